"""GGUF block codecs in numpy: dequantisers for every block type the models use and
quantisers for Q8_0, Q2_K, Q4_K, Q5_K, IQ2_XXS, IQ2_XS, IQ3_XXS and IQ1_M.

Blocks hold 256 weights along the input dimension (32 for Q8_0); `d` / `dmin` are fp16.
Byte layouts follow the public ggml definitions (summarised with the reference's numpy
decoders at src/loader/gguf/tensor_reader.py:592-1009). The reference has no encoders; the
ones here exist so that random-init checkpoints carry real payloads. They favour
clarity over the last bit of quality: scale search is a closed-form min/max fit for the
K-quants and a nearest-codeword search under the sign-parity rule for the IQ types.

`dequantize(blocks, type_name)` takes uint8 [..., nblocks, block_bytes] and returns fp32
[..., nblocks * weights_per_block]; `quantize(x, type_name)` is the inverse direction for
fp32 [..., K].
"""
from __future__ import annotations

from functools import lru_cache

import numpy as np

from .gguf import GGML_TYPE_IDS, GGML_TYPES

QK_K = 256


# --------------------------------------------------------------------------------------
# codebooks (public ggml constants; taken from the installed `gguf` package when present,
# else from the cached copy generated beside this file by `tools_dump_codebooks`)

@lru_cache(maxsize=None)
def codebook(name: str) -> np.ndarray:
    """`iq2_xxs` [256, 8], `iq2_xs` [512, 8], `iq3_xxs` [256, 4] (uint8 magnitudes),
    `iq1` [2048, 8] (int8 in {-1, 0, 1}), `ksigns` [128] (uint8, bit j set = element j negative)."""
    cache = _cache_path()
    if cache.exists():
        with np.load(cache) as z:
            if name in z:
                return z[name]
    books = _codebooks_from_gguf_package()
    return books[name]


def _cache_path():
    from pathlib import Path
    return Path(__file__).with_name("gguf_codebooks.npz")


def _codebooks_from_gguf_package() -> dict[str, np.ndarray]:
    try:
        from gguf import quants as gq
    except Exception as e:  # pragma: no cover - only without the cache and the package
        raise RuntimeError("IQ codebooks need either formats/gguf_codebooks.npz or the `gguf` package") from e
    out = {}
    for key, cls in (("iq2_xxs", gq.IQ2_XXS), ("iq2_xs", gq.IQ2_XS), ("iq3_xxs", gq.IQ3_XXS), ("iq1", gq.IQ1_M)):
        cls.init_grid()
        g = np.asarray(cls.grid).reshape(cls.grid_shape)
        out[key] = g.astype(np.int8 if key == "iq1" else np.uint8)
    out["ksigns"] = np.frombuffer(gq.IQ2_XXS.ksigns, dtype=np.uint8).copy()
    return out


def dump_codebooks() -> None:
    """Write the cache (`gguf_codebooks.npz`) from the installed `gguf` package."""
    np.savez_compressed(_cache_path(), **_codebooks_from_gguf_package())


@lru_cache(maxsize=None)
def _sign_table() -> np.ndarray:
    """[128, 8] of +-1: element j is negative when bit j of ksigns[i] is set."""
    ks = codebook("ksigns").astype(np.uint16)
    bits = (ks[:, None] >> np.arange(8)[None, :]) & 1
    return np.where(bits == 1, -1.0, 1.0).astype(np.float32)


KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def _f16(b: np.ndarray) -> np.ndarray:
    """Two uint8 columns [..., 2] -> fp32."""
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)[..., 0]


def _scale_min_k4(s: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """The 12-byte packed 6-bit (scale, min) pairs of Q4_K / Q5_K -> two [..., 8] uint8 arrays."""
    s = s.astype(np.uint8)
    sc = np.empty(s.shape[:-1] + (8,), dtype=np.uint8)
    mn = np.empty_like(sc)
    sc[..., :4] = s[..., 0:4] & 63
    mn[..., :4] = s[..., 4:8] & 63
    sc[..., 4:] = (s[..., 8:12] & 15) | ((s[..., 0:4] >> 6) << 4)
    mn[..., 4:] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return sc, mn


def _pack_scale_min_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    sc, mn = sc.astype(np.uint8), mn.astype(np.uint8)
    s = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    s[..., 0:4] = (sc[..., :4] & 63) | ((sc[..., 4:] >> 4) << 6)
    s[..., 4:8] = (mn[..., :4] & 63) | ((mn[..., 4:] >> 4) << 6)
    s[..., 8:12] = (sc[..., 4:] & 15) | ((mn[..., 4:] & 15) << 4)
    return s


# --------------------------------------------------------------------------------------
# dequantisers: blocks uint8 [..., nb, bytes] -> fp32 [..., nb, 256 or 32]

def _dq_q8_0(b):
    d = _f16(b[..., 0:2])
    return d[..., None] * b[..., 2:34].view(np.int8).astype(np.float32)


def _dq_q2_k(b):
    sc = b[..., 0:16]
    qs = b[..., 16:80]
    d, dmin = _f16(b[..., 80:82]), _f16(b[..., 82:84])
    out = np.empty(b.shape[:-1] + (256,), dtype=np.float32)
    for g in range(16):
        half, gi = divmod(g, 8)
        shift = (gi // 2) * 2
        byts = qs[..., half * 32 + (gi % 2) * 16: half * 32 + (gi % 2) * 16 + 16]
        q = ((byts >> shift) & 3).astype(np.float32)
        s = sc[..., g]
        out[..., g * 16:(g + 1) * 16] = (d * (s & 15))[..., None] * q - (dmin * (s >> 4))[..., None]
    return out


def _dq_q3_k(b):
    hm, qs, sb = b[..., 0:32], b[..., 32:96], b[..., 96:108]
    d = _f16(b[..., 108:110])
    a = np.ascontiguousarray(sb).view(np.uint32)  # [..., 3]
    a0, a1, tmp = a[..., 0], a[..., 1], a[..., 2]
    k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
    s = np.stack([(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                  ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)], axis=-1)
    scales = np.ascontiguousarray(s).view(np.uint8).astype(np.int32) - 32  # [..., 16]
    out = np.empty(b.shape[:-1] + (256,), dtype=np.float32)
    idx = 0
    m = 1
    for n in range(2):
        q = qs[..., n * 32:(n + 1) * 32]
        for j in range(4):
            shift = 2 * j
            for part in range(2):
                ql = (q[..., part * 16:(part + 1) * 16] >> shift) & 3
                hi = (hm[..., part * 16:(part + 1) * 16] & m) != 0
                val = ql.astype(np.int32) - np.where(hi, 0, 4)
                out[..., idx * 16:(idx + 1) * 16] = (d * scales[..., idx])[..., None] * val
                idx += 1
            m <<= 1
    return out


def _dq_q4_k(b):
    d, dmin = _f16(b[..., 0:2]), _f16(b[..., 2:4])
    sc, mn = _scale_min_k4(b[..., 4:16])
    qs = b[..., 16:144]
    out = np.empty(b.shape[:-1] + (256,), dtype=np.float32)
    for p in range(4):
        q = qs[..., p * 32:(p + 1) * 32]
        for h, nib in ((0, q & 15), (1, q >> 4)):
            j = 2 * p + h
            out[..., p * 64 + h * 32: p * 64 + h * 32 + 32] = (d * sc[..., j])[..., None] * nib - (dmin * mn[..., j])[..., None]
    return out


def _dq_q5_k(b):
    d, dmin = _f16(b[..., 0:2]), _f16(b[..., 2:4])
    sc, mn = _scale_min_k4(b[..., 4:16])
    qh, qs = b[..., 16:48], b[..., 48:176]
    out = np.empty(b.shape[:-1] + (256,), dtype=np.float32)
    for p in range(4):
        q = qs[..., p * 32:(p + 1) * 32]
        for h, nib in ((0, q & 15), (1, q >> 4)):
            j = 2 * p + h
            bit = ((qh >> (2 * p + h)) & 1).astype(np.float32) * 16
            out[..., p * 64 + h * 32: p * 64 + h * 32 + 32] = (d * sc[..., j])[..., None] * (nib + bit) - (dmin * mn[..., j])[..., None]
    return out


def _dq_q6_k(b):
    ql, qh = b[..., 0:128], b[..., 128:192]
    sc = b[..., 192:208].view(np.int8).astype(np.float32)
    d = _f16(b[..., 208:210])
    out = np.empty(b.shape[:-1] + (256,), dtype=np.float32)
    for n in range(2):
        l_ = ql[..., 64 * n: 64 * n + 64]
        h_ = qh[..., 32 * n: 32 * n + 32]
        s_ = sc[..., 8 * n: 8 * n + 8]
        q = [(l_[..., :32] & 15) | ((h_ & 3) << 4), (l_[..., 32:] & 15) | (((h_ >> 2) & 3) << 4),
             (l_[..., :32] >> 4) | (((h_ >> 4) & 3) << 4), (l_[..., 32:] >> 4) | (((h_ >> 6) & 3) << 4)]
        for k in range(4):
            v = q[k].astype(np.float32) - 32
            srep = np.repeat(s_[..., 2 * k: 2 * k + 2], 16, axis=-1)
            out[..., 128 * n + 32 * k: 128 * n + 32 * k + 32] = d[..., None] * srep * v
    return out


def _dq_iq2_xxs(b):
    d = _f16(b[..., 0:2])
    q = b[..., 2:66].reshape(b.shape[:-1] + (8, 8))
    ids = q[..., 0:4]
    aux = np.ascontiguousarray(q[..., 4:8]).view(np.uint32)[..., 0]  # [..., 8]
    ls = (2 * (aux >> 28) + 1).astype(np.float32)
    grid = codebook("iq2_xxs").astype(np.float32)[ids]  # [..., 8, 4, 8]
    sidx = (aux[..., None] >> (7 * np.arange(4, dtype=np.uint32))) & 127
    w = grid * _sign_table()[sidx]
    w = w * (0.125 * d[..., None] * ls)[..., None, None]
    return w.reshape(b.shape[:-1] + (256,))


def _dq_iq2_xs(b):
    d = _f16(b[..., 0:2])
    q = np.ascontiguousarray(b[..., 2:66]).view(np.uint16).reshape(b.shape[:-1] + (8, 4))
    sc = b[..., 66:74]
    nib = np.stack([sc & 15, sc >> 4], axis=-1).astype(np.float32)  # [..., 8, 2]
    db = 0.25 * d[..., None, None] * (nib + 0.5)                     # per pair of parts
    grid = codebook("iq2_xs").astype(np.float32)[q & 511]           # [..., 8, 4, 8]
    w = grid * _sign_table()[q >> 9]
    w = w * np.repeat(db, 2, axis=-1)[..., None]
    return w.reshape(b.shape[:-1] + (256,))


def _dq_iq3_xxs(b):
    d = _f16(b[..., 0:2])
    ids = b[..., 2:66].reshape(b.shape[:-1] + (8, 8))
    aux = np.ascontiguousarray(b[..., 66:98]).view(np.uint32)  # [..., 8]
    ls = (aux >> 28).astype(np.float32)
    grid = codebook("iq3_xxs").astype(np.float32)[ids]  # [..., 8, 8, 4]
    sidx = (aux[..., None] >> (7 * np.arange(4, dtype=np.uint32))) & 127   # [..., 8, 4]
    signs = _sign_table()[sidx].reshape(b.shape[:-1] + (8, 8, 4))           # 8 signs -> two ids
    w = grid * signs * (0.5 * d[..., None] * (ls + 0.5))[..., None, None]
    return w.reshape(b.shape[:-1] + (256,))


def _dq_iq4_xs(b):
    d = _f16(b[..., 0:2])
    sh = np.ascontiguousarray(b[..., 2:4]).view(np.uint16)[..., 0].astype(np.int32)
    sl = b[..., 4:8].astype(np.int32)
    qs = b[..., 8:136].reshape(b.shape[:-1] + (8, 16))
    out = np.empty(b.shape[:-1] + (8, 32), dtype=np.float32)
    for ib in range(8):
        ls = ((sl[..., ib // 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4)
        dl = d * (ls - 32)
        out[..., ib, :16] = dl[..., None] * KVALUES_IQ4NL[qs[..., ib, :] & 15]
        out[..., ib, 16:] = dl[..., None] * KVALUES_IQ4NL[qs[..., ib, :] >> 4]
    return out.reshape(b.shape[:-1] + (256,))


def _dq_iq1_m(b):
    qs = b[..., 0:32].astype(np.int32).reshape(b.shape[:-1] + (8, 4))
    qh = b[..., 32:48].astype(np.int32).reshape(b.shape[:-1] + (8, 2))
    sc = np.ascontiguousarray(b[..., 48:56]).view(np.uint16).astype(np.uint32)  # [..., 4]
    dbits = (sc[..., 0] >> 12) | ((sc[..., 1] >> 8) & 0xF0) | ((sc[..., 2] >> 4) & 0xF00) | (sc[..., 3] & 0xF000)
    d = dbits.astype(np.uint16).view(np.float16).astype(np.float32)
    grid = codebook("iq1").astype(np.float32)
    out = np.empty(b.shape[:-1] + (8, 4, 8), dtype=np.float32)
    for ib in range(8):
        s = sc[..., ib // 2] >> (6 * (ib % 2))
        dl = [d * (2 * ((s >> 0) & 7) + 1).astype(np.float32), d * (2 * ((s >> 3) & 7) + 1).astype(np.float32)]
        for g in range(4):
            h = qh[..., ib, g // 2]
            hi = (h << 8) if g % 2 == 0 else (h << 4)
            idx = qs[..., ib, g] | (hi & 0x700)
            neg = (h & (0x08 if g % 2 == 0 else 0x80)) != 0
            delta = np.where(neg, -0.125, 0.125).astype(np.float32)
            out[..., ib, g, :] = dl[g // 2][..., None] * (grid[idx] + delta[..., None])
    return out.reshape(b.shape[:-1] + (256,))


_DEQUANT = {"q8_0": _dq_q8_0, "q2_k": _dq_q2_k, "q3_k": _dq_q3_k, "q4_k": _dq_q4_k, "q5_k": _dq_q5_k, "q6_k": _dq_q6_k,
            "iq2_xxs": _dq_iq2_xxs, "iq2_xs": _dq_iq2_xs, "iq3_xxs": _dq_iq3_xxs, "iq4_xs": _dq_iq4_xs, "iq1_m": _dq_iq1_m}


def dequantize(blocks: np.ndarray, type_name: str) -> np.ndarray:
    """uint8 [..., nb, block_bytes] (or flat bytes per row [..., nb*block_bytes]) -> fp32 [..., nb*qk]."""
    tid = GGML_TYPE_IDS[type_name]
    _, qk, bs = GGML_TYPES[tid]
    if type_name == "f32":
        return np.ascontiguousarray(blocks).view(np.float32)
    if type_name == "f16":
        return np.ascontiguousarray(blocks).view(np.float16).astype(np.float32)
    if type_name == "bf16":
        u = np.ascontiguousarray(blocks).view(np.uint16).astype(np.uint32) << 16
        return u.view(np.float32)
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    if blocks.shape[-1] != bs:
        blocks = blocks.reshape(blocks.shape[:-1] + (blocks.shape[-1] // bs, bs))
    w = _DEQUANT[type_name](blocks)
    return w.reshape(blocks.shape[:-2] + (blocks.shape[-2] * qk,))


# --------------------------------------------------------------------------------------
# quantisers: fp32 [..., K] -> uint8 [..., K/qk, block_bytes]

def _to_f16_bytes(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x.astype(np.float16)[..., None]).view(np.uint8)


def _q_q8_0(x):
    xb = x.reshape(x.shape[:-1] + (-1, 32))
    d = np.abs(xb).max(-1) / 127.0
    dh = d.astype(np.float16).astype(np.float32)
    q = np.where(dh[..., None] > 0, np.rint(xb / np.where(dh == 0, 1, dh)[..., None]), 0).clip(-127, 127).astype(np.int8)
    out = np.empty(xb.shape[:-1] + (34,), dtype=np.uint8)
    out[..., 0:2] = _to_f16_bytes(d)
    out[..., 2:] = q.view(np.uint8)
    return out


def _affine_fit(xg: np.ndarray, qmax: int) -> tuple[np.ndarray, np.ndarray]:
    """Per group: w ~ scale * q - minv with q in [0, qmax], minv >= 0."""
    lo = np.minimum(xg.min(-1), 0.0)
    hi = np.maximum(xg.max(-1), lo + 1e-30)
    return (hi - lo) / qmax, -lo


def _q_k45(x, bits: int):
    qmax = (1 << bits) - 1
    xb = x.reshape(x.shape[:-1] + (-1, 8, 32))
    scale, minv = _affine_fit(xb, qmax)                       # [..., nb, 8]
    d = scale.max(-1) / 63.0
    dmin = minv.max(-1) / 63.0
    dh, dmh = d.astype(np.float16).astype(np.float32), dmin.astype(np.float16).astype(np.float32)
    sc = np.where(dh[..., None] > 0, np.rint(scale / np.where(dh == 0, 1, dh)[..., None]), 0).clip(0, 63)
    mn = np.where(dmh[..., None] > 0, np.rint(minv / np.where(dmh == 0, 1, dmh)[..., None]), 0).clip(0, 63)
    eff = dh[..., None] * sc
    q = np.where(eff[..., None] > 0, np.rint((xb + (dmh[..., None] * mn)[..., None]) / np.where(eff == 0, 1, eff)[..., None]), 0)
    q = q.clip(0, qmax).astype(np.uint8)                      # [..., nb, 8, 32]
    nb_shape = xb.shape[:-2]
    lo4 = q & 15
    qs = np.empty(nb_shape + (128,), dtype=np.uint8)
    for p in range(4):
        qs[..., p * 32:(p + 1) * 32] = lo4[..., 2 * p, :] | (lo4[..., 2 * p + 1, :] << 4)
    if bits == 4:
        out = np.empty(nb_shape + (144,), dtype=np.uint8)
        out[..., 16:] = qs
    else:
        out = np.empty(nb_shape + (176,), dtype=np.uint8)
        qh = np.zeros(nb_shape + (32,), dtype=np.uint8)
        for j in range(8):
            qh |= ((q[..., j, :] >> 4) & 1) << j
        out[..., 16:48] = qh
        out[..., 48:] = qs
    out[..., 0:2] = _to_f16_bytes(d)
    out[..., 2:4] = _to_f16_bytes(dmin)
    out[..., 4:16] = _pack_scale_min_k4(sc, mn)
    return out


def _q_q2_k(x):
    xb = x.reshape(x.shape[:-1] + (-1, 16, 16))
    scale, minv = _affine_fit(xb, 3)
    d = scale.max(-1) / 15.0
    dmin = minv.max(-1) / 15.0
    dh, dmh = d.astype(np.float16).astype(np.float32), dmin.astype(np.float16).astype(np.float32)
    sc = np.where(dh[..., None] > 0, np.rint(scale / np.where(dh == 0, 1, dh)[..., None]), 0).clip(0, 15).astype(np.uint8)
    mn = np.where(dmh[..., None] > 0, np.rint(minv / np.where(dmh == 0, 1, dmh)[..., None]), 0).clip(0, 15).astype(np.uint8)
    eff = dh[..., None] * sc
    q = np.where(eff[..., None] > 0, np.rint((xb + (dmh[..., None] * mn)[..., None]) / np.where(eff == 0, 1, eff)[..., None]), 0)
    q = q.clip(0, 3).astype(np.uint8)
    nb_shape = xb.shape[:-2]
    out = np.zeros(nb_shape + (84,), dtype=np.uint8)
    out[..., 0:16] = sc | (mn << 4)
    for g in range(16):
        half, gi = divmod(g, 8)
        shift = (gi // 2) * 2
        sl = slice(16 + half * 32 + (gi % 2) * 16, 16 + half * 32 + (gi % 2) * 16 + 16)
        out[..., sl] |= q[..., g, :] << shift
    out[..., 80:82] = _to_f16_bytes(d)
    out[..., 82:84] = _to_f16_bytes(dmin)
    return out


def _parity_signs(v: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Signs of 8-vectors constrained to an even number of minus signs.

    Returns (ksigns index [..], sign array [.., 8] of +-1 actually used)."""
    neg = v < 0
    odd = (neg.sum(-1) % 2) == 1
    weakest = np.abs(v).argmin(-1)
    flip = np.zeros_like(neg)
    np.put_along_axis(flip, weakest[..., None], odd[..., None], axis=-1)
    neg = neg ^ flip
    idx7 = (neg[..., :7] * (1 << np.arange(7))).sum(-1).astype(np.uint8)
    return idx7, np.where(neg, -1.0, 1.0).astype(np.float32)


def _nearest(mag: np.ndarray, grid: np.ndarray) -> np.ndarray:
    """Index of the nearest row of `grid` [G, n] for each row of `mag` [N, n] (chunked)."""
    g = grid.astype(np.float32)
    g2 = (g * g).sum(-1)
    out = np.empty(mag.shape[0], dtype=np.int64)
    step = 1 << 15
    for i in range(0, mag.shape[0], step):
        m = mag[i:i + step]
        out[i:i + step] = (g2[None, :] - 2.0 * (m @ g.T)).argmin(-1)
    return out


def _iq_grid_quant(x, grid_name: str, n: int, code_scale: float, ls_bits: int, ls_form: str):
    """Shared part of IQ2_XXS / IQ2_XS / IQ3_XXS: choose the super scale d, the per-sub-block
    integer scale ls, the codeword of each n-vector and the sign pattern of each 8-vector."""
    grid = codebook(grid_name).astype(np.float32)
    xb = x.reshape(x.shape[:-1] + (-1, 8, 32)).astype(np.float32)      # [..., nb, 8 sub-blocks, 32]
    gmax = float(grid.max())
    ls_max = (1 << ls_bits) - 1
    sub_amax = np.abs(xb).max(-1)                                       # [..., nb, 8]
    # effective multiplier of a sub-block: d * code_scale * f(ls)
    f_max = (2 * ls_max + 1) if ls_form == "odd" else (ls_max + 0.5)
    d = sub_amax.max(-1) / (code_scale * f_max * gmax * 0.85)
    dh = np.maximum(d.astype(np.float16).astype(np.float32), 1e-30)
    want = sub_amax / (dh[..., None] * code_scale * gmax * 0.85)        # desired f(ls)
    ls = np.rint((want - 1) / 2) if ls_form == "odd" else np.rint(want - 0.5)
    ls = ls.clip(0, ls_max)
    f = (2 * ls + 1) if ls_form == "odd" else (ls + 0.5)
    eff = dh[..., None] * code_scale * f                                # [..., nb, 8]
    t = xb / np.maximum(eff, 1e-30)[..., None]                          # target in code units
    v8 = t.reshape(t.shape[:-1] + (4, 8))
    sidx, signs = _parity_signs(v8)
    mag = np.abs(v8)
    flat = mag.reshape(-1, n)
    ids = _nearest(flat, grid).reshape(mag.shape[:-1] + (8 // n,))
    return dh, d, ls.astype(np.uint32), ids, sidx


def _q_iq2_xxs(x):
    dh, d, ls, ids, sidx = _iq_grid_quant(x, "iq2_xxs", 8, 0.125, 4, "odd")
    nb_shape = ids.shape[:-3]
    out = np.zeros(nb_shape + (66,), dtype=np.uint8)
    out[..., 0:2] = _to_f16_bytes(d)
    q = np.zeros(nb_shape + (8, 8), dtype=np.uint8)
    q[..., 0:4] = ids[..., 0].astype(np.uint8)
    aux = (ls << 28).astype(np.uint32)
    for p in range(4):
        aux |= sidx[..., p].astype(np.uint32) << (7 * p)
    q[..., 4:8] = np.ascontiguousarray(aux[..., None]).view(np.uint8)
    out[..., 2:] = q.reshape(nb_shape + (64,))
    return out


def _q_iq2_xs(x):
    # the scale is shared by pairs of 8-vectors (16 weights); fit per 32 and store it twice
    dh, d, ls, ids, sidx = _iq_grid_quant(x, "iq2_xs", 8, 0.25, 4, "half")
    nb_shape = ids.shape[:-3]
    out = np.zeros(nb_shape + (74,), dtype=np.uint8)
    out[..., 0:2] = _to_f16_bytes(d)
    q16 = (ids[..., 0].astype(np.uint16) & 511) | (sidx.astype(np.uint16) << 9)     # [..., nb, 8, 4]
    out[..., 2:66] = np.ascontiguousarray(q16).view(np.uint8).reshape(nb_shape + (64,))
    out[..., 66:74] = (ls | (ls << 4)).astype(np.uint8)
    return out


def _q_iq3_xxs(x):
    dh, d, ls, ids, sidx = _iq_grid_quant(x, "iq3_xxs", 4, 0.5, 4, "half")
    nb_shape = ids.shape[:-3]
    out = np.zeros(nb_shape + (98,), dtype=np.uint8)
    out[..., 0:2] = _to_f16_bytes(d)
    out[..., 2:66] = ids.reshape(nb_shape + (64,)).astype(np.uint8)
    aux = (ls << 28).astype(np.uint32)
    for p in range(4):
        aux |= sidx[..., p].astype(np.uint32) << (7 * p)
    out[..., 66:98] = np.ascontiguousarray(aux).view(np.uint8).reshape(nb_shape + (32,))
    return out


def _q_iq1_m(x):
    grid = codebook("iq1").astype(np.float32)
    xb = x.reshape(x.shape[:-1] + (-1, 16, 16)).astype(np.float32)      # [..., nb, 16 groups of 16]
    amax16 = np.abs(xb).max(-1)
    # values are dl * (g + delta), |g + delta| <= 1.125, dl = d * (2 ls + 1), ls in 0..7
    d = amax16.max(-1) / (15.0 * 1.125)
    dh = np.maximum(d.astype(np.float16).astype(np.float32), 1e-30)
    ls = np.rint((amax16 / (dh[..., None] * 1.125) - 1) / 2).clip(0, 7)
    dl = dh[..., None] * (2 * ls + 1)
    t = (xb / np.maximum(dl, 1e-30)[..., None]).reshape(xb.shape[:-2] + (32, 8))   # 32 groups of 8
    flat = t.reshape(-1, 8)
    best_idx = np.zeros(flat.shape[0], dtype=np.int64)
    best_neg = np.zeros(flat.shape[0], dtype=bool)
    best_err = np.full(flat.shape[0], np.inf, dtype=np.float32)
    for neg, delta in ((False, 0.125), (True, -0.125)):
        idx = _nearest(flat - delta, grid)
        err = ((grid[idx] + delta - flat) ** 2).sum(-1)
        take = err < best_err
        best_idx[take], best_neg[take], best_err[take] = idx[take], neg, err[take]
    nb_shape = xb.shape[:-2]
    idx = best_idx.reshape(nb_shape + (8, 4))
    neg = best_neg.reshape(nb_shape + (8, 4))
    out = np.zeros(nb_shape + (56,), dtype=np.uint8)
    out[..., 0:32] = (idx & 0xFF).astype(np.uint8).reshape(nb_shape + (32,))
    hi = ((idx >> 8) & 7).astype(np.uint8) | (neg.astype(np.uint8) << 3)            # nibble per group of 8
    qh = hi[..., 0::2] | (hi[..., 1::2] << 4)                                        # [..., nb, 8, 2]
    out[..., 32:48] = qh.reshape(nb_shape + (16,))
    ls16 = ls.astype(np.uint32).reshape(nb_shape + (4, 4))                           # four 3-bit scales per word
    words = ls16[..., 0] | (ls16[..., 1] << 3) | (ls16[..., 2] << 6) | (ls16[..., 3] << 9)
    dbits = d.astype(np.float16).view(np.uint16).astype(np.uint32)
    words = words | np.stack([(dbits & 0xF) << 12, ((dbits >> 4) & 0xF) << 12, ((dbits >> 8) & 0xF) << 12,
                              ((dbits >> 12) & 0xF) << 12], axis=-1)
    out[..., 48:56] = np.ascontiguousarray(words.astype(np.uint16)).view(np.uint8).reshape(nb_shape + (8,))
    return out


_QUANT = {"q8_0": _q_q8_0, "q4_k": lambda x: _q_k45(x, 4), "q5_k": lambda x: _q_k45(x, 5), "q2_k": _q_q2_k,
          "iq2_xxs": _q_iq2_xxs, "iq2_xs": _q_iq2_xs, "iq3_xxs": _q_iq3_xxs, "iq1_m": _q_iq1_m}

QUANTIZABLE = tuple(_QUANT)


def quantize(x: np.ndarray, type_name: str) -> np.ndarray:
    """fp32 [..., K] -> uint8 [..., K / qk, block_bytes]."""
    tid = GGML_TYPE_IDS[type_name]
    _, qk, bs = GGML_TYPES[tid]
    x = np.asarray(x, dtype=np.float32)
    if type_name == "f32":
        return np.ascontiguousarray(x).view(np.uint8)
    if type_name == "f16":
        return np.ascontiguousarray(x.astype(np.float16)).view(np.uint8)
    if x.shape[-1] % qk:
        raise ValueError(f"last dim {x.shape[-1]} is not a multiple of {qk}")
    out = _QUANT[type_name](x)
    assert out.shape[-1] == bs, (type_name, out.shape)
    return out
