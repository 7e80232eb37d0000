"""CPU expert server process: owns the routed experts of every layer (from a shared weight arena) and serves the
model ranks over shared-memory channels (reference: src/models/deepseek_v4/moe_server.py:24-34,36-104,111-151).

    python -m pocketllm_b200.moe.moe_server --arena NAME --channels chan0,chan1 --max-tokens 64 --hidden 1024 --topk 2
"""
from __future__ import annotations

import argparse
import signal
import time

import torch

from . import cpu_oracle as co
from . import ipc

_FIELDS = ("router", "w13", "s13", "w2", "s2", "shared_w13", "shared_s13", "shared_w2", "shared_s2", "bias")


def pack_layers(layers: dict[int, co.Fp4MoEWeights]) -> dict[str, torch.Tensor]:
    out = {}
    for l, w in layers.items():
        for f in _FIELDS:
            t = getattr(w, f)
            if t is not None:
                out[f"{l}.{f}"] = t
    return out


def unpack_layers(arena: ipc.SharedWeightArena) -> dict[int, co.Fp4MoEWeights]:
    ids = sorted({int(k.split(".")[0]) for k in arena.directory})
    layers = {}
    for l in ids:
        kw = {f: arena.tensor(f"{l}.{f}") for f in _FIELDS if f"{l}.{f}" in arena.directory}
        layers[l] = co.Fp4MoEWeights(**kw)
    return layers


def serve(arena_name: str, channel_names: list[str], max_tokens: int, hidden: int, topk: int, score_func: str = "softmax",
          route_scale: float = 1.0, swiglu_limit: float = 0.0, idle_exit_s: float = 0.0) -> None:
    arena = ipc.SharedWeightArena.attach(arena_name, timeout_s=600.0)
    layers = unpack_layers(arena)
    chans = [ipc.MoEChannel(n, max_tokens, hidden, create=False) for n in channel_names]
    last = [int(c.hdr[ipc.REQ]) for c in chans]
    stop = {"now": False}
    signal.signal(signal.SIGTERM, lambda *_: stop.update(now=True))
    for c in chans:
        c.hdr[ipc.READY] = 1
    idle_since = time.monotonic()
    try:
        while not stop["now"]:
            busy = False
            for i, c in enumerate(chans):
                if c.hdr[ipc.STOP]:
                    stop["now"] = True
                    break
                req = c.poll(last[i])
                if req is None:
                    continue
                seq, layer, x = req
                y, _, _ = co.forward_native(torch.from_numpy(x.copy()), layers[layer], topk, score_func=score_func, route_scale=route_scale,
                                            swiglu_limit=swiglu_limit)
                c.respond(seq, y.numpy())
                last[i] = seq
                busy = True
            if busy:
                idle_since = time.monotonic()
            else:
                if idle_exit_s and time.monotonic() - idle_since > idle_exit_s:
                    break
                time.sleep(0)
    finally:
        for c in chans:
            c.hdr[ipc.STOP] = 1                        # clients see "server stopped" instead of waiting
            c.close(unlink=False)
        del layers
        arena.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arena", required=True)
    ap.add_argument("--channels", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--hidden", type=int, required=True)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--score-func", default="softmax")
    ap.add_argument("--route-scale", type=float, default=1.0)
    ap.add_argument("--swiglu-limit", type=float, default=0.0)
    ap.add_argument("--idle-exit-s", type=float, default=0.0)
    a = ap.parse_args(argv)
    serve(a.arena, a.channels.split(","), a.max_tokens, a.hidden, a.topk, a.score_func, a.route_scale, a.swiglu_limit, a.idle_exit_s)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
