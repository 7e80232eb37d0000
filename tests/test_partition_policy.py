"""Partition policies and the layer pipeline on CPU (gloo) ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pocketllm_b200.parallel import partition as P


def test_policy_names_and_aliases():
    assert P.normalize_policy(None) == "replicated" and P.normalize_policy("baseline_4gpu") == "tp"
    assert P.normalize_policy("layer_pp_4gpu") == "layer_pp"
    with pytest.raises(ValueError):
        P.normalize_policy("zigzag")


def test_rule_kinds():
    assert P.rule_kind("layers.3.ffn.experts.17.w1.weight") == "expert_owned"
    assert P.rule_kind("layers.3.ffn.shared_experts.w1.weight") == "replicated_shared_expert"
    assert P.rule_kind("layers.0.attn.wo_b.weight") == "row_parallel"
    assert P.rule_kind("layers.0.attn.wq_b.scale") == "column_parallel"
    assert P.rule_kind("layers.0.attn.attn_sink") == "attn_sink"
    assert P.rule_kind("embed.weight") == "column_parallel" and P.rule_kind("layers.0.attn_norm.weight") == "replicated"


def test_tp_shards_reassemble():
    w = torch.arange(8 * 12, dtype=torch.float32).reshape(8, 12)
    cols = [P.shard_tensor("layers.0.attn.wq_b.weight", w, "tp", 4, r) for r in range(4)]
    rows = [P.shard_tensor("layers.0.attn.wo_b.weight", w, "tp", 4, r) for r in range(4)]
    assert torch.equal(torch.cat(cols, 0), w) and torch.equal(torch.cat(rows, 1), w)
    g = w[0]
    assert P.shard_tensor("layers.0.attn_norm.weight", g, "tp", 4, 1) is g
    sink = torch.arange(8.0)
    assert torch.equal(P.shard_tensor("layers.0.attn.attn_sink", sink, "tp", 4, 3), sink[6:])
    with pytest.raises(ValueError):
        P.shard_tensor("layers.0.attn.wq_b.weight", w[:6], "tp", 4, 0)


def test_expert_ownership_and_needed_keys():
    keys = [f"layers.0.ffn.experts.{e}.w1.weight" for e in range(8)] + [f"layers.0.ffn.experts.{e}.w1.scale" for e in range(8)] + ["embed.weight"]
    mine = P.needed_keys(keys, "tp", 4, 2, n_experts=8)
    assert mine == ["layers.0.ffn.experts.4.w1.weight", "layers.0.ffn.experts.5.w1.weight", "embed.weight"]
    assert P.shard_tensor("layers.0.ffn.experts.1.w1.weight", torch.zeros(2, 2), "replicated", 4, 2, n_experts=8) is None


def test_quant_block_sharding_keeps_blocks_whole():
    blocks = np.arange(4 * 6 * 34, dtype=np.uint8).reshape(4, 6, 34)          # q8_0: 34-byte blocks
    r = [P.shard_quant_blocks("layers.0.attn.wo_b.weight", blocks, "tp", 2, k) for k in range(2)]
    assert r[0].shape == (4, 3, 34) and np.array_equal(np.concatenate(r, 1), blocks)
    c = [P.shard_quant_blocks("layers.0.attn.wq_b.weight", blocks, "tp", 2, k) for k in range(2)]
    assert c[1].shape == (2, 6, 34) and np.array_equal(np.concatenate(c, 0), blocks)


def test_layer_pp_ownership():
    assert [P.layer_range(43, 4, s) for s in range(4)] == [(0, 10), (10, 21), (21, 32), (32, 43)]
    assert P.parameter_owner("embed.weight", 43, 4) == 0 and P.parameter_owner("head.weight", 43, 4) == 3
    assert P.parameter_owner("mtp.0.attn.wq_a.weight", 43, 4) == 3 and P.parameter_owner("layers.21.ffn.gate.weight", 43, 4) == 2
    assert P.parameter_owner("freqs", 43, 4) is None
    assert not P.shard_for_rank("layers.5.attn.wq_a.weight", (4, 4), "layer_pp", 4, 1, n_layers=43).owned
    line = P.layout_line("layer_pp", 4, 3, n_layers=43, n_experts=256)
    assert "layers=[32,43)" in line and "owns_head=True" in line


def test_forbidden_environment(monkeypatch):
    P.check_environment("tp", 8)
    monkeypatch.setenv("POCKET_CPU_MOE_RANK0_SERVER", "1")
    P.check_environment("replicated", 8)
    with pytest.raises(RuntimeError, match="RANK0_SERVER"):
        P.check_environment("tp", 8)
    monkeypatch.delenv("POCKET_CPU_MOE_RANK0_SERVER")
    monkeypatch.setenv("POCKET_DECODE_MTP_SPEC", "1")
    with pytest.raises(RuntimeError, match="MTP"):
        P.check_environment("layer_pp", 4)


def _pp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from pocketllm_b200.parallel.pipeline import PipelineStage
    torch.manual_seed(0)
    emb = torch.randn(50, 16)
    ws = [torch.randn(16, 16) / 4 for _ in range(6)]
    head = torch.randn(16, 50)
    st = PipelineStage(6)
    tok = torch.tensor([3, 7])
    seq = []
    for _ in range(3):
        tok = st.step(tok, lambda t: emb[t], lambda x, lo, hi: _run(x, ws, lo, hi), lambda x: (x @ head).argmax(-1), (2, 16))
        seq.append(tok.tolist())
    if rank == 0:
        x = torch.tensor([3, 7])
        ref = []
        for _ in range(3):
            x = (_run(emb[x], ws, 0, 6) @ head).argmax(-1)
            ref.append(x.tolist())
        out.put((seq, ref))
    dist.destroy_process_group()


def _run(x, ws, lo, hi):
    for w in ws[lo:hi]:
        x = torch.tanh(x @ w) + x
    return x


def test_pipeline_three_stages_matches_single_process():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pp_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    seq, ref = q.get(timeout=120)
    for p in procs:
        p.join(60)
    assert seq == ref
