"""Debug kernel library (-DPK_DEBUG_BOUNDS=1): a bad index is recorded in a status word and the access is skipped. Runs in
a child process so that the debug library is the one every op of that process uses."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r'''
import json, torch
from pocketllm_b200 import ops
from pocketllm_b200.ops import lib, gguf_ops as gk
assert lib.kernels().pk_debug_bounds_enabled() == 1          # nothing below may run on the release build
out = {"clean": lib.debug_bounds()}
# KV append at a position outside the cache: recorded, row not written
M, Hq, Hkv, D, cap = 2, 4, 2, 128, 64
proj = torch.randn(M, Hq * 2 * D + 2 * Hkv * D, device="cuda").to(torch.bfloat16)
kc = torch.zeros(Hkv, cap, D, device="cuda", dtype=torch.bfloat16); vc = torch.zeros_like(kc)
pos = torch.tensor([5, cap + 3], device="cuda", dtype=torch.int32)
g = torch.zeros(D, device="cuda")
ops.qk_norm_rope_append(proj, Hq, Hkv, pos, g, g, 1e-6, 32, 1e6, kc, vc)
out["kv"] = lib.debug_bounds()
out["kv_written_rows"] = int((kc.abs().sum(-1) > 0).sum())
# a routed expert id outside the expert range: recorded and left out of the groups
ids = torch.tensor([[0, 3], [9, 1]], device="cuda", dtype=torch.int32)
w = torch.ones(2, 2, device="cuda")
seg, tok, rw = gk.group_routes(ids, w, 4)[:3]
out["route"] = lib.debug_bounds()
out["seg"] = seg.tolist()
out["after_clear"] = lib.debug_bounds()
print(json.dumps(out))
'''


def test_debug_library_records_bad_indices_and_skips_the_access():
    env = dict(os.environ, POCKET_KERNELS_DEBUG="1", PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=300, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["clean"]["code"] == 0
    assert res["kv"]["code"] == 101 and res["kv"]["index"] == 67 and res["kv"]["limit"] == 64 and res["kv"]["skipped"] == 2   # two KV heads
    assert res["kv_written_rows"] == 2                                     # only position 5, for both KV heads
    assert res["route"]["code"] == 102 and res["route"]["index"] == 9 and res["route"]["limit"] == 4
    assert res["seg"] == [0, 1, 2, 2, 3]                                   # experts 0, 1, 3 got one route each
    assert res["after_clear"]["code"] == 0
