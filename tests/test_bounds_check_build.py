"""The checked-index debug build of the kernel library (-DFT_BOUNDS_CHECK=1): guarded indices
that are out of range are recorded and the access is skipped; nothing here reads or writes
out of bounds.  Runs in a child process because the library variant is chosen at load time."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import ctypes, json, torch
from torchft_b200.ops import _native as N, kernels as K
lib = N.lib()
dev = torch.device("cuda")
out = {}
ok = torch.zeros(1, dtype=torch.int32, device=dev)
assert lib.ftb200_bounds_selftest(ctypes.c_int(3), ctypes.c_int(4), N.ptr(ok), N.stream_ptr()) == 0
torch.cuda.synchronize()
out["in_range"] = (int(ok.item()), N.bounds_status())
assert lib.ftb200_bounds_selftest(ctypes.c_int(5), ctypes.c_int(4), N.ptr(ok), N.stream_ptr()) == 0
torch.cuda.synchronize()
out["out_of_range"] = (int(ok.item()), N.bounds_status())
out["cleared"] = N.bounds_status()
# a token id outside the vocabulary: recorded, and row 0 is read instead
V, D = 64, 128
table = torch.randn(V, D, device=dev).bfloat16()
tok = torch.tensor([1, 2, V + 7, 3], device=dev)
emb = K.embedding_fwd(tok, table)
torch.cuda.synchronize()
out["embedding"] = (N.bounds_status(), bool(torch.equal(emb[2], table[0])), bool(torch.equal(emb[1], table[2])))
# ordinary kernels leave the status clean
x = torch.randn(256, 512, device=dev).bfloat16()
w = torch.ones(512, device=dev).bfloat16()
K.rmsnorm_fwd(x, w, 1e-5)
logits = torch.randn(64, 1024, device=dev).bfloat16()
K.cross_entropy_(logits, torch.randint(0, 1024, (64,), device=dev), 1.0)
a = torch.randn(256, 128, device=dev).bfloat16(); b = torch.randn(256, 128, device=dev).bfloat16()
K.gemm(a, b)
torch.cuda.synchronize()
out["clean"] = N.bounds_status()
print(json.dumps(out))
"""


def test_checked_build_records_and_skips():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, FTB200_KERNEL_LIB="checked", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert res["in_range"] == [1, [0, 0]]
    assert res["out_of_range"] == [0, [4, 5]]
    assert res["cleared"] == [0, 0]
    assert res["embedding"] == [[4, 64 + 7], True, True]
    assert res["clean"] == [0, 0]
