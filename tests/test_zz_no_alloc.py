"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the library live inside a GPU memory pool they do not control (a serving
runtime that owns all device memory, a callback that runs while the pool is locked) and so
cannot allocate scratch; for them the library carries its scratch inside its own image.
This test checks that entry point against the regular one, twice in a row because all calls
share the same scratch, and checks that an oversized problem is refused.  It is collected
last so that a failure here cannot hide any other test's result.
"""
import ctypes

import pytest
import torch

from torchft_b200.ops import _native as N
from torchft_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def _call(lib, dy, x, w, rstd, dres, dx, dw, accumulate):
    T, D = x.shape
    return lib.ftb200_rmsnorm_bwd_noalloc(
        N.ptr(dy), N.ptr(x), N.ptr(w), N.ptr(rstd), N.ptr(dres), N.ptr(dx), N.ptr(dw), ctypes.c_int(T), ctypes.c_int(D),
        ctypes.c_int(int(accumulate)), N.stream_ptr())


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_matches_regular_entry_point_twice():
    lib = N.lib()
    dev = "cuda"
    for call, (T, D) in enumerate([(777, 4096), (64, 1024)]):  # second call reuses the shared scratch
        torch.manual_seed(call)
        x = torch.randn(T, D, device=dev).bfloat16()
        dy = torch.randn(T, D, device=dev).bfloat16()
        dres = torch.randn(T, D, device=dev).bfloat16()
        w = (1 + 0.1 * torch.randn(D, device=dev)).bfloat16()
        _, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
        want_dx, want_dw = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.zeros(D, device=dev, dtype=torch.bfloat16)
        before = torch.cuda.memory_allocated()
        assert _call(lib, dy, x, w, rstd, dres, dx, dw, False) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call > 0:
            # torch's counter cannot see a raw cudaMalloc; the driver's free-memory figure can.  On a warm
            # call (the address is resolved, the kernels are loaded) it must not move.
            free0, _ = torch.cuda.mem_get_info()
            assert _call(lib, dy, x, w, rstd, dres, dx, dw, False) == 0
            torch.cuda.synchronize()
            free1, _ = torch.cuda.mem_get_info()
            assert free1 == free0
        assert _rel(dx, want_dx) < 1e-2
        assert _rel(dw, want_dw) < 2e-2
        # and against the fp32 reference of the op
        rdx, rdw = K.ref_rmsnorm_bwd(dy, x, w, rstd, dres)
        assert _rel(dx, rdx) < 1e-2 and _rel(dw, rdw) < 2e-2


def test_noalloc_accumulates_into_dw():
    """``accumulate_dw=1`` adds the weight gradient to what ``dw`` holds, as the regular entry point does."""
    lib = N.lib()
    torch.manual_seed(5)
    T, D = 300, 2048
    x = torch.randn(T, D, device="cuda").bfloat16()
    dy = torch.randn(T, D, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    _, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
    _, want_dw = K.rmsnorm_bwd(dy, x, w, rstd)
    start = torch.randn(D, device="cuda").bfloat16()
    dw = start.clone()
    dx = torch.empty_like(x)
    assert _call(lib, dy, x, w, rstd, None, dx, dw, True) == 0
    torch.cuda.synchronize()
    assert _rel(dw, start.float() + want_dw.float()) < 2e-2


def test_noalloc_rejects_oversized():
    lib = N.lib()
    t = torch.zeros(8, 16384, device="cuda", dtype=torch.bfloat16)
    r = torch.zeros(8, device="cuda")
    w = torch.zeros(16384, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, t, t, w, r, None, t.clone(), w.clone(), False) == -4
