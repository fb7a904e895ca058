"""fp8 block quantisation: format round trip, kernels against the PyTorch restatement,
quantised collectives over gloo (CPU) and the fused peer kernel (GPU, emulated team).
Error bounds follow the thresholds the reference asserts (mean relative error <= 0.05)."""
import ctypes
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
from torch.distributed.distributed_c10d import ReduceOp

from torchft_b200 import quantization as Q
from torchft_b200.collectives import allreduce_quantized, reduce_scatter_quantized, allocate_reduce_scatter_output
from torchft_b200.process_group import ProcessGroupGloo


def mean_rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().mean() / b.abs().mean()).item()


def with_outliers(n, seed, mult=100.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g)
    idx = torch.randperm(n, generator=g)[: max(1, n // 1000)]
    x[idx] *= mult
    return x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [128, 4096, 128 * 1000])
def test_roundtrip_cpu(dtype, n):
    x = with_outliers(n, 0).to(dtype)
    buf = torch.empty(Q.quantized_nbytes(n), dtype=torch.uint8)
    Q.quantize_into(x, buf)
    y = torch.empty_like(x)
    Q.dequantize_from(buf, y)
    assert mean_rel_err(y, x) < 0.05
    # a block of zeros stays zero and has a finite scale
    z = torch.zeros(256, dtype=dtype)
    zb = torch.empty(Q.quantized_nbytes(256), dtype=torch.uint8)
    Q.quantize_into(z, zb)
    out = torch.ones(256, dtype=dtype)
    Q.dequantize_from(zb, out)
    assert out.abs().sum() == 0


def test_list_api_and_padding_cpu():
    ts = [torch.randn(5, 7), torch.randn(130), torch.randn(3, 3, 3)]
    orig = [t.clone() for t in ts]
    buf, (n,) = Q.fused_quantize_into_fp8(ts, world_size=3)
    assert n % (128 * 3) == 0 and buf.numel() == Q.quantized_nbytes(n)
    for t in ts:
        t.zero_()
    Q.fused_dequantize_from_fp8(ts, buf, world_size=3)
    for t, o in zip(ts, orig):
        assert mean_rel_err(t, o) < 0.06


def _gloo(world):
    store = dist.TCPStore("localhost", 0, is_master=True, wait_for_workers=False)
    pgs = [ProcessGroupGloo(timeout=timedelta(seconds=20)) for _ in range(world)]
    with ThreadPoolExecutor(max_workers=world) as ex:
        list(ex.map(lambda r: pgs[r].configure(f"localhost:{store.port}/q", "r", r, world), range(world)))
    for r, pg in enumerate(pgs):
        pg._rank = r
    return store, pgs


@pytest.mark.parametrize("op", [ReduceOp.SUM, ReduceOp.AVG])
def test_allreduce_quantized_gloo(op):
    world = 2
    store, pgs = _gloo(world)
    try:
        data = [[with_outliers(1000, 10 * r + i).reshape(10, 100) for i in range(2)] for r in range(world)]
        want = [sum(data[r][i] for r in range(world)) / (world if op == ReduceOp.AVG else 1) for i in range(2)]

        def run(r):
            ts = [t.clone() for t in data[r]]
            allreduce_quantized(ts, op, pgs[r]).wait()
            return ts

        with ThreadPoolExecutor(max_workers=world) as ex:
            outs = list(ex.map(run, range(world)))
        for ts in outs:
            for t, w in zip(ts, want):
                assert mean_rel_err(t, w) < 0.05
        for a, b in zip(outs[0], outs[1]):
            assert torch.equal(a, b)  # every rank ends with identical values
    finally:
        for pg in pgs:
            pg.shutdown()


def test_reduce_scatter_quantized_gloo():
    world = 2
    store, pgs = _gloo(world)
    try:
        data = [[with_outliers(1024, 3 * r)] for r in range(world)]
        total = (data[0][0] + data[1][0])

        def run(r):
            out, n = allocate_reduce_scatter_output(data[r], world)
            reduce_scatter_quantized(out, [t.clone() for t in data[r]], ReduceOp.SUM, pgs[r]).wait()
            return out

        with ThreadPoolExecutor(max_workers=world) as ex:
            outs = list(ex.map(run, range(world)))
        per = 1024 // world
        for r, o in enumerate(outs):
            assert mean_rel_err(o, total[r * per : (r + 1) * per]) < 0.05
    finally:
        for pg in pgs:
            pg.shutdown()


def _factorisations(n):
    return [(a, n // a) for a in range(1, n + 1) if n % a == 0]


def _simulated_allreduce(per_rank, scale):
    """The quantised allreduce for ranks that live in one process: quantise each rank's flat data, hand slice r of
    every rank to rank r, reduce there, gather the reduced slices, dequantise (the data flow of allreduce_quantized
    with the collectives replaced by slicing)."""
    ws = len(per_rank)
    n = Q.padded_numel(per_rank[0].numel(), ws)
    per = n // ws
    qbufs = []
    for x in per_rank:
        flat = torch.zeros(n, dtype=x.dtype)
        flat[: x.numel()] = x.reshape(-1)
        b = torch.empty(Q.quantized_nbytes(n), dtype=torch.uint8)
        Q.quantize_into(flat, b)
        qbufs.append(b)
    full = torch.empty(Q.quantized_nbytes(n), dtype=torch.uint8)
    fc, fs = Q.split_quantized(full, n)
    nb = per // Q.BLOCK
    for r in range(ws):
        parts = []
        for k in range(ws):
            c, sc = Q.split_quantized(qbufs[(r + k) % ws], n)
            b = torch.empty(Q.quantized_nbytes(per), dtype=torch.uint8)
            bc, bs = Q.split_quantized(b, per)
            bc.copy_(c[r * per : (r + 1) * per])
            bs.copy_(sc[r * nb : (r + 1) * nb])
            parts.append(b)
        red = torch.empty(Q.quantized_nbytes(per), dtype=torch.uint8)
        Q.reduce_quantized(parts, per, scale, red)
        rc, rs = Q.split_quantized(red, per)
        fc[r * per : (r + 1) * per].copy_(rc)
        fs[r * nb : (r + 1) * nb].copy_(rs)
    out = torch.empty(n, dtype=per_rank[0].dtype)
    Q.dequantize_from(full, out)
    return out[: per_rank[0].numel()]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("avg", [False, True])
def test_simulated_two_rank_allreduce_matrix(dtype, avg):
    """Sizes x multipliers x every 2-D factorisation of the size, two simulated ranks, against the exact
    reduction; mean relative error <= 0.05 (the matrix of torchft/quantization_test.py:35-131)."""
    ws = 2
    g = torch.Generator().manual_seed(5)
    for size in (128, 512, 4096):
        for mult in (1.0, 100.0, 1000.0):
            if dtype == torch.float16 and mult == 1000.0 and not avg:
                mult = 500.0  # keep the exact sum inside fp16's range
            for rows, cols in _factorisations(size):
                xs = [(torch.rand(rows, cols, generator=g) * mult).to(dtype) for _ in range(ws)]
                want = sum(x.float() for x in xs) * (1.0 / ws if avg else 1.0)
                got = _simulated_allreduce(xs, 1.0 / ws if avg else 1.0).view(rows, cols)
                assert got.dtype == dtype
                assert mean_rel_err(got, want) <= 0.05, (size, mult, rows, cols)


# ------------------------------------------------------------------------------------ GPU


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernels_match_reference_gpu(dtype):
    n = 128 * 4099
    x = with_outliers(n, 1).to(dtype).cuda()
    sub = with_outliers(n, 2).to(dtype).cuda()
    buf = torch.empty(Q.quantized_nbytes(n), dtype=torch.uint8, device="cuda")
    Q.quantize_into(x, buf)
    codes, scales = Q.split_quantized(buf, n)
    rc, rs = Q.ref_quantize(x)
    torch.testing.assert_close(scales, rs, rtol=1e-6, atol=0)
    assert (codes != rc).float().mean().item() < 1e-3  # rounding ties may differ in a handful of codes
    y = torch.empty_like(x)
    Q.dequantize_from(buf, y)
    assert mean_rel_err(y, x) < 0.05
    Q.quantize_into(x, buf, minus=sub)  # fused pseudo-gradient
    Q.dequantize_from(buf, y)
    assert mean_rel_err(y, x.float() - sub.float()) < 0.05


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_allreduce_fp8_emulated(world, dtype):
    from test_team_gpu import Emu
    from torchft_b200.ops import _native as N

    n = 128 * world * 37
    emu = Emu(world, Q.quantized_nbytes(n) + 256)
    arenas = [emu.arenas[r][emu.fb:] for r in range(world)]
    ins = [with_outliers(n, 100 + r).to(dtype).cuda() for r in range(world)]
    outs = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(world)]
    want = sum(t.float() for t in ins) / world
    rc = emu.lib.ftb200_team_allreduce_fp8_emulated(
        emu.descs(), ctypes.c_int(world), emu.ptrs(arenas), emu.ptrs(ins), None, emu.ptrs(outs), ctypes.c_longlong(n),
        ctypes.c_int(0 if dtype == torch.bfloat16 else 1), ctypes.c_float(1.0 / world), ctypes.c_int(2), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert all(int(s.item()) == 0 for s in emu.status)
    for o in outs:
        assert torch.equal(o, outs[0])
        assert mean_rel_err(o, want) < 0.05


@pytest.mark.gpu
def test_diloco_outer_step_kernel_matches_torch_sgd_nesterov():
    from torchft_b200.ops.diloco import outer_step_

    torch.manual_seed(0)
    n = 4 * 1001
    backup = torch.randn(n, device="cuda")
    param = backup + 0.1 * torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(backup.clone())
    opt = torch.optim.SGD([ref_p], lr=0.7, momentum=0.9, nesterov=True)
    mom = torch.zeros(n, device="cuda")
    for step in range(3):
        g = torch.randn(n, device="cuda")
        local = param.clone()
        outer_step_(g, mom, backup, param, lr=0.7, momentum_coef=0.9, alpha=0.25, nesterov=True, first_step=step == 0)
        ref_p.grad = g.clone()
        opt.step()
        torch.testing.assert_close(backup, ref_p.data, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(param, torch.lerp(ref_p.data, local, 0.25), rtol=1e-5, atol=1e-6)
        param = backup + 0.1 * torch.randn(n, device="cuda")
