"""Peer-memory collectives, all ranks of a team emulated by one cooperative launch on a
single GPU (separate launches that wait on one another must not share a GPU), plus the
bounded-wait path: a team whose peer never shows up must return a TIMEOUT status."""
import ctypes

import pytest
import torch

from torchft_b200.ops import _native as N
from torchft_b200.parallel.team import MAX_RANKS, _TeamDesc

pytestmark = pytest.mark.gpu
DEV = "cuda"


class Emu:
    def __init__(self, world, nbytes, timeout_s=5.0, epoch=7):
        self.lib = N.lib()
        self.world = world
        fb = int(self.lib.ftb200_team_flag_bytes())
        self.fb = (fb + 255) // 256 * 256
        self.arenas = [torch.zeros(self.fb + nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
        self.sync = [torch.zeros(8, dtype=torch.int64, device=DEV) for _ in range(world)]
        self.status = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(world)]
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch, self.seq = epoch, 0

    def descs(self, n=None):
        self.seq += 1
        arr = (_TeamDesc * self.world)()
        for r in range(self.world):
            d = arr[r]
            d.rank, d.world = r, self.world
            d.token = (self.epoch << 32) | self.seq
            d.timeout_ns = self.timeout_ns
            for p in range(self.world):
                d.flags[p] = self.arenas[p].data_ptr()
            d.local_sync = self.sync[r].data_ptr()
            d.abort_word = None
            d.status = self.status[r].data_ptr()
        return arr

    def buf(self, r, numel, dtype):
        es = torch.empty((), dtype=dtype).element_size()
        return self.arenas[r][self.fb : self.fb + numel * es].view(dtype)

    def ptrs(self, tensors):
        arr = (ctypes.c_void_p * MAX_RANKS)()
        for i, t in enumerate(tensors):
            arr[i] = t.data_ptr() if t is not None else None
        return arr


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_allreduce_emulated(world, dtype):
    torch.manual_seed(0)
    n = world * 8 * 1000
    emu = Emu(world, n * 4)
    bufs = [emu.buf(r, n, dtype) for r in range(world)]
    data = [torch.randn(n, device=DEV).to(dtype) for _ in range(world)]
    for b, d in zip(bufs, data):
        b.copy_(d)
    ref = sum(d.float() for d in data) / world
    rc = emu.lib.ftb200_team_allreduce_emulated(
        emu.descs(), ctypes.c_int(world), emu.ptrs(bufs), None, None, ctypes.c_longlong(n),
        ctypes.c_int(0 if dtype == torch.bfloat16 else 1), ctypes.c_float(1.0 / world), None, ctypes.c_int(3),
        N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert all(int(s.item()) == 0 for s in emu.status)
    for b in bufs:
        assert torch.equal(b, bufs[0])  # every rank holds bit-identical results
        torch.testing.assert_close(b.float(), ref, rtol=2e-2, atol=2e-2)


def test_allreduce_emulated_staged_and_zero_contribution():
    world, n, dtype = 2, 2 * 8 * 512, torch.bfloat16
    emu = Emu(world, n * 2)
    bufs = [emu.buf(r, n, dtype) for r in range(world)]
    user = [torch.randn(n, device=DEV).to(dtype) for _ in range(world)]
    orig = [u.clone() for u in user]
    zero = (ctypes.c_int * world)(0, 1)  # rank 1 is "healing": contributes zeros
    rc = emu.lib.ftb200_team_allreduce_emulated(
        emu.descs(), ctypes.c_int(world), emu.ptrs(bufs), emu.ptrs(user), emu.ptrs(user), ctypes.c_longlong(n),
        ctypes.c_int(0), ctypes.c_float(1.0), zero, ctypes.c_int(2), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    for u in user:
        torch.testing.assert_close(u.float(), orig[0].float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("world", [2, 4])
def test_allgather_and_reduce_scatter_emulated(world):
    torch.manual_seed(1)
    shard = 8 * 300
    emu = Emu(world, world * shard * 2 + shard * 2 + 1024)
    # all-gather: shards live in the arenas
    shards = [emu.buf(r, shard, torch.bfloat16) for r in range(world)]
    for r, s in enumerate(shards):
        s.copy_(torch.full((shard,), float(r + 1), device=DEV))
    fulls = [torch.zeros(world * shard, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    rc = emu.lib.ftb200_team_allgather_emulated(emu.descs(), ctypes.c_int(world), emu.ptrs(shards), emu.ptrs(fulls),
                                                ctypes.c_longlong(shard * 2), ctypes.c_int(2), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    want = torch.cat([torch.full((shard,), float(r + 1)) for r in range(world)]).to(DEV)
    for f in fulls:
        assert torch.equal(f.float(), want)
    # reduce-scatter: full buffers in the arenas
    emu2 = Emu(world, world * shard * 2)
    srcs = [emu2.buf(r, world * shard, torch.bfloat16) for r in range(world)]
    data = [torch.randn(world * shard, device=DEV).bfloat16() for _ in range(world)]
    for s, d in zip(srcs, data):
        s.copy_(d)
    outs = [torch.zeros(shard, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    rc = emu2.lib.ftb200_team_reduce_scatter_emulated(emu2.descs(), ctypes.c_int(world), emu2.ptrs(srcs), emu2.ptrs(outs),
                                                      ctypes.c_longlong(shard), ctypes.c_int(0), ctypes.c_float(1.0),
                                                      ctypes.c_int(2), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    total = sum(d.float() for d in data)
    for r, o in enumerate(outs):
        torch.testing.assert_close(o.float(), total[r * shard : (r + 1) * shard], rtol=2e-2, atol=2e-2)
    assert all(int(s.item()) == 0 for s in emu.status + emu2.status)


def test_missing_peer_times_out_with_status():
    """World of two, only rank 0 is launched: its wait for rank 1's flag must give up after
    the (short) deadline, record TIMEOUT and leave the context usable."""
    world, n = 2, 2 * 8 * 64
    emu = Emu(world, n * 2, timeout_s=0.2)
    bufs = [emu.buf(r, n, torch.bfloat16) for r in range(world)]
    rc = emu.lib.ftb200_team_allreduce_emulated(
        emu.descs(), ctypes.c_int(1), emu.ptrs(bufs), None, None, ctypes.c_longlong(n), ctypes.c_int(0),
        ctypes.c_float(1.0), None, ctypes.c_int(2), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(emu.status[0].item()) == 1  # FTB200_ST_TIMEOUT
    # the device still works
    assert torch.ones(4, device=DEV).sum().item() == 4.0
