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


def test_missing_peer_with_abort_word_returns_aborted():
    """The other half of the never-hang contract: with the abort word set, a rank whose peer never
    shows up must come back ABORTED long before its (here: 20 s) deadline."""
    import time

    world, n = 2, 2 * 8 * 64
    emu = Emu(world, n * 2, timeout_s=20.0)
    lib = emu.lib
    hp, dp = ctypes.POINTER(ctypes.c_int)(), ctypes.c_void_p()
    assert lib.ftb200_abort_word_create(ctypes.byref(hp), ctypes.byref(dp)) == 0
    try:
        hp[0] = 1  # aborted before the launch
        descs = emu.descs()
        descs[0].abort_word = dp.value
        bufs = [emu.buf(r, n, torch.bfloat16) for r in range(world)]
        t0 = time.perf_counter()
        rc = lib.ftb200_team_allreduce_emulated(
            descs, ctypes.c_int(1), emu.ptrs(bufs), None, None, ctypes.c_longlong(n), ctypes.c_int(0),
            ctypes.c_float(1.0), None, ctypes.c_int(2), N.stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 5.0
        assert int(emu.status[0].item()) == 2  # FTB200_ST_ABORTED
        assert torch.ones(4, device=DEV).sum().item() == 4.0
    finally:
        lib.ftb200_abort_word_destroy(hp)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_allreduce_oneshot_emulated(world, dtype):
    torch.manual_seed(2)
    n = 8 * 700
    emu = Emu(world, n * 4)
    window = [emu.buf(r, n, dtype) for r in range(world)]
    data = [torch.randn(n, device=DEV).to(dtype) for _ in range(world)]
    outs = [torch.empty(n, dtype=dtype, device=DEV) for _ in range(world)]
    ref = sum(d.float() for d in data) / world
    rc = emu.lib.ftb200_team_allreduce_oneshot_emulated(
        emu.descs(), ctypes.c_int(world), emu.ptrs(window), emu.ptrs(data), emu.ptrs(outs), ctypes.c_longlong(n),
        ctypes.c_int(0 if dtype == torch.bfloat16 else 1), ctypes.c_float(1.0 / world), ctypes.c_int(2), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert all(int(s.item()) == 0 for s in emu.status)
    for o in outs:
        assert torch.equal(o, outs[0])  # same summation order on every rank
        torch.testing.assert_close(o.float(), ref, rtol=2e-2, atol=2e-2)


def _pull_tables(world, rows):
    """rows[r] = list of (src_ptr, dst_ptr, nbytes) for rank r -> flat ctypes tables."""
    src = (ctypes.c_void_p * (world * MAX_RANKS))()
    dst = (ctypes.c_void_p * (world * MAX_RANKS))()
    nb = (ctypes.c_longlong * (world * MAX_RANKS))()
    cnt = (ctypes.c_int * world)()
    for r, segs in enumerate(rows):
        cnt[r] = len(segs)
        for i, (s, d, b) in enumerate(segs):
            src[r * MAX_RANKS + i], dst[r * MAX_RANKS + i], nb[r * MAX_RANKS + i] = s, d, b
    return src, dst, nb, cnt


def test_pull_emulated_alltoall_and_broadcast():
    world, chunk = 4, 16 * 50
    emu = Emu(world, world * chunk)
    stage = [emu.buf(r, world * chunk, torch.uint8) for r in range(world)]
    for r, s in enumerate(stage):
        s.copy_(torch.arange(world * chunk, device=DEV).remainder(251).add(r).to(torch.uint8))
    outs = [torch.zeros(world * chunk, dtype=torch.uint8, device=DEV) for _ in range(world)]
    # all-to-all: rank r takes chunk r of every rank's window
    rows = [[(stage[p].data_ptr() + r * chunk, outs[r].data_ptr() + p * chunk, chunk) for p in range(world)]
            for r in range(world)]
    src, dst, nb, cnt = _pull_tables(world, rows)
    assert emu.lib.ftb200_team_pull_emulated(emu.descs(), ctypes.c_int(world), src, dst, nb, cnt, ctypes.c_int(2),
                                             N.stream_ptr()) == 0
    torch.cuda.synchronize()
    for r in range(world):
        for p in range(world):
            assert torch.equal(outs[r][p * chunk : (p + 1) * chunk], stage[p][r * chunk : (r + 1) * chunk])
    # broadcast from rank 2: the root fetches nothing
    outs = [torch.zeros(chunk, dtype=torch.uint8, device=DEV) for _ in range(world)]
    rows = [[] if r == 2 else [(stage[2].data_ptr(), outs[r].data_ptr(), chunk)] for r in range(world)]
    src, dst, nb, cnt = _pull_tables(world, rows)
    assert emu.lib.ftb200_team_pull_emulated(emu.descs(), ctypes.c_int(world), src, dst, nb, cnt, ctypes.c_int(2),
                                             N.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert all(int(s.item()) == 0 for s in emu.status)
    for r in range(world):
        if r != 2:
            assert torch.equal(outs[r], stage[2][:chunk])


def test_sendrecv_emulated_and_receiver_alone_times_out():
    world, nbytes = 4, 16 * 1000
    emu = Emu(world, nbytes, timeout_s=0.3)
    window = emu.buf(1, nbytes, torch.uint8)  # rank 1 sends to rank 3
    window.copy_(torch.arange(nbytes, device=DEV).remainder(253).to(torch.uint8))
    dst = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    descs = emu.descs()
    token = (emu.epoch << 32) | 1
    rc = emu.lib.ftb200_team_sendrecv_emulated(ctypes.byref(descs[1]), ctypes.byref(descs[3]), ctypes.c_int(1),
                                               ctypes.c_ulonglong(token), ctypes.c_void_p(window.data_ptr()),
                                               ctypes.c_void_p(dst.data_ptr()), ctypes.c_longlong(nbytes), ctypes.c_int(2),
                                               N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dst, window) and int(emu.status[1].item()) == 0 and int(emu.status[3].item()) == 0
    # a receiver whose sender never posts gives up with TIMEOUT and leaves the destination alone
    dst.zero_()
    token = (emu.epoch << 32) | 2
    rc = emu.lib.ftb200_team_sendrecv_emulated(ctypes.byref(descs[1]), ctypes.byref(descs[3]), ctypes.c_int(0),
                                               ctypes.c_ulonglong(token), ctypes.c_void_p(window.data_ptr()),
                                               ctypes.c_void_p(dst.data_ptr()), ctypes.c_longlong(nbytes), ctypes.c_int(2),
                                               N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(emu.status[3].item()) == 1 and int(dst.sum().item()) == 0
    assert torch.ones(4, device=DEV).sum().item() == 4.0


def test_a_peer_that_is_already_one_call_ahead_does_not_stall_the_round():
    """Tokens of a team only grow and every flag word has one writer, so a word that already holds a later token of
    the same epoch proves that the awaited one was posted (a peer may overwrite it when a single-round collective is
    followed at once by the next one).  A later token passes; a token of another epoch does not."""
    world, n = 2, 2 * 8 * 64

    def run(peer_token_of):
        emu = Emu(world, n * 2, timeout_s=0.2)
        bufs = [emu.buf(r, n, torch.bfloat16) for r in range(world)]
        for b in bufs:
            b.fill_(1.0)
        descs = emu.descs()
        words = emu.arenas[0][: emu.fb].view(torch.int64)
        for slot in (0, 1):  # what rank 1 would have written into rank 0's ready and done words
            words[slot * MAX_RANKS + 1] = peer_token_of(int(descs[0].token))
        rc = emu.lib.ftb200_team_allreduce_emulated(
            descs, ctypes.c_int(1), emu.ptrs(bufs), None, None, ctypes.c_longlong(n), ctypes.c_int(0),
            ctypes.c_float(1.0), None, ctypes.c_int(2), N.stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        return int(emu.status[0].item())

    assert run(lambda tok: tok) == 0          # the awaited token itself
    assert run(lambda tok: tok + 3) == 0      # the peer is three calls further on in the same epoch
    assert run(lambda tok: tok - 1) == 1      # an earlier call: TIMEOUT
    assert run(lambda tok: tok + (1 << 32)) == 1  # another epoch: never matches
