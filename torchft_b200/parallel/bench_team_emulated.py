"""The peer-memory kernels on ONE GPU: all ranks of a team emulated by one cooperative launch.

Kernels that wait on one another must not run as separate launches on one GPU, so each collective here is a single
cooperative launch whose blocks are the blocks of all ranks (``blockIdx.y`` is the rank) over arenas that all live on
this GPU.  Nothing crosses NVLink: the figures say what the kernels cost in instructions and local memory traffic
(and give ``ncu`` a single-GPU target for them), not what the links deliver -- that is ``bench_team.py`` and
``bench_quant_sweep.py`` on real ranks.

    python -m torchft_b200.parallel.bench_team_emulated [--world 4] [--mb 64] [--ctas 32]

Prints one JSON line per kernel: the two-shot allreduce (bf16), the fused fp8 allreduce (fp32 in and out) and the
segment-table copy kernel of the live-recovery transport.
"""

from __future__ import annotations

import argparse
import ctypes
import json

import torch

from .. import quantization as Q
from ..ops import _native as N
from .team import MAX_RANKS, _TeamDesc


class EmulatedTeam:
    """Arenas, flag words, local sync words and status words of ``world`` ranks on the current GPU."""

    def __init__(self, world: int, nbytes: int, timeout_s: float = 1.0, epoch: int = 7) -> None:
        self.lib = N.lib()
        self.world = world
        fb = int(self.lib.ftb200_team_flag_bytes())
        self.fb = (fb + 255) // 256 * 256
        self.arenas = [torch.zeros(self.fb + nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        self.sync = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
        self.status = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(world)]
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch, self.seq = epoch, 0

    def descs(self):
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

    def payload(self, r: int) -> torch.Tensor:
        return self.arenas[r][self.fb:]

    @staticmethod
    def ptrs(tensors):
        arr = (ctypes.c_void_p * MAX_RANKS)()
        for i, t in enumerate(tensors):
            arr[i] = t.data_ptr()
        return arr

    def check(self) -> None:
        torch.cuda.synchronize()
        bad = [int(s.item()) for s in self.status]
        if any(bad):
            raise RuntimeError(f"emulated team ended with status {bad}")


def _time(fn, iters: int) -> float:
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--mb", type=float, default=64.0, help="payload per rank in MB")
    ap.add_argument("--ctas", type=int, default=32, help="blocks per emulated rank (world x ctas must fit the GPU)")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    W = a.world
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if W * a.ctas > sms:
        raise SystemExit(f"{W} ranks x {a.ctas} blocks do not fit {sms} SMs in one cooperative launch")
    lib = N.lib()

    # ---- two-shot allreduce, bf16, in place in the arenas
    n = int(a.mb * (1 << 20)) // 2 // (W * 8) * (W * 8)
    team = EmulatedTeam(W, n * 2)
    bufs = [team.payload(r)[: n * 2].view(torch.bfloat16) for r in range(W)]
    for r, b in enumerate(bufs):
        b.copy_(torch.randn(n, device="cuda").bfloat16())

    def allreduce() -> None:
        N.check(lib.ftb200_team_allreduce_emulated(team.descs(), ctypes.c_int(W), team.ptrs(bufs), None, None,
                                                   ctypes.c_longlong(n), ctypes.c_int(0), ctypes.c_float(1.0 / W), None,
                                                   ctypes.c_int(a.ctas), N.stream_ptr()), "allreduce_emulated", 0)

    ms = _time(allreduce, a.iters)
    team.check()
    print(json.dumps({"kernel": "allreduce_emul_kernel<bf16>", "world": W, "mb_per_rank": n * 2 / 2**20, "ms": round(ms, 4),
                      "note": "includes the launcher's staging of the descriptors and its stream sync"}), flush=True)

    # ---- fused fp8 allreduce, fp32 in and out
    m = int(a.mb * (1 << 20)) // 4 // (W * Q.BLOCK) * (W * Q.BLOCK)
    team8 = EmulatedTeam(W, Q.quantized_nbytes(m) + 256)
    arenas = [team8.payload(r) for r in range(W)]
    ins = [torch.randn(m, device="cuda") for _ in range(W)]
    outs = [torch.empty(m, device="cuda") for _ in range(W)]

    def allreduce_fp8() -> None:
        N.check(lib.ftb200_team_allreduce_fp8_emulated(team8.descs(), ctypes.c_int(W), team8.ptrs(arenas), team8.ptrs(ins),
                                                       None, team8.ptrs(outs), ctypes.c_longlong(m), ctypes.c_int(1),
                                                       ctypes.c_float(1.0 / W), ctypes.c_int(a.ctas), N.stream_ptr()),
                "allreduce_fp8_emulated", 0)

    ms = _time(allreduce_fp8, a.iters)
    team8.check()
    want = sum(ins) / W
    err = float(((outs[0] - want).abs().mean() / want.abs().mean()).item())
    print(json.dumps({"kernel": "allreduce_fp8_emul_kernel<float>", "world": W, "mb_per_rank": m * 4 / 2**20,
                      "ms": round(ms, 4), "mean_rel_err": round(err, 5)}), flush=True)

    # ---- segment-table copy (live recovery), local source and destination
    from ..checkpointing.p2p_transport import _seg_table

    nb = int(a.mb * (1 << 20)) * W // 16 * 16
    src = torch.randint(0, 255, (nb,), dtype=torch.uint8, device="cuda")
    dst = torch.empty_like(src)
    third = nb // 3 // 16 * 16
    segs = [(src.data_ptr(), dst.data_ptr(), third), (src.data_ptr() + third, dst.data_ptr() + third, third),
            (src.data_ptr() + 2 * third, dst.data_ptr() + 2 * third, nb - 2 * third)]
    table = _seg_table(segs, torch.device("cuda"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sums = torch.zeros(len(segs), dtype=torch.int64, device="cuda")

    def copy() -> None:
        sums.zero_()
        N.check(lib.ftb200_p2p_copy_checked(N.ptr(table), ctypes.c_int(len(segs)), ctypes.c_longlong(nb), None, N.ptr(status),
                                            ctypes.c_ulonglong(int(5e9)), N.ptr(sums), ctypes.c_int(0), N.stream_ptr()),
                "p2p_copy", 0)

    ms = _time(copy, a.iters)
    ok = bool(torch.equal(src, dst)) and int(status.item()) == 0
    print(json.dumps({"kernel": "p2p_copy_kernel", "mb": nb / 2**20, "ms": round(ms, 4),
                      "gbs_read_plus_write": round(2 * nb / ms / 1e6, 1), "copied_ok": ok}), flush=True)


if __name__ == "__main__":
    main()
