"""Quantised-allreduce sweep: fp32 and bf16 tensors of 1 MB to 4 GB, N(0,1) with 0.1 % outliers at
x100, averaged over the ranks of one NVSwitch box with

* ``peer``      the peer-memory allreduce of :class:`~torchft_b200.parallel.team.ProcessGroupB200` in the
                tensor's own dtype (in place in the arena),
* ``peer-fp8``  its fused block-scaled fp8 allreduce (e4m3, 128-element blocks, fp32 scales),
* ``nccl``      ``dist.all_reduce`` + divide in the tensor's own dtype,
* ``ref-fp8``   the reference's quantised allreduce, unmodified (``torchft/quantization.py`` Triton kernels
                through ``torchft/collectives.py:297-415``, loaded by file path from ``baseline/_ref``) on a plain
                NCCL group, with the tensor shaped ``[n/4096, 4096]`` like a parameter matrix, and (up to 16 MB)
                as the flat 1-D bucket that the reference's bucketised DiLoCo path passes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29544 -m torchft_b200.parallel.bench_quant_sweep

One JSON line per (dtype, size, method): device time (CUDA events, max over ranks), bus bandwidth
``2(n-1)/n x bytes_of_the_unquantised_tensor / t`` (for the fp8 methods that is the *effective* bandwidth an
unquantised allreduce would need), and the error against the fp32 reduction of the same inputs:
``max_err`` = max |x - ref| / max |ref| and ``mean_rel_err`` = mean |x - ref| / mean |ref| (the reference's
test metric).
"""

from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import types
from datetime import timedelta

import torch
import torch.distributed as dist

from .team import ProcessGroupB200

NVLINK_GBS = 770.0


def _time(fn, iters, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def _load_reference_quantized_allreduce():
    """``torchft.collectives.allreduce_quantized`` of the reference, without importing the reference package's
    ``__init__`` (which needs its native extension): a bare package object whose path is the reference folder."""
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline", "_ref", "torchft")
    if not os.path.isfile(os.path.join(root, "collectives.py")):
        return None, f"{root} not found"
    try:
        if "torchft" not in sys.modules:
            pkg = types.ModuleType("torchft")
            pkg.__path__ = [root]  # type: ignore[attr-defined]
            sys.modules["torchft"] = pkg
        return importlib.import_module("torchft.collectives").allreduce_quantized, None
    except Exception as e:  # noqa: BLE001 - triton missing or incompatible: the row is reported as unavailable
        return None, f"{type(e).__name__}: {e}"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[1, 4, 16, 64, 256, 1024, 4096])
    ap.add_argument("--dtypes", nargs="+", default=["bf16", "fp32"], choices=["bf16", "fp32"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--no-reference", action="store_true")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    max_bytes = int(max(a.sizes_mb) * (1 << 20))
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 79, world, is_master=(rank == 0),
                          wait_for_workers=False)
    pg = ProcessGroupB200(timeout=timedelta(seconds=60), arena_bytes=max_bytes + (1 << 20), device=dev)
    pg.configure(f"127.0.0.1:{store.port}/torchft/1/0", "sweep", rank, world)
    ref_fn, ref_why = (None, "disabled") if a.no_reference else _load_reference_quantized_allreduce()
    if rank == 0 and ref_fn is None:
        print(json.dumps({"method": "ref-fp8", "unavailable": ref_why}), flush=True)
    factor = 2 * (world - 1) / world

    def emit(dtype_name, mb, method, ms, got, ref, nbytes, note=None):
        err = (got.float() - ref).abs()
        mx = (err.max() / ref.abs().max()).item()
        mean = (err.mean() / ref.abs().mean()).item()
        if rank == 0:
            bus = nbytes * factor / ms / 1e6
            row = {"dtype": dtype_name, "mb": mb, "world": world, "method": method, "ms": round(ms, 4),
                   "bus_gbs": round(bus, 1), "frac_of_measured_nvlink_770": round(bus / NVLINK_GBS, 3),
                   "max_err": round(mx, 5), "mean_rel_err": round(mean, 5)}
            if note:
                row["note"] = note
            print(json.dumps(row), flush=True)

    arena_bytes = pg.alloc(max_bytes, torch.uint8)
    for dtype_name in a.dtypes:
        dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
        es = 2 if dtype == torch.bfloat16 else 4
        arena_buf = arena_bytes.view(dtype)
        for mb in a.sizes_mb:
            n = int(mb * (1 << 20)) // es // (world * 4096) * (world * 4096)
            nbytes = n * es
            g = torch.Generator(device=dev).manual_seed(1000 * rank + int(mb))
            xf = torch.randn(n, device=dev, generator=g)
            idx = torch.randint(0, n, (max(1, n // 1000),), device=dev, generator=g)
            xf[idx] *= 100.0  # 0.1 % outliers at x100
            x = xf.to(dtype)
            del xf, idx
            ref = x.float()
            dist.all_reduce(ref)
            ref /= world  # the fp32 reduction of exactly these inputs

            t = arena_buf[:n]
            off = pg._team.arena.contains(t)
            t.copy_(x)
            pg._team.allreduce_(off, n, dtype, 1.0 / world)
            got = t.clone()
            ms = _time(lambda: pg._team.allreduce_(off, n, dtype, 1.0 / world), a.iters)
            emit(dtype_name, mb, "peer", ms, got, ref, nbytes)

            y = x.clone()
            dist.all_reduce(y)
            y.div_(world)
            ms = _time(lambda: (dist.all_reduce(y), y.div_(world)), a.iters)
            y.copy_(x)
            dist.all_reduce(y)
            y.div_(world)
            emit(dtype_name, mb, "nccl", ms, y, ref, nbytes)

            y.copy_(x)
            pg.allreduce_fp8(y, y, 1.0 / world)
            got = y.clone()
            ms = _time(lambda: pg.allreduce_fp8(y, y, 1.0 / world), a.iters)
            emit(dtype_name, mb, "peer-fp8", ms, got, ref, nbytes, "effective bandwidth")
            K_err = pg.errored()
            if K_err is not None:
                raise SystemExit(f"peer group errored: {K_err}")

            # The reference's Triton kernels index with 32-bit offsets: at 4 GB (bf16: 2^31 elements) they made
            # an illegal memory access on a B200 (Triton 3.6), so they are run up to 1 GB only.
            if ref_fn is not None and nbytes <= (1 << 30):
                shapes = [("ref-fp8 [n/4096, 4096]", (n // 4096, 4096))]
                if mb <= 16:
                    shapes.append(("ref-fp8 flat 1-D bucket", (n,)))
                for name, shape in shapes:
                    try:
                        z = x.clone().view(*shape)
                        stream = torch.cuda.current_stream()
                        ref_fn([z], dist.ReduceOp.AVG, dist.group.WORLD, stream).wait()
                        got = z.reshape(-1).clone()

                        def run():
                            ref_fn([z], dist.ReduceOp.AVG, dist.group.WORLD, stream).wait()

                        ms = _time(run, max(2, a.iters // 2), warmup=1)
                        emit(dtype_name, mb, name, ms, got, ref, nbytes, "effective bandwidth; reference Triton kernels + NCCL")
                    except Exception as e:  # noqa: BLE001
                        if rank == 0:
                            print(json.dumps({"dtype": dtype_name, "mb": mb, "method": name,
                                              "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}), flush=True)
            del x, y, ref, got
            torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps({"errored": str(pg.errored())}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
