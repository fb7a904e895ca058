"""Bus-bandwidth benchmark of the peer-memory collectives against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29544 -m torchft_b200.parallel.bench_team --sizes-mb 1 16 256 1024

One JSON line per (op, size): device-timed (CUDA events, max over ranks) time, algorithm
and bus bandwidth (allreduce: 2(n-1)/n x bytes / t; all-gather and reduce-scatter:
(n-1)/n x bytes / t) and the fraction of 770 GB/s, a measured per-direction NVLink peer-copy
bandwidth of an HGX B200 box.
"""

from __future__ import annotations

import argparse
import json
import os
from datetime import timedelta

import torch
import torch.distributed as dist

from .team import PeerShardComm, ProcessGroupB200

NVLINK_GBS = 770.0


def _time(fn, iters=10, warmup=3):
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[1, 16, 256, 1024])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", type=int, nargs="+", default=[0], help="CTA counts to sweep for the peer kernels (0 = default)")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    es = 2 if dtype == torch.bfloat16 else 4
    max_bytes = int(max(a.sizes_mb) * (1 << 20))

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 77, world, is_master=(rank == 0),
                          wait_for_workers=False)
    pg = ProcessGroupB200(timeout=timedelta(seconds=30), arena_bytes=max_bytes + (1 << 20), device=dev)
    pg.configure(f"127.0.0.1:{store.port}/torchft/1/0", "bench", rank, world)
    comm = PeerShardComm(dist.group.WORLD, dev, arena_bytes=2 * max_bytes + (16 << 20))
    buf = pg.alloc(max_bytes // es, dtype)
    full_peer = comm.alloc(max_bytes // es, dtype, dev)
    full_local = torch.empty(max_bytes // es, dtype=dtype, device=dev)
    buf.normal_()
    full_peer.normal_()

    ms = _time(lambda: comm.team.barrier(), a.iters)
    if rank == 0:
        print(json.dumps({"op": "barrier", "impl": "peer", "world": world, "ms": round(ms, 4)}), flush=True)
    for mb in a.sizes_mb:
        n = int(mb * (1 << 20)) // es // (world * 8) * (world * 8)
        nbytes = n * es
        t = buf[:n]
        xf = torch.randn(n, device=dev)
        idx = torch.randint(0, n, (max(1, n // 1000),), device=dev)
        xf[idx] *= 100.0  # 0.1 % outliers at x100
        x = xf.to(dtype)
        del xf
        rows = []
        off = pg._team.arena.contains(t)
        for c in a.ctas:
            ms = _time(lambda: pg._team.allreduce_(off, n, dtype, 1.0 / world, ctas=c), a.iters)
            rows.append(("allreduce", f"peer(ctas={c})", ms, 2 * (world - 1) / world))
        ms = _time(lambda: (dist.all_reduce(x), x.div_(world)), a.iters)
        rows.append(("allreduce", "nccl+div", ms, 2 * (world - 1) / world))
        if n % (128 * world) == 0 and n * es <= (200 << 20) * 2:
            # block-scaled fp8 on the wire, fused quantise/reduce/dequantise kernel; "bus_gbs" counts the
            # bytes of the unquantised tensor, i.e. the effective bandwidth an unquantised allreduce would need
            xq = x.clone()
            ms = _time(lambda: pg.allreduce_fp8(xq, xq, 1.0 / world), a.iters)
            rows.append(("allreduce", "peer-fp8(effective)", ms, 2 * (world - 1) / world))
            ref = x.float().clone()
            dist.all_reduce(ref)
            ref /= world
            y = x.clone()
            pg.allreduce_fp8(y, y, 1.0 / world)
            torch.cuda.synchronize()
            err = ((y.float() - ref).abs().mean() / ref.abs().mean()).item()
            mx = ((y.float() - ref).abs().max() / ref.abs().max()).item()
            if rank == 0:
                print(json.dumps({"op": "allreduce", "impl": "peer-fp8", "world": world, "mb": mb, "mean_rel_err": round(err, 5),
                                  "max_abs_err_over_max": round(mx, 5)}), flush=True)
        shard = n // world
        sh = full_peer[:shard]
        for c in a.ctas:
            ms = _time(lambda: comm.team.allgather(comm._off(sh), shard * es, full_local[:n], ctas=c), a.iters)
            rows.append(("all_gather", f"peer(ctas={c})", ms, (world - 1) / world))
        xs = x[:shard].clone()
        ms = _time(lambda: dist.all_gather_into_tensor(full_local[:n], xs), a.iters)
        rows.append(("all_gather", "nccl", ms, (world - 1) / world))
        out = torch.empty(shard, dtype=dtype, device=dev)
        for c in a.ctas:
            ms = _time(lambda: comm.team.reduce_scatter(comm._off(full_peer), out, shard, dtype, ctas=c), a.iters)
            rows.append(("reduce_scatter", f"peer(ctas={c})", ms, (world - 1) / world))
        ms = _time(lambda: dist.reduce_scatter_tensor(out, x), a.iters)
        rows.append(("reduce_scatter", "nccl", ms, (world - 1) / world))
        if rank == 0:
            for op, impl, ms, f in rows:
                bus = nbytes * f / ms / 1e6
                print(json.dumps({"op": op, "impl": impl, "world": world, "mb": mb, "dtype": a.dtype, "ms": round(ms, 4),
                                  "bus_gbs": round(bus, 1), "frac_of_measured_nvlink_770": round(bus / NVLINK_GBS, 3)}),
                      flush=True)
    err = pg.errored()
    comm.team.check()
    if rank == 0:
        print(json.dumps({"errored": str(err)}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
