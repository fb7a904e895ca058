"""Checkpoint-transport benchmark: time one ``send_checkpoint`` / ``recv_checkpoint`` pair of a
synthetic state dict over each transport.

    python -m torchft_b200.checkpointing.bench_transports --transport http --total-mb 12000 --chunk-mb 3
    python -m torchft_b200.checkpointing.bench_transports --transport http --num-chunks 8 --device cuda
    python -m torchft_b200.checkpointing.bench_transports --transport pg --device cuda      # 2 GPUs, NCCL
    python -m torchft_b200.checkpointing.bench_transports --transport p2p                   # 2 GPUs, peer memory

The state dict is ``total / chunk`` fp32 tensors of ``chunk`` megabytes, the shape the
reference's harnesses use (torchft/checkpointing/http_transport_bench.py:19-51,
pg_transport_bench.py:21-89: 12 GB of 3 MB tensors).  ``http`` runs sender and receiver in
one process; ``pg`` and ``p2p`` spawn a second process on the next GPU (gloo on CPU for
``pg --device cpu``).  Prints one JSON line with wall-clock seconds and GB/s.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from datetime import timedelta

import torch
import torch.multiprocessing as mp


def _state(total_mb: float, chunk_mb: float, device: torch.device):
    n = max(1, int(total_mb / chunk_mb))
    numel = int(chunk_mb * 1e6 / 4)
    return {f"t{i}": torch.full((numel,), float(i), dtype=torch.float32, device=device) for i in range(n)}


def _nbytes(sd) -> int:
    return sum(t.numel() * t.element_size() for t in sd.values())


def bench_http(a) -> dict:
    from .http_transport import HTTPTransport

    dev = torch.device(a.device)
    sd = _state(a.total_mb, a.chunk_mb, dev)
    timeout = timedelta(seconds=a.timeout)
    send = HTTPTransport(timeout, num_chunks=a.num_chunks)
    dst = _state(a.total_mb, a.chunk_mb, dev) if a.inplace else None
    recv = HTTPTransport(timeout, num_chunks=a.num_chunks, state_dict=(lambda: dst) if a.inplace else None)
    try:
        t0 = time.perf_counter()
        send.send_checkpoint([1], step=1, state_dict=sd, timeout=timeout)
        t1 = time.perf_counter()
        got = recv.recv_checkpoint(0, send.metadata(), 1, timeout)
        t2 = time.perf_counter()
        assert float(got[f"t{len(sd) - 1}"][0]) == float(len(sd) - 1)
    finally:
        send.shutdown()
        recv.shutdown()
    b = _nbytes(sd)
    return {"transport": "http", "num_chunks": a.num_chunks, "device": a.device, "inplace": a.inplace, "gb": b / 1e9, "stage_s": t1 - t0,
            "recv_s": t2 - t1, "recv_gbs": b / 1e9 / (t2 - t1)}


def _pair_worker(rank: int, a, port: int, q) -> None:
    dev = torch.device("cuda", rank) if a.device == "cuda" else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    timeout = timedelta(seconds=a.timeout)
    store_addr = f"127.0.0.1:{port}/bench"
    sd = _state(a.total_mb, a.chunk_mb, dev)
    if a.transport == "pg":
        from ..process_group import ProcessGroupGloo, ProcessGroupNCCL
        from .pg_transport import PGTransport

        pg = ProcessGroupNCCL(timeout=timeout) if dev.type == "cuda" else ProcessGroupGloo(timeout=timeout)
        pg.configure(store_addr, "bench", rank, 2)
        tr = PGTransport(pg, timeout, dev, state_dict=(lambda: sd) if a.inplace else None)
        meta = tr.metadata()
    else:
        from .p2p_transport import P2PTransport

        tr = P2PTransport(timeout, dev, state_dict=(lambda: sd) if a.inplace else None)
        meta = None
    store = torch.distributed.TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    if rank == 0:
        t0 = time.perf_counter()
        if a.transport == "p2p":
            tr.send_checkpoint([1], 1, sd, timeout)
            store.set("meta", tr.metadata())
            store.get("done")  # the receiver has pulled everything
        else:
            store.set("meta", meta)
            tr.send_checkpoint([1], 1, sd, timeout)
        q.put(("send_s", time.perf_counter() - t0))
    else:
        meta = store.get("meta").decode()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        got = tr.recv_checkpoint(0, meta, 1, timeout)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert float(got[f"t{len(sd) - 1}"][0]) == float(len(sd) - 1)
        store.set("done", "1")
        extra = getattr(tr, "last_recv", {})
        q.put(("recv", {"recv_s": dt, "gb": _nbytes(sd) / 1e9, "recv_gbs": _nbytes(sd) / 1e9 / dt,
                        **({"copy_kernel_gbs": extra["bytes"] / 1e6 / extra["copy_ms"]} if extra.get("copy_ms") else {})}))
    if a.transport == "pg":
        pg.shutdown()
    tr.shutdown(wait=False) if hasattr(tr, "shutdown") else None


def bench_pair(a) -> dict:
    store = torch.distributed.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pair_worker, args=(r, a, store.port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = {"transport": a.transport, "device": a.device, "inplace": a.inplace}
    for _ in range(2):
        k, v = q.get(timeout=a.timeout + 60)
        if k == "recv":
            out.update(v)
        else:
            out[k] = v
    for p in procs:
        p.join(30)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", default="http", choices=["http", "pg", "p2p"])
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--total-mb", type=float, default=12000.0)
    ap.add_argument("--chunk-mb", type=float, default=3.0)
    ap.add_argument("--num-chunks", type=int, default=0, help="http: parallel chunk streams (0 = one stream)")
    ap.add_argument("--inplace", action="store_true", help="receive into existing tensors")
    ap.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args()
    if a.transport == "p2p":
        a.device = "cuda"
    res = bench_http(a) if a.transport == "http" else bench_pair(a)
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
