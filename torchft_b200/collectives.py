"""Quantised collectives: allreduce and reduce-scatter that move block-scaled fp8 instead
of the tensors' own dtype (about half the bytes of bf16, a quarter of fp32).

Two implementations behind one API (that of torchft/collectives.py:159-415):

* any process group with ``alltoall_base`` and ``allgather_into_tensor_coalesced``:
  quantise -> all-to-all (every rank receives its slice from everybody) -> local fp32
  reduce + requantise -> all-gather -> dequantise;
* :class:`~torchft_b200.parallel.team.ProcessGroupB200`: one fused kernel per rank that
  quantises into the peer-visible arena, reduces its slice straight out of the peers'
  arenas and writes the requantised slice back into them.

Only ``SUM`` and ``AVG`` are meaningful for quantised data.
"""

from __future__ import annotations

from typing import List, Optional

import torch
from torch.distributed.distributed_c10d import AllgatherOptions, AllToAllOptions, ReduceOp, Work

from . import quantization as Q
from .work import _DummyWork


def _check_op(op) -> None:
    if op not in (ReduceOp.SUM, ReduceOp.AVG):
        raise NotImplementedError(f"quantised collectives support SUM and AVG, got {op}")


def get_padded_sizes(tensors: List[torch.Tensor], world_size: int) -> int:
    """Total element count of ``tensors`` padded so each rank's slice is whole 128-blocks."""
    return Q.padded_numel(sum(t.numel() for t in tensors), world_size)


class _StreamOrderedWork(Work):
    """Completion = the side stream reached ``event``; ``wait`` orders the caller's stream."""

    def __init__(self, event: Optional["torch.cuda.Event"], result: object) -> None:
        super().__init__()
        self._event, self._result = event, result
        self._fut: torch.futures.Future = torch.futures.Future()
        self._fut.set_result(result)

    def wait(self, timeout=None) -> bool:
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)
        return True

    def synchronize(self) -> None:
        if self._event is not None:
            self._event.synchronize()

    def block_current_stream(self, timeout=None) -> None:
        self.wait()

    def is_completed(self) -> bool:
        return self._event is None or self._event.query()

    def get_future(self) -> torch.futures.Future:
        return self._fut


def _flatten(tensors: List[torch.Tensor], n: int) -> torch.Tensor:
    flat = torch.zeros(n, dtype=tensors[0].dtype, device=tensors[0].device)
    off = 0
    for t in tensors:
        flat[off : off + t.numel()].copy_(t.reshape(-1))
        off += t.numel()
    return flat


def _unflatten(flat: torch.Tensor, tensors: List[torch.Tensor]) -> None:
    off = 0
    for t in tensors:
        t.copy_(flat[off : off + t.numel()].view_as(t))
        off += t.numel()


def _exchange_and_reduce(flat: torch.Tensor, n: int, ws: int, rank: int, scale: float, pg) -> torch.Tensor:
    """Quantise ``flat``, all-to-all the slices, reduce this rank's slice; returns the
    quantised reduced slice (``n/ws`` elements)."""
    dev = flat.device
    per = n // ws
    qbuf = torch.empty(Q.quantized_nbytes(n), dtype=torch.uint8, device=dev)
    Q.quantize_into(flat, qbuf)
    codes, scales = Q.split_quantized(qbuf, n)
    rcodes = torch.empty_like(codes)
    rscales = torch.empty_like(scales)
    pg.alltoall_base(rcodes, codes, [], [], AllToAllOptions()).wait()
    pg.alltoall_base(rscales, scales, [], [], AllToAllOptions()).wait()
    # rebuild one quantised buffer per source rank for my slice, reduce in a fixed order starting at my own
    parts = []
    for k in range(ws):
        p = (rank + k) % ws
        b = torch.empty(Q.quantized_nbytes(per), dtype=torch.uint8, device=dev)
        c, s = Q.split_quantized(b, per)
        c.copy_(rcodes[p * per : (p + 1) * per])
        s.copy_(rscales[p * (per // Q.BLOCK) : (p + 1) * (per // Q.BLOCK)])
        parts.append(b)
    out = torch.empty(Q.quantized_nbytes(per), dtype=torch.uint8, device=dev)
    Q.reduce_quantized(parts, per, scale, out)
    return out


def allreduce_quantized(tensors: List[torch.Tensor], opts, pg, sync_stream: Optional["torch.cuda.Stream"] = None) -> Work:
    """Allreduce ``tensors`` in place through fp8.  ``opts`` is a ``ReduceOp`` (SUM or AVG)
    or an options object carrying one.  On CUDA the work runs on ``sync_stream`` (a fresh
    side stream when None) and the returned work orders the caller's stream behind it."""
    op = opts if isinstance(opts, (ReduceOp, ReduceOp.RedOpType)) else opts.reduceOp
    _check_op(op)
    if not tensors:
        return _DummyWork(tensors)
    ws, rank = pg.size(), pg.rank() if hasattr(pg, "rank") else 0
    rank = getattr(pg, "_rank", rank)
    dev = tensors[0].device
    scale = 1.0 / ws if op == ReduceOp.AVG else 1.0
    n = get_padded_sizes(tensors, ws)

    def body() -> None:
        if hasattr(pg, "allreduce_fp8"):
            if len(tensors) == 1 and tensors[0].is_contiguous() and tensors[0].numel() == n:
                pg.allreduce_fp8(tensors[0].view(-1), tensors[0].view(-1), scale)
            else:
                flat = _flatten(tensors, n)
                pg.allreduce_fp8(flat, flat, scale)
                _unflatten(flat, tensors)
            return
        flat = _flatten(tensors, n)
        reduced = _exchange_and_reduce(flat, n, ws, rank, scale, pg)
        per = n // ws
        rc, rs = Q.split_quantized(reduced, per)
        full = torch.empty(Q.quantized_nbytes(n), dtype=torch.uint8, device=dev)
        fc, fs = Q.split_quantized(full, n)
        pg.allgather_into_tensor_coalesced([fc], [rc.contiguous()], AllgatherOptions()).wait()
        pg.allgather_into_tensor_coalesced([fs.view(torch.uint8)], [rs.contiguous().view(torch.uint8)], AllgatherOptions()).wait()
        Q.dequantize_from(full, flat)
        _unflatten(flat, tensors)

    if dev.type != "cuda":
        body()
        return _DummyWork(tensors)
    stream = sync_stream if sync_stream is not None else torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        body()
        ev = torch.cuda.Event()
        ev.record(stream)
    for t in tensors:
        t.record_stream(stream)
    return _StreamOrderedWork(ev, tensors)


def allocate_reduce_scatter_output(tensors: List[torch.Tensor], world_size: int) -> tuple:
    """Flat output tensor for :func:`reduce_scatter_quantized` (this rank's slice) and the
    padded total size."""
    n = get_padded_sizes(tensors, world_size)
    return torch.empty(n // world_size, dtype=tensors[0].dtype, device=tensors[0].device), n


def reduce_scatter_quantized(output: torch.Tensor, inputs: List[torch.Tensor], opts, pg,
                             sync_stream: Optional["torch.cuda.Stream"] = None) -> Work:
    """``output`` (flat, ``padded_total / world`` elements) receives this rank's slice of
    the reduction of ``inputs`` (viewed as one flat, padded vector), moved as fp8."""
    op = opts if isinstance(opts, (ReduceOp, ReduceOp.RedOpType)) else opts.reduceOp
    _check_op(op)
    ws = pg.size()
    rank = getattr(pg, "_rank", pg.rank() if hasattr(pg, "rank") else 0)
    n = get_padded_sizes(inputs, ws)
    if output.numel() != n // ws:
        raise ValueError(f"output must have {n // ws} elements, got {output.numel()}")
    scale = 1.0 / ws if op == ReduceOp.AVG else 1.0
    dev = inputs[0].device

    def body() -> None:
        flat = _flatten(inputs, n)
        reduced = _exchange_and_reduce(flat, n, ws, rank, scale, pg)
        Q.dequantize_from(reduced, output.view(-1))

    if dev.type != "cuda":
        body()
        return _DummyWork(output)
    stream = sync_stream if sync_stream is not None else torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        body()
        ev = torch.cuda.Event()
        ev.record(stream)
    return _StreamOrderedWork(ev, output)
