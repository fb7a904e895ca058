"""Live-recovery transport over NVLink peer memory.

The healthy replica does not copy anything: it publishes, over the small HTTP channel of
:class:`~torchft_b200.checkpointing.http_transport.HTTPTransport`, a state dict in which
every CUDA tensor is replaced by a reference (CUDA IPC handle of the allocation, offset,
shape, dtype).  The healing replica maps those allocations and *pulls* all tensors with
one grid-stride copy kernel straight into its own live tensors (when given an in-place
state dict) or into fresh ones -- the bytes cross NVLink once and never touch the host.
Pulling means a source that goes away cannot block the healer: every few tens of megabytes
the copy kernel looks at this transport's abort word (:meth:`P2PTransport.abort`, also set by
``shutdown``) and at a deadline (the ``timeout`` of ``recv_checkpoint``), gives up with a status
that ``recv_checkpoint`` raises, and the transfer is retried at the next quorum.  The source
publishes a checksum of every tensor's bytes; the copy kernel computes the same sum over what it
moved and ``recv_checkpoint`` raises on a mismatch.

The source's tensors must stay unmodified until the step commits; the manager guarantees
that (the optimizer only runs after the step's allreduce, which the healing replica joins
after its transfer).  Non-CUDA leaves travel inside the HTTP payload.  Same-host GPUs
only; use ``HTTPTransport`` across hosts.  Replaces the payload path of
torchft/checkpointing/http_transport.py and pg_transport.py.
"""

from __future__ import annotations

import ctypes
import time
import logging
from dataclasses import dataclass
from datetime import timedelta
from typing import Callable, Dict, Generic, List, Optional, Tuple, TypeVar

import torch
from torch.utils._pytree import tree_flatten, tree_unflatten

from ..ops import _native as N
from .http_transport import HTTPTransport

logger = logging.getLogger(__name__)
T = TypeVar("T")


@dataclass
class _PeerTensorRef:
    handle: bytes
    offset: int
    nbytes: int
    shape: Tuple[int, ...]
    dtype: torch.dtype
    checksum: Optional[int] = None  # 64-bit sum of the 32-bit words of the 16-byte-aligned bulk; None: not checked


class _CopySeg(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("bytes", ctypes.c_longlong)]


def _seg_table(segs: List[Tuple[int, int, int]], device: torch.device) -> torch.Tensor:
    table = (_CopySeg * len(segs))()
    for i, (src, dst, nb) in enumerate(segs):
        table[i].src, table[i].dst, table[i].bytes = src, dst, nb
    return torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8).to(device)


def _checksums(tensors: List[torch.Tensor], device: torch.device) -> List[Optional[int]]:
    """Per-tensor checksum of the bytes a receiver's copy kernel will move (the 16-byte-aligned bulk)."""
    idx, segs = [], []
    for i, t in enumerate(tensors):
        nb = t.numel() * t.element_size() // 16 * 16
        if nb and t.data_ptr() % 16 == 0:
            idx.append(i)
            segs.append((t.data_ptr(), 0, nb))
    out: List[Optional[int]] = [None] * len(tensors)
    if segs:
        with torch.cuda.device(device):
            table = _seg_table(segs, device)
            sums = torch.zeros(len(segs), dtype=torch.int64, device=device)
            N.check(N.lib().ftb200_checksum(N.ptr(table), ctypes.c_int(len(segs)),
                                            ctypes.c_longlong(sum(s[2] for s in segs)), N.ptr(sums), N.stream_ptr()),
                    "checksum")
            for i, v in zip(idx, sums.tolist()):
                out[i] = v & 0xFFFFFFFFFFFFFFFF
    return out


def _export(t: torch.Tensor) -> _PeerTensorRef:
    buf = (ctypes.c_ubyte * 64)()
    off, size = ctypes.c_ulonglong(), ctypes.c_ulonglong()
    with torch.cuda.device(t.device):
        N.check(N.lib().ftb200_ipc_export_any(N.ptr(t), buf, ctypes.byref(off), ctypes.byref(size)), "ipc_export_any", 0)
    return _PeerTensorRef(bytes(buf), int(off.value), t.numel() * t.element_size(), tuple(t.shape), t.dtype)


class P2PTransport(HTTPTransport[T], Generic[T]):
    """
    Args:
        timeout: for the metadata exchange
        device: this rank's GPU
        state_dict: optional callable returning the receiver's current state dict; tensors
            whose shape and dtype match are filled in place
        snapshot: publish device-side copies instead of the live tensors.  Needed when the
            source keeps mutating its weights before the step commits (LocalSGD / DiLoCo
            inner steps); FT-DDP / HSDP leave weights untouched until the commit and can
            stay zero-copy
        checksum: publish and verify per-tensor checksums (one extra read of the state on the
            source, at HBM speed; nothing extra on the receiver)
    """

    def __init__(self, timeout: timedelta, device: torch.device, state_dict: Optional[Callable[[], T]] = None,
                 snapshot: bool = False, checksum: bool = True) -> None:
        super().__init__(timeout=timeout, num_chunks=0)
        self._snapshot = snapshot
        self._checksum = checksum
        hp, dp = ctypes.POINTER(ctypes.c_int)(), ctypes.c_void_p()
        with torch.cuda.device(device):
            N.check(N.lib().ftb200_abort_word_create(ctypes.byref(hp), ctypes.byref(dp)), "abort_word_create", 0)
        self._abort_host, self._abort_dev = hp, int(dp.value)
        self._device = torch.device(device)
        self._state_dict_fn = state_dict
        self._keepalive: List[torch.Tensor] = []
        self._status = torch.zeros(1, dtype=torch.int32, device=self._device)
        # what the last recv_checkpoint moved: bytes, device time of the copies, host time of the whole call
        self.last_recv: Dict[str, float] = {}

    def abort(self) -> None:
        """Makes a copy kernel of this transport that is in flight (or launched later) give up within a fraction of a
        millisecond; ``recv_checkpoint`` then raises.  A plain memory write, callable from any thread."""
        self._abort_host[0] = 1

    def shutdown(self, wait: bool = True) -> None:
        self.abort()
        super().shutdown(wait)

    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: T, timeout: timedelta) -> None:
        leaves, spec = tree_flatten(state_dict)
        out: List[object] = []
        keep: List[torch.Tensor] = []
        for v in leaves:
            if isinstance(v, torch.Tensor) and v.is_cuda:
                c = v.detach()
                if self._snapshot:
                    c = c.clone(memory_format=torch.contiguous_format)
                elif not c.is_contiguous():
                    c = c.contiguous()
                keep.append(c)
                out.append(_export(c))
            else:
                out.append(v)
        if self._checksum and keep:
            # stream-ordered behind whatever produced the tensors; reading the sums back is also
            # the synchronisation that makes everything published here materialised
            sums = iter(_checksums(keep, self._device))
            for ref in out:
                if isinstance(ref, _PeerTensorRef):
                    ref.checksum = next(sums)
        else:
            torch.cuda.current_stream(self._device).synchronize()  # what we publish must be materialised
        self._keepalive = keep
        self._spec = spec
        self._chunks = None
        self._state = tree_unflatten(out, spec)
        self.allow_checkpoint(step)

    def disallow_checkpoint(self) -> None:
        super().disallow_checkpoint()
        self._keepalive = []

    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> T:
        t_begin = time.perf_counter()
        remote = self._fetch(f"{metadata}{step}/full", timeout)
        leaves, spec = tree_flatten(remote, is_leaf=lambda x: isinstance(x, _PeerTensorRef))
        inplace: Optional[List[object]] = None
        if self._state_dict_fn is not None:
            inplace, _ = tree_flatten(self._state_dict_fn())
        lib = N.lib()
        opened: Dict[bytes, int] = {}
        segs: List[Tuple[int, int, int]] = []
        want: List[Optional[int]] = []
        result: List[object] = []
        self._abort_host[0] = 0
        with torch.cuda.device(self._device):
            try:
                for i, v in enumerate(leaves):
                    if not isinstance(v, _PeerTensorRef):
                        result.append(v)
                        continue
                    base = opened.get(v.handle)
                    if base is None:
                        p = ctypes.c_void_p()
                        N.check(lib.ftb200_ipc_import((ctypes.c_ubyte * 64).from_buffer_copy(v.handle), ctypes.byref(p)),
                                "ipc_import", 0)
                        base = int(p.value)
                        opened[v.handle] = base
                    dst: Optional[torch.Tensor] = None
                    if inplace is not None and i < len(inplace):
                        cand = inplace[i]
                        if (isinstance(cand, torch.Tensor) and cand.is_cuda and tuple(cand.shape) == v.shape
                                and cand.dtype == v.dtype and cand.is_contiguous()):
                            dst = cand
                    if dst is None:
                        dst = torch.empty(v.shape, dtype=v.dtype, device=self._device)
                    result.append(dst)
                    if v.nbytes:
                        segs.append((base + v.offset, dst.data_ptr(), v.nbytes))
                        want.append(getattr(v, "checksum", None))
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
                mismatch = self._pull(segs, want, timeout)
                ev1.record()
                ev1.synchronize()
                self.last_recv = {"bytes": float(sum(nb for _, _, nb in segs)), "copy_ms": ev0.elapsed_time(ev1),
                                  "total_s": time.perf_counter() - t_begin}
            finally:
                torch.cuda.current_stream().synchronize()
                for base in opened.values():
                    lib.ftb200_ipc_close(ctypes.c_void_p(base))
        code = int(self._status.item())
        if code:
            self._status.zero_()
            raise RuntimeError(f"peer-memory state transfer failed: {N.STATUS.get(code, code)}")
        bad = mismatch()
        if bad:
            raise RuntimeError(f"peer-memory state transfer: checksum mismatch in {len(bad)} tensor(s) (first: segment {bad[0]})")
        return tree_unflatten(result, spec)

    def _pull(self, segs: List[Tuple[int, int, int]], want: Optional[List[Optional[int]]] = None,
              timeout: Optional[timedelta] = None) -> Callable[[], List[int]]:
        """One kernel for all 16-byte-aligned bulk; ragged heads/tails go through memcpy.  Returns a function that,
        once the stream has been synchronised, lists the segments whose checksum differs from the published one."""
        if not segs:
            return lambda: []
        bulk_segs: List[Tuple[int, int, int]] = []
        expect: List[Optional[int]] = []
        tails: List[Tuple[int, int, int]] = []
        for k, (src, dst, nb) in enumerate(segs):
            if (src % 16) or (dst % 16):
                tails.append((src, dst, nb))
                continue
            bulk = nb // 16 * 16
            if bulk:
                bulk_segs.append((src, dst, bulk))
                expect.append(want[k] if want is not None else None)
            if nb - bulk:
                tails.append((src + bulk, dst + bulk, nb - bulk))
        sums = None
        if bulk_segs:
            dev_table = _seg_table(bulk_segs, self._device)
            sums = torch.zeros(len(bulk_segs), dtype=torch.int64, device=self._device)
            timeout_ns = int(timeout.total_seconds() * 1e9) if timeout is not None else 0
            N.check(N.lib().ftb200_p2p_copy_checked(
                N.ptr(dev_table), ctypes.c_int(len(bulk_segs)), ctypes.c_longlong(sum(s[2] for s in bulk_segs)),
                ctypes.c_void_p(self._abort_dev), N.ptr(self._status), ctypes.c_ulonglong(timeout_ns), N.ptr(sums),
                ctypes.c_int(0), N.stream_ptr()), "p2p_copy")
            self._table_keepalive = dev_table
        for src, dst, nb in tails:
            N.check(N.lib().ftb200_memcpy_d2d(ctypes.c_void_p(dst), ctypes.c_void_p(src), ctypes.c_longlong(nb),
                                              N.stream_ptr()), "memcpy_d2d", 0)

        def mismatch() -> List[int]:
            if sums is None:
                return []
            got = [v & 0xFFFFFFFFFFFFFFFF for v in sums.tolist()]
            return [i for i, (g, e) in enumerate(zip(got, expect)) if e is not None and g != e]

        return mismatch
