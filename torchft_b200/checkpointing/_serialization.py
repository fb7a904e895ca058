"""Streaming (de)serialisation of state dicts for the transports.

Format: ``MAGIC | u64 header length | header | tensor bytes ...``.  The header is a pickle of the
pytree spec and one entry per leaf: plain tensors are described by dtype and shape and their bytes
follow the header back to back, in leaf order; every other leaf (Python objects, tensor subclasses
such as DTensor) travels inside the header.  The writer hands each tensor's memory to the stream
without copying it into a byte string; the reader allocates each tensor and receives straight
into its memory (``readinto``), so a multi-GB state dict costs one pass over its bytes on either
side.  The payloads contain arbitrary Python leaves -- the transports only ever talk to replicas
of the same job.

The reference wraps ``torch.distributed._serialization._streaming_save/_streaming_load`` with a
``torch.save`` fallback (torchft/checkpointing/_serialization.py:8-33); on a 1.2 GB state dict of
3 MB tensors that private API took 3 s to write and 11 s to read on the build machine, which made it,
not the network, the limit of the HTTP transport.
"""

from __future__ import annotations

import io
import pickle
import struct
from typing import IO, List, Optional, Tuple

import torch
from torch.utils._pytree import TreeSpec, tree_flatten, tree_unflatten, treespec_dumps, treespec_loads

MAGIC = b"FTB2SD01"
_CHUNK = 64 << 20  # upper bound of one write / readinto call


def pack_treespec(spec: TreeSpec) -> object:
    """A tree spec in the form it travels in: torch's JSON form for the standard containers (stable across torch
    versions), the object itself (to be pickled) for specs that contain types without a registered serialiser."""
    try:
        return ("json", treespec_dumps(spec))
    except Exception:
        return ("obj", spec)


def unpack_treespec(packed: object) -> TreeSpec:
    kind, value = packed  # type: ignore[misc]
    return treespec_loads(value) if kind == "json" else value


def _is_plain_tensor(x: object) -> bool:
    return type(x) is torch.Tensor or type(x) is torch.nn.Parameter


def _bytes_view(t: torch.Tensor) -> memoryview:
    """The memory of a contiguous CPU tensor as a flat byte view (works for bf16 and other dtypes
    NumPy does not know)."""
    flat = t.reshape(-1)
    if flat.numel() == 0:
        return memoryview(b"")
    return memoryview(flat.view(torch.uint8).numpy())


def streaming_save(obj: object, f: IO[bytes]) -> None:
    leaves, spec = tree_flatten(obj)
    metas: List[Tuple] = []
    tensors: List[torch.Tensor] = []
    for leaf in leaves:
        if _is_plain_tensor(leaf):
            t = leaf.detach()
            if t.device.type != "cpu":
                t = t.cpu()
            t = t.contiguous()
            metas.append(("T", t.dtype, tuple(t.shape)))
            tensors.append(t)
        elif isinstance(leaf, torch.Tensor):  # a tensor subclass: let torch serialise it whole
            buf = io.BytesIO()
            torch.save(leaf, buf)
            metas.append(("S", buf.getvalue()))
        else:
            metas.append(("O", leaf))
    header = pickle.dumps((pack_treespec(spec), metas), protocol=pickle.HIGHEST_PROTOCOL)
    f.write(MAGIC + struct.pack("<Q", len(header)))
    f.write(header)
    for t in tensors:
        mv = _bytes_view(t)
        for off in range(0, len(mv), _CHUNK):
            f.write(mv[off : off + _CHUNK])


def _read_exact(f: IO[bytes], n: int) -> bytes:
    parts, got = [], 0
    while got < n:
        b = f.read(n - got)
        if not b:
            raise EOFError(f"stream ended after {got} of {n} bytes")
        parts.append(b)
        got += len(b)
    return b"".join(parts)


def _read_into(f: IO[bytes], mv: memoryview) -> None:
    got, n = 0, len(mv)
    readinto = getattr(f, "readinto", None)
    while got < n:
        if readinto is not None:
            k = readinto(mv[got : min(n, got + _CHUNK)])
            if not k:
                raise EOFError(f"stream ended after {got} of {n} tensor bytes")
        else:
            b = f.read(min(n - got, _CHUNK))
            if not b:
                raise EOFError(f"stream ended after {got} of {n} tensor bytes")
            k = len(b)
            mv[got : got + k] = b
        got += k


def streaming_load(f: IO[bytes], into: Optional[List[object]] = None) -> object:
    """``into``: optional flattened leaves of a state dict of the same structure; tensor leaves whose
    shape and dtype match receive the data in place (CPU tensors straight from the stream, tensors on
    other devices through one host bounce) and are returned as the leaves of the result.  Receiving into
    memory that already exists also avoids faulting in fresh pages, which on some hosts costs more than
    the transfer itself."""
    head = _read_exact(f, len(MAGIC) + 8)
    if head[: len(MAGIC)] != MAGIC:
        raise ValueError("not a torchft_b200 state-dict stream")
    (hlen,) = struct.unpack("<Q", head[len(MAGIC) :])
    packed_spec, metas = pickle.loads(_read_exact(f, hlen))
    spec = unpack_treespec(packed_spec)
    leaves: List[object] = []
    for i, m in enumerate(metas):
        if m[0] == "T":
            dst = into[i] if into is not None and i < len(into) else None
            ok = isinstance(dst, torch.Tensor) and _is_plain_tensor(dst) and dst.dtype == m[1] and tuple(dst.shape) == m[2]
            if ok and dst.device.type == "cpu" and dst.is_contiguous():
                _read_into(f, _bytes_view(dst.detach()))
                leaves.append(dst)
                continue
            t = torch.empty(m[2], dtype=m[1])
            mv = _bytes_view(t)
            if len(mv) >= (1 << 20):
                # touch the pages from user space first: faulting them in one by one inside recv() is several
                # times slower than a memset (an order of magnitude on virtualised hosts)
                t.reshape(-1).view(torch.uint8).zero_()
            _read_into(f, mv)
            if ok:
                with torch.no_grad():
                    dst.copy_(t)
                leaves.append(dst)
            else:
                leaves.append(t)
        elif m[0] == "S":
            leaves.append(torch.load(io.BytesIO(m[1]), weights_only=False))
        else:
            leaves.append(m[1])
    return tree_unflatten(leaves, spec)
