"""Streaming (de)serialisation of state dicts for the transports.

Uses ``torch.distributed._serialization`` when the installed PyTorch has it (tensors
stream straight to/from the socket without an intermediate byte string) and falls back
to ``torch.save``/``torch.load``.  Payloads contain arbitrary Python leaves, hence
``weights_only=False`` -- the transports only ever talk to replicas of the same job.
"""

from __future__ import annotations

from typing import IO

import torch

try:  # pragma: no cover - depends on the torch build
    from torch.distributed._serialization import _streaming_load as _sload
    from torch.distributed._serialization import _streaming_save as _ssave

    _HAVE_STREAMING = True
except Exception:  # pragma: no cover
    _HAVE_STREAMING = False


def streaming_save(obj: object, f: IO[bytes]) -> None:
    if _HAVE_STREAMING:
        _ssave(obj, f)
    else:
        torch.save(obj, f)


def streaming_load(f: IO[bytes]) -> object:
    if _HAVE_STREAMING:
        return _sload(f, weights_only=False)
    return torch.load(f, weights_only=False)
