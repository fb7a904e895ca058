"""Stream/event helpers that work on hosts without an accelerator."""

from __future__ import annotations

from contextlib import nullcontext
from typing import ContextManager, Optional

import torch


def get_stream_context(stream: Optional[torch.cuda.Stream]) -> ContextManager:
    """``with`` context that makes ``stream`` current, or a no-op when ``stream`` is None
    or no CUDA device exists."""
    if stream is not None and torch.cuda.is_available():
        return torch.cuda.stream(stream)
    return nullcontext()


def record_event() -> Optional[torch.cuda.Event]:
    """Record and return an event on the current CUDA stream (None on CPU-only hosts).

    The reference's helper of the same name is declared ``-> None`` and drops the event
    (torchft/utils.py:46-56); here the event is returned so callers can wait on it."""
    if torch.cuda.is_available():
        return torch.cuda.current_stream().record_event()
    return None


def synchronize() -> None:
    """Block the host until the current CUDA stream has drained (no-op on CPU)."""
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
