"""Interface of the live-recovery checkpoint transports."""

from __future__ import annotations

from abc import ABC, abstractmethod
from datetime import timedelta
from typing import Generic, List, TypeVar

T = TypeVar("T")


class CheckpointTransport(Generic[T], ABC):
    """Moves a state dict from an up-to-date replica to recovering ones.

    The manager calls :meth:`metadata` every step (the string travels through the quorum
    so a recovering peer knows where to fetch from), :meth:`send_checkpoint` on the
    source, :meth:`recv_checkpoint` on every destination and
    :meth:`disallow_checkpoint` once the step commits and the weights are about to
    change.  Contract of torchft/checkpointing/transport.py:14-68."""

    @abstractmethod
    def metadata(self) -> str:
        """Opaque string handed to the peers that will call :meth:`recv_checkpoint`."""

    @abstractmethod
    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: T, timeout: timedelta) -> None:
        """Make ``state_dict`` of ``step`` available to the replica ranks ``dst_ranks``."""

    def disallow_checkpoint(self) -> None:
        """Called after the commit vote: the state is about to be mutated, so serving of
        the staged checkpoint must stop.  Default: nothing to do."""

    @abstractmethod
    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> T:
        """Fetch the state dict of ``step`` from replica rank ``src_rank``."""

    def shutdown(self, wait: bool = True) -> None:
        """Release sockets/threads. ``wait`` blocks until they are gone."""
