"""Trivially completed ``Work`` objects."""

from __future__ import annotations

from typing import Generic, TypeVar

import torch
import torch.distributed as dist

T = TypeVar("T")


class _DummyWork(dist._Work, Generic[T]):
    """An already finished ``Work`` whose future holds ``result``; what a fault-tolerant
    collective returns once the step is known to be lost (role of torchft/work.py:9-20)."""

    def __init__(self, result: T) -> None:
        super().__init__()
        self.result_ = result
        self.future_: torch.futures.Future[T] = torch.futures.Future()
        self.future_.set_result(result)

    def wait(self, timeout=None) -> bool:
        return True

    def get_future(self) -> torch.futures.Future[T]:
        return self.future_

    def is_completed(self) -> bool:
        return True

    def synchronize(self) -> None:
        pass

    def block_current_stream(self, timeout=None) -> None:
        pass
