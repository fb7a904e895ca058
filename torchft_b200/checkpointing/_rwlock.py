"""Readers/writer lock whose acquires all time out.

Guards the user's state dict: many checkpoint readers (peers healing from this replica)
may hold it at once, the optimizer step takes it exclusively.  Role of
torchft/checkpointing/_rwlock.py:41-131; implemented here with one condition variable
and writer preference (a waiting writer blocks new readers, so the training loop cannot
be starved by a stream of checkpoint fetches).
"""

from __future__ import annotations

import threading
import time
from contextlib import contextmanager
from typing import Generator


class RWLock:
    def __init__(self, timeout: float = -1) -> None:
        """``timeout`` in seconds for every acquire; negative waits forever."""
        self.timeout = timeout
        self._cond = threading.Condition()
        self._readers = 0
        self._writer = False
        self._writers_waiting = 0

    def _wait_for(self, pred) -> bool:
        if self.timeout < 0:
            self._cond.wait_for(pred)
            return True
        return self._cond.wait_for(pred, timeout=self.timeout)

    # ---- read side
    def r_acquire(self) -> None:
        with self._cond:
            if not self._wait_for(lambda: not self._writer and self._writers_waiting == 0):
                raise TimeoutError(f"timed out after {self.timeout}s waiting for the read lock")
            self._readers += 1

    def r_release(self) -> None:
        with self._cond:
            assert self._readers > 0, "read lock released more often than acquired"
            self._readers -= 1
            if self._readers == 0:
                self._cond.notify_all()

    @contextmanager
    def r_lock(self) -> Generator[None, None, None]:
        self.r_acquire()
        try:
            yield
        finally:
            self.r_release()

    # ---- write side
    def w_acquire(self) -> None:
        with self._cond:
            self._writers_waiting += 1
            try:
                if not self._wait_for(lambda: not self._writer and self._readers == 0):
                    raise TimeoutError(f"timed out after {self.timeout}s waiting for the write lock")
                self._writer = True
            finally:
                self._writers_waiting -= 1
                self._cond.notify_all()

    def w_release(self) -> None:
        with self._cond:
            assert self._writer, "write lock released without being held"
            self._writer = False
            self._cond.notify_all()

    def w_locked(self) -> bool:
        with self._cond:
            return self._writer

    @contextmanager
    def w_lock(self) -> Generator[None, None, None]:
        self.w_acquire()
        try:
            yield
        finally:
            self.w_release()
