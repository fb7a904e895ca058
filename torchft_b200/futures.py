"""Timeouts for futures, CUDA streams and blocks of host code.

One daemon *timer thread* owns a deadline heap; everything that needs a timeout
registers an entry and gets a handle it can cancel.  A second *watchdog thread* checks
that the timer thread keeps making progress: a timeout callback that blocks for longer
than ``TORCHFT_WATCHDOG_TIMEOUT_SEC`` (default 30 s) means aborts can no longer be
delivered, so the process exits and lets the job launcher restart it.

Same module-level API as the reference (torchft/futures.py:273-347), which builds it on
an asyncio loop; here it is a heap + condition variable so a timeout costs one heap
push and no coroutine.
"""

from __future__ import annotations

import heapq
import itertools
import os
import queue
import sys
import threading
import time
from contextlib import contextmanager
from datetime import timedelta
from typing import Callable, Generator, List, Optional, Tuple, TypeVar

import torch
from torch.futures import Future

T = TypeVar("T")

WATCHDOG_TIMEOUT_SEC = "TORCHFT_WATCHDOG_TIMEOUT_SEC"


_COMPACT_ABOVE = 4096  # timers in the heap above which cancelled ones are swept out


class _TimerHandle:
    __slots__ = ("_cancelled", "_lock")

    def __init__(self) -> None:
        self._cancelled = False
        self._lock = threading.Lock()

    def cancel(self) -> bool:
        """Returns True if the callback had not fired yet."""
        with self._lock:
            was = self._cancelled
            self._cancelled = True
            return not was

    def _claim(self) -> bool:
        with self._lock:
            if self._cancelled:
                return False
            self._cancelled = True
            return True


class _TimeoutManager:
    def __init__(self) -> None:
        self._cond = threading.Condition()
        self._heap: List[Tuple[float, int, _TimerHandle, Callable[[], None]]] = []
        self._seq = itertools.count()
        self._thread: Optional[threading.Thread] = None
        self._watchdog: Optional[threading.Thread] = None
        self._stop = False
        self._last_beat = time.monotonic()
        self._busy_since: Optional[float] = None
        self._watchdog_interval = timedelta(seconds=float(os.environ.get(WATCHDOG_TIMEOUT_SEC, "30")))
        # CUDA events must not be destroyed on the timer thread (cudaEventDestroy can block
        # behind a hung collective); they are parked here and dropped by the next caller.
        self._del_queue: "queue.SimpleQueue[object]" = queue.SimpleQueue()

    # ------------------------------------------------------------------ lifecycle
    def _ensure_started(self) -> None:
        with self._cond:
            if self._thread is not None and self._thread.is_alive():
                return
            self._stop = False
            self._thread = threading.Thread(target=self._run, name="torchft_b200_timer", daemon=True)
            self._thread.start()
            self._watchdog = threading.Thread(target=self._watch, name="torchft_b200_watchdog", daemon=True)
            self._watchdog.start()

    def shutdown(self) -> None:
        with self._cond:
            self._stop = True
            self._cond.notify_all()
        t, w = self._thread, self._watchdog
        if t is not None:
            t.join(timeout=5)
        if w is not None:
            w.join(timeout=5)
        self._thread = self._watchdog = None

    # ------------------------------------------------------------------ threads
    def _run(self) -> None:
        while True:
            with self._cond:
                while not self._stop:
                    self._last_beat = time.monotonic()
                    if self._heap and self._heap[0][0] <= self._last_beat:
                        break
                    wait = 0.5
                    if self._heap:
                        wait = min(wait, max(0.0, self._heap[0][0] - self._last_beat))
                    self._cond.wait(wait)
                if self._stop:
                    return
                _, _, handle, cb = heapq.heappop(self._heap)
                self._busy_since = time.monotonic()
            if handle._claim():
                try:
                    cb()
                except Exception as e:  # a failing timeout callback must not kill the timer
                    print(f"torchft_b200: timeout callback raised {e!r}", file=sys.stderr)
            with self._cond:
                self._busy_since = None

    def _watch(self) -> None:
        limit = self._watchdog_interval.total_seconds()
        while True:
            with self._cond:
                if self._stop:
                    return
                busy = self._busy_since
            if busy is not None and time.monotonic() - busy > limit:
                print(
                    f"torchft_b200 watchdog: a timeout callback has been stuck for more than {limit} s; exiting",
                    file=sys.stderr,
                )
                sys.stderr.flush()
                self._exit()
                return
            time.sleep(min(1.0, max(0.01, limit / 10)))

    @staticmethod
    def _exit() -> None:  # separate so tests can patch it
        os._exit(1)

    # ------------------------------------------------------------------ API
    def call_later(self, timeout: timedelta, cb: Callable[[], None]) -> _TimerHandle:
        self._ensure_started()
        self._drain_del_queue()
        handle = _TimerHandle()
        deadline = time.monotonic() + timeout.total_seconds()
        with self._cond:
            # the timer thread only has to be woken when this deadline becomes the earliest one: almost every timer
            # is cancelled long before it is due, and a wake-up per armed timer is a context switch per collective
            wake = not self._heap or deadline < self._heap[0][0]
            heapq.heappush(self._heap, (deadline, next(self._seq), handle, cb))
            if len(self._heap) > _COMPACT_ABOVE:
                live = [e for e in self._heap if not e[2]._cancelled]
                if len(live) < len(self._heap) // 2:  # cancelled timers otherwise stay until their deadline
                    heapq.heapify(live)
                    self._heap = live
            if wake:
                self._cond.notify_all()
        return handle

    def register(self, fut: Future, timeout: timedelta) -> Future:
        """A future that mirrors ``fut`` but fails with ``TimeoutError`` after ``timeout``."""
        timed: Future = Future()
        done = threading.Lock()
        state = {"set": False}

        def settle(fn: Callable[[], None]) -> None:
            with done:
                if state["set"]:
                    return
                state["set"] = True
            fn()

        handle = self.call_later(
            timeout, lambda: settle(lambda: timed.set_exception(TimeoutError(f"future did not complete within {timeout}")))
        )

        def on_done(f: Future) -> None:
            handle.cancel()
            try:
                v = f.value()
            except Exception as e:
                settle(lambda: timed.set_exception(e))
            else:
                settle(lambda: timed.set_result(v))

        fut.add_done_callback(on_done)
        return timed

    def stream_timeout(self, callback: Callable[[], None], timeout: timedelta) -> None:
        """Calls ``callback`` if the work queued so far on the current CUDA stream has not
        finished ``timeout`` from now."""
        if not torch.cuda.is_available():
            return
        event = torch.cuda.Event()
        event.record()

        def check() -> None:
            try:
                if not event.query():
                    callback()
            finally:
                self._del_queue.put(event)

        self.call_later(timeout, check)

    @contextmanager
    def context_timeout(self, callback: Callable[[], None], timeout: timedelta) -> Generator[None, None, None]:
        handle = self.call_later(timeout, callback)
        try:
            yield
        finally:
            handle.cancel()

    def _drain_del_queue(self) -> int:
        n = 0
        while True:
            try:
                self._del_queue.get_nowait()
                n += 1
            except queue.Empty:
                return n


_TIMEOUT_MANAGER = _TimeoutManager()


def future_timeout(fut: Future, timeout: timedelta) -> Future:
    """Return a future that completes like ``fut`` or, after ``timeout``, with ``TimeoutError``."""
    return _TIMEOUT_MANAGER.register(fut, timeout)


def future_wait(fut: Future, timeout: timedelta) -> T:
    """Block until ``fut`` completes and return its value; ``TimeoutError`` after ``timeout``."""
    ev = threading.Event()
    fut.add_done_callback(lambda f: ev.set())
    if not ev.wait(timeout.total_seconds()):
        raise TimeoutError(f"future did not complete within {timeout}")
    return fut.value()


def stream_timeout(callback: Callable[[], None], timeout: timedelta) -> None:
    """Arm a timeout on everything enqueued so far on the current CUDA stream."""
    _TIMEOUT_MANAGER.stream_timeout(callback, timeout)


def context_timeout(callback: Callable[[], None], timeout: timedelta):
    """``with context_timeout(cb, t):`` -- ``cb`` runs on the timer thread if the block is
    still executing after ``t``."""
    return _TIMEOUT_MANAGER.context_timeout(callback, timeout)
