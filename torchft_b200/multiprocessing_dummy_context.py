"""A thread-backed stand-in for a ``multiprocessing`` context.

``DummyContext().Process(...)`` runs its target on a daemon thread of the calling process and
``Pipe()`` is a pair of in-memory endpoints, so code written against ``mp.get_context("spawn")`` --
the subprocess-backed process groups above all -- can be exercised inside one interpreter: no
interpreter start-up per worker, breakpoints and coverage work, and objects cross the "pipe" by
reference instead of being pickled.  It is a test and debugging helper (same role as the
reference's torchft/multiprocessing_dummy_context.py:24-135, which builds on
``multiprocessing.dummy``); it gives none of a subprocess's isolation: ``kill()`` cannot stop a
thread, it only closes the endpoints handed to the thread so that a worker blocked on ``recv()``
sees ``EOFError`` and leaves.

    from torchft_b200.multiprocessing_dummy_context import DummyContext
    ProcessGroupBabyGloo._mp_context = staticmethod(DummyContext)      # in a test
"""

from __future__ import annotations

import itertools
import queue
import threading
import time
from typing import Any, Callable, Dict, Iterable, Optional, Tuple

_pids = itertools.count(1)


class _Channel:
    """One direction of a pipe: a queue plus a closed flag that wakes blocked readers."""

    def __init__(self) -> None:
        self.items: "queue.SimpleQueue[object]" = queue.SimpleQueue()
        self.cond = threading.Condition()
        self.pending = 0
        self.closed = False

    def put(self, obj: object) -> None:
        with self.cond:
            if self.closed:
                raise BrokenPipeError("the other end of the pipe is closed")
            self.items.put(obj)
            self.pending += 1
            self.cond.notify_all()

    def wait(self, timeout: Optional[float]) -> bool:
        """True when an item is ready or the writer has closed (a read will then not block)."""
        end = None if timeout is None else time.monotonic() + timeout
        with self.cond:
            while self.pending == 0 and not self.closed:
                left = None if end is None else end - time.monotonic()
                if left is not None and left <= 0:
                    return False
                self.cond.wait(left)
            return True

    def get(self) -> object:
        self.wait(None)
        with self.cond:
            if self.pending == 0:
                raise EOFError("pipe closed")
            self.pending -= 1
            return self.items.get_nowait()

    def close(self) -> None:
        with self.cond:
            self.closed = True
            self.cond.notify_all()


class ThreadConnection:
    """One endpoint of an in-memory duplex pipe with the part of ``multiprocessing.connection.Connection``
    that pipe users rely on: ``send``, ``recv``, ``poll``, ``close``, ``closed``."""

    def __init__(self, inbox: _Channel, outbox: _Channel) -> None:
        self._in, self._out = inbox, outbox
        self._closed = False
        # An endpoint handed to a ThreadProcess is shared the way a forked file descriptor is: parent and
        # "child" each hold it, and it is really closed when both have closed it (or the child is killed).
        self._holders = 1
        self._holders_lock = threading.Lock()

    def send(self, obj: object) -> None:
        if self._closed:
            raise OSError("handle is closed")
        self._out.put(obj)

    def recv(self) -> object:
        if self._closed:
            raise OSError("handle is closed")
        return self._in.get()

    def poll(self, timeout: Optional[float] = 0.0) -> bool:
        if self._closed:
            raise OSError("handle is closed")
        return self._in.wait(timeout)

    def _share(self) -> None:
        with self._holders_lock:
            self._holders += 1

    def close(self, force: bool = False) -> None:
        with self._holders_lock:
            self._holders = 0 if force else max(0, self._holders - 1)
            if self._holders > 0:
                return
        # closing an endpoint ends both directions it takes part in: the peer's reads see EOF, its writes fail
        self._closed = True
        self._out.close()
        self._in.close()

    @property
    def closed(self) -> bool:
        return self._closed


class ThreadProcess:
    """``multiprocessing.Process`` look-alike running ``target`` on a daemon thread."""

    def __init__(self, group: None = None, target: Optional[Callable[..., object]] = None, name: Optional[str] = None,
                 args: Iterable[Any] = (), kwargs: Optional[Dict[str, Any]] = None, daemon: Optional[bool] = None) -> None:
        self._target, self._args, self._kwargs = target, tuple(args), dict(kwargs or {})
        self.name = name or f"ThreadProcess-{next(_pids)}"
        self.daemon = True if daemon is None else daemon
        self.pid: Optional[int] = None
        self.exitcode: Optional[int] = None
        self._thread: Optional[threading.Thread] = None

    def _run(self) -> None:
        try:
            if self._target is not None:
                self._target(*self._args, **self._kwargs)
            self.exitcode = 0
        except SystemExit as e:
            self.exitcode = e.code if isinstance(e.code, int) else 1
        except BaseException:
            self.exitcode = 1
            raise

    def start(self) -> None:
        assert self._thread is None, "cannot start a process twice"
        self.pid = next(_pids)
        for a in itertools.chain(self._args, self._kwargs.values()):
            if isinstance(a, ThreadConnection):
                a._share()
        self._thread = threading.Thread(target=self._run, name=self.name, daemon=True)
        self._thread.start()

    def join(self, timeout: Optional[float] = None) -> None:
        if self._thread is not None:
            self._thread.join(timeout)

    def is_alive(self) -> bool:
        return self._thread is not None and self._thread.is_alive()

    def kill(self) -> None:
        """Threads cannot be killed: close every pipe endpoint among the arguments so that the worker unblocks."""
        for a in itertools.chain(self._args, self._kwargs.values()):
            if isinstance(a, ThreadConnection):
                a.close(force=True)

    terminate = kill

    def close(self) -> None:
        pass


class DummyContext:
    """Drop-in for ``multiprocessing.get_context(...)`` whose processes are threads."""

    Process = ThreadProcess

    def __init__(self, method: object = None) -> None:
        self._method = method

    def get_start_method(self, allow_none: bool = False) -> str:
        return "thread"

    def Pipe(self, duplex: bool = True) -> Tuple[ThreadConnection, ThreadConnection]:
        a, b = _Channel(), _Channel()
        return ThreadConnection(a, b), ThreadConnection(b, a)

    def Queue(self, maxsize: int = 0) -> "queue.Queue[object]":
        return queue.Queue(maxsize)

    SimpleQueue = staticmethod(queue.SimpleQueue)
    Event = staticmethod(threading.Event)
    Lock = staticmethod(threading.Lock)
    RLock = staticmethod(threading.RLock)
    Semaphore = staticmethod(threading.Semaphore)
    BoundedSemaphore = staticmethod(threading.BoundedSemaphore)
    Condition = staticmethod(threading.Condition)
    Barrier = staticmethod(threading.Barrier)


def get_context(method: object = None) -> DummyContext:
    return DummyContext(method)
