"""Pipe with receive deadlines, used between a process group and its worker subprocess."""

from __future__ import annotations

from datetime import timedelta
from multiprocessing.connection import Connection
from typing import Union


class _MonitoredPipe:
    """Wraps a ``multiprocessing`` connection: ``recv`` gives up with ``TimeoutError``
    after a deadline and re-raises exceptions that the peer sent as payload
    (role of torchft/multiprocessing.py:10-32)."""

    def __init__(self, pipe: "Connection[object, object]") -> None:
        self._pipe = pipe

    def send(self, obj: object) -> None:
        self._pipe.send(obj)

    def recv(self, timeout: Union[float, timedelta]) -> object:
        secs = timeout.total_seconds() if isinstance(timeout, timedelta) else float(timeout)
        if not self._pipe.poll(secs):
            raise TimeoutError(f"pipe.recv() timed out after {secs} seconds")
        out = self._pipe.recv()
        if isinstance(out, Exception):
            raise out
        return out

    def close(self) -> None:
        self._pipe.close()

    def closed(self) -> bool:
        return self._pipe.closed
