"""Pipe with receive deadlines, used between a process group and its worker subprocess."""

from __future__ import annotations

from datetime import timedelta
from typing import Union


def _seconds(t: Union[float, timedelta]) -> float:
    return t.total_seconds() if isinstance(t, timedelta) else float(t)


class _MonitoredPipe:
    """One end of a ``multiprocessing`` pipe (or anything with ``send/recv/poll/close``) whose ``recv`` gives up
    with ``TimeoutError`` after a deadline and re-raises exceptions that the peer sent as payload, so that a
    child's failure surfaces in the parent as the same exception (role of torchft/multiprocessing.py:10-32)."""

    def __init__(self, pipe) -> None:
        self._pipe = pipe

    def send(self, obj: object) -> None:
        self._pipe.send(obj)

    def recv(self, timeout: Union[float, timedelta]) -> object:
        wait = _seconds(timeout)
        if not self._pipe.poll(wait):
            raise TimeoutError(f"pipe.recv() timed out after {wait} seconds")
        payload = self._pipe.recv()
        if isinstance(payload, BaseException):
            raise payload
        return payload

    def close(self) -> None:
        self._pipe.close()

    def closed(self) -> bool:
        return bool(self._pipe.closed)
