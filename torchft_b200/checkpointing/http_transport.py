"""HTTP checkpoint transport: a recovering replica pulls the state dict of an up-to-date
peer over HTTP/1.1.

Works across hosts and for CPU state; for GPUs on one NVSwitch domain the peer-memory
transport (:mod:`torchft_b200.checkpointing.p2p_transport`) moves tensor payloads over
NVLink instead.  Wire behaviour follows torchft/checkpointing/http_transport.py:39-267:

* URL ``/checkpoint/<step>/<key>`` with ``key`` = ``full`` (whole state dict),
  ``metadata`` (the pytree spec) or a chunk index; a step other than the staged one is
  answered with HTTP 400;
* nothing is served before the first :meth:`send_checkpoint`, and
  :meth:`disallow_checkpoint` blocks readers again while the optimizer mutates state;
* with ``num_chunks > 0`` the flattened leaves are dealt round-robin into chunks that
  the receiver fetches on parallel connections.
"""

from __future__ import annotations

import io
import logging
import socket
import threading
import time
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Generic, List, Optional, TypeVar

import torch
from torch.utils._pytree import TreeSpec, tree_flatten, tree_unflatten

from ._rwlock import RWLock
from ._serialization import pack_treespec, streaming_load, streaming_save, unpack_treespec
from .transport import CheckpointTransport

logger = logging.getLogger(__name__)
T = TypeVar("T")


class _DualStackServer(ThreadingHTTPServer):
    address_family = socket.AF_INET6
    request_queue_size = 1024
    daemon_threads = True

    def server_bind(self) -> None:
        try:
            self.socket.setsockopt(socket.IPPROTO_IPV6, socket.IPV6_V6ONLY, 0)
        except OSError:
            pass
        super().server_bind()


def _leaf_to_cpu(v: object, pin: bool) -> object:
    """Host snapshot of a leaf.  Tensors are always copied: what is staged must not change
    when the trainer goes on mutating its weights (LocalSGD/DiLoCo take inner steps while a
    peer is still fetching)."""
    if isinstance(v, torch.Tensor):
        if v.device.type != "cpu":
            out = torch.empty(v.shape, dtype=v.dtype, device="cpu", pin_memory=pin)
            out.copy_(v, non_blocking=True)
            return out
        return v.detach().clone()
    return v


class HTTPTransport(CheckpointTransport[T], Generic[T]):
    """Checkpoint transport over HTTP: every rank runs a small threaded server; a healthy rank stages a snapshot of
    its state (``send_checkpoint``) and recovering ranks download it (``recv_checkpoint``) from
    ``/checkpoint/<step>/full``, or in ``num_chunks`` parallel streams from ``/checkpoint/<step>/<i>``.  Nothing is served
    before the first ``send_checkpoint`` or after ``disallow_checkpoint``; a request for another step gets HTTP 400.
    Works between any two hosts that can reach each other (torchft/checkpointing/http_transport.py:39-267)."""

    def __init__(self, timeout: timedelta, num_chunks: int = 0, pin_memory: bool = False,
                 state_dict: Optional[Callable[[], T]] = None) -> None:
        """``state_dict``: optional callable returning the receiver's current state dict; tensors whose shape
        and dtype match are then filled in place instead of being allocated (as the process-group and
        peer-memory transports do)."""
        self._timeout = timeout
        self._state_dict_fn = state_dict
        self._num_chunks = num_chunks
        self._pin = pin_memory and torch.cuda.is_available()
        self._lock = RWLock(timeout=timeout.total_seconds())
        self._serving = True  # flipped by the disallow below
        self._step = -1
        self._state: Optional[T] = None
        self._spec: Optional[TreeSpec] = None
        self._chunks: Optional[List[List[object]]] = None
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.disallow_checkpoint()  # serve nothing until something has been staged

        transport = self
        sock_timeout = timeout.total_seconds()

        class Handler(BaseHTTPRequestHandler):
            timeout = sock_timeout
            # The serialiser emits a small header before every tensor's bytes.  Unbuffered, each is its own
            # TCP segment and Nagle's algorithm against delayed ACKs stalls ~10-40 ms per tensor.
            wbufsize = 4 << 20
            disable_nagle_algorithm = True

            def log_message(self, fmt, *args):  # keep stderr quiet
                logger.debug(fmt, *args)

            def _reply(self, payload: object) -> None:
                self.send_response(200)
                self.send_header("Content-type", "application/octet-stream")
                self.end_headers()
                streaming_save(payload, self.wfile)

            def do_GET(self) -> None:
                try:
                    with transport._lock.r_lock():
                        parts = self.path.split("/")
                        if len(parts) != 4 or parts[1] != "checkpoint":
                            self.send_error(400, f"invalid url format, expected /checkpoint/step/key but got {self.path}")
                            return
                        want = int(parts[2])
                        if want != transport._step:
                            self.send_error(
                                400, f"invalid checkpoint requested, serving {transport._step} but got step={want}"
                            )
                            return
                        key = parts[3]
                        if key == "full":
                            self._reply(transport._state)
                        elif key == "metadata":
                            self._reply(pack_treespec(transport._spec))
                        else:
                            assert transport._chunks is not None, "checkpoint was not staged in chunks"
                            self._reply(transport._chunks[int(key)])
                except Exception as e:
                    logger.exception("checkpoint server failed on %s: %s", self.path, e)
                    try:
                        self.send_error(500, str(e))
                    except Exception:
                        pass

        self._server = _DualStackServer(("", 0), Handler)
        self._thread = threading.Thread(target=self._server.serve_forever, name="torchft_b200_ckpt_http", daemon=True)
        self._thread.start()
        logger.info("checkpoint server listening on %s", self.address())

    # ------------------------------------------------------------------ addressing
    def address(self) -> str:
        """``http://host:port/checkpoint/`` prefix; append ``<step>/<key>``."""
        port = self._server.socket.getsockname()[1]
        return f"http://{socket.gethostname()}:{port}/checkpoint/"

    def metadata(self) -> str:
        return self.address()

    # ------------------------------------------------------------------ lock state machine
    def allow_checkpoint(self, step: int) -> None:
        self._step = step
        if not self._serving:
            self._serving = True
            self._lock.w_release()

    def disallow_checkpoint(self) -> None:
        if self._serving:
            self._serving = False
            self._lock.w_acquire()

    # ------------------------------------------------------------------ send / recv
    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: T, timeout: timedelta) -> None:
        leaves, spec = tree_flatten(state_dict)
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                leaves = [_leaf_to_cpu(v, self._pin) for v in leaves]
            self._stream.synchronize()
        else:
            leaves = [_leaf_to_cpu(v, False) for v in leaves]
        self._spec = spec
        if self._num_chunks > 0:
            self._chunks = [leaves[i :: self._num_chunks] for i in range(self._num_chunks)]
            self._state = None
        else:
            self._chunks = None
            self._state = tree_unflatten(leaves, spec)
        self.allow_checkpoint(step)

    @staticmethod
    def _fetch(url: str, timeout: timedelta, into: Optional[List[object]] = None) -> object:
        # resolve our own hostname locally: containers often cannot resolve it via DNS
        host = socket.gethostname()
        if f"//{host}:" in url:
            url = url.replace(f"//{host}:", "//localhost:")
        # Deserialise straight from the socket through a large read buffer.  Reading the whole body first
        # (`f.read()` on a response of unknown length) goes through 8 KB receives and a growing byte string:
        # 60 MB/s on a 1.2 GB state dict; streaming reaches the speed of the loopback/NIC.
        with urllib.request.urlopen(url, timeout=timeout.total_seconds()) as f:
            return streaming_load(io.BufferedReader(f, buffer_size=4 << 20), into=into)

    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> T:
        t0 = time.perf_counter()
        try:
            return self._recv_checkpoint(metadata, step, timeout)
        finally:
            logger.info("recv_checkpoint of step %d from rank %d took %.3fs", step, src_rank, time.perf_counter() - t0)

    def _recv_checkpoint(self, metadata: str, step: int, timeout: timedelta) -> T:
        base = f"{metadata}{step}"
        into: Optional[List[object]] = None
        if self._state_dict_fn is not None:
            into, _ = tree_flatten(self._state_dict_fn())
        if self._num_chunks == 0:
            return self._fetch(f"{base}/full", timeout, into)  # type: ignore[return-value]
        spec = unpack_treespec(self._fetch(f"{base}/metadata", timeout))
        n_chunks = self._num_chunks
        with ThreadPoolExecutor(max_workers=n_chunks, thread_name_prefix="torchft_b200_ckpt_fetch") as ex:
            chunks = list(ex.map(lambda i: self._fetch(f"{base}/{i}", timeout, into[i::n_chunks] if into is not None else None),
                                 range(n_chunks)))
        n = sum(len(c) for c in chunks)
        leaves: List[object] = [None] * n
        for i, c in enumerate(chunks):
            leaves[i :: self._num_chunks] = c
        return tree_unflatten(leaves, spec)

    def shutdown(self, wait: bool = True) -> None:
        if not wait:
            # serve_forever polls; closing the socket makes handlers fail fast
            threading.Thread(target=self._server.shutdown, daemon=True).start()
        else:
            self._server.shutdown()
            self._thread.join()
        self._server.server_close()
