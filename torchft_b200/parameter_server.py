"""Prototype parameter server on reconfigurable process groups.

A server process exposes ``GET /new_session``; each call creates a fresh TCPStore prefix,
answers ``{"session_id", "store_addr"}`` and then -- on the HTTP handler's own thread --
configures a new two-member process group (server rank 0, client rank 1) and runs the
user's :meth:`ParameterServer.forward` over it until the session ends.  No lighthouse is
involved; sessions fail independently.  Shape of torchft/parameter_server.py:31-195.
"""

from __future__ import annotations

import json
import logging
import socket
import threading
import urllib.request
import uuid
from abc import ABC, abstractmethod
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from torch.distributed import TCPStore

from .process_group import ProcessGroup

logger = logging.getLogger(__name__)


class _Server(ThreadingHTTPServer):
    address_family = socket.AF_INET6
    request_queue_size = 1024
    daemon_threads = True

    def server_bind(self) -> None:
        try:
            self.socket.setsockopt(socket.IPPROTO_IPV6, socket.IPV6_V6ONLY, 0)
        except OSError:
            pass
        super().server_bind()


class ParameterServer(ABC):
    """Subclass and implement :meth:`new_process_group` and :meth:`forward`."""

    def __init__(self, port: int, store_port: int = 0) -> None:
        self.store = TCPStore(host_name="0.0.0.0", port=store_port, is_master=True, wait_for_workers=False)
        ps = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, fmt, *args):
                logger.debug(fmt, *args)

            def do_GET(self) -> None:
                if self.path != "/new_session":
                    self.send_error(400, f"invalid path, got {self.path}")
                    return
                try:
                    session_id = str(uuid.uuid4())
                    store_addr = f"{socket.gethostname()}:{ps.store.port}/session/{session_id}"
                    local_store_addr = f"localhost:{ps.store.port}/session/{session_id}"
                    body = (json.dumps({"session_id": session_id, "store_addr": store_addr}) + "\n").encode()
                    self.send_response(200)
                    self.send_header("Content-type", "application/json")
                    self.send_header("Content-Length", str(len(body)))
                    self.end_headers()
                    self.wfile.write(body)
                    self.wfile.flush()
                    # the handler thread now becomes the session's worker
                    ps._handle_session(session_id, local_store_addr)
                except Exception:
                    logger.exception("parameter server session failed")

        self._server = _Server(("", port), Handler)
        self._thread = threading.Thread(target=self._server.serve_forever, name="torchft_b200_ps", daemon=True)
        self._thread.start()

    def address(self) -> str:
        """URL a client passes to :meth:`new_session`."""
        return f"http://{socket.gethostname()}:{self._server.socket.getsockname()[1]}/new_session"

    def shutdown(self) -> None:
        self._server.shutdown()
        self._thread.join()
        self._server.server_close()

    @classmethod
    @abstractmethod
    def new_process_group(cls) -> ProcessGroup:
        """A fresh, unconfigured process group (called on both sides of a session)."""

    @classmethod
    def new_session(cls, address: str) -> ProcessGroup:
        """Client side: open a session and return a configured group (this side is rank 1)."""
        host = socket.gethostname()
        if f"//{host}:" in address:
            address = address.replace(f"//{host}:", "//localhost:")
        with urllib.request.urlopen(address) as f:
            data = json.load(f)
        store_addr = data["store_addr"]
        if store_addr.startswith(f"{host}:"):
            store_addr = "localhost:" + store_addr[len(host) + 1:]
        logger.info("connecting to session %s at %s", data["session_id"], store_addr)
        pg = cls.new_process_group()
        pg.configure(store_addr, replica_id="0", rank=1, world_size=2)
        return pg

    def _handle_session(self, session_id: str, store_addr: str) -> None:
        pg = self.new_process_group()
        pg.configure(store_addr, replica_id="0", rank=0, world_size=2)
        self.forward(session_id, pg)

    @abstractmethod
    def forward(self, session_id: str, pg: ProcessGroup) -> None:
        """Server side of one session; runs on a dedicated thread, returns to end it."""
