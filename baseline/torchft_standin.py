"""Pure-Python stand-in for the reference's native module ``torchft._torchft``.

The reference's control plane is a Rust extension that cannot be built offline (no cargo,
rustc, protoc or maturin).  Everything else in the reference is plain Python.  This module
implements the interface of ``torchft/_torchft.pyi`` over plain TCP sockets (length-prefixed
pickle frames) so that the *unmodified* reference Python (``Manager``, ``ProcessGroupNCCL``,
``OptimizerWrapper``, ``DiLoCo``, the checkpoint transports) can run as the comparison arm
of the benchmarks.  It is used by the reference arm only; it is registered as
``sys.modules["torchft._torchft"]`` before ``torchft`` is imported
(:func:`install`).  It imports nothing from the product package and loads no native code.

Behaviour follows the reference's services: ``quorum_compute`` (``src/lighthouse.rs:141-269``),
the quorum RPC (``src/lighthouse.rs:484-551``), ``compute_quorum_results``
(``src/manager.rs:489-624``), the manager's quorum aggregation and ``should_commit`` barrier
(``src/manager.rs:332-479``).  A Python control plane costs a few hundred microseconds more per
round trip than the Rust one; against training steps of hundreds of milliseconds that is noise,
and the benchmark lines say that the control plane is a stand-in.
"""

from __future__ import annotations

import os
import pickle
import socket
import socketserver
import struct
import sys
import threading
import time
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Dict, Hashable, List, Optional
from urllib.parse import urlparse

# ----------------------------------------------------------------------------- wire


def _send(sock: socket.socket, obj) -> None:
    raw = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    sock.sendall(struct.pack("!I", len(raw)) + raw)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return bytes(buf)


def _recv(sock: socket.socket):
    (n,) = struct.unpack("!I", _recv_exact(sock, 4))
    return pickle.loads(_recv_exact(sock, n))


def _host_port(addr: str):
    if "//" not in addr:
        addr = "http://" + addr
    u = urlparse(addr)
    host = u.hostname or "127.0.0.1"
    if host in ("::", "0.0.0.0", "[::]"):
        host = "127.0.0.1"
    return host, int(u.port)


class _Client:
    """One persistent connection; a call is (method, kwargs, timeout_s) -> ("ok", value) | ("err", kind, text)."""

    def __init__(self, addr: str, connect_timeout: timedelta) -> None:
        self._addr = _host_port(addr)
        self._lock = threading.Lock()
        self._sock: Optional[socket.socket] = None
        deadline = time.monotonic() + connect_timeout.total_seconds()
        delay = 0.1
        while True:
            try:
                self._connect()
                return
            except OSError:
                if time.monotonic() + delay > deadline:
                    raise TimeoutError(f"could not connect to {addr} within {connect_timeout}")
                time.sleep(delay)
                delay = min(delay * 1.5, 10.0)

    def _connect(self) -> None:
        s = socket.create_connection(self._addr, timeout=5.0)
        s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._sock = s

    def call(self, method: str, timeout: timedelta, **kwargs):
        t = timeout.total_seconds()
        with self._lock:
            try:
                if self._sock is None:
                    self._connect()
                assert self._sock is not None
                self._sock.settimeout(t + 1.0)
                _send(self._sock, (method, kwargs, t))
                reply = _recv(self._sock)
            except socket.timeout:
                self._close()
                raise TimeoutError(f"{method} timed out after {t}s")
            except (OSError, ConnectionError) as e:
                self._close()
                raise RuntimeError(f"{method} failed: {e}")
        if reply[0] == "ok":
            return reply[1]
        _, kind, text = reply
        if kind == "timeout":
            raise TimeoutError(text)
        raise RuntimeError(text)

    def _close(self) -> None:
        if self._sock is not None:
            try:
                self._sock.close()
            finally:
                self._sock = None


class _Server:
    """Thread-per-connection request loop; ``handler(method, kwargs, deadline)`` returns the value."""

    def __init__(self, bind: str, handler) -> None:
        port = int(bind.rsplit(":", 1)[1])
        outer = self

        class H(socketserver.BaseRequestHandler):
            def handle(self):
                self.request.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                while not outer._stop.is_set():
                    try:
                        method, kwargs, t = _recv(self.request)
                    except (ConnectionError, OSError, EOFError):
                        return
                    try:
                        out = ("ok", handler(method, kwargs, time.monotonic() + t))
                    except TimeoutError as e:
                        out = ("err", "timeout", str(e))
                    except Exception as e:  # noqa: BLE001 - forwarded to the caller
                        out = ("err", "runtime", f"{type(e).__name__}: {e}")
                    try:
                        _send(self.request, out)
                    except OSError:
                        return

        class S(socketserver.ThreadingTCPServer):
            allow_reuse_address = True
            daemon_threads = True
            request_queue_size = 1024

        self._stop = threading.Event()
        self._srv = S(("0.0.0.0", port), H)
        self.port = self._srv.server_address[1]
        self._thread = threading.Thread(target=self._srv.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True)
        self._thread.start()

    def shutdown(self) -> None:
        self._stop.set()
        self._srv.shutdown()
        self._srv.server_close()


# ----------------------------------------------------------------------------- data types


@dataclass
class QuorumMember:
    replica_id: str
    address: str
    store_address: str
    step: int
    world_size: int
    shrink_only: bool
    data: Optional[Dict[Hashable, object]] = None
    commit_failures: int = 0


@dataclass
class Timestamp:
    seconds: int
    nanos: int


@dataclass
class Quorum:
    quorum_id: int
    participants: List[QuorumMember]
    created: Timestamp


@dataclass
class QuorumResult:
    quorum_id: int = 0
    replica_rank: int = 0
    replica_world_size: int = 1
    recover_src_manager_address: str = ""
    recover_src_replica_rank: Optional[int] = None
    recover_dst_replica_ranks: List[int] = field(default_factory=list)
    store_address: str = ""
    max_step: int = 0
    max_replica_rank: Optional[int] = None
    max_world_size: int = 1
    heal: bool = False
    commit_failures: int = 0


# ----------------------------------------------------------------------------- lighthouse


def quorum_compute(now: float, participants: Dict[str, tuple], heartbeats: Dict[str, float],
                   prev_quorum: Optional[Quorum], min_replicas: int, join_timeout_s: float,
                   heartbeat_timeout_s: float):
    """Returns ``(members or None, reason)``.  ``participants`` maps replica id to ``(joined_at, member)``."""
    healthy = {r for r, t in heartbeats.items() if now - t < heartbeat_timeout_s}
    cand = sorted((m for r, (_, m) in participants.items() if r in healthy), key=lambda m: m.replica_id)
    shrink_only = any(m.shrink_only for m in cand)
    meta = f"[{len(cand)}/{len(participants)} participants healthy][{len(healthy)} heartbeating][shrink_only={str(shrink_only).lower()}]"
    if prev_quorum is not None:
        prev_ids = {m.replica_id for m in prev_quorum.participants}
        if shrink_only:
            cand = [m for m in cand if m.replica_id in prev_ids]
        cand_ids = {m.replica_id for m in cand}
        if prev_ids and prev_ids <= cand_ids:
            return cand, f"Fast quorum found! {meta}"
    if len(cand) < min_replicas:
        return None, f"New quorum not ready, only have {len(cand)} participants, need min_replicas {min_replicas} {meta}"
    if len(cand) <= len(healthy) // 2:
        return None, f"No quorum, only have {len(cand)} participants, need at least half of {len(healthy)} healthy workers {meta}"
    if len(cand) < len(healthy):
        first = min((t for r, (t, _) in participants.items() if r in healthy), default=now)
        if now - first < join_timeout_s:
            return None, f"Valid quorum with {len(cand)} participants, waiting for {len(healthy) - len(cand)} healthy but not participating stragglers due to join timeout {meta}"
    return cand, f"Valid quorum found {meta}"


class LighthouseServer:
    def __init__(self, bind: str, min_replicas: int, join_timeout_ms: Optional[int] = None,
                 quorum_tick_ms: Optional[int] = None, heartbeat_timeout_ms: Optional[int] = None) -> None:
        self._min = min_replicas
        self._join = (100 if join_timeout_ms is None else join_timeout_ms) / 1e3
        self._tick = (100 if quorum_tick_ms is None else quorum_tick_ms) / 1e3
        self._hb_timeout = (5000 if heartbeat_timeout_ms is None else heartbeat_timeout_ms) / 1e3
        self._cv = threading.Condition()
        self._participants: Dict[str, tuple] = {}
        self._heartbeats: Dict[str, float] = {}
        self._prev: Optional[Quorum] = None
        self._quorum_id = 0
        self._issued = 0  # generation counter of broadcast quorums
        self._stop = threading.Event()
        self._server = _Server(bind, self._handle)
        self._ticker = threading.Thread(target=self._run_tick, daemon=True)
        self._ticker.start()

    def address(self) -> str:
        return f"http://{socket.gethostname()}:{self._server.port}"

    def shutdown(self) -> None:
        self._stop.set()
        self._server.shutdown()

    def _run_tick(self) -> None:
        while not self._stop.wait(self._tick):
            with self._cv:
                self._quorum_tick()

    def _quorum_tick(self) -> None:
        members, _ = quorum_compute(time.monotonic(), self._participants, self._heartbeats, self._prev,
                                    self._min, self._join, self._hb_timeout)
        if members is None:
            return
        changed = self._prev is None or [m.replica_id for m in members] != [m.replica_id for m in self._prev.participants]
        if changed or any(m.commit_failures > 0 for m in members):
            self._quorum_id += 1
        now = time.time()
        self._prev = Quorum(self._quorum_id, members, Timestamp(int(now), int((now % 1) * 1e9)))
        self._participants.clear()
        self._issued += 1
        self._cv.notify_all()

    def _handle(self, method: str, kw: dict, deadline: float):
        if method == "heartbeat":
            with self._cv:
                self._heartbeats[kw["replica_id"]] = time.monotonic()
            return None
        if method == "quorum":
            member: QuorumMember = kw["member"]
            with self._cv:
                while True:
                    self._heartbeats[member.replica_id] = time.monotonic()
                    self._participants[member.replica_id] = (time.monotonic(), member)
                    seen = self._issued
                    self._quorum_tick()
                    while self._issued == seen:
                        left = deadline - time.monotonic()
                        if left <= 0:
                            raise TimeoutError("lighthouse quorum timed out")
                        self._cv.wait(min(left, self._tick))
                        if self._issued == seen:
                            self._heartbeats[member.replica_id] = time.monotonic()
                            self._quorum_tick()
                    q = self._prev
                    assert q is not None
                    if any(m.replica_id == member.replica_id for m in q.participants):
                        return q
        raise RuntimeError(f"unknown lighthouse method {method}")


class LighthouseClient:
    def __init__(self, addr: str, connect_timeout: timedelta) -> None:
        self._c = _Client(addr, connect_timeout)

    def quorum(self, replica_id: str, timeout: timedelta, address: Optional[str] = None,
               store_address: Optional[str] = None, step: Optional[int] = None, world_size: Optional[int] = None,
               shrink_only: Optional[bool] = None, data: Optional[Dict[Hashable, object]] = None) -> Quorum:
        m = QuorumMember(replica_id, address or "", store_address or "", step or 0, world_size or 1,
                         bool(shrink_only), data)
        if data and "commit_failures" in data:
            m.commit_failures = int(data["commit_failures"])  # type: ignore[arg-type]
        return self._c.call("quorum", timeout, member=m)

    def heartbeat(self, replica_id: str, timeout: timedelta = timedelta(seconds=5)) -> None:
        self._c.call("heartbeat", timeout, replica_id=replica_id)


# ----------------------------------------------------------------------------- manager


def compute_quorum_results(replica_id: str, group_rank: int, quorum: Quorum, init_sync: bool) -> QuorumResult:
    parts = sorted(quorum.participants, key=lambda m: m.replica_id)
    ids = [m.replica_id for m in parts]
    if replica_id not in ids:
        raise RuntimeError(f"replica {replica_id} not participating in returned quorum")
    replica_rank = ids.index(replica_id)
    max_step = max(m.step for m in parts)
    max_parts = [m for m in parts if m.step == max_step]
    max_ids = [m.replica_id for m in max_parts]
    max_replica_rank = max_ids.index(replica_id) if replica_id in max_ids else None
    primary = max_parts[group_rank % len(max_parts)]
    force_recover = init_sync and max_step == 0
    recovering = [i for i, m in enumerate(parts)
                  if m.step != max_step or (force_recover and m.replica_id != primary.replica_id)]
    up_to_date = [i for i in range(len(parts)) if i not in recovering]
    assign: Dict[int, int] = {}
    for k, dst in enumerate(recovering):
        assign[dst] = up_to_date[(k + group_rank) % len(up_to_date)]
    heal = replica_rank in assign
    src = assign.get(replica_rank)
    return QuorumResult(
        quorum_id=quorum.quorum_id,
        replica_rank=replica_rank,
        replica_world_size=len(parts),
        recover_src_manager_address=parts[src].address if src is not None else "",
        recover_src_replica_rank=src,
        recover_dst_replica_ranks=[d for d, s in assign.items() if s == replica_rank],
        store_address=primary.store_address,
        max_step=max_step,
        max_replica_rank=max_replica_rank,
        max_world_size=len(max_parts),
        heal=heal,
        commit_failures=max(m.commit_failures for m in parts),
    )


class ManagerServer:
    def __init__(self, replica_id: str, lighthouse_addr: str, hostname: str, bind: str, store_addr: str,
                 world_size: int, heartbeat_interval: timedelta, connect_timeout: timedelta,
                 quorum_retries: int) -> None:
        self._replica_id = replica_id
        self._lh_addr = lighthouse_addr
        self._hostname = hostname
        self._store_addr = store_addr
        self._world = world_size
        self._connect_timeout = connect_timeout
        self._retries = quorum_retries
        self._cv = threading.Condition()
        self._meta: Dict[int, str] = {}
        self._round = 0  # quorum rounds completed
        self._arrived: Dict[int, dict] = {}
        self._result = None  # (round, Quorum | Exception)
        self._commit_round = 0
        self._votes: Dict[int, bool] = {}
        self._decision = None  # (round, bool)
        self._stop = threading.Event()
        self._server = _Server(bind, self._handle)
        self._hb_client = LighthouseClient(lighthouse_addr, connect_timeout)
        self._hb = threading.Thread(target=self._run_heartbeat, args=(heartbeat_interval.total_seconds(),), daemon=True)
        self._hb.start()

    def address(self) -> str:
        return f"http://{self._hostname}:{self._server.port}"

    def shutdown(self) -> None:
        self._stop.set()
        self._server.shutdown()

    def _run_heartbeat(self, interval: float) -> None:
        while not self._stop.wait(interval):
            try:
                self._hb_client.heartbeat(self._replica_id)
            except Exception:  # noqa: BLE001 - the lighthouse may be restarting
                pass

    def _lighthouse_quorum(self, req: dict, timeout_s: float):
        last: Optional[Exception] = None
        for attempt in range(self._retries + 1):
            try:
                c = LighthouseClient(self._lh_addr, self._connect_timeout)
                return c.quorum(self._replica_id, timedelta(seconds=timeout_s), address=self.address(),
                                store_address=self._store_addr, step=req["step"], world_size=self._world,
                                shrink_only=req["shrink_only"], data={"commit_failures": req["commit_failures"]})
            except Exception as e:  # noqa: BLE001
                last = e
                time.sleep(max(0.1, timeout_s / (self._retries + 1)))
        assert last is not None
        return last

    def _handle(self, method: str, kw: dict, deadline: float):
        if method == "quorum":
            with self._cv:
                rnd = self._round
                self._meta[kw["group_rank"]] = kw["checkpoint_metadata"]
                self._arrived[kw["group_rank"]] = kw
                last = len(self._arrived) == self._world
                if last:
                    self._arrived = {}
            if last:
                q = self._lighthouse_quorum(kw, max(deadline - time.monotonic(), 0.1))
                with self._cv:
                    self._result = (rnd, q)
                    self._round += 1
                    self._cv.notify_all()
            with self._cv:
                while self._result is None or self._result[0] != rnd:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        raise TimeoutError("manager quorum timed out")
                    self._cv.wait(left)
                q = self._result[1]
            if isinstance(q, Exception):
                raise q
            return compute_quorum_results(self._replica_id, kw["group_rank"], q, kw["init_sync"])
        if method == "checkpoint_metadata":
            with self._cv:
                if kw["rank"] not in self._meta:
                    raise RuntimeError("rank not found")
                return self._meta[kw["rank"]]
        if method == "should_commit":
            with self._cv:
                rnd = self._commit_round
                self._votes[kw["group_rank"]] = kw["should_commit"]
                if len(self._votes) == self._world:
                    self._decision = (rnd, all(self._votes.values()))
                    self._votes = {}
                    self._commit_round += 1
                    self._cv.notify_all()
                while self._decision is None or self._decision[0] != rnd:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        raise TimeoutError("should_commit timed out")
                    self._cv.wait(left)
                return self._decision[1]
        if method == "kill":
            os._exit(1)
        raise RuntimeError(f"unknown manager method {method}")


class ManagerClient:
    def __init__(self, addr: str, connect_timeout: timedelta) -> None:
        self._c = _Client(addr, connect_timeout)

    def _quorum(self, group_rank: int, step: int, checkpoint_metadata: str, shrink_only: bool,
                timeout: timedelta, init_sync: bool = True, commit_failures: int = 0) -> QuorumResult:
        return self._c.call("quorum", timeout, group_rank=group_rank, step=step,
                            checkpoint_metadata=checkpoint_metadata, shrink_only=shrink_only,
                            init_sync=init_sync, commit_failures=commit_failures)

    def _checkpoint_metadata(self, rank: int, timeout: timedelta) -> str:
        return self._c.call("checkpoint_metadata", timeout, rank=rank)

    def should_commit(self, group_rank: int, step: int, should_commit: bool, timeout: timedelta) -> bool:
        return self._c.call("should_commit", timeout, group_rank=group_rank, step=step,
                            should_commit=should_commit)


def lighthouse_main() -> None:
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--bind", default="[::]:29510")
    ap.add_argument("--min_replicas", type=int, required=True)
    ap.add_argument("--join_timeout_ms", type=int, default=60000)
    ap.add_argument("--quorum_tick_ms", type=int, default=100)
    ap.add_argument("--heartbeat_timeout_ms", type=int, default=5000)
    a = ap.parse_args()
    srv = LighthouseServer(a.bind, a.min_replicas, a.join_timeout_ms, a.quorum_tick_ms, a.heartbeat_timeout_ms)
    print(f"lighthouse (stand-in) listening on {srv.address()}", flush=True)
    threading.Event().wait()


def install(ref_root: str) -> None:
    """Puts the reference's Python package on ``sys.path`` and registers this module as its
    native extension.  ``ref_root`` is the folder that contains the ``torchft`` package."""
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    sys.modules["torchft._torchft"] = sys.modules[__name__]
