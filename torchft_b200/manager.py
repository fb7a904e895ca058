"""Manager: the per-rank state machine of fault-tolerant training.

One :class:`Manager` per trainer process.  Each step it

1. joins the quorum (:meth:`Manager.start_quorum`) -- on a background thread when
   ``use_async_quorum`` so the round trips overlap the forward pass;
2. if the membership changed, reconfigures the replica-dimension process group with the
   store prefix ``<store>/torchft/<quorum_id>/<group_rank>``;
3. serves its state to recovering peers and/or fetches state when it is behind
   (checkpoint transport, on a dedicated CUDA stream);
4. averages tensors over the *participating* replicas (:meth:`Manager.allreduce`), never
   raising: a failed collective latches an error and the step is simply not committed;
5. votes (:meth:`Manager.should_commit`); only when every rank of the group and enough
   replicas are healthy does the step count advance and may the optimizer step.

Public surface and semantics follow torchft/manager.py:137-988 of the reference; the
server side (quorum aggregation, commit barrier) is the C++ control plane.
"""

from __future__ import annotations

import concurrent.futures
import logging
import os
import socket
import threading
import time
import traceback
import uuid
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta
from enum import Enum
from typing import TYPE_CHECKING, Callable, Dict, List, Optional, TypeVar, cast

import torch
import torch.distributed as dist
from torch.distributed import ReduceOp, TCPStore
from torch.distributed.distributed_c10d import AllreduceOptions, Work

from ._ftcp import ManagerClient, ManagerServer
from .checkpointing._rwlock import RWLock
from .checkpointing.http_transport import HTTPTransport
from .checkpointing.transport import CheckpointTransport
from .futures import future_timeout
from .utils.streams import get_stream_context, synchronize
from .work import _DummyWork

if TYPE_CHECKING:
    from .process_group import ProcessGroup

MANAGER_ADDR_KEY: str = "manager_addr"
MANAGER_PORT_ENV: str = "TORCHFT_MANAGER_PORT"
REPLICA_ID_KEY: str = "replica_id"

# Environment overrides (they win over constructor arguments).
TIMEOUT_SEC_ENV: str = "TORCHFT_TIMEOUT_SEC"
PROGRESS_DIR_ENV: str = "FTB200_PROGRESS_DIR"
QUORUM_TIMEOUT_SEC_ENV: str = "TORCHFT_QUORUM_TIMEOUT_SEC"
CONNECT_TIMEOUT_SEC_ENV: str = "TORCHFT_CONNECT_TIMEOUT_SEC"
QUORUM_RETRIES_ENV: str = "TORCHFT_QUORUM_RETRIES"

T = TypeVar("T")


def get_timeout(env_value: Optional[str], default: timedelta) -> timedelta:
    """``env_value`` (seconds, as a string) if set, else ``default``."""
    if env_value is not None:
        return timedelta(seconds=float(env_value))
    return default


class WorldSizeMode(Enum):
    """How the number of participating replicas is chosen.

    DYNAMIC: every healthy replica participates; batch size varies with membership.
    FIXED_WITH_SPARES: exactly ``min_replica_size`` replicas contribute, the others run as
    hot spares whose gradients are zeroed.
    """

    DYNAMIC = 0
    FIXED_WITH_SPARES = 1


class ExceptionWithTraceback(Exception):
    """What :meth:`Manager.errored` returns: the latched exception (``original_exception``) with the stack trace of
    the place where it was reported (``stack_trace``)."""

    def __init__(self, e: Exception) -> None:
        self.original_exception = e
        self.stack_trace: str = traceback.format_exc()
        super().__init__(f"{e}\n{self.stack_trace}")


class _ManagerLogger:
    def __init__(self, manager: "Manager", replica_id: str, group_rank: int) -> None:
        self._logger = logging.getLogger(__name__)
        self._replica_id, self._group_rank, self._manager = replica_id, group_rank, manager

    def prefix(self) -> str:
        return f"[{self._replica_id}/{self._group_rank} - step {self._manager.current_step()}]"

    def info(self, msg: str) -> None:
        self._logger.info(f"{self.prefix()} {msg}")

    def warn(self, msg: str) -> None:
        self._logger.warning(f"{self.prefix()} {msg}")

    def exception(self, msg: str) -> None:
        self._logger.exception(f"{self.prefix()} {msg}")


class Manager:
    """See the module docstring.  When saving durable checkpoints, save and restore this
    object's :meth:`state_dict` as well (step and batch counters)."""

    def __init__(
        self,
        pg: "ProcessGroup",
        load_state_dict: Optional[Callable[[T], None]],
        state_dict: Optional[Callable[[], T]],
        min_replica_size: int,
        use_async_quorum: bool = True,
        timeout: timedelta = timedelta(seconds=60),
        quorum_timeout: timedelta = timedelta(seconds=60),
        connect_timeout: timedelta = timedelta(seconds=60),
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        world_size_mode: WorldSizeMode = WorldSizeMode.DYNAMIC,
        store_addr: Optional[str] = None,
        store_port: Optional[int] = None,
        lighthouse_addr: Optional[str] = None,
        replica_id: Optional[str] = None,
        port: Optional[int] = None,
        hostname: str = socket.gethostname(),
        heartbeat_interval: timedelta = timedelta(milliseconds=100),
        checkpoint_transport: Optional[CheckpointTransport[Dict[str, T]]] = None,
        init_sync: bool = True,
        max_retries: Optional[int] = None,
        quorum_retries: int = 0,
    ) -> None:
        """
        Args:
            pg: reconfigurable process group spanning the replica dimension
            load_state_dict / state_dict: callables that restore / snapshot the user's
                state when a replica heals (may be None if ``register_state_dict_fn`` is used)
            min_replica_size: minimum number of participating replicas for a step to commit
            use_async_quorum: overlap the quorum with the forward pass
            timeout: default for collectives, should_commit, checkpoint operations, wrap_future
            quorum_timeout: how long a quorum request may wait (should exceed the step time)
            connect_timeout: for connections to the manager server and the lighthouse
            rank / world_size: position inside the replica group (default: RANK / WORLD_SIZE)
            store_addr / store_port: the replica group's TCPStore (default: MASTER_ADDR / MASTER_PORT)
            lighthouse_addr: on group rank 0, the lighthouse (default: TORCHFT_LIGHTHOUSE)
            replica_id: on group rank 0, a prefix for this group's identity; a fresh UUID is
                appended on every start so that a quick restart counts as a new member
            port: on group rank 0, manager server port (then TORCHFT_MANAGER_PORT, then any)
            checkpoint_transport: how healing replicas get state (default HTTPTransport)
            init_sync: synchronise weights from the primary replica at step 0
            max_retries: consecutive failed commits tolerated before raising (None: forever)
            quorum_retries: lighthouse quorum attempts before the round fails
        """
        self.quorum_logger: logging.Logger = logging.getLogger("torchft_quorums")
        self.commits_logger: logging.Logger = logging.getLogger("torchft_commits")
        self.errors_logger: logging.Logger = logging.getLogger("torchft_errors")

        self._load_state_dict_fns: Dict[str, Callable[[object], None]] = {}
        self._user_state_dicts: Dict[str, Callable[[], object]] = {}
        self._replica_id = replica_id

        self._timeout = get_timeout(os.environ.get(TIMEOUT_SEC_ENV), timeout)
        self._quorum_timeout = get_timeout(os.environ.get(QUORUM_TIMEOUT_SEC_ENV), quorum_timeout)
        self._connect_timeout = get_timeout(os.environ.get(CONNECT_TIMEOUT_SEC_ENV), connect_timeout)
        self._state_dict_lock = RWLock(timeout=self._timeout.total_seconds())
        if load_state_dict and state_dict:
            self.register_state_dict_fn("default", load_state_dict, state_dict)

        self._pending_state_dict: Optional[Dict[str, object]] = None
        self._use_async_quorum = use_async_quorum
        self._replica_world_size_mode = world_size_mode
        self._init_sync = init_sync
        self._max_retries = max_retries
        self._commit_failures = 0
        self._quorum_retries = int(os.environ.get(QUORUM_RETRIES_ENV, str(quorum_retries)))

        store_addr = store_addr or os.environ["MASTER_ADDR"]
        store_port = store_port or int(os.environ["MASTER_PORT"])
        self._group_rank: int = rank if rank is not None else int(os.environ["RANK"])
        group_world_size = world_size or int(os.environ["WORLD_SIZE"])
        self._group_world_size = group_world_size
        self._min_replica_size = min_replica_size

        if checkpoint_transport is None:
            checkpoint_transport = HTTPTransport[Dict[str, T]](timeout=self._timeout, num_chunks=0)
        self._checkpoint_transport = checkpoint_transport
        self._executor = ThreadPoolExecutor(max_workers=1, thread_name_prefix="torchft_quorum")
        self._quorum_future: Optional[concurrent.futures.Future] = None

        # connect_timeout bounds reaching the group's store and, below, waiting for rank 0 to publish the manager
        # address (torch's default of five minutes turns a wrong address into a very long silence)
        self._store = TCPStore(host_name=store_addr, port=store_port, is_master=False, wait_for_workers=False,
                               timeout=self._connect_timeout)
        self._pg = pg
        self._manager: Optional[ManagerServer] = None
        self._recovery_stream: Optional[torch.cuda.Stream] = torch.cuda.Stream() if torch.cuda.is_available() else None
        self._recovery_event: Optional[torch.cuda.Event] = None

        if self._group_rank == 0:
            if port is None:
                port = int(os.environ.get(MANAGER_PORT_ENV, 0))
            lighthouse_addr = lighthouse_addr or os.environ["TORCHFT_LIGHTHOUSE"]
            unique = str(uuid.uuid4())
            replica_id = unique if not replica_id else f"{replica_id}:{unique}"
            self._manager = ManagerServer(
                replica_id=replica_id,
                lighthouse_addr=lighthouse_addr,
                hostname=hostname,
                bind=f"[::]:{port}",
                store_addr=f"{store_addr}:{store_port}",
                world_size=group_world_size,
                heartbeat_interval=heartbeat_interval,
                connect_timeout=self._connect_timeout,
                quorum_retries=self._quorum_retries,
            )
            self._store.set(MANAGER_ADDR_KEY, self._manager.address())
            self._store.set(REPLICA_ID_KEY, replica_id)

        # the other ranks of the group block here until rank 0's server is up
        addr = self._store.get(MANAGER_ADDR_KEY).decode("utf-8")
        self._client = ManagerClient(self._local_addr(addr, hostname), connect_timeout=self._connect_timeout)
        replica_id = self._store.get(REPLICA_ID_KEY).decode("utf-8")
        self._replica_id = replica_id
        self._logger = _ManagerLogger(manager=self, replica_id=replica_id or "", group_rank=self._group_rank)
        # Progress beacon for a supervisor (launch/runner.py): a file rewritten at every commit vote.  Heartbeats
        # come from the manager server's own thread and keep flowing while a trainer is stuck; this does not.
        self._progress_file: Optional[str] = None
        progress_dir = os.environ.get(PROGRESS_DIR_ENV)
        if progress_dir:
            group = os.environ.get("REPLICA_GROUP_ID", (replica_id or "replica").split(":")[0])
            self._progress_file = os.path.join(progress_dir, f"group{group}.rank{self._group_rank}")

        self._step = 0
        self._quorum_id = -1
        self._errored: Optional[ExceptionWithTraceback] = None
        self._healing = False
        self.last_quorum_phases: Dict[str, float] = {}
        self._batches_committed = 0
        self._participating_replica_rank: Optional[int] = None
        self._participating_replica_world_size: int = 0
        self._is_state_dict_read_allowed = True

    @staticmethod
    def _local_addr(addr: str, hostname: str) -> str:
        """Managers advertise ``http://<hostname>:port``; when that host is this machine,
        dial ``localhost`` so an unresolvable container hostname does not matter."""
        if hostname and f"//{hostname}:" in addr and hostname == socket.gethostname():
            return addr.replace(f"//{hostname}:", "//localhost:")
        return addr

    # ------------------------------------------------------------------ user state
    def allow_state_dict_read(self) -> None:
        """Let peers read the state dict again (after the optimizer finished mutating it)."""
        if self._is_state_dict_read_allowed:
            return
        self._is_state_dict_read_allowed = True
        self._state_dict_lock.w_release()

    def disallow_state_dict_read(self) -> None:
        """Block state-dict readers (call before the optimizer mutates the weights)."""
        if not self._is_state_dict_read_allowed:
            return
        self._is_state_dict_read_allowed = False
        self._state_dict_lock.w_acquire()

    def register_state_dict_fn(self, key: str, load_state_dict: Callable[[T], None], state_dict: Callable[[], T]) -> None:
        """Add a named piece of user state to what healing transfers."""
        assert key not in self._load_state_dict_fns, f"{key} already registered"
        assert key not in self._user_state_dicts, f"{key} already registered"
        self._load_state_dict_fns[key] = cast(Callable[[object], None], load_state_dict)
        self._user_state_dicts[key] = state_dict

    def set_state_dict_fns(self, load_state_dict: Callable[[T], None], state_dict: Callable[[], T]) -> None:
        self._load_state_dict_fns["default"] = cast(Callable[[object], None], load_state_dict)
        self._user_state_dicts["default"] = state_dict

    # ------------------------------------------------------------------ lifecycle
    def shutdown(self, wait: bool = True) -> None:
        """Stop the manager server, the checkpoint transport and the quorum thread."""
        self._checkpoint_transport.shutdown(wait=wait)
        if self._manager is not None:
            self._manager.shutdown()
        self._executor.shutdown(wait=wait)

    # ------------------------------------------------------------------ collectives
    def allreduce(self, tensor: torch.Tensor, should_quantize: bool = False,
                  reduce_op: ReduceOp = ReduceOp.AVG) -> Work:
        """Fault-tolerant allreduce over the participating replicas.

        ``AVG`` (default) divides by the number of participants.  Never raises: after the
        first error of a step every call returns a completed dummy work, the tensor's
        content is then undefined and the step will not commit.  A replica that is healing
        or is a spare contributes zeros.  ``should_quantize`` sends block-scaled fp8
        instead of the tensor's dtype (CUDA tensors only).
        """
        with torch.profiler.record_function("torchft::manager::allreduce"):
            if self.errored():
                return _DummyWork(tensor)
            self.wait_quorum()
            num_participants = self.num_participants()
            if not self.is_participating():
                tensor.zero_()

            pg_op = reduce_op
            if reduce_op == ReduceOp.AVG:
                if not torch.is_floating_point(tensor):
                    raise ValueError("average reduce op is only supported for floating point tensors")
                pg_op = ReduceOp.SUM
            try:
                quantized = should_quantize and tensor.is_cuda
                # (the quantised collective reduces with SUM: the division below must then happen here, whatever
                # the group could have fused into an unquantised allreduce)
                fused_scale = (getattr(self._pg, "supports_fused_scale", False) and reduce_op == ReduceOp.AVG
                               and not quantized)
                if quantized:
                    from .collectives import allreduce_quantized

                    work = allreduce_quantized([tensor], pg_op, self._pg, torch.cuda.current_stream())
                elif fused_scale:
                    # the peer-memory kernel folds 1/num_participants (and the cast) into the reduction
                    work = self._pg.allreduce([tensor], pg_op, scale=1.0 / max(1, num_participants))  # type: ignore[call-arg]
                else:
                    opts = AllreduceOptions()
                    opts.reduceOp = pg_op
                    work = self._pg.allreduce([tensor], opts)

                def normalize(fut: torch.futures.Future) -> torch.Tensor:
                    with torch.profiler.record_function("torchft::manager::allreduce::callback"):
                        nonlocal tensor
                        if reduce_op == ReduceOp.AVG and not fused_scale:
                            tensor /= num_participants
                        return tensor

                managed = _ManagedWork(self, work, tensor)
                managed.get_future().then(normalize)
                return managed
            except Exception as e:
                self._logger.exception(f"got exception in all reduce -- skipping remaining: {e}")
                self.report_error(e)
                return _DummyWork(tensor)

    def allreduce_delta(self, out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, should_quantize: bool = False) -> Work:
        """``out`` = average over the participating replicas of ``a - b`` (flat tensors of one
        dtype and size); the pseudo-gradient exchange of LocalSGD/DiLoCo.  On a process group
        with a fused quantised allreduce (``allreduce_fp8``) and ``should_quantize``, the
        difference, the quantisation, the reduction and the division are one kernel per rank
        and ``a - b`` is never written to memory; otherwise this is ``out = a - b`` followed
        by :meth:`allreduce`.  Error behaviour is that of :meth:`allreduce`.
        """
        fused = (should_quantize and out.is_cuda and hasattr(self._pg, "allreduce_fp8")
                 and out.is_contiguous() and a.is_contiguous() and b.is_contiguous())
        if fused:
            if self.errored():
                return _DummyWork(out)
            self.wait_quorum()
            fused = out.numel() % (128 * max(1, self._pg.size())) == 0
        if not fused:
            torch.sub(a, b, out=out)
            return self.allreduce(out, should_quantize=should_quantize)
        with torch.profiler.record_function("torchft::manager::allreduce_delta"):
            try:
                self._pg.allreduce_fp8(  # type: ignore[attr-defined]
                    a.view(-1), out.view(-1), 1.0 / max(1, self.num_participants()), minus=b.view(-1),
                    zero_contribution=not self.is_participating())
                ev = torch.cuda.Event()
                ev.record()
                from .collectives import _StreamOrderedWork

                return _ManagedWork(self, _StreamOrderedWork(ev, [out]), out)
            except Exception as e:
                self._logger.exception(f"got exception in allreduce_delta -- skipping remaining: {e}")
                self.report_error(e)
                return _DummyWork(out)

    def report_error(self, e: Exception) -> None:
        """Latch an error: the current step will not commit and the rest of its
        collectives become no-ops.  Cleared by the next :meth:`start_quorum`."""
        self._errored = ExceptionWithTraceback(e)

    def errored(self) -> Optional[ExceptionWithTraceback]:
        return self._errored

    def wrap_future(self, fut: torch.futures.Future, default: T, timeout: Optional[timedelta] = None) -> torch.futures.Future:
        """Bound ``fut`` by a timeout and swallow its failure: on error or timeout the
        returned future resolves to ``default`` and the error is latched."""
        timed = future_timeout(fut, timeout or self._timeout)
        stream = torch.cuda.current_stream() if torch.cuda.is_available() else None

        def swallow(f: torch.futures.Future) -> T:
            with get_stream_context(stream):
                try:
                    return f.value()
                except Exception as e:
                    self._logger.exception(f"got exception in future -- skipping remaining: {e}")
                    self.report_error(e)
                    return default

        return timed.then(swallow)

    # ------------------------------------------------------------------ quorum
    def start_quorum(self, allow_heal: bool = True, shrink_only: bool = False,
                     timeout: Optional[timedelta] = None) -> None:
        """Begin a step: join the quorum (asynchronously when configured so) and clear the
        error latch.  Call before the forward pass.  ``allow_heal=False`` keeps a behind
        replica from fetching state (all replicas must pass the same value);
        ``shrink_only`` forbids this quorum to grow."""
        if self._quorum_future is not None:
            self._quorum_future.result()  # previous round must be over
        self._errored = None
        self._healing = False
        self._quorum_future = self._executor.submit(
            self._async_quorum,
            allow_heal=allow_heal,
            shrink_only=shrink_only,
            quorum_timeout=timeout or self._quorum_timeout,
            curr_device=torch.cuda.current_device() if torch.cuda.is_available() else -1,
        )
        if not self._use_async_quorum:
            self.wait_quorum()
            if self._healing:
                # synchronous mode: restore state now so the forward pass runs on good weights
                self._apply_pending_state_dict()
                self._healing = False

    def wait_quorum(self) -> None:
        """Block until the quorum round (and any reconfiguration/recovery it started) is done."""
        assert self._quorum_future is not None, "must call start_quorum before wait_quorum"
        with torch.profiler.record_function("torchft::manager::wait_quorum"):
            self._quorum_future.result()

    def _async_quorum(self, allow_heal: bool, shrink_only: bool, quorum_timeout: timedelta, curr_device: int) -> None:
        with torch.profiler.record_function("torchft::manager::_async_quorum"):
            self._async_quorum_impl(allow_heal, shrink_only, quorum_timeout, curr_device)

    def _async_quorum_impl(self, allow_heal: bool, shrink_only: bool, quorum_timeout: timedelta, curr_device: int) -> None:
        threading.current_thread().name = "torchft_quorum"
        if curr_device >= 0 and torch.cuda.is_available():
            torch.cuda.set_device(curr_device)

        # host time of the phases of this quorum (seconds): what a slow step of a serving or healing replica is made of
        phases: Dict[str, float] = {}
        self.last_quorum_phases = phases
        t_phase = time.perf_counter()
        with torch.profiler.record_function("torchft::manager::_client::_quorum"):
            quorum = self._client._quorum(
                group_rank=self._group_rank,
                step=self._step,
                checkpoint_metadata=self._checkpoint_transport.metadata(),
                shrink_only=shrink_only,
                timeout=quorum_timeout,
                init_sync=self._init_sync,
                commit_failures=self._commit_failures,
            )

        phases["quorum_rpc_s"] = time.perf_counter() - t_phase
        # With async quorum (or healing disabled) only replicas already at the max step
        # count; with a synchronous quorum everyone has healed before the step runs.
        if self._use_async_quorum or not allow_heal:
            self._participating_replica_rank = quorum.max_replica_rank
            self._participating_replica_world_size = quorum.max_world_size
        else:
            self._participating_replica_rank = quorum.replica_rank
            self._participating_replica_world_size = quorum.replica_world_size

        if self._replica_world_size_mode == WorldSizeMode.FIXED_WITH_SPARES:
            self._participating_replica_world_size = min(self._participating_replica_world_size, self._min_replica_size)
            if (self._participating_replica_rank is not None
                    and self._participating_replica_rank >= self._min_replica_size):
                self._participating_replica_rank = None

        if quorum.quorum_id != self._quorum_id:
            self.quorum_logger.info(
                "",
                extra={
                    "job_id": os.environ.get("JOB_ID", "unknown"),
                    "replica_id": self._replica_id,
                    "rank": self._group_rank,
                    "quorum_id": quorum.quorum_id,
                    "step": quorum.max_step,
                },
            )
            prefixed = f"{quorum.store_address}/torchft/{quorum.quorum_id}/{self._group_rank}"
            self._logger.info(f"reconfiguring for quorum_id={quorum.quorum_id} store_prefixed_addr={prefixed}")
            t_phase = time.perf_counter()
            try:
                with torch.profiler.record_function("torchft::manager::_pg::configure"):
                    if torch.cuda.is_available():
                        torch.cuda.synchronize()
                    # all replicas join the group, also those that are still behind
                    self._pg.configure(prefixed, self._replica_id if self._replica_id is not None else "0",
                                       quorum.replica_rank, quorum.replica_world_size)
                self._quorum_id = quorum.quorum_id
                phases["configure_s"] = time.perf_counter() - t_phase
            except Exception as e:
                self._logger.exception(f"got exception in pg configure: {e}")
                self.report_error(e)
                return

        if allow_heal:
            with get_stream_context(self._recovery_stream):
                try:
                    if quorum.recover_dst_replica_ranks:
                        self._logger.info(f"peers need recovery from us {quorum.recover_dst_replica_ranks}")
                        t_phase = time.perf_counter()
                        with torch.profiler.record_function("torchft::manager::_checkpoint_transport::send_checkpoint"):
                            self._checkpoint_transport.send_checkpoint(
                                dst_ranks=quorum.recover_dst_replica_ranks,
                                step=quorum.max_step,
                                state_dict=self._manager_state_dict(),
                                timeout=self._timeout,
                            )
                        phases["send_checkpoint_s"] = time.perf_counter() - t_phase
                    if quorum.heal:
                        self._healing = True
                        src_addr = quorum.recover_src_manager_address
                        self._logger.info(f"healing required, fetching checkpoint metadata from {src_addr} max_step={quorum.max_step}")
                        primary = ManagerClient(self._local_addr(src_addr, socket.gethostname()),
                                                connect_timeout=self._connect_timeout)
                        metadata = primary._checkpoint_metadata(self._group_rank, timeout=self._timeout)
                        src_rank = quorum.recover_src_replica_rank
                        assert src_rank is not None, "must have a recover rank when healing"
                        self._logger.info(f"fetching checkpoint from recover_src_replica_rank={src_rank} with metadata={metadata}")
                        t_phase = time.perf_counter()
                        with torch.profiler.record_function("torchft::manager::_checkpoint_transport::recv_checkpoint"):
                            # the user part is applied later from the main thread (should_commit)
                            self._pending_state_dict = self._checkpoint_transport.recv_checkpoint(
                                src_rank=src_rank, metadata=metadata, step=quorum.max_step, timeout=self._timeout)
                        phases["recv_checkpoint_s"] = time.perf_counter() - t_phase
                        self.load_state_dict(cast(Dict[str, int], self._pending_state_dict["torchft"]))
                        self._step = quorum.max_step
                except Exception as e:
                    self._logger.exception(f"got exception in recovery: {e}")
                    self.report_error(e)
                self._recovery_event = (
                    torch.cuda.current_stream().record_event() if self._recovery_stream is not None else None
                )

    def _apply_pending_state_dict(self) -> None:
        assert self._healing, "must be in healing state"
        assert self._quorum_future is not None, "must call step before should_commit"
        self._quorum_future.result()
        pending = self._pending_state_dict
        if pending is None:
            assert self.errored(), "checkpoint was not staged and no error occured"
            return
        self._logger.info("applying pending state dict")
        assert len(self._load_state_dict_fns) > 0, "user load_state_dict is not initialized."
        user = cast(Dict[str, object], pending["user"])
        for key, load in self._load_state_dict_fns.items():
            load(user[key])
        self._pending_state_dict = None
        self._logger.info("Loaded state dict.")

    # ------------------------------------------------------------------ commit
    def should_commit(self, timeout: Optional[timedelta] = None) -> bool:
        """Vote on the step; call after backward, exactly once per step, on every rank of
        the group.  Returns True iff the optimizer may step (same answer on all ranks of
        the group; groups may differ).  Raises ``RuntimeError`` after more than
        ``max_retries`` consecutive failures."""
        with torch.profiler.record_function("torchft::manager::should_commit"):
            if self._recovery_event is not None:
                self._recovery_event.synchronize()
                self._recovery_event = None
            if torch.cuda.is_available():
                synchronize()  # this is where asynchronous collective failures surface
            err = self._pg.errored()
            if err:
                self.report_error(err)
            if self._healing:
                self._apply_pending_state_dict()

            enough_replicas = self.num_participants() >= self._min_replica_size
            local = enough_replicas and self._errored is None
            decision = self._client.should_commit(self._group_rank, self._step, local, timeout=timeout or self._timeout)
            self._logger.info(f"should_commit={decision} enough_replicas={enough_replicas}, errored={self._errored}")
            self.commits_logger.info(
                "",
                extra={
                    "job_id": os.environ.get("JOB_ID", "unknown"),
                    "replica_id": self._replica_id,
                    "rank": self._group_rank,
                    "quorum_id": self._quorum_id,
                    "step": self._step,
                    "commit_result": decision,
                },
            )
            self._checkpoint_transport.disallow_checkpoint()
            if decision:
                self._step += 1
                self._batches_committed += self.num_participants()
                self._commit_failures = 0
            else:
                self._commit_failures += 1
                if self._max_retries is not None and self._commit_failures > self._max_retries:
                    msg = (f"should_commit failed {self._commit_failures} times consecutively, "
                           f"exceeding max_retries={self._max_retries}")
                    self._logger.exception(msg)
                    raise RuntimeError(msg)
            self._write_progress()
            return decision

    def _write_progress(self) -> None:
        if self._progress_file is None:
            return
        try:
            os.makedirs(os.path.dirname(self._progress_file), exist_ok=True)
            with open(self._progress_file, "w") as f:
                f.write(f"{self._step}\n")
        except OSError:  # a beacon must never take training down
            pass

    # ------------------------------------------------------------------ state
    def load_state_dict(self, state_dict: Dict[str, int]) -> None:
        """Restore step and batch counters from a previous :meth:`state_dict`."""
        self._step = state_dict["step"]
        self._batches_committed = state_dict["batches_committed"]

    def _manager_state_dict(self) -> Dict[str, object]:
        with self._state_dict_lock.r_lock():
            assert len(self._user_state_dicts) > 0, "user state_dict is not initialized."
            return {
                "user": {key: fn() for key, fn in self._user_state_dicts.items()},
                "torchft": self.state_dict(),
            }

    def state_dict(self) -> Dict[str, int]:
        return {"step": self._step, "batches_committed": self._batches_committed}

    def current_step(self) -> int:
        """Number of committed steps."""
        return self._step

    def batches_committed(self) -> int:
        """Sum over committed steps of the number of participating replicas."""
        return self._batches_committed

    def participating_rank(self) -> Optional[int]:
        """Rank of this replica among the participants (None when not participating).
        Blocks on an unfinished quorum."""
        if self._quorum_future is None:
            return None
        self.wait_quorum()
        return self._participating_replica_rank

    def num_participants(self) -> int:
        """Number of replicas whose data counts this step.  Blocks on an unfinished quorum."""
        if self._quorum_future is None:
            return 0
        self.wait_quorum()
        assert self._participating_replica_world_size >= 0, "internal error"
        return self._participating_replica_world_size

    def is_participating(self) -> bool:
        if self._participating_replica_rank is None:
            return False
        if self._healing:
            assert self._use_async_quorum
            return False
        return True


class _ManagedFuture(torch.futures.Future):
    """Future handed out by :class:`_ManagedWork`: ``then`` callbacks are recorded, not
    attached, until the work is waited on -- they then run in order, on the stream that
    was current when the work was created, and the first link is guarded by
    ``Manager.wrap_future`` (timeout + error latch)."""

    def __init__(self, owner: "_ManagedWork") -> None:
        super().__init__()
        self._owner = owner

    def then(self, callback: Callable[[torch.futures.Future], object]) -> "_ManagedFuture":
        self._owner._callbacks.append(callback)
        return self

    def wait(self) -> object:
        self._owner.wait()
        return self._owner._final().wait()

    def value(self) -> object:
        return self._owner._final().value()

    def done(self) -> bool:
        f = self._owner._resolved
        return f is not None and f.done()

    def add_done_callback(self, callback: Callable[[torch.futures.Future], None]) -> None:
        self._owner._callbacks.append(lambda f: (callback(f), f.value())[1])


class _ManagedWork(dist._Work):
    """``Work`` returned by :meth:`Manager.allreduce`."""

    def __init__(self, manager: Manager, work: Work, value: object) -> None:
        super().__init__()
        self._manager = manager
        self._work = work
        self._value = value
        self._callbacks: List[Callable[[torch.futures.Future], object]] = []
        self._resolved: Optional[torch.futures.Future] = None
        self._future = _ManagedFuture(self)
        self._stream = torch.cuda.current_stream() if torch.cuda.is_available() else None
        self._lock = threading.Lock()

    def _final(self) -> torch.futures.Future:
        self._attach()
        assert self._resolved is not None
        return self._resolved

    def _attach(self) -> None:
        with self._lock:
            if self._resolved is not None:
                return
            callbacks = self._callbacks
            stream = self._stream

            def chain(f: torch.futures.Future) -> object:
                # runs once the collective is done; apply the recorded callbacks in order
                with get_stream_context(stream):
                    f.value()  # a failed collective fails the whole chain (reported by wrap_future)
                    cur: torch.futures.Future = f
                    for cb in callbacks:
                        nxt: torch.futures.Future = torch.futures.Future()
                        try:
                            nxt.set_result(cb(cur))
                        except Exception as e:
                            nxt.set_exception(e)
                        cur = nxt
                    return cur.value()

            fut = self._work.get_future().then(chain)
            self._resolved = self._manager.wrap_future(fut, self._value)

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        with get_stream_context(self._stream):
            try:
                if timeout is not None:
                    self._work.wait(timeout)
                else:
                    self._work.wait()
            except Exception as e:
                self._manager._logger.exception(f"got exception waiting for work: {e}")
                self._manager.report_error(e)
                return True
            self._attach()
            assert self._resolved is not None
            self._resolved.wait()
        return True

    def block_current_stream(self, timeout: Optional[timedelta] = None) -> None:
        self.wait(timeout)

    def synchronize(self) -> None:
        self.wait()

    def get_future(self) -> torch.futures.Future:
        return self._future

    def is_completed(self) -> bool:
        return self._resolved is not None and self._resolved.done()
