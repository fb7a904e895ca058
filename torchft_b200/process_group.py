"""Reconfigurable, abortable process groups.

A fault-tolerant job changes its replica world on (almost) any step, so a process group
here is a long-lived *shell* whose communicator is rebuilt by :meth:`ProcessGroup.configure`
each time the quorum changes, can be aborted from a timer thread when a peer dies mid
collective, and reports such failures through :meth:`ProcessGroup.errored` instead of
hanging or raising inside the training loop.

Classes (the same cast as torchft/process_group.py in the reference):

* :class:`ProcessGroup` -- the c10d-compatible base with ``configure/abort/shutdown/
  errored/set_timeout/register``;
* :class:`ProcessGroupWrapper` -- owns an inner ``torch.distributed`` backend recreated on
  every ``configure`` from a ``host:port/prefix`` store address;
* :class:`ProcessGroupGloo`, :class:`ProcessGroupNCCL` -- concrete back-ends; the NCCL
  one uses non-blocking communicators, aborts on host or stream timeouts and latches the
  error;
* :class:`ProcessGroupDummy` -- world of one that copies inputs to outputs;
* :class:`ErrorSwallowingProcessGroupWrapper`, :class:`FakeProcessGroupWrapper` -- error
  containment and fault injection;
* :class:`ManagedProcessGroup` -- facade whose allreduce goes through a ``Manager``;
* the subprocess-isolated ``ProcessGroupBaby*`` family lives in
  :mod:`torchft_b200.process_group_baby` and is re-exported here.

The NVLink peer-memory group (``ProcessGroupB200``) is in :mod:`torchft_b200.parallel.team`.
"""

from __future__ import annotations

import logging
import os
from contextlib import contextmanager
from datetime import timedelta
from typing import TYPE_CHECKING, Callable, Generator, List, Optional

import torch
import torch.distributed as dist
from torch.distributed import ProcessGroup as BaseProcessGroup, ProcessGroupGloo as BaseProcessGroupGloo, Store
from torch.distributed.distributed_c10d import (
    AllgatherOptions,
    AllreduceCoalescedOptions,
    AllreduceOptions,
    AllToAllOptions,
    BarrierOptions,
    BroadcastOptions,
    ReduceOp,
    ReduceScatterOptions,
    Work,
)
from torch.futures import Future

from .futures import context_timeout, stream_timeout
from .work import _DummyWork

if TYPE_CHECKING:
    from .manager import Manager

try:
    from torch.distributed import ProcessGroupNCCL as BaseProcessGroupNCCL
except ImportError:  # pragma: no cover - CPU-only torch builds
    BaseProcessGroupNCCL = None  # type: ignore

logger = logging.getLogger(__name__)

TORCH_NCCL_DEBUG_INFO_PIPE_FILE_ENV_VAR = "TORCH_NCCL_DEBUG_INFO_PIPE_FILE"
TORCHFT_TRIGGER_FR_ON_ABORT = "TORCHFT_TRIGGER_FR_ON_ABORT"


def trigger_nccl_fr_trace_through_pipe(rank: int) -> bool:
    """Ask NCCL's flight recorder to dump by writing to the debug pipe that
    ``TORCH_NCCL_DEBUG_INFO_PIPE_FILE`` names (``<path><rank>.pipe``)."""
    base = os.environ.get(TORCH_NCCL_DEBUG_INFO_PIPE_FILE_ENV_VAR)
    if base is None:
        return False
    path = f"{base}{rank}.pipe"
    try:
        with open(path, "w") as f:
            f.write("1\n")
        return True
    except OSError as e:
        logger.warning("could not trigger flight-recorder dump through %s: %s", path, e)
        return False


from ._pg_base import ProcessGroup, _reduce_op, create_store_client  # noqa: E402,F401


class _TimedWork(Work):
    """Delegating ``Work`` whose ``wait`` is bounded by a host timeout that aborts the group."""

    def __init__(self, pg: "ProcessGroupWrapper", work: Work, timeout: timedelta) -> None:
        super().__init__()
        self._pg, self._work, self._timeout = pg, work, timeout

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        t = timeout or self._timeout
        with self._pg._run_context():
            with context_timeout(self._pg._timeout_abort, t):
                ok = self._work.wait(t) if timeout is not None else self._work.wait()
        return ok

    def get_future(self) -> Future:
        return self._work.get_future()

    def is_completed(self) -> bool:
        return self._work.is_completed()

    def synchronize(self) -> None:
        self._work.synchronize()

    def block_current_stream(self, timeout: Optional[timedelta] = None) -> None:
        try:
            self._work.block_current_stream()
        except (AttributeError, RuntimeError):
            self._work.wait()


class ProcessGroupWrapper(ProcessGroup):
    """Shell around an inner torch.distributed process group recreated on every ``configure``."""

    def __init__(self, timeout: timedelta = timedelta(seconds=60), pg: Optional[ProcessGroup] = None) -> None:
        super().__init__(0, 1)
        self._pg: Optional[BaseProcessGroup] = pg
        self._timeout = timeout
        self._replica_id: Optional[str] = None
        self._rank: Optional[int] = None
        self._quorum_id: Optional[int] = None
        self.errors_logger = logging.getLogger("torchft_errors")

    # ---- hooks for subclasses
    def _create_pg(self, store: Store, rank: int, world_size: int) -> BaseProcessGroup:
        raise NotImplementedError("_create_pg")

    def _wrap_work(self, work: Work, opts: object) -> Work:
        return _TimedWork(self, work, self._timeout)

    def _opts_hook(self, opts):
        return opts

    @contextmanager
    def _run_context(self) -> Generator[None, None, None]:
        yield

    def _timeout_abort(self) -> None:
        logger.error("%s: collective timed out after %s, aborting", self, self._timeout)
        self.abort()

    # ---- lifecycle
    def set_timeout(self, timeout: timedelta) -> None:
        self._timeout = timeout

    def getBackendName(self) -> str:
        pg = self._pg
        if isinstance(pg, ProcessGroup):
            return pg.getBackendName()
        raise NotImplementedError("getBackendName")

    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int,
                  quorum_id: Optional[int] = None) -> None:
        pg = self._pg
        self._replica_id, self._rank, self._quorum_id = replica_id, rank, quorum_id
        if isinstance(pg, ProcessGroup):
            pg.configure(store_addr, replica_id, rank, world_size)
            return
        # abort the previous communicator first: its peers may be gone
        self.abort(errored=False)
        store = create_store_client(store_addr, timeout=self._timeout)
        self._pg = self._create_pg(store, rank, world_size)

    def abort(self, errored: bool = True) -> None:
        if errored:
            self.errors_logger.info(
                "",
                extra={
                    "job_id": os.environ.get("JOB_ID", "unknown"),
                    "replica_id": self._replica_id,
                    "rank": self._rank,
                    "quorum_id": self._quorum_id,
                    "error": "process_group_abort",
                },
            )
        pg = self._pg
        if pg is not None:
            if hasattr(pg, "abort"):
                pg.abort()
            else:
                try:
                    backend = pg._get_backend(torch.device("cuda"))
                    backend.abort()
                except Exception:
                    pass
        self._pg = None

    def shutdown(self) -> None:
        pg = self._pg
        if pg is not None:
            if hasattr(pg, "shutdown"):
                pg.shutdown()
            self._pg = None

    def size(self) -> int:
        return self.parent.size()

    @property
    def parent(self) -> BaseProcessGroup:
        pg = self._pg
        if pg is None:
            raise RuntimeError("process group is not configured (or was aborted)")
        return pg

    # ---- collectives: forward to the inner group inside the run context, bounded by a host timeout
    def _run(self, fn: Callable[[BaseProcessGroup], Work], opts: object = None) -> Work:
        with self._run_context():
            with context_timeout(self._timeout_abort, self._timeout):
                work = fn(self.parent)
        return self._wrap_work(work, opts)

    def allgather(self, output_tensors, input_tensor, opts=None) -> Work:
        opts = self._opts_hook(opts or AllgatherOptions())
        return self._run(lambda pg: pg.allgather(output_tensors, input_tensor, opts), opts)

    def allgather_into_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        opts = self._opts_hook(opts or AllgatherOptions())
        return self._run(lambda pg: pg.allgather_into_tensor_coalesced(output_tensors, input_tensors, opts), opts)

    def allreduce(self, tensors, opts=None) -> Work:
        if not isinstance(opts, AllreduceOptions):
            o = AllreduceOptions()
            o.reduceOp = _reduce_op(opts)
            opts = o
        opts = self._opts_hook(opts)
        return self._run(lambda pg: pg.allreduce(tensors, opts), opts)

    def allreduce_coalesced(self, tensors, opts=None) -> Work:
        if not isinstance(opts, AllreduceCoalescedOptions):
            o = AllreduceCoalescedOptions()
            if opts is not None:
                o.reduceOp = _reduce_op(opts)
            opts = o
        opts = self._opts_hook(opts)
        return self._run(lambda pg: pg.allreduce_coalesced(tensors, opts), opts)

    def alltoall_base(self, output_buffer, input_buffer, output_split_sizes, input_split_sizes, opts=None) -> Work:
        opts = self._opts_hook(opts or AllToAllOptions())
        return self._run(
            lambda pg: pg.alltoall_base(output_buffer, input_buffer, output_split_sizes, input_split_sizes, opts), opts
        )

    def barrier(self, opts=None) -> Work:
        opts = self._opts_hook(opts or BarrierOptions())
        return self._run(lambda pg: pg.barrier(opts), opts)

    def broadcast(self, tensor_list, opts=None) -> Work:
        opts = self._opts_hook(opts or BroadcastOptions())
        return self._run(lambda pg: pg.broadcast(tensor_list, opts), opts)

    def recv(self, tensors, src_rank, tag) -> Work:
        return self._run(lambda pg: pg.recv(tensors, src_rank, tag))

    def reduce_scatter(self, output_tensors, input_tensors, opts=None) -> Work:
        opts = self._opts_hook(opts or ReduceScatterOptions())
        return self._run(lambda pg: pg.reduce_scatter(output_tensors, input_tensors, opts), opts)

    def reduce_scatter_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        opts = self._opts_hook(opts or ReduceScatterOptions())
        return self._run(lambda pg: pg.reduce_scatter_tensor_coalesced(output_tensors, input_tensors, opts), opts)

    def send(self, tensors, dst_rank, tag) -> Work:
        return self._run(lambda pg: pg.send(tensors, dst_rank, tag))

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(pg={self._pg})"


class ProcessGroupGloo(ProcessGroupWrapper):
    """Gloo back-end (CPU tensors, and CUDA tensors staged through the host)."""

    def _create_pg(self, store: Store, rank: int, world_size: int) -> BaseProcessGroup:
        pg = BaseProcessGroup(store, rank, world_size)
        pg._set_default_backend(BaseProcessGroup.BackendType.GLOO)
        backend = BaseProcessGroupGloo(store, rank, world_size, self._timeout)
        backend._set_sequence_number_for_group()
        pg._register_backend(torch.device("cpu"), BaseProcessGroup.BackendType.GLOO, backend)
        if torch.cuda.is_available():
            pg._register_backend(torch.device("cuda"), BaseProcessGroup.BackendType.GLOO, backend)
        return pg

    def getBackendName(self) -> str:
        return "torchft-b200-gloo"

    def reduce_scatter(self, output_tensors, input_tensors, opts=None) -> Work:
        raise RuntimeError("ProcessGroupGloo does not support reduce_scatter.")

    def reduce_scatter_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        raise RuntimeError("ProcessGroupGloo does not support reduce_scatter_tensor_coalesced.")


class _StreamTimedWork(Work):
    """``Work`` of an accelerator collective: waiting arms both a host timeout around the
    call and a stream timeout behind it, each of which aborts the communicator."""

    def __init__(self, pg: "ProcessGroupNCCL", work: Work, timeout: timedelta) -> None:
        super().__init__()
        self._pg, self._work, self._timeout = pg, work, timeout

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        t = timeout or self._timeout
        with self._pg._run_context():
            with context_timeout(self._pg._timeout_abort, t):
                ok = self._work.wait()
            # the wait above only orders the stream; watch the stream itself too
            stream_timeout(self._pg._timeout_abort, t)
        return ok

    def get_future(self) -> Future:
        return self._work.get_future()

    def is_completed(self) -> bool:
        return self._work.is_completed()

    def synchronize(self) -> None:
        self.wait()

    def block_current_stream(self, timeout: Optional[timedelta] = None) -> None:
        self.wait(timeout)


class ProcessGroupNCCL(ProcessGroupWrapper):
    """NCCL back-end made safe for membership changes.

    The communicator is created non-blocking so that initialisation and collectives can be
    abandoned; every issue and wait runs under a host timeout, every wait additionally arms
    a stream timeout; both call :meth:`abort` (``ncclCommAbort``), which first latches
    ``errored()`` so the manager discards the step.  Needs NCCL >= 2.25 for a safe abort.
    Behaviour of torchft/process_group.py:738-846.
    """

    def __init__(self, timeout: timedelta = timedelta(seconds=60.0)) -> None:
        super().__init__(timeout)
        self._use_abort: bool = torch.cuda.is_available() and torch.cuda.nccl.version() >= (2, 25)
        self._errored: Optional[Exception] = None
        nb = "TORCH_NCCL_NONBLOCKING_TIMEOUT"
        if nb not in os.environ:
            os.environ[nb] = str(timeout.total_seconds())

    def _opts_hook(self, opts):
        if not self._use_abort:
            return opts
        # the per-op c10d timeout would fight with the abort-based timeouts: clear it
        if hasattr(opts, "timeout"):
            try:
                opts.timeout = timedelta(milliseconds=-1)
            except Exception:
                pass
        return opts

    def _wrap_work(self, work: Work, opts: object) -> Work:
        if not self._use_abort:
            return work
        return _StreamTimedWork(self, work, self._timeout)

    @contextmanager
    def _run_context(self) -> Generator[None, None, None]:
        yield

    def _create_pg(self, store: Store, rank: int, world_size: int) -> BaseProcessGroup:
        assert BaseProcessGroupNCCL is not None, "this torch build has no NCCL"
        self._errored = None
        pg = BaseProcessGroup(store, rank, world_size)
        pg._set_default_backend(BaseProcessGroup.BackendType.NCCL)
        opts = BaseProcessGroupNCCL.Options()
        opts.config.blocking = False
        opts.global_ranks_in_group = list(range(world_size))
        opts._timeout = self._timeout
        backend = BaseProcessGroupNCCL(store, rank, world_size, opts)
        backend._set_sequence_number_for_group()
        backend.eager_connect_single_device(torch.device("cuda", torch.cuda.current_device()))
        pg._register_backend(torch.device("cuda"), BaseProcessGroup.BackendType.NCCL, backend)
        return pg

    def abort(self, errored: bool = True) -> None:
        # latch first: a collective unblocked by the abort must be seen as failed
        if errored:
            self._errored = RuntimeError("aborted")
            if os.environ.get(TORCHFT_TRIGGER_FR_ON_ABORT, "0").lower() in ("1", "true"):
                trigger_nccl_fr_trace_through_pipe(dist.get_rank() if dist.is_initialized() else (self._rank or 0))
        super().abort(errored)

    def errored(self) -> Optional[Exception]:
        pg = self._pg
        if pg is not None and torch.cuda.is_available():
            # surface asynchronous NCCL failures before the answer is trusted
            try:
                torch.cuda.current_stream().synchronize()
            except Exception as e:  # pragma: no cover
                self._errored = e
        return self._errored

    def getBackendName(self) -> str:
        return "torchft-b200-nccl"


class ProcessGroupDummy(ProcessGroup):
    """World of one: every collective completes at once, copying inputs to outputs.
    Soaks up DDP's construction-time broadcasts and is handy in unit tests."""

    def __init__(self, rank: int = 0, world: int = 1) -> None:
        super().__init__(rank, world)
        assert rank == 0 and world == 1
        self._rank, self._world = rank, world
        self.wait_count = 0
        self.get_future_count = 0
        self._work: List[Work] = []
        self.configure_count = 0

    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int) -> None:
        self.configure_count += 1

    def _done(self, result: object) -> Work:
        w = _DummyWork(result)
        self._work.append(w)
        return w

    def allgather(self, output_tensors, input_tensor, opts=None) -> Work:
        for o, i in zip(output_tensors[0], input_tensor):
            o.copy_(i)
        return self._done(output_tensors)

    def allgather_into_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        for o, i in zip(output_tensors, input_tensors):
            o.copy_(i)
        return self._done(output_tensors)

    def allreduce(self, tensors, opts=None) -> Work:
        return self._done(tensors)

    def allreduce_coalesced(self, tensors, opts=None) -> Work:
        return self._done(tensors)

    def alltoall_base(self, output_buffer, input_buffer, output_split_sizes, input_split_sizes, opts=None) -> Work:
        output_buffer.copy_(input_buffer)
        return self._done([output_buffer])

    def barrier(self, opts=None) -> Work:
        return self._done(None)

    def broadcast(self, tensor_list, opts=None) -> Work:
        return self._done(tensor_list)

    def recv(self, tensors, src_rank, tag) -> Work:
        return self._done(tensors)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None) -> Work:
        for o, i in zip(output_tensors, input_tensors[0]):
            o.copy_(i)
        return self._done(output_tensors)

    def reduce_scatter_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        for o, i in zip(output_tensors, input_tensors):
            o.copy_(i)
        return self._done(output_tensors)

    def send(self, tensors, dst_rank, tag) -> Work:
        return self._done(tensors)

    def size(self) -> int:
        return self._world

    def getBackendName(self) -> str:
        return "torchft-b200-dummy"


class _ErrorSwallowingWork(Work):
    def __init__(self, pg: "ErrorSwallowingProcessGroupWrapper", work: Work, default_result: object) -> None:
        super().__init__()
        self._pg, self._work, self._default = pg, work, default_result

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        try:
            self._work.wait()
        except Exception as e:
            self._pg.report_error(e)
        return True

    def get_future(self) -> Future:
        fut = self._work.get_future()

        def swallow(f: Future) -> object:
            try:
                return f.value()
            except Exception as e:
                self._pg.report_error(e)
                return self._default

        return fut.then(swallow)


class ErrorSwallowingProcessGroupWrapper(ProcessGroupWrapper):
    """Turns allreduce failures into a latched error: once one happened every further
    allreduce is a no-op until the next ``configure``."""

    def __init__(self, pg: ProcessGroup) -> None:
        super().__init__(pg=pg)
        self._error: Optional[Exception] = None

    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int, quorum_id=None) -> None:
        self._error = None
        super().configure(store_addr, replica_id, rank, world_size)

    def report_error(self, e: Exception) -> None:
        self._error = e

    def error(self) -> Optional[Exception]:
        return self._error

    def allreduce(self, tensors, opts=None) -> Work:
        if self._error is not None:
            return _DummyWork(tensors)
        try:
            return _ErrorSwallowingWork(self, super().allreduce(tensors, opts), tensors)
        except Exception as e:
            self.report_error(e)
            return _DummyWork(tensors)


class FakeProcessGroupWrapper(ProcessGroupWrapper):
    """Fault injection: ``report_future_error(e)`` makes the next allreduce's future fail,
    ``report_error(e)`` makes ``errored()`` return ``e`` until the next configure."""

    def __init__(self, pg: ProcessGroup) -> None:
        super().__init__(pg=pg)
        self._future_error: Optional[Exception] = None
        self._latched: Optional[Exception] = None

    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int, quorum_id=None) -> None:
        self._future_error = None
        self._latched = None
        super().configure(store_addr, replica_id, rank, world_size)

    def report_future_error(self, e: Exception) -> None:
        self._future_error = e

    def report_error(self, e: Exception) -> None:
        self._latched = e

    def errored(self) -> Optional[Exception]:
        if self._latched is not None:
            return self._latched
        pg = self._pg
        return pg.errored() if isinstance(pg, ProcessGroup) else None

    def allreduce(self, tensors, opts=None) -> Work:
        work = super().allreduce(tensors, opts)
        if self._future_error is None:
            return work
        err, self._future_error = self._future_error, None
        fut = work.get_future()

        def fail(f: Future) -> object:
            raise err

        failed = fut.then(fail)

        class _FailedWork(Work):
            def wait(self_inner, timeout=None) -> bool:
                failed.wait()
                return True

            def get_future(self_inner) -> Future:
                return failed

        return _FailedWork()


class ManagedProcessGroup(ProcessGroupWrapper):
    """Process-group facade over a ``Manager``: ``allreduce`` is the manager's
    fault-tolerant allreduce and ``size()`` the current number of participants.  This is
    what the replicate dimension of an HSDP device mesh is made of."""

    def __init__(self, manager: "Manager") -> None:
        super().__init__(pg=manager._pg)
        self._manager = manager

    def allreduce(self, tensors, opts=None) -> Work:
        assert len(tensors) == 1, "ManagedProcessGroup reduces one tensor per call"
        op = _reduce_op(opts)
        if op == ReduceOp.SUM:
            return self._manager.allreduce(tensors[0], reduce_op=ReduceOp.SUM)
        if op == ReduceOp.AVG:
            return self._manager.allreduce(tensors[0], reduce_op=ReduceOp.AVG)
        raise AssertionError(f"ManagedProcessGroup supports SUM and AVG, got {op}")

    def size(self) -> int:
        return self._manager.num_participants()

    def getBackendName(self) -> str:
        return self._manager._pg.getBackendName()


from .process_group_baby import (  # noqa: E402,F401
    ProcessGroupBaby,
    ProcessGroupBabyGloo,
    ProcessGroupBabyNCCL,
)
