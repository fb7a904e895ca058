"""Subprocess-isolated process groups.

The real communicator lives in a spawned child process; the parent only holds pipes.
When a collective wedges (a peer died inside NCCL, a socket never answers) the parent
kills the child and spawns a fresh one on the next ``configure`` -- no library state of
the hung communicator survives in the training process.  The price is a second CUDA
context per rank (about 1 GB) and host-synchronous completion.

Protocol (parent -> child on the request pipe, one reply per request; completions arrive
asynchronously on the future pipe):
    ("op", op_id, method, tensors..., options-as-dict)  -> ("ok", op_id) | exception
    ("num_active_work",)                                -> int
    child -> parent future pipe: (op_id, None | exception)
CPU tensors cross as shared memory, CUDA tensors as CUDA IPC handles (both through
``torch.multiprocessing``'s pickler), so the child works on the parent's memory.
Role of torchft/process_group.py:1358-2023.
"""

from __future__ import annotations

import logging
import threading
from datetime import timedelta
from typing import Dict, List, Optional, Tuple

import torch
import torch.multiprocessing as mp
from torch.distributed import ProcessGroup as BaseProcessGroup
from torch.distributed import ProcessGroupGloo as BaseProcessGroupGloo
from torch.distributed import Store
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

from ._pg_base import ProcessGroup, create_store_client
from .multiprocessing import _MonitoredPipe

logger = logging.getLogger(__name__)

_OPTS = {
    "AllreduceOptions": (AllreduceOptions, ("reduceOp",)),
    "AllreduceCoalescedOptions": (AllreduceCoalescedOptions, ("reduceOp",)),
    "AllgatherOptions": (AllgatherOptions, ()),
    "AllToAllOptions": (AllToAllOptions, ()),
    "BarrierOptions": (BarrierOptions, ()),
    "BroadcastOptions": (BroadcastOptions, ("rootRank", "rootTensor")),
    "ReduceScatterOptions": (ReduceScatterOptions, ("reduceOp",)),
}


def _op_name(op) -> str:
    for name in ("SUM", "AVG", "PRODUCT", "MIN", "MAX", "BAND", "BOR", "BXOR"):
        if op == getattr(ReduceOp, name):
            return name
    raise ValueError(f"unsupported reduce op {op}")


def _pack_opts(opts) -> Optional[Tuple[str, Dict[str, object]]]:
    """c10d option objects do not pickle: ship the class name and the fields that matter."""
    if opts is None:
        return None
    if isinstance(opts, (ReduceOp, ReduceOp.RedOpType)):
        return ("AllreduceOptions", {"reduceOp": _op_name(opts)})
    name = type(opts).__name__
    _, fields = _OPTS[name]
    out: Dict[str, object] = {}
    for f in fields:
        v = getattr(opts, f)
        out[f] = _op_name(v) if f == "reduceOp" else v
    return (name, out)


def _unpack_opts(packed):
    if packed is None:
        return None
    name, fields = packed
    cls, _ = _OPTS[name]
    o = cls()
    for k, v in fields.items():
        setattr(o, k, getattr(ReduceOp, v) if k == "reduceOp" else v)
    return o


class _BabyWork(Work):
    def __init__(self, pg: "ProcessGroupBaby", op_id: int, result: object) -> None:
        super().__init__()
        self._pg, self._op_id, self._result = pg, op_id, result
        self._done = threading.Event()
        self._exc: Optional[Exception] = None
        self._fut: Future = Future()

    def _complete(self, exc: Optional[Exception]) -> None:
        self._exc = exc
        if exc is None:
            self._fut.set_result(self._result)
        else:
            self._fut.set_exception(exc)
        self._done.set()

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        t = (timeout or self._pg._timeout).total_seconds()
        if not self._done.wait(t):
            raise TimeoutError(f"collective {self._op_id} did not complete within {t} s")
        if self._exc is not None:
            raise self._exc
        return True

    def get_future(self) -> Future:
        return self._fut

    def is_completed(self) -> bool:
        return self._done.is_set()

    def synchronize(self) -> None:
        self.wait()

    def block_current_stream(self, timeout: Optional[timedelta] = None) -> None:
        self.wait(timeout)


def _worker(cls, store_addr: str, rank: int, world_size: int, req, fut, timeout: timedelta, device: Optional[int]) -> None:
    """Child process main loop."""
    import queue as _queue

    try:
        if device is not None and torch.cuda.is_available():
            torch.cuda.set_device(device)
        store = create_store_client(store_addr, timeout)
        pg = cls._create_pg(store, rank, world_size, timeout)
        req.send("ready")
    except Exception as e:  # report and die; the parent raises from configure()
        req.send(e)
        return

    pending: "_queue.Queue[Optional[Tuple[int, Work, bool]]]" = _queue.Queue()
    active = {"n": 0}
    lock = threading.Lock()

    def completer() -> None:
        while True:
            item = pending.get()
            if item is None:
                return
            op_id, work, on_cuda = item
            err: Optional[Exception] = None
            try:
                work.wait()
                if on_cuda:
                    torch.cuda.current_stream().synchronize()
            except Exception as e:
                err = e
            with lock:
                active["n"] -= 1
            try:
                fut.send((op_id, err))
            except Exception:
                return

    threading.Thread(target=completer, daemon=True).start()
    try:
        while True:
            cmd = req.recv()
            kind = cmd[0]
            if kind == "op":
                _, op_id, method, args, packed = cmd
                try:
                    opts = _unpack_opts(packed)
                    call_args = list(args) + ([opts] if opts is not None else [])
                    work = getattr(pg, method)(*call_args)
                    on_cuda = any(
                        isinstance(t, torch.Tensor) and t.is_cuda
                        for a in args
                        for t in (a if isinstance(a, (list, tuple)) else [a])
                        for t in (t if isinstance(t, (list, tuple)) else [t])
                    )
                    with lock:
                        active["n"] += 1
                    pending.put((op_id, work, on_cuda))
                    req.send(("ok", op_id))
                except Exception as e:
                    req.send(e)
            elif kind == "num_active_work":
                with lock:
                    req.send(active["n"])
            elif kind == "stop":
                break
    except (EOFError, OSError):  # the parent closed the pipe (or "killed" a thread-backed worker)
        pass
    finally:
        pending.put(None)


class ProcessGroupBaby(ProcessGroup):
    """Base of the subprocess-backed groups; subclasses provide ``_create_pg``."""

    def __init__(self, timeout: timedelta = timedelta(seconds=60.0)) -> None:
        super().__init__(0, 1)
        self._timeout = timeout
        self._world_size = -1
        self._rank = -1
        self._proc: Optional[mp.Process] = None
        self._req: Optional[_MonitoredPipe] = None
        self._fut: Optional[_MonitoredPipe] = None
        self._fut_thread: Optional[threading.Thread] = None
        self._works: Dict[int, _BabyWork] = {}
        self._lock = threading.Lock()
        self._next_op = 0
        self._errored: Optional[Exception] = None

    @classmethod
    def _create_pg(cls, store: Store, rank: int, world_size: int, timeout: timedelta) -> BaseProcessGroup:
        raise NotImplementedError

    @staticmethod
    def _mp_context():
        """The context that provides ``Process`` and ``Pipe``.  Tests may replace it by
        ``multiprocessing_dummy_context.DummyContext`` to run the worker on a thread."""
        return mp.get_context("spawn")

    # ---- lifecycle ------------------------------------------------------------------------
    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int) -> None:
        self.shutdown()
        self._errored = None
        self._rank, self._world_size = rank, world_size
        ctx = self._mp_context()
        req_parent, req_child = ctx.Pipe()
        fut_parent, fut_child = ctx.Pipe()
        device = torch.cuda.current_device() if torch.cuda.is_available() else None
        self._proc = ctx.Process(
            target=_worker,
            args=(type(self), store_addr, rank, world_size, req_child, fut_child, self._timeout, device),
            daemon=True,
        )
        self._proc.start()
        req_child.close()
        fut_child.close()
        self._req, self._fut = _MonitoredPipe(req_parent), _MonitoredPipe(fut_parent)
        ready = self._req.recv(self._timeout)  # raises what the child raised
        assert ready == "ready", ready
        self._fut_thread = threading.Thread(target=self._pump, args=(self._fut,), daemon=True)
        self._fut_thread.start()

    def _pump(self, pipe: _MonitoredPipe) -> None:
        while True:
            try:
                op_id, err = pipe.recv(timedelta(seconds=1))
            except TimeoutError:
                if pipe.closed():
                    break
                continue
            except (EOFError, OSError, TypeError, ValueError):
                break
            with self._lock:
                w = self._works.pop(op_id, None)
            if w is not None:
                w._complete(err)
        # child is gone: fail whatever is still outstanding
        with self._lock:
            works, self._works = list(self._works.values()), {}
        for w in works:
            w._complete(RuntimeError("process group worker exited"))

    def shutdown(self) -> None:
        proc, req, fut = self._proc, self._req, self._fut
        self._proc = self._req = self._fut = None
        if req is not None:
            try:
                req.send(("stop",))
            except Exception:
                pass
            req.close()
        if proc is not None:
            proc.kill()
            proc.join(timeout=10)
        if fut is not None:
            fut.close()
        t = self._fut_thread
        self._fut_thread = None
        if t is not None and t is not threading.current_thread():
            t.join(timeout=5)

    def abort(self) -> None:
        self._errored = RuntimeError("aborted")
        self.shutdown()

    def errored(self) -> Optional[Exception]:
        return self._errored

    def set_timeout(self, timeout: timedelta) -> None:
        self._timeout = timeout

    def size(self) -> int:
        return self._world_size

    def num_active_work(self) -> int:
        assert self._req is not None
        self._req.send(("num_active_work",))
        return int(self._req.recv(self._timeout))  # type: ignore[arg-type]

    # ---- op plumbing ------------------------------------------------------------------------
    def _run(self, method: str, args: tuple, opts, result: object) -> Work:
        req = self._req
        if req is None:
            raise RuntimeError("process group not configured (or aborted)")
        with self._lock:
            op_id = self._next_op
            self._next_op += 1
            work = _BabyWork(self, op_id, result)
            self._works[op_id] = work
        try:
            req.send(("op", op_id, method, args, _pack_opts(opts)))
            reply = req.recv(self._timeout)
            assert reply == ("ok", op_id), reply
        except Exception as e:
            with self._lock:
                self._works.pop(op_id, None)
            self._errored = e if isinstance(e, Exception) else RuntimeError(str(e))
            raise
        return work

    def allreduce(self, tensors: List[torch.Tensor], opts=None) -> Work:
        if not isinstance(opts, AllreduceOptions):
            o = AllreduceOptions()
            if opts is not None:
                o.reduceOp = opts
            opts = o
        return self._run("allreduce", (tensors,), opts, tensors)

    def allreduce_coalesced(self, tensors, opts=None) -> Work:
        return self._run("allreduce_coalesced", (tensors,), opts or AllreduceCoalescedOptions(), tensors)

    def allgather(self, output_tensors, input_tensor, opts=None) -> Work:
        return self._run("allgather", (output_tensors, input_tensor), opts or AllgatherOptions(), output_tensors)

    def allgather_into_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        return self._run("allgather_into_tensor_coalesced", (output_tensors, input_tensors), opts or AllgatherOptions(),
                         output_tensors)

    def alltoall_base(self, output_buffer, input_buffer, output_split_sizes, input_split_sizes, opts=None) -> Work:
        return self._run("alltoall_base", (output_buffer, input_buffer, output_split_sizes, input_split_sizes),
                         opts or AllToAllOptions(), [output_buffer])

    def barrier(self, opts=None) -> Work:
        return self._run("barrier", (), opts or BarrierOptions(), None)

    def broadcast(self, tensor_list, opts=None) -> Work:
        return self._run("broadcast", (tensor_list,), opts or BroadcastOptions(), tensor_list)

    def recv(self, tensors, src_rank: int, tag: int) -> Work:
        return self._run("recv", (tensors, src_rank, tag), None, tensors)

    def send(self, tensors, dst_rank: int, tag: int) -> Work:
        return self._run("send", (tensors, dst_rank, tag), None, tensors)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None) -> Work:
        return self._run("reduce_scatter", (output_tensors, input_tensors), opts or ReduceScatterOptions(), output_tensors)

    def reduce_scatter_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        return self._run("reduce_scatter_tensor_coalesced", (output_tensors, input_tensors),
                         opts or ReduceScatterOptions(), output_tensors)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(rank={self._rank}, world={self._world_size})"

    def __del__(self) -> None:
        try:
            self.shutdown()
        except Exception:
            pass


class ProcessGroupBabyGloo(ProcessGroupBaby):
    """Gloo in a subprocess (CPU tensors through shared memory)."""

    @classmethod
    def _create_pg(cls, store: Store, rank: int, world_size: int, timeout: timedelta) -> BaseProcessGroup:
        pg = BaseProcessGroup(store, rank, world_size)
        pg._set_default_backend(BaseProcessGroup.BackendType.GLOO)
        backend = BaseProcessGroupGloo(store, rank, world_size, timeout)
        backend._set_sequence_number_for_group()
        pg._register_backend(torch.device("cpu"), BaseProcessGroup.BackendType.GLOO, backend)
        return pg

    def getBackendName(self) -> str:
        return "torchft-b200-baby-gloo"

    def reduce_scatter(self, output_tensors, input_tensors, opts=None) -> Work:
        raise RuntimeError("ProcessGroupBabyGloo does not support reduce_scatter.")

    def reduce_scatter_tensor_coalesced(self, output_tensors, input_tensors, opts=None) -> Work:
        raise RuntimeError("ProcessGroupBabyGloo does not support reduce_scatter_tensor_coalesced.")


class ProcessGroupBabyNCCL(ProcessGroupBaby):
    """NCCL in a subprocess: a hung communicator is disposed of by killing the child.
    Costs an extra CUDA context (~1 GB) per rank; tensors cross as CUDA IPC handles."""

    @classmethod
    def _create_pg(cls, store: Store, rank: int, world_size: int, timeout: timedelta) -> BaseProcessGroup:
        from torch.distributed import ProcessGroupNCCL as BaseProcessGroupNCCL

        pg = BaseProcessGroup(store, rank, world_size)
        pg._set_default_backend(BaseProcessGroup.BackendType.NCCL)
        opts = BaseProcessGroupNCCL.Options()
        opts._timeout = timeout
        backend = BaseProcessGroupNCCL(store, rank, world_size, opts)
        backend._set_sequence_number_for_group()
        pg._register_backend(torch.device("cuda"), BaseProcessGroup.BackendType.NCCL, backend)
        return pg

    def getBackendName(self) -> str:
        return "torchft-b200-baby-nccl"
