"""NVLink peer-memory communication: symmetric arenas, kernel collectives, and the two
things built on them -- :class:`PeerShardComm` (FSDP traffic inside a replica group) and
:class:`ProcessGroupB200` (the reconfigurable replica-dimension group).

Every rank owns an *arena* of device memory that its peers map through CUDA IPC.  Arenas
are carved up identically on all ranks, so "the same buffer on rank p" is simply
``peer_base[p] + offset``.  Collectives are single kernels (see ``csrc/team/team.cu``)
that read and write peers' arenas directly; they poll an abort word, carry an
epoch-stamped token and give up after a deadline, reporting through a status word
instead of hanging.  Reconfiguring a team (new quorum) is: bump the epoch, clear local
flags, close old mappings, exchange handles through the store, map -- milliseconds, no
communicator bootstrap.
"""

from __future__ import annotations

import ctypes
import logging
import os
import threading
from datetime import timedelta
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch.distributed import Store
from torch.distributed.distributed_c10d import ReduceOp, Work
from torch.futures import Future

from .._pg_base import ProcessGroup, _reduce_op, create_store_client
from ..ops import _native as N
from .shard_comm import ShardComm

logger = logging.getLogger(__name__)

MAX_RANKS = 8
_DT = {torch.bfloat16: 0, torch.float32: 1}
# CTAs per peer-memory collective (0 = sized from the message, up to 128).  Collectives that
# overlap with compute can be given fewer so that they leave SMs to the GEMMs.
DEFAULT_CTAS = int(os.environ.get("FTB200_COMM_CTAS", "0"))


class _TeamDesc(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
        ("token", ctypes.c_ulonglong),
        ("timeout_ns", ctypes.c_ulonglong),
        ("flags", ctypes.c_void_p * MAX_RANKS),
        ("local_sync", ctypes.c_void_p),
        ("abort_word", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
    ]


class _RawMemory:
    """Exposes a raw device pointer to ``torch.as_tensor`` (zero-copy)."""

    def __init__(self, ptr: int, nbytes: int, owner: object) -> None:
        self._owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class _FdServer:
    """Hands one file descriptor to whoever connects to an abstract Unix-domain socket (SCM_RIGHTS): how a rank's
    arena descriptor reaches its peers in other processes of the same host."""

    def __init__(self, fd: int) -> None:
        import socket

        self._fd = fd
        self._sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.address = f"\0ftb200-arena-{os.getpid()}-{id(self):x}"
        self._sock.bind(self.address)
        self._sock.listen(64)
        self._stop = False
        self._thread = threading.Thread(target=self._serve, name="ftb200-arena-fd", daemon=True)
        self._thread.start()

    def _serve(self) -> None:
        import socket

        while not self._stop:
            try:
                conn, _ = self._sock.accept()
            except OSError:
                return
            try:
                socket.send_fds(conn, [b"fd"], [self._fd])
            except OSError:
                pass
            finally:
                conn.close()

    @staticmethod
    def fetch(address: str, timeout_s: float) -> int:
        import socket

        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
            c.settimeout(timeout_s)
            c.connect(address)
            _, fds, _, _ = socket.recv_fds(c, 16, 1)
        if not fds:
            raise TeamError(f"no descriptor received from {address!r}")
        return fds[0]

    def close(self) -> None:
        self._stop = True
        try:
            self._sock.close()
        except OSError:
            pass


class Arena:
    """One exported slab of device memory with a bump allocator (256-byte granules).

    By default the slab is a ``cuMemCreate`` allocation shared with the peers as a POSIX file descriptor
    (``kind == "vmm"``): a peer that has imported it holds a reference of its own, so its mapping stays valid by
    the documented semantics of the driver even after the exporting process is gone.  ``FTB200_ARENA=ipc`` (or a
    driver without these entry points) selects a ``cudaMalloc`` slab shared through a legacy CUDA IPC handle."""

    def __init__(self, nbytes: int, device: torch.device) -> None:
        self.device = device
        self.nbytes = int(nbytes)
        self.kind = "ipc"
        self._fd_server: Optional[_FdServer] = None
        p = ctypes.c_void_p()
        with torch.cuda.device(device):
            if os.environ.get("FTB200_ARENA", "vmm") != "ipc":
                fd, padded = ctypes.c_int(-1), ctypes.c_ulonglong(0)
                rc = N.lib().ftb200_vmm_alloc(ctypes.byref(p), ctypes.c_ulonglong(self.nbytes), ctypes.byref(fd),
                                              ctypes.byref(padded))
                if rc == 0:
                    self.kind, self.mapped_bytes = "vmm", int(padded.value)
                    self._fd_server = _FdServer(int(fd.value))
                else:
                    logger.warning("VMM arena unavailable (code %d): falling back to a legacy CUDA IPC arena", rc)
            if self.kind == "ipc":
                N.check(N.lib().ftb200_arena_alloc(ctypes.byref(p), ctypes.c_ulonglong(self.nbytes)), "arena_alloc", 0)
            self.base = int(p.value)
            self.bytes_view = torch.as_tensor(_RawMemory(self.base, self.nbytes, self), device=device)
        self._off = 0
        self._lock = threading.Lock()

    def alloc(self, nbytes: int) -> int:
        with self._lock:
            off = self._off
            self._off = (off + nbytes + 255) // 256 * 256
            if self._off > self.nbytes:
                raise MemoryError(f"arena of {self.nbytes} bytes exhausted (asked for {nbytes} at {off})")
            return off

    def tensor(self, off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nb = numel * torch.empty((), dtype=dtype).element_size()
        return self.bytes_view[off : off + nb].view(dtype)

    def export_handle(self) -> bytes:
        """What a peer needs to map this arena: for a VMM arena the address of the descriptor server and the
        mapped size, for a legacy arena the 64-byte CUDA IPC handle."""
        if self.kind == "vmm":
            assert self._fd_server is not None
            return b"vmm:" + f"{self.mapped_bytes}:".encode() + self._fd_server.address.encode()
        buf = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            N.check(N.lib().ftb200_ipc_export(ctypes.c_void_p(self.base), buf), "ipc_export", 0)
        return b"ipc:" + bytes(buf)

    @staticmethod
    def import_handle(handle: bytes, timeout_s: float = 30.0) -> tuple:
        """Maps a peer's arena for the current device; returns ``(base address, kind)``."""
        ptr = ctypes.c_void_p()
        if handle.startswith(b"vmm:"):
            size, _, address = handle[4:].partition(b":")
            fd = _FdServer.fetch(address.decode(), timeout_s)
            try:
                N.check(N.lib().ftb200_vmm_import(ctypes.c_int(fd), ctypes.c_ulonglong(int(size)), ctypes.byref(ptr)),
                        "vmm_import", 0)
            finally:
                os.close(fd)
            return int(ptr.value), "vmm"
        raw = handle[4:] if handle.startswith(b"ipc:") else handle
        N.check(N.lib().ftb200_ipc_import((ctypes.c_ubyte * 64).from_buffer_copy(raw), ctypes.byref(ptr)), "ipc_import", 0)
        return int(ptr.value), "ipc"

    @staticmethod
    def release_import(base: int, kind: str) -> None:
        if kind == "vmm":
            N.lib().ftb200_vmm_free(ctypes.c_void_p(base))
        else:
            N.lib().ftb200_ipc_close(ctypes.c_void_p(base))

    def contains(self, t: torch.Tensor) -> Optional[int]:
        """Offset of ``t`` inside the arena, or None."""
        p = t.data_ptr()
        if self.base <= p and p + t.numel() * t.element_size() <= self.base + self.nbytes:
            return p - self.base
        return None


class TeamError(RuntimeError):
    """A peer-memory collective ended with a status other than OK (timeout, abort, epoch mismatch) or the team could
    not be set up."""


class SymmetricTeam:
    """A set of ranks with mutually mapped arenas plus the flag/abort/status plumbing."""

    def __init__(self, device: torch.device, arena_bytes: int, timeout: timedelta = timedelta(seconds=30)) -> None:
        self.device = torch.device(device)
        self.lib = N.lib()
        self.lib.ftb200_team_flag_bytes.restype = ctypes.c_int
        self.timeout = timeout
        self.arena = Arena(arena_bytes, self.device)
        self._flag_off = self.arena.alloc(int(self.lib.ftb200_team_flag_bytes()))
        self._sync = torch.zeros(8, dtype=torch.int64, device=self.device)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        hp, dp = ctypes.POINTER(ctypes.c_int)(), ctypes.c_void_p()
        with torch.cuda.device(self.device):
            N.check(self.lib.ftb200_abort_word_create(ctypes.byref(hp), ctypes.byref(dp)), "abort_word_create", 0)
        self._abort_host, self._abort_dev = hp, int(dp.value)
        self.rank, self.world = 0, 1
        self.epoch = 0
        self._seq = 0
        self.peer_base: List[int] = [self.arena.base]
        self._imported: List[tuple] = []
        self._lock = threading.Lock()

    # ---- membership -----------------------------------------------------------------------
    def connect(self, store: Store, rank: int, world: int, epoch: int) -> None:
        """(Re)build the peer mappings for a new membership.  ``store`` must be a fresh
        prefix shared by exactly these ranks."""
        if world > MAX_RANKS:
            raise ValueError(f"team supports at most {MAX_RANKS} ranks")
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            self._close_peers()
            self.rank, self.world, self.epoch, self._seq = rank, world, int(epoch) & 0xFFFFFFFF, 0
            self._abort_host[0] = 0
            self._status.zero_()
            self._sync.zero_()
            self.arena.bytes_view[self._flag_off : self._flag_off + int(self.lib.ftb200_team_flag_bytes())].zero_()
            torch.cuda.synchronize(self.device)
            store.set(f"arena/{rank}", self.arena.export_handle())
            bases: List[int] = []
            for p in range(world):
                if p == rank:
                    bases.append(self.arena.base)
                    continue
                handle = store.get(f"arena/{p}")
                base, kind = Arena.import_handle(bytes(handle), self.timeout.total_seconds())
                self._imported.append((base, kind))
                bases.append(base)
            self.peer_base = bases
            # nobody may signal into flags that a slower peer has not cleared yet
            store.set(f"mapped/{rank}", b"1")
            for p in range(world):
                store.get(f"mapped/{p}")

    def _close_peers(self) -> None:
        for base, kind in self._imported:
            Arena.release_import(base, kind)
        self._imported = []
        self.peer_base = [self.arena.base]

    def close(self) -> None:
        with torch.cuda.device(self.device):
            self._close_peers()

    # ---- failure plumbing -------------------------------------------------------------------
    def abort(self) -> None:
        """Make every in-flight and future kernel of this team return (a plain memory write)."""
        self._abort_host[0] = 1

    def status(self) -> int:
        """Synchronising read of the status word (0 ok, 1 timeout, 2 aborted, 3 epoch)."""
        return int(self._status.item())

    def check(self) -> None:
        code = self.status()
        if code:
            raise TeamError(f"peer-memory collective failed: {N.STATUS.get(code, code)}")

    # ---- kernels ------------------------------------------------------------------------------
    def _desc(self) -> _TeamDesc:
        with self._lock:
            self._seq += 1
            seq = self._seq
        d = _TeamDesc()
        d.rank, d.world = self.rank, self.world
        d.token = (self.epoch << 32) | (seq & 0xFFFFFFFF)
        d.timeout_ns = int(self.timeout.total_seconds() * 1e9)
        for p in range(MAX_RANKS):
            d.flags[p] = (self.peer_base[p] + self._flag_off) if p < self.world else None
        d.local_sync = self._sync.data_ptr()
        d.abort_word = self._abort_dev
        d.status = self._status.data_ptr()
        return d

    def _desc_nocount(self) -> _TeamDesc:
        """Descriptor for a point-to-point kernel: those count per pair of ranks, so the team's
        collective sequence number (which every rank must advance identically) stays untouched."""
        with self._lock:
            self._seq -= 1
        return self._desc()

    def _peer_ptrs(self, off: int) -> ctypes.Array:
        arr = (ctypes.c_void_p * MAX_RANKS)()
        for p in range(self.world):
            arr[p] = self.peer_base[p] + off
        return arr

    def allreduce_(self, off: int, numel: int, dtype: torch.dtype, scale: float = 1.0,
                   user_in: Optional[torch.Tensor] = None, user_out: Optional[torch.Tensor] = None,
                   zero_contribution: bool = False, ctas: int = 0) -> None:
        """In-place allreduce of the symmetric buffer at ``off`` (``numel`` must be a
        multiple of ``world * 16 bytes``); optionally staged from/to user tensors."""
        d = self._desc()
        N.check(
            self.lib.ftb200_team_allreduce(ctypes.byref(d), self._peer_ptrs(off), N.ptr(user_in), N.ptr(user_out),
                                           ctypes.c_longlong(numel), ctypes.c_int(_DT[dtype]), ctypes.c_float(scale),
                                           ctypes.c_int(int(zero_contribution)), ctypes.c_int(ctas or DEFAULT_CTAS), N.stream_ptr()),
            "team_allreduce",
        )

    def allgather(self, shard_off: int, shard_bytes: int, dst: torch.Tensor, ctas: int = 0) -> None:
        d = self._desc()
        N.check(
            self.lib.ftb200_team_allgather(ctypes.byref(d), self._peer_ptrs(shard_off), N.ptr(dst),
                                           ctypes.c_longlong(shard_bytes), ctypes.c_int(ctas or DEFAULT_CTAS), N.stream_ptr()),
            "team_allgather",
        )

    def reduce_scatter(self, full_off: int, dst: torch.Tensor, shard_elems: int, dtype: torch.dtype, scale: float = 1.0,
                       ctas: int = 0) -> None:
        d = self._desc()
        N.check(
            self.lib.ftb200_team_reduce_scatter(ctypes.byref(d), self._peer_ptrs(full_off), N.ptr(dst),
                                                ctypes.c_longlong(shard_elems), ctypes.c_int(_DT[dtype]),
                                                ctypes.c_float(scale), ctypes.c_int(ctas or DEFAULT_CTAS), N.stream_ptr()),
            "team_reduce_scatter",
        )

    def reduce_local_slices(self, stage_off: int, dst: torch.Tensor, shard_elems: int, dtype: torch.dtype,
                            scale: float = 1.0, ctas: int = 0) -> None:
        """Second half of the GEMM-fused reduce-scatter: after a ready round (every peer's
        GEMM epilogue has stored its contribution into this rank's staging area
        ``[world, shard_elems]`` at ``stage_off``), sum the ``world`` slices locally into
        ``dst``; a done round then releases the staging area for reuse."""
        es = torch.empty((), dtype=dtype).element_size()
        arr = (ctypes.c_void_p * MAX_RANKS)()
        lo = shard_elems * self.rank
        for p in range(self.world):
            # the kernel reads src[p] + lo + i; make that land on slice p of the local staging area
            arr[p] = self.arena.base + stage_off + (p * shard_elems - lo) * es
        d = self._desc()
        N.check(
            self.lib.ftb200_team_reduce_scatter(ctypes.byref(d), arr, N.ptr(dst), ctypes.c_longlong(shard_elems),
                                                ctypes.c_int(_DT[dtype]), ctypes.c_float(scale),
                                                ctypes.c_int(ctas or DEFAULT_CTAS), N.stream_ptr()),
            "team_reduce_local_slices",
        )

    def barrier(self) -> None:
        d = self._desc()
        N.check(self.lib.ftb200_team_barrier(ctypes.byref(d), N.stream_ptr()), "team_barrier")

    def allreduce_oneshot(self, half_off: int, src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0,
                          zero_contribution: bool = False) -> None:
        """Small-message allreduce: one round instead of two.  ``half_off`` is the half of the small-message window
        that this call uses (callers alternate the halves); ``src``/``dst`` are local, 16-byte aligned, and may be
        the same tensor."""
        d = self._desc()
        N.check(
            self.lib.ftb200_team_allreduce_oneshot(ctypes.byref(d), self._peer_ptrs(half_off), N.ptr(src), N.ptr(dst),
                                                   ctypes.c_longlong(src.numel()), ctypes.c_int(_DT[src.dtype]),
                                                   ctypes.c_float(scale), ctypes.c_int(int(zero_contribution)),
                                                   N.stream_ptr()),
            "team_allreduce_oneshot",
        )

    def pull(self, segs: List[tuple], ctas: int = 0) -> None:
        """One collective launch in which this rank copies ``segs`` = ``[(src_ptr, dst_ptr, nbytes), ...]`` (at most
        one per rank; peer or local sources) between a ready and a done round.  Every rank of the team calls it, with
        an empty list if it has nothing to fetch."""
        src = (ctypes.c_void_p * MAX_RANKS)()
        dst = (ctypes.c_void_p * MAX_RANKS)()
        nb = (ctypes.c_longlong * MAX_RANKS)()
        for i, (sp, dp, b) in enumerate(segs):
            src[i], dst[i], nb[i] = sp, dp, b
        d = self._desc()
        N.check(self.lib.ftb200_team_pull(ctypes.byref(d), src, dst, nb, ctypes.c_int(len(segs)),
                                          ctypes.c_int(ctas or DEFAULT_CTAS), N.stream_ptr()), "team_pull")

    def sendrecv(self, peer: int, is_send: bool, pair_seq: int, src_ptr: int, dst_ptr: int, nbytes: int) -> None:
        """One side of a point-to-point transfer; ``pair_seq`` counts the transfers of this ordered pair."""
        d = self._desc_nocount()
        # the sender's rank is part of the token: a receiver's local go-word must never see the same value for
        # transfers from two different senders
        sender = self.rank if is_send else peer
        token = (self.epoch << 32) | (sender << 28) | (pair_seq & 0x0FFFFFFF)
        N.check(self.lib.ftb200_team_sendrecv(ctypes.byref(d), ctypes.c_int(peer), ctypes.c_int(int(is_send)),
                                              ctypes.c_ulonglong(token), ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst_ptr),
                                              ctypes.c_longlong(nbytes), ctypes.c_int(DEFAULT_CTAS), N.stream_ptr()),
                "team_sendrecv")


# ======================================================================================= FSDP


class PeerShardComm(ShardComm):
    """FSDP traffic of one replica group as peer-memory kernels.

    Buffers handed out by :meth:`alloc` live in the team arena, so the all-gather pulls
    parameter shards straight out of the peers' shard buffers into the local full unit and
    the reduce-scatter pulls this rank's slice out of the peers' full gradient units
    (fp32 accumulation, bf16 result).  Membership is static for the life of the group:
    losing a rank loses the replica group, which is the granularity of fault tolerance.
    """

    def __init__(self, group: dist.ProcessGroup, device: torch.device, arena_bytes: Optional[int] = None,
                 timeout: timedelta = timedelta(seconds=120)) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.device = torch.device(device)
        if arena_bytes is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            arena_bytes = int(free * 0.45)
        self.team = SymmetricTeam(self.device, arena_bytes, timeout)
        # exchange IPC handles through the (static) group itself
        handle = self.team.arena.export_handle()
        allh: List[Optional[bytes]] = [None] * self.size
        dist.all_gather_object(allh, handle, group=group)

        class _ListStore:
            def __init__(s) -> None:
                s.kv: Dict[str, bytes] = {f"arena/{p}": bytes(allh[p]) for p in range(self.size)}

            def set(s, k: str, v: bytes) -> None:
                s.kv[k] = v

            def get(s, k: str) -> bytes:
                return s.kv.get(k, b"1")

        self.team.connect(_ListStore(), self.rank, self.size, epoch=1)  # type: ignore[arg-type]
        dist.barrier(group=group)
        # scalars (the gradient norm) are reduced through the team too, so that nothing inside a step
        # is out of reach of the team's abort word and deadline
        self._scalar_n = 4 * MAX_RANKS
        self._scalar = self.alloc(self._scalar_n, torch.float32, self.device)

    def alloc(self, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        off = self.team.arena.alloc(numel * es)
        return self.team.arena.tensor(off, numel, dtype)

    def _off(self, t: torch.Tensor) -> int:
        off = self.team.arena.contains(t)
        if off is None:
            raise ValueError("tensor was not allocated by PeerShardComm.alloc")
        return off

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        self.team.allgather(self._off(shard), shard.numel() * shard.element_size(), full)

    def reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        self.team.reduce_scatter(self._off(full), shard, shard.numel(), shard.dtype)

    def all_reduce_sum_(self, t: torch.Tensor) -> None:
        n = t.numel()
        if t.dtype != torch.float32 or n > self._scalar_n:
            dist.all_reduce(t, group=self.group)
            return
        self._scalar.zero_()
        self._scalar[:n].copy_(t.reshape(-1))
        self.team.allreduce_(self._off(self._scalar), self._scalar_n, torch.float32, ctas=1)
        t.copy_(self._scalar[:n].view(t.shape))

    # ---- GEMM-fused reduce-scatter ------------------------------------------------------------
    supports_fused_scatter = True

    def stage_peers(self, stage: torch.Tensor):
        """Peer pointers of a staging buffer allocated with :meth:`alloc` (same offset in every arena)."""
        return self.team._peer_ptrs(self._off(stage))

    def reduce_stage(self, stage: torch.Tensor, shard: torch.Tensor) -> None:
        self.team.reduce_local_slices(self._off(stage), shard, shard.numel(), shard.dtype)

    def copy_segments(self, table: torch.Tensor, nsegs: int, total_bytes: int, ctas: int = 4) -> None:
        """One copy kernel over a device table of ``(peer source, local destination, bytes)`` segments (16-byte
        multiples), bounded by the team's abort word and reporting into its status word.  No rounds: the caller
        orders it after a collective that has told every rank that the sources are final."""
        N.check(N.lib().ftb200_p2p_copy(N.ptr(table), ctypes.c_int(nsegs), ctypes.c_longlong(total_bytes),
                                        ctypes.c_void_p(self.team._abort_dev), N.ptr(self.team._status), ctypes.c_int(ctas),
                                        N.stream_ptr()), "p2p_copy")

    def barrier(self) -> None:
        self.team.barrier()

    def shutdown(self) -> None:
        self.team.close()


# ======================================================================================= replica dim


class _StreamWork(Work):
    """Work of a kernel collective: complete when the launching stream reaches the event."""

    def __init__(self, pg: "ProcessGroupB200", result: object) -> None:
        super().__init__()
        self._pg = pg
        self._event = torch.cuda.Event()
        self._event.record()
        self._result = result
        self._fut: Optional[Future] = None

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        torch.cuda.current_stream().wait_event(self._event)
        return True

    def synchronize(self) -> None:
        self._event.synchronize()

    def block_current_stream(self, timeout: Optional[timedelta] = None) -> None:
        self.wait()

    def is_completed(self) -> bool:
        return self._event.query()

    def get_future(self) -> Future:
        # stream semantics as with NCCL futures: "done" means ordered on the stream
        if self._fut is None:
            self._fut = Future()
            self._fut.set_result(self._result)
        return self._fut


class ProcessGroupB200(ProcessGroup):
    """Reconfigurable replica-dimension group over NVLink peer memory.

    ``configure`` keeps this rank's arena, bumps the epoch, exchanges IPC handles under the
    given store prefix and maps the new peers.  ``allreduce`` is one fused kernel: stage
    (unless the tensor already lives in the arena, see :meth:`alloc`), two-shot reduce with
    fp32 accumulation, ``scale`` (the manager passes ``1/num_participants``), write back;
    messages up to 256 KB take a one-shot kernel with a single cross-rank round.
    ``abort`` is a store to a host-mapped word that all kernels poll; ``errored`` reads the
    status word after synchronising the stream.

    The rest of the c10d surface of the reference's groups (torchft/process_group.py:141-280)
    is built from three more kernels over a staging window of the arena: a generic *pull*
    (ready round, copies from peers' windows, done round) carries ``allgather``,
    ``allgather_into_tensor_coalesced``, ``broadcast``/``broadcast_one`` and ``alltoall_base``
    (equal splits) for any dtype; the pulling reduce-scatter carries ``reduce_scatter`` and
    ``reduce_scatter_tensor_coalesced`` (SUM/AVG, bf16/fp32); ``send``/``recv`` are a pair of
    kernels that hand a window from one rank to another without involving the rest of the
    team.  All of them are ordered on the current stream and return a stream-ordered work.
    A rank must not post a ``send`` to a peer that is itself blocked in a ``send`` to this
    rank on the same stream (as with NCCL outside of a group call).
    """

    supports_fused_scale = True

    SMALL_BYTES = 256 << 10  # messages up to this size take the one-shot allreduce

    def __init__(self, timeout: timedelta = timedelta(seconds=60), arena_bytes: int = 1 << 30,
                 staging_bytes: int = 256 << 20, device: Optional[torch.device] = None,
                 p2p_bytes: int = 64 << 20) -> None:
        super().__init__(0, 1)
        self._timeout = timeout
        self._device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._team = SymmetricTeam(self._device, arena_bytes + staging_bytes + p2p_bytes + 2 * self.SMALL_BYTES + (1 << 16),
                                   timeout)
        self._staging_bytes = staging_bytes
        self._staging_off = self._team.arena.alloc(staging_bytes)
        # send window of point-to-point transfers: its own, because a transfer (live recovery on
        # the manager's recovery stream) may run beside a collective that uses the staging window
        self._p2p_bytes = p2p_bytes // 16 * 16
        self._p2p_off = self._team.arena.alloc(p2p_bytes)
        self._small_off = self._team.arena.alloc(2 * self.SMALL_BYTES)
        self._small_calls = 0
        self._pair_seq: Dict[tuple, int] = {}
        self._rank, self._world = 0, 1
        self._errored: Optional[Exception] = None
        self._configured = False
        self._epoch = 0

    # ---- memory ---------------------------------------------------------------------------
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A tensor inside the exported arena: collectives on it run in place, without
        staging copies.  All replicas must allocate in the same order."""
        es = torch.empty((), dtype=dtype).element_size()
        return self._team.arena.tensor(self._team.arena.alloc(numel * es), numel, dtype)

    # ---- lifecycle --------------------------------------------------------------------------
    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int) -> None:
        store = create_store_client(store_addr, timeout=self._timeout)
        self._epoch += 1
        # the epoch must be common to all members: take it from the store prefix (quorum id)
        try:
            epoch = int(store_addr.rstrip("/").split("/")[-2])
        except (ValueError, IndexError):
            epoch = self._epoch
        self._team.connect(store, rank, world_size, epoch)
        self._rank, self._world = rank, world_size
        self._small_calls = 0
        self._pair_seq = {}
        self._errored = None
        self._configured = True

    def abort(self) -> None:
        self._errored = RuntimeError("aborted")
        self._team.abort()

    def shutdown(self) -> None:
        self._team.close()

    def errored(self) -> Optional[Exception]:
        if self._errored is None and self._configured:
            code = self._team.status()
            if code:
                self._errored = TeamError(f"peer-memory collective failed: {N.STATUS.get(code, code)}")
        return self._errored

    def set_timeout(self, timeout: timedelta) -> None:
        self._timeout = timeout
        self._team.timeout = timeout

    def size(self) -> int:
        return self._world

    def getBackendName(self) -> str:
        return "torchft-b200-peer"

    # ---- collectives --------------------------------------------------------------------------
    def allreduce(self, tensors: List[torch.Tensor], opts=None, scale: float = 1.0,
                  zero_contribution: bool = False) -> Work:
        op = _reduce_op(opts)
        if op == ReduceOp.AVG:
            scale = scale / self._world
        elif op != ReduceOp.SUM:
            raise NotImplementedError(f"ProcessGroupB200.allreduce supports SUM and AVG, got {op}")
        for t in tensors:
            if self._world == 1:
                # nothing to reduce: only the scale (and the zeroing of a spare) remains
                if zero_contribution:
                    t.zero_()
                elif scale != 1.0:
                    t.mul_(scale)
                continue
            self._allreduce_one(t, scale, zero_contribution)
        return _StreamWork(self, tensors)

    def _allreduce_one(self, t: torch.Tensor, scale: float, zero: bool) -> None:
        if t.dtype not in _DT:
            raise NotImplementedError(f"dtype {t.dtype} not supported by the peer-memory allreduce")
        if not t.is_contiguous():
            raise ValueError("allreduce needs contiguous tensors")
        es = t.element_size()
        gran = self._world * (16 // es)
        off = self._team.arena.contains(t)
        flat = t.view(-1)
        n = flat.numel()
        if off is not None and n % gran == 0 and off % 16 == 0:
            self._team.allreduce_(off, n, t.dtype, scale, zero_contribution=zero)
            return
        if n * es <= self.SMALL_BYTES:
            vec = 16 // es
            half = self._small_off + (self._small_calls % 2) * self.SMALL_BYTES
            self._small_calls += 1
            if n % vec == 0 and flat.data_ptr() % 16 == 0:
                self._team.allreduce_oneshot(half, flat, flat, scale, zero_contribution=zero)
            else:
                tmp = torch.zeros((n + vec - 1) // vec * vec, dtype=t.dtype, device=t.device)
                tmp[:n].copy_(flat)
                self._team.allreduce_oneshot(half, tmp, tmp, scale, zero_contribution=zero)
                flat.copy_(tmp[:n])
            return
        # staged path, in chunks of the staging window
        cap = (self._staging_bytes // es) // gran * gran
        pos = 0
        while pos < n:
            m = min(cap, n - pos)
            padded = (m + gran - 1) // gran * gran
            chunk = flat[pos : pos + m]
            if padded != m or (chunk.data_ptr() % 16):
                stage = self._team.arena.tensor(self._staging_off, padded, t.dtype)
                stage[:m].copy_(chunk)
                if padded != m:
                    stage[m:].zero_()
                self._team.allreduce_(self._staging_off, padded, t.dtype, scale, zero_contribution=zero)
                chunk.copy_(stage[:m])
            else:
                self._team.allreduce_(self._staging_off, m, t.dtype, scale, user_in=chunk, user_out=chunk,
                                      zero_contribution=zero)
            pos += m

    def allreduce_fp8(self, src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0,
                      minus: Optional[torch.Tensor] = None, zero_contribution: bool = False) -> None:
        """Quantised allreduce of flat ``src`` (or ``src - minus``) into ``dst`` as one fused
        kernel per rank: block-scaled e4m3 on the wire, fp32 accumulation, ``scale`` folded
        in.  ``numel`` must be a multiple of ``128 * world``; runs on the current stream.
        With ``zero_contribution`` this rank takes part but adds nothing (a healing or spare
        replica)."""
        from .. import quantization as Q

        n = src.numel()
        if n % (Q.BLOCK * self._world) or src.dtype not in _DT or not src.is_contiguous():
            raise ValueError("allreduce_fp8 needs a contiguous bf16/fp32 tensor of 128*world-multiple length")
        cap = self._staging_bytes * Q.BLOCK // (Q.BLOCK + 4) // (Q.BLOCK * self._world) * (Q.BLOCK * self._world)
        if self._world > 1:
            # Wait for the slowest rank in a one-warp kernel first.  The exchange kernel holds up to 96 CTAs of 512
            # threads at 96 registers, beside which no GEMM CTA fits on an SM: when it is the one that waits (tens
            # of milliseconds between drifting DiLoCo groups) the training stream that runs next to it crawls.
            self._team.barrier()
        pos = 0
        while pos < n:
            m = min(cap, n - pos)
            d = self._team._desc()
            N.check(
                self._team.lib.ftb200_team_allreduce_fp8(
                    ctypes.byref(d), self._team._peer_ptrs(self._staging_off), N.ptr(src[pos : pos + m]),
                    N.ptr(minus[pos : pos + m] if minus is not None else None), N.ptr(dst[pos : pos + m]),
                    ctypes.c_longlong(m), ctypes.c_int(_DT[src.dtype]), ctypes.c_float(scale),
                    ctypes.c_int(int(zero_contribution)), ctypes.c_int(0), N.stream_ptr()),
                "team_allreduce_fp8",
            )
            pos += m

    def barrier(self, opts=None) -> Work:
        self._team.barrier()
        return _StreamWork(self, None)

    def allreduce_coalesced(self, tensors: List[torch.Tensor], opts=None) -> Work:
        return self.allreduce(tensors, opts)

    # ---- byte-moving collectives over the staging window --------------------------------------------
    @staticmethod
    def _u8(t: torch.Tensor) -> torch.Tensor:
        if not t.is_contiguous():
            raise ValueError("ProcessGroupB200 collectives need contiguous tensors")
        return t.view(-1).view(torch.uint8)

    def _check_cuda(self, *tensors: torch.Tensor) -> None:
        for t in tensors:
            if t.device != self._device:
                raise ValueError(f"tensor on {t.device}, group on {self._device}")

    def _stage(self, nbytes: int) -> torch.Tensor:
        return self._team.arena.bytes_view[self._staging_off : self._staging_off + nbytes]

    def _gather_bytes(self, out_u8: torch.Tensor, in_u8: torch.Tensor) -> None:
        """out_u8[p * nb : (p + 1) * nb] = rank p's in_u8."""
        nb, world = in_u8.numel(), self._world
        if world == 1:
            out_u8.copy_(in_u8)
            return
        cap = self._staging_bytes // 16 * 16
        direct = nb % 16 == 0 and out_u8.data_ptr() % 16 == 0
        pos = 0
        while pos < nb:
            m = min(cap, nb - pos)
            mp = (m + 15) // 16 * 16
            self._stage(mp)[:m].copy_(in_u8[pos : pos + m])
            tmp = None if direct else torch.empty(world * mp, dtype=torch.uint8, device=self._device)
            segs = []
            for p in range(world):
                dst = out_u8.data_ptr() + p * nb + pos if direct else tmp.data_ptr() + p * mp
                segs.append((self._team.peer_base[p] + self._staging_off, dst, mp))
            self._team.pull(segs)
            if tmp is not None:
                for p in range(world):
                    out_u8[p * nb + pos : p * nb + pos + m].copy_(tmp[p * mp : p * mp + m])
            pos += m

    def allgather_into_tensor_coalesced(self, output_tensors: List[torch.Tensor], input_tensors: List[torch.Tensor],
                                        opts=None) -> Work:
        for out, inp in zip(output_tensors, input_tensors):
            self._check_cuda(out, inp)
            if out.numel() != inp.numel() * self._world or out.dtype != inp.dtype:
                raise ValueError("allgather_into_tensor: output must hold world_size inputs of the same dtype")
            self._gather_bytes(self._u8(out), self._u8(inp.contiguous()))
        return _StreamWork(self, output_tensors)

    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor], opts=None) -> Work:
        for outs, inp in zip(output_tensors, input_tensor):
            self._check_cuda(inp, *outs)
            if len(outs) != self._world:
                raise ValueError("allgather: one output tensor per rank")
            flat = torch.empty(self._world * inp.numel(), dtype=inp.dtype, device=self._device)
            self._gather_bytes(self._u8(flat), self._u8(inp.contiguous()))
            for p, o in enumerate(outs):
                o.copy_(flat[p * inp.numel() : (p + 1) * inp.numel()].view(inp.shape))
        return _StreamWork(self, output_tensors)

    def broadcast(self, tensor_list: List[torch.Tensor], opts=None) -> Work:
        root = int(getattr(opts, "rootRank", 0)) if opts is not None else 0
        for t in tensor_list:
            self._check_cuda(t)
            if self._world == 1:
                continue
            contiguous = t if t.is_contiguous() else t.contiguous()
            u8 = self._u8(contiguous)
            nb = u8.numel()
            cap = self._staging_bytes // 16 * 16
            direct = u8.data_ptr() % 16 == 0
            pos = 0
            while pos < nb:
                m = min(cap, nb - pos)
                mp = (m + 15) // 16 * 16
                direct_here = direct and m % 16 == 0
                if self._rank == root:
                    self._stage(mp)[:m].copy_(u8[pos : pos + m])
                    self._team.pull([])
                else:
                    tmp = None if direct_here else torch.empty(mp, dtype=torch.uint8, device=self._device)
                    dst = u8.data_ptr() + pos if direct_here else tmp.data_ptr()
                    self._team.pull([(self._team.peer_base[root] + self._staging_off, dst, mp)])
                    if tmp is not None:
                        u8[pos : pos + m].copy_(tmp[:m])
                pos += m
            if contiguous is not t:
                t.copy_(contiguous)
        return _StreamWork(self, tensor_list)

    def alltoall_base(self, output_buffer: torch.Tensor, input_buffer: torch.Tensor, output_split_sizes: List[int],
                      input_split_sizes: List[int], opts=None) -> Work:
        world = self._world
        for splits, buf in ((output_split_sizes, output_buffer), (input_split_sizes, input_buffer)):
            if splits and (len(splits) != world or len(set(splits)) != 1):
                raise NotImplementedError("ProcessGroupB200.alltoall_base supports equal splits only")
        self._check_cuda(output_buffer, input_buffer)
        out_u8, in_u8 = self._u8(output_buffer), self._u8(input_buffer.contiguous())
        if out_u8.numel() != in_u8.numel() or in_u8.numel() % world:
            raise ValueError("alltoall_base: buffers must have the same size, divisible by the world size")
        if world == 1:
            out_u8.copy_(in_u8)
            return _StreamWork(self, output_buffer)
        chunk = in_u8.numel() // world
        cap = (self._staging_bytes // world) // 16 * 16
        direct = chunk % 16 == 0 and out_u8.data_ptr() % 16 == 0
        in2, out2 = in_u8.view(world, chunk), out_u8.view(world, chunk)
        pos = 0
        while pos < chunk:
            m = min(cap, chunk - pos)
            mp = (m + 15) // 16 * 16
            self._stage(world * mp).view(world, mp)[:, :m].copy_(in2[:, pos : pos + m])
            tmp = None if direct else torch.empty(world, mp, dtype=torch.uint8, device=self._device)
            segs = []
            for p in range(world):
                dst = out_u8.data_ptr() + p * chunk + pos if direct else tmp.data_ptr() + p * mp
                segs.append((self._team.peer_base[p] + self._staging_off + self._rank * mp, dst, mp))
            self._team.pull(segs)
            if tmp is not None:
                out2[:, pos : pos + m].copy_(tmp[:, :m])
            pos += m
        return _StreamWork(self, output_buffer)

    def reduce_scatter_tensor_coalesced(self, output_tensors: List[torch.Tensor], input_tensors: List[torch.Tensor],
                                        opts=None) -> Work:
        op = _reduce_op(opts)
        if op not in (ReduceOp.SUM, ReduceOp.AVG):
            raise NotImplementedError(f"ProcessGroupB200.reduce_scatter supports SUM and AVG, got {op}")
        world = self._world
        scale = 1.0 / world if op == ReduceOp.AVG else 1.0
        for out, inp in zip(output_tensors, input_tensors):
            self._check_cuda(out, inp)
            if inp.dtype not in _DT or out.dtype != inp.dtype:
                raise NotImplementedError(f"dtype {inp.dtype} not supported by the peer-memory reduce-scatter")
            if inp.numel() != out.numel() * world:
                raise ValueError("reduce_scatter_tensor: input must hold world_size outputs")
            if not out.is_contiguous():
                raise ValueError("reduce_scatter_tensor needs a contiguous output")
            shard = out.numel()
            if world == 1:
                out.view(-1).copy_(inp.reshape(-1))
                if scale != 1.0:
                    out.mul_(scale)
                continue
            es = inp.element_size()
            vec = 16 // es
            in2 = inp.contiguous().view(world, shard)
            out1 = out.view(-1)
            cap = (self._staging_bytes // es // world) // vec * vec
            direct = shard % vec == 0 and out1.data_ptr() % 16 == 0
            pos = 0
            while pos < shard:
                m = min(cap, shard - pos)
                mp = (m + vec - 1) // vec * vec
                stage = self._team.arena.tensor(self._staging_off, world * mp, inp.dtype).view(world, mp)
                stage[:, :m].copy_(in2[:, pos : pos + m])
                if mp != m:
                    stage[:, m:].zero_()
                dst = out1[pos : pos + m] if direct else torch.empty(mp, dtype=inp.dtype, device=self._device)
                self._team.reduce_scatter(self._staging_off, dst, mp, inp.dtype, scale)
                if not direct:
                    out1[pos : pos + m].copy_(dst[:m])
                pos += m
        return _StreamWork(self, output_tensors)

    def reduce_scatter(self, output_tensors: List[torch.Tensor], input_tensors: List[List[torch.Tensor]],
                       opts=None) -> Work:
        flat = [torch.cat([t.reshape(-1) for t in ins]) for ins in input_tensors]
        return self.reduce_scatter_tensor_coalesced(output_tensors, flat, opts)

    # ---- point to point -----------------------------------------------------------------------------
    def _next_pair(self, src: int, dst: int) -> int:
        k = self._pair_seq.get((src, dst), 0) + 1
        self._pair_seq[(src, dst)] = k
        return k

    def send(self, tensors: List[torch.Tensor], dst_rank: int, tag: int = 0) -> Work:
        """Hands ``tensors`` to ``dst_rank`` through this rank's send window; transfers between a pair of ranks
        match in posting order (``tag`` is not used for matching)."""
        for t in tensors:
            self._check_cuda(t)
            u8 = self._u8(t.contiguous())
            nb, pos = u8.numel(), 0
            while pos < nb or nb == 0:
                m = min(self._p2p_bytes, nb - pos)
                mp = (m + 15) // 16 * 16
                window = self._team.arena.bytes_view[self._p2p_off : self._p2p_off + mp]
                window[:m].copy_(u8[pos : pos + m])
                self._team.sendrecv(dst_rank, True, self._next_pair(self._rank, dst_rank), 0, 0, mp)
                pos += m
                if nb == 0:
                    break
        return _StreamWork(self, tensors)

    def recv(self, tensors: List[torch.Tensor], src_rank: int, tag: int = 0) -> Work:
        for t in tensors:
            self._check_cuda(t)
            if not t.is_contiguous():
                raise ValueError("recv needs contiguous tensors")
            u8 = self._u8(t)
            nb, pos = u8.numel(), 0
            src = self._team.peer_base[src_rank] + self._p2p_off
            while pos < nb or nb == 0:
                m = min(self._p2p_bytes, nb - pos)
                mp = (m + 15) // 16 * 16
                direct = m % 16 == 0 and (u8.data_ptr() + pos) % 16 == 0
                tmp = None if direct else torch.empty(mp, dtype=torch.uint8, device=self._device)
                dst = u8.data_ptr() + pos if direct else tmp.data_ptr()
                self._team.sendrecv(src_rank, False, self._next_pair(src_rank, self._rank), src, dst, mp)
                if tmp is not None:
                    u8[pos : pos + m].copy_(tmp[:m])
                pos += m
                if nb == 0:
                    break
        return _StreamWork(self, tensors)

    def __repr__(self) -> str:
        return f"ProcessGroupB200(rank={self._rank}, world={self._world}, epoch={self._team.epoch})"
