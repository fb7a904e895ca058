"""Base class of the reconfigurable process groups and the store-address helper.

Kept in its own module so that both :mod:`torchft_b200.process_group` and
:mod:`torchft_b200.process_group_baby` can build on it without importing each other.
"""

from __future__ import annotations

from datetime import timedelta
from typing import List, Optional, Union

import torch
import torch.distributed as dist
from torch.distributed import PrefixStore, ProcessGroup as BaseProcessGroup, Store, TCPStore
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


def create_store_client(store_addr: str, timeout: timedelta) -> Store:
    """``host:port/some/prefix`` -> a ``PrefixStore`` over a ``TCPStore`` client."""
    host_port, _, prefix = store_addr.partition("/")
    host, _, port = host_port.rpartition(":")
    if host.startswith("[") and host.endswith("]"):
        host = host[1:-1]
    store = TCPStore(host_name=host, port=int(port), is_master=False, wait_for_workers=False, timeout=timeout)
    return PrefixStore(prefix, store)


def _reduce_op(opts: Union[AllreduceOptions, ReduceOp, ReduceOp.RedOpType, None]) -> ReduceOp.RedOpType:
    """The reduction of an options object (or of a bare op) as the plain enum value, so that
    ``op in (ReduceOp.SUM, ReduceOp.AVG)`` works (a ``ReduceOp`` object only compares equal to
    the enum when it is the left operand)."""
    if opts is None:
        return ReduceOp.SUM
    op = opts if isinstance(opts, (ReduceOp, ReduceOp.RedOpType)) else opts.reduceOp
    return getattr(op, "op", op)  # a ReduceOp object carries its enum value in .op


class ProcessGroup(BaseProcessGroup):
    """Base class.  Subclasses implement the collectives they support; everything else
    raises ``NotImplementedError`` so a missing op is loud."""

    def __init__(self, *args: object, **kwargs: object) -> None:
        super().__init__(*args, **kwargs)
        self._group_name: Optional[str] = None

    # ---- collectives (c10d signatures) ---------------------------------------------------
    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor],
                  opts: Optional[AllgatherOptions] = None) -> Work:
        raise NotImplementedError("allgather")

    def allgather_into_tensor_coalesced(self, output_tensors: List[torch.Tensor], input_tensors: List[torch.Tensor],
                                        opts: Optional[AllgatherOptions] = None) -> Work:
        raise NotImplementedError("allgather_into_tensor_coalesced")

    def allreduce(self, tensors: List[torch.Tensor], opts: Union[AllreduceOptions, ReduceOp, None] = None) -> Work:
        raise NotImplementedError("allreduce")

    def allreduce_coalesced(self, tensors: List[torch.Tensor], opts: Optional[AllreduceCoalescedOptions] = None) -> Work:
        raise NotImplementedError("allreduce_coalesced")

    def alltoall_base(self, output_buffer: torch.Tensor, input_buffer: torch.Tensor, output_split_sizes: List[int],
                      input_split_sizes: List[int], opts: Optional[AllToAllOptions] = None) -> Work:
        raise NotImplementedError("alltoall_base")

    def barrier(self, opts: Optional[BarrierOptions] = None) -> Work:
        raise NotImplementedError("barrier")

    def broadcast(self, tensor_list: List[torch.Tensor], opts: Optional[BroadcastOptions] = None) -> Work:
        raise NotImplementedError("broadcast")

    def broadcast_one(self, tensor: torch.Tensor, root: int) -> Work:
        opts = BroadcastOptions()
        opts.rootRank = root
        return self.broadcast([tensor], opts)

    def recv(self, tensors: List[torch.Tensor], src_rank: int, tag: int) -> Work:
        raise NotImplementedError("recv")

    def reduce_scatter(self, output_tensors: List[torch.Tensor], input_tensors: List[List[torch.Tensor]],
                       opts: Optional[ReduceScatterOptions] = None) -> Work:
        raise NotImplementedError("reduce_scatter")

    def reduce_scatter_tensor_coalesced(self, output_tensors: List[torch.Tensor], input_tensors: List[torch.Tensor],
                                        opts: Optional[ReduceScatterOptions] = None) -> Work:
        raise NotImplementedError("reduce_scatter_tensor_coalesced")

    def send(self, tensors: List[torch.Tensor], dst_rank: int, tag: int) -> Work:
        raise NotImplementedError("send")

    # ---- lifecycle ------------------------------------------------------------------------
    def configure(self, store_addr: str, replica_id: str, rank: int, world_size: int) -> None:
        """(Re)build the communicator.  ``store_addr`` (``host:port/prefix``) must be unique
        per call; blocks until the group is usable, raises on failure."""
        raise NotImplementedError("configure")

    def size(self) -> int:
        raise NotImplementedError("size")

    def getBackendName(self) -> str:
        raise NotImplementedError("getBackendName")

    def abort(self) -> None:
        """Tear the communicator down without waiting for peers (callable from any thread)."""

    def shutdown(self) -> None:
        """Release every resource of the group."""

    def errored(self) -> Optional[Exception]:
        """The asynchronous error that requires a reconfigure, if one happened."""
        return None

    def set_timeout(self, timeout: timedelta) -> None:
        raise NotImplementedError("set_timeout")

    # ---- registration with torch.distributed's global registry ------------------------------
    def _register(self, name: str) -> str:
        group_name = f"{self.getBackendName()}:{name}"

        def create_pg(prefix_store: PrefixStore, rank: int, world_size: int, timeout: float) -> "ProcessGroup":
            return self

        devices = ["cpu"]
        if torch.cuda.is_available():
            devices.append("cuda")
        dist.Backend.register_backend(group_name, create_pg, devices=devices)
        return group_name

    def register(self, name: str) -> BaseProcessGroup:
        """Register under a unique ``name`` so DeviceMesh / functional collectives can
        resolve this object; returns the world-of-one group torch.distributed hands out.
        Call once."""
        group_name = self._register(name)
        return dist.new_group(ranks=[dist.get_rank()], backend=group_name, group_desc=group_name,
                              timeout=timedelta(seconds=60.0))

    @property
    def group_name(self) -> str:
        if self._group_name is None:
            raise ValueError("ProcessGroup name not set")
        return self._group_name

    def _set_group_name(self, name: str) -> None:
        self._group_name = name

    def unregister(self) -> None:
        dist.destroy_process_group(self)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}()"


