"""Intra-replica-group communication used by the sharded (FSDP-style) trainer.

The trainer needs three operations over the shard group: all-gather of parameter
shards into a full unit, reduce-scatter of a full gradient unit into gradient shards,
and a scalar all-reduce for the gradient norm.  Three interchangeable back-ends:

* :class:`LocalShardComm` -- group of one, everything is a no-op/alias;
* :class:`TorchShardComm` -- ``torch.distributed`` collectives (NCCL on GPUs, gloo on
  CPU); the measured baseline and the CPU test vehicle;
* :class:`PeerShardComm` (in :mod:`torchft_b200.parallel.team`) -- hand-written
  kernels that read peers' memory directly over NVLink.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class ShardComm:
    rank: int = 0
    size: int = 1

    def alloc(self, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        """Allocate a buffer that the back-end can communicate from/into."""
        return torch.empty(numel, dtype=dtype, device=device)

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        raise NotImplementedError

    def reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        """``shard = sum_over_ranks(full[rank slice])`` (fp32 accumulation)."""
        raise NotImplementedError

    def all_reduce_sum_(self, t: torch.Tensor) -> None:
        raise NotImplementedError

    def barrier(self) -> None:
        pass

    def shutdown(self) -> None:
        pass


class LocalShardComm(ShardComm):
    def all_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        if shard.data_ptr() != full.data_ptr():
            full[: shard.numel()].copy_(shard)

    def reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        if shard.data_ptr() != full.data_ptr():
            shard.copy_(full[: shard.numel()])

    def all_reduce_sum_(self, t: torch.Tensor) -> None:
        pass


class TorchShardComm(ShardComm):
    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        dist.all_gather_into_tensor(full, shard, group=self.group)

    def reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        if full.is_cuda:
            dist.reduce_scatter_tensor(shard, full, op=dist.ReduceOp.SUM, group=self.group)
        else:  # gloo has no reduce_scatter: all-reduce a fp32 copy and slice
            tmp = full.float()
            dist.all_reduce(tmp, group=self.group)
            n = shard.numel()
            shard.copy_(tmp[self.rank * n : (self.rank + 1) * n].to(shard.dtype))

    def all_reduce_sum_(self, t: torch.Tensor) -> None:
        dist.all_reduce(t, group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)
