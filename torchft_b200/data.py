"""Data sharding across replica groups."""

from __future__ import annotations

from typing import Optional

import torch.distributed as dist
from torch.utils import data


class DistributedSampler(data.distributed.DistributedSampler):
    """``DistributedSampler`` for a job made of ``num_replica_groups`` groups of
    ``num_replicas`` ranks: the shard of rank ``group_rank`` in group ``replica_rank`` is
    ``group_rank + num_replicas * replica_rank`` out of
    ``num_replicas * num_replica_groups`` (torchft/data.py:24-77).

    The sharding is static: when a group is down its shard is simply not visited that
    step, and a group that restarts gets the same shard back, so restoring the
    dataloader position from a checkpoint stays meaningful.  Jobs whose membership
    changes often may prefer drawing batches at random per replica.
    """

    def __init__(self, dataset: data.Dataset, replica_rank: int, num_replica_groups: int,
                 group_rank: Optional[int] = None, num_replicas: Optional[int] = None, **kwargs: object) -> None:
        if group_rank is None:
            group_rank = dist.get_rank()
        if num_replicas is None:
            num_replicas = dist.get_world_size()
        self.global_rank: int = group_rank + num_replicas * replica_rank
        self.global_world_size: int = num_replicas * num_replica_groups
        super().__init__(dataset, rank=self.global_rank, num_replicas=self.global_world_size, **kwargs)  # type: ignore[arg-type]
