"""Fault-tolerant data parallel wrappers.

The replica dimension of a fault-tolerant job has a world size that changes from step to
step, so gradient averaging goes through ``Manager.allreduce`` instead of a fixed
communicator.
"""


from typing import TYPE_CHECKING

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import parallel

from .process_group import ProcessGroupDummy

if TYPE_CHECKING:
    from .manager import Manager


class DistributedDataParallel(parallel.DistributedDataParallel):
    """``torch.nn.parallel.DistributedDataParallel`` whose gradient buckets are averaged
    by a :class:`~torchft_b200.manager.Manager`.

    torch's reducer does the bucketing and overlaps communication with backward; a
    communication hook hands each bucket to ``manager.allreduce`` (which also applies the
    ``1/num_participants`` scale).  The module is built on a world-of-one dummy group, so
    DDP's construction-time broadcast and shape verification are no-ops: weights must be
    synchronised at step 0 by the manager (``init_sync=True``) or by identical seeding.
    ``find_unused_parameters`` is forced on to stop the reducer from rebuilding its
    buckets after the first iteration -- a replica that heals later must end up with the
    same bucket layout as its peers.  (Behaviour of torchft/ddp.py:32-79.)
    """

    def __init__(self, manager: "Manager", module: nn.Module, **kwargs: object) -> None:
        pg = ProcessGroupDummy(0, 1)
        super().__init__(module, process_group=pg, find_unused_parameters=True, **kwargs)  # type: ignore[arg-type]
        self.register_comm_hook(manager, self._comm_hook)

    @staticmethod
    def _comm_hook(state: "Manager", bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
        work = state.allreduce(bucket.buffer())
        work.wait()
        fut = work.get_future()
        # the reducer needs a plain torch future resolving to the bucket tensor
        out: torch.futures.Future[torch.Tensor] = torch.futures.Future()
        out.set_result(bucket.buffer())
        return out


class PureDistributedDataParallel(nn.Module):
    """Minimal variant: one ``manager.allreduce`` per parameter, issued from a
    post-accumulate-grad hook.  No bucketing, no overlap tuning -- useful as a readable
    reference and for models with few, large parameters."""

    def __init__(self, manager: "Manager", module: nn.Module) -> None:
        super().__init__()
        self.module = module

        def post_grad_hook(p: torch.Tensor) -> None:
            if p.grad is not None:
                manager.allreduce(p.grad).wait()

        for p in module.parameters():
            p.register_post_accumulate_grad_hook(post_grad_hook)

    def forward(self, *args: object) -> object:
        return self.module(*args)
