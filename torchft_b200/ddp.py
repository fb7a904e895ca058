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
        if "process_group" in kwargs or "find_unused_parameters" in kwargs:
            raise TypeError("process_group and find_unused_parameters are fixed by the fault-tolerant wrapper")
        super().__init__(
            module,
            process_group=ProcessGroupDummy(0, 1),  # swallows construction-time collectives
            find_unused_parameters=True,  # keeps the bucket layout fixed, see above
            **kwargs,  # type: ignore[arg-type]
        )
        self.register_comm_hook(manager, _average_bucket)


def _average_bucket(manager: "Manager", bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """DDP communication hook: average one gradient bucket over the participating replica groups.  The manager's
    work is waited here (errors are latched inside the manager, never raised), and the reducer gets an already
    completed plain future holding the bucket."""
    flat = bucket.buffer()
    manager.allreduce(flat).wait()
    done: torch.futures.Future[torch.Tensor] = torch.futures.Future()
    done.set_result(flat)
    return done


class PureDistributedDataParallel(nn.Module):
    """Minimal variant: one ``manager.allreduce`` per parameter, issued from a
    post-accumulate-grad hook.  No bucketing, no overlap tuning -- useful as a readable
    reference and for models with few, large parameters."""

    def __init__(self, manager: "Manager", module: nn.Module) -> None:
        super().__init__()
        self.module = module
        self._hooks = [p.register_post_accumulate_grad_hook(self._make_hook(manager)) for p in module.parameters()]

    @staticmethod
    def _make_hook(manager: "Manager"):
        def average(param: torch.Tensor) -> None:
            grad = param.grad
            if grad is not None:
                manager.allreduce(grad).wait()

        return average

    def forward(self, *args: object, **kwargs: object) -> object:
        return self.module(*args, **kwargs)
