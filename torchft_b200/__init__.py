"""torchft_b200: per-step fault tolerance for PyTorch training, built natively for B200.

Public surface mirrors ``torchft``: ``Manager``, ``Optimizer`` (the commit-gated
optimizer wrapper), ``DistributedDataParallel``, ``DistributedSampler`` and the
reconfigurable process groups; plus ``ProcessGroupB200``, the NVLink peer-memory group.
Importing the package configures the three structured event loggers.
"""

try:
    from . import _ftcp  # noqa: F401  (C++ control plane)
except ImportError:  # first import of a fresh checkout: compile it in-tree
    from . import _build

    _build.build_control()
    from . import _ftcp  # noqa: F401

from .data import DistributedSampler
from .ddp import DistributedDataParallel
from .manager import Manager
from .optim import OptimizerWrapper as Optimizer
from .otel import setup_logger
from .process_group import (
    ProcessGroupBabyGloo,
    ProcessGroupBabyNCCL,
    ProcessGroupGloo,
    ProcessGroupNCCL,
)

setup_logger("torchft_quorums")
setup_logger("torchft_commits")
setup_logger("torchft_errors")

__all__ = (
    "DistributedDataParallel",
    "DistributedSampler",
    "Manager",
    "Optimizer",
    "ProcessGroupNCCL",
    "ProcessGroupBabyNCCL",
    "ProcessGroupGloo",
    "ProcessGroupBabyGloo",
)


def __getattr__(name):
    # the peer-memory group pulls in the kernel library bindings: resolved on first use
    if name == "ProcessGroupB200":
        from .parallel.team import ProcessGroupB200

        return ProcessGroupB200
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
