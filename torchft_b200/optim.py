"""Optimizer wrapper that ties an optimizer to the fault-tolerance protocol."""

from __future__ import annotations

from typing import TYPE_CHECKING, Any, Dict, List, Mapping, Optional

import torch
from torch.optim import Optimizer

if TYPE_CHECKING:
    from .manager import Manager


class OptimizerWrapper(Optimizer):
    """``zero_grad()`` starts the step's quorum, ``step()`` applies the update only when
    the manager's commit vote passes.  Everything else is forwarded to the wrapped
    optimizer.  Closures are not supported.  (Contract of torchft/optim.py:24-63.)

    Typical loop::

        optim = OptimizerWrapper(manager, torch.optim.AdamW(model.parameters()))
        for batch in data:
            optim.zero_grad()      # quorum
            loss(model(batch)).backward()
            optim.step()           # commit-gated
    """

    def __init__(self, manager: "Manager", optim: Optimizer) -> None:
        self.optim = optim
        self.manager = manager

    def add_param_group(self, param_group: Dict[str, Any]) -> None:
        self.optim.add_param_group(param_group)

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        self.optim.load_state_dict(state_dict)

    def state_dict(self) -> Dict[str, Any]:
        return self.optim.state_dict()

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.manager.start_quorum()
        self.optim.zero_grad(set_to_none)

    def step(self, closure: Optional[object] = None) -> None:
        assert closure is None, "optimizers that use closures are not supported"
        if self.manager.should_commit():
            self.optim.step()

    @property
    def param_groups(self) -> List[Dict[str, Any]]:
        return self.optim.param_groups

    @property
    def state(self) -> Mapping[torch.Tensor, Any]:  # type: ignore[override]
        return self.optim.state
