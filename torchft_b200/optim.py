"""Optimizer wrapper that ties an optimizer to the fault-tolerance protocol."""

from __future__ import annotations

from typing import TYPE_CHECKING, Callable, Optional

from torch.optim import Optimizer

if TYPE_CHECKING:
    from .manager import Manager

# Everything that is not part of the protocol goes to the wrapped optimizer unchanged, so that checkpointing code,
# learning-rate schedulers and hook users see the real optimizer's state.
_FORWARDED_METHODS = (
    "state_dict",
    "load_state_dict",
    "add_param_group",
    "register_step_pre_hook",
    "register_step_post_hook",
    "register_state_dict_pre_hook",
    "register_state_dict_post_hook",
    "register_load_state_dict_pre_hook",
    "register_load_state_dict_post_hook",
)
_FORWARDED_ATTRIBUTES = ("param_groups", "state", "defaults")


class OptimizerWrapper(Optimizer):
    """A view of ``optim`` whose ``zero_grad()`` opens the step (joins the quorum) and whose ``step()`` applies the
    update only when the manager's commit vote passes; a step that does not commit leaves weights and optimizer
    state untouched.  ``last_step_committed`` tells which of the two happened.  The wrapper owns no parameters of
    its own: state, parameter groups, hooks and (de)serialisation are the wrapped optimizer's.  Closures are not
    supported.  (Same contract as torchft/optim.py:24-63.)

    Typical loop::

        optim = OptimizerWrapper(manager, torch.optim.AdamW(model.parameters()))
        for batch in data:
            optim.zero_grad()      # quorum
            loss(model(batch)).backward()
            optim.step()           # commit-gated
    """

    def __init__(self, manager: "Manager", optim: Optimizer) -> None:
        # no Optimizer.__init__ on purpose: there is nothing to register here, see the class docstring
        self.manager = manager
        self.optim = optim
        self.last_step_committed: Optional[bool] = None

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.manager.start_quorum()
        self.optim.zero_grad(set_to_none)

    def step(self, closure: Optional[object] = None) -> None:
        if closure is not None:
            raise AssertionError("optimizers that use closures are not supported: the commit vote needs the finished backward pass")
        self.last_step_committed = bool(self.manager.should_commit())
        if self.last_step_committed:
            self.optim.step()

    def __repr__(self) -> str:
        return f"OptimizerWrapper({self.optim!r})"


def _forward_method(name: str) -> Callable[..., object]:
    def call(self: OptimizerWrapper, *args: object, **kwargs: object) -> object:
        return getattr(self.optim, name)(*args, **kwargs)

    call.__name__ = name
    call.__qualname__ = f"OptimizerWrapper.{name}"
    call.__doc__ = f"Forwards to the wrapped optimizer's ``{name}``."
    return call


def _forward_attribute(name: str) -> property:
    def read(self: OptimizerWrapper) -> object:
        return getattr(self.optim, name)

    return property(read, doc=f"The wrapped optimizer's ``{name}``.")


for _name in _FORWARDED_METHODS:
    setattr(OptimizerWrapper, _name, _forward_method(_name))
for _name in _FORWARDED_ATTRIBUTES:
    setattr(OptimizerWrapper, _name, _forward_attribute(_name))
del _name
