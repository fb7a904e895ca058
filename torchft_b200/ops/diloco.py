"""Fused multi-tensor operations of the DiLoCo outer loop on flat buffers.

``outer_step_`` is the whole post-commit part of a fragment synchronisation in one kernel:
Nesterov (or plain) momentum SGD on the averaged pseudo-gradient, write of the new global
weights into the backup, and blending of the live weights with the local ones
(``fragment_update_alpha``).  The reference does this as four passes of eager per-tensor
ops (torchft/local_sgd.py:465-470 with ``torch.optim.SGD``).  The pseudo-gradient itself
(``backup - param``) is formed inside the quantised allreduce kernel
(:meth:`torchft_b200.parallel.team.ProcessGroupB200.allreduce_fp8` with ``minus=``).
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native as N

_DT = {torch.bfloat16: 0, torch.float32: 1}


def ref_outer_step(g, momentum, backup, param, lr, mu, alpha, nesterov, first_step):
    gf = g.float()
    if mu != 0:
        if first_step:
            momentum.copy_(gf)
        else:
            momentum.mul_(mu).add_(gf)
        u = gf + mu * momentum if nesterov else momentum
    else:
        u = gf
    G = backup.float() - lr * u
    local = param.float()
    backup.copy_(G.to(backup.dtype))
    param.copy_((G + alpha * (local - G)).to(param.dtype))


def outer_step_(g: torch.Tensor, momentum: Optional[torch.Tensor], backup: torch.Tensor, param: torch.Tensor, lr: float,
                momentum_coef: float = 0.0, alpha: float = 0.0, nesterov: bool = True, first_step: bool = False) -> None:
    """``v = mu v + g; u = g + mu v (nesterov) or v; G = backup - lr u; backup = G;
    param = G + alpha (param - G)`` on flat, contiguous tensors of one dtype (fp32 or bf16;
    the momentum buffer ``momentum`` is always fp32; ``momentum_coef`` is mu)."""
    mu = float(momentum_coef)
    n = g.numel()
    if not g.is_cuda:
        ref_outer_step(g, momentum, backup, param, lr, mu, alpha, nesterov, first_step)
        return
    if n % 4 or g.dtype not in _DT or backup.dtype != g.dtype or param.dtype != g.dtype:
        ref_outer_step(g, momentum, backup, param, lr, mu, alpha, nesterov, first_step)
        return
    N.check(
        N.lib().ftb200_diloco_outer_step(N.ptr(g), N.ptr(momentum), N.ptr(backup), N.ptr(param), ctypes.c_longlong(n),
                                         ctypes.c_int(_DT[g.dtype]), ctypes.c_float(lr), ctypes.c_float(mu),
                                         ctypes.c_float(alpha), ctypes.c_int(int(nesterov)), ctypes.c_int(int(first_step)),
                                         N.stream_ptr()),
        "diloco_outer_step",
    )
