"""Python entry points of the sm_100a kernels, with plain-PyTorch references.

Every public function dispatches on the device of its arguments:

* CUDA tensors run the hand-written kernel from ``libftb200_kernels.so`` on the
  current stream (never an eager fallback);
* CPU tensors run the ``ref_*`` function of the same name, an fp32 PyTorch
  restatement of the kernel's math.  The ``ref_*`` functions are also the oracles of
  the GPU numerics tests.
"""

from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _native as N
from ._native import c_float, c_int, c_ll, ptr, stream_ptr

# --------------------------------------------------------------------------- status word

_status_words: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write a code into."""
    key = (device.type, device.index)
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = w
    return w


def check_status(device: torch.device) -> None:
    """Synchronising read of the status word; raises if any kernel reported a failure."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise N.KernelError(f"device-side status: {N.STATUS.get(code, code)}")


# --------------------------------------------------------------------------- GEMM


def _check_2d_bf16(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.dtype != torch.bfloat16 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D bf16 tensor with unit inner stride")


# Which GEMM kernel `gemm` launches: "2cta" (pairs of CTAs, tcgen05.mma.cta_group::2) or
# "1cta".  Overridable per call and through the FTB200_GEMM environment variable.
GEMM_IMPL = os.environ.get("FTB200_GEMM", "2cta")


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    out_dtype: torch.dtype = torch.bfloat16,
    max_ctas: int = 0,
    impl: Optional[str] = None,
) -> torch.Tensor:
    """``out (+)= A @ B^T`` with logical ``A [M,K]`` and ``B [N,K]``.

    ``a_mn_major`` says ``a`` is stored as the row-major ``[K, M]`` matrix (and likewise
    for ``b``), which is how the dgrad and wgrad GEMMs of a linear layer read their
    operands without transposed copies.
    """
    _check_2d_bf16(a, "a")
    _check_2d_bf16(b, "b")
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, Nn = b.shape
    else:
        Nn, Kb = b.shape
    if K != Kb:
        raise ValueError(f"reduction dims differ: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an output tensor")
        out = torch.empty(M, Nn, dtype=out_dtype, device=a.device)
    if out.shape != (M, Nn) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("bad output tensor")
    if not a.is_cuda:
        af = a.float().t() if a_mn_major else a.float()
        bf = b.float() if b_mn_major else b.float().t()
        r = af @ bf
        if accumulate:
            r = r + out.float()
        out.copy_(r.to(out.dtype))
        return out
    flags = (1 if out.dtype == torch.float32 else 0) | (2 if accumulate else 0)
    fn = N.lib().ftb200_gemm_bf16_2cta if (impl or GEMM_IMPL) == "2cta" else N.lib().ftb200_gemm_bf16
    rc = fn(
        ptr(a), ptr(b), ptr(out), c_int(M), c_int(Nn), c_int(K), c_int(int(a_mn_major)), c_int(int(b_mn_major)),
        c_ll(a.stride(0)), c_ll(b.stride(0)), c_ll(out.stride(0)), c_int(flags), ptr(status_word(a.device)),
        c_int(max_ctas), stream_ptr(),
    )
    N.check(rc, "gemm_bf16")
    return out


class ScatterField:
    """Destination of a weight-gradient GEMM whose epilogue performs the reduce-scatter's
    transfer: a ``[rows, cols]`` field at element offset ``unit_off`` of a flat gradient unit
    sharded over ``world`` ranks; ``peers`` are the ranks' staging areas (``[world, shard]``)."""

    def __init__(self, peers, world: int, src_rank: int, shard_elems: int, unit_off: int, shape) -> None:
        self.peers, self.world, self.src_rank = peers, world, src_rank
        self.shard_elems, self.unit_off, self.shape = shard_elems, unit_off, tuple(shape)


def gemm_scatter(a: torch.Tensor, b: torch.Tensor, a_mn_major: bool, b_mn_major: bool, dst: ScatterField) -> None:
    """``A @ B^T`` written straight into the owners' staging areas (see :class:`ScatterField`)."""
    _check_2d_bf16(a, "a")
    _check_2d_bf16(b, "b")
    K_, M = a.shape if a_mn_major else a.shape[::-1]
    Kb, Nn = b.shape if b_mn_major else b.shape[::-1]
    if K_ != Kb or (M, Nn) != dst.shape:
        raise ValueError(f"shape mismatch: {(M, Nn)} vs field {dst.shape}")
    rc = N.lib().ftb200_gemm_bf16_scatter(
        ptr(a), ptr(b), c_int(M), c_int(Nn), c_int(K_), c_int(int(a_mn_major)), c_int(int(b_mn_major)), c_ll(a.stride(0)),
        c_ll(b.stride(0)), dst.peers, c_int(dst.world), c_int(dst.src_rank), c_ll(dst.shard_elems), c_ll(dst.unit_off),
        ptr(status_word(a.device)), c_int(0), stream_ptr())
    N.check(rc, "gemm_bf16_scatter")


def scatter_to_stage(src: torch.Tensor, dst: ScatterField) -> None:
    """Copy a small bf16 field (e.g. a norm-weight gradient) to its owners' staging areas."""
    N.check(N.lib().ftb200_scatter_to_stage(ptr(src), c_ll(src.numel()), c_ll(dst.unit_off), c_ll(dst.shard_elems), dst.peers,
                                            c_int(dst.world), c_int(dst.src_rank), stream_ptr()), "scatter_to_stage")


class GatherField:
    """A weight that is still spread over its shard group: ``local`` is its ``[N, K]`` place in this rank's gathered
    copy of a flat parameter unit (``unit_off`` elements from the unit's start), ``peers`` the ranks' shard buffers
    of that unit (``shard_elems`` elements each).  The first forward GEMM that consumes the field gathers it while
    it multiplies (:func:`gemm_gather`) and clears ``pending``; from then on ``local`` is the gathered weight."""

    def __init__(self, local: torch.Tensor, peers, world: int, shard_elems: int, unit_off: int, sync: torch.Tensor) -> None:
        self.local, self.peers, self.world = local, peers, world
        self.shard_elems, self.unit_off, self.sync = shard_elems, unit_off, sync
        self.pending = True

    @staticmethod
    def supported(shape, shard_elems: int) -> bool:
        return len(shape) == 2 and shape[0] % 128 == 0 and shape[1] % 64 == 0 and shard_elems >= 8192 and shard_elems % 8 == 0


def gemm_gather(x: torch.Tensor, w: GatherField, out: torch.Tensor, aux: Optional[torch.Tensor] = None) -> None:
    """``out = x @ W^T`` with the all-gather of ``W`` fused into the GEMM: extra warps of the kernel pull ``W``'s
    rows out of the shard owners' memory over NVLink in tile order while the tensor cores already work on the
    rows that have arrived.  ``aux`` as in :func:`linear_swiglu_fwd`."""
    _check_2d_bf16(x, "x")
    Nn, Kd = w.local.shape
    T = x.shape[0]
    if x.shape[1] != Kd or tuple(out.shape) != (T, Nn) or w.sync.numel() < 1 + Nn // 128:
        raise ValueError(f"shape mismatch: x {tuple(x.shape)}, w {(Nn, Kd)}, out {tuple(out.shape)}")
    rc = N.lib().ftb200_gemm_bf16_gather(
        ptr(x), ptr(w.local), ptr(out), c_int(T), c_int(Nn), c_int(Kd), c_ll(x.stride(0)), c_ll(out.stride(0)), w.peers,
        c_int(w.world), c_ll(w.shard_elems), c_ll(w.unit_off), ptr(w.sync), ptr(aux) if aux is not None else None,
        c_ll(aux.stride(0) if aux is not None else 0), ptr(status_word(x.device)), c_int(0), stream_ptr())
    N.check(rc, "gemm_bf16_gather")
    w.pending = False


def linear_fwd(x: torch.Tensor, w, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = x @ w^T`` (x ``[T,K]``, w ``[N,K]`` or a :class:`GatherField`)."""
    if isinstance(w, GatherField):
        if w.pending:
            if out is None:
                out = torch.empty(x.shape[0], w.local.shape[0], dtype=x.dtype, device=x.device)
            gemm_gather(x, w, out)
            return out
        w = w.local
    return gemm(x, w, False, False, out=out)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False) -> torch.Tensor:
    """``dx = dy @ w`` (dy ``[T,N]``, w ``[N,K]``)."""
    return gemm(dy, w, False, True, out=out, accumulate=accumulate)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``dw = dy^T @ x`` (dy ``[T,N]``, x ``[T,K]``) -> ``[N,K]``.  ``out`` may be a
    :class:`ScatterField`: the result then goes straight to the shard owners."""
    if isinstance(out, ScatterField):
        if accumulate:
            raise ValueError("a scattered weight gradient cannot accumulate")
        gemm_scatter(dy, x, True, True, out)
        return out  # type: ignore[return-value]
    return gemm(dy, x, True, True, out=out, accumulate=accumulate, out_dtype=out_dtype)


# --------------------------------------------------------------------------- embedding


def embedding_fwd(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = tokens.numel()
    V, D = table.shape
    if out is None:
        out = torch.empty(T, D, dtype=table.dtype, device=table.device)
    if not table.is_cuda:
        out.copy_(table[tokens.reshape(-1)])
        return out
    N.check(N.lib().ftb200_embedding_fwd(ptr(tokens), ptr(table), ptr(out), c_int(T), c_int(D), c_int(V), stream_ptr()),
            "embedding_fwd")
    return out


def embedding_bwd(tokens: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor) -> torch.Tensor:
    """``dtable[tokens[t]] += dout[t]`` (``dtable`` must be zeroed by the caller)."""
    T = tokens.numel()
    V, D = dtable.shape
    if not dtable.is_cuda:
        dtable.copy_(dtable.float().index_add_(0, tokens.reshape(-1), dout.float()).to(dtable.dtype))
        return dtable
    N.check(N.lib().ftb200_embedding_bwd(ptr(tokens), ptr(dout), ptr(dtable), c_int(T), c_int(D), c_int(V), stream_ptr()),
            "embedding_bwd")
    return dtable


# --------------------------------------------------------------------------- RMSNorm


def ref_rmsnorm_fwd(x, w, eps, res=None):
    h = x.float()
    if res is not None:
        h = (h + res.float()).to(x.dtype).float()
    rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return (h * rstd * w.float()).to(x.dtype), rstd.squeeze(-1), h.to(x.dtype)


def rmsnorm_fwd(
    x: torch.Tensor,
    w: torch.Tensor,
    eps: float = 1e-5,
    res: Optional[torch.Tensor] = None,
    h_out: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    rstd: Optional[torch.Tensor] = None,
    want_out: bool = True,
) -> Tuple[Optional[torch.Tensor], torch.Tensor, torch.Tensor]:
    """Returns ``(normed, rstd, h)`` where ``h = x + res`` (or ``x``)."""
    T, D = x.shape
    if rstd is None:
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    if res is not None and h_out is None:
        h_out = torch.empty_like(x)
    if want_out and out is None:
        out = torch.empty_like(x)
    if not x.is_cuda:
        o, r, h = ref_rmsnorm_fwd(x, w, eps, res)
        rstd.copy_(r)
        if res is not None:
            h_out.copy_(h)
        if want_out:
            out.copy_(o)
        return (out if want_out else None), rstd, (h_out if res is not None else x)
    N.check(
        N.lib().ftb200_rmsnorm_fwd(ptr(x), ptr(res), ptr(h_out), ptr(w), ptr(out if want_out else None), ptr(rstd),
                                   c_int(T), c_int(D), c_float(eps), stream_ptr()),
        "rmsnorm_fwd",
    )
    return (out if want_out else None), rstd, (h_out if res is not None else x)


def ref_rmsnorm_bwd(dy, x, w, rstd, dres=None):
    dyf, xf, wf = dy.float(), x.float(), w.float()
    r = rstd.float().unsqueeze(-1)
    D = x.shape[-1]
    dot = (dyf * wf * xf).sum(-1, keepdim=True)
    dx = r * wf * dyf - xf * dot * r.pow(3) / D
    if dres is not None:
        dx = dx + dres.float()
    dw = (dyf * xf * r).sum(0)
    return dx.to(x.dtype), dw


_rms_scratch: dict = {}


def rmsnorm_bwd(
    dy: torch.Tensor,
    x: torch.Tensor,
    w: torch.Tensor,
    rstd: torch.Tensor,
    dres: Optional[torch.Tensor] = None,
    dx: Optional[torch.Tensor] = None,
    dw: Optional[torch.Tensor] = None,
    accumulate_dw: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    T, D = x.shape
    if dx is None:
        dx = torch.empty_like(x)
    if dw is None:
        dw = torch.zeros(D, dtype=w.dtype, device=x.device)
    if not x.is_cuda:
        rdx, rdw = ref_rmsnorm_bwd(dy, x, w, rstd, dres)
        dx.copy_(rdx)
        dw.copy_(((dw.float() if accumulate_dw else 0) + rdw).to(dw.dtype))
        return dx, dw
    L = N.lib()
    L.ftb200_rmsnorm_bwd_scratch_floats.restype = c_ll
    need = int(L.ftb200_rmsnorm_bwd_scratch_floats(c_int(D)))
    key = (x.device.index, need)
    scratch = _rms_scratch.get(key)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=x.device)
        _rms_scratch[key] = scratch
    N.check(
        L.ftb200_rmsnorm_bwd(ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(dw), ptr(scratch), c_int(T),
                             c_int(D), c_int(int(accumulate_dw)), stream_ptr()),
        "rmsnorm_bwd",
        launches=2,
    )
    return dx, dw


# --------------------------------------------------------------------------- RoPE


def rope_table(seq_len: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """``[S, head_dim/2, 2]`` fp32 table of (cos, sin) for interleaved-pair rotation."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).float().to(device).contiguous()


def ref_rope(buf, table, S, n_heads, head_dim, backward=False):
    T = buf.shape[0]
    rot = buf[:, : n_heads * head_dim].float().reshape(T, n_heads, head_dim // 2, 2)
    pos = torch.arange(T, device=buf.device) % S
    cs = table[pos].unsqueeze(1)  # T,1,Dh/2,2
    c, s = cs[..., 0], cs[..., 1]
    if backward:
        s = -s
    x0, x1 = rot[..., 0], rot[..., 1]
    o = torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).reshape(T, n_heads * head_dim)
    res = buf.clone()
    res[:, : n_heads * head_dim] = o.to(buf.dtype)
    return res


def rope_(buf: torch.Tensor, table: torch.Tensor, seq_len: int, n_heads: int, head_dim: int,
          backward: bool = False) -> torch.Tensor:
    """Rotate the first ``n_heads`` heads of every row of ``buf`` ``[T, >= n_heads*head_dim]`` in place."""
    T = buf.shape[0]
    if not buf.is_cuda:
        buf.copy_(ref_rope(buf, table, seq_len, n_heads, head_dim, backward))
        return buf
    N.check(
        N.lib().ftb200_rope(ptr(buf), ptr(table), c_ll(T), c_int(seq_len), c_int(n_heads), c_int(head_dim),
                            c_ll(buf.stride(0)), c_int(int(backward)), stream_ptr()),
        "rope",
    )
    return buf


# --------------------------------------------------------------------------- SwiGLU


def ref_swiglu_fwd(gu):
    """``gu`` rows are interleaved (gate, up) pairs."""
    g, u = gu[:, 0::2].float(), gu[:, 1::2].float()
    return (F.silu(g) * u).to(gu.dtype)


def swiglu_fwd(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[:, j] = silu(gu[:, 2j]) * gu[:, 2j+1]`` (interleaved gate/up columns)."""
    T, F2 = gu.shape
    Fd = F2 // 2
    if out is None:
        out = torch.empty(T, Fd, dtype=gu.dtype, device=gu.device)
    if not gu.is_cuda:
        out.copy_(ref_swiglu_fwd(gu))
        return out
    N.check(N.lib().ftb200_swiglu_fwd(ptr(gu), ptr(out), c_ll(T), c_int(Fd), stream_ptr()), "swiglu_fwd")
    return out


def ref_swiglu_bwd(ds, gu):
    g, u, d = gu[:, 0::2].float(), gu[:, 1::2].float(), ds.float()
    sg = torch.sigmoid(g)
    silu = g * sg
    out = torch.empty(gu.shape, dtype=torch.float32, device=gu.device)
    out[:, 0::2] = d * u * (sg + silu * (1 - sg))
    out[:, 1::2] = d * silu
    return out.to(gu.dtype)


def swiglu_bwd(ds: torch.Tensor, gu: torch.Tensor, dgu: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dgu`` may alias ``gu`` (in place)."""
    T, F2 = gu.shape
    if dgu is None:
        dgu = torch.empty_like(gu)
    if not gu.is_cuda:
        dgu.copy_(ref_swiglu_bwd(ds, gu))
        return dgu
    N.check(N.lib().ftb200_swiglu_bwd(ptr(ds), ptr(gu), ptr(dgu), c_ll(T), c_int(F2 // 2), stream_ptr()), "swiglu_bwd")
    return dgu


def linear_swiglu_fwd(x: torch.Tensor, w_gu: torch.Tensor, gu_out: torch.Tensor, s_out: torch.Tensor) -> None:
    """``gu_out = x @ w_gu^T`` and, from the same accumulator, ``s_out = silu(gate) * up``
    where ``w_gu``'s rows (``gu_out``'s columns) interleave gate and up."""
    if isinstance(w_gu, GatherField):
        if w_gu.pending:
            gemm_gather(x, w_gu, gu_out, aux=s_out)
            return
        w_gu = w_gu.local
    T, Kd = x.shape
    N2 = w_gu.shape[0]
    if not x.is_cuda or N2 % 32 or GEMM_IMPL != "2cta":
        gemm(x, w_gu, False, False, out=gu_out)
        swiglu_fwd(gu_out, out=s_out)
        return
    rc = N.lib().ftb200_gemm_bf16_swiglu(
        ptr(x), ptr(w_gu), ptr(gu_out), ptr(s_out), c_int(T), c_int(N2), c_int(Kd), c_ll(x.stride(0)), c_ll(w_gu.stride(0)),
        c_ll(gu_out.stride(0)), c_ll(s_out.stride(0)), ptr(status_word(x.device)), c_int(0), stream_ptr())
    N.check(rc, "gemm_bf16_swiglu")


# --------------------------------------------------------------------------- cross-entropy


def ref_cross_entropy(logits, target, grad_scale):
    lf = logits.float()
    loss = F.cross_entropy(lf, target, reduction="none")
    p = torch.softmax(lf, dim=-1)
    p[torch.arange(lf.shape[0]), target] -= 1.0
    return loss, (p * grad_scale).to(logits.dtype)


def cross_entropy_(logits: torch.Tensor, target: torch.Tensor, grad_scale: float,
                   loss: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-row loss; ``logits`` is overwritten by ``(softmax - onehot) * grad_scale``."""
    T, V = logits.shape
    if loss is None:
        loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    if not logits.is_cuda:
        l, g = ref_cross_entropy(logits, target, grad_scale)
        loss.copy_(l)
        logits.copy_(g)
        return loss
    N.check(
        N.lib().ftb200_cross_entropy(ptr(logits), ptr(target), ptr(loss), c_int(T), c_int(V), c_ll(logits.stride(0)),
                                     c_float(grad_scale), stream_ptr()),
        "cross_entropy",
    )
    return loss


# --------------------------------------------------------------------------- AdamW / grad norm


def ref_adamw(master, m, v, grad, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    g = grad.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2s = math.sqrt(1 - beta2 ** step)
    denom = v.sqrt() / bc2s + eps
    master.mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)


def adamw_(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
           param_lp: Optional[torch.Tensor], lr: float, beta1: float, beta2: float, eps: float, wd: float,
           step: int, grad_scale: Optional[torch.Tensor] = None) -> None:
    """One fused AdamW step over flat buffers (fp32 state, bf16 or fp32 grads, bf16 write-back)."""
    n = master.numel()
    if not master.is_cuda:
        gs = float(grad_scale.item()) if grad_scale is not None else 1.0
        ref_adamw(master.view(-1), m.view(-1), v.view(-1), grad.reshape(-1), lr, beta1, beta2, eps, wd, step, gs)
        if param_lp is not None:
            param_lp.view(-1).copy_(master.view(-1).to(param_lp.dtype))
        return
    N.check(
        N.lib().ftb200_adamw(ptr(master), ptr(m), ptr(v), ptr(grad), c_int(int(grad.dtype == torch.float32)),
                             ptr(param_lp), c_ll(n), c_float(lr), c_float(beta1), c_float(beta2), c_float(eps),
                             c_float(wd), c_int(step), ptr(grad_scale), stream_ptr()),
        "adamw",
    )


def sumsq_(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out += sum(x^2)`` (``out`` is a 1-element fp32 tensor)."""
    if not x.is_cuda:
        out.add_(x.float().pow(2).sum())
        return out
    N.check(N.lib().ftb200_sumsq(ptr(x), c_int(int(x.dtype == torch.float32)), c_ll(x.numel()), ptr(out), stream_ptr()),
            "sumsq")
    return out


def clip_coef_(sumsq: torch.Tensor, max_norm: float, coef: torch.Tensor, norm_out: Optional[torch.Tensor] = None) -> None:
    if not sumsq.is_cuda:
        nrm = sumsq.sqrt()
        if norm_out is not None:
            norm_out.copy_(nrm)
        coef.copy_(torch.clamp(max_norm / (nrm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(nrm))
        return
    N.check(N.lib().ftb200_clip_coef(ptr(sumsq), c_float(max_norm), ptr(coef), ptr(norm_out), stream_ptr()), "clip_coef")


# --------------------------------------------------------------------------- attention


def ref_attention(q, k, v, causal=True):
    """q ``[B,S,Hq,Dh]``, k/v ``[B,S,Hkv,Dh]`` -> ``[B,S,Hq,Dh]`` (fp32 math)."""
    B, S, Hq, Dh = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(Dh)
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)


def ref_attention_lse(q, k, v, causal=True):
    """Row-wise ``logsumexp(scale * q k^T)`` ``[B,Hq,S]`` (fp32) of the same problem."""
    B, S, Hq, Dh = q.shape
    rep = Hq // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(Dh)
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    return torch.logsumexp(s, dim=-1)


def attention_supported(seq_len: int, head_dim: int) -> bool:
    """Shapes the tcgen05 attention kernels take: head dim 128 with 128-row blocks, or head dim 64 with
    sequences that are a multiple of 256 (the forward kernel for it works on two 128-query tiles per CTA)."""
    return (head_dim == 128 and seq_len % 128 == 0) or (head_dim == 64 and seq_len % 256 == 0)


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, batch: int, seq_len: int, n_heads: int,
                  n_kv_heads: int, head_dim: int, out: torch.Tensor, lse: Optional[torch.Tensor] = None,
                  causal: bool = True) -> None:
    """Causal GQA attention forward.  ``q`` ``[batch*seq, n_heads*head_dim]`` and ``k``/``v``
    ``[batch*seq, n_kv_heads*head_dim]`` are 2-D bf16 views (column slices of the packed QKV
    activation are fine), ``out`` ``[batch*seq, n_heads*head_dim]``, ``lse`` ``[batch, n_heads,
    seq]`` fp32 (saved for the backward pass)."""
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (out, "out")):
        _check_2d_bf16(t, name)
    if not q.is_cuda:
        B, S = batch, seq_len
        q4, k4, v4 = (t.reshape(B, S, -1, head_dim) for t in (q, k, v))
        out.copy_(ref_attention(q4, k4, v4, causal).reshape(B * S, -1))
        if lse is not None:
            lse.copy_(ref_attention_lse(q4, k4, v4, causal))
        return
    scale = 1.0 / math.sqrt(head_dim)
    impl = os.environ.get("FTB200_ATTN_FWD", "auto")
    if impl == "auto":
        impl = "single"  # same speed as "pair" at head dim 128 and fewer registers
    if impl == "pair" or head_dim != 128:
        # two query tiles per CTA, one softmax thread per row (head dim 64 or 128, seq % 256 == 0)
        poly = int(os.environ.get("FTB200_ATTN_POLY", "0"))
        N.check(
            N.lib().ftb200_attention_fwd2(ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), c_int(batch), c_int(seq_len),
                                          c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_ll(q.stride(0)),
                                          c_ll(k.stride(0)), c_ll(v.stride(0)), c_ll(out.stride(0)), c_float(scale),
                                          c_int(int(causal)), c_int(poly), ptr(status_word(q.device)), stream_ptr()),
            "attention_fwd2",
        )
        return
    N.check(
        N.lib().ftb200_attention_fwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), c_int(batch), c_int(seq_len), c_int(n_heads),
                                     c_int(n_kv_heads), c_int(head_dim), c_ll(q.stride(0)), c_ll(k.stride(0)),
                                     c_ll(v.stride(0)), c_ll(out.stride(0)), c_float(scale), c_int(int(causal)),
                                     ptr(status_word(q.device)), stream_ptr()),
        "attention_fwd",
    )


def ref_attention_bwd(q, k, v, d_o, causal=True):
    """(dq, dk, dv) of :func:`ref_attention` by autograd in fp32; 4-D inputs as there."""
    q, k, v = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o = ref_attention(q, k, v, causal)
    return torch.autograd.grad(o, (q, k, v), d_o.float())


_attn_scratch: dict = {}


def attention_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, d_o: torch.Tensor,
                  lse: torch.Tensor, dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor, batch: int, seq_len: int,
                  n_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True) -> None:
    """Backward of :func:`attention_fwd`: writes ``dq``, ``dk``, ``dv`` (2-D bf16 views like
    ``q``, ``k``, ``v``; column slices of a packed dQKV buffer are fine).  The fp32 dQ
    accumulator lives in a per-device scratch buffer that is reused across calls on the same
    stream."""
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (d_o, "d_o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        _check_2d_bf16(t, name)
    if not q.is_cuda:
        B, S = batch, seq_len
        q4, k4, v4, do4 = (t.reshape(B, S, -1, head_dim) for t in (q, k, v, d_o))
        gq, gk, gv = ref_attention_bwd(q4, k4, v4, do4, causal)
        dq.copy_(gq.reshape(B * S, -1))
        dk.copy_(gk.reshape(B * S, -1))
        dv.copy_(gv.reshape(B * S, -1))
        return
    lib = N.lib()
    lib.ftb200_attention_bwd_scratch_bytes.restype = ctypes.c_longlong
    need = int(lib.ftb200_attention_bwd_scratch_bytes(c_int(batch), c_int(seq_len), c_int(n_heads)))
    key = (q.device.index, torch.cuda.current_stream().cuda_stream)
    scratch = _attn_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _attn_scratch[key] = scratch
    scale = 1.0 / math.sqrt(head_dim)
    N.check(
        lib.ftb200_attention_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(d_o), ptr(lse), ptr(dq), ptr(dk), ptr(dv), ptr(scratch),
                                 c_int(batch), c_int(seq_len), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                                 c_ll(q.stride(0)), c_ll(k.stride(0)), c_ll(v.stride(0)), c_ll(o.stride(0)),
                                 c_ll(d_o.stride(0)), c_ll(dq.stride(0)), c_ll(dk.stride(0)), c_ll(dv.stride(0)),
                                 c_float(scale), c_int(int(causal)), ptr(status_word(q.device)), stream_ptr()),
        "attention_bwd", launches=3,
    )
