"""Llama-3 style decoder trained by an explicit (autograd-free) forward/backward engine.

The reference project ships no model code; its Llama runs come from an external
trainer layered on ``torchft``.  Here the model is part of the framework because the
fault-tolerant HSDP step is built around it: parameters live in flat per-layer
*units* (the FSDP sharding granule), every activation that backward needs sits in a
preallocated buffer, and each hot op is one of the sm_100a kernels in
:mod:`torchft_b200.ops.kernels`.

Unit layout (bf16, every field a multiple of 8 elements so all views are 16-byte
aligned)::

    layer unit : attn_norm[D] | wqkv[(Hq+2Hkv)*Dh, D] | wo[D, D] | ffn_norm[D] | wgu[2F, D] | wd[D, F]
                 (rows of wgu interleave gate and up: gate_0, up_0, gate_1, up_1, ...)
    embed unit : tok_embeddings[V, D]
    head  unit : final_norm[D] | lm_head[V, D]

RoPE rotates interleaved pairs ``(2i, 2i+1)`` with ``theta = rope_theta``.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..ops import kernels as K


@dataclass
class LlamaConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    vocab_size: int = 128256
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    name: str = "llama3-8b"

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def layer_fields(self) -> List[Tuple[str, Tuple[int, ...]]]:
        D, Fd = self.dim, self.ffn_dim
        return [
            ("attn_norm", (D,)),
            ("wqkv", (self.qkv_dim, D)),
            ("wo", (D, D)),
            ("ffn_norm", (D,)),
            ("wgu", (2 * Fd, D)),
            ("wd", (D, Fd)),
        ]

    def unit_fields(self, unit: int) -> List[Tuple[str, Tuple[int, ...]]]:
        """Unit 0 is the embedding, 1..n_layers the blocks, n_layers+1 the head."""
        if unit == 0:
            return [("tok_embeddings", (self.vocab_size, self.dim))]
        if unit == self.n_layers + 1:
            return [("final_norm", (self.dim,)), ("lm_head", (self.vocab_size, self.dim))]
        return self.layer_fields()

    @property
    def n_units(self) -> int:
        return self.n_layers + 2

    def unit_numel(self, unit: int) -> int:
        return sum(math.prod(s) for _, s in self.unit_fields(unit))

    def num_params(self) -> int:
        return sum(self.unit_numel(u) for u in range(self.n_units))

    def flops_per_token(self, seq_len: int) -> float:
        """Model FLOPs per token for one training step (matmuls + causal attention)."""
        dense = self.num_params() - self.vocab_size * self.dim  # the embedding lookup is not a matmul
        attn = 6 * self.n_layers * self.dim * seq_len  # 12*L*D*S halved by causality
        return 6.0 * dense + attn


LLAMA3_8B = LlamaConfig()
LLAMA3_1B = LlamaConfig(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim=8192, name="llama3-1b")
LLAMA_TINY = LlamaConfig(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512, vocab_size=1024, name="llama-tiny")
LLAMA_SMALL = LlamaConfig(dim=1024, n_layers=4, n_heads=8, n_kv_heads=2, ffn_dim=2816, vocab_size=8192, name="llama-small")

CONFIGS = {c.name: c for c in (LLAMA3_8B, LLAMA3_1B, LLAMA_TINY, LLAMA_SMALL)}


class _Fields:
    """Named views into one flat unit buffer."""

    def __init__(self, flat: torch.Tensor, fields: List[Tuple[str, Tuple[int, ...]]]):
        off = 0
        for name, shape in fields:
            n = math.prod(shape)
            setattr(self, name, flat[off : off + n].view(*shape))
            off += n


class SdpaAttention:
    """Causal GQA attention through ``torch``'s fused SDPA (library kernel).

    Used where the hand-written attention kernel is not selected; keeps a one-op
    autograd graph per layer so that backward reuses the library's saved statistics.
    """

    def __init__(self, cfg: LlamaConfig):
        self.cfg = cfg
        self._saved: Dict[int, Tuple[torch.Tensor, ...]] = {}

    def forward(self, layer: int, qkv: torch.Tensor, batch: int, seq: int, out: torch.Tensor, need_grad: bool) -> None:
        c = self.cfg
        Hq, Hkv, Dh = c.n_heads, c.n_kv_heads, c.head_dim
        q = qkv[:, : Hq * Dh].view(batch, seq, Hq, Dh).transpose(1, 2)
        k = qkv[:, Hq * Dh : (Hq + Hkv) * Dh].view(batch, seq, Hkv, Dh).transpose(1, 2)
        v = qkv[:, (Hq + Hkv) * Dh :].view(batch, seq, Hkv, Dh).transpose(1, 2)
        if need_grad:
            q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
            with torch.enable_grad():
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            self._saved[layer] = (q, k, v, o)
        else:
            with torch.no_grad():
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        out.view(batch, seq, Hq, Dh).copy_(o.detach().transpose(1, 2))

    def backward(self, layer: int, dout: torch.Tensor, batch: int, seq: int, dqkv: torch.Tensor) -> None:
        c = self.cfg
        Hq, Hkv, Dh = c.n_heads, c.n_kv_heads, c.head_dim
        q, k, v, o = self._saved.pop(layer)
        do = dout.view(batch, seq, Hq, Dh).transpose(1, 2)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
        dqkv[:, : Hq * Dh].view(batch, seq, Hq, Dh).copy_(dq.transpose(1, 2))
        dqkv[:, Hq * Dh : (Hq + Hkv) * Dh].view(batch, seq, Hkv, Dh).copy_(dk.transpose(1, 2))
        dqkv[:, (Hq + Hkv) * Dh :].view(batch, seq, Hkv, Dh).copy_(dv.transpose(1, 2))

    def reset(self) -> None:
        self._saved.clear()


class Tcgen05Attention:
    """Causal GQA attention on the hand-written tcgen05 kernels.  Q, K and V are read in
    place from the packed QKV activation and dQ, dK, dV are written in place into the packed
    dQKV workspace; only the per-row log-sum-exp is saved between the passes."""

    def __init__(self, cfg: LlamaConfig):
        self.cfg = cfg
        self._saved: Dict[int, Tuple[torch.Tensor, ...]] = {}
        self._lse_pool: List[torch.Tensor] = []

    def _views(self, qkv: torch.Tensor):
        c = self.cfg
        a, b = c.n_heads * c.head_dim, (c.n_heads + c.n_kv_heads) * c.head_dim
        return qkv[:, :a], qkv[:, a:b], qkv[:, b:]

    def forward(self, layer: int, qkv: torch.Tensor, batch: int, seq: int, out: torch.Tensor, need_grad: bool) -> None:
        c = self.cfg
        q, k, v = self._views(qkv)
        lse = None
        if need_grad:
            lse = self._lse_pool.pop() if self._lse_pool else torch.empty(batch, c.n_heads, seq, dtype=torch.float32,
                                                                          device=qkv.device)
            self._saved[layer] = (qkv, out, lse)
        K.attention_fwd(q, k, v, batch, seq, c.n_heads, c.n_kv_heads, c.head_dim, out, lse, causal=True)

    def backward(self, layer: int, dout: torch.Tensor, batch: int, seq: int, dqkv: torch.Tensor) -> None:
        c = self.cfg
        qkv, out, lse = self._saved.pop(layer)
        q, k, v = self._views(qkv)
        dq, dk, dv = self._views(dqkv)
        K.attention_bwd(q, k, v, out, dout, lse, dq, dk, dv, batch, seq, c.n_heads, c.n_kv_heads, c.head_dim, causal=True)
        self._lse_pool.append(lse)

    def reset(self) -> None:
        for _, _, lse in self._saved.values():
            self._lse_pool.append(lse)
        self._saved.clear()


def make_attention(cfg: LlamaConfig, seq_len: int, device: torch.device, kind: Optional[str] = None):
    """``kind``: "tcgen05" (hand-written kernels; CUDA, head dim 128 and a sequence that is a multiple of 128,
    or head dim 64 and a multiple of 256), "sdpa" (library), or None for tcgen05 where it applies.  The environment variable
    ``FTB200_ATTENTION`` overrides None."""
    kind = kind or os.environ.get("FTB200_ATTENTION") or "auto"
    ok = device.type == "cuda" and K.attention_supported(seq_len, cfg.head_dim)
    if kind == "tcgen05" and not ok:
        raise ValueError("tcgen05 attention needs CUDA and head_dim 128 with seq_len % 128 == 0 or head_dim 64 with "
                         "seq_len % 256 == 0")
    if kind == "tcgen05" or (kind == "auto" and ok):
        return Tcgen05Attention(cfg)
    return SdpaAttention(cfg)


class LlamaEngine:
    """Forward/backward of a Llama decoder over externally owned parameter/grad units.

    ``param_unit(u)`` returns the full (gathered) bf16 flat buffer of unit ``u`` and
    ``grad_unit(u)`` the full flat gradient buffer to write; ``unit_ready`` /
    ``grad_done`` hooks let a sharding layer prefetch parameters and reduce
    gradients while compute continues.
    """

    def __init__(
        self,
        cfg: LlamaConfig,
        batch: int,
        seq_len: int,
        device: torch.device,
        param_unit: Callable[[int], torch.Tensor],
        grad_unit: Callable[[int], torch.Tensor],
        before_unit: Optional[Callable[[int, bool], None]] = None,
        grad_done: Optional[Callable[[int], None]] = None,
        attention: Optional[object] = None,
        logit_chunks: int = 4,
        grad_fields: Optional[Callable[[int], object]] = None,
        grad_scale: float = 1.0,
        fwd_fields: Optional[Callable[[int], object]] = None,
        wgrad_stream: bool = True,
        save_norms: Optional[bool] = None,
    ):
        self.cfg, self.B, self.S, self.device = cfg, batch, seq_len, device
        self.grad_fields = grad_fields
        # forward-pass view of a unit's parameters, when it differs from the plain views: a sharding layer may hand
        # out `K.GatherField`s, weights that the first consuming GEMM gathers from the shard group as it runs
        self.fwd_fields = fwd_fields
        # multiplies every gradient (not the reported loss): 1/shard-group size when the group's
        # gradients are summed, so that the result is the mean over all of the group's tokens
        self.grad_scale = float(grad_scale)
        self.T = batch * seq_len
        self.param_unit, self.grad_unit = param_unit, grad_unit
        self.before_unit = before_unit or (lambda u, backward: None)
        self.grad_done = grad_done or (lambda u: None)
        if attention is None or isinstance(attention, str):
            attention = make_attention(cfg, seq_len, device, attention)
        self.attn = attention
        self.logit_chunks = max(1, logit_chunks)
        while self.T % self.logit_chunks:
            self.logit_chunks -= 1
        T, D, Fd, QKV, L = self.T, cfg.dim, cfg.ffn_dim, cfg.qkv_dim, cfg.n_layers
        bf = dict(dtype=torch.bfloat16, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        # saved activations
        self.x = [torch.empty(T, D, **bf) for _ in range(L + 1)]  # residual stream entering layer l (x[L]: final)
        self.h = [torch.empty(T, D, **bf) for _ in range(L)]
        self.qkv = [torch.empty(T, QKV, **bf) for _ in range(L)]
        self.att = [torch.empty(T, D, **bf) for _ in range(L)]
        self.gu = [torch.empty(T, 2 * Fd, **bf) for _ in range(L)]
        self.s = [torch.empty(T, Fd, **bf) for _ in range(L)]  # silu(gate)*up, kept for the wd wgrad
        self.rstd1 = [torch.empty(T, **f32) for _ in range(L + 1)]
        self.rstd2 = [torch.empty(T, **f32) for _ in range(L)]
        # workspaces
        self.ws_n = torch.empty(T, D, **bf)
        self.ws_n2 = torch.empty(T, D, **bf)  # the FFN-side norm recomputed in the backward pass (see _wgrad)
        self.ws_proj = torch.empty(T, D, **bf)
        self.ws_s = torch.empty(T, Fd, **bf)
        self.ws_ds = torch.empty(T, Fd, **bf)
        self.ws_dn = torch.empty(T, D, **bf)
        self.ws_dh = torch.empty(T, D, **bf)
        self.ws_dy = torch.empty(T, D, **bf)
        self.ws_dqkv = torch.empty(T, QKV, **bf)
        self.logits = torch.empty(T // self.logit_chunks, cfg.vocab_size, **bf)
        self.loss_rows = torch.empty(T, **f32)
        self.rope = K.rope_table(seq_len, cfg.head_dim, cfg.rope_theta, device)
        self.kernel_launches = 0
        # The normalised inputs of the QKV and gate/up GEMMs are needed again by their weight gradients.  They are
        # recomputed in the backward pass (two more norm kernels per layer) unless `save_norms`: then the forward
        # pass keeps them per layer (2 x T x D bf16 per layer).  None: keep them when the device has room to spare.
        if os.environ.get("FTB200_SAVE_NORMS", "") in ("0", "1"):
            save_norms = os.environ["FTB200_SAVE_NORMS"] == "1"
        if save_norms is None:
            save_norms = False
            if device.type == "cuda":
                need = 2 * L * T * D * 2
                free, _ = torch.cuda.mem_get_info(device)
                save_norms = free > need + (20 << 30)
        self.n1 = [torch.empty(T, D, **bf) for _ in range(L)] if save_norms else None
        self.n2 = [torch.empty(T, D, **bf) for _ in range(L)] if save_norms else None
        # Weight-gradient GEMMs on a stream of their own (`wgrad_stream`; FTB200_WGRAD_STREAM=0/1 overrides).  The
        # weight gradient and the data gradient of a layer are independent, and each of these persistent GEMMs ends
        # with a partial wave that leaves most SMs idle (384 tiles on 74 CTA pairs are 5.2 waves); with the two on
        # different streams the CTAs of one start on the SMs that the tail of the other has left.
        self.wstream = None
        env = os.environ.get("FTB200_WGRAD_STREAM", "")
        if device.type == "cuda" and (env == "1" or (env != "0" and wgrad_stream)):
            self.wstream = torch.cuda.Stream(device=device)
            self._w_events: Dict[Tuple[int, str], Tuple[torch.cuda.Event, torch.cuda.Event]] = {}
            self._w_last: Dict[str, torch.cuda.Event] = {}

    # -- helpers ---------------------------------------------------------------------------
    def _p(self, u: int) -> _Fields:
        return _Fields(self.param_unit(u), self.cfg.unit_fields(u))

    def _pf(self, u: int):
        if self.fwd_fields is not None:
            f = self.fwd_fields(u)
            if f is not None:
                return f
        return self._p(u)

    def _wgrad(self, layer: int, name: str, dy: torch.Tensor, x: torch.Tensor, out, reads: Tuple[str, ...]) -> None:
        """Weight gradient ``out = dy^T x`` of one matrix, on the weight-gradient stream when there is one.  ``reads``
        names the reusable workspaces among its operands: before the main stream overwrites one of them it waits for
        this GEMM (:meth:`_before_overwrite`)."""
        if self.wstream is None:
            K.linear_wgrad(dy, x, out=out)
            return
        evs = self._w_events.get((layer, name))
        if evs is None:
            evs = (torch.cuda.Event(), torch.cuda.Event())
            self._w_events[(layer, name)] = evs
        ready, done = evs
        ready.record()  # the operands are complete on the main stream here
        with torch.cuda.stream(self.wstream):
            self.wstream.wait_event(ready)
            K.linear_wgrad(dy, x, out=out)
            done.record(self.wstream)
        for r in reads:
            self._w_last[r] = done

    def _before_overwrite(self, *names: str) -> None:
        """The main stream is about to overwrite these workspaces: wait for the weight-gradient GEMMs that read them."""
        if self.wstream is None:
            return
        for n in names:
            ev = self._w_last.pop(n, None)
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)

    def _grad_done_after_wgrads(self, u: int) -> None:
        """``grad_done(u)`` once the unit's weight gradients are complete: with a weight-gradient stream the hook runs
        on that stream (after it has caught up with the main stream), so that whatever the hook orders after "the
        current stream" -- the reduce-scatter on the communication stream -- follows both."""
        if self.wstream is None:
            self.grad_done(u)
            return
        evs = self._w_events.get((u, "grad_done"))
        if evs is None:
            evs = (torch.cuda.Event(), torch.cuda.Event())
            self._w_events[(u, "grad_done")] = evs
        ready, done = evs
        ready.record()
        with torch.cuda.stream(self.wstream):
            self.wstream.wait_event(ready)
            self.grad_done(u)
            done.record(self.wstream)
        # the hook may read gradient destinations that the next unit reuses (a sharding layer's staging vectors for
        # the norm-weight gradients): the main stream waits for it before it writes the next norm-weight gradient
        self._w_last["grad_done"] = done

    def _g(self, u: int):
        """Gradient destinations of unit ``u``: views into its flat gradient buffer, or
        whatever ``grad_fields`` supplies (e.g. scatter targets of a GEMM-fused reduce-scatter)."""
        if self.grad_fields is not None:
            g = self.grad_fields(u)
            if g is not None:
                return g
        return _Fields(self.grad_unit(u), self.cfg.unit_fields(u))

    # -- forward ---------------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor], train: bool = True) -> torch.Tensor:
        """Runs the decoder; with ``targets`` returns the mean token loss and leaves
        ``dlogits``-derived gradients of the head computed (head backward is fused into
        the loss pass so that the logits never exist in full)."""
        c, T, B, S = self.cfg, self.T, self.B, self.S
        L = c.n_layers
        tok = tokens.reshape(-1)
        self.before_unit(0, False)
        K.embedding_fwd(tok, self._p(0).tok_embeddings, out=self.x[0])
        delta: Optional[torch.Tensor] = None
        for l in range(L):
            u = l + 1
            self.before_unit(u, False)
            W = self._pf(u)
            keep = train and self.n1 is not None
            n1 = self.n1[l] if keep else self.ws_n
            n2 = self.n2[l] if keep else self.ws_n
            # x[l] = stream (+ delta of the previous block); n1 = norm(x[l])
            if delta is None:
                K.rmsnorm_fwd(self.x[l], W.attn_norm, c.norm_eps, out=n1, rstd=self.rstd1[l])
            else:
                K.rmsnorm_fwd(self.h[l - 1], W.attn_norm, c.norm_eps, res=delta, h_out=self.x[l], out=n1,
                              rstd=self.rstd1[l])
            K.linear_fwd(n1, W.wqkv, out=self.qkv[l])
            K.rope_(self.qkv[l], self.rope, S, c.n_heads + c.n_kv_heads, c.head_dim)
            self.attn.forward(l, self.qkv[l], B, S, self.att[l], train)
            K.linear_fwd(self.att[l], W.wo, out=self.ws_proj)
            K.rmsnorm_fwd(self.x[l], W.ffn_norm, c.norm_eps, res=self.ws_proj, h_out=self.h[l], out=n2,
                          rstd=self.rstd2[l])
            s_buf = self.s[l] if train else self.ws_s
            K.linear_swiglu_fwd(n2, W.wgu, self.gu[l], s_buf)  # activation fused into the GEMM epilogue
            K.linear_fwd(s_buf, W.wd, out=self.ws_proj)
            delta = self.ws_proj
        u = L + 1
        self.before_unit(u, False)
        W = self._pf(u)
        if delta is None:
            K.rmsnorm_fwd(self.x[L], W.final_norm, c.norm_eps, out=self.ws_n, rstd=self.rstd1[L])
        else:
            K.rmsnorm_fwd(self.h[L - 1], W.final_norm, c.norm_eps, res=delta, h_out=self.x[L], out=self.ws_n,
                          rstd=self.rstd1[L])
        if targets is None:
            return K.linear_fwd(self.ws_n[-1:].contiguous(), W.lm_head)
        # head: logits -> loss -> dlogits -> (dW_head, d_norm) chunk by chunk
        tgt = targets.reshape(-1)
        G = self._g(u) if train else None
        rows = T // self.logit_chunks
        for ci in range(self.logit_chunks):
            sl = slice(ci * rows, (ci + 1) * rows)
            K.linear_fwd(self.ws_n[sl], W.lm_head, out=self.logits)
            K.cross_entropy_(self.logits, tgt[sl], self.grad_scale / T, loss=self.loss_rows[sl])
            if train:
                K.linear_wgrad(self.logits, self.ws_n[sl], out=G.lm_head, accumulate=ci > 0)
                K.linear_dgrad(self.logits, getattr(W.lm_head, "local", W.lm_head), out=self.ws_dn[sl])
        return self.loss_rows.mean()

    # -- backward --------------------------------------------------------------------------
    def backward(self, tokens: torch.Tensor) -> None:
        """Backward through the blocks and the embedding; expects :meth:`forward` with
        targets to have run (``ws_dn`` then holds the gradient of the final norm output)."""
        c, T, B, S = self.cfg, self.T, self.B, self.S
        L = c.n_layers
        u = L + 1
        W, G = self._p(u), self._g(u)
        K.rmsnorm_bwd(self.ws_dn, self.x[L], W.final_norm, self.rstd1[L], dres=None, dx=self.ws_dy, dw=G.final_norm)
        self.grad_done(u)
        dy = self.ws_dy
        for l in reversed(range(L)):
            u = l + 1
            self.before_unit(u, True)
            W, G = self._p(u), self._g(u)
            # ---- FFN
            self._wgrad(l, "wd", dy, self.s[l], G.wd, reads=("dy",))
            K.linear_dgrad(dy, W.wd, out=self.ws_ds)
            K.swiglu_bwd(self.ws_ds, self.gu[l], dgu=self.gu[l])
            if self.n2 is not None:
                self._wgrad(l, "wgu", self.gu[l], self.n2[l], G.wgu, reads=())
            else:
                self._before_overwrite("ws_n2")
                K.rmsnorm_fwd(self.h[l], W.ffn_norm, c.norm_eps, out=self.ws_n2, rstd=self.rstd2[l])
                self._wgrad(l, "wgu", self.gu[l], self.ws_n2, G.wgu, reads=("ws_n2",))
            K.linear_dgrad(self.gu[l], W.wgu, out=self.ws_dn)
            self._before_overwrite("ws_dh", "grad_done")
            K.rmsnorm_bwd(self.ws_dn, self.h[l], W.ffn_norm, self.rstd2[l], dres=dy, dx=self.ws_dh, dw=G.ffn_norm)
            # ---- attention
            self._wgrad(l, "wo", self.ws_dh, self.att[l], G.wo, reads=("ws_dh",))
            K.linear_dgrad(self.ws_dh, W.wo, out=self.ws_dn)
            self._before_overwrite("ws_dqkv")
            self.attn.backward(l, self.ws_dn, B, S, self.ws_dqkv)
            K.rope_(self.ws_dqkv, self.rope, S, c.n_heads + c.n_kv_heads, c.head_dim, backward=True)
            if self.n1 is not None:
                self._wgrad(l, "wqkv", self.ws_dqkv, self.n1[l], G.wqkv, reads=("ws_dqkv",))
            else:
                self._before_overwrite("ws_n")
                K.rmsnorm_fwd(self.x[l], W.attn_norm, c.norm_eps, out=self.ws_n, rstd=self.rstd1[l])
                self._wgrad(l, "wqkv", self.ws_dqkv, self.ws_n, G.wqkv, reads=("ws_dqkv", "ws_n"))
            K.linear_dgrad(self.ws_dqkv, W.wqkv, out=self.ws_dn)
            self._before_overwrite("dy")
            K.rmsnorm_bwd(self.ws_dn, self.x[l], W.attn_norm, self.rstd1[l], dres=self.ws_dh, dx=self.ws_dy,
                          dw=G.attn_norm)
            self._grad_done_after_wgrads(u)
            dy = self.ws_dy
        self.before_unit(0, True)
        G = self._g(0)
        G.tok_embeddings.zero_()
        K.embedding_bwd(tokens.reshape(-1), dy, G.tok_embeddings)
        self.grad_done(0)
        if self.wstream is not None:
            # the weight gradients are part of the backward pass: whoever runs after it on this stream sees them
            torch.cuda.current_stream().wait_stream(self.wstream)
            self._w_last.clear()


def init_unit_(cfg: LlamaConfig, unit: int, flat: torch.Tensor, seed: int) -> None:
    """Deterministic random init of one full unit (norm weights 1, matrices N(0, 0.02))."""
    g = torch.Generator(device=flat.device)
    g.manual_seed(seed * 1000 + unit)
    f = _Fields(flat, cfg.unit_fields(unit))
    for name, shape in cfg.unit_fields(unit):
        t = getattr(f, name)
        if len(shape) == 1:
            t.fill_(1.0)
        else:
            std = 0.02
            if name in ("wo", "wd"):
                std = 0.02 / math.sqrt(2 * cfg.n_layers)
            # generate in chunks to bound the fp32 temporary
            flat_t = t.view(-1)
            step = 1 << 26
            for s in range(0, flat_t.numel(), step):
                e = min(flat_t.numel(), s + step)
                flat_t[s:e] = (torch.randn(e - s, generator=g, device=flat.device, dtype=torch.float32) * std).to(flat.dtype)


class TorchLlama(torch.nn.Module):
    """Plain PyTorch (autograd) restatement of the same decoder: the numerical oracle
    of :class:`LlamaEngine` and a module users can wrap with the FT DDP wrapper."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        D, Fd = cfg.dim, cfg.ffn_dim
        self.tok_embeddings = torch.nn.Parameter(torch.empty(cfg.vocab_size, D))
        self.layers = torch.nn.ModuleList()
        for _ in range(cfg.n_layers):
            m = torch.nn.Module()
            for name, shape in cfg.layer_fields():
                setattr(m, name, torch.nn.Parameter(torch.empty(*shape)))
            self.layers.append(m)
        self.final_norm = torch.nn.Parameter(torch.empty(D))
        self.lm_head = torch.nn.Parameter(torch.empty(cfg.vocab_size, D))

    def load_units(self, unit_fn: Callable[[int], torch.Tensor]) -> None:
        cfg = self.cfg
        with torch.no_grad():
            self.tok_embeddings.copy_(_Fields(unit_fn(0), cfg.unit_fields(0)).tok_embeddings)
            for l, m in enumerate(self.layers):
                f = _Fields(unit_fn(l + 1), cfg.unit_fields(l + 1))
                for name, _ in cfg.layer_fields():
                    getattr(m, name).copy_(getattr(f, name))
            f = _Fields(unit_fn(cfg.n_layers + 1), cfg.unit_fields(cfg.n_layers + 1))
            self.final_norm.copy_(f.final_norm)
            self.lm_head.copy_(f.lm_head)

    def _norm(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.norm_eps) * w.float()).to(x.dtype)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        B, S = tokens.shape
        Hq, Hkv, Dh = c.n_heads, c.n_kv_heads, c.head_dim
        x = self.tok_embeddings[tokens]
        table = K.rope_table(S, Dh, c.rope_theta, x.device)
        cos, sin = table[..., 0][None, :, None, :], table[..., 1][None, :, None, :]

        def rot(t):
            t2 = t.float().reshape(*t.shape[:-1], Dh // 2, 2)
            a, b = t2[..., 0], t2[..., 1]
            return torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).reshape(t.shape).to(t.dtype)

        for m in self.layers:
            n1 = self._norm(x, m.attn_norm)
            qkv = n1 @ m.wqkv.t()
            q = rot(qkv[..., : Hq * Dh].reshape(B, S, Hq, Dh))
            k = rot(qkv[..., Hq * Dh : (Hq + Hkv) * Dh].reshape(B, S, Hkv, Dh))
            v = qkv[..., (Hq + Hkv) * Dh :].reshape(B, S, Hkv, Dh)
            rep = Hq // Hkv
            a = F.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(rep, 1), v.transpose(1, 2).repeat_interleave(rep, 1),
                is_causal=True,
            ).transpose(1, 2).reshape(B, S, Hq * Dh)
            x = x + a @ m.wo.t()
            n2 = self._norm(x, m.ffn_norm)
            gu = n2 @ m.wgu.t()
            x = x + (F.silu(gu[..., 0::2]) * gu[..., 1::2]) @ m.wd.t()
        return self._norm(x, self.final_norm) @ self.lm_head.t()
