"""Every kernel family once, with guard zones around everything it writes (tests/canary.py)."""

import pytest
import torch

from canary import Canaries
from torchft_b200 import quantization as Q
from torchft_b200.ops import diloco, kernels as K

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def test_kernel_outputs_stay_inside_their_tensors():
    torch.manual_seed(0)
    c = Canaries(DEV)
    # GEMMs: ragged M/N (partial tiles), all three layouts, fused SwiGLU epilogue
    M, N, Kd = 200, 328, 192
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = torch.randn(N, Kd, device=DEV).bfloat16()
    dy = torch.randn(M, N, device=DEV).bfloat16()
    K.linear_fwd(x, w, out=c.empty((M, N), torch.bfloat16, "fwd"))
    K.linear_dgrad(dy, w, out=c.empty((M, Kd), torch.bfloat16, "dgrad"))
    K.linear_wgrad(dy, x, out=c.empty((N, Kd), torch.bfloat16, "wgrad"))
    Fd = 176
    wgu = (torch.randn(2 * Fd, Kd, device=DEV) * 0.1).bfloat16()
    K.linear_swiglu_fwd(x, wgu, c.empty((M, 2 * Fd), torch.bfloat16, "gu"), c.empty((M, Fd), torch.bfloat16, "s"))
    # attention forward and backward on packed QKV
    B, S, Hq, Hkv, D = 1, 256, 2, 1, 128
    qkv = c.like((torch.randn(B * S, (Hq + 2 * Hkv) * D, device=DEV) * 0.5).bfloat16(), "qkv")
    q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D : (Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D :]
    out = c.empty((B * S, Hq * D), torch.bfloat16, "attn_out")
    lse = c.empty((B, Hq, S), torch.float32, "lse")
    K.attention_fwd(q, k, v, B, S, Hq, Hkv, D, out, lse)
    dqkv = c.empty(tuple(qkv.shape), torch.bfloat16, "dqkv")
    K.attention_bwd(q, k, v, out, torch.randn_like(out), lse, dqkv[:, : Hq * D], dqkv[:, Hq * D : (Hq + Hkv) * D],
                    dqkv[:, (Hq + Hkv) * D :], B, S, Hq, Hkv, D)
    # normalisation, RoPE, SwiGLU backward, cross-entropy, embedding
    T, Dm = 96, 520
    xr = torch.randn(T, Dm, device=DEV).bfloat16()
    wn = torch.ones(Dm, device=DEV).bfloat16()
    rstd = c.empty((T,), torch.float32, "rstd")
    K.rmsnorm_fwd(xr, wn, 1e-5, res=xr, h_out=c.empty((T, Dm), torch.bfloat16, "h"), out=c.empty((T, Dm), torch.bfloat16, "n"),
                  rstd=rstd)
    K.rmsnorm_bwd(xr, xr, wn, rstd, dres=xr, dx=c.empty((T, Dm), torch.bfloat16, "dx"), dw=c.empty((Dm,), torch.bfloat16, "dw"))
    rope_buf = c.like(torch.randn(64, 3 * 64, device=DEV).bfloat16(), "rope")
    K.rope_(rope_buf, K.rope_table(32, 64, 10000.0, DEV), 32, 2, 64)  # only two of three heads are rotated
    gu = c.like(torch.randn(T, 2 * 88, device=DEV).bfloat16(), "gu_bwd")
    K.swiglu_bwd(torch.randn(T, 88, device=DEV).bfloat16(), gu, dgu=gu)
    logits = c.like(torch.randn(T, 1000, device=DEV).bfloat16(), "logits")
    K.cross_entropy_(logits, torch.randint(0, 1000, (T,), device=DEV), 1.0 / T, c.empty((T,), torch.float32, "loss"))
    table = torch.randn(50, 64, device=DEV).bfloat16()
    tok = torch.randint(0, 50, (T,), device=DEV)
    K.embedding_fwd(tok, table, out=c.empty((T, 64), torch.bfloat16, "emb"))
    K.embedding_bwd(tok, torch.randn(T, 64, device=DEV).bfloat16(), c.like(torch.zeros(50, 64, device=DEV).bfloat16(), "dtable"))
    # optimizer state, norms, fp8 quantisation, DiLoCo outer step
    n = 12345 * 4
    master, m, vv = (c.like(torch.randn(n, device=DEV), nm) for nm in ("master", "m", "v"))
    vv.abs_()
    K.adamw_(master, m, vv, torch.randn(n, device=DEV).bfloat16(), c.empty((n,), torch.bfloat16, "p_bf16"), 1e-3, 0.9, 0.95,
             1e-8, 0.1, 3)
    K.sumsq_(master, c.like(torch.zeros(1, device=DEV), "sumsq"))
    nq = 128 * 37
    qbuf = c.empty((Q.quantized_nbytes(nq),), torch.uint8, "quantised")
    Q.quantize_into(torch.randn(nq, device=DEV), qbuf)
    Q.dequantize_from(qbuf, c.empty((nq,), torch.float32, "dequantised"))
    g, mom, backup, param = (c.like(torch.randn(nq, device=DEV), nm) for nm in ("g", "mom", "backup", "param"))
    diloco.outer_step_(g, mom, backup, param, lr=0.7, momentum_coef=0.9, alpha=0.25, nesterov=True)
    K.check_status(DEV)
    c.check()
