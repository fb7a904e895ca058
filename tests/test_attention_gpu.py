"""Numerics of the tcgen05 attention kernels against an fp32 PyTorch restatement."""
import pytest
import torch

from torchft_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def _qkv(B, S, Hq, Hkv, D, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qkv = (torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda", generator=g) * scale).to(torch.bfloat16)
    q = qkv[:, : Hq * D]
    k = qkv[:, Hq * D : (Hq + Hkv) * D]
    v = qkv[:, (Hq + Hkv) * D :]
    return qkv, q, k, v


@pytest.mark.parametrize("B,S,Hq,Hkv,causal,scale", [
    (1, 128, 1, 1, True, 1.0),
    (1, 256, 2, 1, True, 1.0),
    (2, 512, 4, 2, True, 1.0),
    (1, 1024, 8, 2, True, 3.0),   # large scores: the running maximum moves and O is rescaled
    (1, 384, 2, 2, False, 1.0),
])
def test_attention_fwd_matches_reference(B, S, Hq, Hkv, causal, scale):
    D = 128
    _, q, k, v = _qkv(B, S, Hq, Hkv, D, seed=S, scale=scale)
    out = torch.empty(B * S, Hq * D, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    K.attention_fwd(q, k, v, B, S, Hq, Hkv, D, out, lse, causal=causal)
    K.check_status(out.device)
    q4, k4, v4 = (t.reshape(B, S, -1, D) for t in (q, k, v))
    ref = K.ref_attention(q4.float(), k4.float(), v4.float(), causal).reshape(B * S, Hq * D)
    ref_lse = K.ref_attention_lse(q4, k4, v4, causal)
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 1e-2, err
    assert (out.float() - ref).abs().max() < 0.05 * max(1.0, ref.abs().max().item())
    torch.testing.assert_close(lse, ref_lse, rtol=1e-3, atol=2e-3)


def _check_fwd(B, S, Hq, Hkv, D, causal, scale, seed):
    _, q, k, v = _qkv(B, S, Hq, Hkv, D, seed=seed, scale=scale)
    out = torch.empty(B * S, Hq * D, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    K.attention_fwd(q, k, v, B, S, Hq, Hkv, D, out, lse, causal=causal)
    K.check_status(out.device)
    q4, k4, v4 = (t.reshape(B, S, -1, D) for t in (q, k, v))
    ref = K.ref_attention(q4.float(), k4.float(), v4.float(), causal).reshape(B * S, Hq * D)
    ref_lse = K.ref_attention_lse(q4, k4, v4, causal)
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 1e-2, err
    assert (out.float() - ref).abs().max() < 0.05 * max(1.0, ref.abs().max().item())
    torch.testing.assert_close(lse, ref_lse, rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("poly", ["0", "2", "4"])
@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal,scale", [
    (1, 256, 1, 1, 128, True, 1.0),
    (2, 512, 4, 2, 128, True, 1.0),
    (1, 1024, 8, 2, 128, True, 3.0),    # the running maximum moves and O is rescaled
    (1, 512, 2, 2, 128, False, 1.0),
    (1, 256, 2, 1, 64, True, 1.0),      # head dim 64 (Llama-3.2-1B)
    (2, 1024, 8, 2, 64, True, 3.0),
    (1, 768, 4, 4, 64, False, 1.0),
])
def test_attention_fwd_pair_kernel(monkeypatch, poly, B, S, Hq, Hkv, D, causal, scale):
    """The two-tiles-per-CTA forward kernel, with none, a quarter and half of the exponentials on the FMA pipe."""
    monkeypatch.setenv("FTB200_ATTN_FWD", "pair")
    monkeypatch.setenv("FTB200_ATTN_POLY", poly)
    _check_fwd(B, S, Hq, Hkv, D, causal, scale, seed=S + D)


def test_attention_fwd_at_the_benchmark_shape():
    """Sequence 8192, 32 query heads on 8 KV heads, head dim 128: the shape of the Llama-3 8B step.  The fp32
    reference is evaluated on a slice of heads to bound its memory."""
    B, S, Hq, Hkv, D = 1, 8192, 32, 8, 128
    _, q, k, v = _qkv(B, S, Hq, Hkv, D, seed=5)
    out = torch.empty(B * S, Hq * D, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    K.attention_fwd(q, k, v, B, S, Hq, Hkv, D, out, lse, causal=True)
    K.check_status(out.device)
    for kvh in (0, 7):
        qs = q.reshape(B, S, Hq, D)[:, :, kvh * 4 : kvh * 4 + 2]
        ks = k.reshape(B, S, Hkv, D)[:, :, kvh : kvh + 1]
        vs = v.reshape(B, S, Hkv, D)[:, :, kvh : kvh + 1]
        ref = K.ref_attention(qs.float(), ks.float(), vs.float(), True)
        got = out.reshape(B, S, Hq, D)[:, :, kvh * 4 : kvh * 4 + 2].float()
        err = (got - ref).norm() / ref.norm()
        assert err < 1e-2, err
        ref_lse = K.ref_attention_lse(qs, ks, vs, True)
        torch.testing.assert_close(lse[:, kvh * 4 : kvh * 4 + 2], ref_lse, rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("B,S,Hq,Hkv,causal,D", [
    (1, 128, 1, 1, True, 128),
    (1, 256, 2, 1, True, 128),
    (2, 512, 4, 2, True, 128),
    (1, 384, 2, 2, False, 128),
    (1, 256, 1, 1, True, 64),       # head dim 64 (Llama-3.2-1B): the forward needs seq % 256 == 0
    (2, 512, 8, 2, True, 64),
    (1, 2048, 8, 2, True, 64),
    (1, 768, 4, 4, False, 64),
])
def test_attention_bwd_matches_reference(B, S, Hq, Hkv, causal, D):
    qkv, q, k, v = _qkv(B, S, Hq, Hkv, D, seed=7 + S)
    out = torch.empty(B * S, Hq * D, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    K.attention_fwd(q, k, v, B, S, Hq, Hkv, D, out, lse, causal=causal)
    g = torch.Generator(device="cuda").manual_seed(99)
    d_o = torch.randn(B * S, Hq * D, device="cuda", generator=g).to(torch.bfloat16)
    dqkv = torch.full_like(qkv, float("nan"))
    dq, dk, dv = dqkv[:, : Hq * D], dqkv[:, Hq * D : (Hq + Hkv) * D], dqkv[:, (Hq + Hkv) * D :]
    K.attention_bwd(q, k, v, out, d_o, lse, dq, dk, dv, B, S, Hq, Hkv, D, causal=causal)
    K.check_status(out.device)
    q4, k4, v4, do4 = (t.reshape(B, S, -1, D) for t in (q, k, v, d_o))
    rq, rk, rv = K.ref_attention_bwd(q4, k4, v4, do4, causal)
    for name, got, want in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        want = want.reshape(B * S, -1)
        err = (got.float() - want).norm() / want.norm()
        assert err < 2e-2, (name, err)
