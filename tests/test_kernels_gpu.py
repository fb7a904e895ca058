"""Numerics of every sm_100a kernel against an fp32 PyTorch reference of the same op."""
import math

import pytest
import torch

from torchft_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("impl", ["1cta", "2cta"])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K_", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (200, 328, 136), (1024, 1024, 4096)])
def test_gemm_layouts(a_mn, b_mn, M, N, K_, impl):
    torch.manual_seed(1)
    a = torch.randn((K_, M) if a_mn else (M, K_), device=DEV).bfloat16()
    b = torch.randn((K_, N) if b_mn else (N, K_), device=DEV).bfloat16()
    out = K.gemm(a, b, a_mn, b_mn, impl=impl)
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    ref = af @ bf
    K.check_status(out.device)
    assert rel_err(out, ref) < 1e-2
    # fp32 output + accumulate
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    K.gemm(a, b, a_mn, b_mn, out=acc, accumulate=True, impl=impl)
    assert rel_err(acc, ref + 1.0) < 1e-2


@pytest.mark.parametrize("impl", ["1cta", "2cta"])
def test_gemm_many_tiles_persistent(impl):
    torch.manual_seed(2)
    M, N, K_ = 2048, 4096, 512
    a = torch.randn(M, K_, device=DEV).bfloat16()
    b = torch.randn(N, K_, device=DEV).bfloat16()
    ref = a.float() @ b.float().t()
    for ctas in (0, 7, 1):
        out = K.gemm(a, b, max_ctas=ctas, impl=impl)
        assert rel_err(out, ref) < 1e-2
    K.check_status(a.device)


def test_linear_trio_matches_autograd():
    torch.manual_seed(3)
    T, Kd, Nd = 512, 384, 640
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    w = (torch.randn(Nd, Kd, device=DEV) * 0.05).bfloat16()
    dy = torch.randn(T, Nd, device=DEV).bfloat16()
    assert rel_err(K.linear_fwd(x, w), x.float() @ w.float().t()) < 1e-2
    assert rel_err(K.linear_dgrad(dy, w), dy.float() @ w.float()) < 1e-2
    assert rel_err(K.linear_wgrad(dy, x), dy.float().t() @ x.float()) < 1e-2


@pytest.mark.parametrize("T,D", [(64, 256), (33, 4096), (7, 1024), (701, 4096), (613, 8192)])
def test_rmsnorm(T, D):
    torch.manual_seed(4)
    x = torch.randn(T, D, device=DEV).bfloat16()
    res = torch.randn(T, D, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    out, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
    ro, rr, _ = K.ref_rmsnorm_fwd(x, w, 1e-5)
    assert rel_err(out, ro) < 1e-2 and rel_err(rstd, rr) < 1e-4
    out2, rstd2, h = K.rmsnorm_fwd(x, w, 1e-5, res=res)
    ro2, rr2, rh = K.ref_rmsnorm_fwd(x, w, 1e-5, res)
    assert rel_err(out2, ro2) < 1e-2 and rel_err(h, rh) < 1e-2
    dy = torch.randn(T, D, device=DEV).bfloat16()
    dres = torch.randn(T, D, device=DEV).bfloat16()
    dx, dw = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
    rdx, rdw = K.ref_rmsnorm_bwd(dy, x, w, rr, dres)
    assert rel_err(dx, rdx) < 1e-2
    assert rel_err(dw, rdw) < 2e-2


def test_rope_roundtrip_and_ref():
    torch.manual_seed(5)
    S, Hq, Hkv, Dh = 64, 4, 2, 64
    T = 2 * S
    buf = torch.randn(T, (Hq + 2 * Hkv) * Dh, device=DEV).bfloat16()
    orig = buf.clone()
    table = K.rope_table(S, Dh, 500000.0, DEV)
    ref = K.ref_rope(orig, table, S, Hq + Hkv, Dh)
    K.rope_(buf, table, S, Hq + Hkv, Dh)
    assert rel_err(buf, ref) < 1e-2
    assert torch.equal(buf[:, (Hq + Hkv) * Dh:], orig[:, (Hq + Hkv) * Dh:])
    K.rope_(buf, table, S, Hq + Hkv, Dh, backward=True)
    assert rel_err(buf, orig) < 2e-2


def test_swiglu():
    torch.manual_seed(6)
    T, Fd = 96, 512
    gu = torch.randn(T, 2 * Fd, device=DEV).bfloat16()
    ds = torch.randn(T, Fd, device=DEV).bfloat16()
    assert rel_err(K.swiglu_fwd(gu), K.ref_swiglu_fwd(gu)) < 1e-2
    ref = K.ref_swiglu_bwd(ds, gu)
    got = K.swiglu_bwd(ds, gu.clone())
    assert rel_err(got, ref) < 1e-2
    inplace = gu.clone()
    K.swiglu_bwd(ds, inplace, dgu=inplace)
    assert rel_err(inplace, ref) < 1e-2


@pytest.mark.parametrize("T,V", [(16, 1024), (5, 128256), (64, 8192)])
def test_cross_entropy(T, V):
    torch.manual_seed(7)
    logits = (torch.randn(T, V, device=DEV) * 3).bfloat16()
    tgt = torch.randint(0, V, (T,), device=DEV)
    rl, rg = K.ref_cross_entropy(logits, tgt, 1.0 / T)
    loss = K.cross_entropy_(logits, tgt, 1.0 / T)
    assert rel_err(loss, rl) < 1e-3
    assert rel_err(logits, rg) < 1e-2


@pytest.mark.parametrize("gdt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8, 1000, 1 << 20, (1 << 20) + 3])
def test_adamw(gdt, n):
    torch.manual_seed(8)
    master = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    lp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    rm, rmm, rv = master.clone(), m.clone(), v.clone()
    scale = torch.tensor([0.5], device=DEV)
    for step in (1, 2, 3):
        g = torch.randn(n, device=DEV).to(gdt)
        K.adamw_(master, m, v, g, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, scale)
        K.ref_adamw(rm, rmm, rv, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5)
    assert rel_err(master, rm) < 1e-5
    assert rel_err(m, rmm) < 1e-5 and rel_err(v, rv) < 1e-5
    assert torch.equal(lp, master.bfloat16())


def test_sumsq_and_clip():
    torch.manual_seed(9)
    x = torch.randn((1 << 18) + 5, device=DEV).bfloat16()
    out = torch.zeros(1, device=DEV)
    K.sumsq_(x, out)
    ref = x.float().pow(2).sum()
    assert abs(out.item() - ref.item()) / ref.item() < 1e-4
    coef = torch.zeros(1, device=DEV)
    nrm = torch.zeros(1, device=DEV)
    K.clip_coef_(out, 1.0, coef, nrm)
    assert abs(nrm.item() - math.sqrt(ref.item())) / nrm.item() < 1e-4
    assert abs(coef.item() - 1.0 / (nrm.item() + 1e-6)) < 1e-6


def test_embedding():
    torch.manual_seed(10)
    V, D, T = 512, 256, 300
    table = torch.randn(V, D, device=DEV).bfloat16()
    tok = torch.randint(0, V, (T,), device=DEV)
    assert torch.equal(K.embedding_fwd(tok, table), table[tok])
    dout = torch.randn(T, D, device=DEV).bfloat16()
    dtab = torch.zeros(V, D, device=DEV, dtype=torch.bfloat16)
    K.embedding_bwd(tok, dout, dtab)
    ref = torch.zeros(V, D, device=DEV).index_add_(0, tok, dout.float())
    assert rel_err(dtab, ref) < 2e-2


@pytest.mark.parametrize("variant", ["library", "head_dim_128", "head_dim_64"])
def test_engine_matches_autograd_gpu(variant):
    from torchft_b200.models.llama import LLAMA_TINY, LlamaConfig, SdpaAttention, Tcgen05Attention, TorchLlama, _Fields
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer

    torch.manual_seed(0)
    # the tcgen05 attention kernels take head dim 128, and head dim 64 (LLAMA_TINY) when the sequence is a multiple
    # of 256; LLAMA_TINY at sequence 128 falls back to the library
    cfg = (LlamaConfig(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=1024, name="llama-hd128")
           if variant == "head_dim_128" else LLAMA_TINY)
    B, S = 2, (256 if variant == "head_dim_64" else 128)
    native_attention = variant != "library"
    dev = torch.device("cuda")
    tr = ShardedLlamaTrainer(cfg, B, S, dev, logit_chunks=2)
    assert isinstance(tr.engine.attn, Tcgen05Attention if native_attention else SdpaAttention)
    tokens = torch.randint(0, cfg.vocab_size, (B, S), device=dev)
    targets = torch.randint(0, cfg.vocab_size, (B, S), device=dev)
    loss = tr.forward_backward(tokens, targets)
    ref = TorchLlama(cfg).to(dev, torch.float32)
    ref.load_units(lambda u: tr._param_unit(u))
    rl = torch.nn.functional.cross_entropy(ref(tokens).float().view(-1, cfg.vocab_size), targets.view(-1))
    rl.backward()
    K.check_status(dev)
    assert abs(loss.item() - rl.item()) < 3e-2
    g = _Fields(tr._grad_unit(1), cfg.unit_fields(1))
    for name in ("wqkv", "wo", "wgu", "wd", "attn_norm", "ffn_norm"):
        assert rel_err(getattr(g, name), getattr(ref.layers[0], name).grad) < 0.03, name
    l0 = loss.item()
    for _ in range(3):
        tr.optimizer_step()
        l1 = tr.forward_backward(tokens, targets).item()
    assert l1 < l0


def test_engine_matches_autograd_at_the_8b_layer_shape():
    """One decoder layer with the shapes the benchmark runs (dim 4096, ffn 14336, 32 query heads on 8 KV heads,
    sequence 8192: reductions of depth 4096, 8192 and 14336, attention over 64 key blocks) against fp32 autograd.
    The vocabulary is cut to 8192 to bound the oracle's memory."""
    from torchft_b200.models.llama import LlamaConfig, Tcgen05Attention, TorchLlama, _Fields
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer

    torch.manual_seed(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    cfg = LlamaConfig(dim=4096, n_layers=1, n_heads=32, n_kv_heads=8, ffn_dim=14336, vocab_size=8192, name="llama-8b-layer")
    B, S = 1, 8192
    dev = torch.device("cuda")
    tr = ShardedLlamaTrainer(cfg, B, S, dev, logit_chunks=1)
    assert isinstance(tr.engine.attn, Tcgen05Attention)
    tokens = torch.randint(0, cfg.vocab_size, (B, S), device=dev)
    targets = torch.randint(0, cfg.vocab_size, (B, S), device=dev)
    loss = tr.forward_backward(tokens, targets)
    K.check_status(dev)
    ref = TorchLlama(cfg).to(dev, torch.float32)
    ref.load_units(lambda u: tr._param_unit(u))
    rl = torch.nn.functional.cross_entropy(ref(tokens).float().view(-1, cfg.vocab_size), targets.view(-1))
    rl.backward()
    assert abs(loss.item() - rl.item()) < 2e-2, (loss.item(), rl.item())
    g = _Fields(tr._grad_unit(1), cfg.unit_fields(1))
    errs = {name: rel_err(getattr(g, name), getattr(ref.layers[0], name).grad)
            for name in ("wqkv", "wo", "wgu", "wd", "attn_norm", "ffn_norm")}
    print("gradient errors at the 8B layer shape:", {k: round(v, 5) for k, v in errs.items()})
    for name, e in errs.items():
        assert e < 0.02, (name, errs)


def test_linear_swiglu_fused_epilogue():
    torch.manual_seed(11)
    T, Kd, Fd = 384, 256, 352  # 2F = 704 = 22 * 32
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    w = (torch.randn(2 * Fd, Kd, device=DEV) * 0.1).bfloat16()
    gu = torch.empty(T, 2 * Fd, device=DEV, dtype=torch.bfloat16)
    s = torch.empty(T, Fd, device=DEV, dtype=torch.bfloat16)
    K.linear_swiglu_fwd(x, w, gu, s)
    K.check_status(x.device)
    ref_gu = x.float() @ w.float().t()
    assert rel_err(gu, ref_gu) < 1e-2
    assert rel_err(s, K.ref_swiglu_fwd(gu)) < 1e-2
    assert rel_err(s, torch.nn.functional.silu(ref_gu[:, 0::2]) * ref_gu[:, 1::2]) < 2e-2


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("M,N,K_,swiglu", [(256, 256, 64, False), (1024, 1536, 512, False), (2048, 2048, 1024, True),
                                           (200, 640, 192, False)])
def test_gemm_with_fused_all_gather(world, M, N, K_, swiglu):
    """The weight lies spread over `world` shard buffers (here all on this GPU: the kernel only sees pointers) at an
    offset that makes it straddle shard boundaries; the GEMM gathers it into the local unit while it multiplies."""
    import ctypes

    torch.manual_seed(7)
    unit_off = 8 * 331  # some field in front of the weight
    numel = unit_off + N * K_ + 8 * 57
    shard = -(-numel // (world * 8)) * 8
    shard = max(shard, 8192)
    unit = torch.zeros(shard * world, device=DEV, dtype=torch.bfloat16)
    unit[:numel] = (torch.randn(numel, device=DEV) * 0.5).bfloat16()
    shards = [unit[r * shard:(r + 1) * shard].clone() for r in range(world)]
    peers = (ctypes.c_void_p * 8)()
    for r in range(world):
        peers[r] = shards[r].data_ptr()
    full = torch.full((shard * world,), 7.0, device=DEV, dtype=torch.bfloat16)  # stale content must be overwritten
    w_true = unit[unit_off:unit_off + N * K_].view(N, K_)
    sync = torch.full((1 + N // 128,), 12345, device=DEV, dtype=torch.int32)  # the launcher zeroes it
    field = K.GatherField(full[unit_off:unit_off + N * K_].view(N, K_), peers, world, shard, unit_off, sync)
    assert K.GatherField.supported((N, K_), shard)
    x = torch.randn(M, K_, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    if swiglu:
        s_out = torch.empty(M, N // 2, device=DEV, dtype=torch.bfloat16)
        K.linear_swiglu_fwd(x, field, out, s_out)
    else:
        K.linear_fwd(x, field, out=out)
    torch.cuda.synchronize()
    K.check_status(out.device)
    assert not field.pending
    assert torch.equal(field.local, w_true)
    assert torch.all(full[:unit_off] == 7.0) and torch.all(full[unit_off + N * K_:] == 7.0)  # nothing outside the field
    ref = x.float() @ w_true.float().t()
    assert rel_err(out, ref) < 1e-2
    if swiglu:
        g, u = out.float()[:, 0::2], out.float()[:, 1::2]
        assert rel_err(s_out, torch.nn.functional.silu(g) * u) < 1e-2
    # second use: an ordinary GEMM on the gathered weight
    out2 = K.linear_fwd(x, field)
    assert torch.equal(out2, out)
