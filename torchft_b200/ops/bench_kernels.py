"""Micro-benchmarks of the sm_100a kernels (CUDA-event timing, warm-up, L2-exceeding inputs).

    python -m torchft_b200.ops.bench_kernels gemm --m 8192 --n 8192 --k 8192 --layout fwd
    python -m torchft_b200.ops.bench_kernels adamw --n 1073741824
    python -m torchft_b200.ops.bench_kernels all

Each line printed is JSON: achieved TFLOP/s or GB/s and the fraction of the measured
peaks in ``MEASURED_PEAKS.json`` (cuBLAS bf16 burst and STREAM-style copy) when that
file is present next to the package.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Callable

import torch

from . import kernels as K


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn: Callable[[], None], iters: int = 10, warmup: int = 3) -> float:
    """Milliseconds per call (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_gemm(m: int, n: int, k: int, layout: str, iters: int, compare: bool) -> dict:
    dev = "cuda"
    x = torch.randn(m, k, device=dev).bfloat16()
    w = torch.randn(n, k, device=dev).bfloat16()
    dy = torch.randn(m, n, device=dev).bfloat16()
    fns = {
        "fwd": (lambda: K.linear_fwd(x, w), lambda: torch.matmul(x, w.t())),
        "dgrad": (lambda: K.linear_dgrad(dy, w), lambda: torch.matmul(dy, w)),
        "wgrad": (lambda: K.linear_wgrad(dy, x), lambda: torch.matmul(dy.t(), x)),
    }
    ours, lib = fns[layout]
    ms = timeit(ours, iters)
    K.check_status(x.device)
    hbm, tf, how = _peaks()
    fl = 2.0 * m * n * k
    out = {"kernel": "gemm_bf16_tcgen05", "layout": layout, "m": m, "n": n, "k": k, "ms": ms,
           "tflops": fl / ms / 1e9, f"frac_of_{how}_cublas_peak": fl / ms / 1e9 / tf}
    if compare:
        out["cublas_tflops"] = fl / timeit(lib, iters) / 1e9
    return out


def bench_gemm_gather(m: int, n: int, k: int, world: int, iters: int) -> dict:
    """Forward GEMM with the all-gather of its weight fused in, against the same GEMM on a weight that is already
    gathered and against copy-then-GEMM.  On one GPU the `world` shard buffers are local memory: the figure is
    what the gather warps and the tile waits cost the GEMM, not the NVLink transfer."""
    import ctypes

    dev = "cuda"
    x = torch.randn(m, k, device=dev).bfloat16()
    numel = n * k
    shard = -(-numel // (world * 8)) * 8
    shards = [torch.randn(shard, device=dev).bfloat16() for _ in range(world)]
    peers = (ctypes.c_void_p * 8)()
    for r in range(world):
        peers[r] = shards[r].data_ptr()
    full = torch.zeros(shard * world, device=dev, dtype=torch.bfloat16)
    sync = torch.zeros(1 + n // 128, device=dev, dtype=torch.int32)
    field = K.GatherField(full[:numel].view(n, k), peers, world, shard, 0, sync)
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)

    def fused():
        field.pending = True
        K.linear_fwd(x, field, out=out)

    def separate():
        for r in range(world):
            full[r * shard:(r + 1) * shard].copy_(shards[r])
        K.linear_fwd(x, field.local, out=out)

    ms_fused = timeit(fused, iters)
    ref = out.clone()
    ms_plain = timeit(lambda: K.linear_fwd(x, field.local, out=out), iters)
    ms_sep = timeit(separate, iters)
    K.check_status(x.device)
    fl = 2.0 * m * n * k
    return {"kernel": "gemm_bf16_gather", "m": m, "n": n, "k": k, "world": world, "fused_ms": ms_fused,
            "plain_gemm_ms": ms_plain, "copy_then_gemm_ms": ms_sep, "fused_tflops": fl / ms_fused / 1e9,
            "plain_tflops": fl / ms_plain / 1e9, "bit_equal_to_plain": bool(torch.equal(ref, out))}


def bench_adamw(n: int, iters: int) -> dict:
    dev = "cuda"
    master, m, v = (torch.zeros(n, device=dev) for _ in range(3))
    g = torch.randn(n, device=dev, dtype=torch.bfloat16)
    lp = torch.empty(n, device=dev, dtype=torch.bfloat16)
    ms = timeit(lambda: K.adamw_(master, m, v, g, lp, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1), iters)
    hbm, _, how = _peaks()
    gbs = n * 28 / ms / 1e6
    return {"kernel": "adamw", "n": n, "ms": ms, "gbs": gbs, f"frac_of_{how}_copy_bw": gbs / hbm}


def bench_rmsnorm(t: int, d: int, iters: int) -> dict:
    dev = "cuda"
    x = torch.randn(t, d, device=dev).bfloat16()
    r = torch.randn(t, d, device=dev).bfloat16()
    w = torch.ones(d, device=dev).bfloat16()
    h = torch.empty_like(x)
    o = torch.empty_like(x)
    rs = torch.empty(t, device=dev)
    ms = timeit(lambda: K.rmsnorm_fwd(x, w, 1e-5, res=r, h_out=h, out=o, rstd=rs), iters)
    hbm, _, how = _peaks()
    gbs = t * d * 2 * 4 / ms / 1e6
    return {"kernel": "rmsnorm_fwd(add+norm)", "t": t, "d": d, "ms": ms, "gbs": gbs, f"frac_of_{how}_copy_bw": gbs / hbm}


def bench_elementwise(iters: int) -> list:
    """The memory-bound kernels of one Llama-3 8B layer / head at seq 8192: each is timed on tensors of the real
    shape, several of them cycled so that consecutive launches do not hit L2, and reported as algorithmic bytes
    over the measured copy bandwidth."""
    dev = "cuda"
    hbm, _, how = _peaks()
    T, D, Fd, V, QKV, H = 8192, 4096, 14336, 128256, 6144, 40
    out = []

    def row(name, nbytes, ms):
        gbs = nbytes / ms / 1e6
        out.append({"kernel": name, "ms": ms, "gbs": gbs, f"frac_of_{how}_copy_bw": gbs / hbm})

    def cycle(make, n=4):
        bufs = [make() for _ in range(n)]
        state = {"i": 0}

        def nxt():
            state["i"] = (state["i"] + 1) % n
            return bufs[state["i"]]

        return nxt

    # RMSNorm backward (dx and dw): reads dy, x, dres, writes dx
    xs = cycle(lambda: torch.randn(T, D, device=dev).bfloat16())
    w = torch.ones(D, device=dev).bfloat16()
    rstd = torch.rand(T, device=dev) + 0.5
    dx, dw = torch.empty(T, D, device=dev, dtype=torch.bfloat16), torch.zeros(D, device=dev, dtype=torch.bfloat16)
    row("rmsnorm_bwd", T * D * 2 * 4, timeit(lambda: K.rmsnorm_bwd(xs(), xs(), w, rstd, dres=xs(), dx=dx, dw=dw), iters))
    # RoPE in place on the packed QKV activation (Q and K heads)
    qkvs = cycle(lambda: torch.randn(T, QKV, device=dev).bfloat16(), 6)
    table = K.rope_table(T, 128, 500000.0, torch.device(dev))
    row("rope", T * H * 128 * 2 * 2, timeit(lambda: K.rope_(qkvs(), table, T, H, 128), iters))
    # SwiGLU backward in place on the gate/up activation: reads ds, gu, writes dgu
    gus = cycle(lambda: torch.randn(T, 2 * Fd, device=dev).bfloat16(), 3)
    dss = cycle(lambda: torch.randn(T, Fd, device=dev).bfloat16(), 3)

    def swiglu():
        g = gus()
        K.swiglu_bwd(dss(), g, dgu=g)

    row("swiglu_bwd", T * Fd * 2 * 5, timeit(swiglu, iters))
    # cross-entropy with in-place gradient over the full vocabulary: reads and writes the logits once
    logits = torch.randn(T, V, device=dev).bfloat16()
    tgt = torch.randint(0, V, (T,), device=dev)
    loss = torch.empty(T, device=dev)
    row("cross_entropy", T * V * 2 * 2, timeit(lambda: K.cross_entropy_(logits, tgt, 1.0 / T, loss), max(2, iters // 2), warmup=1))
    del logits
    # embedding gather
    table_e = torch.randn(V, D, device=dev).bfloat16()
    eo = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
    row("embedding_fwd", T * D * 2 * 2, timeit(lambda: K.embedding_fwd(tgt, table_e, out=eo), iters))
    # sum of squares (gradient norm) over a 218 M-element layer gradient
    gsq = cycle(lambda: torch.randn(218112000, device=dev).bfloat16(), 2)
    acc = torch.zeros(1, device=dev)
    row("sumsq", 218112000 * 2, timeit(lambda: K.sumsq_(gsq(), acc), iters))
    return out


def bench_attention(batch: int, seq: int, hq: int, hkv: int, iters: int, compare: bool, head_dim: int = 128) -> dict:
    """Causal GQA attention, head dim 128 or 64, forward and backward; FLOPs count the causal half."""
    import torch.nn.functional as F

    dev, D = "cuda", head_dim
    qkv = (torch.randn(batch * seq, (hq + 2 * hkv) * D, device=dev) * 0.5).bfloat16()
    q, k, v = qkv[:, : hq * D], qkv[:, hq * D : (hq + hkv) * D], qkv[:, (hq + hkv) * D :]
    out = torch.empty(batch * seq, hq * D, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(batch, hq, seq, device=dev)
    d_o = torch.randn_like(out)
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = dqkv[:, : hq * D], dqkv[:, hq * D : (hq + hkv) * D], dqkv[:, (hq + hkv) * D :]
    fwd = timeit(lambda: K.attention_fwd(q, k, v, batch, seq, hq, hkv, D, out, lse), iters)
    variants = {}
    if seq % 256 == 0 and D == 128:
        # the forward kernels side by side: one tile per CTA, and two tiles per CTA with none, a quarter
        # and half of the exponentials on the FMA pipe
        saved = {n: os.environ.get(n) for n in ("FTB200_ATTN_FWD", "FTB200_ATTN_POLY")}
        for name, impl, poly in (("single", "single", "0"), ("pair_poly0", "pair", "0"), ("pair_poly2", "pair", "2"),
                                 ("pair_poly4", "pair", "4")):
            os.environ["FTB200_ATTN_FWD"], os.environ["FTB200_ATTN_POLY"] = impl, poly
            variants[name + "_ms"] = timeit(lambda: K.attention_fwd(q, k, v, batch, seq, hq, hkv, D, out, lse), iters)
        for n, val in saved.items():
            if val is None:
                os.environ.pop(n, None)
            else:
                os.environ[n] = val
    bwd = timeit(lambda: K.attention_bwd(q, k, v, out, d_o, lse, dq, dk, dv, batch, seq, hq, hkv, D), iters)
    K.check_status(qkv.device)
    _, tf, how = _peaks()
    fl_fwd = 4.0 * batch * hq * seq * seq * D / 2
    fl_bwd = 2.5 * fl_fwd
    res = {"kernel": "attention_tcgen05", "batch": batch, "seq": seq, "heads": hq, "kv_heads": hkv, "head_dim": D, "fwd_ms": fwd,
           "bwd_ms": bwd, "fwd_tflops": fl_fwd / fwd / 1e9, "bwd_tflops": fl_bwd / bwd / 1e9,
           f"fwd_frac_of_{how}_cublas_peak": fl_fwd / fwd / 1e9 / tf, f"bwd_frac_of_{how}_cublas_peak": fl_bwd / bwd / 1e9 / tf}
    res["fwd_variants"] = variants
    if compare:
        q4 = q.reshape(batch, seq, hq, D).transpose(1, 2).detach().requires_grad_(True)
        k4 = k.reshape(batch, seq, hkv, D).transpose(1, 2).detach().requires_grad_(True)
        v4 = v.reshape(batch, seq, hkv, D).transpose(1, 2).detach().requires_grad_(True)
        do4 = d_o.reshape(batch, seq, hq, D).transpose(1, 2)

        def lib_fwd():
            with torch.no_grad():
                F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True)

        o4 = F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True)
        res["sdpa_fwd_ms"] = timeit(lib_fwd, iters)
        res["sdpa_bwd_ms"] = timeit(lambda: torch.autograd.grad(o4, (q4, k4, v4), do4, retain_graph=True), iters)
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_gather", "adamw", "rmsnorm", "attention", "elementwise", "all"])
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-compare", action="store_true")
    a = ap.parse_args()
    if a.what in ("gemm", "all"):
        layouts = ["fwd", "dgrad", "wgrad"] if a.what == "all" else [a.layout]
        for lay in layouts:
            print(json.dumps(bench_gemm(a.m, a.n, a.k, lay, a.iters, not a.no_compare)), flush=True)
    if a.what == "gemm_gather":
        print(json.dumps(bench_gemm_gather(a.m, a.n, a.k, a.world, a.iters)), flush=True)
    if a.what in ("adamw", "all"):
        print(json.dumps(bench_adamw(1 << 28 if a.what == "all" else a.n, a.iters)), flush=True)
    if a.what in ("attention", "all"):
        print(json.dumps(bench_attention(a.batch, a.seq, a.heads, a.kv_heads, a.iters, not a.no_compare, a.head_dim)), flush=True)
    if a.what in ("elementwise", "all"):
        for r in bench_elementwise(a.iters):
            print(json.dumps(r), flush=True)
    if a.what in ("rmsnorm", "all"):
        print(json.dumps(bench_rmsnorm(8192, 4096, a.iters)), flush=True)


if __name__ == "__main__":
    main()
