"""Event trace of the tcgen05 attention kernels: builds the two kernel files with
``-DFTB200_ATTN_TRACE`` into a scratch library, runs them on the Llama-3 8B attention shape and prints,
for the first blocks of the busiest CTA, ``clock64()`` at the pipeline events of the MMA-issuing
thread and of one softmax thread.

    python -m torchft_b200.ops.attention_trace [--seq 8192 --heads 32 --kv-heads 8]

Forward columns: mma = K of the next block present, S issued, P and V present, P·V issued;
softmax = S complete, scores in registers, row maximum exchanged, exponentials done, P published.
Backward columns: mma = S inputs ready, S and dP issued, P/dS ready, tail issued; softmax = S and dP
complete, scores in registers, math done, P/dS published.  Cycles are relative to the first event.
"""

from __future__ import annotations

import argparse
import ctypes
import math
import subprocess
import tempfile
from pathlib import Path

import torch

from .. import _build
from ._native import c_float, c_int, c_ll, ptr, stream_ptr


def _build_trace_lib(workdir: Path) -> ctypes.CDLL:
    src = _build.CSRC / "kernels"
    out = workdir / "libftb200_attention_trace.so"
    cmd = [_build._nvcc(), *_build.NVCC_FLAGS, "-DFTB200_ATTN_TRACE", f"-I{src}", "-shared", "-Xcompiler", "-fPIC",
           str(src / "attention_tcgen05.cu"), str(src / "attention_bwd_tcgen05.cu"), "-o", str(out), "-lcuda"]
    subprocess.run(cmd, check=True)
    return ctypes.CDLL(str(out))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--blocks", type=int, default=12, help="how many blocks / tiles of the traced CTA to print")
    a = ap.parse_args()
    B, S, hq, hkv, D = 1, a.seq, a.heads, a.kv_heads, 128
    with tempfile.TemporaryDirectory() as tmp:
        lib = _build_trace_lib(Path(tmp))
        lib.ftb200_attention_bwd_scratch_bytes.restype = ctypes.c_longlong
        dev = torch.device("cuda")
        qkv = (torch.randn(B * S, (hq + 2 * hkv) * D, device=dev) * 0.5).bfloat16()
        q, k, v = qkv[:, : hq * D], qkv[:, hq * D : (hq + hkv) * D], qkv[:, (hq + hkv) * D :]
        out = torch.empty(B * S, hq * D, device=dev, dtype=torch.bfloat16)
        n_lse = B * hq * S
        lse = torch.zeros(n_lse + 8 + 2048, device=dev)  # the forward trace lands behind the statistics
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        scale = c_float(1 / math.sqrt(D))
        for _ in range(3):
            rc = lib.ftb200_attention_fwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), c_int(B), c_int(S), c_int(hq), c_int(hkv),
                                          c_int(D), c_ll(q.stride(0)), c_ll(k.stride(0)), c_ll(v.stride(0)), c_ll(out.stride(0)),
                                          scale, c_int(1), ptr(status), stream_ptr())
            assert rc == 0, rc
        torch.cuda.synchronize()
        off = (n_lse + 1) // 2 * 2
        tr = lse[off : off + 1024].view(torch.int64).cpu().view(2, 32, 8)
        t0 = int(tr[1, 0, 0])
        print("forward: block | mma [K_ready, S_issued, P_ready, PV_issued] | softmax [S_done, loaded, max, exp, published]")
        for t in range(2, min(32, 2 + a.blocks)):
            print(t, [int(tr[0, t, e]) - t0 for e in range(4)], [int(tr[1, t, e]) - t0 for e in range(5)])

        d_o = torch.randn_like(out)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, : hq * D], dqkv[:, hq * D : (hq + hkv) * D], dqkv[:, (hq + hkv) * D :]
        need = int(lib.ftb200_attention_bwd_scratch_bytes(c_int(B), c_int(S), c_int(hq)))
        scratch = torch.zeros(need + 8192, dtype=torch.uint8, device=dev)  # the backward trace lands behind the scratch
        for _ in range(3):
            rc = lib.ftb200_attention_bwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(d_o), ptr(lse), ptr(dq), ptr(dk), ptr(dv),
                                          ptr(scratch), c_int(B), c_int(S), c_int(hq), c_int(hkv), c_int(D), c_ll(q.stride(0)),
                                          c_ll(k.stride(0)), c_ll(v.stride(0)), c_ll(out.stride(0)), c_ll(d_o.stride(0)),
                                          c_ll(dq.stride(0)), c_ll(dk.stride(0)), c_ll(dv.stride(0)), scale, c_int(1), ptr(status),
                                          stream_ptr())
            assert rc == 0, rc
        torch.cuda.synchronize()
        tr = scratch[need : need + 4096].view(torch.int64).cpu().view(2, 32, 8)
        t0 = int(tr[0, 0, 0])
        print("backward: tile | mma [S_in_ready, S_dP_issued, PdS_ready, tail_issued] | softmax [SdP_done, loaded, math, published]")
        for t in range(min(32, a.blocks)):
            print(t, [int(tr[0, t, e]) - t0 for e in range(4)], [int(tr[1, t, e]) - t0 for e in range(4)])
        print("status word:", int(status.item()))


if __name__ == "__main__":
    main()
