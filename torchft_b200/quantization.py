"""Block-scaled fp8 (e4m3) quantisation of gradient-like tensors.

Format: consecutive blocks of 128 elements, each stored as 128 e4m3 codes plus one fp32
scale ``s = absmax / 448`` (``value = s * decode(code)``).  A quantised buffer of ``n``
elements (``n`` a multiple of 128) is one ``uint8`` tensor laid out as
``[n codes][n/128 fp32 scales]`` -- 1.03 bytes per element for any tensor shape.

The reference quantises per *row* of each 2-D parameter with Triton kernels
(torchft/quantization.py:53-428), which degenerates to 8 bytes per element for the 1-D
flat buffers DiLoCo sends; the block format here does not depend on the shape.  On CUDA
the functions below launch the sm_100a kernels of ``csrc/team/quant_team.cu``; on CPU they
run the PyTorch restatement (``ref_*``) that also serves as the numerics oracle.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch

from .ops import _native as N

BLOCK = 128
FP8_MAX = 448.0
_DT = {torch.bfloat16: 0, torch.float32: 1}


def quantized_nbytes(n: int) -> int:
    """Bytes of the quantised buffer for ``n`` (padded) elements."""
    assert n % BLOCK == 0
    return n + (n // BLOCK) * 4


def padded_numel(n: int, world_size: int = 1) -> int:
    """``n`` rounded up so that every rank's slice is a whole number of blocks."""
    g = BLOCK * world_size
    return (n + g - 1) // g * g


def split_quantized(buf: torch.Tensor, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Views ``(codes uint8 [n], scales fp32 [n/128])`` into a quantised buffer."""
    return buf[:n], buf[n : n + (n // BLOCK) * 4].view(torch.float32)


# --------------------------------------------------------------------------- reference (any device)


def ref_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """PyTorch restatement of the block quantiser: ``(codes uint8 [n], scales fp32 [n/128])`` with
    ``scale = amax / 448`` per 128 elements (1 for an all-zero block) and ``code = e4m3(x / scale)``."""
    xf = x.float().reshape(-1, BLOCK)
    amax = xf.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    codes = (xf / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return codes.view(torch.uint8).reshape(-1), scale


def ref_dequantize(codes: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Inverse of :func:`ref_quantize`: ``code * scale`` per block, cast to ``dtype``."""
    vals = codes.view(torch.float8_e4m3fn).float().reshape(-1, BLOCK) * scales[:, None]
    return vals.reshape(-1).to(dtype)


# --------------------------------------------------------------------------- kernels


def quantize_into(x: torch.Tensor, out: torch.Tensor, minus: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Quantise flat ``x`` (or ``x - minus``) into the quantised buffer ``out``."""
    n = x.numel()
    assert n % BLOCK == 0 and out.dtype == torch.uint8 and out.numel() >= quantized_nbytes(n)
    codes, scales = split_quantized(out, n)
    if not x.is_cuda:
        src = x if minus is None else (x.float() - minus.float())
        c, s = ref_quantize(src)
        codes.copy_(c)
        scales.copy_(s)
        return out
    N.check(N.lib().ftb200_quantize_fp8(N.ptr(x), N.ptr(minus), N.ptr(codes), N.ptr(scales), ctypes.c_longlong(n),
                                        ctypes.c_int(_DT[x.dtype]), N.stream_ptr()), "quantize_fp8")
    return out


def dequantize_from(buf: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Dequantise the quantised buffer ``buf`` into flat ``out`` (whose length is a multiple of the block size)."""
    n = out.numel()
    assert n % BLOCK == 0
    codes, scales = split_quantized(buf, n)
    if not out.is_cuda:
        out.copy_(ref_dequantize(codes, scales, out.dtype).view_as(out))
        return out
    N.check(N.lib().ftb200_dequantize_fp8(N.ptr(codes), N.ptr(scales), N.ptr(out), ctypes.c_longlong(n),
                                          ctypes.c_int(_DT[out.dtype]), N.stream_ptr()), "dequantize_fp8")
    return out


def reduce_quantized(bufs: List[torch.Tensor], n: int, scale: float, out: torch.Tensor) -> torch.Tensor:
    """``out`` (quantised) = requantise(scale * sum_i dequant(bufs[i])) over ``n`` elements;
    fp32 accumulation in the order given."""
    acc = torch.zeros(n, dtype=torch.float32, device=out.device)
    tmp = torch.empty(n, dtype=torch.float32, device=out.device)
    for b in bufs:
        dequantize_from(b, tmp)
        acc += tmp
    acc *= scale
    return quantize_into(acc, out)


# --------------------------------------------------------------------------- list-of-tensors API


def fused_quantize_into_fp8(tensors: List[torch.Tensor], world_size: int) -> Tuple[torch.Tensor, List[int]]:
    """Pack ``tensors`` (same dtype/device) into one flat quantised buffer whose element
    count is padded to ``128 * world_size`` so it splits evenly across ranks.  Returns the
    buffer and the padded total element count (as a one-element list for symmetry with
    :func:`fused_dequantize_from_fp8`)."""
    assert tensors, "nothing to quantise"
    dtype, device = tensors[0].dtype, tensors[0].device
    assert dtype in _DT, f"unsupported dtype {dtype}"
    total = sum(t.numel() for t in tensors)
    n = padded_numel(total, world_size)
    flat = torch.zeros(n, dtype=dtype, device=device)
    off = 0
    for t in tensors:
        assert t.dtype == dtype and t.device == device
        flat[off : off + t.numel()].copy_(t.reshape(-1))
        off += t.numel()
    buf = torch.empty(quantized_nbytes(n), dtype=torch.uint8, device=device)
    quantize_into(flat, buf)
    return buf, [n]


def fused_dequantize_from_fp8(tensors: List[torch.Tensor], buf: torch.Tensor, world_size: int) -> None:
    """Inverse of :func:`fused_quantize_into_fp8`: write the values back into ``tensors``."""
    dtype, device = tensors[0].dtype, tensors[0].device
    total = sum(t.numel() for t in tensors)
    n = padded_numel(total, world_size)
    flat = torch.empty(n, dtype=dtype, device=device)
    dequantize_from(buf, flat)
    off = 0
    for t in tensors:
        t.copy_(flat[off : off + t.numel()].view_as(t))
        off += t.numel()
