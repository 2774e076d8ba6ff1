"""FP8 with fp32 scales per tensor / row / column: the functions of src/quant/fp8.py, running
on the sm_100a kernels.  ``fp8_gemm`` replaces the reference's ``torch._scaled_mm`` call
(src/quant/fp8.py:59-65) by the tcgen05 kernel behind ``b200q_gemm_fp8``."""

from __future__ import annotations

import torch

from .. import torch_ops as T
from ..ops import fmt_of

HARDWARE_REQUIREMENT = "an NVIDIA B200 (compute capability 10.0); this build has no other backend"


def is_supported() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    return x if x.dim() == 2 else x.reshape(-1, x.shape[-1])


def quantize_fp8(x: torch.Tensor, fp8_dtype: torch.dtype, dim: int | None = None):
    """(x_fp8, scale) with x ~= x_fp8.float() * scale, as src/quant/fp8.py:16-32.

    dim=None: one scale (0-dim).  dim=-1: one per row, shape (rows, 1).  dim=0: one per column,
    shape (1, cols); the codes come back as a (rows, cols) view of column-major storage, the
    layout the GEMM wants for that operand."""
    x2 = _as_2d(x.detach())
    fmt = fmt_of(fp8_dtype)
    if dim is None:
        codes, scale = T.quantize_fp8_tensorwise(x2, fmt, False)
        return codes.view(fp8_dtype).view(x.shape), scale.reshape(())
    if dim in (-1, x.dim() - 1):
        codes, scales = T.quantize_fp8(x2, fmt, 1)
        return codes.view(fp8_dtype).view(x.shape), scales.view(*x.shape[:-1], 1)
    if dim in (0, -2) and x.dim() == 2:
        codes_t, scales = T.quantize_fp8(x2, fmt, 0)
        return codes_t.view(fp8_dtype).t(), scales.view(1, -1)
    raise ValueError(f"quantize_fp8: unsupported dim {dim} for a {x.dim()}-D tensor")


def fake_quantize_fp8(x: torch.Tensor, fp8_dtype: torch.dtype, dim: int | None = None) -> torch.Tensor:
    """dequant(quant(x)) in x.dtype (src/quant/fp8.py:68-78): fp32 multiply, one rounding."""
    codes, scale = quantize_fp8(x, fp8_dtype, dim)
    return (codes.float() * scale).to(x.dtype)


def _k_major(t: torch.Tensor, contraction_dim: int):
    """(matrix, axis) such that quantizing `matrix` along `axis` yields codes with the
    contraction dimension contiguous, without copying `t` first."""
    if contraction_dim == 1:                    # t is (outer, C)
        return (t.t(), 0) if (t.stride(0) == 1 and t.stride(1) != 1) else (t, 1)
    return (t.t(), 1) if (t.stride(0) == 1 and t.stride(1) != 1) else (t, 0)   # t is (C, outer)


def fp8_gemm(a, b, out_dtype, a_dtype, b_dtype, rowwise: bool = False):
    """`a @ b` for a (M, K), b (K, N) high precision; both quantized along K — per row of a
    and per column of b when ``rowwise``, else one scale per tensor (src/quant/fp8.py:35-65).
    Transposed views (``w.t()``, ``g.t()``) are read in place by the transposing quantizer."""
    if a_dtype == torch.float8_e5m2 and b_dtype == torch.float8_e5m2:
        raise ValueError("fp8_gemm: at least one operand must be e4m3")
    fa, fb = fmt_of(a_dtype), fmt_of(b_dtype)
    am, a_axis = _k_major(a, 1)
    bm, b_axis = _k_major(b, 0)
    if rowwise:
        ca, sa = T.quantize_fp8(am, fa, a_axis)
        cb, sb = T.quantize_fp8(bm, fb, b_axis)
    else:
        ca, sa = T.quantize_fp8_tensorwise(am, fa, a_axis == 0)
        cb, sb = T.quantize_fp8_tensorwise(bm, fb, b_axis == 0)
    out = T.gemm_fp8(ca, fa, cb, fb, sa, sb)
    return out if out_dtype == torch.bfloat16 else out.to(out_dtype)
