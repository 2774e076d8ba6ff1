"""Block-scaled formats the reference's TODOs name (src/quant/__init__.py:20,26,30): MXFP8 and
NVFP4 quantizers and GEMMs with the same calling convention as ``fp8_gemm``."""

from __future__ import annotations

import torch

from .. import torch_ops as T
from ..ops import SF_NATURAL, SF_SWIZZLED, fmt_of
from .fp8 import _k_major


def quantize_mxfp8(x: torch.Tensor, fp8_dtype: torch.dtype = torch.float8_e4m3fn, dim: int = -1, swizzle: bool = False):
    """(codes, sf): 32-element blocks along ``dim`` of a 2-D tensor.  codes have the contraction
    dimension last (transposed for dim=0); sf is one E8M0 byte per block, (outer, C/32) natural
    or the flat 128x4-swizzled buffer the GEMM reads."""
    axis = 1 if dim in (-1, 1) else 0
    codes, sf = T.quantize_mxfp8(x.detach(), axis, fmt_of(fp8_dtype), SF_SWIZZLED if swizzle else SF_NATURAL)
    return codes.view(fp8_dtype), (sf if swizzle else sf.view(codes.shape[0], -1))


def quantize_nvfp4(x: torch.Tensor, dim: int = -1, swizzle: bool = False):
    """(packed, sf, tensor_scale): 16-element blocks along ``dim``; two E2M1 codes per byte."""
    axis = 1 if dim in (-1, 1) else 0
    packed, sf, ts = T.quantize_nvfp4(x.detach(), axis, SF_SWIZZLED if swizzle else SF_NATURAL)
    return packed, (sf if swizzle else sf.view(packed.shape[0], -1)), ts


def mxfp8_gemm(a, b, out_dtype, a_dtype=torch.float8_e4m3fn, b_dtype=torch.float8_e4m3fn):
    """`a @ b`, a (M, K), b (K, N), both block-quantized along K."""
    am, a_axis = _k_major(a, 1)
    bm, b_axis = _k_major(b, 0)
    # one library call: both quantizations (one launch when both operands have K contiguous) and the GEMM behind them
    out = T.linear_mxfp8(am, a_axis, bm, b_axis, fmt_of(a_dtype), fmt_of(b_dtype))
    return out if out_dtype == torch.bfloat16 else out.to(out_dtype)


def nvfp4_gemm(a, b, out_dtype):
    am, a_axis = _k_major(a, 1)
    bm, b_axis = _k_major(b, 0)
    pa, sfa, ta = T.quantize_nvfp4(am, a_axis, SF_SWIZZLED)
    pb, sfb, tb = T.quantize_nvfp4(bm, b_axis, SF_SWIZZLED)
    out = T.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb)
    return out if out_dtype == torch.bfloat16 else out.to(out_dtype)
