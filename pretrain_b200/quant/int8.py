"""int8 series (int8 .. int4 in an int8 container) with fp32 scales per tensor / row / column:
the functions of src/quant/int8.py on the sm_100a kernels.  ``int8_gemm`` replaces the
reference's ``torch._int_mm`` + scaling (src/quant/int8.py:49-53) by the tcgen05 ``kind::i8``
kernel behind ``b200q_gemm_int8``; integer accumulation is exact, so both give the same bits."""

from __future__ import annotations

import torch

from .. import torch_ops as T
from .fp8 import _as_2d, _k_major


def quantize_int8(x: torch.Tensor, qmax: int, dim: int | None = None):
    """(x_i8, scale) with x ~= x_i8.float() * scale, as src/quant/int8.py:9-19: dim=None one
    scale (0-dim), dim=-1 one per row (rows, 1), dim=0 one per column (1, cols) with the codes
    returned as a (rows, cols) view of column-major storage."""
    x2 = _as_2d(x.detach())
    if dim is None:
        codes, scale = T.quantize_int8_tensorwise(x2, int(qmax), False)
        return codes.view(x.shape), scale.reshape(())
    if dim in (-1, x.dim() - 1):
        codes, scales = T.quantize_int8(x2, int(qmax), 1)
        return codes.view(x.shape), scales.view(*x.shape[:-1], 1)
    if dim in (0, -2) and x.dim() == 2:
        codes_t, scales = T.quantize_int8(x2, int(qmax), 0)
        return codes_t.t(), scales.view(1, -1)
    raise ValueError(f"quantize_int8: unsupported dim {dim} for a {x.dim()}-D tensor")


def fake_quantize_int8(x: torch.Tensor, qmax: int, dim: int | None = None) -> torch.Tensor:
    """dequant(quant(x)) in x.dtype (src/quant/int8.py:22-26)."""
    codes, scale = quantize_int8(x, qmax, dim)
    return (codes.float() * scale).to(x.dtype)


def int8_gemm(a, b, out_dtype, a_qmax, b_qmax, rowwise: bool = False):
    """`a @ b` for a (M, K), b (K, N) high precision, both quantized along K to the int8 series
    (src/quant/int8.py:29-53).  The tensor-core kernel wants K % 16 == 0 and N % 8 == 0; other shapes
    are padded with zeros (which change neither a maximum nor the integer product) and the result is
    cut back, so every shape runs on the kernel - there is no matmul fallback like the reference's
    (src/quant/int8.py:35-47)."""
    if not (a.is_cuda and b.is_cuda):
        raise RuntimeError("int8_gemm runs on the B200 kernels only (no CPU path)")
    k, n = b.shape
    pad_k, pad_n = (-k) % 16, (-n) % 8
    if pad_k or pad_n:
        a = torch.nn.functional.pad(a, (0, pad_k))
        b = torch.nn.functional.pad(b, (0, pad_n, 0, pad_k))
    am, a_axis = _k_major(a, 1)
    bm, b_axis = _k_major(b, 0)
    if rowwise:
        ca, sa = T.quantize_int8(am, int(a_qmax), a_axis)
        cb, sb = T.quantize_int8(bm, int(b_qmax), b_axis)
    else:
        ca, sa = T.quantize_int8_tensorwise(am, int(a_qmax), a_axis == 0)
        cb, sb = T.quantize_int8_tensorwise(bm, int(b_qmax), b_axis == 0)
    out = T.gemm_int8(ca, cb, sa, sb)
    if pad_n:
        out = out[:, :n]
    return out if out_dtype == torch.bfloat16 else out.to(out_dtype)
