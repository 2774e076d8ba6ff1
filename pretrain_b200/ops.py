"""Tensor-level wrappers of the C-ABI entry points: allocate outputs with torch, pass raw
pointers and the current CUDA stream.  Everything here runs on the GPU through libb200q.so;
nothing has a CPU path."""

from __future__ import annotations

import torch

from . import _lib

E4M3, E5M2 = 0, 1
SF_NATURAL, SF_SWIZZLED = 0, 1
_FMT_OF_DTYPE = {torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}
_DTYPE_OF_FMT = {E4M3: torch.float8_e4m3fn, E5M2: torch.float8_e5m2}


def fmt_of(dtype_or_fmt) -> int:
    return _FMT_OF_DTYPE.get(dtype_or_fmt, dtype_or_fmt)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _mat(x: torch.Tensor) -> torch.Tensor:
    """A bf16 CUDA matrix the kernels can read in place: unit column stride, pitch % 8 == 0,
    16-byte aligned base; otherwise a contiguous copy."""
    if x.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if not x.is_cuda:
        raise RuntimeError("b200q ops need CUDA tensors (no CPU path exists)")
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    if x.stride(1) != 1 or x.stride(0) % 8 or x.stride(0) < x.shape[1] or x.data_ptr() % 16:
        x = x.contiguous()
    return x


def sf_bytes(outer: int, nblk: int, layout: int = SF_SWIZZLED) -> int:
    return _lib.load().b200q_sf_bytes(outer, nblk, layout)


def amax(x: torch.Tensor) -> torch.Tensor:
    x = _mat(x)
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_amax(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), out.data_ptr(), _stream()), "b200q_amax")
    return out


def quantize_fp8(x: torch.Tensor, fmt, axis: int):
    """Per-row (axis=1) or per-column (axis=0, codes transposed) FP8.  Returns
    (codes uint8 [outer, C], scales fp32 [outer])."""
    x = _mat(x)
    rows, cols = x.shape
    outer, c = (rows, cols) if axis == 1 else (cols, rows)
    codes = torch.empty(outer, c, dtype=torch.uint8, device=x.device)
    scales = torch.empty(outer, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_quantize_fp8(x.data_ptr(), rows, cols, x.stride(0), axis, fmt_of(fmt), codes.data_ptr(),
                                              scales.data_ptr(), _stream()), "b200q_quantize_fp8")
    return codes, scales


def quantize_fp8_tensorwise(x: torch.Tensor, fmt, transpose: bool = False, tensor_amax: torch.Tensor | None = None):
    x = _mat(x)
    rows, cols = x.shape
    if tensor_amax is None:
        tensor_amax = amax(x)
    shape = (cols, rows) if transpose else (rows, cols)
    codes = torch.empty(shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_quantize_fp8_tensorwise(x.data_ptr(), rows, cols, x.stride(0), int(transpose), fmt_of(fmt),
                                                         tensor_amax.data_ptr(), codes.data_ptr(), scale.data_ptr(), _stream()),
               "b200q_quantize_fp8_tensorwise")
    return codes, scale


def quantize_mxfp8(x: torch.Tensor, axis: int = 1, fmt=E4M3, layout: int = SF_SWIZZLED):
    """Returns (codes uint8 [outer, C], sf uint8 flat buffer in `layout`)."""
    x = _mat(x)
    rows, cols = x.shape
    outer, c = (rows, cols) if axis == 1 else (cols, rows)
    codes = torch.empty(outer, c, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(outer, c // 32, layout), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.load().b200q_quantize_mxfp8(x.data_ptr(), rows, cols, x.stride(0), axis, fmt_of(fmt), codes.data_ptr(),
                                                sf.data_ptr(), layout, _stream()), "b200q_quantize_mxfp8")
    return codes, sf


def quantize_nvfp4(x: torch.Tensor, axis: int = 1, tensor_amax: torch.Tensor | None = None, layout: int = SF_SWIZZLED):
    """Returns (packed uint8 [outer, C/2], sf uint8 flat buffer, tensor_scale fp32 [1])."""
    x = _mat(x)
    rows, cols = x.shape
    outer, c = (rows, cols) if axis == 1 else (cols, rows)
    if tensor_amax is None:
        tensor_amax = amax(x)
    codes = torch.empty(outer, c // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(outer, c // 16, layout), dtype=torch.uint8, device=x.device)
    ts = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_quantize_nvfp4(x.data_ptr(), rows, cols, x.stride(0), axis, tensor_amax.data_ptr(),
                                                codes.data_ptr(), sf.data_ptr(), layout, ts.data_ptr(), _stream()),
               "b200q_quantize_nvfp4")
    return codes, sf, ts


def _out(m: int, n: int, device, out: torch.Tensor | None) -> torch.Tensor:
    if out is None:
        return torch.empty(m, n, dtype=torch.bfloat16, device=device)
    if out.dtype != torch.bfloat16 or out.shape != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be a bf16 (M, N) tensor with unit column stride")
    return out


def gemm_fp8(a_codes, a_fmt, b_codes, b_fmt, scale_a, scale_b, out=None):
    """D = (A . B^T) * scale_a[:, None] * scale_b[None, :]; scales may have one element."""
    m, k = a_codes.shape
    n = b_codes.shape[0]
    d = _out(m, n, a_codes.device, out)
    _lib.check(_lib.load().b200q_gemm_fp8(a_codes.data_ptr(), fmt_of(a_fmt), b_codes.data_ptr(), fmt_of(b_fmt),
                                          scale_a.data_ptr(), int(scale_a.numel() == 1), scale_b.data_ptr(),
                                          int(scale_b.numel() == 1), m, n, k, d.data_ptr(), d.stride(0), _stream()),
               "b200q_gemm_fp8")
    return d


def gemm_mxfp8(a_codes, a_sf, b_codes, b_sf, a_fmt=E4M3, b_fmt=E4M3, out=None):
    m, k = a_codes.shape
    n = b_codes.shape[0]
    d = _out(m, n, a_codes.device, out)
    _lib.check(_lib.load().b200q_gemm_mxfp8(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                            fmt_of(b_fmt), b_sf.data_ptr(), m, n, k, d.data_ptr(), d.stride(0), _stream()),
               "b200q_gemm_mxfp8")
    return d


def gemm_nvfp4(a_packed, a_sf, a_ts, b_packed, b_sf, b_ts, out=None):
    m, k2 = a_packed.shape
    n = b_packed.shape[0]
    d = _out(m, n, a_packed.device, out)
    _lib.check(_lib.load().b200q_gemm_nvfp4(a_packed.data_ptr(), a_sf.data_ptr(), b_packed.data_ptr(), b_sf.data_ptr(),
                                            a_ts.data_ptr(), b_ts.data_ptr(), m, n, 2 * k2, d.data_ptr(), d.stride(0), _stream()),
               "b200q_gemm_nvfp4")
    return d


def device_status() -> None:
    """Raises if a kernel's bounded wait expired since the last check (synchronizes)."""
    _lib.check(_lib.load().b200q_device_status(), "b200q device status")
