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


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream (the raw-handle query skips building a Stream object per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
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
    """b200q_sf_bytes without the foreign call: 512-byte tiles of 128 rows x 4 blocks, or one byte per block."""
    if layout == SF_SWIZZLED:
        return ((outer + 127) // 128) * ((nblk + 3) // 4) * 512
    return outer * nblk


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


def quantize_fp8_both(x: torch.Tensor, fmt):
    """Per-row and per-column FP8 of x (rows, cols) in two reads: returns (codes_row (rows, cols),
    scales_row (rows), codes_col (cols, rows), scales_col (cols)), equal to quantize_fp8(x, fmt, 1) +
    quantize_fp8(x, fmt, 0).  rows % 16 == 0, cols <= 8192."""
    x = _mat(x)
    rows, cols = x.shape
    lib = _lib.load()
    cr = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    sr = torch.empty(rows, dtype=torch.float32, device=x.device)
    cc = torch.empty(cols, rows, dtype=torch.uint8, device=x.device)
    sc = torch.empty(cols, dtype=torch.float32, device=x.device)
    ws = torch.empty(lib.b200q_quantize_fp8_both_workspace_bytes(cols), dtype=torch.uint8, device=x.device)
    _lib.check(lib.b200q_quantize_fp8_both(x.data_ptr(), rows, cols, x.stride(0), fmt_of(fmt), cr.data_ptr(), sr.data_ptr(),
                                           cc.data_ptr(), sc.data_ptr(), ws.data_ptr(), _stream()), "b200q_quantize_fp8_both")
    return cr, sr, cc, sc


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


def quantize_int8(x: torch.Tensor, qmax: int, axis: int):
    """Per-row (axis=1) or per-column (axis=0, codes transposed) int8-series codes.  Returns
    (codes int8 [outer, C], scales fp32 [outer])."""
    x = _mat(x)
    rows, cols = x.shape
    outer, c = (rows, cols) if axis == 1 else (cols, rows)
    codes = torch.empty(outer, c, dtype=torch.int8, device=x.device)
    scales = torch.empty(outer, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_quantize_int8(x.data_ptr(), rows, cols, x.stride(0), axis, int(qmax), codes.data_ptr(),
                                               scales.data_ptr(), _stream()), "b200q_quantize_int8")
    return codes, scales


def quantize_int8_tensorwise(x: torch.Tensor, qmax: int, transpose: bool = False, tensor_amax: torch.Tensor | None = None):
    x = _mat(x)
    rows, cols = x.shape
    if tensor_amax is None:
        tensor_amax = amax(x)
    shape = (cols, rows) if transpose else (rows, cols)
    codes = torch.empty(shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_quantize_int8_tensorwise(x.data_ptr(), rows, cols, x.stride(0), int(transpose), int(qmax),
                                                          tensor_amax.data_ptr(), codes.data_ptr(), scale.data_ptr(), _stream()),
               "b200q_quantize_int8_tensorwise")
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


def _nt(num_tiles):
    return num_tiles.data_ptr() if num_tiles is not None else None


def quantize_mxfp8_dual(x: torch.Tensor, fmt=E4M3, layout: int = SF_SWIZZLED, num_tiles: torch.Tensor | None = None):
    """One pass over x (rows, cols): returns (codes_row, sf_row, codes_col, sf_col), equal to
    quantize_mxfp8(x, 1) + quantize_mxfp8(x, 0).  rows % 32 == 0 and cols % 32 == 0.  `num_tiles` (device int32):
    only the first num_tiles 128-row tiles are processed, the rest of the outputs is left as allocated."""
    x = _mat(x)
    rows, cols = x.shape
    cr = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    cc = torch.empty(cols, rows, dtype=torch.uint8, device=x.device)
    sr = torch.empty(sf_bytes(rows, cols // 32, layout), dtype=torch.uint8, device=x.device)
    sc = torch.empty(sf_bytes(cols, rows // 32, layout), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.load().b200q_quantize_mxfp8_dual(x.data_ptr(), rows, cols, x.stride(0), fmt_of(fmt), cr.data_ptr(), sr.data_ptr(),
                                                     cc.data_ptr(), sc.data_ptr(), layout, _nt(num_tiles), _stream()), "b200q_quantize_mxfp8_dual")
    return cr, sr, cc, sc


def glu_row_map(n_groups: int, inter: int, device) -> torch.Tensor:
    """dst_row for weights stacked as n_groups x [gate (inter rows); up (inter rows)]: the
    interleaved order the SwiGLU epilogue reads (32 gate rows, then the 32 up rows of the same
    outputs).  inter % 32 == 0."""
    if inter % 32:
        raise ValueError("intermediate size must be a multiple of 32")
    j = torch.arange(inter, device=device)
    gate = (j // 32) * 64 + j % 32
    one = torch.cat([gate, gate + 32])
    base = torch.arange(n_groups, device=device).unsqueeze(1) * (2 * inter)
    return (base + one.unsqueeze(0)).reshape(-1).to(torch.int32)


def quantize_mxfp8_rowmap(x: torch.Tensor, dst_row: torch.Tensor, fmt=E4M3, layout: int = SF_SWIZZLED):
    """Row-wise MXFP8 of x with input row r written as output row dst_row[r] (a permutation)."""
    x = _mat(x)
    rows, cols = x.shape
    if dst_row.numel() != rows or dst_row.dtype != torch.int32 or not dst_row.is_cuda:
        raise ValueError("dst_row: one int32 per row, on the GPU")
    codes = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols // 32, layout), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.load().b200q_quantize_mxfp8_rowmap(x.data_ptr(), rows, cols, x.stride(0), fmt_of(fmt), dst_row.data_ptr(),
                                                       codes.data_ptr(), sf.data_ptr(), layout, _stream()),
               "b200q_quantize_mxfp8_rowmap")
    return codes, sf


def quantize_mxfp8_pair(x0: torch.Tensor, x1: torch.Tensor, dst_row0: torch.Tensor | None = None, dst_row1: torch.Tensor | None = None,
                        fmt=E4M3, layout: int = SF_SWIZZLED):
    """Row-wise MXFP8 of two matrices in one launch (each optionally through an output-row map): (codes0, sf0, codes1, sf1),
    equal to two quantize_mxfp8 / quantize_mxfp8_rowmap calls."""
    x0, x1 = _mat(x0), _mat(x1)
    outs = []
    for x, m in ((x0, dst_row0), (x1, dst_row1)):
        if m is not None and (m.numel() != x.shape[0] or m.dtype != torch.int32 or not m.is_cuda):
            raise ValueError("dst_row: one int32 per row, on the GPU")
        outs.append(torch.empty(x.shape[0], x.shape[1], dtype=torch.uint8, device=x.device))
        outs.append(torch.empty(sf_bytes(x.shape[0], x.shape[1] // 32, layout), dtype=torch.uint8, device=x.device))
    _lib.check(_lib.load().b200q_quantize_mxfp8_pair(
        x0.data_ptr(), x0.shape[0], x0.shape[1], x0.stride(0), dst_row0.data_ptr() if dst_row0 is not None else None, outs[0].data_ptr(),
        outs[1].data_ptr(), x1.data_ptr(), x1.shape[0], x1.shape[1], x1.stride(0), dst_row1.data_ptr() if dst_row1 is not None else None,
        outs[2].data_ptr(), outs[3].data_ptr(), fmt_of(fmt), layout, _stream()), "b200q_quantize_mxfp8_pair")
    return tuple(outs)


def quantize_nvfp4_rowmap(x: torch.Tensor, dst_row: torch.Tensor, tensor_amax: torch.Tensor | None = None, layout: int = SF_SWIZZLED):
    """Row-wise NVFP4 of x with input row r written as output row dst_row[r] (a permutation)."""
    x = _mat(x)
    rows, cols = x.shape
    if dst_row.numel() != rows or dst_row.dtype != torch.int32 or not dst_row.is_cuda:
        raise ValueError("dst_row: one int32 per row, on the GPU")
    if tensor_amax is None:
        tensor_amax = amax(x)
    codes = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, cols // 16, layout), dtype=torch.uint8, device=x.device)
    ts = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().b200q_quantize_nvfp4_rowmap(x.data_ptr(), rows, cols, x.stride(0), tensor_amax.data_ptr(), dst_row.data_ptr(),
                                                       codes.data_ptr(), sf.data_ptr(), layout, ts.data_ptr(), _stream()),
               "b200q_quantize_nvfp4_rowmap")
    return codes, sf, ts


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


def quantize_nvfp4_both(x: torch.Tensor, tensor_amax: torch.Tensor | None = None, layout: int = SF_SWIZZLED):
    """Both NVFP4 copies of x (rows, cols) under ONE tensor scale: (packed_row (rows, cols/2), sf_row, packed_col
    (cols, rows/2), sf_col, tensor_scale) - what quantize_nvfp4(x, 1) and quantize_nvfp4(x, 0) give, with the tensor
    maximum taken once (three passes over x instead of four).  rows % 32 == 0 and cols % 32 == 0."""
    x = _mat(x)
    if tensor_amax is None:
        tensor_amax = amax(x)
    pr, sr, ts = quantize_nvfp4(x, 1, tensor_amax, layout)
    pc, sc, _ = quantize_nvfp4(x, 0, tensor_amax, layout)
    return pr, sr, pc, sc, ts


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


def gemm_int8(a_codes, b_codes, scale_a, scale_b, out=None):
    """D = bf16((float(A . B^T) * scale_a[:, None]) * scale_b[None, :]), int8 codes, exact integer
    accumulation; scales may have one element."""
    m, k = a_codes.shape
    n = b_codes.shape[0]
    d = _out(m, n, a_codes.device, out)
    _lib.check(_lib.load().b200q_gemm_int8(a_codes.data_ptr(), b_codes.data_ptr(), scale_a.data_ptr(), int(scale_a.numel() == 1),
                                           scale_b.data_ptr(), int(scale_b.numel() == 1), m, n, k, d.data_ptr(), d.stride(0),
                                           _stream()), "b200q_gemm_int8")
    return d


def gemm_mxfp8(a_codes, a_sf, b_codes, b_sf, a_fmt=E4M3, b_fmt=E4M3, out=None):
    m, k = a_codes.shape
    n = b_codes.shape[0]
    d = _out(m, n, a_codes.device, out)
    _lib.check(_lib.load().b200q_gemm_mxfp8(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                            fmt_of(b_fmt), b_sf.data_ptr(), m, n, k, d.data_ptr(), d.stride(0), _stream()),
               "b200q_gemm_mxfp8")
    return d


def linear_mxfp8(a: torch.Tensor, a_axis: int, b: torch.Tensor, b_axis: int, a_fmt=E4M3, b_fmt=E4M3, out=None):
    """D = A . B^T with both bf16 operands quantized to MXFP8 along the contraction dimension, in one library call:
    `a` is the (M, K) operand when a_axis == 1, or its (K, M) storage when a_axis == 0 (likewise `b` with N)."""
    a, b = _mat(a), _mat(b)
    m, k = (a.shape if a_axis == 1 else a.shape[::-1])
    n = b.shape[0] if b_axis == 1 else b.shape[1]
    d = _out(m, n, a.device, out)
    lib = _lib.load()
    ws = torch.empty(lib.b200q_linear_mxfp8_workspace_bytes(m, n, k), dtype=torch.uint8, device=a.device)
    _lib.check(lib.b200q_linear_mxfp8(a.data_ptr(), a.shape[0], a.shape[1], a.stride(0), a_axis, fmt_of(a_fmt), b.data_ptr(), b.shape[0],
                                      b.shape[1], b.stride(0), b_axis, fmt_of(b_fmt), d.data_ptr(), d.stride(0), ws.data_ptr(), _stream()),
               "b200q_linear_mxfp8")
    return d


def gemm_nvfp4(a_packed, a_sf, a_ts, b_packed, b_sf, b_ts, out=None):
    m, k2 = a_packed.shape
    n = b_packed.shape[0]
    d = _out(m, n, a_packed.device, out)
    _lib.check(_lib.load().b200q_gemm_nvfp4(a_packed.data_ptr(), a_sf.data_ptr(), b_packed.data_ptr(), b_sf.data_ptr(),
                                            a_ts.data_ptr(), b_ts.data_ptr(), m, n, 2 * k2, d.data_ptr(), d.stride(0), _stream()),
               "b200q_gemm_nvfp4")
    return d


def _ptr_array(ptrs):
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def gemm_mxfp8_allgather(a_codes, a_sf, b_codes, b_sf, out_ptrs, rank: int, n: int, ldd: int, a_fmt=E4M3, b_fmt=E4M3):
    """Fused GEMM + all-gather: this rank's (M, n) block goes to rows [rank*M, rank*M+M) of the gathered
    buffer of every rank; `out_ptrs` are the device pointers of those buffers (own and peer-mapped)."""
    m, k = a_codes.shape
    _lib.check(_lib.load().b200q_gemm_mxfp8_allgather(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                                      fmt_of(b_fmt), b_sf.data_ptr(), m, n, k, _ptr_array(out_ptrs),
                                                      len(out_ptrs), rank, ldd, _stream()), "b200q_gemm_mxfp8_allgather")


def gemm_mxfp8_allgather_mxfp8(a_codes, a_sf, b_codes, b_sf, code_ptrs, sf_ptrs, rank: int, n: int, ldc: int, a_fmt=E4M3, b_fmt=E4M3):
    """Fused GEMM + all-gather with an MXFP8 output: this rank's (M, n) block, rounded to bf16 and quantized
    along its columns, goes to rows [rank*M, rank*M+M) of every rank's gathered codes and swizzled scale
    factors (`code_ptrs` / `sf_ptrs`: device pointers of those buffers, own and peer-mapped)."""
    m, k = a_codes.shape
    _lib.check(_lib.load().b200q_gemm_mxfp8_allgather_mxfp8(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                                            fmt_of(b_fmt), b_sf.data_ptr(), m, n, k, _ptr_array(code_ptrs),
                                                            _ptr_array(sf_ptrs), len(code_ptrs), rank, ldc, _stream()),
               "b200q_gemm_mxfp8_allgather_mxfp8")


def gemm_mxfp8_quantized(a_codes, a_sf, b_codes, b_sf, a_fmt=E4M3, b_fmt=E4M3):
    """(codes uint8 (M, N), swizzled sf) = quantize_mxfp8(gemm_mxfp8(...)) in one kernel: the GEMM's epilogue
    quantizes its bf16 result along the columns.  M % 128 == 0, N % 128 == 0."""
    m, n = a_codes.shape[0], b_codes.shape[0]
    codes = torch.empty(m, n, dtype=torch.uint8, device=a_codes.device)
    sf = torch.empty(sf_bytes(m, n // 32), dtype=torch.uint8, device=a_codes.device)
    gemm_mxfp8_allgather_mxfp8(a_codes, a_sf, b_codes, b_sf, [codes.data_ptr()], [sf.data_ptr()], 0, n, codes.stride(0), a_fmt, b_fmt)
    return codes, sf


def gemm_mxfp8_scatter(a_codes, a_sf, b_codes, b_sf, stage_ptrs, rank: int, n: int, ldd: int, a_fmt=E4M3, b_fmt=E4M3):
    """First half of a fused GEMM + reduce-scatter: block rows [g*M/world, ...) of this rank's (M, n) partial result go
    to slot `rank` of rank g's staging buffer (`stage_ptrs`: device pointers of the ranks' [world, M/world, n] buffers)."""
    m, k = a_codes.shape
    _lib.check(_lib.load().b200q_gemm_mxfp8_scatter(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                                    fmt_of(b_fmt), b_sf.data_ptr(), m, n, k, _ptr_array(stage_ptrs),
                                                    len(stage_ptrs), rank, ldd, _stream()), "b200q_gemm_mxfp8_scatter")


def sum_slots(stage: torch.Tensor) -> torch.Tensor:
    """(slots, rows, cols) bf16 -> (rows, cols) bf16: the slots added in order in fp32, one rounding."""
    slots, rows, cols = stage.shape
    if stage.dtype != torch.bfloat16 or not stage.is_contiguous():
        raise ValueError("expected a contiguous bf16 (slots, rows, cols) tensor")
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=stage.device)
    _lib.check(_lib.load().b200q_sum_slots(stage.data_ptr(), slots, rows, cols, cols, out.data_ptr(), cols, _stream()), "b200q_sum_slots")
    return out


def gemm_nvfp4_allgather(a_packed, a_sf, a_ts, b_packed, b_sf, b_ts, out_ptrs, rank: int, n: int, ldd: int):
    m, k2 = a_packed.shape
    _lib.check(_lib.load().b200q_gemm_nvfp4_allgather(a_packed.data_ptr(), a_sf.data_ptr(), b_packed.data_ptr(), b_sf.data_ptr(),
                                                      a_ts.data_ptr(), b_ts.data_ptr(), m, n, 2 * k2, _ptr_array(out_ptrs),
                                                      len(out_ptrs), rank, ldd, _stream()), "b200q_gemm_nvfp4_allgather")


def gemm_fp8_allgather(a_codes, a_fmt, b_codes, b_fmt, scale_a, scale_b, out_ptrs, rank: int, n: int, ldd: int):
    m, k = a_codes.shape
    _lib.check(_lib.load().b200q_gemm_fp8_allgather(a_codes.data_ptr(), fmt_of(a_fmt), b_codes.data_ptr(), fmt_of(b_fmt),
                                                    scale_a.data_ptr(), int(scale_a.numel() == 1), scale_b.data_ptr(),
                                                    int(scale_b.numel() == 1), m, n, k, _ptr_array(out_ptrs), len(out_ptrs),
                                                    rank, ldd, _stream()), "b200q_gemm_fp8_allgather")


# ---- MoE ------------------------------------------------------------------------------------

class MoEPlan:
    """Device-side tables of the padded expert-sorted layout (see include/b200q.h)."""
    __slots__ = ("offs", "padded_offs", "row_of", "src_of_row", "tile_expert", "num_tiles", "padded_rows", "n_experts")


def moe_padded_rows(n_pairs: int, n_experts: int) -> int:
    return _lib.load().b200q_moe_padded_rows(n_pairs, n_experts)


def _new_plan(n_rows: int, n_experts: int, device) -> MoEPlan:
    p = MoEPlan()
    p.n_experts = n_experts
    p.padded_rows = moe_padded_rows(n_rows, n_experts)
    i32 = dict(dtype=torch.int32, device=device)
    p.offs = torch.empty(n_experts, **i32)
    p.padded_offs = torch.empty(n_experts + 1, **i32)
    p.src_of_row = torch.empty(p.padded_rows, **i32)
    p.tile_expert = torch.empty(p.padded_rows // 128, **i32)
    p.num_tiles = torch.empty(1, **i32)
    p.row_of = None
    return p


def moe_permute_plan(top_indices: torch.Tensor, n_experts: int) -> MoEPlan:
    """top_indices: int64 (T, k) expert ids -> plan (stable sort by expert, reference order)."""
    t, k = top_indices.shape
    idx = top_indices.contiguous().view(-1)
    if idx.dtype != torch.int64:
        idx = idx.to(torch.int64)
    lib = _lib.load()
    p = _new_plan(t * k, n_experts, idx.device)
    p.row_of = torch.empty(t * k, dtype=torch.int32, device=idx.device)
    ws = torch.empty(lib.b200q_moe_plan_workspace_bytes(t * k, n_experts), dtype=torch.uint8, device=idx.device)
    _lib.check(lib.b200q_moe_permute_plan(idx.data_ptr(), t * k, k, n_experts, p.offs.data_ptr(), p.padded_offs.data_ptr(),
                                          p.row_of.data_ptr(), p.src_of_row.data_ptr(), p.tile_expert.data_ptr(),
                                          p.num_tiles.data_ptr(), ws.data_ptr(), _stream()), "b200q_moe_permute_plan")
    return p


def moe_pad_plan(offs: torch.Tensor, n_rows: int) -> MoEPlan:
    """Plan for rows already sorted by expert; offs int32 (E,) cumulative ends."""
    offs = offs.to(torch.int32).contiguous()
    p = _new_plan(n_rows, offs.numel(), offs.device)
    p.offs = offs
    _lib.check(_lib.load().b200q_moe_pad_plan(offs.data_ptr(), offs.numel(), n_rows, p.padded_offs.data_ptr(),
                                              p.src_of_row.data_ptr(), p.tile_expert.data_ptr(), p.num_tiles.data_ptr(),
                                              _stream()), "b200q_moe_pad_plan")
    return p


def moe_gather(x: torch.Tensor, plan: MoEPlan, quantize: bool, fmt=E4M3):
    """Rows of x into the padded layout: bf16 copy, or (codes, swizzled sf) when quantize.
    Rows past the plan's live tiles are left unwritten."""
    x = _mat(x)
    d = x.shape[1]
    if quantize:
        out = torch.empty(plan.padded_rows, d, dtype=torch.uint8, device=x.device)
        sf = torch.empty(sf_bytes(plan.padded_rows, d // 32), dtype=torch.uint8, device=x.device)
    else:
        out = torch.empty(plan.padded_rows, d, dtype=torch.bfloat16, device=x.device)
        sf = None
    _lib.check(_lib.load().b200q_moe_gather(x.data_ptr(), d, x.stride(0), plan.src_of_row.data_ptr(), plan.num_tiles.data_ptr(),
                                            plan.padded_rows, int(quantize), fmt_of(fmt), out.data_ptr(),
                                            sf.data_ptr() if quantize else None, _stream()), "b200q_moe_gather")
    return (out, sf) if quantize else out


def grouped_gemm_mxfp8(a_codes, a_sf, b_codes, b_sf, plan: MoEPlan, n: int, a_fmt=E4M3, b_fmt=E4M3, out=None):
    """D[padded_rows, n]: row tile i times the (n, K) weight of expert plan.tile_expert[i];
    b_codes is (E * n, K)."""
    rows, k = a_codes.shape
    d = _out(rows, n, a_codes.device, out)
    _lib.check(_lib.load().b200q_grouped_gemm_mxfp8(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                                    fmt_of(b_fmt), b_sf.data_ptr(), plan.tile_expert.data_ptr(),
                                                    plan.num_tiles.data_ptr(), rows, plan.n_experts, n, k, d.data_ptr(),
                                                    d.stride(0), _stream()), "b200q_grouped_gemm_mxfp8")
    return d


def gemm_mxfp8_swiglu(a_codes, a_sf, b_codes, b_sf, a_fmt=E4M3, b_fmt=E4M3):
    """MXFP8 (codes [M, N/2], sf) of silu(gate) * up where [gate | up] = A . B^T and B's rows are in
    the interleaved order of glu_row_map: the GEMM, the activation and the quantization in one kernel."""
    m, k = a_codes.shape
    n = b_codes.shape[0]
    h = torch.empty(m, n // 2, dtype=torch.uint8, device=a_codes.device)
    sf = torch.empty(sf_bytes(m, n // 64), dtype=torch.uint8, device=a_codes.device)
    _lib.check(_lib.load().b200q_gemm_mxfp8_swiglu(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                                   fmt_of(b_fmt), b_sf.data_ptr(), m, n, k, h.data_ptr(), h.stride(0),
                                                   sf.data_ptr(), _stream()), "b200q_gemm_mxfp8_swiglu")
    return h, sf


def grouped_gemm_mxfp8_dgrad(a_codes, a_sf, bt_codes, bt_sf, plan: MoEPlan, n: int, a_fmt=E4M3, b_fmt=E4M3, out=None):
    """D[r] = A[r] . W_e(r) for the padded layout, where the weight stack (E*K, n) was quantized along
    axis 0 as a whole: bt_codes is (n, E*K).  A is (padded_rows, K)."""
    rows, k = a_codes.shape
    d = _out(rows, n, a_codes.device, out)
    _lib.check(_lib.load().b200q_grouped_gemm_mxfp8_dgrad(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), bt_codes.data_ptr(),
                                                          fmt_of(b_fmt), bt_sf.data_ptr(), plan.tile_expert.data_ptr(),
                                                          plan.num_tiles.data_ptr(), rows, plan.n_experts, n, k, d.data_ptr(),
                                                          d.stride(0), _stream()), "b200q_grouped_gemm_mxfp8_dgrad")
    return d


def grouped_gemm_mxfp8_wgrad(at_codes, at_sf, bt_codes, bt_sf, plan: MoEPlan, a_fmt=E4M3, b_fmt=E4M3):
    """D[e] = At[:, rows of e] . Bt[:, rows of e]^T for every expert: at_codes (M, padded_rows), bt_codes
    (N, padded_rows), both quantized along the row dimension of the padded layout.  Returns (E, M, N) bf16."""
    m, rows = at_codes.shape
    n = bt_codes.shape[0]
    e = plan.n_experts
    d = torch.empty(e * m, n, dtype=torch.bfloat16, device=at_codes.device)
    _lib.check(_lib.load().b200q_grouped_gemm_mxfp8_wgrad(at_codes.data_ptr(), fmt_of(a_fmt), at_sf.data_ptr(), bt_codes.data_ptr(),
                                                          fmt_of(b_fmt), bt_sf.data_ptr(), plan.padded_offs.data_ptr(), e, m, n, rows,
                                                          d.data_ptr(), d.stride(0), _stream()), "b200q_grouped_gemm_mxfp8_wgrad")
    return d.view(e, m, n)


def gemm_nvfp4_swiglu(a_codes, a_sf, a_ts, b_codes, b_sf, b_ts):
    """(h bf16 [M, N/2], max|h| fp32 [1]) with h = silu(gate) * up, [gate | up] = A . B^T in NVFP4 and B's
    rows in the interleaved order of glu_row_map: GEMM, activation and the amax pass in one kernel."""
    m = a_codes.shape[0]
    k = a_codes.shape[1] * 2
    n = b_codes.shape[0]
    h = torch.empty(m, n // 2, dtype=torch.bfloat16, device=a_codes.device)
    am = torch.empty(1, dtype=torch.float32, device=a_codes.device)
    _lib.check(_lib.load().b200q_gemm_nvfp4_swiglu(a_codes.data_ptr(), a_sf.data_ptr(), b_codes.data_ptr(), b_sf.data_ptr(),
                                                   a_ts.data_ptr(), b_ts.data_ptr(), m, n, k, h.data_ptr(), h.stride(0), am.data_ptr(),
                                                   _stream()), "b200q_gemm_nvfp4_swiglu")
    return h, am


def grouped_gemm_mxfp8_swiglu(a_codes, a_sf, b_codes, b_sf, plan: MoEPlan, n: int, a_fmt=E4M3, b_fmt=E4M3):
    """Grouped form of gemm_mxfp8_swiglu: b_codes is (E * n, K) with every expert's n = 2I rows interleaved."""
    rows, k = a_codes.shape
    h = torch.empty(rows, n // 2, dtype=torch.uint8, device=a_codes.device)
    sf = torch.empty(sf_bytes(rows, n // 64), dtype=torch.uint8, device=a_codes.device)
    _lib.check(_lib.load().b200q_grouped_gemm_mxfp8_swiglu(a_codes.data_ptr(), fmt_of(a_fmt), a_sf.data_ptr(), b_codes.data_ptr(),
                                                           fmt_of(b_fmt), b_sf.data_ptr(), plan.tile_expert.data_ptr(),
                                                           plan.num_tiles.data_ptr(), rows, plan.n_experts, n, k, h.data_ptr(),
                                                           h.stride(0), sf.data_ptr(), _stream()),
               "b200q_grouped_gemm_mxfp8_swiglu")
    return h, sf


def swiglu(g: torch.Tensor, quantize: bool, fmt=E4M3):
    """g (rows, 2I) bf16 = [gate | up] -> silu(gate) * up as bf16 (rows, I), or MXFP8 (codes, sf)."""
    g = _mat(g)
    rows, i2 = g.shape
    i = i2 // 2
    if quantize:
        out = torch.empty(rows, i, dtype=torch.uint8, device=g.device)
        sf = torch.empty(sf_bytes(rows, i // 32), dtype=torch.uint8, device=g.device)
    else:
        out, sf = torch.empty(rows, i, dtype=torch.bfloat16, device=g.device), None
    _lib.check(_lib.load().b200q_swiglu(g.data_ptr(), rows, i, g.stride(0), int(quantize), fmt_of(fmt), out.data_ptr(),
                                        sf.data_ptr() if quantize else None, _stream()), "b200q_swiglu")
    return (out, sf) if quantize else out


def _dual_outputs(rows: int, cols: int, device):
    return (torch.empty(rows, cols, dtype=torch.uint8, device=device), torch.empty(sf_bytes(rows, cols // 32), dtype=torch.uint8, device=device),
            torch.empty(cols, rows, dtype=torch.uint8, device=device), torch.empty(sf_bytes(cols, rows // 32), dtype=torch.uint8, device=device))


def moe_gather_quantize_dual(x: torch.Tensor, plan: MoEPlan, fmt=E4M3, live_only: bool = False):
    """quantize_mxfp8_dual(moe_gather(x, plan, False)) without the bf16 copy of the gathered rows (all
    padded_rows rows are defined: rows without a source are zero)."""
    x = _mat(x)
    d = x.shape[1]
    cr, sr, cc, sc = _dual_outputs(plan.padded_rows, d, x.device)
    _lib.check(_lib.load().b200q_moe_gather_quantize_dual(x.data_ptr(), d, x.stride(0), plan.src_of_row.data_ptr(), plan.padded_rows,
                                                          fmt_of(fmt), cr.data_ptr(), sr.data_ptr(), cc.data_ptr(), sc.data_ptr(),
                                                          _nt(plan.num_tiles if live_only else None), _stream()), "b200q_moe_gather_quantize_dual")
    return cr, sr, cc, sc


def moe_pair_of_row(plan: MoEPlan) -> torch.Tensor:
    """Inverse of plan.row_of: the routed pair that owns every padded row, -1 for rows nobody owns."""
    inv = torch.empty(plan.padded_rows, dtype=torch.int32, device=plan.row_of.device)
    _lib.check(_lib.load().b200q_moe_pair_of_row(plan.row_of.data_ptr(), plan.row_of.numel(), plan.padded_rows, inv.data_ptr(), _stream()),
               "b200q_moe_pair_of_row")
    return inv


def moe_unpermute_backward_quantize_dual(dout: torch.Tensor, weights: torch.Tensor, pair_of_row: torch.Tensor, fmt=E5M2,
                                         y: torch.Tensor | None = None, row_of: torch.Tensor | None = None):
    """quantize_mxfp8_dual of dy[row] = weights[pair] * dout[pair // k] without writing dy.  With the
    expert outputs `y` (padded rows) and the plan's `row_of`, the same pass also returns the routing
    weights' gradient dw (T, k) fp32 = <dout[token], y[row of the pair]> as a fifth result."""
    dout = _mat(dout)
    d = dout.shape[1]
    w = weights.to(torch.bfloat16).contiguous()
    rows = pair_of_row.numel()
    cr, sr, cc, sc = _dual_outputs(rows, d, dout.device)
    dw = ws = None
    if y is not None:
        y = _mat(y)
        if row_of is None or y.shape != (rows, d):
            raise ValueError("dw needs row_of and y of shape (padded_rows, D)")
        dw = torch.empty(w.shape, dtype=torch.float32, device=dout.device)
        ws = torch.empty(d // 128, rows, dtype=torch.float32, device=dout.device)
    _lib.check(_lib.load().b200q_moe_unpermute_backward_quantize_dual(
        dout.data_ptr(), dout.stride(0), w.data_ptr(), pair_of_row.data_ptr(), w.shape[1], rows, d, fmt_of(fmt), cr.data_ptr(),
        sr.data_ptr(), cc.data_ptr(), sc.data_ptr(), y.data_ptr() if y is not None else None, y.stride(0) if y is not None else 0,
        row_of.data_ptr() if y is not None else None, w.numel(), ws.data_ptr() if ws is not None else None,
        dw.data_ptr() if dw is not None else None, _stream()), "b200q_moe_unpermute_backward_quantize_dual")
    return (cr, sr, cc, sc) if dw is None else (cr, sr, cc, sc, dw)


def swiglu_quantize_dual(g: torch.Tensor, fmt=E4M3, num_tiles: torch.Tensor | None = None):
    """quantize_mxfp8_dual(swiglu(g, False)) without the bf16 h."""
    g = _mat(g)
    rows, i2 = g.shape
    cr, sr, cc, sc = _dual_outputs(rows, i2 // 2, g.device)
    _lib.check(_lib.load().b200q_swiglu_quantize_dual(g.data_ptr(), rows, i2 // 2, g.stride(0), fmt_of(fmt), cr.data_ptr(), sr.data_ptr(),
                                                      cc.data_ptr(), sc.data_ptr(), _nt(num_tiles), _stream()), "b200q_swiglu_quantize_dual")
    return cr, sr, cc, sc


def swiglu_backward_quantize_dual(g: torch.Tensor, dh: torch.Tensor, fmt=E5M2, num_tiles: torch.Tensor | None = None):
    """quantize_mxfp8_dual(swiglu_backward(g, dh)) without the bf16 dg."""
    g, dh = _mat(g), _mat(dh)
    rows, i2 = g.shape
    cr, sr, cc, sc = _dual_outputs(rows, i2, g.device)
    _lib.check(_lib.load().b200q_swiglu_backward_quantize_dual(g.data_ptr(), rows, i2 // 2, g.stride(0), dh.data_ptr(), dh.stride(0),
                                                               fmt_of(fmt), cr.data_ptr(), sr.data_ptr(), cc.data_ptr(), sc.data_ptr(),
                                                               _nt(num_tiles), _stream()), "b200q_swiglu_backward_quantize_dual")
    return cr, sr, cc, sc


def moe_dispatch_peers(x: torch.Tensor, plan: MoEPlan, row_base: torch.Tensor, experts_per_rank: int, peer_codes, peer_sf):
    """Quantize this rank's routed rows (plan over ALL experts) to MXFP8 and store them into their owners'
    buffers; peer_codes / peer_sf are the device pointers of every rank's buffers (own and peer-mapped)."""
    x = _mat(x)
    _lib.check(_lib.load().b200q_moe_dispatch_peers(x.data_ptr(), x.shape[1], x.stride(0), plan.src_of_row.data_ptr(),
                                                    plan.tile_expert.data_ptr(), plan.padded_offs.data_ptr(), plan.num_tiles.data_ptr(),
                                                    plan.padded_rows, row_base.data_ptr(), experts_per_rank, len(peer_codes),
                                                    _ptr_array(peer_codes), _ptr_array(peer_sf), _stream()), "b200q_moe_dispatch_peers")


def moe_zero_pad_rows(plan: MoEPlan, d: int, codes: torch.Tensor, sf: torch.Tensor):
    _lib.check(_lib.load().b200q_moe_zero_pad_rows(plan.src_of_row.data_ptr(), plan.num_tiles.data_ptr(), plan.padded_rows, d,
                                                   codes.data_ptr(), sf.data_ptr(), _stream()), "b200q_moe_zero_pad_rows")


def moe_combine_peers(peer_y, ldy: int, weights: torch.Tensor, pair_peer: torch.Tensor, pair_row: torch.Tensor, d: int):
    """out[t] = sum_j weights[t, j] * y_{pair_peer[t, j]}[pair_row[t, j]], the rows read from their owners' buffers."""
    t, k = weights.shape
    w = weights.to(torch.bfloat16).contiguous()
    out = torch.empty(t, d, dtype=torch.bfloat16, device=w.device)
    _lib.check(_lib.load().b200q_moe_combine_peers(_ptr_array(peer_y), len(peer_y), ldy, w.data_ptr(), pair_peer.data_ptr(),
                                                   pair_row.data_ptr(), t, k, d, out.data_ptr(), _stream()), "b200q_moe_combine_peers")
    return out


def moe_ep_index(all_offs: torch.Tensor, rank: int, top_indices: torch.Tensor, plan: MoEPlan):
    """(row_base (E,), own_offs (E / world,), pair_peer (T*k,), pair_row (T*k,)), all int32: the expert-parallel index
    tables of this rank from the gathered cumulative counts all_offs (world, E) and its own permute plan."""
    world, e = all_offs.shape
    idx = top_indices.contiguous().view(-1)
    n = idx.numel()
    i32 = dict(dtype=torch.int32, device=idx.device)
    row_base, own_offs = torch.empty(e, **i32), torch.empty(e // world, **i32)
    pair_peer, pair_row = torch.empty(n, **i32), torch.empty(n, **i32)
    _lib.check(_lib.load().b200q_moe_ep_index(all_offs.data_ptr(), world, rank, e, idx.data_ptr(), plan.row_of.data_ptr(),
                                              plan.padded_offs.data_ptr(), n, row_base.data_ptr(), own_offs.data_ptr(), pair_peer.data_ptr(),
                                              pair_row.data_ptr(), _stream()), "b200q_moe_ep_index")
    return row_base, own_offs, pair_peer, pair_row


def moe_ep_forward_workspace_bytes(own_padded_rows: int, inter: int) -> int:
    return int(_lib.load().b200q_moe_ep_forward_workspace_bytes(own_padded_rows, inter))


def moe_ep_forward(x: torch.Tensor, top_weights: torch.Tensor, plan: MoEPlan, own: MoEPlan, row_base: torch.Tensor, pair_peer: torch.Tensor,
                   pair_row: torch.Tensor, experts_per_rank: int, rank: int, epoch: int, codes_ptrs, sf_ptrs, y_ptrs, flag_ptrs,
                   w1_codes: torch.Tensor, w1_sf: torch.Tensor, w2_codes: torch.Tensor, w2_sf: torch.Tensor, inter: int,
                   workspace: torch.Tensor | None = None) -> torch.Tensor:
    """The expert-parallel forward after the index tables as one library call (b200q_moe_ep_forward): pad rows zeroed,
    dispatch into the owners' buffers, rendezvous, both grouped GEMMs over the experts this rank owns, rendezvous, combine,
    rendezvous (epochs epoch + 1 .. epoch + 3).  Returns out (T, D) bf16."""
    lib = _lib.load()
    x = _mat(x)
    t, d = x.shape
    k = top_weights.shape[1]
    w = top_weights.to(torch.bfloat16).contiguous()
    need = lib.b200q_moe_ep_forward_workspace_bytes(own.padded_rows, inter)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    out = torch.empty(t, d, dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.b200q_moe_ep_forward(x.data_ptr(), x.stride(0), w.data_ptr(), t, k, d, inter, experts_per_rank, len(codes_ptrs), rank, epoch,
                                        plan.src_of_row.data_ptr(), plan.tile_expert.data_ptr(), plan.padded_offs.data_ptr(),
                                        plan.num_tiles.data_ptr(), plan.padded_rows, row_base.data_ptr(), pair_peer.data_ptr(),
                                        pair_row.data_ptr(), own.src_of_row.data_ptr(), own.tile_expert.data_ptr(), own.num_tiles.data_ptr(),
                                        own.padded_rows, _ptr_array(codes_ptrs), _ptr_array(sf_ptrs), _ptr_array(y_ptrs), _ptr_array(flag_ptrs),
                                        w1_codes.data_ptr(), w1_sf.data_ptr(), w2_codes.data_ptr(), w2_sf.data_ptr(), out.data_ptr(),
                                        workspace.data_ptr(), _stream()), "b200q_moe_ep_forward")
    return out


def peer_barrier(flag_ptrs, rank: int, epoch: int):
    """Stream-ordered rendezvous of the ranks through flag words in peer-mapped memory (bounded wait)."""
    _lib.check(_lib.load().b200q_peer_barrier(_ptr_array(flag_ptrs), len(flag_ptrs), rank, epoch, _stream()), "b200q_peer_barrier")


def moe_scatter_rows_peers(x: torch.Tensor, weights: torch.Tensor | None, pair_peer: torch.Tensor, pair_row: torch.Tensor, k: int,
                           peer_bufs, ldy: int):
    """bf16 rows of x (T, D), scaled by the pairs' weights when given, stored into row pair_row[p] of rank pair_peer[p]'s buffer."""
    x = _mat(x)
    t, d = x.shape
    w = weights.to(torch.bfloat16).contiguous() if weights is not None else None
    _lib.check(_lib.load().b200q_moe_scatter_rows_peers(x.data_ptr(), x.stride(0), w.data_ptr() if w is not None else None,
                                                        pair_peer.data_ptr(), pair_row.data_ptr(), t, k, d, _ptr_array(peer_bufs),
                                                        len(peer_bufs), ldy, _stream()), "b200q_moe_scatter_rows_peers")


def moe_zero_pad_rows_bf16(plan: MoEPlan, buf: torch.Tensor):
    _lib.check(_lib.load().b200q_moe_zero_pad_rows_bf16(plan.src_of_row.data_ptr(), plan.num_tiles.data_ptr(), plan.padded_rows, buf.shape[1],
                                                        buf.data_ptr(), buf.stride(0), _stream()), "b200q_moe_zero_pad_rows_bf16")


def moe_pair_dots_peers(dout: torch.Tensor, peer_y, ldy: int, pair_peer: torch.Tensor, pair_row: torch.Tensor, k: int) -> torch.Tensor:
    """dw (T, k) fp32 = <dout[t], y_owner[row of the pair]>, the rows read from their owners' buffers."""
    dout = _mat(dout)
    t, d = dout.shape
    dw = torch.empty(t, k, dtype=torch.float32, device=dout.device)
    _lib.check(_lib.load().b200q_moe_pair_dots_peers(dout.data_ptr(), dout.stride(0), _ptr_array(peer_y), len(peer_y), ldy, pair_peer.data_ptr(),
                                                     pair_row.data_ptr(), t, k, d, dw.data_ptr(), _stream()), "b200q_moe_pair_dots_peers")
    return dw


def swiglu_backward(g: torch.Tensor, dh: torch.Tensor) -> torch.Tensor:
    """dg (rows, 2I) bf16 from g = [gate | up] (rows, 2I) and dh (rows, I)."""
    g, dh = _mat(g), _mat(dh)
    rows, i2 = g.shape
    dg = torch.empty(rows, i2, dtype=torch.bfloat16, device=g.device)
    _lib.check(_lib.load().b200q_swiglu_backward(g.data_ptr(), rows, i2 // 2, g.stride(0), dh.data_ptr(), dh.stride(0), dg.data_ptr(),
                                                 dg.stride(0), _stream()), "b200q_swiglu_backward")
    return dg


def moe_ffn_forward(x: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor, w1_codes: torch.Tensor, w1_sf: torch.Tensor,
                    w2_codes: torch.Tensor, w2_sf: torch.Tensor, n_experts: int, inter: int, workspace: torch.Tensor | None = None):
    """The expert path of the MoE block in one library call (src/layers/mlp.py:446-477 around grouped_mlp): permute plan,
    gather + MXFP8, grouped GEMM with SwiGLU + MXFP8 epilogue, grouped GEMM, weighted unpermute.  x (T, D) bf16;
    top_idx (T, k) int64; top_w (T, k); w1: the gate / up stack quantized through glu_row_map (E * 2I, D); w2: the down
    stack (E * D, I), both MXFP8 along their last axis.  Returns (out (T, D) bf16, offs (E,) int32: cumulative pairs per
    expert).  `workspace` (uint8, 256-byte aligned, moe_ffn_workspace_bytes long) may be passed to keep the call free of
    allocations besides the results."""
    x = _mat(x)
    t, d = x.shape
    k = top_idx.shape[1]
    w = top_w.to(torch.bfloat16).contiguous()
    idx = top_idx.contiguous()
    lib = _lib.load()
    need = lib.b200q_moe_ffn_workspace_bytes(t, k, d, n_experts, inter)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    elif workspace.numel() < need or workspace.dtype != torch.uint8:
        raise ValueError(f"workspace: {need} bytes of uint8 wanted")
    out = torch.empty(t, d, dtype=torch.bfloat16, device=x.device)
    offs = torch.empty(n_experts, dtype=torch.int32, device=x.device)
    _lib.check(lib.b200q_moe_ffn_forward(x.data_ptr(), x.stride(0), idx.data_ptr(), w.data_ptr(), t, k, d, n_experts, inter,
                                         w1_codes.data_ptr(), w1_sf.data_ptr(), w2_codes.data_ptr(), w2_sf.data_ptr(), out.data_ptr(),
                                         offs.data_ptr(), workspace.data_ptr(), _stream()), "b200q_moe_ffn_forward")
    return out, offs


def moe_ffn_train_forward(x: torch.Tensor, top_w: torch.Tensor, plan: MoEPlan, w1r, w1sr, w2r, w2sr, inter: int):
    """Forward of the trainable expert path in one library call: (out (T, D) bf16, ac, asc, g, hc, hsc, y), the last six
    being what the backward needs (transposed MXFP8 copies of the gathered rows and of h, bf16 g and y)."""
    x = _mat(x)
    t, d = x.shape
    r, e = plan.padded_rows, plan.n_experts
    w = top_w.to(torch.bfloat16).contiguous()
    dev = x.device
    u8 = dict(dtype=torch.uint8, device=dev)
    ac, asc = torch.empty(d, r, **u8), torch.empty(sf_bytes(d, r // 32), **u8)
    hc, hsc = torch.empty(inter, r, **u8), torch.empty(sf_bytes(inter, r // 32), **u8)
    g = torch.empty(r, 2 * inter, dtype=torch.bfloat16, device=dev)
    y = torch.empty(r, d, dtype=torch.bfloat16, device=dev)
    out = torch.empty(t, d, dtype=torch.bfloat16, device=dev)
    lib = _lib.load()
    ws = torch.empty(lib.b200q_moe_ffn_train_forward_workspace_bytes(r, d, inter), **u8)
    _lib.check(lib.b200q_moe_ffn_train_forward(
        x.data_ptr(), x.stride(0), w.data_ptr(), t, w.shape[1], d, e, inter, r, plan.row_of.data_ptr(), plan.src_of_row.data_ptr(),
        plan.tile_expert.data_ptr(), plan.num_tiles.data_ptr(), w1r.data_ptr(), w1sr.data_ptr(), w2r.data_ptr(), w2sr.data_ptr(),
        ac.data_ptr(), asc.data_ptr(), g.data_ptr(), hc.data_ptr(), hsc.data_ptr(), y.data_ptr(), out.data_ptr(), ws.data_ptr(), _stream()),
        "b200q_moe_ffn_train_forward")
    return out, ac, asc, g, hc, hsc, y


def moe_ffn_train_backward(dout: torch.Tensor, top_w: torch.Tensor, plan: MoEPlan, y, g, ac, asc, hc, hsc, w1c, w1sc, w2c, w2sc):
    """Backward of the trainable expert path in one library call: (dx (T, D) bf16, dw (T, k) fp32, dw1 (E, 2I, D) bf16,
    dw2 (E, D, I) bf16)."""
    dout = _mat(dout)
    t, d = dout.shape
    r, e = plan.padded_rows, plan.n_experts
    inter = g.shape[1] // 2
    w = top_w.to(torch.bfloat16).contiguous()
    dev = dout.device
    dx = torch.empty(t, d, dtype=torch.bfloat16, device=dev)
    dw = torch.empty(w.shape, dtype=torch.float32, device=dev)
    dw1 = torch.empty(e, 2 * inter, d, dtype=torch.bfloat16, device=dev)
    dw2 = torch.empty(e, d, inter, dtype=torch.bfloat16, device=dev)
    lib = _lib.load()
    ws = torch.empty(lib.b200q_moe_ffn_train_backward_workspace_bytes(r, d, inter), dtype=torch.uint8, device=dev)
    _lib.check(lib.b200q_moe_ffn_train_backward(
        dout.data_ptr(), dout.stride(0), w.data_ptr(), t, w.shape[1], d, e, inter, r, plan.row_of.data_ptr(), plan.padded_offs.data_ptr(),
        plan.tile_expert.data_ptr(), plan.num_tiles.data_ptr(), y.data_ptr(), g.data_ptr(), ac.data_ptr(), asc.data_ptr(), hc.data_ptr(),
        hsc.data_ptr(), w1c.data_ptr(), w1sc.data_ptr(), w2c.data_ptr(), w2sc.data_ptr(), dx.data_ptr(), dw.data_ptr(), dw1.data_ptr(),
        dw2.data_ptr(), ws.data_ptr(), _stream()), "b200q_moe_ffn_train_backward")
    return dx, dw, dw1, dw2


def moe_ffn_workspace_bytes(tokens: int, top_k: int, d_model: int, n_experts: int, inter: int) -> int:
    return _lib.load().b200q_moe_ffn_workspace_bytes(tokens, top_k, d_model, n_experts, inter)


def moe_unpermute_backward(dout: torch.Tensor, weights: torch.Tensor, y: torch.Tensor | None, plan: MoEPlan, want_dy: bool = True):
    """(dy bf16 (padded_rows, D), dw fp32 (T, k) | None): gradients of moe_unpermute w.r.t. the expert
    outputs and, when y is given, the routing weights.  want_dy=False returns dw alone."""
    dout = _mat(dout)
    t, d = dout.shape
    w = weights.to(torch.bfloat16).contiguous()
    k = w.shape[1]
    dw = torch.empty(t, k, dtype=torch.float32, device=dout.device) if y is not None else None
    if not want_dy:
        _lib.check(_lib.load().b200q_moe_unpermute_backward(dout.data_ptr(), w.data_ptr(), y.data_ptr(), y.stride(0), plan.row_of.data_ptr(),
                                                            plan.src_of_row.data_ptr(), t, k, d, plan.padded_rows, None, dw.data_ptr(),
                                                            _stream()), "b200q_moe_unpermute_backward")
        return dw
    dy = torch.empty(plan.padded_rows, d, dtype=torch.bfloat16, device=dout.device)
    _lib.check(_lib.load().b200q_moe_unpermute_backward(dout.data_ptr(), w.data_ptr(), y.data_ptr() if y is not None else None,
                                                        y.stride(0) if y is not None else 0, plan.row_of.data_ptr(),
                                                        plan.src_of_row.data_ptr(), t, k, d, plan.padded_rows, dy.data_ptr(),
                                                        dw.data_ptr() if dw is not None else None, _stream()),
               "b200q_moe_unpermute_backward")
    return dy, dw


def moe_router_topk(logits: torch.Tensor, k: int, score_fn: str = "softmax", normalize: bool = True, want_probs: bool = True,
                    want_counts: bool = True, select_bias: torch.Tensor | None = None, fp32_out: bool = False):
    """fp32 logits (T, E) -> (top_idx int64 (T, k), top_w (T, k), probs (T, E) | None, expert_counts int32 (E) | None):
    score function, top-k, normalisation, casts and histogram in one launch.  top_w and probs are bf16, or fp32
    when `fp32_out`."""
    if not logits.is_cuda:
        raise RuntimeError("b200q ops need CUDA tensors (no CPU path exists)")
    logits = logits.float().contiguous()
    t, e = logits.shape
    idx = torch.empty(t, k, dtype=torch.int64, device=logits.device)
    odt = torch.float32 if fp32_out else torch.bfloat16
    w = torch.empty(t, k, dtype=odt, device=logits.device)
    probs = torch.empty(t, e, dtype=odt, device=logits.device) if want_probs else None
    counts = torch.empty(e, dtype=torch.int32, device=logits.device) if want_counts else None
    bias = select_bias.float().contiguous() if select_bias is not None else None      # chosen by score + bias, weighted by score
    if bias is not None and bias.shape != (e,):
        raise ValueError("select_bias must have one entry per expert")
    _lib.check(_lib.load().b200q_moe_router_topk(logits.data_ptr(), t, e, k, {"softmax": 0, "sigmoid": 1}[score_fn], int(normalize),
                                                 idx.data_ptr(), w.data_ptr(), probs.data_ptr() if want_probs else None,
                                                 counts.data_ptr() if want_counts else None,
                                                 bias.data_ptr() if bias is not None else None, int(fp32_out), _stream()),
               "b200q_moe_router_topk")
    return idx, w, probs, counts


def moe_unpermute(y: torch.Tensor, weights: torch.Tensor | None, row_of: torch.Tensor, n_tokens: int):
    """out[t] = sum_j weights[t, j] * y[row_of[t*k + j]] (fp32 accumulate, bf16 out); weights None = all ones."""
    k = row_of.numel() // n_tokens
    w = weights.to(torch.bfloat16).contiguous() if weights is not None else None
    d = y.shape[1]
    out = torch.empty(n_tokens, d, dtype=torch.bfloat16, device=y.device)
    _lib.check(_lib.load().b200q_moe_unpermute(y.data_ptr(), y.stride(0), w.data_ptr() if w is not None else None, row_of.data_ptr(), n_tokens, k, d,
                                               out.data_ptr(), _stream()), "b200q_moe_unpermute")
    return out


def device_status() -> None:
    """Raises if a kernel's bounded wait expired since the last check (synchronizes)."""
    _lib.check(_lib.load().b200q_device_status(), "b200q device status")
