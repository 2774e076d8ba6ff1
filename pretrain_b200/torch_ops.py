"""torch custom-op shim over the C-ABI: each kernel entry is a ``torch.library.custom_op`` in
the ``b200q`` namespace with a fake (meta) implementation, so that a model compiled with
``torch.compile`` after the module swap (as the reference's trainer does,
src/training/trainer.py:151,176-177) traces through the quantized linears without graph
breaks.  The real implementations call ``pretrain_b200.ops`` (CUDA only)."""

from __future__ import annotations

from typing import Tuple

import torch

from . import ops

_lib_def = torch.library.custom_op


def _outer_c(x, axis):
    rows, cols = x.shape
    return (rows, cols) if axis == 1 else (cols, rows)


def _sf_numel(outer, nblk, layout):
    if layout == ops.SF_SWIZZLED:
        return ((outer + 127) // 128) * ((nblk + 3) // 4) * 512
    return outer * nblk


@_lib_def("b200q::amax", mutates_args=())
def amax(x: torch.Tensor) -> torch.Tensor:
    return ops.amax(x)


@amax.register_fake
def _(x):
    return x.new_empty(1, dtype=torch.float32)


@_lib_def("b200q::quantize_fp8", mutates_args=())
def quantize_fp8(x: torch.Tensor, fmt: int, axis: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.quantize_fp8(x, fmt, axis)


@quantize_fp8.register_fake
def _(x, fmt, axis):
    outer, c = _outer_c(x, axis)
    return x.new_empty(outer, c, dtype=torch.uint8), x.new_empty(outer, dtype=torch.float32)


@_lib_def("b200q::quantize_fp8_both", mutates_args=())
def quantize_fp8_both(x: torch.Tensor, fmt: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return ops.quantize_fp8_both(x, fmt)


@quantize_fp8_both.register_fake
def _(x, fmt):
    rows, cols = x.shape
    return (x.new_empty(rows, cols, dtype=torch.uint8), x.new_empty(rows, dtype=torch.float32),
            x.new_empty(cols, rows, dtype=torch.uint8), x.new_empty(cols, dtype=torch.float32))


@_lib_def("b200q::quantize_fp8_tensorwise", mutates_args=())
def quantize_fp8_tensorwise(x: torch.Tensor, fmt: int, transpose: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.quantize_fp8_tensorwise(x, fmt, transpose)


@quantize_fp8_tensorwise.register_fake
def _(x, fmt, transpose):
    outer, c = _outer_c(x, 0 if transpose else 1)
    return x.new_empty(outer, c, dtype=torch.uint8), x.new_empty(1, dtype=torch.float32)


@_lib_def("b200q::quantize_int8", mutates_args=())
def quantize_int8(x: torch.Tensor, qmax: int, axis: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.quantize_int8(x, qmax, axis)


@quantize_int8.register_fake
def _(x, qmax, axis):
    outer, c = _outer_c(x, axis)
    return x.new_empty(outer, c, dtype=torch.int8), x.new_empty(outer, dtype=torch.float32)


@_lib_def("b200q::quantize_int8_tensorwise", mutates_args=())
def quantize_int8_tensorwise(x: torch.Tensor, qmax: int, transpose: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.quantize_int8_tensorwise(x, qmax, transpose)


@quantize_int8_tensorwise.register_fake
def _(x, qmax, transpose):
    outer, c = _outer_c(x, 0 if transpose else 1)
    return x.new_empty(outer, c, dtype=torch.int8), x.new_empty(1, dtype=torch.float32)


@_lib_def("b200q::gemm_int8", mutates_args=())
def gemm_int8(a: torch.Tensor, b: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    return ops.gemm_int8(a, b, scale_a, scale_b)


@gemm_int8.register_fake
def _(a, b, scale_a, scale_b):
    return a.new_empty(a.shape[0], b.shape[0], dtype=torch.bfloat16)


@_lib_def("b200q::quantize_mxfp8", mutates_args=())
def quantize_mxfp8(x: torch.Tensor, axis: int, fmt: int, layout: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.quantize_mxfp8(x, axis, fmt, layout)


@quantize_mxfp8.register_fake
def _(x, axis, fmt, layout):
    outer, c = _outer_c(x, axis)
    return x.new_empty(outer, c, dtype=torch.uint8), x.new_empty(_sf_numel(outer, c // 32, layout), dtype=torch.uint8)


@_lib_def("b200q::quantize_mxfp8_dual", mutates_args=())
def quantize_mxfp8_dual(x: torch.Tensor, fmt: int, layout: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return ops.quantize_mxfp8_dual(x, fmt, layout)


@quantize_mxfp8_dual.register_fake
def _(x, fmt, layout):
    rows, cols = x.shape
    return (x.new_empty(rows, cols, dtype=torch.uint8), x.new_empty(_sf_numel(rows, cols // 32, layout), dtype=torch.uint8),
            x.new_empty(cols, rows, dtype=torch.uint8), x.new_empty(_sf_numel(cols, rows // 32, layout), dtype=torch.uint8))


@_lib_def("b200q::quantize_nvfp4", mutates_args=())
def quantize_nvfp4(x: torch.Tensor, axis: int, layout: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return ops.quantize_nvfp4(x, axis, None, layout)


@quantize_nvfp4.register_fake
def _(x, axis, layout):
    outer, c = _outer_c(x, axis)
    return (x.new_empty(outer, c // 2, dtype=torch.uint8), x.new_empty(_sf_numel(outer, c // 16, layout), dtype=torch.uint8),
            x.new_empty(1, dtype=torch.float32))


@_lib_def("b200q::gemm_fp8", mutates_args=())
def gemm_fp8(a: torch.Tensor, a_fmt: int, b: torch.Tensor, b_fmt: int, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    return ops.gemm_fp8(a, a_fmt, b, b_fmt, scale_a, scale_b)


@gemm_fp8.register_fake
def _(a, a_fmt, b, b_fmt, scale_a, scale_b):
    return a.new_empty(a.shape[0], b.shape[0], dtype=torch.bfloat16)


@_lib_def("b200q::gemm_mxfp8", mutates_args=())
def gemm_mxfp8(a: torch.Tensor, a_sf: torch.Tensor, b: torch.Tensor, b_sf: torch.Tensor, a_fmt: int, b_fmt: int) -> torch.Tensor:
    return ops.gemm_mxfp8(a, a_sf, b, b_sf, a_fmt, b_fmt)


@gemm_mxfp8.register_fake
def _(a, a_sf, b, b_sf, a_fmt, b_fmt):
    return a.new_empty(a.shape[0], b.shape[0], dtype=torch.bfloat16)


@_lib_def("b200q::gemm_nvfp4", mutates_args=())
def gemm_nvfp4(a: torch.Tensor, a_sf: torch.Tensor, a_ts: torch.Tensor, b: torch.Tensor, b_sf: torch.Tensor, b_ts: torch.Tensor) -> torch.Tensor:
    return ops.gemm_nvfp4(a, a_sf, a_ts, b, b_sf, b_ts)


@gemm_nvfp4.register_fake
def _(a, a_sf, a_ts, b, b_sf, b_ts):
    return a.new_empty(a.shape[0], b.shape[0], dtype=torch.bfloat16)
