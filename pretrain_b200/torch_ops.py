"""torch custom-op shim over the C-ABI: each kernel entry is a ``torch.library.custom_op`` in
the ``b200q`` namespace with a fake (meta) implementation, so that a model compiled with
``torch.compile`` after the module swap (as the reference's trainer does,
src/training/trainer.py:151,176-177) traces through the quantized linears without graph
breaks.  The real implementations call ``pretrain_b200.ops`` (CUDA only)."""

from __future__ import annotations

import functools
from typing import NamedTuple, Optional, Tuple

import torch

from . import ops

def _lib_def(name: str, mutates_args=()):
    """``torch.library.custom_op`` whose result, called outside the compiler, runs the Python
    implementation directly: the dispatcher's per-call cost (tens of microseconds) would otherwise
    make a step of ~30 small launches host-bound.  Under ``torch.compile`` the registered op (with
    its fake kernel) is what gets traced."""
    def decorate(fn):
        op = torch.library.custom_op(name, mutates_args=mutates_args)(fn)

        @functools.wraps(fn)
        def call(*args, **kwargs):
            if torch.compiler.is_compiling():
                return op(*args, **kwargs)
            return fn(*args, **kwargs)

        call.register_fake = op.register_fake
        call.op = op
        return call
    return decorate


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


@_lib_def("b200q::quantize_nvfp4_both", mutates_args=())
def quantize_nvfp4_both(x: torch.Tensor, layout: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return ops.quantize_nvfp4_both(x, None, layout)


@quantize_nvfp4_both.register_fake
def _(x, layout):
    rows, cols = x.shape
    return (x.new_empty(rows, cols // 2, dtype=torch.uint8), x.new_empty(_sf_numel(rows, cols // 16, layout), dtype=torch.uint8),
            x.new_empty(cols, rows // 2, dtype=torch.uint8), x.new_empty(_sf_numel(cols, rows // 16, layout), dtype=torch.uint8),
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


@_lib_def("b200q::linear_mxfp8", mutates_args=())
def linear_mxfp8(a: torch.Tensor, a_axis: int, b: torch.Tensor, b_axis: int, a_fmt: int, b_fmt: int) -> torch.Tensor:
    return ops.linear_mxfp8(a, a_axis, b, b_axis, a_fmt, b_fmt)


@linear_mxfp8.register_fake
def _(a, a_axis, b, b_axis, a_fmt, b_fmt):
    m = a.shape[0] if a_axis == 1 else a.shape[1]
    n = b.shape[0] if b_axis == 1 else b.shape[1]
    return a.new_empty(m, n, dtype=torch.bfloat16)


@_lib_def("b200q::gemm_nvfp4", mutates_args=())
def gemm_nvfp4(a: torch.Tensor, a_sf: torch.Tensor, a_ts: torch.Tensor, b: torch.Tensor, b_sf: torch.Tensor, b_ts: torch.Tensor) -> torch.Tensor:
    return ops.gemm_nvfp4(a, a_sf, a_ts, b, b_sf, b_ts)


@gemm_nvfp4.register_fake
def _(a, a_sf, a_ts, b, b_sf, b_ts):
    return a.new_empty(a.shape[0], b.shape[0], dtype=torch.bfloat16)


# ---- MoE expert path ---------------------------------------------------------------------------
# The plan travels as a tuple of tensors (a NamedTuple traces through torch.compile; an opaque
# Python object would not); every size is an upper bound known on the host.

class MoEPlan(NamedTuple):
    """Tables of the padded expert-sorted layout (see include/b200q.h); row_of is empty for a plan
    built from already sorted rows."""
    offs: torch.Tensor
    padded_offs: torch.Tensor
    row_of: torch.Tensor
    src_of_row: torch.Tensor
    tile_expert: torch.Tensor
    num_tiles: torch.Tensor

    @property
    def padded_rows(self) -> int:
        return self.src_of_row.shape[0]

    @property
    def n_experts(self) -> int:
        return self.offs.shape[0]


def _plan(n_experts: int, *, padded_offs=None, row_of=None, src_of_row=None, tile_expert=None, num_tiles=None, padded_rows=0):
    p = ops.MoEPlan()
    p.n_experts, p.padded_offs, p.row_of, p.src_of_row, p.tile_expert, p.num_tiles = (
        n_experts, padded_offs, row_of, src_of_row, tile_expert, num_tiles)
    p.offs = None
    p.padded_rows = padded_rows or (src_of_row.shape[0] if src_of_row is not None else tile_expert.shape[0] * 128)
    return p


def _padded_rows(n_pairs: int, n_experts: int) -> int:
    return (n_pairs + n_experts * 127 + 127) // 128 * 128


def _dual_fake(x, rows, cols):
    u8 = dict(dtype=torch.uint8)
    return (x.new_empty(rows, cols, **u8), x.new_empty(_sf_numel(rows, cols // 32, ops.SF_SWIZZLED), **u8),
            x.new_empty(cols, rows, **u8), x.new_empty(_sf_numel(cols, rows // 32, ops.SF_SWIZZLED), **u8))


_T4 = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


@_lib_def("b200q::moe_permute_plan", mutates_args=())
def _moe_permute_plan(top_idx: torch.Tensor, n_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    p = ops.moe_permute_plan(top_idx, n_experts)
    return p.offs, p.padded_offs, p.row_of, p.src_of_row, p.tile_expert, p.num_tiles


@_moe_permute_plan.register_fake
def _(top_idx, n_experts):
    n = top_idx.numel()
    rows = _padded_rows(n, n_experts)
    i32 = dict(dtype=torch.int32)
    return (top_idx.new_empty(n_experts, **i32), top_idx.new_empty(n_experts + 1, **i32), top_idx.new_empty(n, **i32),
            top_idx.new_empty(rows, **i32), top_idx.new_empty(rows // 128, **i32), top_idx.new_empty(1, **i32))


def moe_permute_plan(top_idx: torch.Tensor, n_experts: int) -> MoEPlan:
    return MoEPlan(*_moe_permute_plan(top_idx, n_experts))


@_lib_def("b200q::moe_pad_plan", mutates_args=())
def _moe_pad_plan(offs: torch.Tensor, n_rows: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    p = ops.moe_pad_plan(offs, n_rows)
    return p.padded_offs, p.src_of_row, p.tile_expert, p.num_tiles


@_moe_pad_plan.register_fake
def _(offs, n_rows):
    e = offs.shape[0]
    rows = _padded_rows(n_rows, e)
    i32 = dict(dtype=torch.int32)
    return (offs.new_empty(e + 1, **i32), offs.new_empty(rows, **i32), offs.new_empty(rows // 128, **i32), offs.new_empty(1, **i32))


def moe_pad_plan(offs: torch.Tensor, n_rows: int) -> MoEPlan:
    offs = offs.to(torch.int32).contiguous()
    padded_offs, src_of_row, tile_expert, num_tiles = _moe_pad_plan(offs, n_rows)
    return MoEPlan(offs, padded_offs, offs.new_empty(0), src_of_row, tile_expert, num_tiles)


@_lib_def("b200q::moe_gather_mxfp8", mutates_args=())
def _moe_gather_mxfp8(x: torch.Tensor, src_of_row: torch.Tensor, num_tiles: torch.Tensor, fmt: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.moe_gather(x, _plan(0, src_of_row=src_of_row, num_tiles=num_tiles), True, fmt)


@_moe_gather_mxfp8.register_fake
def _(x, src_of_row, num_tiles, fmt):
    rows, d = src_of_row.shape[0], x.shape[1]
    return x.new_empty(rows, d, dtype=torch.uint8), x.new_empty(_sf_numel(rows, d // 32, ops.SF_SWIZZLED), dtype=torch.uint8)


def moe_gather_mxfp8(x, plan: MoEPlan, fmt: int = ops.E4M3):
    return _moe_gather_mxfp8(x, plan.src_of_row, plan.num_tiles, fmt)


@_lib_def("b200q::moe_gather_quantize_dual", mutates_args=())
def _moe_gather_quantize_dual(x: torch.Tensor, src_of_row: torch.Tensor, fmt: int) -> _T4:
    return ops.moe_gather_quantize_dual(x, _plan(0, src_of_row=src_of_row), fmt)


@_moe_gather_quantize_dual.register_fake
def _(x, src_of_row, fmt):
    return _dual_fake(x, src_of_row.shape[0], x.shape[1])


def moe_gather_quantize_dual(x, plan: MoEPlan, fmt: int = ops.E4M3):
    return _moe_gather_quantize_dual(x, plan.src_of_row, fmt)


@_lib_def("b200q::grouped_gemm_mxfp8", mutates_args=())
def _grouped_gemm_mxfp8(a: torch.Tensor, a_sf: torch.Tensor, b: torch.Tensor, b_sf: torch.Tensor, tile_expert: torch.Tensor,
                        num_tiles: torch.Tensor, n_experts: int, n: int, a_fmt: int, b_fmt: int, form: int) -> torch.Tensor:
    plan = _plan(n_experts, tile_expert=tile_expert, num_tiles=num_tiles)
    fn = ops.grouped_gemm_mxfp8 if form == 0 else ops.grouped_gemm_mxfp8_dgrad
    return fn(a, a_sf, b, b_sf, plan, n, a_fmt, b_fmt)


@_grouped_gemm_mxfp8.register_fake
def _(a, a_sf, b, b_sf, tile_expert, num_tiles, n_experts, n, a_fmt, b_fmt, form):
    return a.new_empty(a.shape[0], n, dtype=torch.bfloat16)


def grouped_gemm_mxfp8(a, a_sf, b, b_sf, plan: MoEPlan, n: int, a_fmt: int = ops.E4M3, b_fmt: int = ops.E4M3):
    """Row tile i of A times the (n, K) weight of its expert; b is (E * n, K)."""
    return _grouped_gemm_mxfp8(a, a_sf, b, b_sf, plan.tile_expert, plan.num_tiles, plan.n_experts, n, a_fmt, b_fmt, 0)


def grouped_gemm_mxfp8_dgrad(a, a_sf, bt, bt_sf, plan: MoEPlan, n: int, a_fmt: int = ops.E4M3, b_fmt: int = ops.E4M3):
    """The same with the weight stack quantized along axis 0 as a whole: bt is (n, E * K)."""
    return _grouped_gemm_mxfp8(a, a_sf, bt, bt_sf, plan.tile_expert, plan.num_tiles, plan.n_experts, n, a_fmt, b_fmt, 1)


@_lib_def("b200q::grouped_gemm_mxfp8_swiglu", mutates_args=())
def _grouped_gemm_mxfp8_swiglu(a: torch.Tensor, a_sf: torch.Tensor, b: torch.Tensor, b_sf: torch.Tensor, tile_expert: torch.Tensor,
                               num_tiles: torch.Tensor, n_experts: int, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.grouped_gemm_mxfp8_swiglu(a, a_sf, b, b_sf, _plan(n_experts, tile_expert=tile_expert, num_tiles=num_tiles), n)


@_grouped_gemm_mxfp8_swiglu.register_fake
def _(a, a_sf, b, b_sf, tile_expert, num_tiles, n_experts, n):
    rows = a.shape[0]
    return a.new_empty(rows, n // 2, dtype=torch.uint8), a.new_empty(_sf_numel(rows, n // 64, ops.SF_SWIZZLED), dtype=torch.uint8)


def grouped_gemm_mxfp8_swiglu(a, a_sf, b, b_sf, plan: MoEPlan, n: int):
    return _grouped_gemm_mxfp8_swiglu(a, a_sf, b, b_sf, plan.tile_expert, plan.num_tiles, plan.n_experts, n)


@_lib_def("b200q::grouped_gemm_mxfp8_wgrad", mutates_args=())
def _grouped_gemm_mxfp8_wgrad(at: torch.Tensor, at_sf: torch.Tensor, bt: torch.Tensor, bt_sf: torch.Tensor, padded_offs: torch.Tensor,
                              a_fmt: int, b_fmt: int) -> torch.Tensor:
    return ops.grouped_gemm_mxfp8_wgrad(at, at_sf, bt, bt_sf, _plan(padded_offs.shape[0] - 1, padded_offs=padded_offs, padded_rows=at.shape[1]),
                                        a_fmt, b_fmt)


@_grouped_gemm_mxfp8_wgrad.register_fake
def _(at, at_sf, bt, bt_sf, padded_offs, a_fmt, b_fmt):
    return at.new_empty(padded_offs.shape[0] - 1, at.shape[0], bt.shape[0], dtype=torch.bfloat16)


def grouped_gemm_mxfp8_wgrad(at, at_sf, bt, bt_sf, plan: MoEPlan, a_fmt: int = ops.E4M3, b_fmt: int = ops.E4M3):
    """(E, M, N): per expert, At[:, its rows] . Bt[:, its rows]^T."""
    return _grouped_gemm_mxfp8_wgrad(at, at_sf, bt, bt_sf, plan.padded_offs, a_fmt, b_fmt)


@_lib_def("b200q::swiglu", mutates_args=())
def swiglu(g: torch.Tensor) -> torch.Tensor:
    return ops.swiglu(g, False)


@swiglu.register_fake
def _(g):
    return g.new_empty(g.shape[0], g.shape[1] // 2, dtype=torch.bfloat16)


@_lib_def("b200q::swiglu_mxfp8", mutates_args=())
def swiglu_mxfp8(g: torch.Tensor, fmt: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.swiglu(g, True, fmt)


@swiglu_mxfp8.register_fake
def _(g, fmt):
    rows, i = g.shape[0], g.shape[1] // 2
    return g.new_empty(rows, i, dtype=torch.uint8), g.new_empty(_sf_numel(rows, i // 32, ops.SF_SWIZZLED), dtype=torch.uint8)


@_lib_def("b200q::swiglu_quantize_dual", mutates_args=())
def swiglu_quantize_dual(g: torch.Tensor, fmt: int) -> _T4:
    return ops.swiglu_quantize_dual(g, fmt)


@swiglu_quantize_dual.register_fake
def _(g, fmt):
    return _dual_fake(g, g.shape[0], g.shape[1] // 2)


@_lib_def("b200q::swiglu_backward_quantize_dual", mutates_args=())
def swiglu_backward_quantize_dual(g: torch.Tensor, dh: torch.Tensor, fmt: int) -> _T4:
    return ops.swiglu_backward_quantize_dual(g, dh, fmt)


@swiglu_backward_quantize_dual.register_fake
def _(g, dh, fmt):
    return _dual_fake(g, g.shape[0], g.shape[1])


@_lib_def("b200q::moe_unpermute", mutates_args=())
def moe_unpermute(y: torch.Tensor, weights: Optional[torch.Tensor], row_of: torch.Tensor, n_tokens: int) -> torch.Tensor:
    return ops.moe_unpermute(y, weights, row_of, n_tokens)


@moe_unpermute.register_fake
def _(y, weights, row_of, n_tokens):
    return y.new_empty(n_tokens, y.shape[1], dtype=torch.bfloat16)


@_lib_def("b200q::moe_ffn_forward", mutates_args=())
def moe_ffn_forward(x: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor, w1_codes: torch.Tensor, w1_sf: torch.Tensor,
                    w2_codes: torch.Tensor, w2_sf: torch.Tensor, n_experts: int, inter: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The expert path in one library call: (out (T, D) bf16, offs (E,) int32)."""
    return ops.moe_ffn_forward(x, top_idx, top_w, w1_codes, w1_sf, w2_codes, w2_sf, n_experts, inter)


@moe_ffn_forward.register_fake
def _(x, top_idx, top_w, w1_codes, w1_sf, w2_codes, w2_sf, n_experts, inter):
    return x.new_empty(x.shape[0], x.shape[1], dtype=torch.bfloat16), x.new_empty(n_experts, dtype=torch.int32)


_T7 = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


@_lib_def("b200q::moe_ffn_train_forward", mutates_args=())
def moe_ffn_train_forward(x: torch.Tensor, top_w: torch.Tensor, w1r: torch.Tensor, w1sr: torch.Tensor, w2r: torch.Tensor, w2sr: torch.Tensor,
                          n_experts: int, inter: int, row_of: torch.Tensor, src_of_row: torch.Tensor, tile_expert: torch.Tensor,
                          num_tiles: torch.Tensor) -> _T7:
    """Forward of the trainable expert path in one library call: (out, ac, asc, g, hc, hsc, y)."""
    plan = _plan(n_experts, row_of=row_of, src_of_row=src_of_row, tile_expert=tile_expert, num_tiles=num_tiles)
    return ops.moe_ffn_train_forward(x, top_w, plan, w1r, w1sr, w2r, w2sr, inter)


@moe_ffn_train_forward.register_fake
def _(x, top_w, w1r, w1sr, w2r, w2sr, n_experts, inter, row_of, src_of_row, tile_expert, num_tiles):
    r, d = src_of_row.shape[0], x.shape[1]
    u8, bf = dict(dtype=torch.uint8), dict(dtype=torch.bfloat16)
    return (x.new_empty(x.shape[0], d, **bf), x.new_empty(d, r, **u8), x.new_empty(ops.sf_bytes(d, r // 32), **u8),
            x.new_empty(r, 2 * inter, **bf), x.new_empty(inter, r, **u8), x.new_empty(ops.sf_bytes(inter, r // 32), **u8),
            x.new_empty(r, d, **bf))


@_lib_def("b200q::moe_ffn_train_backward", mutates_args=())
def moe_ffn_train_backward(dout: torch.Tensor, top_w: torch.Tensor, y: torch.Tensor, g: torch.Tensor, ac: torch.Tensor, asc: torch.Tensor,
                           hc: torch.Tensor, hsc: torch.Tensor, w1c: torch.Tensor, w1sc: torch.Tensor, w2c: torch.Tensor, w2sc: torch.Tensor,
                           n_experts: int, padded_offs: torch.Tensor, row_of: torch.Tensor, tile_expert: torch.Tensor,
                           num_tiles: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward of the trainable expert path in one library call: (dx, dw fp32, dw1, dw2)."""
    plan = _plan(n_experts, padded_offs=padded_offs, row_of=row_of, tile_expert=tile_expert, num_tiles=num_tiles, padded_rows=y.shape[0])
    return ops.moe_ffn_train_backward(dout, top_w, plan, y, g, ac, asc, hc, hsc, w1c, w1sc, w2c, w2sc)


@moe_ffn_train_backward.register_fake
def _(dout, top_w, y, g, ac, asc, hc, hsc, w1c, w1sc, w2c, w2sc, n_experts, padded_offs, row_of, tile_expert, num_tiles):
    d, inter = dout.shape[1], g.shape[1] // 2
    bf = dict(dtype=torch.bfloat16)
    return (dout.new_empty(dout.shape[0], d, **bf), dout.new_empty(top_w.shape, dtype=torch.float32),
            dout.new_empty(n_experts, 2 * inter, d, **bf), dout.new_empty(n_experts, d, inter, **bf))


@_lib_def("b200q::moe_unpermute_backward_quantize_dual", mutates_args=())
def moe_unpermute_backward_quantize_dual(dout: torch.Tensor, weights: torch.Tensor, row_of: torch.Tensor, padded_rows: int, fmt: int,
                                         y: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Both MXFP8 copies of dy[row] = w[pair] * dout[token of the pair] and dw[pair] = <dout[token], y[row]> (fp32)."""
    plan = _plan(0, row_of=row_of, padded_rows=padded_rows)
    return ops.moe_unpermute_backward_quantize_dual(dout, weights, ops.moe_pair_of_row(plan), fmt, y=y, row_of=row_of)


@moe_unpermute_backward_quantize_dual.register_fake
def _(dout, weights, row_of, padded_rows, fmt, y):
    return (*_dual_fake(dout, padded_rows, dout.shape[1]), dout.new_empty(weights.shape, dtype=torch.float32))


@_lib_def("b200q::moe_router_topk", mutates_args=())
def moe_router_topk(logits: torch.Tensor, k: int, score_fn: str, normalize: bool, select_bias: Optional[torch.Tensor],
                    fp32_out: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    idx, w, probs, _ = ops.moe_router_topk(logits, k, score_fn, normalize, want_counts=False, select_bias=select_bias,
                                           fp32_out=fp32_out)
    return idx, w, probs


@moe_router_topk.register_fake
def _(logits, k, score_fn, normalize, select_bias, fp32_out=False):
    t, e = logits.shape
    odt = torch.float32 if fp32_out else torch.bfloat16
    return (logits.new_empty(t, k, dtype=torch.int64), logits.new_empty(t, k, dtype=odt), logits.new_empty(t, e, dtype=odt))


_GLU_ROW_MAPS: dict = {}


@_lib_def("b200q::quantize_mxfp8_glu_rows", mutates_args=())
def quantize_mxfp8_glu_rows(w: torch.Tensor, n_groups: int, inter: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row-wise MXFP8 of a (n_groups * 2 * inter, K) weight with every group's gate and up rows interleaved in
    blocks of 32, the order the SwiGLU epilogue expects."""
    key = (n_groups, inter, str(w.device))
    if key not in _GLU_ROW_MAPS:
        _GLU_ROW_MAPS[key] = ops.glu_row_map(n_groups, inter, w.device)
    return ops.quantize_mxfp8_rowmap(w, _GLU_ROW_MAPS[key])


@quantize_mxfp8_glu_rows.register_fake
def _(w, n_groups, inter):
    rows, k = w.shape
    return w.new_empty(rows, k, dtype=torch.uint8), w.new_empty(_sf_numel(rows, k // 32, ops.SF_SWIZZLED), dtype=torch.uint8)


@_lib_def("b200q::moe_unpermute_backward", mutates_args=())
def _moe_unpermute_backward(dout: torch.Tensor, weights: torch.Tensor, y: torch.Tensor, row_of: torch.Tensor,
                            src_of_row: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    plan = _plan(0, row_of=row_of, src_of_row=src_of_row)
    return ops.moe_unpermute_backward(dout, weights, y, plan)


@_moe_unpermute_backward.register_fake
def _(dout, weights, y, row_of, src_of_row):
    return dout.new_empty(src_of_row.shape[0], dout.shape[1], dtype=torch.bfloat16), dout.new_empty(weights.shape, dtype=torch.float32)


def moe_unpermute_backward(dout, weights, y, plan: MoEPlan):
    """(dy bf16 (padded_rows, D) with zero pad rows, dw fp32 (T, k)): the gradients of moe_unpermute."""
    return _moe_unpermute_backward(dout, weights, y, plan.row_of, plan.src_of_row)
