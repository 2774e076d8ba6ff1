"""Quantized linear: ``_gemm``, ``QuantizedLinearFn`` and ``QuantLinear`` with the signatures and
conventions of src/quant/linear.py, on the sm_100a kernels.

``_gemm(a, b, ...)`` always receives a (rows, C) and b (C, cols) — possibly as transposed views
(``w.t()``, ``g.t()``) — and scales run along C.  Same-family quantized operands go to the fused
tensor-core GEMM; mixed or one-sided formats are fake-quantized and multiplied in high
precision, as the reference does (src/quant/linear.py:27-56)."""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import torch_ops as T
from ..ops import SF_NATURAL, SF_SWIZZLED, fmt_of
from . import cache as weight_cache
from .config import QuantConfig
from .fp8 import _k_major, fake_quantize_fp8, fp8_gemm
from .int8 import fake_quantize_int8, int8_gemm
from .mx import mxfp8_gemm, nvfp4_gemm
from .utils import is_fp8, is_int8s, is_mxfp8, is_nvfp4, is_quantized, str_to_dtype_fp8, str_to_qmax_int8s

_E2M1_LUT = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _fake_quant_block(x: torch.Tensor, fmt: str, contraction_dim: int) -> torch.Tensor:
    """dequant(quant(x)) for a block-scaled format, blocks along ``contraction_dim`` of the 2-D
    view x; quantization on the CUDA kernels, dequantization in plain torch."""
    m, axis = _k_major(x, contraction_dim)
    if is_mxfp8(fmt):
        dt = str_to_dtype_fp8(fmt)
        codes, sf = T.quantize_mxfp8(m, axis, fmt_of(dt), SF_NATURAL)
        outer, c = codes.shape
        scale = torch.exp2(sf.view(outer, c // 32).float() - 127.0)
        deq = (codes.view(dt).float().view(outer, c // 32, 32) * scale.unsqueeze(-1)).view(outer, c)
    else:
        packed, sf, ts = T.quantize_nvfp4(m, axis, SF_NATURAL)
        outer, c = packed.shape[0], packed.shape[1] * 2
        lut = torch.tensor(_E2M1_LUT + [-v for v in _E2M1_LUT], device=x.device)
        vals = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1).view(outer, c)
        eff = sf.view(outer, c // 16).view(torch.float8_e4m3fn).float() * ts
        deq = (vals.view(outer, c // 16, 16) * eff.unsqueeze(-1)).view(outer, c)
    deq = deq.to(x.dtype)                       # (outer, C)
    return deq if contraction_dim == 1 else deq.t()


def _fake_quant(x, fmt, dim, contraction_dim):
    """dequant(quant(x)) for one operand in its format; identity for passthrough formats."""
    if is_fp8(fmt):
        return fake_quantize_fp8(x, str_to_dtype_fp8(fmt), dim=dim)
    if is_mxfp8(fmt) or is_nvfp4(fmt):
        return _fake_quant_block(x, fmt, contraction_dim)
    if is_int8s(fmt):
        return fake_quantize_int8(x, str_to_qmax_int8s(fmt), dim=dim)
    return x


def _gemm(a, b, a_fmt, b_fmt, out_dtype, rowwise=False):
    """`a @ b` dispatched on the operands' format families."""
    if is_fp8(a_fmt) and is_fp8(b_fmt):
        return fp8_gemm(a, b, out_dtype, str_to_dtype_fp8(a_fmt), str_to_dtype_fp8(b_fmt), rowwise=rowwise)
    if is_mxfp8(a_fmt) and is_mxfp8(b_fmt):
        return mxfp8_gemm(a, b, out_dtype, str_to_dtype_fp8(a_fmt), str_to_dtype_fp8(b_fmt))
    if is_nvfp4(a_fmt) and is_nvfp4(b_fmt):
        return nvfp4_gemm(a, b, out_dtype)
    if is_int8s(a_fmt) and is_int8s(b_fmt):
        return int8_gemm(a, b, out_dtype, str_to_qmax_int8s(a_fmt), str_to_qmax_int8s(b_fmt), rowwise=rowwise)
    if is_quantized(a_fmt):
        a = _fake_quant(a, a_fmt, -1 if rowwise else None, 1)
    if is_quantized(b_fmt):
        b = _fake_quant(b, b_fmt, 0 if rowwise else None, 0)
    return (a @ b).to(out_dtype)


def _mx_training_formats(cfg: QuantConfig):
    """(act, weight, grad) fp8 dtypes when every operand of the three GEMMs is MXFP8 and both uses
    of the output gradient share a format (the ``mxfp8`` recipe); None otherwise."""
    d = cfg.dtype
    if not all(is_mxfp8(d[k]) for k in ("act", "weight", "input_grad", "weight_grad")):
        return None
    if str_to_dtype_fp8(d["input_grad"]) != str_to_dtype_fp8(d["weight_grad"]):
        return None
    return str_to_dtype_fp8(d["act"]), str_to_dtype_fp8(d["weight"]), str_to_dtype_fp8(d["input_grad"])


def _fp8_training_formats(cfg: QuantConfig):
    """(act, weight, grad) fp8 dtypes when the three GEMMs are row-wise-scaled FP8 and both uses of the
    output gradient share a format (the ``fp8`` recipe with ``granularity: rowwise``); None otherwise."""
    d = cfg.dtype
    if cfg.scaling["granularity"] != "rowwise" or not all(is_fp8(d[k]) for k in ("act", "weight", "input_grad", "weight_grad")):
        return None
    if d["input_grad"] != d["weight_grad"]:
        return None
    fa, fw, fg = (str_to_dtype_fp8(d[k]) for k in ("act", "weight", "input_grad"))
    e5 = torch.float8_e5m2
    if (fa == e5 and fw == e5) or (fg == e5 and fw == e5) or (fg == e5 and fa == e5):
        return None                       # fp8_gemm wants at least one e4m3 operand in every GEMM
    return fa, fw, fg


def _nv_training(cfg: QuantConfig) -> bool:
    """Every operand of the three GEMMs is NVFP4 (the ``nvfp4`` recipe)."""
    return all(is_nvfp4(cfg.dtype[k]) for k in ("act", "weight", "input_grad", "weight_grad"))


def _both_nv_weight(weight: torch.Tensor, w: torch.Tensor):
    """Both NVFP4 copies of the weight under one tensor scale, kept on the parameter until it is written again."""
    return weight_cache.cached(weight, "nv", (w.dtype,), lambda: T.quantize_nvfp4_both(w.detach(), SF_SWIZZLED))


def _both_fp8_weight(weight: torch.Tensor, w: torch.Tensor, fmt: torch.dtype):
    """Per-row and per-column FP8 copies of the weight, kept on the parameter until it is written again
    (see ``pretrain_b200.quant.cache`` for what "written" covers)."""
    return weight_cache.cached(weight, "fp8", (w.dtype, fmt), lambda: T.quantize_fp8_both(w.detach(), fmt_of(fmt)))


def _dual_mx_weight(weight: torch.Tensor, w: torch.Tensor, fmt: torch.dtype):
    """Both MXFP8 copies of the weight (along in_features for fprop, along out_features for
    dgrad).  Outside torch.compile they are kept on the parameter until it is next written, so a
    step made of several micro-batches quantizes each weight once (the reference re-quantizes in
    every forward and again in every backward, src/quant/linear.py:73-76,98)."""
    return weight_cache.cached(weight, "mx", (w.dtype, fmt), lambda: T.quantize_mxfp8_dual(w.detach(), fmt_of(fmt), SF_SWIZZLED))


class QuantizedLinearFn(torch.autograd.Function):
    """y = x . W^T (+ bias) with the three GEMMs of a linear layer quantized per ``cfg``:
    fprop act x weight, dgrad input_grad x weight, wgrad weight_grad x act
    (src/quant/linear.py:59-115).

    When all of them are MXFP8 and a backward pass will follow, every tensor is quantized ONCE,
    in both directions by one kernel, and the codes - not the bf16 tensors - are what is saved
    for backward: three quantize passes per layer and step instead of six, half the saved bytes,
    the same results bit for bit."""

    @staticmethod
    def forward(ctx, x, weight, bias, cfg: QuantConfig, recording=None, dp=None):
        # `recording`: whether autograd is recording this call (grad mode is always off in here, and
        # needs_input_grad only mirrors requires_grad); QuantLinear passes it, direct callers with the
        # reference's four arguments leave it None = "assume a backward pass may follow"
        # `dp`: a pretrain_b200.dist.DataParallelGrad - the weight gradient is summed over the ranks of its group inside
        # the wgrad GEMM (epilogue stores into the owners' staging buffers) instead of by a collective afterwards
        ctx.n_inputs = 4 if recording is None else (5 if dp is None else 6)
        ctx.dp = dp
        dev = x.device.type
        compute_dtype = torch.get_autocast_dtype(dev) if torch.is_autocast_enabled(dev) else x.dtype
        rowwise = cfg.scaling["granularity"] == "rowwise"
        x2d = x.reshape(-1, x.shape[-1]).to(compute_dtype)
        w = weight.to(compute_dtype)
        mx = _mx_training_formats(cfg)
        ctx.mx = (mx is not None and compute_dtype == torch.bfloat16 and any(ctx.needs_input_grad[:2]) and recording is not False
                  and x2d.shape[0] % 32 == 0 and x2d.shape[1] % 32 == 0 and w.shape[0] % 32 == 0)
        ctx.f8 = ctx.nv = False
        if ctx.mx:
            fa, fw, _ = mx
            xr, xsr, xc, xsc = T.quantize_mxfp8_dual(x2d, fmt_of(fa), SF_SWIZZLED)
            wr, wsr, wc, wsc = _dual_mx_weight(weight, w, fw)
            y = T.gemm_mxfp8(xr, xsr, wr, wsr, fmt_of(fa), fmt_of(fw))
            if bias is not None:
                y = y + bias.to(compute_dtype)
            ctx.save_for_backward(xc, xsc, wc, wsc)
            ctx.cfg, ctx.has_bias = cfg, bias is not None
            ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, weight.dtype
            return y.reshape(*x.shape[:-1], weight.shape[0])
        ctx.nv = (_nv_training(cfg) and compute_dtype == torch.bfloat16 and any(ctx.needs_input_grad[:2]) and recording is not False
                  and x2d.shape[0] % 32 == 0 and x2d.shape[1] % 32 == 0 and w.shape[0] % 32 == 0)
        if ctx.nv:
            # NVFP4 the same way: each tensor's maximum taken once, both directions quantized under that one tensor scale,
            # the transposed codes (not the bf16 tensors) saved for backward, the weight's two copies kept on the parameter
            xr, xsr, xc, xsc, tx = T.quantize_nvfp4_both(x2d, SF_SWIZZLED)          # (M, K/2) | (K, M/2)
            wr, wsr, wc, wsc, tw = _both_nv_weight(weight, w)                        # (N, K/2) | (K, N/2)
            y = T.gemm_nvfp4(xr, xsr, tx, wr, wsr, tw)
            if bias is not None:
                y = y + bias.to(compute_dtype)
            ctx.save_for_backward(xc, xsc, tx, wc, wsc, tw)
            ctx.cfg, ctx.has_bias = cfg, bias is not None
            ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, weight.dtype
            return y.reshape(*x.shape[:-1], weight.shape[0])
        f8 = _fp8_training_formats(cfg)
        ctx.f8 = (f8 is not None and compute_dtype == torch.bfloat16 and any(ctx.needs_input_grad[:2]) and recording is not False
                  and x2d.shape[0] % 16 == 0 and w.shape[0] % 16 == 0 and x2d.shape[1] % 16 == 0
                  and max(x2d.shape[1], w.shape[0]) <= 8192)
        if ctx.f8:
            # the same idea for row-wise FP8: each tensor quantized per row and per column in two reads
            # (not three), codes and scales saved for backward, the weight's copies kept on the parameter
            fa, fw, _ = f8
            xr, xsr, xc, xsc = T.quantize_fp8_both(x2d, fmt_of(fa))            # (M, K) | (K, M)
            wr, wsr, wc, wsc = _both_fp8_weight(weight, w, fw)                 # (N, K) | (K, N)
            y = T.gemm_fp8(xr, fmt_of(fa), wr, fmt_of(fw), xsr, wsr)
            if bias is not None:
                y = y + bias.to(compute_dtype)
            ctx.save_for_backward(xc, xsc, wc, wsc)
            ctx.cfg, ctx.has_bias = cfg, bias is not None
            ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, weight.dtype
            return y.reshape(*x.shape[:-1], weight.shape[0])
        y = _gemm(x2d, w.t(), cfg.dtype["act"], cfg.dtype["weight"], compute_dtype, rowwise)
        if bias is not None:
            y = y + bias.to(compute_dtype)
        ctx.save_for_backward(x2d, w)
        ctx.cfg, ctx.has_bias = cfg, bias is not None
        ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, weight.dtype
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.mx:
            xc, xsc, wc, wsc = ctx.saved_tensors          # x^T codes (K, M), w^T codes (K, N)
            fa, fw, fg = (fmt_of(t) for t in _mx_training_formats(ctx.cfg))
            g = grad_out.reshape(-1, grad_out.shape[-1]).to(torch.bfloat16)             # (M, N)
            gr, gsr, gc, gsc = T.quantize_mxfp8_dual(g, fg, SF_SWIZZLED)
            dx = T.gemm_mxfp8(gr, gsr, wc, wsc, fg, fw) if ctx.needs_input_grad[0] else None    # (M, N) . (K, N)^T
            dw = None
            if ctx.needs_input_grad[1]:
                if ctx.dp is not None:
                    dw = ctx.dp.wgrad(gc, gsc, xc, xsc, fg, fa)                                 # summed over the ranks in the GEMM
                else:
                    dw = T.gemm_mxfp8(gc, gsc, xc, xsc, fg, fa)                                 # (N, M) . (K, M)^T
            db = g.sum(dim=0).to(ctx.w_dtype) if ctx.has_bias else None
            if db is not None and ctx.dp is not None:
                db = ctx.dp.reduce_small(db)
            return (dx.reshape(*ctx.x_shape).to(ctx.x_dtype) if dx is not None else None,
                    dw.to(ctx.w_dtype) if dw is not None else None, db, None, None, None)[:ctx.n_inputs]
        if ctx.nv:
            xc, xsc, tx, wc, wsc, tw = ctx.saved_tensors   # x^T (K, M/2), w^T (K, N/2) with their tensor scales
            g = grad_out.reshape(-1, grad_out.shape[-1]).to(torch.bfloat16)                     # (M, N)
            gr, gsr, gc, gsc, tg = T.quantize_nvfp4_both(g, SF_SWIZZLED)                        # (M, N/2) | (N, M/2)
            dx = T.gemm_nvfp4(gr, gsr, tg, wc, wsc, tw) if ctx.needs_input_grad[0] else None    # (M, N) . (K, N)^T
            dw = T.gemm_nvfp4(gc, gsc, tg, xc, xsc, tx) if ctx.needs_input_grad[1] else None    # (N, M) . (K, M)^T
            db = g.sum(dim=0).to(ctx.w_dtype) if ctx.has_bias else None
            if ctx.dp is not None:                   # no fused form for this format: a plain sum over the ranks
                dw = ctx.dp.reduce_small(dw) if dw is not None else None
                db = ctx.dp.reduce_small(db) if db is not None else None
            return (dx.reshape(*ctx.x_shape).to(ctx.x_dtype) if dx is not None else None,
                    dw.to(ctx.w_dtype) if dw is not None else None, db, None, None, None)[:ctx.n_inputs]
        if ctx.f8:
            xc, xsc, wc, wsc = ctx.saved_tensors          # x^T codes (K, M) + per-column scales, w^T codes (K, N)
            fa, fw, fg = (fmt_of(t) for t in _fp8_training_formats(ctx.cfg))
            g = grad_out.reshape(-1, grad_out.shape[-1]).to(torch.bfloat16)             # (M, N)
            gr, gsr, gc, gsc = T.quantize_fp8_both(g, fg)                                # (M, N) | (N, M)
            dx = T.gemm_fp8(gr, fg, wc, fw, gsr, wsc) if ctx.needs_input_grad[0] else None      # (M, N) . (K, N)^T
            dw = T.gemm_fp8(gc, fg, xc, fa, gsc, xsc) if ctx.needs_input_grad[1] else None      # (N, M) . (K, M)^T
            db = g.sum(dim=0).to(ctx.w_dtype) if ctx.has_bias else None
            if ctx.dp is not None:                   # no fused form for this format: a plain sum over the ranks
                dw = ctx.dp.reduce_small(dw) if dw is not None else None
                db = ctx.dp.reduce_small(db) if db is not None else None
            return (dx.reshape(*ctx.x_shape).to(ctx.x_dtype) if dx is not None else None,
                    dw.to(ctx.w_dtype) if dw is not None else None, db, None, None, None)[:ctx.n_inputs]
        x2d, w = ctx.saved_tensors
        cfg = ctx.cfg
        dt = x2d.dtype
        g = grad_out.reshape(-1, grad_out.shape[-1]).to(dt)          # (M, N)
        rowwise = cfg.scaling["granularity"] == "rowwise"
        dx = _gemm(g, w, cfg.dtype["input_grad"], cfg.dtype["weight"], dt, rowwise)        # (M,N)@(N,K)
        dw = _gemm(g.t(), x2d, cfg.dtype["weight_grad"], cfg.dtype["act"], dt, rowwise)    # (N,M)@(M,K)
        db = g.sum(dim=0).to(ctx.w_dtype) if ctx.has_bias else None
        if ctx.dp is not None:                       # formats without the fused form: a plain sum over the ranks
            dw = ctx.dp.reduce_small(dw)
            db = ctx.dp.reduce_small(db) if db is not None else None
        return (dx.reshape(*ctx.x_shape).to(ctx.x_dtype), dw.to(ctx.w_dtype), db, None, None, None)[:ctx.n_inputs]


class QuantLinear(nn.Module):
    """Drop-in for ``nn.Linear``: same parameter names and shapes (state-dict compatible), keeps
    the high-precision master weight; only the GEMMs run quantized."""

    def __init__(self, in_features, out_features, bias, cfg: QuantConfig):
        super().__init__()
        self.in_features, self.out_features, self.cfg = in_features, out_features, cfg
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None

    @classmethod
    def from_linear(cls, linear: nn.Linear, cfg: QuantConfig) -> "QuantLinear":
        q = cls(linear.in_features, linear.out_features, linear.bias is not None, cfg)
        with torch.no_grad():
            q.weight.copy_(linear.weight)
            if linear.bias is not None:
                q.bias.copy_(linear.bias)
        return q.to(linear.weight.device, linear.weight.dtype)

    def forward(self, x):
        packed = getattr(self, "_packed", None)
        if packed is not None:
            y = self._forward_packed(x, packed)
            if y is not None:
                return y
        dp = getattr(self, "_dp", None)
        if dp is not None:
            return QuantizedLinearFn.apply(x, self.weight, self.bias, self.cfg, torch.is_grad_enabled(), dp)
        return QuantizedLinearFn.apply(x, self.weight, self.bias, self.cfg, torch.is_grad_enabled())

    def enable_data_parallel(self, group=None) -> "QuantLinear":
        """Data-parallel training of this layer inside one NVLink domain: every rank runs the layer on its own shard of the
        batch, and ``weight.grad`` (and ``bias.grad``) come out already SUMMED over the ranks of `group` - for the all-MXFP8
        rule the sum happens inside the wgrad GEMM (its epilogue stores each block into the staging buffer of the rank that
        owns those rows; an owner adds its slots; an all-gather hands every rank the whole gradient), for other rules by a
        plain all-reduce.  Replaces the gradient all-reduce a DDP wrapper would do for this parameter."""
        from ..dist import DataParallelGrad
        self._dp = DataParallelGrad(self.out_features, self.in_features, group)
        return self

    # ---- pre-quantized weight (pretrain_b200.quant.wire) ---------------------------------------------------------
    def attach_quantized(self, qw) -> None:
        """Use a pre-quantized form of this layer's weight (a ``wire.QuantizedWeight`` in the rule's weight format, shape
        (out_features, in_features)) for forwards that record no gradient: the activation is quantized, the weight is
        not.  It is dropped as soon as the master weight is written again (version counter) or ``post_step`` runs;
        it is an attribute, not a buffer, so the state dict stays that of ``nn.Linear``."""
        from . import wire
        want = wire._CANON.get(self.cfg.dtype["weight"], self.cfg.dtype["weight"])
        if qw.format != want:
            raise ValueError(f"layer quantizes its weight as {want!r}, the container entry is {qw.format!r}")
        if tuple(qw.shape) != (self.out_features, self.in_features):
            raise ValueError(f"container entry has shape {tuple(qw.shape)}, the layer's weight is {(self.out_features, self.in_features)}")
        self._packed = (qw.to(self.weight.device), self.weight._version)

    def _forward_packed(self, x, packed):
        qw, version = packed
        if version != self.weight._version:
            self._packed = None                     # the master weight moved on
            return None
        d = self.cfg.dtype
        if (torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad)) or not x.is_cuda:
            return None                             # training goes through the autograd function
        if torch.is_autocast_enabled("cuda"):
            out_dtype = torch.get_autocast_dtype("cuda")
        else:
            out_dtype = x.dtype
        x2d = x.reshape(-1, x.shape[-1]).to(torch.bfloat16)
        if is_mxfp8(d["act"]) and qw.format.startswith("mxfp8"):
            fa, fw = fmt_of(str_to_dtype_fp8(d["act"])), fmt_of(str_to_dtype_fp8(d["weight"]))
            ca, sfa = T.quantize_mxfp8(x2d, 1, fa, SF_SWIZZLED)
            y = T.gemm_mxfp8(ca, sfa, qw.codes, qw.sf, fa, fw)
        elif is_nvfp4(d["act"]) and qw.format == "nvfp4":
            pa, sfa, ta = T.quantize_nvfp4(x2d, 1, SF_SWIZZLED)
            y = T.gemm_nvfp4(pa, sfa, ta, qw.codes, qw.sf, qw.tensor_scale)
        elif is_fp8(d["act"]) and qw.format.startswith("fp8") and self.cfg.scaling["granularity"] == "rowwise":
            fa, fw = fmt_of(str_to_dtype_fp8(d["act"])), fmt_of(str_to_dtype_fp8(d["weight"]))
            ca, sa = T.quantize_fp8(x2d, fa, 1)
            y = T.gemm_fp8(ca, fa, qw.codes, fw, sa, qw.scales)
        else:
            return None
        y = y if out_dtype == torch.bfloat16 else y.to(out_dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*x.shape[:-1], self.out_features)

    @torch.no_grad()
    def post_step(self):
        """Called by the training loop after every optimizer step (src/training/trainer.py:367 through
        src/model/transformer.py:144-147): the weight has just been written, so its cached quantized copies go -
        also when the optimizer wrote through ``.data``, which the version counter does not see."""
        weight_cache.invalidate(self.weight)
        self._packed = None

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
