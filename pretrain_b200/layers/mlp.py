"""MoE expert FFN on the sm_100a kernels, behind the call signatures of the reference's
``src/layers/mlp.py``: ``grouped_mlp`` (:55-100), ``MoERouter`` (:248-302) and
``SparseMoEBlock`` (:324-494).

The two bf16 ``torch._grouped_mm`` calls of the reference become ragged MXFP8 grouped GEMMs on
the tensor cores; the permute is a stable counting sort (same row order as the reference's
``sort(stable=True)``) whose gather is fused with the MXFP8 quantization; SwiGLU is fused with
the re-quantization of the hidden activations; the unpermute is a gather-reduce in fp32.
``SparseMoEBlock`` is trainable (bias-free SwiGLU experts): its backward runs the four grouped
backward GEMMs in MXFP8 as well.  ``grouped_mlp`` on its own is forward-only.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .. import torch_ops as T
from ..quant import cache as weight_cache


def silu_glu(gate, up):
    """SwiGLU, the gated activation of the reference's default experts (src/layers/activation.py:80-81)."""
    return F.silu(gate) * up


def _powlu(x, m: float = 3.0):
    """PowLU with m = 3: x * x^(m / (sqrt(x) + 1)) * sigmoid(x) for x > 0 and x^2 * sigmoid(x) otherwise.  The positive
    branch is evaluated on max(x, 1-where-negative) so that the unselected side stays finite for autograd."""
    base = torch.where(x > 0, x, torch.ones_like(x))
    pos = x * base ** (m / (base.sqrt() + 1.0)) * torch.sigmoid(x)
    return torch.where(x > 0, pos, x * x * torch.sigmoid(x))


# The reference's activation registries (src/layers/activation.py): unary activations, their squares
# ("relu2", ...), and for gated blocks unary(gate) * up, plus the gate-only forms.  Only SwiGLU has a
# fused kernel here; the others run as torch element-wise ops between the two quantized GEMMs.
_UNARY = {"relu": F.relu, "gelu": F.gelu, "silu": F.silu, "leaky_relu": lambda x: F.leaky_relu(x, 0.01)}
UNGATED_ACTIVATIONS = dict(_UNARY)
UNGATED_ACTIVATIONS.update({name + "2": (lambda x, f=f: f(x) ** 2) for name, f in _UNARY.items()})
GATED_ACTIVATIONS = {name: (lambda g, u, f=f: f(g) * u) for name, f in UNGATED_ACTIVATIONS.items()}
GATED_ACTIVATIONS.update({"silu": silu_glu, "bilinear": lambda g, u: g * u, "bilinear2": lambda g, u: g ** 2 * u,
                          "powlu": lambda g, u: _powlu(g) * u})


def _add_bias(y, b):
    return y if b is None else y + (b if b.ndim == 1 else b.unsqueeze(-2))


def gated_mlp(x, w_gate_up, w_down, act_fn, b_gate_up=None, b_down=None):
    """down(act(gate, up)) with (gate, up) = chunk(x @ w_gate_up^T): the reference's unquantized helper
    (src/layers/mlp.py:7-30), kept as plain matmuls."""
    gate, up = _add_bias(x @ w_gate_up.mT, b_gate_up).chunk(2, dim=-1)
    return _add_bias(act_fn(gate, up) @ w_down.mT, b_down)


def ungated_mlp(x, w_up, w_down, act_fn, b_up=None, b_down=None):
    """down(act(x @ w_up^T)), the ungated counterpart (src/layers/mlp.py:33-52)."""
    return _add_bias(act_fn(_add_bias(x @ w_up.mT, b_up)) @ w_down.mT, b_down)


MOE_ROUTER_SCORE_FNS = {
    "softmax": lambda logits: logits.softmax(dim=-1),
    "sigmoid": lambda logits: logits.sigmoid(),
}


def _wants_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


E4M3, E5M2, SWZ = ops.E4M3, ops.E5M2, ops.SF_SWIZZLED


class _ExpertFFN(torch.autograd.Function):
    """Permuted SwiGLU expert FFN + weighted unpermute with a backward pass, all GEMMs in MXFP8 on
    the padded expert-sorted layout (the reference differentiates src/layers/mlp.py:446-477 through
    torch._grouped_mm with autograd).

    forward : gather -> quantize x both ways -> GEMM 1 -> SwiGLU -> quantize h both ways -> GEMM 2
              -> weighted unpermute; the weights are quantized both ways too (row-wise for fprop,
              transposed for dgrad).
    backward: dy = w * dout (and dw = <dout, y>) -> dgrad 2 / wgrad 2 -> SwiGLU backward -> dgrad 1 /
              wgrad 1 -> sum over the k slots.  Activations and weights E4M3, gradients E5M2, as in
              the `mxfp8` recipe."""

    @staticmethod
    def forward(ctx, x, top_w, w_in, w_down, w1r, w1sr, w1c, w1sc, w2r, w2sr, w2c, w2sc, *plan_tensors):
        # w1* / w2*: both MXFP8 copies of the weight stacks, (E*2I, D) | (D, E*2I) and (E*D, I) | (I, E*D)
        plan = T.MoEPlan(*plan_tensors)
        t, d = x.shape
        e, n1, _ = w_in.shape
        inter = n1 // 2
        # every element-wise step hands its result to the both-directions quantizer inside one kernel
        if inter % 128 == 0:
            # the five launches below as one library call (issued back to back, each may be scheduled while its predecessor drains)
            out, ac, asc, g, hc, hsc, y = T.moe_ffn_train_forward(x, top_w.to(torch.bfloat16), w1r, w1sr, w2r, w2sr, e, inter, plan.row_of,
                                                                  plan.src_of_row, plan.tile_expert, plan.num_tiles)
        else:
            ar, asr, ac, asc = T.moe_gather_quantize_dual(x, plan, E4M3)                      # (R, D) | (D, R), pad rows zero
            g = T.grouped_gemm_mxfp8(ar, asr, w1r, w1sr, plan, n1)                    # (R, 2I) bf16, kept for backward
            hr, hsr, hc, hsc = T.quantize_mxfp8_dual(T.swiglu(g), E4M3, SWZ)
            y = T.grouped_gemm_mxfp8(hr, hsr, w2r, w2sr, plan, d)                     # (R, D) bf16
            out = T.moe_unpermute(y, top_w, plan.row_of, t)
        ctx.save_for_backward(top_w, ac, asc, g, hc, hsc, w1c, w1sc, w2c, w2sc, y, *plan_tensors)
        ctx.shapes = (t, d, e, inter, top_w.shape[1])
        ctx.dtypes = (x.dtype, top_w.dtype, w_in.dtype, w_down.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        top_w, ac, asc, g, hc, hsc, w1c, w1sc, w2c, w2sc, y, *plan_tensors = ctx.saved_tensors
        plan = T.MoEPlan(*plan_tensors)
        t, d, e, inter, k = ctx.shapes
        dout = dout.reshape(t, d).to(torch.bfloat16)
        xd, twd, w1d, w2d = ctx.dtypes
        if inter % 128 == 0:
            dx, dw, dw1, dw2 = T.moe_ffn_train_backward(dout.contiguous(), top_w.to(torch.bfloat16), y, g, ac, asc, hc, hsc, w1c, w1sc, w2c,
                                                        w2sc, e, plan.padded_offs, plan.row_of, plan.tile_expert, plan.num_tiles)
            return (dx.to(xd), dw.to(twd), dw1.to(w1d), dw2.to(w2d)) + (None,) * (8 + len(plan_tensors))
        dyr, dysr, dyc, dysc, dw = T.moe_unpermute_backward_quantize_dual(                      # dw (T, k) fp32
            dout, top_w.to(torch.bfloat16), plan.row_of, plan.padded_rows, E5M2, y)
        dh = T.grouped_gemm_mxfp8_dgrad(dyr, dysr, w2c, w2sc, plan, inter, E5M2, E4M3)         # (R, I)
        dw2 = T.grouped_gemm_mxfp8_wgrad(dyc, dysc, hc, hsc, plan, E5M2, E4M3)                 # (E, D, I)
        dgr, dgsr, dgc, dgsc = T.swiglu_backward_quantize_dual(g, dh, E5M2)                    # of dg (R, 2I)
        da = T.grouped_gemm_mxfp8_dgrad(dgr, dgsr, w1c, w1sc, plan, d, E5M2, E4M3)             # (R, D)
        dw1 = T.grouped_gemm_mxfp8_wgrad(dgc, dgsc, ac, asc, plan, E5M2, E4M3)                 # (E, 2I, D)
        dx = T.moe_unpermute(da, None, plan.row_of, t)                                           # sum over the k slots
        return (dx.to(xd), dw.to(twd), dw1.to(w1d), dw2.to(w2d)) + (None,) * (8 + len(plan_tensors))


class _GroupedLinearFn(torch.autograd.Function):
    """y[r] = a[r] @ w[expert of r]^T on the padded expert-sorted layout, MXFP8 forward and backward: one piece of
    the general trainable expert path (any activation, biases), which keeps the element-wise steps between its two
    grouped linears in plain torch under autograd.  With `gather` the input is the (T, D) token matrix and the
    permute is fused into the quantizer; otherwise it is a (padded_rows, K) matrix."""

    @staticmethod
    def forward(ctx, a, w, gather, wr, wsr, wc, wsc, *plan_tensors):
        # wr .. wsc: both MXFP8 copies of the (E*N, K) weight matrix (_expert_weight_copies)
        plan = T.MoEPlan(*plan_tensors)
        e, n, k = w.shape
        if gather:
            ar, asr, ac, asc = T.moe_gather_quantize_dual(a, plan, E4M3)
        else:
            ar, asr, ac, asc = T.quantize_mxfp8_dual(a, E4M3, SWZ)
        ctx.save_for_backward(ac, asc, wc, wsc, *plan_tensors)
        ctx.gather, ctx.tokens, ctx.k = gather, a.shape[0], k
        ctx.dtypes = (a.dtype, w.dtype)
        return T.grouped_gemm_mxfp8(ar, asr, wr, wsr, plan, n)

    @staticmethod
    def backward(ctx, dy):
        ac, asc, wc, wsc, *plan_tensors = ctx.saved_tensors
        plan = T.MoEPlan(*plan_tensors)
        gr, gsr, gc, gsc = T.quantize_mxfp8_dual(dy.to(torch.bfloat16).contiguous(), E5M2, SWZ)
        da = T.grouped_gemm_mxfp8_dgrad(gr, gsr, wc, wsc, plan, ctx.k, E5M2, E4M3)            # (R, K)
        dw = T.grouped_gemm_mxfp8_wgrad(gc, gsc, ac, asc, plan, E5M2, E4M3)                  # (E, N, K)
        if ctx.gather:
            da = T.moe_unpermute(da, None, plan.row_of, ctx.tokens)                           # sum over the k slots
        return (da.to(ctx.dtypes[0]), dw.to(ctx.dtypes[1]), None) + (None,) * (4 + len(plan_tensors))


class _UnpermuteFn(torch.autograd.Function):
    """out[t] = sum_j w[t, j] * y[row of (t, j)] with its backward (dy scattered into the padded layout, pad rows
    zero; dw = <dout, y>)."""

    @staticmethod
    def forward(ctx, y, top_w, tokens, *plan_tensors):
        plan = T.MoEPlan(*plan_tensors)
        ctx.save_for_backward(y, top_w, *plan_tensors)
        return T.moe_unpermute(y, top_w.to(torch.bfloat16), plan.row_of, tokens)

    @staticmethod
    def backward(ctx, dout):
        y, top_w, *plan_tensors = ctx.saved_tensors
        dy, dw = T.moe_unpermute_backward(dout.to(torch.bfloat16).contiguous(), top_w.to(torch.bfloat16), y, T.MoEPlan(*plan_tensors))
        return (dy.to(y.dtype), dw.to(top_w.dtype), None) + (None,) * len(plan_tensors)


def _trainable_widths(d: int, width: int, inter: int) -> None:
    if d % 128 or width % 128 or inter % 32:
        raise NotImplementedError("the backward of the MXFP8 expert path needs d_model and the first layer's width "
                                  "(2 * intermediate_size when gated) to be multiples of 128 and intermediate_size "
                                  "a multiple of 32")


def _expert_ffn_general(x, w_in, w_down, b_in, b_down, act_fn, gated, plan):
    """The trainable expert path for any activation and optional biases, up to the expert outputs in the padded
    layout: grouped linear (permute fused) -> (+ bias, activation in torch) -> grouped linear -> (+ bias).  Pad rows
    carry no gradient: their output gradient is zero, so whatever the biases put there never reaches a weight."""
    g = _GroupedLinearFn.apply(x, w_in, True, *_expert_weight_copies(w_in, "dual"), *plan)
    rows = _expert_of_padded_row(plan)
    if b_in is not None:
        g = g + b_in.to(g.dtype)[rows]
    # rows past the live tiles are never written by the grouped GEMMs (forward or backward): select them away, so
    # that neither their contents nor the gradients that come back for them reach a weight or a bias
    live = (plan.tile_expert >= 0).repeat_interleave(128).unsqueeze(-1)
    g = torch.where(live, g, torch.zeros((), dtype=g.dtype, device=g.device))
    h = act_fn(*g.chunk(2, dim=-1)) if gated else act_fn(g)
    y = _GroupedLinearFn.apply(h.contiguous(), w_down, False, *_expert_weight_copies(w_down, "dual"), *plan)
    if b_down is not None:
        y = y + b_down.to(y.dtype)[rows]
    return y


def _quantize_expert_weights(w: torch.Tensor):
    """(E, out, in) weight stack -> MXFP8 codes (E*out, in) + swizzled scales, blocks along `in`."""
    e, n, k = w.shape
    if n % 128:
        # scale-factor tiles hold 128 rows and must not straddle experts: pad every expert's rows
        w = torch.cat([w, w.new_zeros(e, 128 - n % 128, k)], dim=1)
    return T.quantize_mxfp8(w.reshape(-1, k), 1, E4M3, SWZ)


def _expert_of_padded_row(plan) -> torch.Tensor:
    return plan.tile_expert.clamp_min(0).repeat_interleave(128).long()


_ROW_MAPS: dict = {}


def _glu_row_map(e: int, inter: int, device) -> torch.Tensor:
    key = (e, inter, str(device))
    if key not in _ROW_MAPS:
        _ROW_MAPS[key] = ops.glu_row_map(e, inter, device)
    return _ROW_MAPS[key]


def _grouped_ffn_padded(a, sfa, plan, w_in, w_down, act_fn, gated, b_in=None, b_down=None, out=None):
    """Both grouped GEMMs and the activation on the padded layout; returns (padded_rows, D_out) bf16
    (written into `out` when given and the expert width needs no padding)."""
    n1, n2 = w_in.shape[1], w_down.shape[1]
    wq2, wsf2 = _expert_weight_copies(w_down, "rows")
    e = w_in.shape[0]
    if gated and act_fn is silu_glu and b_in is None and n1 % 128 == 0:
        # SwiGLU and the re-quantization run in the first GEMM's epilogue: the weights are stored with
        # gate and up rows interleaved so that a thread of the epilogue holds a whole block of h
        wq1, wsf1 = _expert_weight_copies(w_in, "glu")
        hq, hsf = T.grouped_gemm_mxfp8_swiglu(a, sfa, wq1, wsf1, plan, n1)
    else:
        wq1, wsf1 = _expert_weight_copies(w_in, "rows")
        h = T.grouped_gemm_mxfp8(a, sfa, wq1, wsf1, plan, wq1.shape[0] // e)[:, :n1]
        if b_in is not None:
            h = h + b_in.to(h.dtype)[_expert_of_padded_row(plan)]
        if gated and act_fn is silu_glu:
            hq, hsf = T.swiglu_mxfp8(h, E4M3)                 # fused silu(gate)*up + MXFP8
        else:
            act = act_fn(*h.chunk(2, dim=-1)) if gated else act_fn(h)
            hq, hsf = T.quantize_mxfp8(act.contiguous(), 1, E4M3, SWZ)
    if out is not None and n2 % 128 == 0:       # straight into the caller's buffer (expert-parallel combine reads it in place)
        return ops.grouped_gemm_mxfp8(hq, hsf, wq2, wsf2, plan, wq2.shape[0] // e, out=out)
    out = T.grouped_gemm_mxfp8(hq, hsf, wq2, wsf2, plan, wq2.shape[0] // e)[:, :n2]
    if b_down is not None:
        out = out + b_down.to(out.dtype)[_expert_of_padded_row(plan)]
    return out


def grouped_mlp(x, w_in, w_down, act_fn, offs, gated, row_expert_ids=None, b_in=None, b_down=None):
    """Dropless MoE expert FFN over expert-sorted rows.

    x is (R, D) with rows grouped by expert and ``offs`` the (E,) int32 cumulative end offsets
    (offs[-1] == R); weights are (E, out, in); empty groups are fine; biases, when given, are
    (E, out) and are added per row.  Returns (R, D_out), rows in the input order (computed in MXFP8 with bf16
    outputs, returned in the autocast dtype or else x's dtype).  With inputs that
    require grad the general trainable path runs (MXFP8 backward GEMMs; widths as _trainable_widths says).
    """
    if not x.is_cuda:
        raise RuntimeError("grouped_mlp runs on the B200 kernels only (no CPU path)")
    r = x.shape[0]
    e = w_in.shape[0]
    in_dtype = x.dtype
    plan = T.moe_pad_plan(offs, r)
    # padded row of every input row (the inverse of the plan's src_of_row): its expert's padded start + its rank there
    rows = torch.arange(r, device=x.device)
    expert = torch.searchsorted(plan.offs.long(), rows, right=True).clamp_max(e - 1)
    starts = torch.cat([plan.offs.new_zeros(1), plan.offs[:-1]]).long()
    row_of = plan.padded_offs.long()[expert] + rows - starts[expert]
    if _wants_grad(x, w_in, w_down, b_in, b_down):
        _trainable_widths(x.shape[1], w_in.shape[1], w_down.shape[2])
        plan = plan._replace(row_of=row_of.to(torch.int32))          # one "slot" per row: the backward of the gather sums over it
        out_p = _expert_ffn_general(x.to(torch.bfloat16), w_in, w_down, b_in, b_down, act_fn, gated, plan)
    else:
        x, w_in, w_down = x.to(torch.bfloat16), w_in.to(torch.bfloat16), w_down.to(torch.bfloat16)
        a, sfa = T.moe_gather_mxfp8(x, plan)
        out_p = _grouped_ffn_padded(a, sfa, plan, w_in, w_down, act_fn, gated, b_in, b_down)
    # back to the caller's unpadded row order, in the dtype the reference's matmuls would return: the autocast
    # dtype when autocast is on, else the input's (tests/fast/layers/test_mlp.py:1065-1084)
    out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else in_dtype
    return out_p[row_of].to(out_dtype)


def _cached(param: torch.Tensor, slot: str, key, make):
    """Quantized copies of a weight, kept on the parameter until it is written again (pretrain_b200.quant.cache)."""
    return weight_cache.cached(param, slot[len("_b200q_"):] if slot.startswith("_b200q_") else slot, key, make)


def _expert_weight_copies(param: torch.Tensor, kind: str):
    """Quantized copies of an expert weight stack (E, out, in), kept on the parameter until it is next written
    (a step made of several micro-batches, or evaluation, quantizes each stack once; under torch.compile they are
    recomputed in the graph).  kind "dual": (codes, sf) along `in` and along `out` of the (E*out, in) matrix, for
    fprop / dgrad; "glu": row-wise with gate / up rows interleaved for the SwiGLU epilogue; "rows": row-wise."""
    e, n, k = param.shape

    def make():
        w = param.detach().to(torch.bfloat16)
        if kind == "dual":
            return T.quantize_mxfp8_dual(w.reshape(e * n, k), E4M3, SWZ)
        if kind == "glu":
            return T.quantize_mxfp8_glu_rows(w.reshape(e * n, k), e, n // 2)
        return _quantize_expert_weights(w)

    return _cached(param, kind, kind, make)


def _ffn_flops(d_model: int, d_ff: int, gated: bool, bias: bool) -> int:
    """Forward FLOPs per token of one feed-forward network: 2 FLOPs per weight (three d x d_ff matrices when gated,
    two otherwise) plus one add per bias entry - the accounting of src/layers/mlp.py:152-162."""
    return (6 if gated else 4) * d_model * d_ff + _ffn_bias_terms(d_model, d_ff, gated, bias)


def _ffn_bias_terms(d_model: int, d_ff: int, gated: bool, bias: bool) -> int:
    return ((2 if gated else 1) * d_ff + d_model) if bias else 0


def _ffn_parameters(d_model: int, d_ff: int, gated: bool, bias: bool) -> int:
    return (3 if gated else 2) * d_model * d_ff + _ffn_bias_terms(d_model, d_ff, gated, bias)


class DenseMLPBlock(nn.Module):
    """Dense feed-forward block with the reference's constructor and (out, None) contract
    (src/layers/mlp.py:103-150): ``down_proj(act(gate, up))`` with ``(gate, up) =
    chunk(gate_up_proj(x))`` when gated, ``down_proj(act(up_proj(x)))`` otherwise.  Its Linears are
    plain ``nn.Linear`` that ``apply_quantization`` swaps for ``QuantLinear`` like any other.

    When both projections carry an all-MXFP8 or all-NVFP4 rule, the block is SwiGLU without biases
    and no gradient is being recorded, the forward is three launches shorter than the composition:
    the gate/up GEMM applies SwiGLU in its epilogue and hands the down projection MXFP8 codes, or
    bf16 h plus its absolute maximum for NVFP4 (b200q_gemm_{mxfp8,nvfp4}_swiglu)."""

    def __init__(self, d_model, *, intermediate_size, activation="silu", gated=True, bias=False, dropout=0.0):
        super().__init__()
        registry = GATED_ACTIVATIONS if gated else UNGATED_ACTIVATIONS
        self.gated = gated
        self.act_fn = registry[activation]
        if gated:
            self.gate_up_proj = nn.Linear(d_model, 2 * intermediate_size, bias=bias)
        else:
            self.up_proj = nn.Linear(d_model, intermediate_size, bias=bias)
        self.down_proj = nn.Linear(intermediate_size, d_model, bias=bias)
        self.dropout = nn.Dropout(dropout)

    @classmethod
    def compute_flops(cls, d_model, *, intermediate_size, gated=True, bias=False, **_):
        return _ffn_flops(d_model, intermediate_size, gated, bias)

    @classmethod
    def compute_parameters(cls, d_model, *, intermediate_size, gated=True, bias=False, active=False, **_):
        return _ffn_parameters(d_model, intermediate_size, gated, bias)

    def _fused_kind(self, x):
        """'mxfp8' / 'nvfp4' when the epilogue form applies to this call, else None."""
        from ..quant.linear import QuantLinear
        from ..quant.utils import is_mxfp8, is_nvfp4
        if not (self.gated and self.act_fn is silu_glu and x.is_cuda and x.dtype == torch.bfloat16):
            return None
        if torch.compiler.is_compiling():        # the cached weight copies are Python-side state: the composition traces cleanly
            return None
        up, down = self.gate_up_proj, self.down_proj
        if not (isinstance(up, QuantLinear) and isinstance(down, QuantLinear)) or up.bias is not None or down.bias is not None:
            return None
        if _wants_grad(x, up.weight, down.weight) or up.weight.dtype != torch.bfloat16 and not torch.is_autocast_enabled("cuda"):
            return None
        inter, d = down.in_features, up.in_features
        if inter % 64 or d % 32:
            return None
        fmts = [m.cfg.dtype[o] for m in (up, down) for o in ("act", "weight")]
        if all(is_mxfp8(f) and not f.endswith("e5m2") for f in fmts):
            return "mxfp8"
        if all(is_nvfp4(f) for f in fmts):
            return "nvfp4"
        return None

    def forward(self, x):
        kind = self._fused_kind(x)
        if kind is None:
            if self.gated:
                gate, up = self.gate_up_proj(x).chunk(2, dim=-1)
                hidden = self.act_fn(gate, up)
            else:
                hidden = self.act_fn(self.up_proj(x))
            return self.dropout(self.down_proj(hidden)), None
        w_gu, w_d = self.gate_up_proj.weight, self.down_proj.weight
        inter = self.down_proj.in_features
        x2 = x.reshape(-1, x.shape[-1])
        row_map = _glu_row_map(1, inter, x.device)
        if kind == "mxfp8":
            gq = _cached(w_gu, "_b200q_glu", "mx", lambda: ops.quantize_mxfp8_rowmap(w_gu.detach().to(torch.bfloat16), row_map))
            dq = _cached(w_d, "_b200q_row", "mx", lambda: ops.quantize_mxfp8(w_d.detach().to(torch.bfloat16), 1))
            xq, xsf = ops.quantize_mxfp8(x2, 1)
            hq, hsf = ops.gemm_mxfp8_swiglu(xq, xsf, *gq)
            out = ops.gemm_mxfp8(hq, hsf, *dq)
        else:
            gq = _cached(w_gu, "_b200q_glu", "nv", lambda: ops.quantize_nvfp4_rowmap(w_gu.detach().to(torch.bfloat16), row_map))
            dq = _cached(w_d, "_b200q_row", "nv", lambda: ops.quantize_nvfp4(w_d.detach().to(torch.bfloat16), 1))
            px, sx, tx = ops.quantize_nvfp4(x2, 1)
            h, h_amax = ops.gemm_nvfp4_swiglu(px, sx, tx, *gq)
            ph, sh, th = ops.quantize_nvfp4(h, 1, h_amax)
            out = ops.gemm_nvfp4(ph, sh, th, *dq)
        return self.dropout(out.reshape(*x.shape[:-1], out.shape[-1])), None


class ExpertBias(nn.Module):
    """Auxiliary-loss-free load-balancing bias (src/layers/mlp.py:182-216): added to the gating scores for the
    top-k selection only, nudged toward uniform load by a fixed-rate sign rule; an fp32 buffer, not a parameter."""

    def __init__(self, n_experts: int, update_rate: float = 0.001):
        super().__init__()
        self.update_rate = update_rate
        self.register_buffer("bias", torch.zeros(n_experts))

    def _apply(self, fn, recurse=True):
        result = super()._apply(fn, recurse)
        if self.bias.dtype != torch.float32:
            self.bias = self.bias.float()
        return result

    def forward(self, scores):
        return scores + self.bias

    @torch.no_grad()
    def update(self, expert_counts):
        err = expert_counts.float().mean() - expert_counts.float()
        self.bias += self.update_rate * err.sign()

    @classmethod
    def compute_flops(cls, n_experts: int) -> int:
        return n_experts                   # one add per expert score

    @classmethod
    def compute_parameters(cls, n_experts: int) -> int:
        return 0                           # a buffer, not a parameter


class ExpertLoad(nn.Module):
    """Tokens per expert seen in training (accumulated) and in the last evaluation pass (src/layers/mlp.py:219-239)."""

    def __init__(self, n_experts: int):
        super().__init__()
        self.register_buffer("train_load", torch.zeros(n_experts, dtype=torch.long), persistent=False)
        self.register_buffer("eval_load", torch.zeros(n_experts, dtype=torch.long), persistent=False)

    def record_load(self, counts, training: bool) -> None:
        if training:
            self.train_load += counts
        else:
            self.eval_load.copy_(counts)

    def reset_train_load(self) -> None:
        self.train_load.zero_()

    def reset_eval_load(self) -> None:
        self.eval_load.zero_()


class MoERouter(nn.Module):
    """Top-k router with an fp32-pinned gate (src/layers/mlp.py:248-302): fp32 logits, score
    function, top-k, weights normalised by their sum + 1e-9."""

    def __init__(self, d_model, n_routed_experts, n_routed_experts_per_token, normalize=True, expert_bias=False,
                 expert_bias_update_rate=0.001, router_score_fn="sigmoid"):
        super().__init__()
        self.n_routed_experts = n_routed_experts
        self.n_routed_experts_per_token = n_routed_experts_per_token
        self.normalize = normalize
        self.score_fn = MOE_ROUTER_SCORE_FNS[router_score_fn]
        self.score_name = router_score_fn
        self.gate = nn.Linear(d_model, n_routed_experts, bias=False)
        self.expert_bias = ExpertBias(n_routed_experts, expert_bias_update_rate) if expert_bias else None

    @classmethod
    def compute_flops(cls, d_model: int, n_experts: int, *, expert_bias=False) -> int:
        return 2 * d_model * n_experts + (ExpertBias.compute_flops(n_experts) if expert_bias else 0)

    @classmethod
    def compute_parameters(cls, d_model: int, n_experts: int, *, expert_bias=False) -> int:
        return d_model * n_experts + (ExpertBias.compute_parameters(n_experts) if expert_bias else 0)

    def update_expert_bias(self, expert_counts):
        """Nudge the load-balancing bias toward uniform load; no-op without one."""
        if self.expert_bias is not None:
            self.expert_bias.update(expert_counts)

    def _apply(self, fn, recurse=True):
        result = super()._apply(fn, recurse)
        if self.gate.weight.dtype != torch.float32:
            self.gate.weight.data = self.gate.weight.data.float()
        return result

    def forward(self, x):
        with torch.amp.autocast(device_type=x.device.type, enabled=False):
            logits = self.gate(x.float())                  # the fp32 gate GEMM stays the reference's own op
        if not x.is_cuda:
            raise RuntimeError("MoERouter runs on the B200 kernels only (no CPU path)")
        if self.n_routed_experts > 256:
            raise NotImplementedError("the router kernel handles at most 256 experts")
        bias = self.expert_bias.bias if self.expert_bias is not None else None
        # weights and probs come back in the activations' dtype (src/layers/mlp.py:302): bf16 straight from the
        # kernel, anything else from its fp32 results
        fp32_out = x.dtype != torch.bfloat16
        top_i, top_w, probs = _RouterBackEnd.apply(logits, self.n_routed_experts_per_token, self.score_name, self.normalize, bias,
                                                   fp32_out)
        return (top_i, top_w.to(x.dtype), probs.to(x.dtype)) if fp32_out else (top_i, top_w, probs)


class _RouterBackEnd(torch.autograd.Function):
    """Score function, top-k, normalisation and casts of MoERouter.forward in one kernel
    (b200q_moe_router_topk); the backward is the closed form of those steps on the (T, E) tensors."""

    @staticmethod
    def forward(ctx, logits, k, score_name, normalize, select_bias=None, fp32_out=False):
        top_i, top_w, probs = T.moe_router_topk(logits.float().contiguous(), k, score_name, normalize, select_bias, fp32_out)
        ctx.save_for_backward(logits, top_i)
        ctx.score_name, ctx.normalize = score_name, normalize
        ctx.mark_non_differentiable(top_i)
        return top_i, top_w, probs

    @staticmethod
    def backward(ctx, _g_idx, g_w, g_p):
        logits, top_i = ctx.saved_tensors
        p = logits.softmax(-1) if ctx.score_name == "softmax" else logits.sigmoid()
        dp = g_p.float() if g_p is not None else torch.zeros_like(p)
        if g_w is not None:
            g_w = g_w.float()
            w_raw = p.gather(-1, top_i)
            if ctx.normalize:
                s = w_raw.sum(-1, keepdim=True) + 1e-9
                d_raw = g_w / s - (g_w * w_raw).sum(-1, keepdim=True) / (s * s)
            else:
                d_raw = g_w
            dp = dp.scatter_add(-1, top_i, d_raw)
        if ctx.score_name == "softmax":
            dlogits = p * (dp - (dp * p).sum(-1, keepdim=True))
        else:
            dlogits = dp * p * (1 - p)
        return dlogits, None, None, None, None, None


class SparseMoEBlock(nn.Module):
    """Sparse MoE MLP block, dropless dispatch (src/layers/mlp.py:324-494): route, permute by
    expert, grouped FFN, weighted unpermute, Switch auxiliary loss.  Parameters keep the
    reference's names and (E, out, in) shapes: ``expert_gate_up`` / ``expert_up``, ``expert_down``."""

    def __init__(self, d_model, *, intermediate_size, n_routed_experts, n_routed_experts_per_token, n_shared_experts=0,
                 aux_loss=True, aux_loss_coef=0.001, expert_bias=False, expert_bias_update_rate=0.001,
                 router_score_fn="sigmoid", activation="silu", gated=True, bias=False, dropout=0.0):
        super().__init__()
        if aux_loss and expert_bias:
            raise ValueError("aux_loss and expert_bias are mutually exclusive MoE balancing strategies")
        self.n_routed_experts = n_routed_experts
        self.n_shared_experts = n_shared_experts
        self.expert_bias, self.expert_bias_update_rate = expert_bias, expert_bias_update_rate
        self.n_routed_experts_per_token = n_routed_experts_per_token
        self.aux_loss, self.aux_loss_coef = aux_loss, aux_loss_coef
        self.router_score_fn, self.gated = router_score_fn, gated
        self.act_fn = (GATED_ACTIVATIONS if gated else UNGATED_ACTIVATIONS)[activation]
        self.router = MoERouter(d_model, n_routed_experts, n_routed_experts_per_token, expert_bias=expert_bias,
                                expert_bias_update_rate=expert_bias_update_rate, router_score_fn=router_score_fn)
        width = 2 * intermediate_size if gated else intermediate_size
        name = "expert_gate_up" if gated else "expert_up"
        setattr(self, name, nn.Parameter(torch.empty(n_routed_experts, width, d_model)))
        setattr(self, name + "_bias", nn.Parameter(torch.zeros(n_routed_experts, width)) if bias else None)
        self.expert_down = nn.Parameter(torch.empty(n_routed_experts, d_model, intermediate_size))
        self.expert_down_bias = nn.Parameter(torch.zeros(n_routed_experts, d_model)) if bias else None
        # DeepSeekMoE shared experts: one always-on dense block of width n_shared_experts * intermediate_size
        self.shared_expert = (DenseMLPBlock(d_model, intermediate_size=n_shared_experts * intermediate_size, activation=activation,
                                            gated=gated, bias=bias) if n_shared_experts > 0 else None)
        # the reference drops elements of weight * expert_out (src/layers/mlp.py:472-473); the weights multiply
        # element-wise, so dropping the expert outputs before the weighted unpermute is the same operation
        self.expert_dropout = nn.Dropout(dropout)
        self.expert_load = ExpertLoad(n_routed_experts)

    @torch.no_grad()
    def post_step(self):
        weight_cache.invalidate(self)      # the optimizer has just written the experts: their quantized copies go
        if self.expert_bias:
            self.router.update_expert_bias(self.expert_load.train_load)
            self.expert_load.reset_train_load()

    def forward_meta(self) -> dict:
        """Routing metadata of the last forward: accumulated counts in training, the batch's counts in evaluation."""
        return {"expert_load": self.expert_load.train_load if self.training else self.expert_load.eval_load}

    @classmethod
    def compute_flops(cls, d_model, *, intermediate_size, n_routed_experts, n_routed_experts_per_token=2, n_shared_experts=0,
                      gated=True, bias=False, expert_bias=False, **_):
        """Per token: the router, k routed experts and the always-on shared block (src/layers/mlp.py:510-545)."""
        shared = _ffn_flops(d_model, n_shared_experts * intermediate_size, gated, bias) if n_shared_experts > 0 else 0
        return (MoERouter.compute_flops(d_model, n_routed_experts, expert_bias=expert_bias)
                + n_routed_experts_per_token * _ffn_flops(d_model, intermediate_size, gated, bias) + shared)

    @classmethod
    def compute_parameters(cls, d_model, *, intermediate_size, n_routed_experts, n_routed_experts_per_token=2, n_shared_experts=0,
                           gated=True, bias=False, expert_bias=False, active=False, **_):
        """All experts, or with `active` only the k that run per token; shared experts count either way."""
        n = n_routed_experts_per_token if active else n_routed_experts
        shared = _ffn_parameters(d_model, n_shared_experts * intermediate_size, gated, bias) if n_shared_experts > 0 else 0
        return (MoERouter.compute_parameters(d_model, n_routed_experts, expert_bias=expert_bias)
                + n * _ffn_parameters(d_model, intermediate_size, gated, bias) + shared)

    def forward(self, x):
        b, s, d = x.shape
        e = self.n_routed_experts
        x_flat = x.reshape(b * s, d)
        top_indices, top_weights, router_probs = self.router(x_flat)
        w_in = self.expert_gate_up if self.gated else self.expert_up
        b_in = self.expert_gate_up_bias if self.gated else self.expert_up_bias
        wants_grad = _wants_grad(x, top_weights, w_in, self.expert_down, b_in, self.expert_down_bias)
        if (not wants_grad and self.gated and self.act_fn is silu_glu and b_in is None and self.expert_down_bias is None
                and not (self.training and self.expert_dropout.p > 0) and d % 128 == 0 and w_in.shape[1] % 128 == 0
                and self.expert_down.shape[2] % 64 == 0 and x_flat.is_cuda):
            # bias-free SwiGLU experts without gradients: plan, gather + MXFP8, both grouped GEMMs (SwiGLU in the first one's
            # epilogue) and the weighted unpermute as one library call
            out, offs = T.moe_ffn_forward(x_flat.to(torch.bfloat16), top_indices, top_weights.to(torch.bfloat16),
                                          *_expert_weight_copies(w_in, "glu"), *_expert_weight_copies(self.expert_down, "rows"),
                                          e, self.expert_down.shape[2])
            return self._finish(x, out.to(x.dtype), offs, router_probs)
        plan = T.moe_permute_plan(top_indices, e)                          # stable sort by expert
        if wants_grad:
            _trainable_widths(d, w_in.shape[1], self.expert_down.shape[2])
            dropping = self.training and self.expert_dropout.p > 0
            if self.gated and self.act_fn is silu_glu and b_in is None and self.expert_down_bias is None and not dropping:
                # SwiGLU without biases: every element-wise step runs inside a quantizer kernel
                out = _ExpertFFN.apply(x_flat.to(torch.bfloat16), top_weights, w_in, self.expert_down,
                                       *_expert_weight_copies(w_in, "dual"), *_expert_weight_copies(self.expert_down, "dual"),
                                       *plan).to(x.dtype)
            else:
                y = _expert_ffn_general(x_flat.to(torch.bfloat16), w_in, self.expert_down, b_in, self.expert_down_bias,
                                        self.act_fn, self.gated, plan)
                out = _UnpermuteFn.apply(self.expert_dropout(y), top_weights, b * s, *plan).to(x.dtype)
        else:
            a, sfa = T.moe_gather_mxfp8(x_flat.to(torch.bfloat16), plan)      # permute fused with MXFP8
            y = _grouped_ffn_padded(a, sfa, plan, w_in, self.expert_down, self.act_fn, self.gated, b_in, self.expert_down_bias)
            out = T.moe_unpermute(self.expert_dropout(y), top_weights.to(torch.bfloat16), plan.row_of, b * s).to(x.dtype)

        return self._finish(x, out, plan.offs, router_probs)

    def _finish(self, x, out, offs, router_probs):
        """Load bookkeeping, auxiliary loss and shared experts (src/layers/mlp.py:479-494)."""
        b, s, d = x.shape
        e = self.n_routed_experts
        counts = torch.diff(offs, prepend=offs.new_zeros(1))
        self.expert_load.record_load(counts.detach(), self.training)
        aux = None
        if self.aux_loss:
            f = counts.to(x.dtype) / (b * s)
            probs = router_probs
            if self.router_score_fn == "sigmoid":
                probs = probs / (probs.sum(-1, keepdim=True) + 1e-9)
            aux = self.aux_loss_coef * e * (f * probs.mean(0)).sum()
        out = out.view(b, s, d)
        if self.shared_expert is not None:
            out = out + self.shared_expert(x)[0]
        return out, aux


MLP_REGISTRY = {"dense": DenseMLPBlock, "moe": SparseMoEBlock}
