"""CPU oracle for the low-precision linear path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: it is the checker that
the tests, the smoke check and the bench's CPU-baseline leg compare the CUDA
kernels against.  Everything here runs on torch-CPU / numpy.

Two kinds of functions live here:

* restatements of code the reference really has, each citing the lines it
  follows (``src/quant/fp8.py``, ``src/quant/linear.py``, ``src/layers/mlp.py``
  of gongyisheng/pretrain).  ``tests/golden/make_golden.py`` runs the reference's
  own functions on seeded inputs and commits the results, and
  ``tests/test_oracle.py`` pins these restatements to those vectors bit for bit;

* block-scaled extensions (MXFP8, NVFP4, scale-factor swizzle) that the
  reference only names in TODOs (``src/quant/__init__.py:20,26,30``).  They
  extend ``quantize_fp8``'s formula (``src/quant/fp8.py:16-32``) to block
  granularity.  PARITY UNPINNED at the reference for these: the reference holds
  no implementation or vector for them, so they are pinned only by this file's
  own contract (stated in each docstring).
"""

from __future__ import annotations

import numpy as np
import torch

E4M3 = torch.float8_e4m3fn
E5M2 = torch.float8_e5m2
FP8_MAX = {E4M3: 448.0, E5M2: 57344.0}
EPS = 1e-12  # src/quant/fp8.py:6

MX_BLOCK = 32
MX_NAN_EXP = 128  # scale exponent of a block that holds a NaN: byte 0xFF, the E8M0 NaN
NV_BLOCK = 16
E2M1_MAX = 6.0
NV_TENSOR_DIV = 2688.0  # 448 * 6
_E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


# ---------------------------------------------------------------------------
# FP8 with per-tensor / per-row / per-column fp32 scales (reference code exists)
# ---------------------------------------------------------------------------

def quantize_fp8(x: torch.Tensor, fp8_dtype: torch.dtype, dim: int | None = None):
    """Restates ``quantize_fp8`` (src/quant/fp8.py:16-32).

    amax over the whole tensor (dim=None) or over ``dim`` (keepdim), taken in
    x's dtype then widened; ``scale = max(amax / fp8_max, 1e-12)`` in fp32 with
    a true division; ``codes = cast(clamp(x.float() / scale, +-fp8_max))`` with
    torch's round-to-nearest-even cast.
    """
    fp8_max = FP8_MAX[fp8_dtype]
    if dim is None:
        amax = x.abs().max().float()
    else:
        amax = x.abs().amax(dim=dim, keepdim=True).float()
    scale = (amax / fp8_max).clamp_min(EPS)
    codes = (x.float() / scale).clamp(-fp8_max, fp8_max).to(fp8_dtype)
    return codes, scale


def fake_quantize_fp8(x: torch.Tensor, fp8_dtype: torch.dtype, dim: int | None = None):
    """Restates ``fake_quantize_fp8`` (src/quant/fp8.py:68-78): fp32 dequant
    multiply, one rounding back to x's dtype."""
    codes, scale = quantize_fp8(x, fp8_dtype, dim)
    return (codes.float() * scale).to(x.dtype)


def fp8_gemm_ref(a, b, out_dtype, a_dtype, b_dtype, rowwise=False):
    """The reference's CPU form of its FP8 GEMM: fake-quantise ``a`` per row
    (dim=-1) and ``b`` per column (dim=0) — or per tensor — and matmul
    (src/quant/linear.py:52-56; the same form tests/fast/quant/test_linear.py:82-85
    uses as the oracle of the real kernel)."""
    fa = fake_quantize_fp8(a, a_dtype, dim=-1 if rowwise else None)
    fb = fake_quantize_fp8(b, b_dtype, dim=0 if rowwise else None)
    return (fa.float() @ fb.float()).to(out_dtype)


# ---------------------------------------------------------------------------
# int8 series: symmetric integers of 8..4 bits in an int8 container (reference code exists)
# ---------------------------------------------------------------------------
INT_QMAX = {"int8": 127, "int7": 63, "int6": 31, "int5": 15, "int4": 7}   # src/quant/utils.py:19


def quantize_int8(x: torch.Tensor, qmax: int, dim: int | None = None):
    """Restates ``quantize_int8`` (src/quant/int8.py:9-19): ``scale = max(amax / qmax, 1e-12)``
    in fp32, ``codes = clamp(round(x.float() / scale), +-qmax)`` as int8 (``torch.round`` rounds
    halves to even)."""
    if dim is None:
        amax = x.abs().max().float()
    else:
        amax = x.abs().amax(dim=dim, keepdim=True).float()
    scale = (amax / qmax).clamp_min(EPS)
    codes = torch.round(x.float() / scale).clamp(-qmax, qmax).to(torch.int8)
    return codes, scale


def fake_quantize_int8(x: torch.Tensor, qmax: int, dim: int | None = None):
    """Restates ``fake_quantize_int8`` (src/quant/int8.py:22-26)."""
    codes, scale = quantize_int8(x, qmax, dim)
    return (codes.float() * scale).to(x.dtype)


def int8_gemm_ref(a, b, out_dtype, a_qmax, b_qmax, rowwise=False):
    """The reference's int8 GEMM with the real kernel's arithmetic (src/quant/int8.py:49-53):
    integer codes, exact integer accumulation (what ``torch._int_mm`` returns; it lives in
    torch 2.10 / cuBLAS, outside the reference checkout), then
    ``(acc.float() * a_scale * b_scale).to(out_dtype)``."""
    ca, sa = quantize_int8(a, a_qmax, dim=-1 if rowwise else None)
    cb, sb = quantize_int8(b, b_qmax, dim=0 if rowwise else None)
    acc = (ca.to(torch.int64) @ cb.to(torch.int64)).to(torch.int32)
    return (acc.float() * sa * sb).to(out_dtype)


def int8_gemm_fake_ref(a, b, out_dtype, a_qmax, b_qmax, rowwise=False):
    """The reference's CPU / fallback form of the same GEMM (src/quant/int8.py:41-47):
    fake-quantise both operands and matmul in their dtype."""
    fa = fake_quantize_int8(a, a_qmax, dim=-1 if rowwise else None)
    fb = fake_quantize_int8(b, b_qmax, dim=0 if rowwise else None)
    return (fa @ fb).to(out_dtype)


# ---------------------------------------------------------------------------
# MXFP8: 32-element blocks, E4M3/E5M2 codes, E8M0 power-of-two scale
# ---------------------------------------------------------------------------

def mx_scale_exponent(amax: torch.Tensor, fp8_dtype: torch.dtype = E4M3) -> torch.Tensor:
    """Unbiased exponent e of the block scale 2**e for a block maximum.

    Contract: 2**e is the smallest power of two >= max(amax / fp8_max, 1e-12),
    i.e. quantize_fp8's scale (src/quant/fp8.py:30) rounded UP to a power of two
    so that the block maximum never clips.  With amax = m * 2**E, m in [1, 2),
    and fp8_max = 1.75 * 2**P (P = 8 for E4M3, 15 for E5M2):
    e = E - P + (m > 1.75), floored at -39 (1e-12 rounds up to 2**-39) and
    capped at 127.  Integer-only: no division, no log.

    A NaN maximum (torch's amax propagates NaN, as in src/quant/fp8.py:26-29) gives
    e = 128: the scale max(NaN / fp8_max, 1e-12) is NaN, which E8M0 stores as 0xFF.
    """
    p = 8 if fp8_dtype == E4M3 else 15
    bits = amax.float().contiguous().view(torch.int32)
    expf = (bits >> 23) & 0xFF
    mant = bits & 0x7FFFFF
    e = expf - 127 - p + (mant > 0x600000).to(torch.int32)
    # fp32 subnormals / zero have expf == 0 and land far below the floor anyway
    e = e.clamp(min=-39, max=127)
    return torch.where(amax.float().isnan(), torch.full_like(e, MX_NAN_EXP), e)


def mx_scale_exponent_by_division(amax: torch.Tensor, fp8_dtype: torch.dtype = E4M3):
    """The same exponent computed the long way — ceil(log2(max(amax/fp8_max, 1e-12)))
    with the fp32 division of the reference's formula — used only to cross-check
    the integer rule above."""
    s = (amax.float() / FP8_MAX[fp8_dtype]).clamp_min(EPS).double()
    return torch.ceil(torch.log2(s)).to(torch.int32).clamp(min=-39, max=127)


def quantize_mxfp8(x: torch.Tensor, axis: int = -1, fp8_dtype: torch.dtype = E4M3):
    """Block-quantise a 2-D tensor along ``axis`` (the contraction dimension).

    Returns (codes, sf): ``codes`` is uint8 with the contraction dimension LAST
    (for axis=0 the result is transposed, shape (cols, rows)); ``sf`` is the
    uint8 E8M0 byte e+127 per block, shape (outer, C/32), natural layout.
    codes = e4m3_rne(clamp(x * 2**-e, +-fp8_max)) — an exact scaling followed by
    the same cast quantize_fp8 uses.  A block that holds a NaN follows quantize_fp8's
    arithmetic literally: NaN maximum -> NaN scale (byte 0xFF) -> every code of the
    block is NaN (0x7F).
    """
    assert x.dim() == 2
    xt = x.t() if axis in (0, -2) else x
    xt = xt.contiguous()
    outer, c = xt.shape
    assert c % MX_BLOCK == 0, "contraction dim must be a multiple of 32"
    xb = xt.float().view(outer, c // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(dim=-1)
    e = mx_scale_exponent(amax, fp8_dtype)
    inv = torch.ldexp(torch.ones_like(amax), -e)  # exact 2**-e
    inv = torch.where(e == MX_NAN_EXP, torch.full_like(inv, float("nan")), inv)
    fp8_max = FP8_MAX[fp8_dtype]
    codes = (xb * inv.unsqueeze(-1)).clamp(-fp8_max, fp8_max).to(fp8_dtype).view(torch.uint8)
    codes = torch.where((e == MX_NAN_EXP).unsqueeze(-1), torch.full_like(codes, 0x7F), codes)   # +NaN whatever the operands' signs
    return codes.view(outer, c), (e + 127).to(torch.uint8)


def dequantize_mxfp8(codes: torch.Tensor, sf: torch.Tensor, fp8_dtype: torch.dtype = E4M3):
    """codes * 2**(sf-127) as fp32 (exactly representable in bf16 for E4M3)."""
    outer, c = codes.shape
    v = codes.view(fp8_dtype).float().view(outer, c // MX_BLOCK, MX_BLOCK)
    scale = torch.ldexp(torch.ones(sf.shape, dtype=torch.float32), sf.to(torch.int32) - 127)
    return (v * scale.unsqueeze(-1)).view(outer, c)


# ---------------------------------------------------------------------------
# NVFP4: 16-element blocks, E2M1 codes, E4M3 block scale, fp32 tensor scale
# ---------------------------------------------------------------------------

def e2m1_rne(v: np.ndarray) -> np.ndarray:
    """Round fp32 values (already clamped to [-6, 6]) to E2M1 codes 0..15:
    magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the even code, sign in bit 3
    (-0 keeps its sign).  E2M1 has no NaN: a NaN becomes +6 (code 7), the saturating
    conversion's answer."""
    v = np.asarray(v, dtype=np.float32)
    nan = np.isnan(v)
    v = np.where(nan, np.float32(6.0), v)
    a = np.abs(v)
    hi = np.searchsorted(_E2M1_VALUES, a, side="left").clip(0, 7)
    lo = (hi - 1).clip(0, 7)
    dlo = a - _E2M1_VALUES[lo]
    dhi = _E2M1_VALUES[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    sign = np.signbit(v).astype(np.uint8) << 3
    return code | sign


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    mag = _E2M1_VALUES[code & 7]
    return np.where(code & 8, -mag, mag).astype(np.float32)


def nvfp4_tensor_scale(amax_tensor: torch.Tensor) -> torch.Tensor:
    """s_t = max(amax / 2688, 1e-12) in fp32 (2688 = 448 * 6): quantize_fp8's scale
    formula (src/quant/fp8.py:30) with the two-level maximum."""
    return (amax_tensor.float() / NV_TENSOR_DIV).clamp_min(EPS)


def quantize_nvfp4(x: torch.Tensor, axis: int = -1, tensor_amax: torch.Tensor | None = None):
    """Two-level NVFP4 quantisation of a 2-D tensor along ``axis``.

    Contract (every ``/`` an IEEE fp32 division):
      s_t  = max(amax_tensor / 2688, 1e-12)
      d_b  = max(amax_block / 6, 1e-12);  sq_b = e4m3_rne(min(d_b / s_t, 448))
      eff  = float(sq_b) * s_t;  codes = e2m1_rne(clamp(x.float() / eff, +-6)),
      all +0 when sq_b == 0.
    A NaN anywhere makes the tensor maximum, hence s_t, hence every block scale byte
    (0x7F, the E4M3 NaN) and every effective scale NaN: the whole tensor dequantizes to
    NaN, as a per-tensor quantize_fp8 of it would (src/quant/fp8.py:26-31).
    Returns (packed, sf, s_t): ``packed`` uint8 (outer, C/2), element 2i in the low
    nibble; ``sf`` uint8 E4M3 bytes (outer, C/16); ``s_t`` a 0-dim fp32 tensor.
    """
    assert x.dim() == 2
    xt = x.t() if axis in (0, -2) else x
    xt = xt.contiguous()
    outer, c = xt.shape
    assert c % NV_BLOCK == 0
    if tensor_amax is None:
        tensor_amax = x.abs().max().float()
    s_t = nvfp4_tensor_scale(tensor_amax)
    xb = xt.float().view(outer, c // NV_BLOCK, NV_BLOCK)
    d_b = (xb.abs().amax(dim=-1) / E2M1_MAX).clamp_min(EPS)
    sq = (d_b / s_t).clamp(max=448.0).to(E4M3)
    sq = torch.where(sq.float().isnan(), torch.full_like(sq.view(torch.uint8), 0x7F).view(E4M3), sq)   # +NaN byte
    eff = sq.float() * s_t
    q = (xb / eff.unsqueeze(-1)).clamp(-E2M1_MAX, E2M1_MAX)
    q = torch.where((sq.float() == 0).unsqueeze(-1), torch.zeros_like(q), q)
    codes = torch.from_numpy(e2m1_rne(q.numpy())).view(outer, c)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed.contiguous(), sq.view(torch.uint8), s_t


def dequantize_nvfp4(packed: torch.Tensor, sf: torch.Tensor, s_t: torch.Tensor):
    outer, half = packed.shape
    c = half * 2
    codes = torch.empty(outer, c, dtype=torch.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    v = torch.from_numpy(e2m1_decode(codes.numpy())).view(outer, c // NV_BLOCK, NV_BLOCK)
    eff = sf.view(E4M3).float() * s_t
    return (v * eff.unsqueeze(-1)).view(outer, c)


# ---------------------------------------------------------------------------
# Scale-factor storage: natural (outer, nblk) bytes <-> 128x4 swizzled tiles
# ---------------------------------------------------------------------------

def sf_swizzled_size(outer: int, nblk: int) -> int:
    return ((outer + 127) // 128) * ((nblk + 3) // 4) * 512


def swizzle_sf(sf: torch.Tensor) -> torch.Tensor:
    """Byte permutation of natural scale factors into the layout the tensor core's
    scale-factor copy consumes: rows padded to 128, blocks padded to 4, each
    (128 rows x 4 blocks) tile stored as 512 contiguous bytes with in-tile offset
    (r % 32) * 16 + (r % 128) // 32 * 4 + kb % 4, tiles ordered K-tile fastest.
    Pad bytes are zero."""
    outer, nblk = sf.shape
    rt, kt = (outer + 127) // 128, (nblk + 3) // 4
    out = torch.zeros(rt * kt * 512, dtype=torch.uint8)
    r = torch.arange(outer).unsqueeze(1).expand(outer, nblk)
    kb = torch.arange(nblk).unsqueeze(0).expand(outer, nblk)
    off = ((r // 128) * kt + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    out[off.reshape(-1)] = sf.reshape(-1)
    return out


def unswizzle_sf(buf: torch.Tensor, outer: int, nblk: int) -> torch.Tensor:
    kt = (nblk + 3) // 4
    r = torch.arange(outer).unsqueeze(1).expand(outer, nblk)
    kb = torch.arange(nblk).unsqueeze(0).expand(outer, nblk)
    off = ((r // 128) * kt + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    return buf[off.reshape(-1)].view(outer, nblk)


# ---------------------------------------------------------------------------
# GEMM references: dequantise, then matmul with fp32 accumulation
# ---------------------------------------------------------------------------

def gemm_dequant_ref(a_deq: torch.Tensor, b_deq: torch.Tensor, out_dtype=torch.bfloat16):
    """D = A . B^T for dequantised K-major operands A (M,K), B (N,K)."""
    return (a_deq.float() @ b_deq.float().t()).to(out_dtype)


def mxfp8_gemm_ref(a, b, out_dtype=torch.bfloat16, a_dtype=E4M3, b_dtype=E4M3):
    """Block-scaled analogue of the reference's fake-quant GEMM form
    (src/quant/linear.py:52-56): a (M,K) and b (K,N), both scaled along K."""
    ca, sa = quantize_mxfp8(a, -1, a_dtype)
    cb, sb = quantize_mxfp8(b, 0, b_dtype)
    return gemm_dequant_ref(dequantize_mxfp8(ca, sa, a_dtype), dequantize_mxfp8(cb, sb, b_dtype), out_dtype)


def nvfp4_gemm_ref(a, b, out_dtype=torch.bfloat16):
    pa, sa, ta = quantize_nvfp4(a, -1)
    pb, sb, tb = quantize_nvfp4(b, 0)
    return gemm_dequant_ref(dequantize_nvfp4(pa, sa, ta), dequantize_nvfp4(pb, sb, tb), out_dtype)


# ---------------------------------------------------------------------------
# MoE permute / grouped FFN / weighted unpermute (reference code exists)
# ---------------------------------------------------------------------------

def moe_permute(top_indices: torch.Tensor, n_experts: int):
    """Restates the permute of ``SparseMoEBlock.forward`` (src/layers/mlp.py:446-457):
    flatten (token, slot) token-major, stable sort by expert.  Returns
    (order, token_ids_sorted, expert_counts, offs int32)."""
    t, k = top_indices.shape
    expert_ids = top_indices.reshape(-1)
    token_ids = torch.arange(t).repeat_interleave(k)
    _, order = expert_ids.sort(stable=True)
    counts = torch.bincount(expert_ids, minlength=n_experts)
    offs = counts.cumsum(0).to(torch.int32)
    return order, token_ids[order], counts, offs


def moe_padded_plan(top_indices: torch.Tensor, n_experts: int):
    """Host restatement of the padded expert-sorted layout the kernels use between permute and unpermute: the reference's
    stable expert order (src/layers/mlp.py:447-452) with every expert's segment starting on a multiple of 128 rows.
    Returns (offs (E,) cumulative unpadded ends, padded_offs (E+1,), row_of (T*k,) padded row of every pair)."""
    flat = top_indices.reshape(-1)
    order, _, counts, offs = moe_permute(top_indices, n_experts)
    padded = (counts + 127) // 128 * 128
    padded_offs = torch.cat([padded.new_zeros(1), padded.cumsum(0)])
    starts = offs - counts
    row_of = torch.empty(flat.numel(), dtype=torch.int64)
    sorted_e = flat[order]
    row_of[order] = padded_offs[sorted_e] + torch.arange(flat.numel()) - starts[sorted_e]
    return offs.to(torch.int32), padded_offs.to(torch.int32), row_of.to(torch.int32)


def ep_index(all_offs: torch.Tensor, rank: int, top_indices: torch.Tensor, row_of: torch.Tensor, padded_offs: torch.Tensor):
    """Host restatement of the expert-parallel index tables (no counterpart in the reference, which is single-GPU).

    all_offs (world, E): every sender's cumulative per-expert counts.  An owner's buffer holds the segments of its
    E / world experts in order, each padded to 128 rows; inside a segment the senders' rows follow in rank order, each
    sender's in its own stable order.  Returns (row_base (E,): where `rank`'s rows for every expert start at the owner;
    own_offs (E / world,): cumulative ends of the segments `rank` owns; pair_peer, pair_row (T*k,))."""
    world, e = all_offs.shape
    el = e // world
    counts = torch.diff(all_offs.long(), dim=1, prepend=torch.zeros(world, 1, dtype=torch.long))       # [sender][expert]
    totals = counts.sum(0)
    padded = (totals + 127) // 128 * 128
    seg = padded.view(world, el)
    seg_start = (seg.cumsum(1) - seg).reshape(-1)
    row_base = seg_start + counts[:rank].sum(0)
    own_offs = totals.view(world, el)[rank].cumsum(0)
    flat = top_indices.reshape(-1).long()
    pair_peer = flat // el
    pair_row = row_base[flat] + row_of.long() - padded_offs.long()[flat]
    return row_base.to(torch.int32), own_offs.to(torch.int32), pair_peer.to(torch.int32), pair_row.to(torch.int32)


def silu_glu(gate, up):
    """src/layers/activation.py:80-81."""
    return torch.nn.functional.silu(gate) * up


def grouped_mlp_ref(x_sorted, w_in, w_down, offs, fake_quant=None):
    """Per-expert loop form of ``grouped_mlp`` (src/layers/mlp.py:55-100; the loop the
    reference's own tests compare against, tests/fast/layers/test_mlp.py:929-992),
    gated SwiGLU experts, optional operand fake-quantiser applied to both GEMMs'
    operands along their contraction dimension."""
    fq = fake_quant or (lambda t: t)
    out = torch.zeros(x_sorted.shape[0], w_down.shape[1], dtype=x_sorted.dtype)
    start = 0
    for e, end in enumerate(offs.tolist()):
        if end > start:
            xe = x_sorted[start:end]
            h = (fq(xe).float() @ fq(w_in[e]).float().t()).to(x_sorted.dtype)
            g, u = h.chunk(2, dim=-1)
            h = silu_glu(g, u)
            out[start:end] = (fq(h).float() @ fq(w_down[e]).float().t()).to(x_sorted.dtype)
        start = end
    return out


def moe_unpermute_ref(expert_out, weights_sorted, token_ids_sorted, n_tokens):
    """src/layers/mlp.py:472-477 — scale rows by their routing weight, index_add_
    into a zero tensor (the reference accumulates in the activations' dtype)."""
    out = torch.zeros(n_tokens, expert_out.shape[1], dtype=expert_out.dtype)
    out.index_add_(0, token_ids_sorted, expert_out * weights_sorted.reshape(-1, 1))
    return out


def moe_unpermute_fp32(expert_out, weights_sorted, token_ids_sorted, n_tokens):
    """The same reduction with fp32 accumulation and one final rounding (what the
    CUDA kernel computes; compared with the bf16 form under a tolerance)."""
    out = torch.zeros(n_tokens, expert_out.shape[1], dtype=torch.float32)
    out.index_add_(0, token_ids_sorted, expert_out.float() * weights_sorted.float().reshape(-1, 1))
    return out.to(expert_out.dtype)


def router_topk(logits: torch.Tensor, k: int, dtype=torch.bfloat16):
    """softmax -> top-k -> normalise, as MoERouter.forward (src/layers/mlp.py:294-302)."""
    probs = logits.float().softmax(dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    w = w / (w.sum(-1, keepdim=True) + 1e-9)
    return idx, w.to(dtype)


def router_backend(logits: torch.Tensor, k: int, score_fn: str = "softmax", normalize: bool = True, dtype=torch.bfloat16):
    """Everything after the gate GEMM in MoERouter.forward (src/layers/mlp.py:292-301) and the
    bincount of SparseMoEBlock.forward (:455): (top_idx, top_w, probs, expert_counts)."""
    lf = logits.float()
    probs = lf.softmax(dim=-1) if score_fn == "softmax" else lf.sigmoid()
    w, idx = torch.topk(probs, k, dim=-1)
    if normalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-9)
    counts = torch.bincount(idx.reshape(-1), minlength=logits.shape[-1])
    return idx, w.to(dtype), probs.to(dtype), counts


# ---------------------------------------------------------------------------
# Seeded synthetic inputs for the benchmark configurations
# ---------------------------------------------------------------------------

def _gen(seed=0):
    return torch.Generator(device="cpu").manual_seed(seed)


def inputs_mxfp8_linear(m=8192, k=768, n=3072, seed=0):
    g = _gen(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    return x, w


def inputs_nvfp4_mlp(tokens=16384, hidden=1024, inter=3072, seed=0):
    g = _gen(seed)
    x = torch.randn(tokens, hidden, generator=g)
    mask = torch.rand(tokens, hidden, generator=g) < 1e-3
    x = torch.where(mask, x * 50.0, x).to(torch.bfloat16)
    w_gu = (0.02 * torch.randn(2 * inter, hidden, generator=g)).to(torch.bfloat16)
    w_d = (0.02 * torch.randn(hidden, inter, generator=g)).to(torch.bfloat16)
    return x, w_gu, w_d


def inputs_fp8_triple(m=16384, k=2048, n=2048, seed=0):
    g = _gen(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    dy = (1e-3 * torch.randn(m, n, generator=g)).to(torch.bfloat16)
    return x, w, dy


def inputs_moe(tokens=16384, hidden=768, experts=64, topk=4, inter=384, seed=0):
    g = _gen(seed)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, generator=g)
    w_gu = (0.02 * torch.randn(experts, 2 * inter, hidden, generator=g)).to(torch.bfloat16)
    w_d = (0.02 * torch.randn(experts, hidden, inter, generator=g)).to(torch.bfloat16)
    return x, logits, w_gu, w_d


def inputs_square(n=4096, seed=0):
    g = _gen(seed)
    a = torch.randn(n, n, generator=g).to(torch.bfloat16)
    b = torch.randn(n, n, generator=g).to(torch.bfloat16)
    return a, b
