"""MoE path on the GPU through the C-ABI: permute plan bit-exact against the reference's own
sort (golden vectors), gather / quantize bit-exact against the oracle, ragged grouped GEMM,
SwiGLU and weighted unpermute within tolerance, including empty experts first / middle / last
(the group patterns of the reference's tests/fast/layers/test_mlp.py:929)."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import restate as R
from conftest import bf16_from_bits
import gpu_ref as G

pytestmark = pytest.mark.gpu
E4 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def ops():
    from pretrain_b200 import build, ops
    build.build()
    return ops


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm()).item()


def _check_plan(plan, top_i, n_experts):
    order, tok, counts, offs = R.moe_permute(top_i, n_experts)
    assert torch.equal(plan.offs.cpu(), offs)
    pstart = torch.zeros(n_experts + 1, dtype=torch.int64)
    pstart[1:] = ((counts + 127) // 128 * 128).cumsum(0)
    assert torch.equal(plan.padded_offs.cpu().long(), pstart)
    assert plan.num_tiles.item() == pstart[-1] // 128
    starts = offs.long() - counts
    expert_sorted = top_i.reshape(-1)[order]
    want_rows = pstart[expert_sorted] + torch.arange(order.numel()) - starts[expert_sorted]
    row_of = plan.row_of.cpu().long()
    assert torch.equal(row_of[order], want_rows)                      # stable: the reference's row order
    src = plan.src_of_row.cpu().long()
    assert torch.equal(src[want_rows], tok)
    mask = torch.ones(plan.padded_rows, dtype=torch.bool)
    mask[want_rows] = False
    assert (src[mask] == -1).all()
    te = plan.tile_expert.cpu()
    for e in range(n_experts):
        assert (te[pstart[e] // 128: pstart[e + 1] // 128] == e).all()
    assert (te[pstart[-1] // 128:] == -1).all()
    return want_rows, tok


def test_permute_plan_matches_reference_golden(ops, golden):
    top_i = torch.from_numpy(golden["moe_top_i"])
    plan = ops.moe_permute_plan(top_i.cuda(), 6)
    assert np.array_equal(plan.offs.cpu().numpy(), golden["moe_offs"])
    want_rows, tok = _check_plan(plan, top_i, 6)
    assert np.array_equal(tok.numpy(), golden["moe_token_ids_sorted"])
    x = bf16_from_bits(golden["moe_x"])
    xs = ops.moe_gather(x.cuda(), plan, False).cpu()
    assert np.array_equal(xs[want_rows].view(torch.int16).numpy(), golden["moe_x_sorted"])
    live = plan.num_tiles.item() * 128
    pad = torch.ones(live, dtype=torch.bool)
    pad[want_rows] = False
    assert (xs[:live][pad] == 0).all()


@pytest.mark.parametrize("t,k,e", [(16384, 4, 64), (1000, 2, 8), (3000, 8, 256), (7, 1, 4)])
def test_permute_plan_large_and_ragged(ops, t, k, e):
    g = torch.Generator().manual_seed(t)
    logits = torch.randn(t, e, generator=g)
    if e >= 8:
        logits[:, 3] = -1e9                                            # an expert nobody picks
    top_i = torch.topk(logits, k, dim=-1).indices
    plan = ops.moe_permute_plan(top_i.cuda(), e)
    _check_plan(plan, top_i, e)


def test_fused_permute_quantize_is_bit_exact(ops):
    x, logits, _, _ = R.inputs_moe(2048, 768, 64, 4, 384)
    top_i, _ = R.router_topk(logits, 4)
    plan = ops.moe_permute_plan(top_i.cuda(), 64)
    want_rows, tok = _check_plan(plan, top_i, 64)
    codes, sf = ops.moe_gather(x.cuda(), plan, True)
    rc, rs = R.quantize_mxfp8(x[tok])
    assert torch.equal(codes.cpu()[want_rows], rc)
    sf_nat = G.unswizzle(sf, plan.padded_rows, 768 // 32).cpu()
    assert torch.equal(sf_nat[want_rows], rs)


# 37 experts, every fifth one empty, up to 6 row tiles each: odd and even tile counts in a row
_MANY = [int(c) for c in torch.randint(0, 700, (37,), generator=torch.Generator().manual_seed(3)) * (torch.arange(37) % 5 != 2)]


@pytest.mark.parametrize("counts", [[5, 0, 7, 4], [200, 0, 0, 131], [128, 256, 1, 0], [0, 0, 300, 0], "many"])
@pytest.mark.parametrize("k,n", [(256, 384), (768, 384), (384, 768)])
@pytest.mark.parametrize("bn", [0, 128, 192, 256, "pair", "bstat", "rowstat"])   # tile width of the one-CTA kernel (0 = by shape) / CTA pairs / weight tile kept in shared memory / rows of A kept in shared memory (dgrad)
def test_grouped_backward_gemms(ops, counts, k, n, bn):
    """dgrad (operand = transposed weight stack, expert offset along K) and wgrad (ragged K range per
    expert, one output matrix per expert, zeros for experts without rows) against dequantize-then-matmul."""
    from pretrain_b200 import _lib
    counts = _MANY if counts == "many" else counts
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    r, e = sum(counts), len(counts)
    gy = torch.randn(r, k, generator=g).bfloat16().cuda()               # "output gradient" rows, K = the layer's out features
    w = (0.05 * torch.randn(e, k, n, generator=g)).bfloat16().cuda()     # weight stack (E, out = k, in = n)
    xin = torch.randn(r, n, generator=g).bfloat16().cuda()               # layer input rows
    offs = torch.tensor(counts).cumsum(0).int().cuda()
    plan = ops.moe_pad_plan(offs, r)
    pstart = plan.padded_offs.cpu().tolist()
    a, sfa = ops.moe_gather(gy, plan, True)                              # (padded_rows, k) codes along k
    wt, wtsf = ops.quantize_mxfp8(w.reshape(e * k, n), 0)                # (n, E*k): every expert's operand at column e*k
    gy_pad, x_pad = ops.moe_gather(gy, plan, False), ops.moe_gather(xin, plan, False)
    live = int(plan.num_tiles.item()) * 128
    # rows past the live tiles are never written by the forward's kernels and may hold anything: an expert
    # without rows must not read them (a product with them "scaled to zero" would be NaN)
    gy_pad[live:] = float("nan"); x_pad[live:] = float("nan")
    gt, gtsf = ops.quantize_mxfp8(gy_pad, 0)                             # (k, padded_rows)
    xt, xtsf = ops.quantize_mxfp8(x_pad, 0)                              # (n, padded_rows)
    _lib.load().b200q_debug_set_gemm_pair(1 if bn == "pair" else 0)
    _lib.load().b200q_debug_set_gemm_bn(0 if bn in ("pair", "bstat", "rowstat") else bn)
    _lib.load().b200q_debug_set_gemm_bstat(1 if bn == "bstat" else -1)
    _lib.load().b200q_debug_set_gemm_rowstat(1 if bn == "rowstat" else -1)
    try:
        dx = ops.grouped_gemm_mxfp8_dgrad(a, sfa, wt, wtsf, plan, n)     # (padded_rows, n)
        dw = ops.grouped_gemm_mxfp8_wgrad(gt, gtsf, xt, xtsf, plan)      # (E, k, n)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_bn(0)
        _lib.load().b200q_debug_set_gemm_pair(0)
        _lib.load().b200q_debug_set_gemm_bstat(0)
        _lib.load().b200q_debug_set_gemm_rowstat(0)
    a_deq = G.deq_mxfp8(a, sfa)
    wt_deq = G.deq_mxfp8(wt, wtsf)                                       # (n, E*k)
    gt_deq, xt_deq = G.deq_mxfp8(gt, gtsf), G.deq_mxfp8(xt, xtsf)
    for ei, c in enumerate(counts):
        lo, hi = pstart[ei], pstart[ei + 1]
        if c:
            ref = G.matmul_fp32(a_deq[lo:lo + c], wt_deq[:, ei * k:(ei + 1) * k])
            mx, fro = G.rel_errors(dx[lo:lo + c], ref)
            assert mx <= 1e-2 and fro <= 1e-2, ("dgrad", ei, mx, fro)
            refw = G.matmul_fp32(gt_deq[:, lo:hi], xt_deq[:, lo:hi])
            mx, fro = G.rel_errors(dw[ei], refw)
            assert mx <= 1e-2 and fro <= 1e-2, ("wgrad", ei, mx, fro)
        else:
            assert (dw[ei] == 0).all()


def test_grouped_entry_points_want_whole_scale_groups_per_expert(ops):
    """N % 128 != 0 would start an expert's weight rows inside a 128-row scale-factor group: refused, not mis-computed."""
    from pretrain_b200 import _lib
    lib = _lib.load()
    z = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    i32 = torch.zeros(8, dtype=torch.int32, device="cuda")
    for n in (64, 96, 160, 320):
        rc = lib.b200q_grouped_gemm_mxfp8(z.data_ptr(), 0, z.data_ptr(), z.data_ptr(), 0, z.data_ptr(), i32.data_ptr(), i32.data_ptr(),
                                          128, 2, n, 128, z.data_ptr(), n, None)
        assert rc == -2, (n, rc)
        if n % 64 == 0:
            rc = lib.b200q_grouped_gemm_mxfp8_swiglu(z.data_ptr(), 0, z.data_ptr(), z.data_ptr(), 0, z.data_ptr(), i32.data_ptr(),
                                                     i32.data_ptr(), 128, 2, n, 128, z.data_ptr(), n // 2, z.data_ptr(), None)
            assert rc == -2, (n, rc)


def test_expert_ffn_backward_with_trailing_empty_experts_and_poisoned_scratch(ops, monkeypatch):
    """Every buffer the layer allocates starts as 0xFF bytes (bf16 / fp32 NaN): rows past the live tiles, which no
    grouped GEMM writes, then hold NaN when the both-directions quantizers and the wgrad GEMMs pass over them.
    Experts without tokens - trailing ones, whose K range lies past the live tiles, included - must still get
    exactly zero weight gradients, and every other gradient must be finite."""
    from pretrain_b200.layers.mlp import _ExpertFFN, _expert_weight_copies
    from pretrain_b200 import torch_ops as T
    real_empty = torch.empty

    def poisoned_empty(*args, **kwargs):
        t = real_empty(*args, **kwargs)
        if t.is_cuda and t.numel() and t.is_contiguous():
            t.view(-1).view(torch.uint8).fill_(0xFF)
        return t

    t_, d, e, k, inter = 512, 256, 16, 2, 128
    x, logits, w_gu, w_d = R.inputs_moe(t_, d, e, k, inter, seed=3)
    logits[:, 3] = -1e9                      # an empty expert in the middle
    logits[:, e - 3:] = -1e9                 # and three trailing ones
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    x.requires_grad_(True); top_w.requires_grad_(True); w_gu.requires_grad_(True); w_d.requires_grad_(True)
    dout = torch.randn(t_, d, device="cuda", dtype=torch.bfloat16)
    monkeypatch.setattr(torch, "empty", poisoned_empty)
    out = _ExpertFFN.apply(x, top_w, w_gu, w_d, *_expert_weight_copies(w_gu, "dual"), *_expert_weight_copies(w_d, "dual"),
                           *T.moe_permute_plan(top_i, e))
    gx, gtw, g1, g2 = torch.autograd.grad(out, (x, top_w, w_gu, w_d), dout)
    monkeypatch.undo()
    ops.device_status()
    for g in (out, gx, gtw, g1, g2):
        assert torch.isfinite(g.float()).all()
    for ei in (3, e - 3, e - 2, e - 1):
        assert (g1[ei] == 0).all() and (g2[ei] == 0).all()
    assert (g1[0] != 0).any() and (g2[e - 4] != 0).any()


def test_gather_and_swiglu_from_rows_that_are_only_16_byte_aligned(ops):
    """Views whose start and pitch rule out 256-bit loads give the same bytes as aligned copies."""
    x, logits, _, _ = R.inputs_moe(512, 256, 8, 2, 128)
    top_i, _ = R.router_topk(logits, 2)
    plan = ops.moe_permute_plan(top_i.cuda(), 8)
    big = torch.zeros(512, 256 + 24, dtype=torch.bfloat16, device="cuda")
    big[:, 8:264] = x.cuda()
    view = big[:, 8:264]
    assert view.data_ptr() % 32 == 16 and view.stride(0) % 16 == 8
    for quant in (True, False):
        a = ops.moe_gather(view, plan, quant)
        b = ops.moe_gather(x.cuda(), plan, quant)
        live = int(plan.num_tiles.item()) * 128
        if quant:
            n_sf = live // 128 * (256 // 32 // 4) * 512       # scale bytes of the live row tiles
            assert torch.equal(a[0][:live], b[0][:live]) and torch.equal(a[1][:n_sf], b[1][:n_sf])
        else:
            assert torch.equal(a[:live], b[:live])
    h = torch.zeros(384, 512 + 24, dtype=torch.bfloat16, device="cuda")
    hv = h[:, 8:520]
    hv.copy_(2.0 * torch.randn(384, 512, device="cuda"))
    for quant in (True, False):
        a, b = ops.swiglu(hv, quant), ops.swiglu(hv.contiguous(), quant)
        if quant:
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
        else:
            assert torch.equal(a, b)


def _grouped_ref(a_deq, w_deq, counts):
    out = torch.zeros(a_deq.shape[0], w_deq.shape[1], device=a_deq.device)
    s = 0
    for e, c in enumerate(counts):
        if c:
            out[s:s + c] = G.matmul_fp32(a_deq[s:s + c], w_deq[e])
        s += c
    return out


@pytest.mark.parametrize("pair", [1, -1, "bstat", "rowstat"])   # CTA pairs formed inside every expert (opt-in) / the one-CTA kernel / the B-stationary kernel / the row-stationary pair kernel
@pytest.mark.parametrize("counts", [[5, 0, 7, 4], [0, 5, 7, 4], [5, 7, 4, 0], [200, 0, 0, 131], [128, 256, 1, 0], [300, 129, 0, 513, 1], _MANY])
@pytest.mark.parametrize("d,n", [(256, 384), (768, 768)])
def test_grouped_gemm_with_empty_experts(ops, counts, d, n, pair):
    from pretrain_b200 import _lib
    g = torch.Generator().manual_seed(sum(counts) + d)
    r, e = sum(counts), len(counts)
    x = torch.randn(r, d, generator=g).bfloat16().cuda()
    w = (0.05 * torch.randn(e, n, d, generator=g)).bfloat16().cuda()
    offs = torch.tensor(counts).cumsum(0).int().cuda()
    plan = ops.moe_pad_plan(offs, r)
    a, sfa = ops.moe_gather(x, plan, True)
    wq, wsf = ops.quantize_mxfp8(w.reshape(e * n, d), 1)
    _lib.load().b200q_debug_set_gemm_pair(0 if pair in ("bstat", "rowstat") else pair)
    _lib.load().b200q_debug_set_gemm_bstat(1 if pair == "bstat" else -1)
    _lib.load().b200q_debug_set_gemm_rowstat(1 if pair == "rowstat" else -1)
    try:
        out = ops.grouped_gemm_mxfp8(a, sfa, wq, wsf, plan, n)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_pair(0)
        _lib.load().b200q_debug_set_gemm_bstat(0)
        _lib.load().b200q_debug_set_gemm_rowstat(0)
    xq, xsf = ops.quantize_mxfp8(x, 1)
    ref = _grouped_ref(G.deq_mxfp8(xq, xsf), G.deq_mxfp8(wq, wsf).view(e, n, d), counts)
    pstart = plan.padded_offs.cpu().tolist()
    s = 0
    for ei, c in enumerate(counts):
        if c:
            got = out[pstart[ei]: pstart[ei] + c]
            mx, fro = G.rel_errors(got, ref[s:s + c])
            assert mx <= 1e-2 and fro <= 1e-2, (ei, mx, fro)
            assert (out[pstart[ei] + c: pstart[ei + 1]] == 0).all()   # pad rows stay zero
        s += c


@pytest.mark.parametrize("counts", [[5, 0, 7, 4], [200, 0, 0, 131], [128, 256, 1, 0]])
@pytest.mark.parametrize("d,inter", [(256, 64), (768, 384), (512, 192)])
@pytest.mark.parametrize("bn", [0, 128, 192, 256, "pair", "bstat", "rowstat"])
def test_swiglu_epilogue_equals_gemm_then_swiglu(ops, counts, d, inter, bn):
    """Grouped GEMM with the SwiGLU + MXFP8 epilogue over interleaved weights == grouped GEMM to
    bf16 followed by the stand-alone SwiGLU + MXFP8 kernel over the plain weights, byte for byte."""
    from pretrain_b200 import _lib
    g = torch.Generator().manual_seed(sum(counts) + d + inter)
    r, e = sum(counts), len(counts)
    x = torch.randn(r, d, generator=g).bfloat16().cuda()
    w = (0.08 * torch.randn(e, 2 * inter, d, generator=g)).bfloat16().cuda()
    offs = torch.tensor(counts).cumsum(0).int().cuda()
    plan = ops.moe_pad_plan(offs, r)
    a, sfa = ops.moe_gather(x, plan, True)
    live = int(plan.num_tiles.item()) * 128
    # plain chain (every expert's 2I rows padded to 128 so that scale-factor tiles do not straddle experts)
    n_pad = (2 * inter + 127) // 128 * 128
    wp = torch.cat([w, w.new_zeros(e, n_pad - 2 * inter, d)], 1) if n_pad != 2 * inter else w
    wq, wsf = ops.quantize_mxfp8(wp.reshape(e * n_pad, d), 1)
    hb = ops.grouped_gemm_mxfp8(a, sfa, wq, wsf, plan, n_pad)[:live, : 2 * inter].contiguous()
    want_codes, want_sf = ops.swiglu(hb, True)
    _lib.load().b200q_debug_set_gemm_pair(1 if bn == "pair" else 0)
    _lib.load().b200q_debug_set_gemm_bn(0 if bn in ("pair", "bstat", "rowstat") else bn)
    _lib.load().b200q_debug_set_gemm_bstat(1 if bn == "bstat" else -1)
    _lib.load().b200q_debug_set_gemm_rowstat(1 if bn == "rowstat" else -1)
    try:
        wqi, wsfi = ops.quantize_mxfp8_rowmap(w.reshape(e * 2 * inter, d), ops.glu_row_map(e, inter, "cuda"))
        got_codes, got_sf = ops.grouped_gemm_mxfp8_swiglu(a, sfa, wqi, wsfi, plan, 2 * inter)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_bn(0)
        _lib.load().b200q_debug_set_gemm_pair(0)
        _lib.load().b200q_debug_set_gemm_bstat(0)
        _lib.load().b200q_debug_set_gemm_rowstat(0)
    assert torch.equal(got_codes[:live], want_codes)
    n_sf = live // 128 * ((inter // 32 + 3) // 4) * 512
    assert torch.equal(got_sf[:n_sf], want_sf[:n_sf])


def test_rowmap_quantizer_is_a_row_permutation(ops):
    e, inter, d = 3, 96, 160
    g = torch.Generator().manual_seed(9)
    w = torch.randn(e * 2 * inter, d, generator=g).bfloat16().cuda()
    m = ops.glu_row_map(e, inter, "cuda")
    assert sorted(m.tolist()) == list(range(e * 2 * inter))
    assert m[:32].tolist() == list(range(32)) and m[inter: inter + 32].tolist() == list(range(32, 64))   # gate block, then its up block
    codes, sf = ops.quantize_mxfp8_rowmap(w, m, layout=0)
    rc, rs = ops.quantize_mxfp8(w, 1, layout=0)
    assert torch.equal(codes[m.long()], rc)
    assert torch.equal(sf.view(-1, d // 32)[m.long()], rs.view(-1, d // 32))


@pytest.mark.parametrize("pair", [-1, 1])
@pytest.mark.parametrize("m_,d,inter", [(300, 512, 256), (1024, 768, 384)])
def test_dense_gemm_with_swiglu_epilogue(ops, pair, m_, d, inter):
    from pretrain_b200 import _lib
    g = torch.Generator().manual_seed(4)
    x = torch.randn(m_, d, generator=g).bfloat16().cuda()
    w = (0.06 * torch.randn(2 * inter, d, generator=g)).bfloat16().cuda()
    xq, xsf = ops.quantize_mxfp8(x, 1)
    wq, wsf = ops.quantize_mxfp8(w, 1)
    want_codes, want_sf = ops.swiglu(ops.gemm_mxfp8(xq, xsf, wq, wsf), True)
    wqi, wsfi = ops.quantize_mxfp8_rowmap(w, ops.glu_row_map(1, inter, "cuda"))
    _lib.load().b200q_debug_set_gemm_pair(pair)                   # never / always the CTA-pair kernel
    try:
        got_codes, got_sf = ops.gemm_mxfp8_swiglu(xq, xsf, wqi, wsfi)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_pair(0)
    assert torch.equal(got_codes, want_codes)
    assert torch.equal(G.unswizzle(got_sf, m_, inter // 32), G.unswizzle(want_sf, m_, inter // 32))
    # and against the oracle's arithmetic on the dequantized operands
    h_ref = R.silu_glu(*(G.matmul_fp32(G.deq_mxfp8(xq, xsf), G.deq_mxfp8(wq, wsf)).bfloat16()).chunk(2, dim=-1))
    h_got = G.deq_mxfp8(got_codes, got_sf)
    mx, fro = G.rel_errors(h_got, h_ref.float())
    assert mx <= 6e-2 and fro <= 4e-2, (mx, fro)      # one E4M3 rounding (2^-4 relative) on top of the GEMM tolerance


@pytest.mark.parametrize("score_fn", ["softmax", "sigmoid"])
@pytest.mark.parametrize("normalize", [True, False])
@pytest.mark.parametrize("t,e,k", [(4096, 64, 4), (1000, 8, 2), (777, 200, 6), (64, 256, 8), (16384, 64, 4)])
def test_router_back_end(ops, score_fn, normalize, t, e, k):
    """Indices and counts exactly as torch.topk / bincount on the same fp32 logits; weights and
    probs within one bf16 ulp of the reference's fp32 arithmetic (the kernel's exp and sum differ
    from torch's in the last fp32 bit at most)."""
    g = torch.Generator().manual_seed(t + e + k)
    logits = torch.randn(t, e, generator=g)
    if t == 1000:
        logits = logits * 30                                       # saturated router (tests/fast/layers/test_mlp.py:808-822)
    idx, w, probs, counts = ops.moe_router_topk(logits.cuda(), k, score_fn, normalize)
    ri, rw, rp, rc = R.router_backend(logits, k, score_fn, normalize)
    # positions where the reference's own probs tie (saturation) may be ordered either way: compare as sets there
    pf = logits.softmax(-1) if score_fn == "softmax" else logits.sigmoid()
    tied = (pf.gather(-1, ri)[:, 1:] == pf.gather(-1, ri)[:, :-1]).any(-1) | (pf.gather(-1, ri)[:, -1:] == pf.topk(min(k + 1, e), -1).values[:, -1:]).any(-1)
    assert torch.equal(idx.cpu()[~tied], ri[~tied])
    # Rows with exact ties (a saturated softmax sends many probs to 0.0 or 1.0; sigmoid saturates likewise): which of two
    # equal probs torch.topk returns first is its implementation's choice, so the indices may differ - but only among
    # experts of EQUAL prob: the chosen experts' probs must be the reference's, position by position, and no expert
    # may be chosen twice.
    ti, tr = idx.cpu()[tied], ri[tied]
    assert torch.equal(pf[tied].gather(-1, ti), pf[tied].gather(-1, tr))
    assert (ti.sort(-1).values.diff(dim=-1) != 0).all()
    # ... and among equal probs the kernel's documented order holds: larger logit first, then lower index
    lt, pt = logits[tied].gather(-1, ti), pf[tied].gather(-1, ti)
    same = pt[:, 1:] == pt[:, :-1]
    assert ((lt[:, :-1] > lt[:, 1:]) | ((lt[:, :-1] == lt[:, 1:]) & (ti[:, :-1] < ti[:, 1:])))[same].all()
    clean = ~tied
    ulp = lambda a, b: ((a.view(torch.int16).int() - b.view(torch.int16).int()).abs().max().item() if a.numel() else 0)
    assert ulp(w.cpu()[clean], rw[clean]) <= 1
    assert ulp(probs.cpu(), rp) <= 1
    assert torch.equal(counts.cpu().long(), torch.bincount(idx.cpu().reshape(-1), minlength=e))
    if not tied.any():
        assert torch.equal(counts.cpu().long(), rc)


@pytest.mark.parametrize("score_fn", ["softmax", "sigmoid"])
def test_router_back_end_with_selection_bias(ops, score_fn):
    """Experts chosen by prob + bias (src/layers/mlp.py:295-297), weights from the unbiased probs."""
    g = torch.Generator().manual_seed(21)
    t, e, k = 2048, 64, 4
    logits = torch.randn(t, e, generator=g)
    bias = 0.05 * torch.randn(e, generator=g)
    bias[7] = 5.0                                                   # always chosen
    bias[9] = -5.0                                                  # never chosen
    idx, w, probs, counts = ops.moe_router_topk(logits.cuda(), k, score_fn, True, select_bias=bias.cuda())
    p = logits.softmax(-1) if score_fn == "softmax" else logits.sigmoid()
    biased = p + bias
    ri = torch.topk(biased, k, dim=-1).indices
    # rows where the k-th and (k+1)-th biased scores are within rounding of each other may legitimately differ
    top = biased.topk(k + 1, -1).values
    clear = (top[:, :-1] - top[:, 1:]).min(-1).values > 1e-6
    assert clear.float().mean() > 0.99
    assert torch.equal(idx.cpu()[clear], ri[clear])
    assert (idx.cpu() == 7).any(-1).all() and not (idx.cpu() == 9).any()
    raw = p.gather(-1, idx.cpu())
    rw = (raw / (raw.sum(-1, keepdim=True) + 1e-9)).bfloat16()
    ulp = (w.cpu().view(torch.int16).int() - rw.view(torch.int16).int()).abs().max().item()
    assert ulp <= 1
    assert torch.equal(counts.cpu().long(), torch.bincount(idx.cpu().reshape(-1), minlength=e))


@pytest.mark.parametrize("compiled", [False, True])
def test_block_with_shared_experts_and_expert_bias(ops, compiled):
    from pretrain_b200.layers.mlp import SparseMoEBlock
    torch.manual_seed(3)
    d, inter, e, k, t = 256, 128, 8, 2, 512
    blk = SparseMoEBlock(d, intermediate_size=inter, n_routed_experts=e, n_routed_experts_per_token=k, n_shared_experts=2,
                         router_score_fn="sigmoid", aux_loss=False, expert_bias=True, expert_bias_update_rate=0.01).cuda().bfloat16()
    with torch.no_grad():
        blk.expert_gate_up.normal_(std=0.05)
        blk.expert_down.normal_(std=0.05)
        blk.router.expert_bias.bias[5] = 3.0                        # every token is routed to expert 5
    assert blk.router.gate.weight.dtype == torch.float32 and blk.router.expert_bias.bias.dtype == torch.float32
    fn = torch.compile(blk, fullgraph=True) if compiled else blk
    x = torch.randn(2, t // 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out, aux = fn(x)
    assert aux is None and out.shape == x.shape
    out.float().square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in blk.parameters())
    load = blk.expert_load.train_load
    assert load.sum().item() == t * k and load[5].item() == t
    # routed part + shared part: the shared block alone gives the difference to a block without it
    with torch.no_grad():
        shared = blk.shared_expert(x)[0]
        blk_shared, blk.shared_expert = blk.shared_expert, None
        routed = blk(x)[0]
        blk.shared_expert = blk_shared
    assert _rel(out.detach(), routed + shared) < 1e-2
    blk.post_step()                                                  # expert 5 is overloaded: its bias drops by the rate
    assert abs(blk.router.expert_bias.bias[5].item() - 2.99) < 1e-6 and blk.expert_load.train_load.sum().item() == 0


def test_router_module_matches_torch_router_and_backpropagates(ops):
    from pretrain_b200.layers.mlp import MoERouter
    torch.manual_seed(0)
    for score in ("softmax", "sigmoid"):
        r = MoERouter(128, 16, 4, router_score_fn=score).cuda()
        x = torch.randn(512, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        ti, tw, pr = r(x)
        # the same module on its plain torch path (fp32 input switches the fused back end off)
        logits = r.gate(x.float())
        p = logits.softmax(-1) if score == "softmax" else logits.sigmoid()
        rw, ri = torch.topk(p, 4, dim=-1)
        rw = rw / (rw.sum(-1, keepdim=True) + 1e-9)
        assert torch.equal(ti, ri)
        assert (tw.float() - rw).abs().max() <= 2 ** -8 * rw.abs().max()
        coef_w, coef_p = torch.randn_like(rw), torch.randn_like(p)
        (gx,) = torch.autograd.grad((tw.float() * coef_w).sum() + (pr.float() * coef_p).sum(), x, retain_graph=True)
        (rx,) = torch.autograd.grad((rw * coef_w).sum() + (p * coef_p).sum(), x)
        assert _rel(gx, rx) < 2e-2


def test_swiglu_backward_and_unpermute_backward(ops):
    g = torch.Generator().manual_seed(2)
    gu = (1.5 * torch.randn(300, 512, generator=g)).bfloat16().cuda().requires_grad_(True)
    dh = torch.randn(300, 256, generator=g).bfloat16().cuda()
    ref_h = F.silu(gu[:, :256].float()) * gu[:, 256:].float()
    (ref_dg,) = torch.autograd.grad(ref_h, gu, dh.float())
    dg = ops.swiglu_backward(gu.detach(), dh)
    assert _rel(dg, ref_dg) < 4e-3
    # unpermute backward against autograd through the gather-reduce written in torch
    t, k, d, e = 256, 2, 128, 8
    logits = torch.randn(t, e, generator=g)
    top_i, top_w = R.router_topk(logits, k)
    plan = ops.moe_permute_plan(top_i.cuda(), e)
    y = torch.randn(plan.padded_rows, d, generator=g).bfloat16().cuda().requires_grad_(True)
    w = top_w.cuda().float().requires_grad_(True)
    dout = torch.randn(t, d, generator=g).bfloat16().cuda()
    out = (y.float()[plan.row_of.long()].view(t, k, d) * w.unsqueeze(-1)).sum(1)
    ref_dy, ref_dw = torch.autograd.grad(out, (y, w), dout.float())
    dy, dw = ops.moe_unpermute_backward(dout, top_w.cuda(), y.detach(), plan)
    assert _rel(dy, ref_dy) < 4e-3 and _rel(dw, ref_dw) < 4e-3
    assert (dy[plan.src_of_row < 0] == 0).all()


def test_elementwise_steps_fused_with_the_dual_quantizer(ops):
    """gather / swiglu / unpermute-backward / swiglu-backward feeding the both-directions MXFP8 quantizer inside
    one kernel == the step's own kernel followed by quantize_mxfp8_dual, byte for byte."""
    g = torch.Generator().manual_seed(11)
    t, k, d, e, inter = 640, 2, 256, 8, 128
    x = torch.randn(t, d, generator=g).bfloat16().cuda()
    logits = torch.randn(t, e, generator=g)
    logits[:, 2] = -1e9
    top_i, top_w = R.router_topk(logits, k)
    plan = ops.moe_permute_plan(top_i.cuda(), e)
    live = int(plan.num_tiles.item()) * 128
    eq = lambda a, b: all(torch.equal(u, v) for u, v in zip(a, b))
    # gather (rows past the live tiles are zero rows in the fused form; the plain gather leaves them unwritten)
    a = ops.moe_gather(x, plan, False)
    a[live:] = 0
    assert eq(ops.moe_gather_quantize_dual(x, plan), ops.quantize_mxfp8_dual(a))
    # swiglu
    gu = (1.5 * torch.randn(plan.padded_rows, 2 * inter, generator=g)).bfloat16().cuda()
    assert eq(ops.swiglu_quantize_dual(gu), ops.quantize_mxfp8_dual(ops.swiglu(gu, False)))
    # unpermute backward
    dout = torch.randn(t, d, generator=g).bfloat16().cuda()
    dy, _ = ops.moe_unpermute_backward(dout, top_w.cuda(), torch.zeros(plan.padded_rows, d, dtype=torch.bfloat16, device="cuda"), plan)
    E5 = torch.float8_e5m2
    assert eq(ops.moe_unpermute_backward_quantize_dual(dout, top_w.cuda(), ops.moe_pair_of_row(plan), E5), ops.quantize_mxfp8_dual(dy, E5))
    # ... and with the routing weights' gradient from the same pass
    y = torch.randn(plan.padded_rows, d, generator=g).bfloat16().cuda()
    _, dw = ops.moe_unpermute_backward(dout, top_w.cuda(), y, plan)
    *codes, dw_fused = ops.moe_unpermute_backward_quantize_dual(dout, top_w.cuda(), ops.moe_pair_of_row(plan), E5, y=y, row_of=plan.row_of)
    assert eq(codes, ops.quantize_mxfp8_dual(dy, E5))
    ref_dw = (dout.float().unsqueeze(1) * y.float()[plan.row_of.long()].view(t, k, d)).sum(-1)
    assert dw_fused.shape == (t, k) and dw_fused.dtype == torch.float32
    assert _rel(dw_fused, ref_dw) < 1e-5 and _rel(dw_fused, dw) < 1e-5
    # swiglu backward (expert widths of one tile, and of one and a half tiles)
    for width in (inter, 192):
        gu = (1.5 * torch.randn(plan.padded_rows, 2 * width, generator=g)).bfloat16().cuda()
        dh = torch.randn(plan.padded_rows, width, generator=g).bfloat16().cuda()
        assert eq(ops.swiglu_backward_quantize_dual(gu, dh, E5), ops.quantize_mxfp8_dual(ops.swiglu_backward(gu, dh), E5))


def _moe_block_reference(x, gate_w, w_gu, w_d, k):
    """SparseMoEBlock.forward of the reference (src/layers/mlp.py:432-494, softmax router, SwiGLU experts,
    no aux loss) written as a per-expert loop in fp32."""
    t, d = x.shape
    e = w_gu.shape[0]
    probs = (x.float() @ gate_w.float().t()).softmax(-1)
    top_w, top_i = torch.topk(probs, k, dim=-1)
    top_w = top_w / (top_w.sum(-1, keepdim=True) + 1e-9)
    out = torch.zeros(t, d, device=x.device)
    for ei in range(e):
        tok, slot = (top_i == ei).nonzero(as_tuple=True)
        if tok.numel():
            hgu = x.float()[tok] @ w_gu[ei].float().t()
            gate, up = hgu.chunk(2, dim=-1)
            out = out.index_add(0, tok, (F.silu(gate) * up) @ w_d[ei].float().t() * top_w[tok, slot].unsqueeze(-1))
    return out


def test_sparse_moe_block_trains(ops):
    """Forward + backward of the block against the fp32 loop form under autograd: MXFP8 noise only."""
    from pretrain_b200.layers.mlp import SparseMoEBlock
    torch.manual_seed(0)
    d, inter, e, k, t = 256, 128, 8, 2, 1024
    blk = SparseMoEBlock(d, intermediate_size=inter, n_routed_experts=e, n_routed_experts_per_token=k, router_score_fn="softmax",
                         aux_loss=False).cuda()
    with torch.no_grad():
        blk.expert_gate_up.normal_(std=0.05)
        blk.expert_down.normal_(std=0.05)
        blk.router.gate.weight.normal_(std=0.5)
        blk.router.gate.weight[3] = -10.0 * blk.router.gate.weight[3].abs()       # an expert that gets (almost) nothing
    x = torch.randn(4, t // 4, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    coef = torch.randn(4, t // 4, d, device="cuda")
    out, aux = blk(x)
    assert aux is None and out.shape == x.shape
    (out.float() * coef).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    params = [p.detach().clone().requires_grad_(True) for p in (blk.router.gate.weight, blk.expert_gate_up, blk.expert_down)]
    ref = _moe_block_reference(xr.reshape(t, d), params[0], params[1].bfloat16(), params[2].bfloat16(), k)
    (ref * coef.reshape(t, d)).sum().backward()
    # the loop form is not quantized at all: every GEMM of the block adds a few % of MXFP8 rounding noise (E4M3
    # activations and weights, E5M2 gradients); measured 6.6 / 7.9 / 9.3 / 8.0 / 6.6 %.  A wiring error (a wrong
    # transposition, offset or expert) shows as ~100 %; the kernels themselves are held to 1e-2 in their own tests
    errs = {"out": _rel(out.reshape(t, d), ref), "dx": _rel(x.grad.reshape(t, d), xr.grad.reshape(t, d)),
            "dw_gate_up": _rel(blk.expert_gate_up.grad, params[1].grad), "dw_down": _rel(blk.expert_down.grad, params[2].grad),
            "dw_router": _rel(blk.router.gate.weight.grad, params[0].grad)}
    assert errs["out"] < 8e-2 and errs["dx"] < 1.2e-1 and errs["dw_gate_up"] < 1.2e-1 and errs["dw_down"] < 1.2e-1, errs
    assert errs["dw_router"] < 1.5e-1, errs
    opt = torch.optim.SGD(blk.parameters(), lr=1e-3)
    opt.step()
    assert all(torch.isfinite(p).all() for p in blk.parameters())


@pytest.mark.parametrize("gated,activation,bias", [(False, "relu2", True), (True, "gelu", True), (True, "silu", True), (False, "silu", False)])
@pytest.mark.parametrize("compiled", [False, True])
def test_block_trains_with_any_activation_and_biases(ops, gated, activation, bias, compiled):
    """The general trainable path (grouped linears with MXFP8 forward and backward, element-wise steps in torch)
    against the same block written as a per-expert fp32 loop under autograd."""
    from pretrain_b200.layers.mlp import GATED_ACTIVATIONS, UNGATED_ACTIVATIONS, SparseMoEBlock
    torch.manual_seed(4)
    d, inter, e, k, t = 256, 128, 8, 2, 1024
    blk = SparseMoEBlock(d, intermediate_size=inter, n_routed_experts=e, n_routed_experts_per_token=k, router_score_fn="softmax",
                         aux_loss=False, activation=activation, gated=gated, bias=bias).cuda()
    w_in = blk.expert_gate_up if gated else blk.expert_up
    b_in = blk.expert_gate_up_bias if gated else blk.expert_up_bias
    with torch.no_grad():
        w_in.normal_(std=0.05)
        blk.expert_down.normal_(std=0.05)
        blk.router.gate.weight.normal_(std=0.5)
        if bias:
            b_in.normal_(std=0.1)
            blk.expert_down_bias.normal_(std=0.1)
    fn = torch.compile(blk, fullgraph=True) if compiled else blk
    x = torch.randn(2, t // 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    coef = torch.randn(2, t // 2, d, device="cuda")
    out, _ = fn(x)
    (out.float() * coef).sum().backward()
    # fp32 loop form
    act = (GATED_ACTIVATIONS if gated else UNGATED_ACTIVATIONS)[activation]
    xr = x.detach().float().reshape(t, d).requires_grad_(True)
    params = [p.detach().float().clone().requires_grad_(True) for p in ([w_in, blk.expert_down] + ([b_in, blk.expert_down_bias] if bias else []))]
    probs = (xr @ blk.router.gate.weight.detach().float().t()).softmax(-1)
    tw, ti = torch.topk(probs, k, dim=-1)
    tw = tw / (tw.sum(-1, keepdim=True) + 1e-9)
    ref = torch.zeros(t, d, device="cuda")
    for ei in range(e):
        tok, slot = (ti == ei).nonzero(as_tuple=True)
        if tok.numel():
            pre = xr[tok].bfloat16().float() @ params[0][ei].bfloat16().float().t() + (params[2][ei] if bias else 0)
            hid = act(*pre.chunk(2, -1)) if gated else act(pre)
            y = hid @ params[1][ei].bfloat16().float().t() + (params[3][ei] if bias else 0)
            ref = ref.index_add(0, tok, y * tw[tok, slot].unsqueeze(-1))
    (ref * coef.reshape(t, d)).sum().backward()
    got = [w_in.grad, blk.expert_down.grad] + ([b_in.grad, blk.expert_down_bias.grad] if bias else [])
    errs = [_rel(out.reshape(t, d), ref)] + [_rel(a_, b_.grad) for a_, b_ in zip(got, params)]
    # MXFP8 noise of two chained GEMMs with E5M2 gradients; the first layer's bias gradient is a sum of signed
    # per-row terms that largely cancel, which amplifies that noise relative to the sum (a wiring error gives >= 1)
    limits = [1.3e-1, 1.3e-1, 1.3e-1, 3.5e-1, 1.3e-1]
    assert all(err < lim for err, lim in zip(errs, limits)), errs
    assert _rel(x.grad.reshape(t, d), xr.grad) < 1.5e-1


def test_expert_weight_copies_are_kept_until_the_weights_change(ops):
    from pretrain_b200.layers.mlp import SparseMoEBlock
    torch.manual_seed(8)
    blk = SparseMoEBlock(256, intermediate_size=128, n_routed_experts=8, n_routed_experts_per_token=2, router_score_fn="softmax",
                         aux_loss=False).cuda()
    with torch.no_grad():
        blk.expert_gate_up.normal_(std=0.05)
        blk.expert_down.normal_(std=0.05)
    x = torch.randn(1, 512, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        first = blk(x)[0]
        kept = blk.expert_gate_up._b200q_glu[1][0]
        assert blk(x)[0].equal(first) and blk.expert_gate_up._b200q_glu[1][0] is kept          # evaluation: quantized once
        blk.expert_gate_up.mul_(2.0)                                                            # what an optimizer step does
        second = blk(x)[0]
        assert blk.expert_gate_up._b200q_glu[1][0] is not kept and not second.equal(first)
    # training: two micro-batches share the copies, the optimizer step invalidates them
    xg = x.clone().requires_grad_(True)
    blk(xg)[0].float().sum().backward()
    dual = blk.expert_down._b200q_dual[1][0]
    blk(xg)[0].float().sum().backward()
    assert blk.expert_down._b200q_dual[1][0] is dual
    torch.optim.SGD(blk.parameters(), lr=1e-3).step()
    blk(xg)[0].float().sum().backward()
    assert blk.expert_down._b200q_dual[1][0] is not dual


def test_expert_dropout(ops):
    from pretrain_b200.layers.mlp import SparseMoEBlock
    torch.manual_seed(6)
    d, inter, e, k, t = 256, 128, 8, 2, 1024
    kw = dict(intermediate_size=inter, n_routed_experts=e, n_routed_experts_per_token=k, router_score_fn="softmax", aux_loss=False)
    plain, drop = SparseMoEBlock(d, **kw).cuda(), SparseMoEBlock(d, dropout=0.5, **kw).cuda()
    with torch.no_grad():
        plain.expert_gate_up.normal_(std=0.05)
        plain.expert_down.normal_(std=0.05)
    drop.load_state_dict(plain.state_dict())
    x = torch.randn(1, t, d, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = plain.eval()(x)[0]
        assert torch.equal(drop.eval()(x)[0], want)                       # identity outside training
    xg = x.clone().requires_grad_(True)
    out = drop.train()(xg)[0]
    out.float().square().mean().backward()
    assert torch.isfinite(xg.grad).all() and torch.isfinite(drop.expert_down.grad).all()
    # each expert output element survives with probability 1/2 and is doubled: same mean, about twice the energy
    ratio = (out.float().norm() / want.float().norm()).item()
    assert 1.1 < ratio < 1.8 and _rel(out, want) > 0.5


@pytest.mark.parametrize("train", [True, False])
def test_sparse_moe_block_traces_with_torch_compile(ops, train):
    """The reference compiles the whole model (src/training/trainer.py:176-177): the block must trace without a
    graph break, forward and backward, and give what it gives eagerly: the same kernels run, so the expert path is
    bit-identical; the router's torch arithmetic is re-fused by the compiler and may round differently."""
    from pretrain_b200.layers.mlp import SparseMoEBlock
    torch.manual_seed(1)
    d, inter, e, k, t = 256, 128, 8, 2, 512
    blk = SparseMoEBlock(d, intermediate_size=inter, n_routed_experts=e, n_routed_experts_per_token=k, router_score_fn="sigmoid",
                         aux_loss=True).cuda()
    with torch.no_grad():
        blk.expert_gate_up.normal_(std=0.05)
        blk.expert_down.normal_(std=0.05)
    compiled = torch.compile(blk, fullgraph=True)
    coef = torch.randn(2, t // 2, d, device="cuda")

    def run(fn):
        x = torch.randn(2, t // 2, d, device="cuda", dtype=torch.bfloat16, generator=torch.Generator("cuda").manual_seed(5))
        if not train:
            with torch.no_grad():
                out, aux = fn(x)
            return out, aux
        x.requires_grad_(True)
        blk.zero_grad()
        out, aux = fn(x)
        ((out.float() * coef).sum() + aux.float()).backward()
        return out, aux, x.grad, blk.expert_gate_up.grad.clone(), blk.expert_down.grad.clone(), blk.router.gate.weight.grad.clone()

    eager, traced = run(blk), run(compiled)
    assert torch.equal(eager[0], traced[0])
    for a, b in zip(eager[1:], traced[1:]):
        assert _rel(a.reshape(1, -1), b.reshape(1, -1)) < 2e-3


def test_swiglu(ops):
    g = torch.Generator().manual_seed(0)
    h = (2.0 * torch.randn(384, 768, generator=g)).bfloat16().cuda()
    ref = F.silu(h[:, :384]) * h[:, 384:]                             # the reference's bf16 tensor ops
    out = ops.swiglu(h, False)
    assert (out.float() - ref.float()).abs().max() <= 2 ** -7 * ref.float().abs().max()
    assert _rel(out, ref) < 3e-3
    codes, sf = ops.swiglu(h, True)
    rc, rsf = ops.quantize_mxfp8(out, 1)
    assert torch.equal(codes, rc) and torch.equal(sf, rsf)            # fused == unfused


def test_unpermute(ops, golden):
    top_i = torch.from_numpy(golden["moe_top_i"])
    top_w = bf16_from_bits(golden["moe_top_w"])
    eo = bf16_from_bits(golden["moe_expert_out"])
    plan = ops.moe_permute_plan(top_i.cuda(), 6)
    want_rows, tok = _check_plan(plan, top_i, 6)
    y_pad = torch.zeros(plan.padded_rows, eo.shape[1], dtype=torch.bfloat16)
    y_pad[want_rows] = eo
    out = ops.moe_unpermute(y_pad.cuda(), top_w.cuda(), plan.row_of, top_i.shape[0]).cpu()
    order = torch.from_numpy(golden["moe_order"])
    ref32 = R.moe_unpermute_fp32(eo, top_w.reshape(-1)[order], tok, top_i.shape[0])
    assert (out.float() - ref32.float()).abs().max() <= 2 ** -7 * ref32.float().abs().max()
    gold = bf16_from_bits(golden["moe_y"])                            # the reference's bf16 index_add_
    assert (out.float() - gold.float()).abs().max() <= 2e-2 * gold.float().abs().max()
    # no weights = unit weights; pair_of_row is the inverse of row_of with -1 on pad rows
    ones = torch.ones_like(top_w).cuda()
    assert torch.equal(ops.moe_unpermute(y_pad.cuda(), None, plan.row_of, top_i.shape[0]),
                       ops.moe_unpermute(y_pad.cuda(), ones, plan.row_of, top_i.shape[0]))
    inv = ops.moe_pair_of_row(plan).cpu()
    want = torch.full((plan.padded_rows,), -1, dtype=torch.int32)
    want[plan.row_of.cpu().long()] = torch.arange(top_i.numel(), dtype=torch.int32)
    assert torch.equal(inv, want)


def _mx_fake(t):
    c, s = R.quantize_mxfp8(t)
    return R.dequantize_mxfp8(c, s).to(t.dtype)


@pytest.mark.parametrize("counts", [[5, 0, 7, 4], [0, 5, 7, 4], [5, 7, 4, 0], [300, 40, 0, 129]])
def test_grouped_mlp_drop_in(ops, counts):
    from pretrain_b200.layers.mlp import grouped_mlp, silu_glu
    g = torch.Generator().manual_seed(len(counts) + counts[0])
    r, e, d, i = sum(counts), len(counts), 256, 128
    x = torch.randn(r, d, generator=g).bfloat16()
    w_in = (0.05 * torch.randn(e, 2 * i, d, generator=g)).bfloat16()
    w_down = (0.05 * torch.randn(e, d, i, generator=g)).bfloat16()
    offs = torch.tensor(counts).cumsum(0).int()
    with torch.no_grad():
        out = grouped_mlp(x.cuda(), w_in.cuda(), w_down.cuda(), silu_glu, offs.cuda(), True)
    assert out.shape == (r, d)
    ref = R.grouped_mlp_ref(x, w_in, w_down, offs, fake_quant=_mx_fake)
    assert _rel(out, ref) < 2e-2
    plain = R.grouped_mlp_ref(x, w_in, w_down, offs)                   # unquantized reference: only quantization noise apart
    assert _rel(out, plain) < 0.08
    # with gradients: the same function under autograd against the plain loop form in fp32
    xg, wi, wd = (t.cuda().requires_grad_(True) for t in (x, w_in, w_down))
    coef = torch.randn(r, d, generator=g).cuda()
    (grouped_mlp(xg, wi, wd, silu_glu, offs.cuda(), True).float() * coef).sum().backward()
    xr, wir, wdr = (t.cuda().float().requires_grad_(True) for t in (x, w_in, w_down))
    starts = [0] + offs.tolist()
    ref_rows = []
    for ei in range(e):
        seg = xr[starts[ei]:starts[ei + 1]]
        gate, up = (seg @ wir[ei].t()).chunk(2, -1)
        ref_rows.append((F.silu(gate) * up) @ wdr[ei].t())
    (torch.cat(ref_rows) * coef).sum().backward()
    assert _rel(xg.grad, xr.grad) < 1.5e-1
    live = [ei for ei, c in enumerate(counts) if c]
    assert _rel(wi.grad[live], wir.grad[live]) < 1.5e-1 and _rel(wd.grad[live], wdr.grad[live]) < 1.5e-1
    dead = [ei for ei, c in enumerate(counts) if not c]
    assert (wi.grad[dead] == 0).all() and (wd.grad[dead] == 0).all()      # experts without rows get exact zeros
    with pytest.raises(NotImplementedError):                               # widths the backward GEMMs cannot tile
        grouped_mlp(x.cuda()[:, :192].requires_grad_(True), w_in.cuda()[:, :, :192], w_down.cuda()[:, :192], silu_glu, offs.cuda(), True)


def test_grouped_mlp_against_reference_golden(ops, golden):
    from pretrain_b200.layers.mlp import grouped_mlp, silu_glu
    xs = bf16_from_bits(golden["moe_x_sorted"])
    w_in, w_down = bf16_from_bits(golden["moe_w_in"]), bf16_from_bits(golden["moe_w_down"])
    offs = torch.from_numpy(golden["moe_offs"])
    with torch.no_grad():
        out = grouped_mlp(xs.cuda(), w_in.cuda(), w_down.cuda(), silu_glu, offs.cuda(), True)
    gold = bf16_from_bits(golden["moe_expert_out"])                    # the reference's bf16 grouped_mlp
    assert _rel(out, gold) < 0.08


def test_sparse_moe_block_full_config(ops):
    """16384 tokens, hidden 768, 64 experts, top-4, intermediate 384: the block against the
    oracle's per-expert loop with fake-quantized operands on a sample of tokens, plus exact
    conservation of the routing (every pair lands in exactly one row)."""
    from pretrain_b200.layers.mlp import SparseMoEBlock
    x, logits, w_gu, w_d = R.inputs_moe()
    blk = SparseMoEBlock(768, intermediate_size=384, n_routed_experts=64, n_routed_experts_per_token=4,
                         router_score_fn="softmax").cuda()
    with torch.no_grad():
        blk.expert_gate_up.copy_(w_gu)
        blk.expert_down.copy_(w_d)
        torch.nn.init.normal_(blk.router.gate.weight, std=0.02)
        out, aux = blk(x.cuda().view(16, 1024, 768))
        top_i, top_w, _ = blk.router(x.cuda())
    assert out.shape == (16, 1024, 768) and torch.isfinite(out).all() and aux is not None and torch.isfinite(aux)
    top_i, top_w = top_i.cpu(), top_w.cpu()
    sample = torch.arange(0, 16384, 257)
    ref = torch.zeros(len(sample), 768)
    for n, t in enumerate(sample.tolist()):
        for j in range(4):
            e = top_i[t, j].item()
            h = (_mx_fake(x[t:t + 1]).float() @ _mx_fake(w_gu[e]).float().t()).bfloat16()
            h = R.silu_glu(*h.chunk(2, dim=-1))
            y = (_mx_fake(h).float() @ _mx_fake(w_d[e]).float().t()).bfloat16()
            ref[n] += top_w[t, j].float() * y[0].float()
    assert _rel(out.view(-1, 768)[sample], ref) < 2e-2


def test_fake_kernels_of_the_moe_ops_describe_the_real_outputs(ops):
    """torch.compile trusts every custom op's fake kernel for shapes, dtypes and strides: check them against what the
    real kernels return (torch.library.opcheck, fake-tensor test) on one routed batch."""
    from pretrain_b200 import torch_ops as T
    g = torch.Generator().manual_seed(12)
    t, k, d, e, inter = 384, 2, 256, 8, 128
    x = torch.randn(t, d, generator=g).bfloat16().cuda()
    logits = torch.randn(t, e, generator=g).cuda()
    check = lambda fn, *args: torch.library.opcheck(fn.op, args, test_utils="test_faketensor")
    check(T.moe_router_topk, logits, k, "softmax", True, None)
    check(T.moe_router_topk, logits, k, "sigmoid", False, torch.zeros(e, device="cuda"))
    top_i, top_w, _ = T.moe_router_topk(logits, k, "softmax", True, None)
    check(T._moe_permute_plan, top_i, e)
    plan = T.moe_permute_plan(top_i, e)
    check(T._moe_pad_plan, plan.offs, t * k)
    check(T._moe_gather_mxfp8, x, plan.src_of_row, plan.num_tiles, 0)
    check(T._moe_gather_quantize_dual, x, plan.src_of_row, 0)
    w_in = (0.05 * torch.randn(e, 2 * inter, d, generator=g)).bfloat16().cuda()
    w_down = (0.05 * torch.randn(e, d, inter, generator=g)).bfloat16().cuda()
    ar, asr, ac, asc = T.moe_gather_quantize_dual(x, plan, 0)
    w1r, w1sr, w1c, w1sc = T.quantize_mxfp8_dual(w_in.reshape(-1, d), 0, 1)
    check(T._grouped_gemm_mxfp8, ar, asr, w1r, w1sr, plan.tile_expert, plan.num_tiles, e, 2 * inter, 0, 0, 0)
    check(T.quantize_mxfp8_glu_rows, w_in.reshape(-1, d), e, inter)
    wg, wgs = T.quantize_mxfp8_glu_rows(w_in.reshape(-1, d), e, inter)
    check(T._grouped_gemm_mxfp8_swiglu, ar, asr, wg, wgs, plan.tile_expert, plan.num_tiles, e, 2 * inter)
    gu = T.grouped_gemm_mxfp8(ar, asr, w1r, w1sr, plan, 2 * inter)
    check(T.swiglu, gu)
    check(T.swiglu_mxfp8, gu, 0)
    check(T.swiglu_quantize_dual, gu, 0)
    hr, hsr, hc, hsc = T.swiglu_quantize_dual(gu, 0)
    w2r, w2sr, w2c, w2sc = T.quantize_mxfp8_dual(w_down.reshape(-1, inter), 0, 1)
    y = T.grouped_gemm_mxfp8(hr, hsr, w2r, w2sr, plan, d)
    check(T.moe_unpermute, y, top_w, plan.row_of, t)
    check(T.moe_unpermute, y, None, plan.row_of, t)
    dout = torch.randn(t, d, generator=g).bfloat16().cuda()
    check(T.moe_unpermute_backward_quantize_dual, dout, top_w, plan.row_of, plan.padded_rows, 1, y)
    check(T._moe_unpermute_backward, dout, top_w, y, plan.row_of, plan.src_of_row)
    dyr, dysr, dyc, dysc, _ = T.moe_unpermute_backward_quantize_dual(dout, top_w, plan.row_of, plan.padded_rows, 1, y)
    check(T._grouped_gemm_mxfp8, dyr, dysr, w2c, w2sc, plan.tile_expert, plan.num_tiles, e, inter, 1, 0, 1)
    check(T._grouped_gemm_mxfp8_wgrad, dyc, dysc, hc, hsc, plan.padded_offs, 1, 0)
    dh = T.grouped_gemm_mxfp8_dgrad(dyr, dysr, w2c, w2sc, plan, inter, 1, 0)
    check(T.swiglu_backward_quantize_dual, gu, dh, 1)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_expert_parallel_index_kernel_matches_its_restatement(ops, world):
    """b200q_moe_ep_index against oracle.restate.ep_index, for every rank of a simulated group (the counts of the other
    ranks are made up on the host; no second GPU is involved)."""
    t, e, k = 777, 64, 4
    g = torch.Generator().manual_seed(world)
    logits = torch.randn(world * t, e, generator=g)
    logits[:, 5] = -1e9
    top_all, _ = R.router_topk(logits, k)
    offs_all = torch.stack([R.moe_padded_plan(top_all[r * t:(r + 1) * t], e)[0] for r in range(world)])
    for rank in sorted({0, world // 2, world - 1}):
        mine = top_all[rank * t:(rank + 1) * t]
        plan = ops.moe_permute_plan(mine.cuda(), e)
        offs, padded_offs, row_of = R.moe_padded_plan(mine, e)
        assert torch.equal(plan.offs.cpu(), offs) and torch.equal(plan.padded_offs.cpu(), padded_offs) and torch.equal(plan.row_of.cpu(), row_of)
        got = ops.moe_ep_index(offs_all.cuda(), rank, mine.cuda(), plan)
        want = R.ep_index(offs_all, rank, mine, row_of, padded_offs)
        for a, b in zip(got, want):
            assert torch.equal(a.cpu(), b)


def test_peer_scatter_dots_and_barrier_on_one_rank(ops):
    """The expert-parallel row movers with a group of one (every "peer" is this GPU): the scatter is the inverse of the
    combine, the dot products are the routing weights' gradient, the flag barrier returns at once and stays clean."""
    t, d, e, k = 512, 256, 8, 2
    x, logits, _, _ = R.inputs_moe(t, d, e, k, 64, seed=4)
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w = x.cuda(), top_i.cuda(), top_w.cuda()
    plan = ops.moe_permute_plan(top_i, e)
    row_base, own_offs, pair_peer, pair_row = ops.moe_ep_index(plan.offs.view(1, e).contiguous(), 0, top_i, plan)
    assert torch.equal(pair_row, plan.row_of) and (pair_peer == 0).all() and torch.equal(own_offs, plan.offs)
    own = ops.moe_pad_plan(own_offs, t * k)
    buf = torch.full((own.padded_rows, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.moe_zero_pad_rows_bf16(own, buf)
    ops.moe_scatter_rows_peers(x, None, pair_peer, pair_row, k, [buf.data_ptr()], d)
    live = int(own.num_tiles.item()) * 128
    assert torch.equal(buf[:live], ops.moe_gather(x, plan, False)[:live])                 # the same padded layout, pad rows zero
    ops.moe_scatter_rows_peers(x, top_w, pair_peer, pair_row, k, [buf.data_ptr()], d)
    want = (top_w.float().reshape(-1, 1) * x.float().repeat_interleave(k, 0)).bfloat16()
    assert torch.equal(buf[plan.row_of.long()], want)
    dots = ops.moe_pair_dots_peers(x, [buf.data_ptr()], d, pair_peer, pair_row, k)
    ref = (x.float().repeat_interleave(k, 0) * want.float()).sum(1).view(t, k)
    assert ((dots - ref).abs().max() / ref.abs().max()).item() < 1e-5
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        ops.peer_barrier([flags.data_ptr()], 0, epoch)
    torch.cuda.synchronize()
    assert flags[0].item() == 3
    ops.device_status()


@pytest.mark.parametrize("form", ["bstat", "rowstat"])
@pytest.mark.parametrize("d,inter", [(768, 384), (512, 256), (256, 128)])
def test_stationary_grouped_gemms_equal_the_general_kernel_bit_for_bit(ops, d, inter, form):
    """The grouped GEMMs with the expert's weight tile, or the pair's rows of A, kept in shared memory against the general grouped kernel on a
    routing of BASELINE config 4's kind (many experts, ragged and empty ones, several thousand rows): same codes and
    scale bytes from the SwiGLU epilogue form, same bf16 outputs from the plain and the dgrad forms."""
    from pretrain_b200 import _lib
    lib = _lib.load()
    t, e, k = 4096, 32, 4
    x, logits, w_gu, w_d = R.inputs_moe(t, d, e, k, inter, seed=12)
    logits[:, 7] = -1e9
    logits[:, e - 1] = -1e9
    logits[:, 3] += 2.0
    top_i, _ = R.router_topk(logits, k)
    x, top_i, w_gu, w_d = x.cuda(), top_i.cuda(), w_gu.cuda(), w_d.cuda()
    plan = ops.moe_permute_plan(top_i, e)
    a, sfa = ops.moe_gather(x, plan, True)
    w1q, w1s = ops.quantize_mxfp8_rowmap(w_gu.view(e * 2 * inter, d), ops.glu_row_map(e, inter, "cuda"))
    w1p, w1ps = ops.quantize_mxfp8(w_gu.view(e * 2 * inter, d), 1)
    w2q, w2s = ops.quantize_mxfp8(w_d.view(e * d, inter), 1)
    w2t, w2ts = ops.quantize_mxfp8(w_d.view(e * d, inter), 0)                       # (inter, E*d): dgrad operand
    live = int(plan.num_tiles.item()) * 128
    res = {}
    for mode in (-1, 1):
        lib.b200q_debug_set_gemm_bstat(mode if form == "bstat" else -1)
        lib.b200q_debug_set_gemm_rowstat(mode if form == "rowstat" else -1)
        try:
            hq, hs = ops.grouped_gemm_mxfp8_swiglu(a, sfa, w1q, w1s, plan, 2 * inter)
            g = ops.grouped_gemm_mxfp8(a, sfa, w1p, w1ps, plan, 2 * inter)
            y = ops.grouped_gemm_mxfp8(hq, hs, w2q, w2s, plan, d)
            gy, gys = ops.quantize_mxfp8(y, 1, ops.E5M2)
            dh = ops.grouped_gemm_mxfp8_dgrad(gy, gys, w2t, w2ts, plan, inter, ops.E5M2, ops.E4M3)
            ops.device_status()
        finally:
            lib.b200q_debug_set_gemm_bstat(0)
            lib.b200q_debug_set_gemm_rowstat(0)
        n_sf = live // 128 * ((inter // 32 + 3) // 4) * 512
        res[mode] = (hq[:live].clone(), hs[:n_sf].clone(), g[:live].clone(), y[:live].clone(), dh[:live].clone())
    for got, want in zip(res[1], res[-1]):
        assert torch.equal(got, want)


@pytest.mark.parametrize("t,d,inter,e,k", [(4096, 768, 384, 64, 4), (1000, 256, 128, 8, 2), (512, 128, 64, 16, 1)])
def test_expert_path_in_one_call_equals_the_five_calls(ops, t, d, inter, e, k):
    """b200q_moe_ffn_forward against permute plan, gather + MXFP8, grouped GEMM with the SwiGLU epilogue, grouped GEMM and
    unpermute called one by one: the same output bits and the same per-expert offsets, with experts that get no token, twice
    in a row on one workspace (nothing in it needs to be cleared)."""
    x, logits, w_gu, w_d = R.inputs_moe(t, d, e, k, inter, seed=21)
    logits[:, 1] = -1e9                                               # an expert without tokens
    logits[:, e - 1] = -1e9
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = x.cuda(), top_i.cuda(), top_w.cuda(), w_gu.cuda(), w_d.cuda()
    w1q, w1s = ops.quantize_mxfp8_rowmap(w_gu.view(e * 2 * inter, d), ops.glu_row_map(e, inter, "cuda"))
    w2q, w2s = ops.quantize_mxfp8(w_d.view(e * d, inter), 1)
    plan = ops.moe_permute_plan(top_i, e)
    a, sfa = ops.moe_gather(x, plan, True)
    hq, hs = ops.grouped_gemm_mxfp8_swiglu(a, sfa, w1q, w1s, plan, 2 * inter)
    y = ops.grouped_gemm_mxfp8(hq, hs, w2q, w2s, plan, d)
    want = ops.moe_unpermute(y, top_w, plan.row_of, t)
    ws = torch.empty(ops.moe_ffn_workspace_bytes(t, k, d, e, inter), dtype=torch.uint8, device="cuda")
    ws.fill_(0xA5)
    for rep in range(2):
        got, offs = ops.moe_ffn_forward(x, top_i, top_w, w1q, w1s, w2q, w2s, e, inter, workspace=ws)
        ops.device_status()
        assert torch.equal(offs, plan.offs), rep
        assert torch.equal(got, want), (rep, int((got != want).sum()), int((got != want).any(1).sum()))
    got, offs = ops.moe_ffn_forward(x, top_i, top_w, w1q, w1s, w2q, w2s, e, inter)
    assert torch.equal(got, want)


@pytest.mark.parametrize("t,d,inter,e,k", [(4096, 768, 384, 64, 4), (1000, 256, 128, 8, 2)])
def test_trainable_expert_path_in_one_call_equals_the_separate_calls(ops, t, d, inter, e, k):
    """b200q_moe_ffn_train_forward / _backward against the same steps called one by one: every saved tensor, the output and
    all four gradients bit for bit (live rows; experts without tokens included)."""
    x, logits, w_gu, w_d = R.inputs_moe(t, d, e, k, inter, seed=31)
    logits[:, 2] = -1e9
    top_i, top_w = R.router_topk(logits, k)
    g0 = torch.Generator().manual_seed(7)
    dout = (0.01 * torch.randn(t, d, generator=g0)).bfloat16().cuda()
    x, top_i, top_w, w_gu, w_d = x.cuda(), top_i.cuda(), top_w.cuda(), w_gu.cuda(), w_d.cuda()
    w1r, w1sr, w1c, w1sc = ops.quantize_mxfp8_dual(w_gu.view(e * 2 * inter, d))
    w2r, w2sr, w2c, w2sc = ops.quantize_mxfp8_dual(w_d.view(e * d, inter))
    plan = ops.moe_permute_plan(top_i, e)
    live = int(plan.num_tiles.item()) * 128
    # one by one
    ar, asr, ac, asc = ops.moe_gather_quantize_dual(x, plan)
    g = ops.grouped_gemm_mxfp8(ar, asr, w1r, w1sr, plan, 2 * inter)
    hr, hsr, hc, hsc = ops.swiglu_quantize_dual(g)
    y = ops.grouped_gemm_mxfp8(hr, hsr, w2r, w2sr, plan, d)
    out = ops.moe_unpermute(y, top_w, plan.row_of, t)
    got = ops.moe_ffn_train_forward(x, top_w, plan, w1r, w1sr, w2r, w2sr, inter)
    ops.device_status()
    assert torch.equal(got[0], out) and torch.equal(got[1], ac) and torch.equal(got[2], asc)
    assert torch.equal(got[3][:live], g[:live]) and torch.equal(got[6][:live], y[:live])
    # the transposed copies of h cover every padded row, the dead ones included, whose gate / up rows no GEMM wrote: compare
    # the columns of the live rows
    assert torch.equal(got[4][:, :live], hc[:, :live])
    # backward, fed with the one-by-one forward's tensors on both sides
    dyr, dysr, dyc, dysc, dw = ops.moe_unpermute_backward_quantize_dual(dout, top_w, ops.moe_pair_of_row(plan), ops.E5M2, y=y, row_of=plan.row_of)
    dh = ops.grouped_gemm_mxfp8_dgrad(dyr, dysr, w2c, w2sc, plan, inter, ops.E5M2, ops.E4M3)
    dw2 = ops.grouped_gemm_mxfp8_wgrad(dyc, dysc, hc, hsc, plan, ops.E5M2, ops.E4M3)
    dgr, dgsr, dgc, dgsc = ops.swiglu_backward_quantize_dual(g, dh, ops.E5M2)
    da = ops.grouped_gemm_mxfp8_dgrad(dgr, dgsr, w1c, w1sc, plan, d, ops.E5M2, ops.E4M3)
    dw1 = ops.grouped_gemm_mxfp8_wgrad(dgc, dgsc, ac, asc, plan, ops.E5M2, ops.E4M3)
    dx = ops.moe_unpermute(da, None, plan.row_of, t)
    gdx, gdw, gdw1, gdw2 = ops.moe_ffn_train_backward(dout, top_w, plan, y, g, ac, asc, hc, hsc, w1c, w1sc, w2c, w2sc)
    ops.device_status()
    assert torch.equal(gdx, dx) and torch.equal(gdw, dw) and torch.equal(gdw1, dw1) and torch.equal(gdw2, dw2)
