"""Parity of the tcgen05 GEMMs (through the C-ABI) with dequantize-then-matmul in fp32:
max|out-ref|/max|ref| <= 1e-2 and Frobenius-relative <= 1e-2 (bf16 output, fp32 accumulate)."""

import pytest
import torch

from oracle import restate as R
from conftest import bf16_from_bits
import gpu_ref as G

pytestmark = pytest.mark.gpu
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
TOL = 1e-2


@pytest.fixture(scope="module")
def ops():
    from pretrain_b200 import build, ops
    build.build()
    return ops


def _check(out, ref):
    mx, fro = G.rel_errors(out, ref)
    assert mx <= TOL and fro <= TOL, (mx, fro)


def _rand(m, k, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(m, k, generator=g)).to(torch.bfloat16).cuda()


SHAPES = [(128, 128, 128), (128, 256, 512), (256, 512, 2048), (64, 96, 128), (32, 48, 64), (200, 264, 96),
          (1024, 768, 768), (384, 3072, 768)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("a_dt,b_dt", [(E4, E4), (E5, E4)])
def test_fp8_rowwise(ops, m, n, k, a_dt, b_dt):
    a, b = _rand(m, k, 1), _rand(n, k, 2, 0.02)
    ca, sa = ops.quantize_fp8(a, a_dt, 1)
    cb, sb = ops.quantize_fp8(b, b_dt, 1)
    out = ops.gemm_fp8(ca, a_dt, cb, b_dt, sa, sb)
    ops.device_status()
    ref = G.matmul_fp32(G.deq_fp8(ca, a_dt) * sa[:, None], G.deq_fp8(cb, b_dt) * sb[:, None])
    _check(out, ref)


def test_fp8_tensorwise_scalar_scales(ops):
    a, b = _rand(256, 512, 3), _rand(384, 512, 4)
    ca, sa = ops.quantize_fp8_tensorwise(a, E4)
    cb, sb = ops.quantize_fp8_tensorwise(b, E4)
    out = ops.gemm_fp8(ca, E4, cb, E4, sa, sb)
    ref = G.matmul_fp32(G.deq_fp8(ca, E4) * sa, G.deq_fp8(cb, E4) * sb)
    _check(out, ref)


def test_fp8_gemm_against_reference_golden(ops, golden):
    """The reference's own CPU result for its rowwise FP8 GEMM form (64 x 128 x 96)."""
    a, b = bf16_from_bits(golden["in_a"]).cuda(), bf16_from_bits(golden["in_b"]).cuda()
    ca, sa = ops.quantize_fp8(a, E4, 1)
    cb, sb = ops.quantize_fp8(b, E4, 0)          # b is (K, N): scales per column, codes as (N, K)
    out = ops.gemm_fp8(ca, E4, cb, E4, sa, sb).cpu()
    gold = bf16_from_bits(golden["gemm_rowwise_e4m3"])
    _check(out, gold)
    rel = (out.float() - gold.float()).norm() / gold.float().norm()
    assert rel < 0.02                             # the reference's own tolerance (tests/fast/quant/test_fp8.py:75)


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("a_dt,b_dt", [(E4, E4), (E5, E4)])
def test_mxfp8(ops, m, n, k, a_dt, b_dt):
    if k % 32:
        pytest.skip("K % 32")
    a, b = _rand(m, k, 5), _rand(n, k, 6, 0.02)
    ca, sfa = ops.quantize_mxfp8(a, 1, a_dt)
    cb, sfb = ops.quantize_mxfp8(b, 1, b_dt)
    out = ops.gemm_mxfp8(ca, sfa, cb, sfb, a_dt, b_dt)
    ops.device_status()
    ref = G.matmul_fp32(G.deq_mxfp8(ca, sfa, a_dt), G.deq_mxfp8(cb, sfb, b_dt))
    _check(out, ref)


def test_mxfp8_single_scale_factor_lands_where_expected(ops):
    """All-ones codes, unit scales except one (row, K-block): exactly that row of D changes,
    by exactly that block's contribution — checks the scale-factor layout end to end."""
    m, n, k = 256, 256, 512
    one = torch.full((1,), 1.0).to(E4).view(torch.uint8).item()
    ca = torch.full((m, k), one, dtype=torch.uint8, device="cuda")
    cb = torch.full((n, k), one, dtype=torch.uint8, device="cuda")
    for (row, kb, on_a) in [(5, 0, True), (37, 3, True), (130, 9, True), (255, 15, True), (70, 6, False), (200, 12, False)]:
        sfa = torch.full((m, k // 32), 127, dtype=torch.uint8, device="cuda")
        sfb = torch.full((n, k // 32), 127, dtype=torch.uint8, device="cuda")
        (sfa if on_a else sfb)[row, kb] = 130    # x8
        out = ops.gemm_mxfp8(ca, G.swizzle(sfa), cb, G.swizzle(sfb)).float()
        want = torch.full((m, n), float(k), device="cuda")
        if on_a:
            want[row, :] = k + 7 * 32
        else:
            want[:, row] = k + 7 * 32
        assert torch.equal(out, want), (row, kb, on_a)


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_nvfp4(ops, m, n, k):
    if k % 32:
        pytest.skip("K % 32")
    a, b = _rand(m, k, 7), _rand(n, k, 8, 0.02)
    pa, sfa, ta = ops.quantize_nvfp4(a, 1)
    pb, sfb, tb = ops.quantize_nvfp4(b, 1)
    out = ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb)
    ops.device_status()
    ref = G.matmul_fp32(G.deq_nvfp4(pa, sfa, ta), G.deq_nvfp4(pb, sfb, tb))
    _check(out, ref)


def test_nvfp4_single_scale_factor_lands_where_expected(ops):
    m, n, k = 256, 256, 512
    ca = torch.full((m, k // 2), 0x22, dtype=torch.uint8, device="cuda")      # E2M1 code 2 = 1.0, twice
    cb = torch.full((n, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    unit = torch.full((1,), 1.0).to(E4).view(torch.uint8).item()
    four = torch.full((1,), 4.0).to(E4).view(torch.uint8).item()
    one = torch.ones(1, device="cuda")
    for (row, kb, on_a) in [(3, 0, True), (45, 7, True), (129, 17, True), (250, 31, True), (66, 5, False), (222, 30, False)]:
        sfa = torch.full((m, k // 16), unit, dtype=torch.uint8, device="cuda")
        sfb = torch.full((n, k // 16), unit, dtype=torch.uint8, device="cuda")
        (sfa if on_a else sfb)[row, kb] = four
        out = ops.gemm_nvfp4(ca, G.swizzle(sfa), one, cb, G.swizzle(sfb), one).float()
        want = torch.full((m, n), float(k), device="cuda")
        if on_a:
            want[row, :] = k + 3 * 16
        else:
            want[:, row] = k + 3 * 16
        assert torch.equal(out, want), (row, kb, on_a)


@pytest.mark.parametrize("bn", [128, 192, 256])
@pytest.mark.parametrize("kind", ["fp8", "mxfp8", "nvfp4"])
@pytest.mark.parametrize("n", [768, 1000])
def test_every_tile_width(ops, bn, kind, n):
    """Width 192 starts every other B tile off the 128-row scale-factor groups (column offset into
    the tensor-memory scale block); n = 1000 adds a ragged last tile."""
    from pretrain_b200 import _lib
    a, b = _rand(512, 1024, 9), _rand(n, 1024, 10)
    _lib.load().b200q_debug_set_gemm_bn(bn)
    try:
        if kind == "fp8":
            ca, sa = ops.quantize_fp8(a, E4, 1); cb, sb = ops.quantize_fp8(b, E4, 1)
            out = ops.gemm_fp8(ca, E4, cb, E4, sa, sb)
            ref = G.matmul_fp32(G.deq_fp8(ca, E4) * sa[:, None], G.deq_fp8(cb, E4) * sb[:, None])
        elif kind == "mxfp8":
            ca, sfa = ops.quantize_mxfp8(a); cb, sfb = ops.quantize_mxfp8(b)
            out = ops.gemm_mxfp8(ca, sfa, cb, sfb)
            ref = G.matmul_fp32(G.deq_mxfp8(ca, sfa), G.deq_mxfp8(cb, sfb))
        else:
            pa, sfa, ta = ops.quantize_nvfp4(a); pb, sfb, tb = ops.quantize_nvfp4(b)
            out = ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb)
            ref = G.matmul_fp32(G.deq_nvfp4(pa, sfa, ta), G.deq_nvfp4(pb, sfb, tb))
    finally:
        _lib.load().b200q_debug_set_gemm_bn(0)
    _check(out, ref)


@pytest.mark.parametrize("kind", ["fp8", "mxfp8", "nvfp4"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 512, 1024), (300, 520, 256), (2048, 1024, 4096), (128, 256, 96)])
def test_cta_pair_kernel(ops, kind, m, n, k):
    """The dense GEMMs on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2), forced on for shapes
    with ragged rows / columns / K as well."""
    from pretrain_b200 import _lib
    a, b = _rand(m, k, 11), _rand(n, k, 12)
    _lib.load().b200q_debug_set_gemm_pair(1)
    try:
        if kind == "fp8":
            ca, sa = ops.quantize_fp8(a, E4, 1); cb, sb = ops.quantize_fp8(b, E4, 1)
            out = ops.gemm_fp8(ca, E4, cb, E4, sa, sb)
            ref = G.matmul_fp32(G.deq_fp8(ca, E4) * sa[:, None], G.deq_fp8(cb, E4) * sb[:, None])
        elif kind == "mxfp8":
            ca, sfa = ops.quantize_mxfp8(a); cb, sfb = ops.quantize_mxfp8(b)
            out = ops.gemm_mxfp8(ca, sfa, cb, sfb)
            ref = G.matmul_fp32(G.deq_mxfp8(ca, sfa), G.deq_mxfp8(cb, sfb))
        else:
            pa, sfa, ta = ops.quantize_nvfp4(a); pb, sfb, tb = ops.quantize_nvfp4(b)
            out = ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb)
            ref = G.matmul_fp32(G.deq_nvfp4(pa, sfa, ta), G.deq_nvfp4(pb, sfb, tb))
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_pair(0)
    _check(out, ref)


@pytest.mark.parametrize("bn,pair", [(0, -1), (128, -1), (192, -1), (256, -1), (0, 1)])
@pytest.mark.parametrize("m,d,inter", [(300, 512, 256), (1024, 1024, 384)])
def test_nvfp4_gemm_with_swiglu_epilogue(ops, bn, pair, m, d, inter):
    """GEMM with the SwiGLU -> bf16 + amax epilogue over interleaved NVFP4 weights == GEMM to bf16,
    stand-alone SwiGLU, amax kernel: the same bits."""
    from pretrain_b200 import _lib
    x, w = _rand(m, d, 31), _rand(2 * inter, d, 32) * 0.05
    px, sx, tx = ops.quantize_nvfp4(x)
    pw, sw, tw = ops.quantize_nvfp4(w)
    want = ops.swiglu(ops.gemm_nvfp4(px, sx, tx, pw, sw, tw), False)
    pwi, swi, twi = ops.quantize_nvfp4_rowmap(w, ops.glu_row_map(1, inter, "cuda"))
    assert torch.equal(twi, tw)
    _lib.load().b200q_debug_set_gemm_bn(bn)
    _lib.load().b200q_debug_set_gemm_pair(pair)                   # never / always the CTA-pair kernel
    try:
        h, am = ops.gemm_nvfp4_swiglu(px, sx, tx, pwi, swi, twi)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_bn(0)
        _lib.load().b200q_debug_set_gemm_pair(0)
    assert torch.equal(h, want)
    assert am.item() == ops.amax(want).item() == want.float().abs().max().item()


@pytest.mark.parametrize("bn,pair", [(0, -1), (128, -1), (256, -1), (0, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (1024, 768, 768), (2048, 2048, 1024), (384, 1280, 96)])
def test_gemm_with_mxfp8_quantized_output(ops, bn, pair, m, n, k):
    """The GEMM whose epilogue quantizes its own bf16 result along the columns == the plain GEMM followed by
    the row-wise MXFP8 quantizer: the same codes and the same swizzled scale bytes."""
    from pretrain_b200 import _lib
    a, b = _rand(m, k, 41), _rand(n, k, 42, 0.05)
    ca, sfa = ops.quantize_mxfp8(a); cb, sfb = ops.quantize_mxfp8(b)
    want_c, want_sf = ops.quantize_mxfp8(ops.gemm_mxfp8(ca, sfa, cb, sfb), 1)
    _lib.load().b200q_debug_set_gemm_bn(bn)
    _lib.load().b200q_debug_set_gemm_pair(pair)
    try:
        got_c, got_sf = ops.gemm_mxfp8_quantized(ca, sfa, cb, sfb)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_bn(0)
        _lib.load().b200q_debug_set_gemm_pair(0)
    assert torch.equal(got_c, want_c)
    assert torch.equal(got_sf, want_sf)
    # and it is a valid A operand for the next GEMM
    w2 = _rand(256, n, 43, 0.05)
    c2, sf2 = ops.quantize_mxfp8(w2)
    assert torch.equal(ops.gemm_mxfp8(got_c, got_sf, c2, sf2), ops.gemm_mxfp8(want_c, want_sf, c2, sf2))


def test_quantized_output_refuses_partial_tiles(ops):
    from pretrain_b200 import _lib
    import ctypes
    z = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    one = (ctypes.c_void_p * 1)(z.data_ptr())
    for m, n in ((96, 128), (128, 96), (128, 192 + 32)):
        assert _lib.load().b200q_gemm_mxfp8_allgather_mxfp8(z.data_ptr(), 0, z.data_ptr(), z.data_ptr(), 0, z.data_ptr(), m, n, 128,
                                                            one, one, 1, 0, 256, None) == -2


def _int8_ref(ca, cb, sa, sb):
    """The reference's formula (src/quant/int8.py:52-53) with an exact integer product."""
    acc = (ca.double() @ cb.double().t()).to(torch.int32)            # |acc| < 2^31: exact in fp64
    return (acc.float() * sa.view(-1, 1) * sb.view(1, -1)).bfloat16()


@pytest.mark.parametrize("bn,pair", [(0, 0), (128, 0), (192, 0), (256, 0), (0, 1)])
@pytest.mark.parametrize("m,n,k", [(512, 768, 1024), (300, 520, 256), (128, 256, 96), (2048, 1024, 4096)])
def test_int8_gemm_is_bit_exact(ops, bn, pair, m, n, k):
    """kind::i8 accumulates exactly, so every tile width and both kernels must give the reference's
    bits; per-row scales and one-per-tensor scales."""
    from pretrain_b200 import _lib
    a, b = _rand(m, k, 21), _rand(n, k, 22)
    ca, sa = ops.quantize_int8(a, 127, 1)
    cb, sb = ops.quantize_int8(b, 31, 1)
    ta, tsa = ops.quantize_int8_tensorwise(a, 127)
    tb, tsb = ops.quantize_int8_tensorwise(b, 127)
    _lib.load().b200q_debug_set_gemm_bn(bn)
    _lib.load().b200q_debug_set_gemm_pair(1 if pair else -1)       # always / never the CTA-pair kernel
    try:
        out = ops.gemm_int8(ca, cb, sa, sb)
        out_t = ops.gemm_int8(ta, tb, tsa, tsb)
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_bn(0)
        _lib.load().b200q_debug_set_gemm_pair(0)
    assert torch.equal(out, _int8_ref(ca, cb, sa, sb))
    assert torch.equal(out_t, _int8_ref(ta, tb, tsa.expand(m), tsb.expand(n)))


def test_mxfp8_linear_config_against_cpu_oracle(ops):
    """GPT-2 MLP up-projection (X[8192,768] . W[3072,768]^T, seed 0): the full path against
    the CPU oracle's dequantize-then-matmul on a row sample."""
    x, w = R.inputs_mxfp8_linear()
    ca, sfa = ops.quantize_mxfp8(x.cuda())
    cb, sfb = ops.quantize_mxfp8(w.cuda())
    out = ops.gemm_mxfp8(ca, sfa, cb, sfb).cpu()
    rows = torch.arange(0, 8192, 61)
    ref = R.mxfp8_gemm_ref(x[rows], w.t())
    _check(out[rows], ref)


def test_largest_square_16384(ops):
    """16384^3, the largest benchmark size (8.8 TFLOP, tile and K-step counts at their maxima for the
    configurations of record): sampled rows against the fp32 reference, and the GEMM of the row-reversed
    operand equals the row-reversed GEMM (the output rows are independent), bit for bit."""
    g = torch.Generator(device="cuda").manual_seed(3)
    n = 16384
    a = torch.randn(n, n, generator=g, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, n, generator=g, device="cuda", dtype=torch.bfloat16)
    ca, sfa = ops.quantize_mxfp8(a); cb, sfb = ops.quantize_mxfp8(b)
    out = ops.gemm_mxfp8(ca, sfa, cb, sfb)
    ops.device_status()
    rows = torch.arange(5, n, 331, device="cuda")
    _check(out[rows], G.matmul_fp32(G.deq_mxfp8(ca, sfa)[rows], G.deq_mxfp8(cb, sfb)))
    del cb, sfb
    ca2, sfa2 = ops.quantize_mxfp8(a.flip(0).contiguous())
    cb, sfb = ops.quantize_mxfp8(b)
    out2 = ops.gemm_mxfp8(ca2, sfa2, cb, sfb)
    assert torch.equal(out2.flip(0), out)


def test_large_square_linearity(ops):
    """8192^3 (the headline size): compared on sampled rows with an fp32 reference, plus
    linearity in the scale factors (doubling every A scale doubles D exactly)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(8192, 8192, generator=g, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(8192, 8192, generator=g, device="cuda", dtype=torch.bfloat16)
    ca, sfa = ops.quantize_mxfp8(a); cb, sfb = ops.quantize_mxfp8(b)
    out = ops.gemm_mxfp8(ca, sfa, cb, sfb)
    ops.device_status()
    rows = torch.arange(0, 8192, 97, device="cuda")
    ref = G.matmul_fp32(G.deq_mxfp8(ca, sfa)[rows], G.deq_mxfp8(cb, sfb))
    _check(out[rows], ref)
    out2 = ops.gemm_mxfp8(ca, sfa + 1, cb, sfb)
    assert torch.equal(out2.float(), out.float() * 2)
    pa, sa4, ta = ops.quantize_nvfp4(a); pb, sb4, tb = ops.quantize_nvfp4(b)
    out4 = ops.gemm_nvfp4(pa, sa4, ta, pb, sb4, tb)
    ref4 = G.matmul_fp32(G.deq_nvfp4(pa, sa4, ta)[rows], G.deq_nvfp4(pb, sb4, tb))
    _check(out4[rows], ref4)


@pytest.mark.parametrize("pair", [-1, 1])
def test_scatter_epilogue_and_slot_sum_on_one_gpu(ops, pair):
    """The reduce-scatter form with both "ranks" played in turn on one GPU (no kernel waits on another): every rank's
    partial product lands in its slot of the owner's staging buffer, and the slot sum is the fp32 sum of the bf16
    partials rounded once."""
    from pretrain_b200 import _lib
    world, m, n, k = 2, 512, 384, 256            # result (m, n), contraction k; owner g holds rows [g * 256, ...)
    g = torch.Generator().manual_seed(3)
    stage = [torch.full((world, m // world, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = [t.data_ptr() for t in stage]
    parts = []
    _lib.load().b200q_debug_set_gemm_pair(pair)
    try:
        for rank in range(world):
            a = torch.randn(m, k, generator=g).bfloat16().cuda()
            b = torch.randn(n, k, generator=g).bfloat16().cuda()
            ca, sa = ops.quantize_mxfp8(a, 1)
            cb, sb = ops.quantize_mxfp8(b, 1)
            ops.gemm_mxfp8_scatter(ca, sa, cb, sb, ptrs, rank, n, n)
            parts.append(ops.gemm_mxfp8(ca, sa, cb, sb))
        ops.device_status()
    finally:
        _lib.load().b200q_debug_set_gemm_pair(0)
    for owner in range(world):
        rows = slice(owner * (m // world), (owner + 1) * (m // world))
        for rank in range(world):
            assert torch.equal(stage[owner][rank], parts[rank][rows])
        want = torch.stack([p[rows].float() for p in parts]).sum(0).bfloat16()
        assert torch.equal(ops.sum_slots(stage[owner]), want)
