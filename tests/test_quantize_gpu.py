"""Parity of the CUDA quantizers, called through the C-ABI, with the CPU oracle: codes and
scales bit-exact (integer / byte outputs), on seeded inputs, golden fixtures and edge cases."""

import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import restate as R
from conftest import ROOT, bf16_from_bits

pytestmark = pytest.mark.gpu
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def G_unswizzle(sf, outer, nblk):
    import gpu_ref
    return gpu_ref.unswizzle(sf, outer, nblk)


@pytest.fixture(scope="module")
def ops():
    from pretrain_b200 import build, ops
    build.build()
    return ops


def _cases():
    g = torch.Generator().manual_seed(5)
    x, w = R.inputs_mxfp8_linear(512, 768, 384)
    xo, wgu, _ = R.inputs_nvfp4_mlp(256, 1024, 64)
    wide = torch.randn(96, 160, generator=g) * torch.exp2(torch.randint(-30, 30, (96, 160), generator=g).float())
    tiny = torch.randn(32, 64, generator=g) * 1e-20
    zeros = torch.zeros(32, 32)
    big = torch.randn(64, 4352, generator=g) * 3        # > 4096 columns: re-read path of the per-row kernel
    odd = torch.randn(160, 96, generator=g)             # partial tiles in both directions
    # one huge element per 32-block next to tiny, subnormal and signed-zero ones: the scaled values fall
    # below every format's smallest subnormal and must come out as zeros that keep their sign
    span = torch.randn(64, 128, generator=g) * 1e-30
    span[:, ::32] = 3.0e38 * torch.sign(torch.randn(64, 4, generator=g))
    span[:, 1::32] = -0.0
    span[:, 2::32] = -1e-39
    span[:, 3::32] = 2.0 ** -126
    span[1::2, 4::32] = -(2.0 ** -133)
    return {"span": span.bfloat16(), "x": x, "w": w, "outlier": xo, "wgu": wgu, "wide": wide.bfloat16(), "tiny": tiny.bfloat16(),
            "zeros": zeros.bfloat16(), "long": big.bfloat16(), "odd": odd.bfloat16()}


CASES = _cases()


@pytest.mark.parametrize("name", list(CASES))
def test_amax(ops, name):
    x = CASES[name]
    got = ops.amax(x.cuda()).cpu()
    assert got.item() == x.abs().max().float().item()


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("dt", [E4, E5])
@pytest.mark.parametrize("axis", [1, 0])
def test_fp8_row_and_col(ops, name, dt, axis):
    x = CASES[name]
    codes, scales = ops.quantize_fp8(x.cuda(), dt, axis)
    rc, rs = R.quantize_fp8(x, dt, dim=-1 if axis == 1 else 0)
    rc = rc.view(torch.uint8)
    if axis == 0:
        rc = rc.t().contiguous()
    assert torch.equal(scales.cpu().view(torch.int32), rs.reshape(-1).view(torch.int32))
    assert torch.equal(codes.cpu(), rc)


@pytest.mark.parametrize("name", ["x", "wide", "zeros", "odd"])
@pytest.mark.parametrize("dt", [E4, E5])
@pytest.mark.parametrize("transpose", [False, True])
def test_fp8_tensorwise(ops, name, dt, transpose):
    x = CASES[name]
    codes, scale = ops.quantize_fp8_tensorwise(x.cuda(), dt, transpose)
    rc, rs = R.quantize_fp8(x, dt, None)
    rc = rc.view(torch.uint8)
    assert scale.cpu().view(torch.int32).item() == rs.view(torch.int32).item()
    assert torch.equal(codes.cpu(), rc.t().contiguous() if transpose else rc)


def test_fp8_matches_reference_golden(ops, golden):
    for name in ("a", "b", "grad", "edge"):
        x = bf16_from_bits(golden[f"in_{name}"])
        for dname, dt in (("e4m3", E4), ("e5m2", E5)):
            codes, scales = ops.quantize_fp8(x.cuda(), dt, 1)
            assert np.array_equal(codes.cpu().numpy(), golden[f"q_{name}_{dname}_row_codes"])
            assert np.array_equal(scales.cpu().numpy().view(np.uint32), golden[f"q_{name}_{dname}_row_scale"].view(np.uint32))
            codes, scales = ops.quantize_fp8(x.cuda(), dt, 0)
            assert np.array_equal(codes.cpu().numpy(), golden[f"q_{name}_{dname}_col_codes"].T)
            assert np.array_equal(scales.cpu().numpy().view(np.uint32), golden[f"q_{name}_{dname}_col_scale"].view(np.uint32))
            codes, scale = ops.quantize_fp8_tensorwise(x.cuda(), dt)
            assert np.array_equal(codes.cpu().numpy(), golden[f"q_{name}_{dname}_tensor_codes"])


@pytest.mark.parametrize("name", ["x", "w", "outlier", "wide", "tiny", "zeros", "long", "odd"])
@pytest.mark.parametrize("qmax", [127, 31, 7])
def test_int8_series_row_col_tensor(ops, name, qmax):
    x = CASES[name]
    xc = x.cuda()
    codes, scales = ops.quantize_int8(xc, qmax, 1)
    rc, rs = R.quantize_int8(x, qmax, dim=-1)
    assert torch.equal(codes.cpu(), rc) and torch.equal(scales.cpu().view(torch.int32), rs.reshape(-1).view(torch.int32))
    if x.shape[0] % 16 == 0:
        codes, scales = ops.quantize_int8(xc, qmax, 0)
        rc, rs = R.quantize_int8(x, qmax, dim=0)
        assert torch.equal(codes.cpu(), rc.t()) and torch.equal(scales.cpu().view(torch.int32), rs.reshape(-1).view(torch.int32))
        codes, scale = ops.quantize_int8_tensorwise(xc, qmax, True)
        rc, rs = R.quantize_int8(x, qmax, None)
        assert torch.equal(codes.cpu(), rc.t()) and scale.item() == rs.item()
    codes, scale = ops.quantize_int8_tensorwise(xc, qmax, False)
    rc, rs = R.quantize_int8(x, qmax, None)
    assert torch.equal(codes.cpu(), rc) and scale.item() == rs.item()


def test_int8_matches_reference_golden(ops, golden, golden_int8):
    for name in ("a", "b", "grad", "edge"):
        x = bf16_from_bits(golden[f"in_{name}"]).cuda()
        for qmax in (127, 63, 31, 15, 7):
            codes, scales = ops.quantize_int8(x, qmax, 1)
            assert np.array_equal(codes.cpu().numpy(), golden_int8[f"q_{name}_{qmax}_row_codes"])
            assert np.array_equal(scales.cpu().numpy().view(np.uint32), golden_int8[f"q_{name}_{qmax}_row_scale"].view(np.uint32))
            codes, scales = ops.quantize_int8(x, qmax, 0)
            assert np.array_equal(codes.cpu().numpy(), golden_int8[f"q_{name}_{qmax}_col_codes"].T)
            assert np.array_equal(scales.cpu().numpy().view(np.uint32), golden_int8[f"q_{name}_{qmax}_col_scale"].view(np.uint32))
            codes, scale = ops.quantize_int8_tensorwise(x, qmax)
            assert np.array_equal(codes.cpu().numpy(), golden_int8[f"q_{name}_{qmax}_tensor_codes"])
            assert np.array_equal(scale.cpu().numpy().view(np.uint32), golden_int8[f"q_{name}_{qmax}_tensor_scale"].view(np.uint32))


def test_fp8_digests_at_benchmark_size(ops):
    """FP8 training triple (M=16384, K=N=2048): sha256 of codes and scales equals what the
    reference's quantize_fp8 produced for the same seeded inputs."""
    with open(os.path.join(ROOT, "tests", "golden", "ref_digests.json")) as f:
        dig = json.load(f)
    x, w, dy = R.inputs_fp8_triple()

    def sha(t):
        return hashlib.sha256(t.cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()

    # name -> (tensor, dtype, axis, codes come out transposed relative to the reference's)
    table = {
        "fprop_x_row_e4m3": (x, E4, 1, False), "fprop_wT_col_e4m3": (w, E4, 1, True),
        "dgrad_dy_row_e5m2": (dy, E5, 1, False), "dgrad_w_col_e4m3": (w, E4, 0, True),
        "wgrad_dyT_row_e5m2": (dy, E5, 0, False), "wgrad_x_col_e4m3": (x, E4, 0, True),
    }
    for name, (t, dt, axis, transposed) in table.items():
        codes, scales = ops.quantize_fp8(t.cuda(), dt, axis)
        ref_layout = codes.t().contiguous() if transposed else codes
        assert list(ref_layout.shape) == dig[name]["shape"]
        assert sha(ref_layout) == dig[name]["codes"], name
        assert sha(scales) == dig[name]["scale"], name


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n].shape[1] % 32 == 0])
@pytest.mark.parametrize("dt", [E4, E5])
@pytest.mark.parametrize("layout", [0, 1])
def test_mxfp8_rowwise(ops, name, dt, layout):
    x = CASES[name]
    codes, sf = ops.quantize_mxfp8(x.cuda(), 1, dt, layout)
    rc, rs = R.quantize_mxfp8(x, -1, dt)
    want_sf = R.swizzle_sf(rs) if layout else rs.reshape(-1)
    assert torch.equal(sf.cpu(), want_sf)
    assert torch.equal(codes.cpu(), rc)


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n].shape[0] % 32 == 0])
@pytest.mark.parametrize("dt", [E4, E5])
@pytest.mark.parametrize("layout", [0, 1])
def test_mxfp8_transposing(ops, name, dt, layout):
    x = CASES[name]
    codes, sf = ops.quantize_mxfp8(x.cuda(), 0, dt, layout)
    rc, rs = R.quantize_mxfp8(x, 0, dt)
    want_sf = R.swizzle_sf(rs) if layout else rs.reshape(-1)
    assert codes.shape == (x.shape[1], x.shape[0])
    assert torch.equal(sf.cpu(), want_sf)
    assert torch.equal(codes.cpu(), rc)


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n].shape[1] % 32 == 0])
@pytest.mark.parametrize("layout", [0, 1])
def test_nvfp4_rowwise(ops, name, layout):
    x = CASES[name]
    packed, sf, ts = ops.quantize_nvfp4(x.cuda(), 1, None, layout)
    rp, rs, rt = R.quantize_nvfp4(x)
    assert ts.cpu().view(torch.int32).item() == rt.view(torch.int32).item()
    assert torch.equal(sf.cpu(), R.swizzle_sf(rs) if layout else rs.reshape(-1))
    assert torch.equal(packed.cpu(), rp)


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n].shape[0] % 32 == 0])
@pytest.mark.parametrize("layout", [0, 1])
def test_nvfp4_transposing(ops, name, layout):
    x = CASES[name]
    packed, sf, ts = ops.quantize_nvfp4(x.cuda(), 0, None, layout)
    rp, rs, rt = R.quantize_nvfp4(x, 0)
    assert packed.shape == (x.shape[1], x.shape[0] // 2)
    assert torch.equal(sf.cpu(), R.swizzle_sf(rs) if layout else rs.reshape(-1))
    assert torch.equal(packed.cpu(), rp)


def test_strided_input_is_read_in_place(ops):
    x = CASES["x"]
    big = torch.zeros(x.shape[0], x.shape[1] + 64, dtype=torch.bfloat16)
    big[:, : x.shape[1]] = x
    view = big.cuda()[:, : x.shape[1]]
    codes, sf = ops.quantize_mxfp8(view, 1, E4, 0)
    rc, rs = R.quantize_mxfp8(x, -1, E4)
    assert torch.equal(codes.cpu(), rc) and torch.equal(sf.cpu(), rs.reshape(-1))


@pytest.mark.parametrize("shape", [(512, 768), (96, 160), (32, 32), (160, 96), (384, 4352)])
@pytest.mark.parametrize("dt", [E4, E5])
@pytest.mark.parametrize("layout", [0, 1])
def test_mxfp8_both_directions_in_one_pass(ops, shape, dt, layout):
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    x = (torch.randn(*shape, generator=g) * torch.exp2(torch.randint(-6, 6, shape, generator=g).float())).bfloat16().cuda()
    cr, sr, cc, sc = ops.quantize_mxfp8_dual(x, dt, layout)
    r1, s1 = ops.quantize_mxfp8(x, 1, dt, layout)
    r0, s0 = ops.quantize_mxfp8(x, 0, dt, layout)
    assert torch.equal(cr, r1) and torch.equal(sr, s1) and torch.equal(cc, r0) and torch.equal(sc, s0)
    # and against the oracle directly
    oc, osf = R.quantize_mxfp8(x.cpu(), 0, dt)
    assert torch.equal(cc.cpu(), oc)
    assert torch.equal((G_unswizzle(sc, shape[1], shape[0] // 32) if layout else sc.view(shape[1], -1)).cpu(), osf)


@pytest.mark.parametrize("dt", [E4, E5])
def test_mxfp8_both_directions_on_blocks_that_span_the_exponent_range(ops, dt):
    x = CASES["span"].cuda()
    cr, sr, cc, sc = ops.quantize_mxfp8_dual(x, dt, 0)
    for axis, codes, sf in ((-1, cr, sr), (0, cc, sc)):
        oc, osf = R.quantize_mxfp8(x.cpu(), axis, dt)
        assert torch.equal(codes.cpu(), oc) and torch.equal(sf.cpu().reshape(-1), osf.reshape(-1))


@pytest.mark.parametrize("shape", [(512, 768), (96, 160), (16, 8), (160, 96), (64, 4352), (2048, 8192)])
@pytest.mark.parametrize("dt", [E4, E5])
def test_fp8_rows_and_columns_in_two_reads(ops, shape, dt):
    g = torch.Generator().manual_seed(shape[0] * 7 + shape[1])
    x = (torch.randn(*shape, generator=g) * torch.exp2(torch.randint(-8, 8, shape, generator=g).float())).bfloat16().cuda()
    cr, sr, cc, sc = ops.quantize_fp8_both(x, dt)
    r1, s1 = ops.quantize_fp8(x, dt, 1)
    r0, s0 = ops.quantize_fp8(x, dt, 0)
    assert torch.equal(cr, r1) and torch.equal(sr, s1) and torch.equal(cc, r0) and torch.equal(sc, s0)
    oc, osc = R.quantize_fp8(x.cpu(), dt, dim=0)
    assert torch.equal(cc.cpu(), oc.view(torch.uint8).t()) and torch.equal(sc.cpu(), osc.reshape(-1))


def test_rows_that_are_only_16_byte_aligned(ops):
    """Pitch and start that rule out the 256-bit loads: the 128-bit path must give the same bytes."""
    x = CASES["x"]
    big = torch.zeros(x.shape[0], x.shape[1] + 24, dtype=torch.bfloat16)
    big[:, 8: 8 + x.shape[1]] = x
    view = big.cuda()[:, 8: 8 + x.shape[1]]
    assert view.data_ptr() % 32 == 16 and view.stride(0) % 16 == 8
    for dt in (E4, E5):
        codes, sf = ops.quantize_mxfp8(view, 1, dt, 0)
        rc, rs = R.quantize_mxfp8(x, -1, dt)
        assert torch.equal(codes.cpu(), rc) and torch.equal(sf.cpu(), rs.reshape(-1))
        c8, s8 = ops.quantize_fp8(view, dt, 1)
        r8, rs8 = R.quantize_fp8(x, dt, dim=-1)
        assert torch.equal(c8.cpu(), r8.view(torch.uint8)) and torch.equal(s8.cpu(), rs8.reshape(-1))
    packed, sf, ts = ops.quantize_nvfp4(view, 1, None, 0)
    rp, rs, rt = R.quantize_nvfp4(x, -1)
    assert torch.equal(packed.cpu(), rp) and torch.equal(sf.cpu(), rs.reshape(-1)) and ts.item() == rt.item()


def test_baseline_config_1_operands_bit_exact_at_full_size(ops):
    """MXFP8 linear of the GPT-2 MLP up-projection: X [8192, 768], W [3072, 768], seed 0, both along K - every code and
    every scale byte against the CPU oracle, row-wise, transposing and both-directions kernels."""
    x, w = R.inputs_mxfp8_linear()
    assert x.shape == (8192, 768) and w.shape == (3072, 768)
    for t in (x, w):
        tc = t.cuda()
        rc, rs = R.quantize_mxfp8(t, -1, E4)
        codes, sf = ops.quantize_mxfp8(tc, 1, E4, 0)
        assert torch.equal(codes.cpu(), rc) and torch.equal(sf.cpu().view(rs.shape), rs)
        codes, sf = ops.quantize_mxfp8(tc, 1, E4, 1)
        assert torch.equal(codes.cpu(), rc) and torch.equal(sf.cpu(), R.swizzle_sf(rs))
        r0, s0 = R.quantize_mxfp8(t, 0, E4)
        codes, sf = ops.quantize_mxfp8(tc, 0, E4, 0)
        assert torch.equal(codes.cpu(), r0) and torch.equal(sf.cpu().view(s0.shape), s0)
        cr, sr, cc, sc = ops.quantize_mxfp8_dual(tc, E4, 1)
        assert torch.equal(cr.cpu(), rc) and torch.equal(cc.cpu(), r0)
        assert torch.equal(sr.cpu(), R.swizzle_sf(rs)) and torch.equal(sc.cpu(), R.swizzle_sf(s0))


def test_baseline_config_2_operands_bit_exact_at_full_size(ops):
    """NVFP4 SwiGLU MLP: X [16384, 1024] with 0.1 % outliers x 50, gate/up W [6144, 1024], down W [1024, 3072] - packed
    codes, E4M3 block scales and the fp32 tensor scale against the CPU oracle; then an operand of the hidden activation's
    shape [16384, 3072] with per-row magnitudes, quantized along 3072 as the second GEMM needs it."""
    x, w_gu, w_d = R.inputs_nvfp4_mlp()
    assert x.shape == (16384, 1024) and w_gu.shape == (6144, 1024) and w_d.shape == (1024, 3072)
    for t in (x, w_gu, w_d):
        rp, rs, rt = R.quantize_nvfp4(t, -1)
        p, sf, ts = ops.quantize_nvfp4(t.cuda(), 1, None, 0)
        assert ts.item() == rt.item()
        assert torch.equal(p.cpu(), rp) and torch.equal(sf.cpu().view(rs.shape), rs)
        p, sf, ts = ops.quantize_nvfp4(t.cuda(), 1, None, 1)
        assert torch.equal(p.cpu(), rp) and torch.equal(sf.cpu(), R.swizzle_sf(rs))
    assert x.abs().max().item() > 100 and (rs.view(E4).float() > 0).all()          # the outliers reach the tensor scale
    g = torch.Generator().manual_seed(2)
    h = (torch.randn(16384, 3072, generator=g) * torch.rand(16384, 1, generator=g)).bfloat16()     # an activation-shaped operand
    rp, rs, rt = R.quantize_nvfp4(h, -1)
    p, sf, ts = ops.quantize_nvfp4(h.cuda(), 1, None, 0)
    assert ts.item() == rt.item() and torch.equal(p.cpu(), rp) and torch.equal(sf.cpu().view(rs.shape), rs)


def test_full_size_properties(ops):
    """Benchmark-size square operand (8192 x 8192): properties that need no CPU pass over the
    data — never clips, scale is tight, transposing kernel == row-wise kernel on the transpose."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(8192, 8192, generator=g, device="cuda", dtype=torch.bfloat16)
    codes, sf = ops.quantize_mxfp8(x, 1, E4, 0)
    e = sf.view(8192, 256).float() - 127
    amax = x.float().view(8192, 256, 32).abs().amax(-1)
    scaled = amax * torch.exp2(-e)
    assert (scaled <= 448).all() and (scaled > 224).all()
    deq = (codes.view(E4).float().view(8192, 256, 32) * torch.exp2(e).unsqueeze(-1)).view(8192, 8192)
    assert ((deq - x.float()).norm() / x.float().norm()).item() < 0.04
    ct, sft = ops.quantize_mxfp8(x.t().contiguous(), 0, E4, 0)
    assert torch.equal(ct, codes) and torch.equal(sft, sf)
    p1, s1, t1 = ops.quantize_nvfp4(x, 1, None, 1)
    p2, s2, t2 = ops.quantize_nvfp4(x.t().contiguous(), 0, None, 1)
    assert torch.equal(p1, p2) and torch.equal(s1, s2) and torch.equal(t1, t2)
    c1, sc1 = ops.quantize_fp8(x, E4, 1)
    c2, sc2 = ops.quantize_fp8(x.t().contiguous(), E4, 0)
    assert torch.equal(c1, c2) and torch.equal(sc1, sc2)


def _nan_pattern_equal(codes_u8, gold_u8, fp8_dtype):
    """Equal bytes outside the reference's NaN codes, NaN exactly where it has NaN (the sign / payload of a NaN code
    depends on which torch reduction produced the scale: 0x7F by rows, 0xFF by columns)."""
    got, ref = torch.from_numpy(codes_u8).view(fp8_dtype).float(), torch.from_numpy(np.ascontiguousarray(gold_u8)).view(fp8_dtype).float()
    nan = ref.isnan()
    return bool(torch.equal(got.isnan(), nan)) and np.array_equal(codes_u8[~nan.numpy()], np.ascontiguousarray(gold_u8)[~nan.numpy()])


def _scales_equal_with_nans(got, gold):
    return np.array_equal(np.isnan(got), np.isnan(gold)) and np.array_equal(got[~np.isnan(got)].view(np.uint32), gold[~np.isnan(gold)].view(np.uint32))


@pytest.mark.parametrize("dname,dt", [("e4m3", E4), ("e5m2", E5)])
def test_nan_inputs_reproduce_the_reference(ops, golden, dname, dt):
    """src/quant/fp8.py:26-31 on a tensor with two NaNs, run by the reference itself (tests/golden/make_golden.py): the
    NaN reaches the scale of its row / column / tensor and every code of that group; all other groups are untouched."""
    x = bf16_from_bits(golden["in_nan"]).cuda()
    codes, scales = ops.quantize_fp8(x, dt, 1)
    assert _nan_pattern_equal(codes.cpu().numpy(), golden[f"q_nan_{dname}_row_codes"], dt)
    assert _scales_equal_with_nans(scales.cpu().numpy(), golden[f"q_nan_{dname}_row_scale"])
    codes, scales = ops.quantize_fp8(x, dt, 0)
    assert _nan_pattern_equal(codes.cpu().numpy(), golden[f"q_nan_{dname}_col_codes"].T, dt)
    assert _scales_equal_with_nans(scales.cpu().numpy(), golden[f"q_nan_{dname}_col_scale"])
    for transpose in (False, True):
        codes, scale = ops.quantize_fp8_tensorwise(x, dt, transpose)
        gold = golden[f"q_nan_{dname}_tensor_codes"]
        assert _nan_pattern_equal(codes.cpu().numpy(), gold.T if transpose else gold, dt)
        assert np.isnan(scale.cpu().numpy()).all()
    cr, sr, cc, sc = ops.quantize_fp8_both(x, dt)
    assert _nan_pattern_equal(cr.cpu().numpy(), golden[f"q_nan_{dname}_row_codes"], dt)
    assert _nan_pattern_equal(cc.cpu().numpy(), golden[f"q_nan_{dname}_col_codes"].T, dt)
    assert _scales_equal_with_nans(sr.cpu().numpy(), golden[f"q_nan_{dname}_row_scale"])
    assert _scales_equal_with_nans(sc.cpu().numpy(), golden[f"q_nan_{dname}_col_scale"])


def test_block_scaled_quantizers_follow_the_same_nan_rule(ops):
    """MXFP8 / NVFP4 against the oracle on inputs with NaNs, every kernel form: the block (MXFP8) or the tensor
    (NVFP4) that holds a NaN gets the NaN scale and NaN codes, bit for bit as the oracle states it."""
    g = torch.Generator().manual_seed(17)
    x = torch.randn(128, 256, generator=g).bfloat16()
    x[3, 5] = float("nan")
    x[77, 200] = float("nan")
    xc = x.cuda()
    for dt in (E4, E5):
        for axis in (1, 0):
            codes, sf = ops.quantize_mxfp8(xc, axis, dt, 0)
            rc, rs = R.quantize_mxfp8(x, -1 if axis == 1 else 0, dt)
            assert torch.equal(codes.cpu(), rc) and torch.equal(sf.cpu().view(rs.shape), rs)
            assert int((rs == 255).sum()) == 2
        cr, sr, cc, sc = ops.quantize_mxfp8_dual(xc, dt, 0)
        r1, s1 = R.quantize_mxfp8(x, -1, dt)
        r0, s0 = R.quantize_mxfp8(x, 0, dt)
        assert torch.equal(cr.cpu(), r1) and torch.equal(cc.cpu(), r0)
        assert torch.equal(sr.cpu().view(s1.shape), s1) and torch.equal(sc.cpu().view(s0.shape), s0)
    for axis in (1, 0):
        p, sq, ts = ops.quantize_nvfp4(xc, axis, None, 0)
        rp, rsq, rt = R.quantize_nvfp4(x, -1 if axis == 1 else 0)
        assert ts.isnan().all() and rt.isnan()
        assert torch.equal(p.cpu(), rp) and torch.equal(sq.cpu().view(rsq.shape), rsq)
    assert ops.amax(xc).isnan().all()
    # a GEMM over such operands gives NaN exactly in the output rows / columns the NaN blocks feed
    ca, sfa = ops.quantize_mxfp8(xc, 1)
    w = torch.randn(128, 256, generator=g).bfloat16().cuda()
    cb, sfb = ops.quantize_mxfp8(w, 1)
    out = ops.gemm_mxfp8(ca, sfa, cb, sfb).float().cpu()
    bad = out.isnan().any(1)
    assert bad[3] and bad[77] and int(bad.sum()) == 2


def test_two_matrices_in_one_launch_equal_two_calls(ops):
    """b200q_quantize_mxfp8_pair against quantize_mxfp8 / quantize_mxfp8_rowmap on each matrix: different shapes, one of them
    through a row map, a ragged scale-factor tile, both formats."""
    g = torch.Generator().manual_seed(5)
    a = torch.randn(1000, 768, generator=g).bfloat16().cuda()
    b = (0.02 * torch.randn(384, 96, generator=g)).bfloat16().cuda()
    perm = torch.randperm(1000, generator=g).int().cuda()
    for fmt in (ops.E4M3, ops.E5M2):
        c0, s0, c1, s1 = ops.quantize_mxfp8_pair(a, b, perm, None, fmt)
        w0, t0 = ops.quantize_mxfp8_rowmap(a, perm, fmt)
        w1, t1 = ops.quantize_mxfp8(b, 1, fmt)
        assert torch.equal(c0, w0) and torch.equal(s0, t0) and torch.equal(c1, w1) and torch.equal(s1, t1)
        c0, s0, c1, s1 = ops.quantize_mxfp8_pair(b, a, None, None, fmt)
        w0, t0 = ops.quantize_mxfp8(b, 1, fmt)
        w1, t1 = ops.quantize_mxfp8(a, 1, fmt)
        assert torch.equal(c0, w0) and torch.equal(s0, t0) and torch.equal(c1, w1) and torch.equal(s1, t1)
