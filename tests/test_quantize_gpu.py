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


def test_a_nan_stays_where_it_is(ops):
    """Non-finite inputs are outside the reference's tests; what the kernels do with them is pinned here: a NaN
    becomes a NaN code in place and takes part in no maximum, so every other code and every scale are those of the
    same tensor with the NaN replaced by zero."""
    g = torch.Generator().manual_seed(17)
    x = torch.randn(64, 256, generator=g).bfloat16()
    clean = x.clone()
    x[3, 5] = float("nan")
    clean[3, 5] = 0.0
    is_nan = lambda codes, dt: codes.view(dt).float().isnan()
    for dt in (E4, E5):
        for fn in (lambda t: ops.quantize_fp8(t, dt, 1), lambda t: ops.quantize_mxfp8(t, 1, dt, 0)):
            codes, scales = fn(x.cuda())
            want, want_scales = fn(clean.cuda())
            assert is_nan(codes[3, 5].cpu(), dt)
            codes = codes.clone()
            codes[3, 5] = want[3, 5]
            assert torch.equal(codes, want) and torch.equal(scales.view(torch.uint8), want_scales.view(torch.uint8))
        cr, sr, cc, sc = ops.quantize_mxfp8_dual(x.cuda(), dt, 0)
        wr, wsr, wc, wsc = ops.quantize_mxfp8_dual(clean.cuda(), dt, 0)
        assert is_nan(cr[3, 5].cpu(), dt) and is_nan(cc[5, 3].cpu(), dt)
        cr, cc = cr.clone(), cc.clone()
        cr[3, 5], cc[5, 3] = wr[3, 5], wc[5, 3]
        assert torch.equal(cr, wr) and torch.equal(cc, wc) and torch.equal(sr, wsr) and torch.equal(sc, wsc)
