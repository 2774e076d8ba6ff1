"""Pins the CPU oracle: restatements of reference code must reproduce the golden
vectors the reference itself produced (tests/golden/make_golden.py), bit for bit;
the block-scaled extensions are checked for their stated contract."""

import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import restate as R
from conftest import ROOT, bf16_from_bits

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.mark.parametrize("name", ["a", "b", "grad", "edge"])
@pytest.mark.parametrize("dname,dt", [("e4m3", E4), ("e5m2", E5)])
@pytest.mark.parametrize("dimname,dim", [("tensor", None), ("row", -1), ("col", 0)])
def test_quantize_fp8_matches_reference_vectors(golden, name, dname, dt, dimname, dim):
    x = bf16_from_bits(golden[f"in_{name}"])
    codes, scale = R.quantize_fp8(x, dt, dim)
    assert np.array_equal(codes.view(torch.uint8).numpy(), golden[f"q_{name}_{dname}_{dimname}_codes"])
    assert np.array_equal(scale.reshape(-1).numpy().view(np.uint32),
                          golden[f"q_{name}_{dname}_{dimname}_scale"].view(np.uint32))


def _same_up_to_nan_sign(codes_u8, gold_u8, fp8_dtype):
    """Equal bytes, except that where the reference's code is a NaN ours must be a NaN too (its sign and payload
    depend on which torch kernel reduced the maximum: 0x7F from the row reduction, 0xFF from the column one)."""
    got = torch.from_numpy(np.ascontiguousarray(codes_u8)).view(fp8_dtype).float()
    ref = torch.from_numpy(np.ascontiguousarray(gold_u8)).view(fp8_dtype).float()
    nan = ref.isnan()
    return bool(torch.equal(got.isnan(), nan)) and np.array_equal(codes_u8[~nan.numpy()], gold_u8[~nan.numpy()])


@pytest.mark.parametrize("dname,dt", [("e4m3", E4), ("e5m2", E5)])
@pytest.mark.parametrize("dimname,dim", [("tensor", None), ("row", -1), ("col", 0)])
def test_quantize_fp8_nan_inputs_match_reference_vectors(golden, dname, dt, dimname, dim):
    """The reference's amax carries a NaN into the scale of its row / column / tensor and from there into every code of
    that group (src/quant/fp8.py:26-31); groups without a NaN are untouched."""
    x = bf16_from_bits(golden["in_nan"])
    codes, scale = R.quantize_fp8(x, dt, dim)
    gold_scale = golden[f"q_nan_{dname}_{dimname}_scale"]
    assert _same_up_to_nan_sign(codes.view(torch.uint8).numpy(), golden[f"q_nan_{dname}_{dimname}_codes"], dt)
    got = scale.reshape(-1).numpy()
    assert np.array_equal(np.isnan(got), np.isnan(gold_scale))
    assert np.array_equal(got[~np.isnan(got)].view(np.uint32), gold_scale[~np.isnan(gold_scale)].view(np.uint32))
    n_groups = {"tensor": 1, "row": 2, "col": 2}[dimname]
    assert int(np.isnan(gold_scale).sum()) == n_groups


def test_block_scaled_nan_rule():
    """MXFP8 / NVFP4 follow the same arithmetic at their own granularity: a block with a NaN gets the NaN scale byte
    (E8M0 0xFF) and NaN codes; an NVFP4 tensor with a NaN gets a NaN tensor scale, so every block scale byte is the
    E4M3 NaN (0x7F) and the whole tensor dequantizes to NaN."""
    g = torch.Generator().manual_seed(8)
    x = torch.randn(8, 128, generator=g).bfloat16()
    clean_codes, clean_sf = R.quantize_mxfp8(x)
    x[2, 70] = float("nan")
    for dt in (E4, E5):
        cc, cs = R.quantize_mxfp8(x.nan_to_num(0.0), -1, dt)
        codes, sf = R.quantize_mxfp8(x, -1, dt)
        hit = torch.zeros(8, 4, dtype=torch.bool); hit[2, 2] = True
        assert torch.equal(sf[hit], torch.tensor([255], dtype=torch.uint8)) and torch.equal(sf[~hit], cs[~hit])
        assert (codes[2, 64:96] == 0x7F).all()
        keep = torch.ones(8, 128, dtype=torch.bool); keep[2, 64:96] = False
        assert torch.equal(codes[keep], cc[keep])
        assert R.dequantize_mxfp8(codes, sf, dt)[2, 64:96].isnan().all()
    p, sq, s_t = R.quantize_nvfp4(x)
    assert s_t.isnan() and (sq == 0x7F).all() and (p == 0x77).all()
    assert R.dequantize_nvfp4(p, sq, s_t).isnan().all()


def test_fake_quant_and_gemm_forms_match_reference_vectors(golden):
    a, b, g = (bf16_from_bits(golden[f"in_{n}"]) for n in ("a", "b", "grad"))
    fq = R.fake_quantize_fp8(a, E4, dim=-1)
    assert np.array_equal(fq.view(torch.int16).numpy(), golden["fq_a_e4m3_row"])
    # the reference multiplies the fake-quantised bf16 operands with a bf16 matmul
    out = R.fake_quantize_fp8(a, E4, dim=-1) @ R.fake_quantize_fp8(b, E4, dim=0)
    assert np.array_equal(out.view(torch.int16).numpy(), golden["gemm_rowwise_e4m3"])
    # fp32-accumulated form used for the CUDA parity checks stays within bf16 rounding of it
    ref32 = R.fp8_gemm_ref(a, b, torch.bfloat16, E4, E4, rowwise=True).float()
    gold = bf16_from_bits(golden["gemm_rowwise_e4m3"]).float()
    assert (ref32 - gold).abs().max() / gold.abs().max() < 1e-2
    out2 = R.fake_quantize_fp8(g, E5, dim=-1) @ R.fake_quantize_fp8(b.t(), E4, dim=0)
    assert np.array_equal(out2.view(torch.int16).numpy(), golden["gemm_rowwise_e5m2_e4m3"])


@pytest.mark.parametrize("name", ["a", "b", "grad", "edge"])
@pytest.mark.parametrize("qmax", [127, 63, 31, 15, 7])
@pytest.mark.parametrize("dimname,dim", [("tensor", None), ("row", -1), ("col", 0)])
def test_quantize_int8_matches_reference_vectors(golden, golden_int8, name, qmax, dimname, dim):
    x = bf16_from_bits(golden[f"in_{name}"])
    codes, scale = R.quantize_int8(x, qmax, dim)
    assert np.array_equal(codes.numpy(), golden_int8[f"q_{name}_{qmax}_{dimname}_codes"])
    assert np.array_equal(scale.reshape(-1).numpy().view(np.uint32),
                          golden_int8[f"q_{name}_{qmax}_{dimname}_scale"].view(np.uint32))


def test_int8_fake_quant_and_gemm_forms_match_reference_vectors(golden, golden_int8):
    a, b = (bf16_from_bits(golden[f"in_{n}"]) for n in ("a", "b"))
    assert np.array_equal(R.fake_quantize_int8(a, 127, dim=-1).view(torch.int16).numpy(), golden_int8["fq_a_127_row"])
    out = R.int8_gemm_fake_ref(a, b, torch.bfloat16, 127, 127, rowwise=True)
    assert np.array_equal(out.view(torch.int16).numpy(), golden_int8["gemm_rowwise_127"])
    out = R.int8_gemm_fake_ref(a, b, torch.bfloat16, 127, 7, rowwise=False)
    assert np.array_equal(out.view(torch.int16).numpy(), golden_int8["gemm_tensor_127_7"])
    # the real kernel's form (exact integer accumulation, scales applied in fp32) stays within bf16
    # rounding of the fallback form the reference runs on a CPU
    exact = R.int8_gemm_ref(a, b, torch.bfloat16, 127, 127, rowwise=True).float()
    gold = bf16_from_bits(golden_int8["gemm_rowwise_127"]).float()
    assert (exact - gold).abs().max() / gold.abs().max() < 1e-2


def test_digests_at_benchmark_size():
    with open(os.path.join(ROOT, "tests", "golden", "ref_digests.json")) as f:
        dig = json.load(f)
    x, w, dy = R.inputs_fp8_triple()

    def sha(t):
        return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()

    for name, t, dt, dim in (("fprop_x_row_e4m3", x, E4, -1), ("dgrad_w_col_e4m3", w, E4, 0),
                             ("wgrad_dyT_row_e5m2", dy.t(), E5, -1)):
        codes, scale = R.quantize_fp8(t, dt, dim)
        assert sha(codes) == dig[name]["codes"] and sha(scale) == dig[name]["scale"]


def test_moe_permute_matches_reference_vectors(golden):
    top_i = torch.from_numpy(golden["moe_top_i"])
    order, tok, counts, offs = R.moe_permute(top_i, 6)
    assert np.array_equal(order.numpy(), golden["moe_order"])
    assert np.array_equal(tok.numpy(), golden["moe_token_ids_sorted"])
    assert np.array_equal(counts.numpy(), golden["moe_counts"])
    assert np.array_equal(offs.numpy(), golden["moe_offs"])
    assert counts[3] == 0  # the empty expert of the fixture
    x = bf16_from_bits(golden["moe_x"])
    xs = x[tok]
    assert np.array_equal(xs.view(torch.int16).numpy(), golden["moe_x_sorted"])
    w_in, w_down = bf16_from_bits(golden["moe_w_in"]), bf16_from_bits(golden["moe_w_down"])
    eo = R.grouped_mlp_ref(xs, w_in, w_down, offs)
    gold = bf16_from_bits(golden["moe_expert_out"]).float()
    assert (eo.float() - gold).abs().max() <= 8e-2 * max(1.0, gold.abs().max())  # reference's bf16 COMPOUND atol
    assert (eo.float() - gold).norm() / gold.norm() < 1e-2
    w_sorted = bf16_from_bits(golden["moe_top_w"]).reshape(-1)[order]
    y = R.moe_unpermute_ref(bf16_from_bits(golden["moe_expert_out"]), w_sorted, tok, x.shape[0])
    assert np.array_equal(y.view(torch.int16).numpy(), golden["moe_y"])
    y32 = R.moe_unpermute_fp32(bf16_from_bits(golden["moe_expert_out"]), w_sorted, tok, x.shape[0])
    assert (y32.float() - y.float()).abs().max() <= 2e-2 * y.float().abs().max()


# ---- block-scaled extensions: contract checks (no reference implementation exists) ----

def _all_positive_bf16():
    bits = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16)
    return bits.view(torch.bfloat16).float()


@pytest.mark.parametrize("dt", [E4, E5])
def test_mx_exponent_integer_rule_equals_division_form(dt):
    amax = _all_positive_bf16()
    assert torch.equal(R.mx_scale_exponent(amax, dt), R.mx_scale_exponent_by_division(amax, dt))
    g = torch.Generator().manual_seed(0)
    rnd = torch.randn(1 << 20, generator=g).abs() * torch.exp2(torch.randint(-60, 60, (1 << 20,), generator=g).float())
    assert torch.equal(R.mx_scale_exponent(rnd, dt), R.mx_scale_exponent_by_division(rnd, dt))
    assert R.mx_scale_exponent(torch.zeros(1), dt).item() == -39


@pytest.mark.parametrize("dt", [E4, E5])
def test_mxfp8_never_clips_and_scale_is_tight(dt):
    x, w = R.inputs_mxfp8_linear(256, 768, 128)
    for t in (x, w, x * 1e4, w * 1e-5):
        codes, sf = R.quantize_mxfp8(t, -1, dt)
        e = sf.to(torch.int32) - 127
        amax = t.float().view(t.shape[0], -1, 32).abs().amax(-1)
        scaled = amax * torch.exp2(-e.float())
        assert (scaled <= R.FP8_MAX[dt]).all()
        tight = (scaled > R.FP8_MAX[dt] / 2) | (e == -39)
        assert tight.all()
        deq = R.dequantize_mxfp8(codes, sf, dt)
        assert (deq - t.float()).norm() / t.float().norm() < (0.04 if dt == E4 else 0.08)
        if dt == E4:
            assert torch.equal(deq.to(torch.bfloat16).float(), deq)  # exact in bf16


def test_mxfp8_axis0_is_transpose_of_rowwise():
    x, _ = R.inputs_mxfp8_linear(128, 96, 8)
    c0, s0 = R.quantize_mxfp8(x, 0)
    c1, s1 = R.quantize_mxfp8(x.t().contiguous(), -1)
    assert torch.equal(c0, c1) and torch.equal(s0, s1) and c0.shape == (96, 128)


def test_e2m1_rounding_table():
    v = np.array([0, .25, .26, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 2.51, 3, 3.5, 4, 5, 5.01, 6, -0.0, -0.25, -5], np.float32)
    want = np.array([0, 0, 1, 1, 2, 2, 2, 3, 4, 4, 4, 5, 5, 6, 6, 6, 7, 7, 8, 8, 8 | 6], np.uint8)
    assert np.array_equal(R.e2m1_rne(v), want)
    assert np.array_equal(R.e2m1_decode(np.arange(16, dtype=np.uint8))[:8], R._E2M1_VALUES)


def test_nvfp4_contract_and_noise():
    x, w_gu, _ = R.inputs_nvfp4_mlp(512, 1024, 64)
    for t in (x, w_gu):
        packed, sf, s_t = R.quantize_nvfp4(t)
        assert packed.shape == (t.shape[0], t.shape[1] // 2) and sf.shape == (t.shape[0], t.shape[1] // 16)
        deq = R.dequantize_nvfp4(packed, sf, s_t)
        rel = (deq - t.float()).norm() / t.float().norm()
        assert rel < 0.12
        assert (sf.view(E4).float() <= 448).all()
    z = torch.zeros(4, 32, dtype=torch.bfloat16)
    packed, sf, s_t = R.quantize_nvfp4(z)
    assert packed.eq(0).all() and torch.isfinite(R.dequantize_nvfp4(packed, sf, s_t)).all()


def test_sf_swizzle_roundtrip_and_layout():
    g = torch.Generator().manual_seed(0)
    for outer, nblk in ((128, 4), (200, 24), (3072, 24), (64, 3), (1, 1)):
        sf = torch.randint(1, 255, (outer, nblk), dtype=torch.uint8, generator=g)
        buf = R.swizzle_sf(sf)
        assert buf.numel() == R.sf_swizzled_size(outer, nblk)
        assert torch.equal(R.unswizzle_sf(buf, outer, nblk), sf)
        assert int((buf != 0).sum()) == outer * nblk
    sf = torch.zeros(256, 8, dtype=torch.uint8)
    sf[129, 5] = 7            # row tile 1, k tile 1; r%32 = 1, (r%128)//32 = 0, kb%4 = 1
    assert R.swizzle_sf(sf)[(1 * 2 + 1) * 512 + 1 * 16 + 0 * 4 + 1] == 7
