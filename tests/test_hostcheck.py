"""The numeric core the CUDA quantizers are built from (pretrain_b200/csrc/numeric.cuh),
compiled for the host and driven serially, against the oracle: exhaustive over bf16 for the
hoisted-reciprocal division, bit-exact codes and scales for all three formats."""

import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import restate as R
from conftest import ROOT, bf16_from_bits

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
SRC = os.path.join(ROOT, "tests", "hostcheck", "hostcheck.cpp")
OUT = os.path.join(ROOT, "tests", "hostcheck", "_build", "libhostcheck.so")


@pytest.fixture(scope="module")
def hc():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    deps = [SRC, os.path.join(ROOT, "pretrain_b200", "csrc", "numeric.cuh")]
    if not os.path.exists(OUT) or any(os.path.getmtime(d) > os.path.getmtime(OUT) for d in deps):
        subprocess.check_call(["g++", "-O2", "-ffp-contract=off", "-mfma", "-shared", "-fPIC",
                               "-I/usr/local/cuda/include", "-o", OUT, SRC])
    return ctypes.CDLL(OUT)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _cases():
    g = torch.Generator().manual_seed(3)
    x, w = R.inputs_mxfp8_linear(64, 768, 32)
    xo, _, _ = R.inputs_nvfp4_mlp(64, 1024, 16)
    wide = (torch.randn(32, 256, generator=g) * torch.exp2(torch.randint(-30, 30, (32, 256), generator=g).float()))
    tiny = torch.randn(8, 128, generator=g) * 1e-20
    zeros = torch.zeros(4, 64)
    signed = torch.randn(8, 64, generator=g)
    signed[:, ::3] = -0.0          # negative zeros keep their sign bit through every format
    signed[:, 1::7] *= -1e-30      # negative values that underflow to -0 after scaling
    return [x, w, xo, wide.to(torch.bfloat16), tiny.to(torch.bfloat16), zeros.to(torch.bfloat16),
            signed.to(torch.bfloat16), (-zeros).to(torch.bfloat16)]


@pytest.mark.parametrize("fmt,dt", [(0, E4), (1, E5)])
def test_division_by_hoisted_reciprocal_is_exact(hc, fmt, dt):
    out = (ctypes.c_int64 * 3)()
    hc.hc_div_exhaustive_fp8(fmt, 11, out)   # every 11th bf16 amax x every bf16 |x| <= amax
    assert out[2] > 4e7 and out[0] == 0 and out[1] == 0


def test_packed_pair_quotient_on_negated_operands_gives_the_same_bits(hc):
    out = (ctypes.c_int64 * 2)()
    hc.hc_negated_quotient(400, ctypes.c_uint64(11), out)
    assert out[1] == 400 * 65536 and out[0] == 0


def test_division_random_fp4(hc):
    out = (ctypes.c_int64 * 3)()
    hc.hc_div_random_fp4(ctypes.c_int64(20_000_000), ctypes.c_uint64(7), out)
    assert out[0] == 0 and out[1] == 0


def test_fp4_codes_at_every_rounding_boundary(hc):
    out = (ctypes.c_int64 * 2)()
    hc.hc_quot_fp4_boundaries(5, ctypes.c_int64(2_000_000), ctypes.c_uint64(11), out)
    assert out[1] > 4e7 and out[0] == 0


def test_nvfp4_block_scale_with_hoisted_reciprocals_is_exact(hc):
    out = (ctypes.c_int64 * 3)()
    hc.hc_nv_block_scale_exhaustive(13, out)   # every bf16 block amax x every 13th bf16 tensor amax >= it
    assert out[1] > 3e7 and out[0] == 0


def test_e4m3_decode_table(hc):
    tab = (ctypes.c_float * 256)()
    hc.hc_e4m3_decode_table(tab)
    ref = torch.arange(256, dtype=torch.uint8).view(E4).float().numpy()
    got = np.array(tab, dtype=np.float32)
    ok = (ref.view(np.uint32) == got.view(np.uint32)) | (np.isnan(ref) & np.isnan(got))
    assert ok.all()


@pytest.mark.parametrize("fmt,dt", [(0, E4), (1, E5)])
def test_fp8_rows(hc, golden, fmt, dt):
    cases = _cases() + [bf16_from_bits(golden["in_edge"]), bf16_from_bits(golden["in_a"])]
    for x in cases:
        rows, cols = x.shape
        codes = torch.empty(rows, cols, dtype=torch.uint8)
        scales = torch.empty(rows, dtype=torch.float32)
        hc.hc_quant_fp8_rows(_ptr(x), ctypes.c_int64(rows), ctypes.c_int64(cols), fmt, _ptr(codes), _ptr(scales))
        rc, rs = R.quantize_fp8(x, dt, dim=-1)
        assert torch.equal(codes, rc.view(torch.uint8))
        assert torch.equal(scales.view(torch.int32), rs.reshape(-1).view(torch.int32))


def test_fp8_rows_match_reference_golden(hc, golden):
    x = bf16_from_bits(golden["in_edge"])
    codes = torch.empty(x.shape, dtype=torch.uint8)
    scales = torch.empty(x.shape[0], dtype=torch.float32)
    hc.hc_quant_fp8_rows(_ptr(x), ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), 0, _ptr(codes), _ptr(scales))
    assert np.array_equal(codes.numpy(), golden["q_edge_e4m3_row_codes"])
    assert np.array_equal(scales.numpy().view(np.uint32), golden["q_edge_e4m3_row_scale"].view(np.uint32))


@pytest.mark.parametrize("fmt,dt", [(0, E4), (1, E5)])
def test_mxfp8_rows(hc, fmt, dt):
    for x in _cases():
        rows, cols = x.shape
        codes = torch.empty(rows, cols, dtype=torch.uint8)
        sf = torch.empty(rows, cols // 32, dtype=torch.uint8)
        hc.hc_quant_mxfp8_rows(_ptr(x), ctypes.c_int64(rows), ctypes.c_int64(cols), fmt, _ptr(codes), _ptr(sf))
        rc, rs = R.quantize_mxfp8(x, -1, dt)
        assert torch.equal(codes, rc) and torch.equal(sf, rs)


def test_nvfp4_rows(hc):
    for x in _cases():
        rows, cols = x.shape
        packed = torch.empty(rows, cols // 2, dtype=torch.uint8)
        sf = torch.empty(rows, cols // 16, dtype=torch.uint8)
        ts = ctypes.c_float()
        amax = float(x.abs().max().float())
        hc.hc_quant_nvfp4_rows(_ptr(x), ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_float(amax),
                               _ptr(packed), _ptr(sf), ctypes.byref(ts))
        rp, rs, rt = R.quantize_nvfp4(x)
        assert ts.value == rt.item()
        assert torch.equal(sf, rs) and torch.equal(packed, rp)


def test_sf_offset_matches_oracle_swizzle(hc):
    hc.hc_sf_offset.restype = ctypes.c_int64
    for outer, nblk in ((200, 24), (64, 3)):
        sf = torch.arange(outer * nblk, dtype=torch.int32).remainder(251).add(1).to(torch.uint8).view(outer, nblk)
        buf = R.swizzle_sf(sf)
        for r in range(0, outer, 7):
            for kb in range(nblk):
                off = hc.hc_sf_offset(ctypes.c_int64(r), ctypes.c_int64(kb), ctypes.c_int64(nblk), 1)
                assert buf[off] == sf[r, kb]
