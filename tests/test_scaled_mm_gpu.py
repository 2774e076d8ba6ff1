"""A second implementation reads this library's bytes: torch's scaled matmul (cuBLASLt), the reference's own GPU
call for FP8 (`torch._scaled_mm`, src/quant/fp8.py:59-65) and its block-scaled modes for MXFP8 / NVFP4, is fed the
codes and the (swizzled) scale factors the quantizers here produce and must agree with this library's GEMM within
the north star's 1e-2 (max relative and Frobenius, bf16 output).  That pins, against code this repository did not
write, (a) the E8M0 / E4M3 scale bytes and their 128x4 tiling, (b) the packing of E2M1 pairs, (c) which operand
each scale belongs to.  Where torch refuses a mode on this build the test is skipped with torch's message, which is
also appended to scaled_mm_refusals.txt in the directory B200Q_TEST_ARTIFACTS names (when it is set).  Test
infrastructure only: nothing in the package calls torch's scaled matmul."""

import os

import pytest
import torch

from oracle import restate as R
import gpu_ref as G

pytestmark = pytest.mark.gpu
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
TOL = 1e-2


@pytest.fixture(scope="module")
def ops():
    from pretrain_b200 import build, ops
    build.build()
    return ops


def _refused(what, exc):
    msg = f"{what}: {type(exc).__name__}: {str(exc).splitlines()[0][:300]}"
    out_dir = os.environ.get("B200Q_TEST_ARTIFACTS")
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "scaled_mm_refusals.txt"), "a") as f:
            f.write(msg + "\n")
    pytest.skip(msg)


def _close(out, ref, tol=TOL):
    mx, fro = G.rel_errors(out, ref)
    assert mx <= tol and fro <= tol, (mx, fro)
    return mx, fro


def _inputs(name):
    if name == "cfg1":
        return R.inputs_mxfp8_linear(8192, 768, 3072)
    if name == "cfg3":
        return R.inputs_fp8_triple()[:2]
    if name == "cfg2_gate_up":                                     # activations with the x50 outliers, gate/up weight
        return R.inputs_nvfp4_mlp()[:2]
    return R.inputs_square(8192)                                   # cfg5 at 8192: A, B ~ N(0, 1)


@pytest.mark.parametrize("cfg", ["cfg1", "cfg3", "square8192"])
@pytest.mark.parametrize("a_dt", [E4, E5])
def test_fp8_rowwise_codes_through_torch_scaled_mm(ops, cfg, a_dt):
    """Exactly the reference's call: per-row scales of a, per-column scales of b, b column-major."""
    a, b = (t.cuda() for t in _inputs(cfg))
    ca, sa = ops.quantize_fp8(a, a_dt, 1)
    cb, sb = ops.quantize_fp8(b, E4, 1)
    ours = ops.gemm_fp8(ca, a_dt, cb, E4, sa, sb)
    try:
        theirs = torch._scaled_mm(ca.view(a_dt), cb.view(E4).t(), scale_a=sa.view(-1, 1), scale_b=sb.view(1, -1), out_dtype=torch.bfloat16)
    except Exception as exc:                                           # noqa: BLE001 - whatever torch raises is the finding
        _refused(f"fp8 rowwise {cfg} a={a_dt}", exc)
    _close(ours, theirs)


def _mx_scaled_mm(ca, sfa, cb, sfb, a_dt, b_dt):
    import torch.nn.functional as F
    e8 = torch.float8_e8m0fnu
    return F.scaled_mm(ca.view(a_dt), cb.view(b_dt).t(), sfa.view(e8), F.ScalingType.BlockWise1x32, sfb.view(e8),
                       F.ScalingType.BlockWise1x32, swizzle_a=F.SwizzleType.SWIZZLE_32_4_4, swizzle_b=F.SwizzleType.SWIZZLE_32_4_4,
                       output_dtype=torch.bfloat16)


@pytest.mark.parametrize("cfg", ["cfg1", "cfg3", "square8192"])
def test_mxfp8_codes_and_swizzled_scales_through_torch_scaled_mm(ops, cfg):
    a, b = (t.cuda() for t in _inputs(cfg))
    ca, sfa = ops.quantize_mxfp8(a, 1)
    cb, sfb = ops.quantize_mxfp8(b, 1)
    ours = ops.gemm_mxfp8(ca, sfa, cb, sfb)
    try:
        theirs = _mx_scaled_mm(ca, sfa, cb, sfb, E4, E4)
    except Exception as exc:                                           # noqa: BLE001
        _refused(f"mxfp8 {cfg}", exc)
    _close(ours, theirs)


def test_mxfp8_scale_rule_is_what_a_block_scaled_gemm_needs(ops):
    """Blocks of very different magnitude in one row (2^-20 .. 2^20): if the E8M0 byte of any block were off by one, or
    landed in the wrong slot of the tiled layout, torch's GEMM over the same bytes would be off by a factor of two in
    that block's contribution.  Also the e5m2 gradient format against e4m3 weights."""
    g = torch.Generator().manual_seed(5)
    m, n, k = 384, 256, 1024
    mag = torch.exp2(torch.randint(-20, 21, (m, k // 32), generator=g).float()).repeat_interleave(32, dim=1)
    a = (torch.randn(m, k, generator=g) * mag).bfloat16().cuda()
    b = torch.randn(n, k, generator=g).bfloat16().cuda()
    for a_dt in (E4, E5):
        ca, sfa = ops.quantize_mxfp8(a, 1, a_dt)
        cb, sfb = ops.quantize_mxfp8(b, 1, E4)
        ours = ops.gemm_mxfp8(ca, sfa, cb, sfb, a_dt, E4)
        try:
            theirs = _mx_scaled_mm(ca, sfa, cb, sfb, a_dt, E4)
        except Exception as exc:                                       # noqa: BLE001
            _refused(f"mxfp8 wide-range a={a_dt}", exc)
        _close(ours, theirs)
        # and both against dequantize-then-matmul, per row (rows differ by 2^40 in magnitude)
        ref = G.matmul_fp32(G.deq_mxfp8(ca, sfa, a_dt), G.deq_mxfp8(cb, sfb, E4))
        row_err = ((theirs.float() - ref).abs().amax(1) / ref.abs().amax(1)).max().item()
        assert row_err <= TOL, row_err


def _nv_scaled_mm(pa, sfa, ta, pb, sfb, tb):
    import torch.nn.functional as F
    f4 = torch.float4_e2m1fn_x2
    a4, b4 = pa.view(f4), pb.view(f4).t()
    S, Z = F.ScalingType, F.SwizzleType
    try:                                                               # two-level form: block scales + tensor scales
        return F.scaled_mm(a4, b4, [sfa.view(E4), ta.view(())], [S.BlockWise1x16, S.TensorWise], [sfb.view(E4), tb.view(())],
                           [S.BlockWise1x16, S.TensorWise], swizzle_a=[Z.SWIZZLE_32_4_4, Z.NO_SWIZZLE],
                           swizzle_b=[Z.SWIZZLE_32_4_4, Z.NO_SWIZZLE], output_dtype=torch.bfloat16), "two-level"
    except Exception:                                                  # noqa: BLE001 - fall back to block scales only
        out = F.scaled_mm(a4, b4, sfa.view(E4), S.BlockWise1x16, sfb.view(E4), S.BlockWise1x16, swizzle_a=Z.SWIZZLE_32_4_4,
                          swizzle_b=Z.SWIZZLE_32_4_4, output_dtype=torch.float32)
        return (out * (ta * tb)).bfloat16(), "block scales in torch, tensor scales applied after"


@pytest.mark.parametrize("cfg", ["cfg1", "cfg2_gate_up", "square8192"])
def test_nvfp4_codes_and_scales_through_torch_scaled_mm(ops, cfg):
    a, b = (t.cuda() for t in _inputs(cfg))
    pa, sfa, ta = ops.quantize_nvfp4(a, 1)
    pb, sfb, tb = ops.quantize_nvfp4(b, 1)
    ours = ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb)
    try:
        theirs, how = _nv_scaled_mm(pa, sfa, ta, pb, sfb, tb)
    except Exception as exc:                                           # noqa: BLE001
        _refused(f"nvfp4 {cfg}", exc)
    _close(ours, theirs)
