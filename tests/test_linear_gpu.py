"""QuantLinear / QuantizedLinearFn / _gemm on the GPU, in the style of the reference's
tests/fast/quant/test_linear.py: forward and the two backward GEMMs against the oracle's
fake-quantize-then-matmul, dtype plumbing under autocast, and tracing with torch.compile."""

import pytest
import torch
import torch.nn as nn

from oracle import restate as R

pytestmark = pytest.mark.gpu
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.fixture(scope="module", autouse=True)
def _built():
    from pretrain_b200 import build
    build.build()


def _cfg(recipe, granularity=None, **dtype):
    from pretrain_b200.quant.config import TrainingConfig
    q = {"enabled": True, "dtype_recipe": recipe, "dtype": dict(dtype)}
    if granularity:
        q["scaling"] = {"granularity": granularity}
    return TrainingConfig(quant=q).quant[0]


def _rel(out, ref):
    return ((out.float() - ref.float()).norm() / ref.float().norm()).item()


def _oracle_gemm(kind, a, b, a_dt=E4, b_dt=E4):
    """a (M,K) @ b (K,N) on the CPU oracle, operands scaled along K."""
    if kind == "fp8_rowwise":
        return R.fp8_gemm_ref(a, b, torch.bfloat16, a_dt, b_dt, rowwise=True)
    if kind == "fp8_tensorwise":
        return R.fp8_gemm_ref(a, b, torch.bfloat16, a_dt, b_dt, rowwise=False)
    if kind == "mxfp8":
        return R.mxfp8_gemm_ref(a, b, torch.bfloat16, a_dt, b_dt)
    return R.nvfp4_gemm_ref(a, b)


CASES = [("fp8", "rowwise", "fp8_rowwise"), ("fp8", None, "fp8_tensorwise"), ("mxfp8", None, "mxfp8"), ("nvfp4", None, "nvfp4")]


@pytest.mark.parametrize("recipe,gran,kind", CASES)
def test_gemm_seam_matches_oracle_in_all_three_layouts(recipe, gran, kind):
    """fprop / dgrad / wgrad call shapes of src/quant/linear.py:74,98,102 (views included)."""
    from pretrain_b200.quant.linear import _gemm
    cfg = _cfg(recipe, gran)
    g = torch.Generator().manual_seed(0)
    M, K, N = 256, 128, 192
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (0.05 * torch.randn(N, K, generator=g)).bfloat16()
    dy = (1e-2 * torch.randn(M, N, generator=g)).bfloat16()
    xd, wd, dyd = x.cuda(), w.cuda(), dy.cuda()
    rw = gran == "rowwise"
    e5 = E4 if recipe == "nvfp4" else E5
    y = _gemm(xd, wd.t(), cfg.dtype["act"], cfg.dtype["weight"], torch.bfloat16, rw)
    assert y.shape == (M, N) and _rel(y.cpu(), _oracle_gemm(kind, x, w.t())) < 0.01
    dx = _gemm(dyd, wd, cfg.dtype["input_grad"], cfg.dtype["weight"], torch.bfloat16, rw)
    assert dx.shape == (M, K) and _rel(dx.cpu(), _oracle_gemm(kind, dy, w, e5, E4)) < 0.01
    dw = _gemm(dyd.t(), xd, cfg.dtype["weight_grad"], cfg.dtype["act"], torch.bfloat16, rw)
    assert dw.shape == (N, K) and _rel(dw.cpu(), _oracle_gemm(kind, dy.t(), x, e5, E4)) < 0.01


def test_mixed_formats_fall_to_fake_quant_matmul():
    from pretrain_b200.quant.linear import _gemm
    g = torch.Generator().manual_seed(1)
    a = torch.randn(64, 128, generator=g).bfloat16()
    b = torch.randn(128, 96, generator=g).bfloat16()
    out = _gemm(a.cuda(), b.cuda(), "fp8_e4m3", "bf16", torch.bfloat16, rowwise=True)
    ref = (R.fake_quantize_fp8(a, E4, dim=-1).float() @ b.float()).bfloat16()
    assert _rel(out.cpu(), ref) < 0.01
    out = _gemm(a.cuda(), b.cuda(), "bf16", "mxfp8", torch.bfloat16)
    cb, sb = R.quantize_mxfp8(b, 0)
    ref = (a.float() @ R.dequantize_mxfp8(cb, sb).t()).bfloat16()
    assert _rel(out.cpu(), ref) < 0.01
    out = _gemm(a.cuda(), b.cuda(), "int8", "fp8_e4m3", torch.bfloat16, rowwise=True)      # mixed families
    ref = (R.fake_quantize_int8(a, 127, dim=-1).float() @ R.fake_quantize_fp8(b, E4, dim=0).float()).bfloat16()
    assert _rel(out.cpu(), ref) < 0.01


@pytest.mark.parametrize("a_fmt,b_fmt", [("int8", "int8"), ("int8", "int4"), ("int6", "int7")])
@pytest.mark.parametrize("rowwise", [True, False])
def test_int8_series_gemm_seam_is_bit_exact(a_fmt, b_fmt, rowwise):
    """Integer accumulation is exact, so the tensor-core GEMM must reproduce the reference's
    `torch._int_mm` formula (src/quant/int8.py:49-53) bit for bit, in all three layouts."""
    from pretrain_b200.quant.linear import _gemm
    g = torch.Generator().manual_seed(3)
    x = torch.randn(256, 192, generator=g).bfloat16()
    w = (0.05 * torch.randn(128, 192, generator=g)).bfloat16()
    gr = (1e-2 * torch.randn(256, 128, generator=g)).bfloat16()
    qa, qb = R.INT_QMAX[a_fmt], R.INT_QMAX[b_fmt]
    for a, b in ((x, w.t()), (gr, w), (gr.t(), x)):                       # fprop, dgrad, wgrad
        out = _gemm(a.cuda(), b.cuda(), a_fmt, b_fmt, torch.bfloat16, rowwise=rowwise)
        ref = R.int8_gemm_ref(a, b, torch.bfloat16, qa, qb, rowwise=rowwise)
        assert torch.equal(out.cpu(), ref)


def test_int8_recipe_module_trains():
    from pretrain_b200.quant.linear import QuantLinear
    torch.manual_seed(0)
    lin = nn.Linear(128, 96, bias=True)
    q = QuantLinear.from_linear(lin, _cfg("int8", "rowwise")).cuda()
    x = torch.randn(4, 16, 128)
    xd = x.cuda().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = q(xd)
    ref = R.int8_gemm_ref(x.reshape(-1, 128).bfloat16(), lin.weight.detach().bfloat16().t(), torch.bfloat16, 127, 127, True)
    assert torch.equal(y.reshape(-1, 96).cpu(), (ref + lin.bias.detach().bfloat16()))
    y.float().square().mean().backward()
    assert torch.isfinite(xd.grad).all() and torch.isfinite(q.weight.grad).all()


@pytest.mark.parametrize("recipe,gran,kind", CASES)
def test_module_forward_backward(recipe, gran, kind):
    from pretrain_b200.quant.linear import QuantLinear
    torch.manual_seed(0)
    lin = nn.Linear(128, 96, bias=True)
    q = QuantLinear.from_linear(lin, _cfg(recipe, gran)).cuda()
    assert torch.equal(q.weight.cpu(), lin.weight) and torch.equal(q.bias.cpu(), lin.bias)
    x = torch.randn(4, 16, 128)                       # batch dims are flattened and restored
    xd = x.cuda().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = q(xd)
    assert y.shape == (4, 16, 96) and y.dtype == torch.bfloat16
    ref = _oracle_gemm(kind, x.reshape(-1, 128).bfloat16(), lin.weight.detach().bfloat16().t()).float() + lin.bias.detach()
    assert _rel(y.float().cpu().reshape(-1, 96), ref) < 0.05     # module tolerance of the reference's tests
    y.float().square().mean().backward()
    assert xd.grad.dtype == torch.float32 and xd.grad.shape == x.shape
    assert q.weight.grad.dtype == torch.float32 and q.weight.grad.shape == (96, 128)   # master-weight dtype
    assert q.bias.grad is not None and torch.isfinite(q.weight.grad).all()


def test_mxfp8_training_path_quantizes_once_and_equals_the_per_gemm_path():
    """All-MXFP8 layers quantize x, w and g once each (both directions in one kernel) and save codes
    for backward; y, dx and dw must equal what the three separate `_gemm` calls give, bit for bit."""
    from pretrain_b200.quant.linear import QuantLinear, QuantizedLinearFn, _gemm
    torch.manual_seed(1)
    cfg = _cfg("mxfp8")
    m, k, n = 256, 160, 96
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = nn.Parameter((0.05 * torch.randn(n, k, device="cuda")).bfloat16())
    g = (1e-2 * torch.randn(m, n, device="cuda")).bfloat16()
    y = QuantizedLinearFn.apply(x, w, None, cfg)
    y.backward(g)
    d = cfg.dtype
    with torch.no_grad():
        y_ref = _gemm(x, w.t(), d["act"], d["weight"], torch.bfloat16)
        dx_ref = _gemm(g, w, d["input_grad"], d["weight"], torch.bfloat16)
        dw_ref = _gemm(g.t(), x, d["weight_grad"], d["act"], torch.bfloat16)
    assert torch.equal(y, y_ref) and torch.equal(x.grad, dx_ref) and torch.equal(w.grad, dw_ref)
    # the weight's two MXFP8 copies are kept until the parameter is written again
    cached = w._b200q_mx
    QuantizedLinearFn.apply(x, w, None, cfg).sum().backward()
    assert w._b200q_mx is cached
    with torch.no_grad():
        w.add_(1.0)                                    # what an optimizer step does
    QuantizedLinearFn.apply(x, w, None, cfg)
    assert w._b200q_mx is not cached
    # no backward to come: the plain single-direction path runs and leaves no codes behind
    q = QuantLinear(k, n, False, cfg).cuda().bfloat16()
    with torch.no_grad():
        y2 = q(x.detach())
    assert not hasattr(q.weight, "_b200q_mx") and y2.shape == (m, n)
    q(x.detach()).sum().backward()
    assert hasattr(q.weight, "_b200q_mx") and q.weight.grad is not None


def test_fp8_rowwise_training_path_equals_the_per_gemm_path():
    """Row-wise FP8 layers quantize x, w and g per row and per column in two reads each and save codes;
    y, dx and dw must equal the three separate `_gemm` calls bit for bit."""
    from pretrain_b200.quant.linear import QuantizedLinearFn, _gemm
    torch.manual_seed(2)
    cfg = _cfg("fp8", "rowwise")
    m, k, n = 256, 160, 96
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = nn.Parameter((0.05 * torch.randn(n, k, device="cuda")).bfloat16())
    g = (1e-2 * torch.randn(m, n, device="cuda")).bfloat16()
    y = QuantizedLinearFn.apply(x, w, None, cfg)
    y.backward(g)
    assert hasattr(w, "_b200q_fp8")
    d = cfg.dtype
    with torch.no_grad():
        y_ref = _gemm(x, w.t(), d["act"], d["weight"], torch.bfloat16, rowwise=True)
        dx_ref = _gemm(g, w, d["input_grad"], d["weight"], torch.bfloat16, rowwise=True)
        dw_ref = _gemm(g.t(), x, d["weight_grad"], d["act"], torch.bfloat16, rowwise=True)
    assert torch.equal(y, y_ref) and torch.equal(x.grad, dx_ref) and torch.equal(w.grad, dw_ref)


def test_hp_weight_grad_differs_from_quantized():
    from pretrain_b200.quant.linear import QuantLinear
    torch.manual_seed(0)
    lin = nn.Linear(64, 64, bias=False)
    x = torch.randn(128, 64).cuda()
    grads = []
    for cfg in (_cfg("fp8", "rowwise"), _cfg("fp8", "rowwise", weight_grad="bf16")):
        q = QuantLinear.from_linear(lin, cfg).cuda()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            q(x).float().square().mean().backward()
        grads.append(q.weight.grad.clone())
    assert not torch.equal(grads[0], grads[1]) and _rel(grads[0], grads[1]) < 0.1


@pytest.mark.parametrize("recipe", ["mxfp8", "nvfp4"])
def test_dense_mlp_block_fused_forward_equals_the_composition(recipe):
    """DenseMLPBlock (src/layers/mlp.py:103-150) after the module swap: without grad the gate/up GEMM does
    SwiGLU in its epilogue; with grad it is the plain composition of two QuantLinears.  Same result up to the
    bf16 rounding of silu(gate) * up (the epilogue follows the reference's bf16 steps; torch fuses differently)."""
    from types import SimpleNamespace
    from pretrain_b200.layers.mlp import DenseMLPBlock
    from pretrain_b200.quant.config import TrainingConfig
    from pretrain_b200.quant.convert import apply_quantization
    from pretrain_b200.quant.linear import QuantLinear
    torch.manual_seed(0)
    blk = DenseMLPBlock(256, intermediate_size=384).cuda().bfloat16()
    apply_quantization(blk, SimpleNamespace(training=TrainingConfig(quant={"enabled": True, "dtype_recipe": recipe, "exclude": []})))
    assert isinstance(blk.gate_up_proj, QuantLinear) and isinstance(blk.down_proj, QuantLinear)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        assert blk._fused_kind(x) == recipe
        fused, none = blk(x)
        gate, up = blk.gate_up_proj(x).chunk(2, dim=-1)
        comp = blk.down_proj(torch.nn.functional.silu(gate) * up)
    assert none is None and fused.shape == x.shape
    assert _rel(fused, comp) < 2e-2
    xg = x.clone().requires_grad_(True)
    assert blk._fused_kind(xg) is None
    out, _ = blk(xg)
    out.float().square().mean().backward()
    assert torch.isfinite(xg.grad).all() and blk.gate_up_proj.weight.grad is not None
    assert _rel(out, comp) < 1e-3                    # the recorded path IS the composition


def test_swapped_model_trains_one_step_and_compiles():
    from types import SimpleNamespace
    from pretrain_b200.quant.config import TrainingConfig
    from pretrain_b200.quant.convert import apply_quantization
    from pretrain_b200.quant.linear import QuantLinear
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(128, 256), nn.SiLU(), nn.Linear(256, 128)).cuda()
    cfg = SimpleNamespace(training=TrainingConfig(quant={"enabled": True, "dtype_recipe": "mxfp8", "exclude": []}))
    apply_quantization(model, cfg)
    assert sum(isinstance(m, QuantLinear) for m in model.modules()) == 2
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)
    x = torch.randn(64, 128, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        eager = model(x)
        loss = eager.float().square().mean()
    loss.backward()
    opt.step()
    assert torch.isfinite(loss)
    compiled = torch.compile(model, fullgraph=True)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        a, b = model(x), compiled(x)
    assert _rel(a, b) < 5e-2          # Inductor fuses bias add and SiLU with other roundings; requantization amplifies them


def test_fake_kernels_of_the_linear_ops_describe_the_real_outputs():
    """Shapes, dtypes and strides the compiler assumes for every custom op of the linear path against what the kernels
    return (torch.library.opcheck, fake-tensor test)."""
    from pretrain_b200 import build, torch_ops as T
    build.build()
    g = torch.Generator().manual_seed(2)
    x = torch.randn(256, 384, generator=g).bfloat16().cuda()
    w = torch.randn(512, 384, generator=g).bfloat16().cuda()
    check = lambda fn, *args: torch.library.opcheck(fn.op, args, test_utils="test_faketensor")
    check(T.amax, x)
    for axis in (1, 0):
        check(T.quantize_fp8, x, 0, axis)
        check(T.quantize_int8, x, 127, axis)
        for layout in (0, 1):
            check(T.quantize_mxfp8, x, axis, 1, layout)
            check(T.quantize_nvfp4, x, axis, layout)
    check(T.quantize_fp8_both, x, 1)
    for transpose in (False, True):
        check(T.quantize_fp8_tensorwise, x, 0, transpose)
        check(T.quantize_int8_tensorwise, x, 31, transpose)
    for layout in (0, 1):
        check(T.quantize_mxfp8_dual, x, 0, layout)
    xq, xs = T.quantize_fp8(x, 0, 1)
    wq, ws = T.quantize_fp8(w, 0, 1)
    check(T.gemm_fp8, xq, 0, wq, 0, xs, ws)
    xi, xis = T.quantize_int8(x, 127, 1)
    wi, wis = T.quantize_int8(w, 127, 1)
    check(T.gemm_int8, xi, wi, xis, wis)
    xm, xms = T.quantize_mxfp8(x, 1, 0, 1)
    wm, wms = T.quantize_mxfp8(w, 1, 0, 1)
    check(T.gemm_mxfp8, xm, xms, wm, wms, 0, 0)
    xn, xns, xnt = T.quantize_nvfp4(x, 1, 1)
    wn, wns, wnt = T.quantize_nvfp4(w, 1, 1)
    check(T.gemm_nvfp4, xn, xns, xnt, wn, wns, wnt)


@pytest.mark.parametrize("m,n,k", [(256, 384, 128), (8192, 3072, 768), (200, 264, 96), (64, 4096, 2048)])
def test_one_call_mxfp8_linear_equals_the_three_call_path(m, n, k):
    """b200q_linear_mxfp8 (one launch quantizes both operands, the GEMM follows by programmatic dependent launch) gives
    the bits of quantize + quantize + GEMM, for K-contiguous operands and for transposed storage of either one, and
    repeated back to back (the GEMM's early set-up must never read codes of the call before)."""
    from pretrain_b200 import build, ops
    build.build()
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    b = (0.05 * torch.randn(n, k, generator=g)).bfloat16().cuda()
    ca, sfa = ops.quantize_mxfp8(a, 1); cb, sfb = ops.quantize_mxfp8(b, 1)
    want = ops.gemm_mxfp8(ca, sfa, cb, sfb)
    assert torch.equal(ops.linear_mxfp8(a, 1, b, 1), want)
    for scale in (1.0, 0.5, 2.0, 0.25):                       # different inputs through the same allocator blocks
        a2 = (a * scale).bfloat16()
        c2, s2 = ops.quantize_mxfp8(a2, 1)
        assert torch.equal(ops.linear_mxfp8(a2, 1, b, 1), ops.gemm_mxfp8(c2, s2, cb, sfb))
    if m % 32 == 0:
        at, bt = a.t().contiguous(), b.t().contiguous()       # (K, M) and (K, N) storage: the transposing quantizer
        assert torch.equal(ops.linear_mxfp8(at, 0, b, 1), want)
        assert torch.equal(ops.linear_mxfp8(a, 1, bt, 0), want)
        assert torch.equal(ops.linear_mxfp8(a, 1, b, 1, ops.E5M2, ops.E4M3),
                           ops.gemm_mxfp8(*ops.quantize_mxfp8(a, 1, ops.E5M2), cb, sfb, ops.E5M2, ops.E4M3))
    ops.device_status()


def test_nvfp4_training_path_takes_each_maximum_once_and_equals_the_per_gemm_path():
    """All-NVFP4 layers quantize x, w and g in both directions under one tensor scale each (the tensor maximum taken
    once), save the transposed codes for backward and keep the weight's copies on the parameter; y, dx and dw equal what
    the three separate `_gemm` calls give, bit for bit."""
    from pretrain_b200.quant.linear import QuantLinear, QuantizedLinearFn, _gemm
    torch.manual_seed(2)
    cfg = _cfg("nvfp4")
    m, k, n = 256, 160, 96
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = nn.Parameter((0.05 * torch.randn(n, k, device="cuda")).bfloat16())
    g = (1e-2 * torch.randn(m, n, device="cuda")).bfloat16()
    y = QuantizedLinearFn.apply(x, w, None, cfg)
    y.backward(g)
    d = cfg.dtype
    with torch.no_grad():
        y_ref = _gemm(x, w.t(), d["act"], d["weight"], torch.bfloat16)
        dx_ref = _gemm(g, w, d["input_grad"], d["weight"], torch.bfloat16)
        dw_ref = _gemm(g.t(), x, d["weight_grad"], d["act"], torch.bfloat16)
    assert torch.equal(y, y_ref) and torch.equal(x.grad, dx_ref) and torch.equal(w.grad, dw_ref)
    cached = w._b200q_nv
    QuantizedLinearFn.apply(x, w, None, cfg).sum().backward()
    assert w._b200q_nv is cached
    with torch.no_grad():
        w.mul_(1.5)
    QuantizedLinearFn.apply(x, w, None, cfg)
    assert w._b200q_nv is not cached
    # against the unquantized gradients: NVFP4 noise only
    xf, wf = x.detach().float(), w.detach().float()
    q = QuantLinear(k, n, True, cfg).cuda().bfloat16()
    with torch.no_grad():
        q.weight.copy_(w); q.bias.zero_()
    xi = x.detach().clone().requires_grad_(True)
    q(xi).backward(g)
    assert _rel(q.weight.grad.float(), g.float().t() @ xf) < 0.2 and _rel(xi.grad.float(), g.float() @ wf) < 0.2
    assert torch.equal(q.bias.grad, g.sum(0))
