"""Sentinel guard bands: every buffer the Python layer allocates for a kernel's output sits between two 64 KiB bands of
a known byte pattern, and after the launch both bands of every buffer must be intact.  Run over the cases where an
out-of-range store is most likely: ragged and empty expert groups, partial tiles in rows / columns / K, TMA-stored
tiles that hang over the edge of the matrix, per-expert output matrices."""

import math

import pytest
import torch

from oracle import restate as R

pytestmark = pytest.mark.gpu
GUARD, PATTERN = 64 * 1024, 0xA5


class Guarded:
    """Stands in for torch.empty while active: CUDA buffers come with guard bands on both sides."""

    def __init__(self):
        self.real = torch.empty
        self.bufs = []

    def empty(self, *size, dtype=None, device=None, **kw):
        if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
            size = tuple(size[0])
        dev = torch.device(device) if device is not None else torch.device("cpu")
        if dev.type != "cuda" or kw.get("pin_memory"):
            return self.real(tuple(size), dtype=dtype, device=device, **kw)
        dtype = dtype or torch.get_default_dtype()
        nbytes = math.prod(size) * dtype.itemsize
        body = (nbytes + 255) // 256 * 256
        raw = self.real(2 * GUARD + body, dtype=torch.uint8, device=dev)
        raw.fill_(PATTERN)
        self.bufs.append((raw, nbytes))
        return raw[GUARD:GUARD + nbytes].view(dtype).view(*size)

    def check(self):
        assert self.bufs
        for raw, nbytes in self.bufs:
            assert bool((raw[:GUARD] == PATTERN).all()), "bytes before an output buffer were overwritten"
            assert bool((raw[GUARD + nbytes:] == PATTERN).all()), "bytes after an output buffer were overwritten"
        n = len(self.bufs)
        self.bufs = []
        return n


@pytest.fixture
def guard(monkeypatch):
    from pretrain_b200 import build
    build.build()
    g = Guarded()
    monkeypatch.setattr(torch, "empty", g.empty)
    yield g
    monkeypatch.undo()


_MANY = [37, 0, 129, 1, 0, 0, 256, 5, 300, 0, 64, 127, 128, 2, 0, 91]


@pytest.mark.parametrize("counts", [[5, 0, 7, 4], [0, 5, 7, 4], [5, 7, 4, 0], [0, 0, 300, 0], _MANY])
def test_grouped_forward_and_backward_gemms_stay_inside_their_outputs(guard, counts):
    from pretrain_b200 import ops
    g = torch.Generator().manual_seed(sum(counts))
    r, e, d, inter = sum(counts), len(counts), 256, 128
    x = torch.randn(r, d, generator=g).bfloat16().cuda()
    w1 = (0.05 * torch.randn(e, 2 * inter, d, generator=g)).bfloat16().cuda()
    w2 = (0.05 * torch.randn(e, d, inter, generator=g)).bfloat16().cuda()
    plan = ops.moe_pad_plan(torch.tensor(counts).cumsum(0).int().cuda(), r)
    ar, asr, ac, asc = ops.moe_gather_quantize_dual(x, plan)
    a, sfa = ops.moe_gather(x, plan, True)
    w1q, w1s = ops.quantize_mxfp8_rowmap(w1.view(e * 2 * inter, d), ops.glu_row_map(e, inter, "cuda"))
    hq, hs = ops.grouped_gemm_mxfp8_swiglu(a, sfa, w1q, w1s, plan, 2 * inter)
    w2q, w2s = ops.quantize_mxfp8(w2.view(e * d, inter), 1)
    y = ops.grouped_gemm_mxfp8(hq, hs, w2q, w2s, plan, d)
    w2t, w2ts = ops.quantize_mxfp8(w2.view(e * d, inter), 0)
    gyr, gysr, gyc, gysc = ops.quantize_mxfp8_dual(torch.randn(plan.padded_rows, d, device="cuda").bfloat16(), ops.E5M2)
    dh = ops.grouped_gemm_mxfp8_dgrad(gyr, gysr, w2t, w2ts, plan, inter, ops.E5M2, ops.E4M3)
    hr, hsr, hc, hsc = ops.quantize_mxfp8_dual(torch.randn(plan.padded_rows, inter, device="cuda").bfloat16())
    dw2 = ops.grouped_gemm_mxfp8_wgrad(gyc, gysc, hc, hsc, plan, ops.E5M2, ops.E4M3)
    torch.cuda.synchronize()
    ops.device_status()
    assert guard.check() >= 20
    assert dw2.shape == (e, d, inter) and y.shape[1] == d and dh.shape[1] == inter


def test_permute_plan_gather_and_unpermute_stay_inside_their_outputs(guard):
    from pretrain_b200 import ops
    t, d, e, k = 1000, 256, 24, 3
    x, logits, _, _ = R.inputs_moe(t, d, e, k, 64, seed=2)
    logits[:, 7] = -1e9
    idx, w, probs, counts = ops.moe_router_topk(logits.cuda(), k, "softmax", True)
    plan = ops.moe_permute_plan(idx, e)
    a, sfa = ops.moe_gather(x.cuda(), plan, True)
    ab = ops.moe_gather(x.cuda(), plan, False)
    out = ops.moe_unpermute(ab, w, plan.row_of, t)
    inv = ops.moe_pair_of_row(plan)
    dy, dw = ops.moe_unpermute_backward(out, w, ab, plan)
    torch.cuda.synchronize()
    assert guard.check() >= 12 and out.shape == (t, d)


@pytest.mark.parametrize("m,n,k", [(200, 264, 96), (96, 160, 64), (1000, 520, 288), (2048 + 40, 1024 + 8, 512)])
def test_dense_gemms_and_quantizers_on_partial_tiles(guard, m, n, k):
    from pretrain_b200 import _lib, ops
    E4 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    b = torch.randn(n, k, generator=g).bfloat16().cuda()
    for pair in (-1, 1):
        _lib.load().b200q_debug_set_gemm_pair(pair)
        try:
            ca, sa = ops.quantize_fp8(a, E4, 1); cb, sb = ops.quantize_fp8(b, E4, 1)
            ops.gemm_fp8(ca, E4, cb, E4, sa, sb)
            if k % 32 == 0:
                qa, fa = ops.quantize_mxfp8(a, 1); qb, fb = ops.quantize_mxfp8(b, 1)
                ops.gemm_mxfp8(qa, fa, qb, fb)
                pa, s4a, ta = ops.quantize_nvfp4(a, 1); pb, s4b, tb = ops.quantize_nvfp4(b, 1)
                ops.gemm_nvfp4(pa, s4a, ta, pb, s4b, tb)
        finally:
            _lib.load().b200q_debug_set_gemm_pair(0)
    if m % 32 == 0 and k % 32 == 0:
        ops.quantize_mxfp8_dual(a)
        ops.quantize_mxfp8(a, 0)
        ops.quantize_nvfp4(a, 0)
    if m % 16 == 0:
        ops.quantize_fp8(a, E4, 0)
        ops.quantize_fp8_both(a, E4)
    torch.cuda.synchronize()
    ops.device_status()
    assert guard.check() >= 8


def test_quantized_output_gemm_stays_inside_its_outputs(guard):
    from pretrain_b200 import ops
    a = torch.randn(384, 256, device="cuda").bfloat16()
    b = torch.randn(640, 256, device="cuda").bfloat16()
    ca, sfa = ops.quantize_mxfp8(a); cb, sfb = ops.quantize_mxfp8(b)
    codes, sf = ops.gemm_mxfp8_quantized(ca, sfa, cb, sfb)
    torch.cuda.synchronize()
    assert guard.check() >= 6 and codes.shape == (384, 640)
