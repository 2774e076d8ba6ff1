"""Stream order around the library's launches: a kernel must see what a copy or memset enqueued before it on the same stream
wrote, whatever launch attributes the library uses.  A kernel launched with the programmatic-serialization attribute is not
held back by a preceding copy (it read stale inputs in 27 - 30 of 30 runs of these very sequences), which is why only
kernels that follow another kernel of the same entry point carry it.  Every case repeats the sequence with fresh buffers,
so a kernel that started early would read the previous repetition's (different) contents."""

import pytest
import torch

from oracle import restate as R

pytestmark = pytest.mark.gpu
REPS = 12


@pytest.fixture(scope="module")
def ops():
    from pretrain_b200 import ops as o
    return o


def _inputs(rep, rows=8192, cols=3072):
    g = torch.Generator().manual_seed(100 + rep)
    return (torch.randn(rows, cols, generator=g) * (1.0 + rep)).bfloat16()


def test_quantizers_see_an_async_host_copy(ops):
    for rep in range(REPS):
        h = _inputs(rep).pin_memory()
        want = (h.float().abs().max() / 2688).item()                     # NVFP4 tensor scale = amax / (448 * 6)
        d = h.cuda(non_blocking=True)
        ts = ops.quantize_nvfp4(d, 1, None, 0)[2]                         # memset + amax kernel + quantize kernel
        codes, sf = ops.quantize_mxfp8(h.cuda(non_blocking=True))        # one kernel right behind the copy
        torch.cuda.synchronize()
        assert ts.item() == want, rep
        ref_codes, ref_sf = ops.quantize_mxfp8(d)
        assert torch.equal(codes, ref_codes) and torch.equal(sf, ref_sf), rep


def test_kernels_see_a_device_copy(ops):
    base = [_inputs(rep, 4096, 2048).cuda() for rep in range(REPS)]
    w = (0.02 * torch.randn(1024, 2048)).bfloat16().cuda()
    wq, wsf = ops.quantize_mxfp8(w)
    torch.cuda.synchronize()
    for rep in range(REPS):
        x = base[rep].clone()                                            # cudaMemcpyAsync device to device
        out = ops.linear_mxfp8(x, 1, w, 1)                               # quantize both + GEMM behind the copy
        xq, xsf = ops.quantize_mxfp8(base[rep])
        cq, csf = xq.clone(), xsf.clone()                                # copies of the codes, GEMM right behind them
        out2 = ops.gemm_mxfp8(cq, csf, wq, wsf)
        torch.cuda.synchronize()
        ref = ops.gemm_mxfp8(xq, xsf, wq, wsf)
        assert torch.equal(out, ref) and torch.equal(out2, ref), rep


def test_a_memset_inside_an_entry_point_is_ordered(ops):
    """Per-column FP8 zeroes its scales (used as atomic maxima) and the tensor-wide amax zeroes its word before the kernel."""
    e4 = torch.float8_e4m3fn
    for rep in range(REPS):
        h = _inputs(rep, 4096, 1024)
        x = h.cuda()
        codes, scales = ops.quantize_fp8(x, e4, 0)
        amax = ops.amax(x)
        torch.cuda.synchronize()
        assert amax.item() == h.float().abs().max().item(), rep
        want_codes, want_scales = R.quantize_fp8(h, e4, dim=0)
        assert torch.equal(scales.cpu(), want_scales.reshape(-1)), rep


def test_a_copy_right_behind_an_entry_point_that_zeroes_by_kernel(ops):
    """The tensor maximum and the per-column scales are accumulated with atomics into words that a one-CTA kernel zeroes
    first; that kernel lets its successor be scheduled at once.  A device copy (or a read-back) enqueued directly behind
    the entry point must still see the finished result."""
    e4 = torch.float8_e4m3fn
    keep = []
    for rep in range(REPS):
        h = _inputs(rep, 4096, 1024)
        x = h.cuda()
        got = ops.amax(x).clone()                                        # device copy right behind the reduction
        back = ops.amax(x).cpu()                                         # and a read-back right behind another
        scales = ops.quantize_fp8(x, e4, 0)[1].clone()
        keep.append((h, got, back, scales))
    torch.cuda.synchronize()
    for rep, (h, got, back, scales) in enumerate(keep):
        want = h.float().abs().max().item()
        assert got.item() == want and back.item() == want, rep
        assert torch.equal(scales.cpu(), R.quantize_fp8(h, e4, dim=0)[1].reshape(-1)), rep
