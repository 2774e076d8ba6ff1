"""Failure detection without a GPU fault: a kernel whose bounded wait runs out records a status word and returns; the
host reads it through b200q_device_status and the Python layer raises.  The wait here is on a barrier nothing ever
signals, limited to a few thousand polls (milliseconds); nothing traps, faults or hangs, and the context stays usable."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_an_expired_device_wait_is_reported_and_cleared():
    from pretrain_b200 import _lib, build, ops
    build.build()
    lib = _lib.load()
    ops.device_status()                                        # clean to start with
    assert lib.b200q_debug_expire_wait(2000, None) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        ops.device_status()
    ops.device_status()                                        # reading it cleared it
    # the context is intact: a real kernel runs and is right
    x = torch.randn(128, 256, device="cuda").bfloat16()
    codes, sf = ops.quantize_mxfp8(x, 1)
    w = torch.randn(128, 256, device="cuda").bfloat16()
    cw, sw = ops.quantize_mxfp8(w, 1)
    out = ops.gemm_mxfp8(codes, sf, cw, sw)
    ref = x.float() @ w.float().t()
    assert ((out.float() - ref).norm() / ref.norm()).item() < 0.05
    ops.device_status()
    assert lib.b200q_debug_expire_wait(0, None) == -1 and lib.b200q_debug_expire_wait(10 ** 6, None) == -1
