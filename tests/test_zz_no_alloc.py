"""The workspace-free permute plan (b200q_moe_permute_plan_static), called through the C ABI.

It exists for hosts that cannot allocate device memory when they need a plan (a runtime with a
fixed memory arena, a foreign-language caller that owns only its tensors): its scratch is an
array built into the library.  The plan tables are integers, so its outputs must equal those of
b200q_moe_permute_plan bit for bit — checked on two calls in a row, because the second call
finds the first call's leftovers in the shared scratch.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan_buffers(n_pairs, n_experts, lib):
    rows = lib.b200q_moe_padded_rows(n_pairs, n_experts)
    i32 = dict(dtype=torch.int32, device="cuda")
    return {"offs": torch.full((n_experts,), -7, **i32), "padded_offs": torch.full((n_experts + 1,), -7, **i32),
            "row_of": torch.full((n_pairs,), -7, **i32), "src_of_row": torch.full((rows,), -7, **i32),
            "tile_expert": torch.full((rows // 128,), -7, **i32), "num_tiles": torch.full((1,), -7, **i32)}


def _ptrs(b):
    return [b[k].data_ptr() for k in ("offs", "padded_offs", "row_of", "src_of_row", "tile_expert", "num_tiles")]


@pytest.mark.parametrize("t,k,e", [(16384, 4, 64), (777, 2, 8)])
def test_static_plan_equals_workspace_plan_twice_in_a_row(t, k, e):
    from pretrain_b200 import _lib, build
    build.build()
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        g = torch.Generator().manual_seed(100 * call + t)
        top_idx = torch.topk(torch.randn(t, e, generator=g), k, dim=-1).indices.cuda().contiguous()
        n = t * k
        ref, got = _plan_buffers(n, e, lib), _plan_buffers(n, e, lib)
        ws = torch.empty(lib.b200q_moe_plan_workspace_bytes(n, e), dtype=torch.uint8, device="cuda")
        assert lib.b200q_moe_permute_plan(top_idx.data_ptr(), n, k, e, *_ptrs(ref), ws.data_ptr(), stream) == 0
        before = torch.cuda.memory_allocated()
        assert lib.b200q_moe_permute_plan_static(top_idx.data_ptr(), n, k, e, *_ptrs(got), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        for name in ref:
            assert torch.equal(ref[name], got[name]), (call, name)
        assert int(got["num_tiles"]) * 128 <= got["src_of_row"].numel() and (got["row_of"] >= 0).all()


def test_static_plan_rejects_sizes_beyond_its_scratch():
    from pretrain_b200 import _lib, build
    build.build()
    lib = _lib.load()
    n, e = 1025 * 1024, 256                       # 1025 CTAs x 256 experts > 262144 scratch entries
    dummy = ctypes.c_void_p(256)
    rc = lib.b200q_moe_permute_plan_static(dummy, n, 1, e, dummy, dummy, dummy, dummy, dummy, dummy, None)
    assert rc == -2 and b"shape" in lib.b200q_status_string(rc)
