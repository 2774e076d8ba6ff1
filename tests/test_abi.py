"""The C-ABI library builds for sm_100a without a GPU, loads, and exports every symbol that
include/b200q.h declares (no compute calls here)."""

import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib_path():
    from pretrain_b200 import build
    return build.build()


def _declared():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib_path):
    lib = ctypes.CDLL(lib_path)
    names = _declared()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200q.h but not exported"


def test_binding_table_matches_header(lib_path):
    from pretrain_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()


def test_host_only_entry_points(lib_path):
    from pretrain_b200 import _lib
    lib = _lib.load()
    assert lib.b200q_status_string(0) == b"ok"
    assert b"shape" in lib.b200q_status_string(-2)
    assert lib.b200q_sf_bytes(128, 4, 1) == 512
    assert lib.b200q_sf_bytes(129, 5, 1) == 2 * 2 * 512
    assert lib.b200q_sf_bytes(129, 5, 0) == 129 * 5
    from pretrain_b200 import ops                       # the Python-side size formula is the library's
    for outer in (1, 127, 128, 129, 4096):
        for nblk in (1, 3, 4, 5, 257):
            for layout in (0, 1):
                assert ops.sf_bytes(outer, nblk, layout) == lib.b200q_sf_bytes(outer, nblk, layout)
    # argument validation happens before any CUDA call
    assert lib.b200q_amax(None, 4, 8, 8, None, None) == -1
    assert lib.b200q_quantize_mxfp8(ctypes.c_void_p(16), 4, 12, 16, 1, 0, ctypes.c_void_p(16), ctypes.c_void_p(16), 1, None) == -2
    assert lib.b200q_quantize_mxfp8(ctypes.c_void_p(8), 4, 32, 32, 1, 0, ctypes.c_void_p(16), ctypes.c_void_p(16), 1, None) == -3
    # the composed entry points: workspace sizes are pure functions, and bad shapes / null pointers are refused up front
    p = ctypes.c_void_p(256)
    assert lib.b200q_moe_ffn_workspace_bytes(0, 4, 768, 64, 384) == 0
    assert lib.b200q_moe_ffn_workspace_bytes(16384, 4, 768, 64, 384) % 256 == 0 and lib.b200q_moe_ffn_workspace_bytes(16384, 4, 768, 64, 384) > 0
    assert lib.b200q_moe_ffn_forward(None, 768, p, p, 128, 4, 768, 8, 384, p, p, p, p, p, None, p, None) == -1
    assert lib.b200q_moe_ffn_forward(p, 768, p, p, 128, 4, 760, 8, 384, p, p, p, p, p, None, p, None) == -2       # D % 128
    assert lib.b200q_moe_ffn_forward(p, 768, p, p, 128, 4, 768, 8, 384, p, p, p, p, p, None, ctypes.c_void_p(128), None) == -3
    assert lib.b200q_moe_ep_forward_workspace_bytes(0, 384) == 0
    need = lib.b200q_moe_ep_forward_workspace_bytes(1024, 384)
    assert need >= 1024 * 384 + lib.b200q_sf_bytes(1024, 12, 1) and need % 256 == 0
    ptrs = (ctypes.c_void_p * 2)(256, 512)
    ep_args = [p, 768, p, 128, 4, 768, 384, 4, 2, 0, 0, p, p, p, p, 1024, p, p, p, p, p, p, 1024, ptrs, ptrs, ptrs, ptrs, p, p, p, p, p, p, None]
    bad_rank = list(ep_args); bad_rank[9] = 2
    assert lib.b200q_moe_ep_forward(*bad_rank) == -1
    bad_rows = list(ep_args); bad_rows[22] = 1000                     # rows of the receive buffers: whole 128-row tiles
    assert lib.b200q_moe_ep_forward(*bad_rows) == -2
    bad_inter = list(ep_args); bad_inter[6] = 96
    assert lib.b200q_moe_ep_forward(*bad_inter) == -2


def test_ops_refuse_cpu_tensors(lib_path):
    import torch
    from pretrain_b200 import ops
    with pytest.raises(RuntimeError):
        ops.quantize_mxfp8(torch.zeros(4, 32, dtype=torch.bfloat16))


def test_nvtx_ranges_around_every_entry_point(lib_path, monkeypatch):
    """B200Q_NVTX=1: each C-ABI call runs inside an NVTX range named after the entry point."""
    import torch
    from pretrain_b200 import _lib
    seen = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: seen.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: seen.append(("pop", None)))
    monkeypatch.setenv("B200Q_NVTX", "1")
    monkeypatch.setattr(_lib, "_lib", None)
    lib = _lib.load()
    assert lib.b200q_sf_bytes(128, 4, 1) == 512
    assert lib.b200q_status_string(0) == b"ok"
    assert seen == [("push", "b200q_sf_bytes"), ("pop", None), ("push", "b200q_status_string"), ("pop", None)]
    assert all(hasattr(lib, n) for n in _lib.SIGNATURES)
    monkeypatch.setattr(_lib, "_lib", None)                    # later tests load the plain library again
