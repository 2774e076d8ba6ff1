"""ctypes binding of libb200q.so (declared in include/b200q.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""

from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "_lib", "libb200q.so")

_i64, _int, _vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/b200q.h one to one
SIGNATURES = {
    "b200q_status_string": (ctypes.c_char_p, [_int]),
    "b200q_last_cuda_error": (_int, []),
    "b200q_device_status": (_int, []),
    "b200q_sf_bytes": (_i64, [_i64, _i64, _int]),
    "b200q_amax": (_int, [_vp, _i64, _i64, _i64, _vp, _vp]),
    "b200q_quantize_fp8": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "b200q_quantize_fp8_tensorwise": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp, _vp]),
    "b200q_quantize_mxfp8": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _int, _vp]),
    "b200q_quantize_nvfp4": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _int, _vp, _vp]),
    "b200q_quantize_fp8_both_workspace_bytes": (_i64, [_i64]),
    "b200q_quantize_fp8_both": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_quantize_int8": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "b200q_quantize_int8_tensorwise": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp, _vp]),
    "b200q_gemm_int8": (_int, [_vp, _vp, _vp, _int, _vp, _int, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200q_gemm_fp8": (_int, [_vp, _int, _vp, _int, _vp, _int, _vp, _int, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200q_gemm_mxfp8": (_int, [_vp, _int, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200q_linear_mxfp8_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b200q_linear_mxfp8": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _i64, _i64, _i64, _int, _int, _vp, _i64, _vp, _vp]),
    "b200q_gemm_nvfp4": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200q_gemm_fp8_allgather": (_int, [_vp, _int, _vp, _int, _vp, _int, _vp, _int, _i64, _i64, _i64, _vp, _int, _int, _i64, _vp]),
    "b200q_gemm_mxfp8_allgather": (_int, [_vp, _int, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _int, _int, _i64, _vp]),
    "b200q_gemm_mxfp8_allgather_mxfp8": (_int, [_vp, _int, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _vp, _int, _int, _i64, _vp]),
    "b200q_gemm_mxfp8_scatter": (_int, [_vp, _int, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _int, _int, _i64, _vp]),
    "b200q_sum_slots": (_int, [_vp, _int, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200q_gemm_nvfp4_allgather": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _int, _i64, _vp]),
    "b200q_moe_padded_rows": (_i64, [_i64, _int]),
    "b200q_moe_plan_workspace_bytes": (_i64, [_i64, _int]),
    "b200q_moe_permute_plan": (_int, [_vp, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_permute_plan_static": (_int, [_vp, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_pad_plan": (_int, [_vp, _int, _i64, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_gather": (_int, [_vp, _i64, _i64, _vp, _vp, _i64, _int, _int, _vp, _vp, _vp]),
    "b200q_grouped_gemm_mxfp8": (_int, [_vp, _int, _vp, _vp, _int, _vp, _vp, _vp, _i64, _int, _i64, _i64, _vp, _i64, _vp]),
    "b200q_grouped_gemm_mxfp8_dgrad": (_int, [_vp, _int, _vp, _vp, _int, _vp, _vp, _vp, _i64, _int, _i64, _i64, _vp, _i64, _vp]),
    "b200q_grouped_gemm_mxfp8_wgrad": (_int, [_vp, _int, _vp, _vp, _int, _vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b200q_swiglu": (_int, [_vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "b200q_gemm_mxfp8_swiglu": (_int, [_vp, _int, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "b200q_grouped_gemm_mxfp8_swiglu": (_int, [_vp, _int, _vp, _vp, _int, _vp, _vp, _vp, _i64, _int, _i64, _i64, _vp, _i64,
                                               _vp, _vp]),
    "b200q_quantize_mxfp8_dual": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _int, _vp, _vp]),
    "b200q_gemm_nvfp4_swiglu": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp]),
    "b200q_quantize_nvfp4_rowmap": (_int, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _vp, _vp]),
    "b200q_quantize_mxfp8_rowmap": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _int, _vp]),
    "b200q_quantize_mxfp8_pair": (_int, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _int, _int, _vp]),
    "b200q_moe_gather_quantize_dual": (_int, [_vp, _i64, _i64, _vp, _i64, _int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_unpermute_backward_quantize_dual": (_int, [_vp, _i64, _vp, _vp, _int, _i64, _i64, _int, _vp, _vp, _vp, _vp,
                                                         _vp, _i64, _vp, _i64, _vp, _vp, _vp]),
    "b200q_swiglu_quantize_dual": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_swiglu_backward_quantize_dual": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_dispatch_peers": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _int, _int, _vp, _vp, _vp]),
    "b200q_moe_zero_pad_rows": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "b200q_moe_combine_peers": (_int, [_vp, _int, _i64, _vp, _vp, _vp, _i64, _int, _i64, _vp, _vp]),
    "b200q_moe_ep_index": (_int, [_vp, _int, _int, _int, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp]),
    "b200q_peer_barrier": (_int, [_vp, _int, _int, _int, _vp]),
    "b200q_moe_scatter_rows_peers": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _int, _i64, _vp, _int, _i64, _vp]),
    "b200q_moe_zero_pad_rows_bf16": (_int, [_vp, _vp, _i64, _i64, _vp, _i64, _vp]),
    "b200q_moe_pair_dots_peers": (_int, [_vp, _i64, _vp, _int, _i64, _vp, _vp, _i64, _int, _i64, _vp, _vp]),
    "b200q_swiglu_backward": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "b200q_moe_unpermute_backward": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _int, _i64, _i64, _vp, _vp, _vp]),
    "b200q_moe_router_topk": (_int, [_vp, _i64, _int, _int, _int, _int, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "b200q_moe_unpermute": (_int, [_vp, _i64, _vp, _vp, _i64, _int, _i64, _vp, _vp]),
    "b200q_moe_ffn_workspace_bytes": (_i64, [_i64, _int, _i64, _int, _i64]),
    "b200q_moe_ffn_train_forward_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b200q_moe_ffn_train_forward": (_int, [_vp, _i64, _vp, _i64, _int, _i64, _int, _i64, _i64] + [_vp] * 17),
    "b200q_moe_ffn_train_backward_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b200q_moe_ffn_train_backward": (_int, [_vp, _i64, _vp, _i64, _int, _i64, _int, _i64, _i64] + [_vp] * 20),
    "b200q_moe_ffn_forward": (_int, [_vp, _i64, _vp, _vp, _i64, _int, _i64, _int, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200q_moe_pair_of_row": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "b200q_moe_ep_forward_workspace_bytes": (_i64, [_i64, _i64]),
    "b200q_moe_ep_forward": (_int, [_vp, _i64, _vp, _i64, _int, _i64, _i64, _int, _int, _int, _int, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp,
                                    _vp, _vp, _vp, _i64] + [_vp] * 11),
    # test hooks (process-wide kernel-choice overrides; see the end of include/b200q.h)
    "b200q_debug_set_gemm_bn": (_int, [_int]),
    "b200q_debug_set_gemm_pair": (_int, [_int]),
    "b200q_debug_set_gemm_bstat": (_int, [_int]),
    "b200q_debug_set_gemm_rowstat": (_int, [_int]),
    "b200q_debug_expire_wait": (_int, [_int, _vp]),
}

_lib = None


class _Traced:
    """The library with every entry point inside an NVTX range named after it (B200Q_NVTX=1): a profiler timeline then
    shows which C-ABI call each kernel belongs to, as the reference's profiling script does for its steps
    (profile/profile_model.py:77-108).  Off by default: a range costs about a microsecond of host time per call."""

    def __init__(self, lib):
        import torch
        push, pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop

        def wrap(fn, name):
            def call(*args):
                push(name)
                try:
                    return fn(*args)
                finally:
                    pop()
            return call

        for name in SIGNATURES:
            setattr(self, name, wrap(getattr(lib, name), name))


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m pretrain_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = _Traced(lib) if os.environ.get("B200Q_NVTX") == "1" else lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.b200q_status_string(status).decode()
        extra = f" (cudaError {lib.b200q_last_cuda_error()})" if status == -4 else ""
        raise RuntimeError(f"{what}: {msg}{extra}")
