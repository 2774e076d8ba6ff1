"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own code.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/gongyisheng-pretrain

It imports ``src.quant.fp8`` and ``src.layers.mlp`` from that checkout, feeds them
seeded inputs and stores what they return (``ref_small.npz``: whole small tensors;
``ref_int8.npz``: the int8-series quantizer of ``src.quant.int8``; ``ref_digests.json``:
sha256 of codes and scales at benchmark sizes).  The tests
never need the checkout again: they compare the oracle and the CUDA kernels with
these files.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy()


def _bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def small_inputs():
    """Seeded small inputs; shapes follow the reference's tests
    (tests/fast/quant/test_fp8.py:54 uses M,K,N = 64,128,96)."""
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, 128, generator=g).to(torch.bfloat16)
    b = torch.randn(128, 96, generator=g).to(torch.bfloat16)
    grad = (1e-3 * torch.randn(64, 96, generator=g)).to(torch.bfloat16)
    edge = torch.zeros(16, 64)
    edge[1] = torch.linspace(-500, 500, 64)           # beyond e4m3 max before scaling
    edge[2] = 2.0 ** torch.arange(-40, 24).float()    # wide dynamic range
    edge[3, ::2] = -0.0
    edge[4] = 448.0 * 3
    edge[5, 0] = 1e-30                                # amax below the epsilon floor
    edge[6] = torch.randn(64, generator=g) * 1e-6
    edge[7] = torch.randn(64, generator=g) * 1e4
    edge[8:] = torch.randn(8, 64, generator=g)
    return a, b, grad, edge.to(torch.bfloat16)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from src.quant.fp8 import fake_quantize_fp8, quantize_fp8  # noqa: E402
    from src.layers.mlp import grouped_mlp  # noqa: E402
    from src.layers.activation import GATED_ACTIVATIONS  # noqa: E402

    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import restate  # only for the shared seeded input generators

    e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2
    a, b, grad, edge = small_inputs()
    out: dict[str, np.ndarray] = {}
    for name, t in (("a", a), ("b", b), ("grad", grad), ("edge", edge)):
        out[f"in_{name}"] = _bf16_bits(t)
        for dname, dt in (("e4m3", e4), ("e5m2", e5)):
            for dimname, dim in (("tensor", None), ("row", -1), ("col", 0)):
                codes, scale = quantize_fp8(t, dt, dim)
                out[f"q_{name}_{dname}_{dimname}_codes"] = _u8(codes)
                out[f"q_{name}_{dname}_{dimname}_scale"] = scale.reshape(-1).numpy()
        out[f"fq_{name}_e4m3_row"] = _bf16_bits(fake_quantize_fp8(t, e4, dim=-1))

    # NaN inputs: the reference's amax propagates a NaN into the scale of its group (row / column / tensor), and with
    # it into every code of the group (src/quant/fp8.py:26-31).  Two NaNs, in different rows and columns.
    nan_in = torch.randn(16, 64, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    nan_in[3, 5] = float("nan")
    nan_in[9, 40] = float("nan")
    out["in_nan"] = _bf16_bits(nan_in)
    for dname, dt in (("e4m3", e4), ("e5m2", e5)):
        for dimname, dim in (("tensor", None), ("row", -1), ("col", 0)):
            codes, scale = quantize_fp8(nan_in, dt, dim)
            out[f"q_nan_{dname}_{dimname}_codes"] = _u8(codes)
            out[f"q_nan_{dname}_{dimname}_scale"] = scale.reshape(-1).numpy()

    # The reference's CPU form of its rowwise FP8 GEMM (src/quant/linear.py:52-56).
    out["gemm_rowwise_e4m3"] = _bf16_bits(
        fake_quantize_fp8(a, e4, dim=-1) @ fake_quantize_fp8(b, e4, dim=0)
    )
    out["gemm_tensor_e4m3"] = _bf16_bits(fake_quantize_fp8(a, e4) @ fake_quantize_fp8(b, e4))
    # dgrad-style: e5m2 grad (64,96) x e4m3 b^T (96,128)
    out["gemm_rowwise_e5m2_e4m3"] = _bf16_bits(
        fake_quantize_fp8(grad, e5, dim=-1) @ fake_quantize_fp8(b.t(), e4, dim=0)
    )

    # MoE permute + grouped FFN + unpermute on a small case with empty experts,
    # through the reference's own tensor ops (src/layers/mlp.py:446-477).
    g = torch.Generator().manual_seed(1)
    t_, d_, e_, k_, i_ = 48, 64, 6, 2, 32
    x = torch.randn(t_, d_, generator=g).to(torch.bfloat16)
    logits = torch.randn(t_, e_, generator=g)
    logits[:, 3] = -1e9  # expert 3 never chosen
    probs = logits.softmax(-1)
    top_w, top_i = torch.topk(probs, k_, dim=-1)
    top_w = (top_w / (top_w.sum(-1, keepdim=True) + 1e-9)).to(torch.bfloat16)
    w_in = (0.02 * torch.randn(e_, 2 * i_, d_, generator=g)).to(torch.bfloat16)
    w_down = (0.02 * torch.randn(e_, d_, i_, generator=g)).to(torch.bfloat16)
    expert_ids = top_i.reshape(-1)
    token_ids = torch.arange(t_).repeat_interleave(k_)
    weights = top_w.reshape(-1, 1)
    expert_ids_sorted, order = expert_ids.sort(stable=True)
    token_ids_sorted = token_ids[order]
    weights_sorted = weights[order]
    counts = torch.bincount(expert_ids_sorted, minlength=e_)
    offs = counts.cumsum(0).to(torch.int32)
    x_sorted = x[token_ids_sorted]
    eo = grouped_mlp(x_sorted, w_in, w_down, GATED_ACTIVATIONS["silu"], offs, True)
    eo_w = eo * weights_sorted
    y = torch.zeros_like(x)
    y.index_add_(0, token_ids_sorted, eo_w)
    out.update(
        moe_x=_bf16_bits(x), moe_top_i=top_i.numpy(), moe_top_w=_bf16_bits(top_w),
        moe_w_in=_bf16_bits(w_in), moe_w_down=_bf16_bits(w_down),
        moe_order=order.numpy(), moe_token_ids_sorted=token_ids_sorted.numpy(),
        moe_counts=counts.numpy(), moe_offs=offs.numpy(),
        moe_x_sorted=_bf16_bits(x_sorted), moe_expert_out=_bf16_bits(eo), moe_y=_bf16_bits(y),
    )
    np.savez_compressed(os.path.join(HERE, "ref_small.npz"), **out)

    # int8 series (src/quant/int8.py:9-26): codes, scales and the fake-quant round trip for every
    # width and granularity, plus the reference's CPU form of its int8 GEMM (:41-47).
    from src.quant.int8 import fake_quantize_int8, quantize_int8  # noqa: E402
    i8: dict[str, np.ndarray] = {}
    for name, t in (("a", a), ("b", b), ("grad", grad), ("edge", edge)):
        for qmax in (127, 63, 31, 15, 7):
            for dimname, dim in (("tensor", None), ("row", -1), ("col", 0)):
                codes, scale = quantize_int8(t, qmax, dim)
                i8[f"q_{name}_{qmax}_{dimname}_codes"] = codes.numpy()
                i8[f"q_{name}_{qmax}_{dimname}_scale"] = scale.reshape(-1).numpy()
        i8[f"fq_{name}_127_row"] = _bf16_bits(fake_quantize_int8(t, 127, dim=-1))
    i8["gemm_rowwise_127"] = _bf16_bits(fake_quantize_int8(a, 127, dim=-1) @ fake_quantize_int8(b, 127, dim=0))
    i8["gemm_tensor_127_7"] = _bf16_bits(fake_quantize_int8(a, 127) @ fake_quantize_int8(b, 7))
    np.savez_compressed(os.path.join(HERE, "ref_int8.npz"), **i8)

    # Digests at benchmark sizes (FP8 training triple: M=16384, K=N=2048).
    x3, w3, dy3 = restate.inputs_fp8_triple()
    dig = {}
    for name, t, dt, dim in (
        ("fprop_x_row_e4m3", x3, e4, -1), ("fprop_wT_col_e4m3", w3.t(), e4, 0),
        ("dgrad_dy_row_e5m2", dy3, e5, -1), ("dgrad_w_col_e4m3", w3, e4, 0),
        ("wgrad_dyT_row_e5m2", dy3.t(), e5, -1), ("wgrad_x_col_e4m3", x3, e4, 0),
    ):
        codes, scale = quantize_fp8(t, dt, dim)
        dig[name] = {"codes": _sha(codes), "scale": _sha(scale), "shape": list(codes.shape)}
    with open(os.path.join(HERE, "ref_digests.json"), "w") as f:
        json.dump(dig, f, indent=1, sort_keys=True)
    print("wrote", len(out), "+", len(i8), "arrays and", len(dig), "digests")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/gongyisheng-pretrain")
    main(sys.argv[1])
