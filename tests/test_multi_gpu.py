"""Two-rank NCCL runs of the multi-GPU forms (skipped with fewer than 2 GPUs): the M-sharded GEMM
with output all-gather equals the single-GPU GEMM bit for bit (quantization is row-local), and
the expert-parallel MoE block equals the single-GPU block on the concatenated tokens."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import restate as R

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, fn, world, port, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        fn(rank, world, *args)
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


def _run(fn, world, *args):
    mp.spawn(_entry, args=(fn, world, _free_port(), args), nprocs=world, join=True)


def _sharded_gemm_rank(rank, world, fmt):
    from pretrain_b200 import dist as D
    from pretrain_b200.quant.linear import _gemm
    m, k, n = 1024, 512, 768
    g = torch.Generator().manual_seed(0)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (0.05 * torch.randn(n, k, generator=g)).bfloat16().cuda()
    lo, hi = D.row_shard(m, world, rank)
    full = D.sharded_gemm(a[lo:hi], w.t(), fmt, fmt, torch.bfloat16, m, rowwise=True)
    ref = _gemm(a, w.t(), fmt, fmt, torch.bfloat16, rowwise=True)
    assert full.shape == (m, n)
    if fmt == "nvfp4":       # the tensor-level scale sees only the shard's amax: same values within tolerance
        assert ((full.float() - ref.float()).norm() / ref.float().norm()).item() < 0.1
    else:
        assert torch.equal(full, ref)


@pytest.mark.parametrize("fmt", ["mxfp8", "fp8_e4m3", "nvfp4"])
def test_m_sharded_gemm_matches_single_gpu(fmt):
    _run(_sharded_gemm_rank, 2, fmt)


def _fused_rank(rank, world, fmt):
    from pretrain_b200 import dist as D, ops
    from pretrain_b200.quant.linear import _gemm
    m, k, n = 2048, 1024, 1536                 # per-rank rows; 8 x 6 pair tiles per rank
    g = torch.Generator().manual_seed(rank)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (0.05 * torch.randn(n, k, generator=torch.Generator().manual_seed(77))).bfloat16().cuda()
    out = D.GatheredOutput(m, n)
    # three passes over different inputs: the two buffer sets alternate, and a result stays valid while the next call runs
    inputs = [a, (a * 0.5 + 1.0).bfloat16(), a.flip(0).contiguous()]
    fulls = [D.sharded_gemm_fused(ai, w, fmt, out) for ai in inputs]
    torch.cuda.synchronize()
    for i, ai in enumerate(inputs):
        local = _gemm(ai, w.t(), fmt, fmt, torch.bfloat16, rowwise=True)
        ref = D.all_gather_rows(local, world * m)   # the NCCL all-gather of the same shards
        if i > 0:                                # pass 0's buffer set was reused by pass 2
            assert torch.equal(fulls[i], ref)
    assert fulls[0].data_ptr() == fulls[2].data_ptr() != fulls[1].data_ptr()
    full = fulls[2]
    ops.device_status()
    for small_m in (128, 96):                   # one-CTA kernel path, ragged rows
        o2 = D.GatheredOutput(small_m, n)
        f2 = D.sharded_gemm_fused(a[:small_m], w, fmt, o2)
        r2 = D.all_gather_rows(_gemm(a[:small_m], w.t(), fmt, fmt, torch.bfloat16, rowwise=True), world * small_m, multiple=small_m)
        torch.cuda.synchronize()
        assert torch.equal(f2, r2)


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4", "fp8_e4m3"])
def test_fused_gemm_allgather_equals_nccl_allgather(fmt):
    _run(_fused_rank, 2, fmt)


def _fused_codes_rank(rank, world):
    from pretrain_b200 import dist as D, ops
    m, k, n = 2048, 1024, 1536
    g = torch.Generator().manual_seed(rank)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (0.05 * torch.randn(n, k, generator=torch.Generator().manual_seed(77))).bfloat16().cuda()
    bf = D.GatheredOutput(m, n)
    mx = D.GatheredOutput(m, n, payload="mxfp8")
    for ai in (a, (a * 0.25).bfloat16()):
        full = D.sharded_gemm_fused(ai, w, "mxfp8", bf)
        codes, sf = D.sharded_gemm_fused(ai, w, "mxfp8", mx)
        torch.cuda.synchronize()
        # the gathered codes and scale bytes are the row-wise MXFP8 quantization of the gathered bf16 output
        want_c, want_sf = ops.quantize_mxfp8(full, 1)
        assert torch.equal(codes, want_c) and torch.equal(sf, want_sf)
    ops.device_status()
    for small_m in (128, 256):                  # one-CTA kernel path
        o2 = D.GatheredOutput(small_m, n, payload="mxfp8")
        c2, s2 = D.sharded_gemm_fused(a[:small_m], w, "mxfp8", o2)
        f2 = D.sharded_gemm_fused(a[:small_m], w, "mxfp8", D.GatheredOutput(small_m, n))
        torch.cuda.synchronize()
        wc, ws = ops.quantize_mxfp8(f2, 1)
        assert torch.equal(c2, wc) and torch.equal(s2, ws)


def test_fused_gemm_allgather_with_mxfp8_payload_equals_quantized_bf16_gather():
    _run(_fused_codes_rank, 2)


def _wgrad_rs_rank(rank, world):
    from pretrain_b200 import dist as D, ops
    m, n, k = 1024, 1536, 1024                  # tokens per rank, out features, in features
    g = torch.Generator().manual_seed(10 + rank)
    dy = (1e-2 * torch.randn(m, n, generator=g)).bfloat16().cuda()
    x = torch.randn(m, k, generator=g).bfloat16().cuda()
    out = D.ScatteredSum(n, k)
    for _ in range(3):                          # the staging buffers alternate and are reused
        dw = D.wgrad_reduce_scatter_fused(dy, x, out)
    # the same partial GEMM without the scatter, then the ranks' partials added in fp32 in rank order
    gt, gtsf = ops.quantize_mxfp8(dy, 0, torch.float8_e5m2)
    xt, xtsf = ops.quantize_mxfp8(x, 0, torch.float8_e4m3fn)
    part = ops.gemm_mxfp8(gt, gtsf, xt, xtsf, torch.float8_e5m2, torch.float8_e4m3fn)      # (n, k) bf16
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    rows = n // world
    want = torch.stack([p[rank * rows:(rank + 1) * rows].float() for p in parts]).sum(0).bfloat16()
    torch.cuda.synchronize()
    assert dw.shape == (rows, k) and torch.equal(dw, want)
    # ... and against the unquantized gradient of the whole batch
    full_dy, full_x = [torch.empty_like(dy) for _ in range(world)], [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(full_dy, dy)
    dist.all_gather(full_x, x)
    ref = (torch.cat(full_dy).float().t() @ torch.cat(full_x).float())[rank * rows:(rank + 1) * rows]
    assert ((dw.float() - ref).norm() / ref.norm()).item() < 6e-2        # E5M2 gradients x E4M3 activations
    ops.device_status()


def test_fused_wgrad_reduce_scatter_equals_sum_of_partials():
    _run(_wgrad_rs_rank, 2)


def _dp_linear_rank(rank, world, recipe):
    import torch.nn as nn
    from pretrain_b200.quant.config import TrainingConfig
    from pretrain_b200.quant.linear import QuantLinear
    q = {"enabled": True, "dtype_recipe": recipe}
    if recipe == "fp8":
        q["scaling"] = {"granularity": "rowwise"}
    cfg = TrainingConfig(quant=q).quant[0]
    m, k, n = 512, 256, 384
    torch.manual_seed(0)                                            # the same weights on every rank
    lin = nn.Linear(k, n, bias=True)
    g = torch.Generator().manual_seed(100 + rank)                   # its own shard of the batch
    x = torch.randn(m, k, generator=g).bfloat16().cuda()
    dy = (1e-2 * torch.randn(m, n, generator=g)).bfloat16().cuda()
    plain = QuantLinear.from_linear(lin, cfg).cuda().bfloat16()
    dp = QuantLinear.from_linear(lin, cfg).cuda().bfloat16().enable_data_parallel()
    for _ in range(2):                                              # the staging buffers alternate
        plain.zero_grad(); dp.zero_grad()
        plain(x).backward(dy)
        dp(x).backward(dy)
    # what summing the single-GPU gradients of the ranks gives: bf16 partials added in fp32 in rank order, one rounding
    parts = [torch.empty_like(plain.weight.grad) for _ in range(world)]
    dist.all_gather(parts, plain.weight.grad.contiguous())
    want_w = torch.stack([p.float() for p in parts]).sum(0).bfloat16()
    bparts = [torch.empty_like(plain.bias.grad) for _ in range(world)]
    dist.all_gather(bparts, plain.bias.grad.contiguous())
    want_b = torch.stack([p.float() for p in bparts]).sum(0).bfloat16()
    torch.cuda.synchronize()
    assert torch.equal(dp.weight.grad, want_w), (dp.weight.grad.float() - want_w.float()).abs().max()
    assert torch.equal(dp.bias.grad, want_b)


@pytest.mark.parametrize("recipe", ["mxfp8", "fp8"])
def test_data_parallel_quant_linear_sums_the_weight_gradient_over_the_ranks(recipe):
    """QuantLinear.enable_data_parallel: w.grad == the sum over the ranks of the single-GPU dW, bit for bit - for MXFP8
    through the wgrad GEMM whose epilogue scatters into the owners' staging buffers."""
    _run(_dp_linear_rank, 2, recipe)


def _ep_rank(rank, world):
    from pretrain_b200 import dist as D, ops
    from pretrain_b200.layers.mlp import _grouped_ffn_padded, silu_glu
    t, d, e, k, i = 1024, 256, 16, 4, 128
    x, logits, w_gu, w_d = R.inputs_moe(world * t, d, e, k, i, seed=5)
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    lo, hi, el = rank * t, (rank + 1) * t, e // world
    with torch.no_grad():
        out = D.expert_parallel_moe(x[lo:hi], top_i[lo:hi], top_w[lo:hi], w_gu[rank * el:(rank + 1) * el].contiguous(),
                                    w_d[rank * el:(rank + 1) * el].contiguous(), e)
        # single-GPU block on all tokens with the same kernels
        plan = ops.moe_permute_plan(top_i, e)
        a, sfa = ops.moe_gather(x, plan, True)
        y = _grouped_ffn_padded(a, sfa, plan, w_gu, w_d, silu_glu, True)
        ref = ops.moe_unpermute(y, top_w, plan.row_of, world * t)[lo:hi]
    # per-row arithmetic is identical; only the fp32 reduction order over a token's k rows may differ
    assert ((out.float() - ref.float()).abs().max() <= 2 ** -7 * ref.float().abs().max()).item()
    assert ((out.float() - ref.float()).norm() / ref.float().norm()).item() < 2e-3


def test_expert_parallel_moe_matches_single_gpu():
    _run(_ep_rank, 2)


def _fused_ep_rank(rank, world):
    from pretrain_b200 import dist as D, ops
    from pretrain_b200.layers.mlp import _grouped_ffn_padded, silu_glu
    t, d, e, k, i = 1024, 256, 16, 4, 128
    x, logits, w_gu, w_d = R.inputs_moe(world * t, d, e, k, i, seed=6)
    logits[:, 5] = -1e9                                                 # an expert nobody picks
    logits[: world * t // 2, 9] += 4.0                                  # and one that the first rank's tokens crowd
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    lo, hi, el = rank * t, (rank + 1) * t, e // world
    ep = D.FusedExpertParallel(t, k, d, e)
    with torch.no_grad():
        outs = [ep.forward(x[lo:hi], top_i[lo:hi], top_w[lo:hi], w_gu[rank * el:(rank + 1) * el].contiguous(),
                           w_d[rank * el:(rank + 1) * el].contiguous()) for _ in range(2)]      # buffers are reused
        plan = ops.moe_permute_plan(top_i, e)
        a, sfa = ops.moe_gather(x, plan, True)
        y = _grouped_ffn_padded(a, sfa, plan, w_gu, w_d, silu_glu, True)
        ref = ops.moe_unpermute(y, top_w, plan.row_of, world * t)[lo:hi]
    ops.device_status()
    # same rows, same kernels, same order of the k additions: the same bits as one GPU over all tokens
    assert torch.equal(outs[0], ref) and torch.equal(outs[1], ref)


def test_fused_expert_parallel_equals_single_gpu_bit_for_bit():
    """Dispatch by stores into the owners' buffers, combine by loads from them (no all-to-all)."""
    _run(_fused_ep_rank, 2)


def _fused_ep_train_rank(rank, world):
    from pretrain_b200 import dist as D, ops
    from pretrain_b200 import torch_ops as T
    from pretrain_b200.layers.mlp import _ExpertFFN, _expert_weight_copies
    t, d, e, k, i = 1024, 256, 16, 4, 128
    x, logits, w_gu, w_d = R.inputs_moe(world * t, d, e, k, i, seed=7)
    logits[:, 5] = -1e9                                                 # an expert nobody picks
    logits[: world * t // 2, 9] += 4.0                                  # and one that the first rank's tokens crowd
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    dout = torch.randn(world * t, d, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    lo, hi, el = rank * t, (rank + 1) * t, e // world
    # one GPU, all tokens, all experts: the reference for every result
    xa, wa = x.clone().requires_grad_(True), top_w.clone().requires_grad_(True)
    w1a, w2a = w_gu.clone().requires_grad_(True), w_d.clone().requires_grad_(True)
    ref = _ExpertFFN.apply(xa, wa, w1a, w2a, *_expert_weight_copies(w1a, "dual"), *_expert_weight_copies(w2a, "dual"),
                           *T.moe_permute_plan(top_i, e))
    gx, gw, g1, g2 = torch.autograd.grad(ref, (xa, wa, w1a, w2a), dout)
    # expert-parallel: my tokens, my experts
    ep = D.FusedExpertParallel(t, k, d, e, training=True)
    for _ in range(2):                                                  # buffers and flags are reused
        xl, wl = x[lo:hi].clone().requires_grad_(True), top_w[lo:hi].clone().requires_grad_(True)
        w1l = torch.nn.Parameter(w_gu[rank * el:(rank + 1) * el].clone())
        w2l = torch.nn.Parameter(w_d[rank * el:(rank + 1) * el].clone())
        out = ep.train(xl, top_i[lo:hi], wl, w1l, w2l)
        out.backward(dout[lo:hi])
    ops.device_status()
    assert torch.equal(out, ref[lo:hi])
    assert torch.equal(xl.grad, gx[lo:hi])
    assert torch.equal(w1l.grad, g1[rank * el:(rank + 1) * el]) and torch.equal(w2l.grad, g2[rank * el:(rank + 1) * el])
    rel = ((wl.grad.float() - gw[lo:hi].float()).norm() / gw[lo:hi].float().norm()).item()
    assert rel < 1e-2, rel                                              # a dot product summed in another order, rounded to bf16
    # and the gradient-free path through the same object gives the forward again
    with torch.no_grad():
        fwd = ep.forward(x[lo:hi], top_i[lo:hi], top_w[lo:hi], w_gu[rank * el:(rank + 1) * el].contiguous(),
                         w_d[rank * el:(rank + 1) * el].contiguous())
    from pretrain_b200.layers.mlp import _grouped_ffn_padded, silu_glu
    plan = ops.moe_permute_plan(top_i, e)
    a, sfa = ops.moe_gather(x, plan, True)
    y = _grouped_ffn_padded(a, sfa, plan, w_gu, w_d, silu_glu, True)
    assert torch.equal(fwd, ops.moe_unpermute(y, top_w, plan.row_of, world * t)[lo:hi])
    ops.device_status()


def test_fused_expert_parallel_training_equals_single_gpu():
    """Forward and backward of the expert-parallel block (peer scatter / combine, flag barriers, one index kernel) against the
    single-GPU expert path over all tokens: output, input gradient and expert-weight gradients bit for bit."""
    _run(_fused_ep_train_rank, 2)
