"""Benchmark of the low-precision linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one pass of the path over one batch of synthetic operands already in HBM:
quantize A (bf16 -> MXFP8), quantize B, block-scaled GEMM D = A . B^T (bf16 out) — what
`_gemm(a, b, "mxfp8", "mxfp8", ...)` does for one linear layer.  The default workload is the
square 8192^3 case the GEMM targets are quoted on.  With N > 1 (launched by torchrun, one rank
per GPU) A is sharded by rows over the ranks (B replicated) and the step ends with the all-gather
of the bf16 output shards - fused into the GEMM's epilogue, which stores every tile into all ranks'
gathered buffers over NVLink - and the rendezvous after which the gathered matrix may be read:
`value` includes both.  `--scaling weak` (default): every rank brings the workload's M rows;
`--scaling strong`: the workload's M rows are split over the ranks.  The same step without the
gather ("compute_only"), with `ncclAllGather` after the GEMM and with an MXFP8 payload are reported
beside it under "allgather".

The --steps-long block is repeated (each block bracketed by barrier + synchronize and timed with CUDA
events) until at least --min-seconds of device time have been timed; the median block is reported and
the SM clock is sampled throughout.

Prints ONE JSON line (rank 0).  `value` is device-timed whole-job TFLOPS; `e2e` is the same
metric through the public `_gemm` call with host buffers (H2D of both operands and D2H of the
result inside the timed region); `roofline` is the GEMM kernel against the measured tensor
peak (burst or sustained according to how long the kernel's loop ran); the default line also carries
the NVFP4 GEMM and the quantizers on 8192-sized operands, and `incumbent`: torch's scaled matmul
(cuBLASLt, the reference's own GPU call) on the same codes; `cpu_baseline` is the oracle's
fake-quantize-then-matmul on this box's host cores.  `--impl reference` times that CPU path alone.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "block-scaled GEMM TFLOPS/GPU (linear step: quantize A + quantize B + GEMM)"
WORKLOADS = {
    # name: (kind, M, N, K)
    "mxfp8_square_8192": ("mxfp8", 8192, 8192, 8192),
    "nvfp4_square_8192": ("nvfp4", 8192, 8192, 8192),
    "mxfp8_square_4096": ("mxfp8", 4096, 4096, 4096),
    "mxfp8_square_16384": ("mxfp8", 16384, 16384, 16384),
    "nvfp4_square_16384": ("nvfp4", 16384, 16384, 16384),
    "mxfp8_gpt2_mlp_up": ("mxfp8", 8192, 3072, 768),
    "fp8_rowwise_linear_16384x2048x2048": ("fp8", 16384, 2048, 2048),
    "int8_rowwise_linear_16384x2048x2048": ("int8", 16384, 2048, 2048),
    # MoE block: (kind, tokens, hidden, intermediate); 64 experts, top-4
    "moe_mxfp8_16384x768_e64_top4": ("moe", 16384, 768, 384),
    # the same block, forward + backward (autograd function of SparseMoEBlock, 4 more grouped GEMMs)
    "moe_mxfp8_training_16384x768_e64_top4": ("moe_train", 16384, 768, 384),
    # gated MLP in NVFP4: (kind, tokens, hidden, intermediate): gate_up GEMM, SwiGLU, re-quantize, down GEMM
    "nvfp4_mlp_16384x1024x3072": ("nvfp4_mlp", 16384, 1024, 3072),
    # the three GEMMs of one linear layer and step (fprop, dgrad, wgrad): (kind, M, N, K)
    "fp8_training_triple_16384x2048x2048": ("fp8_triple", 16384, 2048, 2048),
    "mxfp8_training_triple_16384x2048x2048": ("mxfp8_triple", 16384, 2048, 2048),
}
MOE_EXPERTS, MOE_TOPK = 64, 4
NOMINAL_TFLOPS = {"mxfp8": 4500.0, "fp8": 4500.0, "int8": 4500.0, "nvfp4": 9000.0}
# dram__bytes_read.sum + dram__bytes_write.sum per GEMM launch from the ncu captures summarised
# under profiles/ (null until captured for that workload)
GEMM_DRAM_TRAFFIC = {"mxfp8_square_8192": 386.3e6, "nvfp4_square_8192": 273.4e6,
                     "fp8_rowwise_linear_16384x2048x2048": 55.1e6}   # gemm_pair_kernel captures


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML every few milliseconds while the timed
    region runs (read-only queries)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period, self.sm, self.mask, self.max_mhz = index, period_s, [], 0, None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)

            def run():
                while not self._stop.is_set():
                    try:
                        self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        self.mask |= pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:
                        pass
                    time.sleep(self.period)

            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": [n for n, bit in self.REASONS.items() if self.mask & bit], "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle's emulated path (fake-quantize each operand along K, bf16 matmul)
# ------------------------------------------------------------------------------------------
def cpu_step(kind, a, b):
    from oracle import restate as R
    if kind == "mxfp8":
        ca, sa = R.quantize_mxfp8(a, -1)
        cb, sb = R.quantize_mxfp8(b, -1)
        fa, fb = R.dequantize_mxfp8(ca, sa).bfloat16(), R.dequantize_mxfp8(cb, sb).bfloat16()
    elif kind == "nvfp4":
        pa, sa, ta = R.quantize_nvfp4(a, -1)
        pb, sb, tb = R.quantize_nvfp4(b, -1)
        fa, fb = R.dequantize_nvfp4(pa, sa, ta).bfloat16(), R.dequantize_nvfp4(pb, sb, tb).bfloat16()
    elif kind == "int8":
        fa, fb = R.fake_quantize_int8(a, 127, dim=-1), R.fake_quantize_int8(b, 127, dim=-1)
    else:
        fa, fb = R.fake_quantize_fp8(a, torch.float8_e4m3fn, dim=-1), R.fake_quantize_fp8(b, torch.float8_e4m3fn, dim=-1)
    return fa @ fb.t()


def cpu_sample_shape(kind, m, n, k):
    """A bounded slice of the workload: full K, operands cut so one step is ~0.5 TFLOP."""
    budget = 5.5e11
    ms = max(128, min(m, int(budget / (2 * n * k)) // 128 * 128))
    ns = n if 2 * ms * n * k <= 2 * budget else max(128, int(budget / (2 * ms * k)) // 128 * 128)
    return ms, ns, k


def run_cpu(kind, m, n, k, steps, warmup, budget_s=150.0):
    """`steps` timed passes after `warmup` untimed ones, as asked - cut short only if the host is so slow that the whole
    run would pass `budget_s` seconds (the counts actually run are returned and reported)."""
    ms, ns, ks = cpu_sample_shape(kind, m, n, k)
    g = torch.Generator().manual_seed(0)
    a = torch.randn(ms, ks, generator=g).bfloat16()
    b = torch.randn(ns, ks, generator=g).bfloat16()
    start = time.perf_counter()
    cpu_step(kind, a, b)                                    # first pass: also tells how many more fit the budget
    per = time.perf_counter() - start
    fit = max(2, int(budget_s / max(per, 1e-3)))
    warmup = max(1, min(warmup, fit // 4))
    steps = max(1, min(steps, fit - warmup))
    for _ in range(warmup - 1):
        cpu_step(kind, a, b)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(kind, a, b)
    dt = (time.perf_counter() - t0) / steps
    return {"value": 2.0 * ms * ns * ks / dt / 1e12, "unit": "TFLOPS", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{ms}x{ns}x{ks} slice of the {m}x{n}x{k} workload, {steps} step(s) after {warmup} warm-up",
            "ms_per_step": dt * 1e3, "steps": steps, "warmup": warmup}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def _mark(marks):
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    marks.append(e)


def make_step(kind, a, b, out):
    """Returns (step_fn, gemm_only_fn_factory, launches_per_step).  step_fn records CUDA events
    around the GEMM launch into `marks`."""
    from pretrain_b200 import ops
    E4 = torch.float8_e4m3fn

    def step(marks=None):
        ev = (lambda: None) if marks is None else (lambda: _mark(marks))
        ev()                                        # start of the quantize kernels
        if kind == "mxfp8":
            ca, sfa = ops.quantize_mxfp8(a, 1)
            cb, sfb = ops.quantize_mxfp8(b, 1)
            ev()                                    # start of the GEMM
            ops.gemm_mxfp8(ca, sfa, cb, sfb, out=out)
        elif kind == "nvfp4":
            aa, ab = ops.amax(a), ops.amax(b)
            pa, sfa, ta = ops.quantize_nvfp4(a, 1, aa)
            pb, sfb, tb = ops.quantize_nvfp4(b, 1, ab)
            ev()
            ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb, out=out)
        elif kind == "int8":
            ca, sa = ops.quantize_int8(a, 127, 1)
            cb, sb = ops.quantize_int8(b, 127, 1)
            ev()
            ops.gemm_int8(ca, cb, sa, sb, out=out)
        else:
            ca, sa = ops.quantize_fp8(a, E4, 1)
            cb, sb = ops.quantize_fp8(b, E4, 1)
            ev()
            ops.gemm_fp8(ca, E4, cb, E4, sa, sb, out=out)
        ev()                                        # end of the GEMM
        return out

    # nvfp4: each tensor maximum is two kernels (the kernel that zeroes its word, then the reduction)
    launches = {"mxfp8": 3, "nvfp4": 7, "fp8": 3, "int8": 3}[kind]
    return step, launches


def cpu_moe_sample(t, d, inter, ts=1024):
    """The oracle's MoE path on the host cores for a sample of tokens: permute, per-expert loop
    with MXFP8 fake-quantized operands (both GEMMs, SwiGLU between), as grouped_mlp does."""
    from oracle import restate as R
    e, k = MOE_EXPERTS, MOE_TOPK
    x, logits, w_gu, w_d = R.inputs_moe(ts, d, e, k, inter)
    top_i, _ = R.router_topk(logits, k)
    fq = lambda v: R.dequantize_mxfp8(*R.quantize_mxfp8(v)).to(v.dtype)
    tc = time.perf_counter()
    order, tok, counts, offs = R.moe_permute(top_i, e)
    R.grouped_mlp_ref(x[tok], w_gu, w_d, offs, fake_quant=fq)
    dt = time.perf_counter() - tc
    return {"value": 2.0 * ts * k * (2 * inter * d + d * inter) / dt / 1e12, "unit": "TFLOPS", "cores": torch.get_num_threads(),
            "kind": "port", "sample": f"{ts} of {t} tokens through the oracle's per-expert fake-quant loop, 1 pass",
            "ms_per_step": dt * 1e3}



def run_moe(args, t, d, inter, rank, world, local):
    """MoE block workload: one step = permute plan, gather fused with MXFP8, quantize both expert
    weight stacks, grouped GEMM with the SwiGLU + MXFP8 epilogue, grouped GEMM, weighted unpermute
    (what SparseMoEBlock.forward does after the router).  Throughput counts the two grouped GEMMs'
    2*R*N*K FLOP (pad rows not counted)."""
    from oracle import restate as R
    from pretrain_b200 import build, ops
    from pretrain_b200.layers.mlp import SparseMoEBlock
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if dist is not None:
        dist.barrier()
    e, k = MOE_EXPERTS, MOE_TOPK
    x, logits, w_gu, w_d = R.inputs_moe(t, d, e, k, inter, seed=rank)
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    n_pairs = t * k
    flops = 2.0 * n_pairs * (2 * inter * d + d * inter)
    ev = lambda marks: None if marks is None else _mark(marks)
    row_map = ops.glu_row_map(e, inter, x.device)      # gate / up rows interleaved for the SwiGLU epilogue

    def step(marks=None):
        ev(marks)
        plan = ops.moe_permute_plan(top_i, e)
        a, sfa = ops.moe_gather(x, plan, True)
        ev(marks)
        wq1, wsf1 = ops.quantize_mxfp8_rowmap(w_gu.view(e * 2 * inter, d), row_map)
        wq2, wsf2 = ops.quantize_mxfp8(w_d.view(e * d, inter), 1)
        ev(marks)
        hq, hsf = ops.grouped_gemm_mxfp8_swiglu(a, sfa, wq1, wsf1, plan, 2 * inter)
        ev(marks)
        y = ops.grouped_gemm_mxfp8(hq, hsf, wq2, wsf2, plan, d)
        ev(marks)
        out = ops.moe_unpermute(y, top_w, plan.row_of, t)
        ev(marks)
        return out

    ffn_ws = torch.empty(ops.moe_ffn_workspace_bytes(t, k, d, e, inter), dtype=torch.uint8, device=x.device)

    def product_step():
        # the product call: both weight stacks quantized by one launch (every step, as the reference re-reads its weights every forward),
        # then plan, gather + MXFP8, both grouped GEMMs and the unpermute as ONE library call on a standing workspace
        wq1, wsf1, wq2, wsf2 = ops.quantize_mxfp8_pair(w_gu.view(e * 2 * inter, d), w_d.view(e * d, inter), row_map, None)
        return ops.moe_ffn_forward(x, top_i, top_w, wq1, wsf1, wq2, wsf2, e, inter, workspace=ffn_ws)[0]

    for _ in range(max(args.warmup, 3)):
        step()
        product_step()
    torch.cuda.synchronize()
    assert torch.equal(step(), product_step())
    marks = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    with ClockSampler(local) as clk:
        barrier()
        t0.record()
        for _ in range(args.steps):
            product_step()
        t1.record()
        barrier()
    ops.device_status()
    ms_step = t0.elapsed_time(t1) / args.steps
    if dist is not None:
        tt = torch.tensor([ms_step], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_step = tt.item()
    # the same step as seven library calls with events between them: the split into its parts
    barrier()
    t0.record()
    for _ in range(args.steps):
        step(marks)
    t1.record()
    barrier()
    separate_ms = t0.elapsed_time(t1) / args.steps
    seg = [marks[i:i + 6] for i in range(0, len(marks), 6)]
    avg = lambda i: sum(sg[i].elapsed_time(sg[i + 1]) for sg in seg) / len(seg)
    permute_ms, wquant_ms, gemm1_ms, gemm2_ms, unperm_ms = (avg(i) for i in range(5))

    # eight launches of 10-50 us each: also replay the step from a CUDA graph (no host launch cost between them)
    graph = None
    try:
        cg = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            product_step()
            with torch.cuda.graph(cg, stream=side):
                product_step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            cg.replay()
        torch.cuda.synchronize()
        t0.record()
        for _ in range(args.steps):
            cg.replay()
        t1.record()
        torch.cuda.synchronize()
        g_ms = t0.elapsed_time(t1) / args.steps
        graph = {"ms_per_step": g_ms, "value": world * flops / (g_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                 "note": "the same step replayed from a CUDA graph (no host launch cost)"}
    except Exception as ex:
        graph = {"error": str(ex)[:200]}

    blk = SparseMoEBlock(d, intermediate_size=inter, n_routed_experts=e, n_routed_experts_per_token=k, router_score_fn="softmax").cuda()
    with torch.no_grad():
        blk.expert_gate_up.copy_(w_gu)
        blk.expert_down.copy_(w_d)
        torch.nn.init.normal_(blk.router.gate.weight, std=0.02)
    hx = x.cpu().view(16, t // 16, d).pin_memory()
    hout = torch.empty_like(hx).pin_memory()

    def e2e_step():
        with torch.no_grad():
            o, _ = blk(hx.to("cuda", non_blocking=True))
        hout.copy_(o, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    n_e2e = max(3, min(args.steps, 20))
    t0.record()
    for _ in range(n_e2e):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / n_e2e

    # ---- expert parallelism over the ranks (tokens stay sharded, experts split): the exchange by NCCL
    # all-to-all, and by the kernels themselves over peer-mapped memory; reported beside `value`
    expert_parallel = None
    if dist is not None and e % world == 0:
        from pretrain_b200 import dist as D
        el = e // world
        w1l, w2l = w_gu[rank * el:(rank + 1) * el].contiguous(), w_d[rank * el:(rank + 1) * el].contiguous()

        def timed(fn, n=20):
            for _ in range(3):
                fn()
            dist.barrier(); torch.cuda.synchronize()
            t0.record()
            for _ in range(n):
                fn()
            t1.record()
            dist.barrier(); torch.cuda.synchronize()
            tt = torch.tensor([t0.elapsed_time(t1) / n], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return tt.item()

        with torch.no_grad():
            nccl_ms = timed(lambda: D.expert_parallel_moe(x, top_i, top_w, w1l, w2l, e))
            expert_parallel = {"nccl_all_to_all_ms": nccl_ms, "nccl_tflops": world * flops / (nccl_ms * 1e-3) / 1e12}
            try:
                ep = D.FusedExpertParallel(t, k, d, e)
                fused_ms = timed(lambda: ep.forward(x, top_i, top_w, w1l, w2l))
                expert_parallel.update(fused_ms=fused_ms, fused_tflops=world * flops / (fused_ms * 1e-3) / 1e12,
                                       fused="dispatch = gather + MXFP8 kernel storing into the owners' buffers, combine = "
                                             "unpermute kernel loading from them (symmetric memory, NVLink)")
            except Exception as ex:                       # symmetric memory not available on this system
                expert_parallel["fused_error"] = str(ex)[:200]

    # ---- incumbent: the reference's own expert path on this GPU - sort / bincount / gather, two bf16 torch._grouped_mm with
    # SwiGLU between (src/layers/mlp.py:446-477, :89,97), index_add_ - on the same tokens and weights
    incumbent = None
    if world == 1:
        try:
            import torch.nn.functional as F

            def ref_block(marks=None):
                ev(marks)
                expert_ids = top_i.reshape(-1)
                token_ids = torch.arange(t, device="cuda").repeat_interleave(k)
                ids_sorted, order = expert_ids.sort(stable=True)
                tok_sorted, w_sorted = token_ids[order], top_w.reshape(-1, 1)[order]
                offs = torch.bincount(ids_sorted, minlength=e).cumsum(0).to(torch.int32)
                xs = x[tok_sorted]
                ev(marks)
                h = torch._grouped_mm(xs, w_gu.mT, offs=offs)
                ev(marks)
                gate, up = h.chunk(2, dim=-1)
                h = F.silu(gate) * up
                ev(marks)
                y = torch._grouped_mm(h, w_d.mT, offs=offs)
                ev(marks)
                o = torch.zeros_like(x).index_add_(0, tok_sorted, y * w_sorted)
                ev(marks)
                return o

            for _ in range(3):
                ref_block()
            torch.cuda.synchronize()
            rm = []
            t0.record()
            for _ in range(20):
                ref_block(rm)
            t1.record()
            torch.cuda.synchronize()
            ref_ms = t0.elapsed_time(t1) / 20
            rseg = [rm[i:i + 6] for i in range(0, len(rm), 6)]
            ravg = lambda i: sum(sg[i].elapsed_time(sg[i + 1]) for sg in rseg) / len(rseg)
            incumbent = {"call": "the reference's expert path in bf16: sort / bincount / gather, torch._grouped_mm x 2 with SwiGLU between, index_add_ "
                                 "(src/layers/mlp.py:446-477)", "block_ms": ref_ms, "permute_ms": ravg(0), "grouped_mm1_ms": ravg(1), "swiglu_ms": ravg(2),
                         "grouped_mm2_ms": ravg(3), "unpermute_ms": ravg(4), "grouped_mm_tflops": flops / ((ravg(1) + ravg(3)) * 1e-3) / 1e12,
                         "ours_block_ms": ms_step, "speedup_block": ref_ms / ms_step,
                         "speedup_gemms": (ravg(1) + ravg(2) + ravg(3)) / (gemm1_ms + gemm2_ms),
                         "note": "speedup_gemms compares grouped_mm1 + SwiGLU + grouped_mm2 with this library's two grouped GEMMs (SwiGLU in the first one's epilogue)"}
        except Exception as ex:
            incumbent = {"error": f"{type(ex).__name__}: {str(ex)[:200]}"}

    peaks = measured_peaks()
    gemm_ms = gemm1_ms + gemm2_ms
    clocks = clk.summary()
    hbm = lambda nbytes, ms: {k2: v for k2, v in hbm_record(nbytes, ms, peaks).items() if k2 != "bound"}
    line = {"metric": "MoE block grouped-GEMM TFLOPS/GPU (permute + MXFP8 grouped GEMMs + SwiGLU + unpermute)",
            "value": world * flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp8", "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_gpu": t, "hidden": d, "intermediate": inter, "experts": e, "top_k": k,
                       "l2": "weights (108 MB bf16) + permuted activations exceed L2; no flush needed"},
            "clocks": clocks,
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": hx.numel() * 2, "d2h_bytes_per_step": hout.numel() * 2},
            "gpu_launches": 7 * args.steps,
            "roofline": roofline_tensor("grouped MXFP8 GEMMs (2 launches; the first one's epilogue does SwiGLU + MXFP8)", flops, gemm_ms, 2.0,
                                        4500.0, gemm_ms * args.steps * 1e-3, clocks, peaks, gemm1_swiglu_ms=gemm1_ms, gemm2_ms=gemm2_ms),
            "permute": dict(bound="hbm", **hbm(n_pairs * d * 3.03125, permute_ms), note="plan kernels + gather fused with MXFP8"),
            "weight_quantize": dict(bound="hbm", **hbm((w_gu.numel() + w_d.numel()) * 3.03125, wquant_ms)),
            "unpermute": dict(bound="hbm", **hbm(n_pairs * d * 2 + t * d * 2, unperm_ms))}
    line["separate_launches"] = {"ms_per_step": separate_ms, "note": "the same step as seven library calls (plan, gather, two weight quantizations, "
                                 "two grouped GEMMs, unpermute) with CUDA events between them: where the per-part times come from"}
    if graph is not None:
        line["cuda_graph"] = graph
    if expert_parallel is not None:
        line["expert_parallel"] = expert_parallel
    if incumbent is not None:
        line["incumbent"] = incumbent
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_moe_sample(t, d, inter)
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_moe_training(args, t, d, inter, rank, world, local):
    """Forward + backward of the expert path of SparseMoEBlock (after the router): every tensor quantized
    both ways once, 2 + 4 grouped MXFP8 GEMMs, SwiGLU forward and backward, unpermute forward and backward.
    FLOP = 3 x the forward's GEMM FLOP (fprop, dgrad, wgrad of both layers)."""
    from oracle import restate as R
    from pretrain_b200 import build, ops
    from pretrain_b200.layers.mlp import _ExpertFFN, _expert_weight_copies      # plain tensors: quantized every step
    from pretrain_b200 import torch_ops as T
    if rank == 0:
        build.build()
    e, k = MOE_EXPERTS, MOE_TOPK
    x, logits, w_gu, w_d = R.inputs_moe(t, d, e, k, inter, seed=rank)
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    flops = 3 * 2.0 * t * k * (2 * inter * d + d * inter)
    x.requires_grad_(True); top_w.requires_grad_(True); w_gu.requires_grad_(True); w_d.requires_grad_(True)
    dout = torch.randn(t, d, device="cuda", dtype=torch.bfloat16)

    def step():
        out = _ExpertFFN.apply(x, top_w, w_gu, w_d, *_expert_weight_copies(w_gu, "dual"), *_expert_weight_copies(w_d, "dual"),
                               *T.moe_permute_plan(top_i, e))
        return torch.autograd.grad(out, (x, top_w, w_gu, w_d), dout)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        torch.cuda.synchronize()
        t0.record()
        for _ in range(args.steps):
            step()
        t1.record()
        torch.cuda.synchronize()
    ops.device_status()
    ms_step = t0.elapsed_time(t1) / args.steps
    # ~30 launches of 10-60 us each: the eager loop is close to the host's launch rate, so also replay the
    # whole forward + backward from a CUDA graph
    graph = None
    try:
        cg = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            with torch.cuda.graph(cg, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            cg.replay()
        torch.cuda.synchronize()
        t0.record()
        for _ in range(args.steps):
            cg.replay()
        t1.record()
        torch.cuda.synchronize()
        g_ms = t0.elapsed_time(t1) / args.steps
        graph = {"ms_per_step": g_ms, "value": world * flops / (g_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                 "note": "the same forward + backward replayed from a CUDA graph (no host launch cost)"}
    except Exception as ex:
        graph = {"error": str(ex)[:200]}
    hx, hd = x.detach().cpu().pin_memory(), dout.cpu().pin_memory()
    hgx = torch.empty_like(hx).pin_memory()

    def e2e_step():
        xx = hx.to("cuda", non_blocking=True).requires_grad_(True)
        out = _ExpertFFN.apply(xx, top_w, w_gu, w_d, *_expert_weight_copies(w_gu, "dual"), *_expert_weight_copies(w_d, "dual"),
                               *T.moe_permute_plan(top_i, e))
        (gx,) = torch.autograd.grad(out, (xx,), hd.to("cuda", non_blocking=True))
        hgx.copy_(gx, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    n_e2e = max(3, min(args.steps, 10))
    t0.record()
    for _ in range(n_e2e):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / n_e2e
    peaks = measured_peaks()
    achieved = flops / (ms_step * 1e-3) / 1e12
    clocks = clk.summary()
    line = {"metric": "MoE block grouped-GEMM TFLOPS/GPU (forward + backward of the expert path)",
            "value": world * achieved, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8", "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_gpu": t, "hidden": d, "intermediate": inter, "experts": e, "top_k": k,
                       "l2": "weights and permuted activations exceed L2; no flush needed"},
            "clocks": clocks,
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (hx.numel() + hd.numel()) * 2, "d2h_bytes_per_step": hgx.numel() * 2},
            # plan 2, forward 5, backward 10 (fill + pair table 2, dy both ways + its dot partials 2, two dgrads, two wgrads,
            # SwiGLU backward, scatter to tokens), the two weight stacks 2: counted in an ncu launch list of this workload
            "gpu_launches": 19 * args.steps,
            "roofline": roofline_tensor("whole step (6 grouped GEMMs and the HBM-bound kernels between them)", flops, ms_step, 2.0, 4500.0,
                                        ms_step * args.steps * 1e-3, clocks, peaks)}
    if graph is not None:
        line["cuda_graph"] = graph
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_moe_sample(t, d, inter)
        print(json.dumps(line))


def run_composite(args, kind, d0, d1, d2, rank, world, local):
    """Workloads made of several quantize / GEMM / elementwise launches: the NVFP4 gated MLP
    (tokens d0, hidden d1, intermediate d2) and the three GEMMs of a linear layer's step in FP8
    row-wise or MXFP8 (M d0, N d1, K d2).  Every phase is event-timed; `value` counts the GEMMs' FLOP
    over the whole step."""
    from oracle import restate as R
    from pretrain_b200 import build, ops
    if rank == 0:
        build.build()
    E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    rnd = lambda *shape, scale=1.0: (scale * torch.randn(*shape, generator=g, device="cuda")).to(torch.bfloat16)
    phases = []            # (label, kind, work) in execution order; work = FLOP for gemm, bytes otherwise

    if kind == "nvfp4_mlp":
        t, h, inter = d0, d1, d2
        x, w_gu, w_d = rnd(t, h), rnd(2 * inter, h, scale=0.02), rnd(h, inter, scale=0.02)
        flops = 2.0 * t * (2 * inter * h + h * inter)

        row_map = ops.glu_row_map(1, inter, x.device)       # gate / up rows interleaved for the SwiGLU epilogue

        def step(ev):
            ev("quantize", (t * h + 2 * inter * h) * (2 + 2.5625))
            px, sx, tx = ops.quantize_nvfp4(x, 1)
            pw, sw, tw = ops.quantize_nvfp4_rowmap(w_gu, row_map)
            ev("gemm", 2.0 * t * 2 * inter * h)
            hh, h_amax = ops.gemm_nvfp4_swiglu(px, sx, tx, pw, sw, tw)       # GEMM + SwiGLU + max|h| in one kernel
            ev("quantize", t * inter * 2.5625 + h * inter * (2 + 2.5625))
            ph, sh, th = ops.quantize_nvfp4(hh, 1, h_amax)
            pd, sd, td = ops.quantize_nvfp4(w_d, 1)
            ev("gemm", 2.0 * t * h * inter)
            out = ops.gemm_nvfp4(ph, sh, th, pd, sd, td)
            ev(None, 0)
            return out
        # x, w_gu and w_d: zero + tensor maximum + quantize each (9); GEMM 1: zero of its maximum + GEMM (2); h: quantize (1); GEMM 2 (1)
        launches, dtype, peak_ratio, nominal = 13, "nvfp4", 4.0, 9000.0
        desc = {"tokens_per_gpu": t, "hidden": h, "intermediate": inter}
    else:
        m, n, k = d0, d1, d2
        x, w, dy = rnd(m, k), rnd(n, k, scale=0.02), rnd(m, n, scale=1e-3)
        flops = 3 * 2.0 * m * n * k
        if kind == "fp8_triple":
            def step(ev):
                # every tensor quantized per row and per column by one call (two reads of it, 6 B / element)
                ev("quantize", (m * k + n * k) * 6.0)
                cx, sx, cxt, sxt = ops.quantize_fp8_both(x, E4); cw, sw, cwt, swt = ops.quantize_fp8_both(w, E4)
                ev("gemm", 2.0 * m * n * k)
                y = ops.gemm_fp8(cx, E4, cw, E4, sx, sw)                         # fprop  (M,K).(N,K)^T
                ev("quantize", m * n * 6.0)
                cg, sg, cgt, sgt = ops.quantize_fp8_both(dy, E5)
                ev("gemm", 2.0 * m * n * k)
                dx = ops.gemm_fp8(cg, E5, cwt, E4, sg, swt)                      # dgrad  (M,N).(K,N)^T
                ev("gemm", 2.0 * m * n * k)
                dw = ops.gemm_fp8(cgt, E5, cxt, E4, sgt, sxt)                    # wgrad  (N,M).(K,M)^T
                ev(None, 0)
                return y, dx, dw
            launches, dtype = 3 * 3 + 3, "fp8"
        else:
            def step(ev):
                ev("quantize", (m * k + n * k) * 4.0625)
                xr, xsr, xc, xsc = ops.quantize_mxfp8_dual(x, E4); wr, wsr, wc, wsc = ops.quantize_mxfp8_dual(w, E4)
                ev("gemm", 2.0 * m * n * k)
                y = ops.gemm_mxfp8(xr, xsr, wr, wsr)
                ev("quantize", m * n * 4.0625)
                gr, gsr, gc, gsc = ops.quantize_mxfp8_dual(dy, E5)
                ev("gemm", 2.0 * m * n * k)
                dx = ops.gemm_mxfp8(gr, gsr, wc, wsc, E5, E4)
                ev("gemm", 2.0 * m * n * k)
                dw = ops.gemm_mxfp8(gc, gsc, xc, xsc, E5, E4)
                ev(None, 0)
                return y, dx, dw
            launches, dtype = 6, "mxfp8"
        peak_ratio, nominal = 2.0, 4500.0
        desc = {"M_per_gpu": m, "N": n, "K": k, "gemms": "fprop, dgrad, wgrad"}

    def run(record):
        marks = []

        def ev(label, work):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append((label, work, e))
        step(ev if record else (lambda *_: None))
        return marks

    for _ in range(max(args.warmup, 3)):
        run(False)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    all_marks = []
    with ClockSampler(local) as clk:
        torch.cuda.synchronize()
        t0.record()
        for _ in range(args.steps):
            all_marks.append(run(True))
        t1.record()
        torch.cuda.synchronize()
    ops.device_status()
    ms_step = t0.elapsed_time(t1) / args.steps
    acc = {}
    for marks in all_marks:
        for (label, work, e0), (_, _, e1) in zip(marks[:-1], marks[1:]):
            a = acc.setdefault(label, [0.0, 0.0])
            a[0] += e0.elapsed_time(e1)
            a[1] += work
    per = {lab: (ms / args.steps, work / args.steps) for lab, (ms, work) in acc.items()}

    # end to end through the public seam, host buffers in and out
    from pretrain_b200.quant.linear import QuantizedLinearFn, _gemm
    from pretrain_b200.quant.config import TrainingConfig
    import torch.nn.functional as F
    if kind == "nvfp4_mlp":
        hx = x.cpu().pin_memory()
        hout = torch.empty(d0, d1, dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            dxm = hx.to("cuda", non_blocking=True)
            gu = _gemm(dxm, w_gu.t(), "nvfp4", "nvfp4", torch.bfloat16)
            gate, up = gu.chunk(2, dim=-1)
            hout.copy_(_gemm(F.silu(gate) * up, w_d.t(), "nvfp4", "nvfp4", torch.bfloat16), non_blocking=True)
        h2d, d2h = hx.numel() * 2, hout.numel() * 2
    else:
        recipe = "fp8" if kind == "fp8_triple" else "mxfp8"
        q = {"enabled": True, "dtype_recipe": recipe}
        if recipe == "fp8":
            q["scaling"] = {"granularity": "rowwise"}
        cfg = TrainingConfig(quant=q).quant[0]
        hx, hg = x.cpu().pin_memory(), dy.cpu().pin_memory()
        hdx, hdw = torch.empty_like(hx).pin_memory(), torch.empty(d1, d2, dtype=torch.bfloat16).pin_memory()
        wp = torch.nn.Parameter(w.clone())

        def e2e_step():
            dxm = hx.to("cuda", non_blocking=True).requires_grad_(True)
            y = QuantizedLinearFn.apply(dxm, wp, None, cfg)
            gx, gw = torch.autograd.grad(y, (dxm, wp), hg.to("cuda", non_blocking=True))
            hdx.copy_(gx, non_blocking=True)
            hdw.copy_(gw, non_blocking=True)
        h2d, d2h = (hx.numel() + hg.numel()) * 2, (hdx.numel() + hdw.numel()) * 2
    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    n_e2e = max(3, min(args.steps, 10))
    t0.record()
    for _ in range(n_e2e):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / n_e2e

    peaks = measured_peaks()
    gemm_ms, gemm_flops = per["gemm"]
    q_ms, q_bytes = per["quantize"]
    clocks = clk.summary()
    incumbent = None
    if kind == "fp8_triple" and world == 1:
        # the reference's own GPU path for the same three GEMMs: fp8_gemm(rowwise=True) = two quantize_fp8 passes in torch +
        # torch._scaled_mm each (src/quant/fp8.py:35-65, src/quant/linear.py:74,98,102), here written with torch ops on the GPU
        try:
            fmax = {E4: 448.0, E5: 57344.0}

            def q_ref(t_, dt, dim):
                amax = t_.abs().amax(dim=dim, keepdim=True).float()
                sc = (amax / fmax[dt]).clamp_min(1e-12)
                return (t_.float() / sc).clamp(-fmax[dt], fmax[dt]).to(dt), sc

            def ref_gemm(a_, b_, adt, bdt):                      # a_ (M, C), b_ (C, N)
                qa, sa_ = q_ref(a_, adt, -1)
                qb, sb_ = q_ref(b_, bdt, 0)
                return torch._scaled_mm(qa.contiguous(), qb.t().contiguous().t(), scale_a=sa_, scale_b=sb_, out_dtype=torch.bfloat16)

            def ref_step():
                ref_gemm(x, w.t(), E4, E4)
                ref_gemm(dy, w, E5, E4)
                ref_gemm(dy.t(), x, E5, E4)

            ref_ms = time_loop(ref_step, reps=10, warm=3)
            cx, sx, cxt, sxt = ops.quantize_fp8_both(x, E4); cw, sw, cwt, swt = ops.quantize_fp8_both(w, E4)
            cg, sg, cgt, sgt = ops.quantize_fp8_both(dy, E5)
            mm = lambda a_, b_, sa_, sb_: torch._scaled_mm(a_, b_.t(), scale_a=sa_.view(-1, 1), scale_b=sb_.view(1, -1), out_dtype=torch.bfloat16)
            gemms_only = time_loop(lambda: (mm(cx.view(E4), cw.view(E4), sx, sw), mm(cg.view(E5), cwt.view(E4), sg, swt),
                                            mm(cgt.view(E5), cxt.view(E4), sgt, sxt)), reps=20)
            incumbent = {"call": "the reference's GPU path for the three GEMMs: quantize_fp8 (torch ops) x 2 + torch._scaled_mm each "
                                 "(src/quant/fp8.py:16-65)", "step_ms": ref_ms, "ours_step_ms": ms_step, "speedup_step": ref_ms / ms_step,
                         "scaled_mm_x3_ms": gemms_only, "ours_gemms_ms": gemm_ms, "speedup_gemms": gemms_only / gemm_ms,
                         "scaled_mm_tflops": flops / (gemms_only * 1e-3) / 1e12}
        except Exception as ex:
            incumbent = {"error": f"{type(ex).__name__}: {str(ex)[:200]}"}
    line = {"metric": METRIC.replace("linear step: quantize A + quantize B + GEMM", "all quantize + GEMM launches of the workload"),
            "value": world * flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtype, "data": "synthetic",
            "config": dict(workload=args.workload, l2="tensors of a step total > 126 MB (larger than L2); no flush needed", **desc),
            "clocks": clocks,
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches * args.steps,
            "roofline": roofline_tensor("all GEMM launches of the step", gemm_flops, gemm_ms, peak_ratio, nominal, gemm_ms * args.steps * 1e-3,
                                        clocks, peaks),
            "quantize": hbm_record(q_bytes, q_ms, peaks)}
    if "elementwise" in per:
        e_ms, e_bytes = per["elementwise"]
        line["swiglu"] = hbm_record(e_bytes, e_ms, peaks)
    if incumbent is not None:
        line["incumbent"] = incumbent
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_composite_sample(kind, d0, d1, d2)
        print(json.dumps(line))


def cpu_composite_sample(kind, d0, d1, d2, rows=1024):
    """The oracle's form of the composite workloads on the host cores, on a slice of `rows` tokens / rows."""
    from oracle import restate as R
    g = torch.Generator().manual_seed(0)
    E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2
    if kind == "nvfp4_mlp":
        x = torch.randn(rows, d1, generator=g).bfloat16()
        w_gu, w_d = (0.02 * torch.randn(2 * d2, d1, generator=g)).bfloat16(), (0.02 * torch.randn(d1, d2, generator=g)).bfloat16()
        tc = time.perf_counter()
        gu = R.nvfp4_gemm_ref(x, w_gu.t())
        gate, up = gu.chunk(2, dim=-1)
        R.nvfp4_gemm_ref(R.silu_glu(gate, up), w_d.t())
        dt = time.perf_counter() - tc
        fl = 2.0 * rows * (2 * d2 * d1 + d1 * d2)
        what = f"{rows} of {d0} tokens through the oracle's NVFP4 fake-quant MLP, 1 pass"
    else:
        n, k = d1, d2
        x, w, dy = torch.randn(rows, k, generator=g).bfloat16(), (0.02 * torch.randn(n, k, generator=g)).bfloat16(), (1e-3 * torch.randn(rows, n, generator=g)).bfloat16()
        tc = time.perf_counter()
        if kind == "fp8_triple":
            R.fp8_gemm_ref(x, w.t(), torch.bfloat16, E4, E4, rowwise=True)
            R.fp8_gemm_ref(dy, w, torch.bfloat16, E5, E4, rowwise=True)
            R.fp8_gemm_ref(dy.t(), x, torch.bfloat16, E5, E4, rowwise=True)
        else:
            R.mxfp8_gemm_ref(x, w.t(), torch.bfloat16, E4, E4)
            R.mxfp8_gemm_ref(dy, w, torch.bfloat16, E5, E4)
            R.mxfp8_gemm_ref(dy.t(), x, torch.bfloat16, E5, E4)
        dt = time.perf_counter() - tc
        fl = 3 * 2.0 * rows * n * k
        what = f"{rows} of {d0} rows through the oracle's fake-quant fprop + dgrad + wgrad, 1 pass"
    return {"value": fl / dt / 1e12, "unit": "TFLOPS", "cores": torch.get_num_threads(), "kind": "port", "sample": what,
            "ms_per_step": dt * 1e3}


# ------------------------------------------------------------------------------------------
# Timing helpers
# ------------------------------------------------------------------------------------------
MIN_TIMED_SECONDS = 2.0          # the headline loop repeats its --steps-long block until this much device time is timed


def tensor_peak(ratio, region_s, peaks):
    """Tensor-pipe denominator for a kernel timed over `region_s` seconds: `ratio` x the driver-measured bf16 cuBLAS
    rate (FP8 = 2 x, FP4 = 4 x) - the burst figure for a region that ends before the power cap settles the clock
    (under ~1 s), the sustained figure for a longer one.  Both are returned so that either fraction can be read."""
    burst, sustained = ratio * peaks["bf16_tflops"], ratio * peaks["bf16_tflops_sustained"]
    use_sustained = region_s >= 1.0
    return {"peak": sustained if use_sustained else burst, "peak_burst": burst, "peak_sustained": sustained,
            "peak_source": f"{ratio:g} x bf16_tflops{'_sustained' if use_sustained else ''} ({peaks['source']}); timed region {region_s:.2f} s"}


def roofline_tensor(kernel, flops, kernel_ms, ratio, nominal, region_s, clocks, peaks, traffic=None, **extra):
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    pk = tensor_peak(ratio, region_s, peaks)
    out = {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": pk["peak"], "unit": "TFLOP/s", "frac": achieved / pk["peak"],
           "frac_of_burst": achieved / pk["peak_burst"], "frac_of_sustained": achieved / pk["peak_sustained"], "peak_source": pk["peak_source"],
           "frac_of_nominal": achieved / nominal, "nominal_peak": nominal, "traffic": traffic, "kernel_ms": kernel_ms}
    mhz, mx = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    if mhz and mx:
        # the same kernel time expressed at the maximum SM clock: separates what the kernel loses from what the
        # power cap takes (no GPU setting is touched: the clock is only sampled)
        out["clock_normalized"] = {"sm_mhz_median": mhz, "sm_max_mhz": mx, "kernel_ms_x_mhz_over_max": kernel_ms * mhz / mx,
                                   "achieved_at_max_clock": achieved * mx / mhz, "frac_of_nominal_at_max_clock": achieved * mx / mhz / nominal}
    out.update(extra)
    return out


def hbm_record(nbytes, ms, peaks, **extra):
    gbs = nbytes / (ms * 1e-3) / 1e9
    return dict({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                 "peak_source": f"hbm_gbs, {peaks['source']}", "kernels_ms": ms, "bytes": nbytes}, **extra)


def time_loop(fn, reps=20, warm=5):
    """Mean CUDA-event time of fn() over `reps` back-to-back calls after `warm` warm-ups (ms)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(reps):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / reps


def time_kernel(fn, reps=40, inner=10):
    """Mean duration of one fn() (ms) with the launches replayed back to back from a CUDA graph of `inner` calls, timed
    with CUDA events: what a short kernel takes once the host's launch gap (about 2 us per eager launch, 5 - 10 % of a
    20 - 40 us quantizer) is out of the loop.  Returns (graph_ms, eager_ms); graph_ms is None if capture failed."""
    eager = time_loop(fn, reps=reps)
    try:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
            with torch.cuda.graph(g, stream=side):
                for _ in range(inner):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        return time_loop(g.replay, reps=max(1, reps // inner), warm=2) / inner, eager
    except Exception:
        return None, eager


def hbm_kernel_record(nbytes, fn, peaks, **extra):
    """hbm_record of one kernel-sized call: the graph-replayed duration where available, the eager loop's beside it."""
    g_ms, e_ms = time_kernel(fn)
    rec = hbm_record(nbytes, g_ms if g_ms is not None else e_ms, peaks, **extra)
    rec["timing"] = ("launches replayed back to back from a CUDA graph" if g_ms is not None else "eager loop (graph capture failed)")
    rec["eager_loop_ms"] = e_ms
    return rec


def timed_blocks(run_block, min_seconds, barrier, dist=None, max_blocks=5000):
    """run_block() enqueues exactly --steps steps.  Each block is bracketed by barrier + synchronize on both sides
    and timed with CUDA events; blocks repeat until `min_seconds` of device time have been timed (the count is
    agreed over the ranks after the first block).  Returns the per-block times in ms, max over ranks."""
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one():
        barrier()
        t0.record()
        run_block()
        t1.record()
        barrier()
        return t0.elapsed_time(t1)

    first = one()
    if dist is not None:
        t = torch.tensor([first], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        first = t.item()
    n_more = max(0, min(max_blocks, int(min_seconds * 1e3 / max(first, 1e-3)) + 1) - 1)
    times = [first] + [one() for _ in range(n_more)]
    if dist is not None:
        t = torch.tensor(times, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = t.tolist()
        times[0] = first
    return times


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


# ------------------------------------------------------------------------------------------
# Incumbents: the library kernels the reference itself calls on a GPU, timed on the same box
# ------------------------------------------------------------------------------------------
def incumbent_scaled_mm(ops, kinds, shapes, seed=7):
    """torch's scaled matmul (cuBLASLt) - `torch._scaled_mm`, the reference's GPU call at src/quant/fp8.py:59-65, and
    its block-scaled modes - on this library's own codes and scale factors, beside this library's GEMM on the same
    operands.  GEMM kernels only (operands quantized beforehand), 20 launches after 5 warm-ups each."""
    import torch.nn.functional as F
    E4, e8, f4 = torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float4_e2m1fn_x2
    S, Z = F.ScalingType, F.SwizzleType
    out = {}
    for kind, (m, n, k) in zip(kinds, shapes):
        g = torch.Generator(device="cuda").manual_seed(seed)
        a = torch.randn(m, k, generator=g, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(n, k, generator=g, device="cuda", dtype=torch.bfloat16)
        d = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        rec = {"shape": f"{m}x{n}x{k}"}
        try:
            if kind == "fp8":
                ca, sa = ops.quantize_fp8(a, E4, 1); cb, sb = ops.quantize_fp8(b, E4, 1)
                ours = lambda: ops.gemm_fp8(ca, E4, cb, E4, sa, sb, out=d)
                av, bv, sav, sbv = ca.view(E4), cb.view(E4).t(), sa.view(-1, 1), sb.view(1, -1)
                theirs = lambda: torch._scaled_mm(av, bv, scale_a=sav, scale_b=sbv, out_dtype=torch.bfloat16)
                rec["call"] = "torch._scaled_mm, per-row scales (src/quant/fp8.py:59-65)"
            elif kind == "mxfp8":
                ca, sfa = ops.quantize_mxfp8(a, 1); cb, sfb = ops.quantize_mxfp8(b, 1)
                ours = lambda: ops.gemm_mxfp8(ca, sfa, cb, sfb, out=d)
                av, bv, sav, sbv = ca.view(E4), cb.view(E4).t(), sfa.view(e8), sfb.view(e8)
                theirs = lambda: F.scaled_mm(av, bv, sav, S.BlockWise1x32, sbv, S.BlockWise1x32, swizzle_a=Z.SWIZZLE_32_4_4,
                                             swizzle_b=Z.SWIZZLE_32_4_4, output_dtype=torch.bfloat16)
                rec["call"] = "torch.nn.functional.scaled_mm, BlockWise1x32 E8M0 scales, SWIZZLE_32_4_4 (cuBLASLt)"
            else:
                pa, sfa, ta = ops.quantize_nvfp4(a, 1); pb, sfb, tb = ops.quantize_nvfp4(b, 1)
                ours = lambda: ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb, out=d)
                av, bv, sav, sbv = pa.view(f4), pb.view(f4).t(), sfa.view(E4), sfb.view(E4)
                theirs = lambda: F.scaled_mm(av, bv, sav, S.BlockWise1x16, sbv, S.BlockWise1x16, swizzle_a=Z.SWIZZLE_32_4_4,
                                             swizzle_b=Z.SWIZZLE_32_4_4, output_dtype=torch.bfloat16)
                rec["call"] = ("torch.nn.functional.scaled_mm, BlockWise1x16 E4M3 scales, SWIZZLE_32_4_4 (cuBLASLt); the fp32 tensor "
                               "scales, which this library applies in its epilogue, are left out of torch's launch")
            ours_ms = time_loop(ours)
            rec.update(ours_ms=ours_ms, ours_tflops=2.0 * m * n * k / (ours_ms * 1e-3) / 1e12)
            theirs()
            torch.cuda.synchronize()
            their_ms = time_loop(theirs)
            rec.update(incumbent_ms=their_ms, incumbent_tflops=2.0 * m * n * k / (their_ms * 1e-3) / 1e12, speedup=their_ms / ours_ms)
        except Exception as ex:                                   # torch refused this mode on this build: say so
            rec["error"] = f"{type(ex).__name__}: {str(ex).splitlines()[0][:200]}" if str(ex) else type(ex).__name__
        out[f"{kind}_{m}x{n}x{k}"] = rec
    return out


def secondary_kernels(ops, peaks, clocks):
    """The other targets quoted on the 8192-sized problem, each with its own short event-timed loop: the NVFP4 GEMM, and
    the NVFP4 / FP8 / MXFP8 quantizers on 8192 x 8192 and 16384 x 2048 bf16 operands (inputs of 128 and 64 MiB; with
    their outputs every call moves more than the 126 MB L2 holds)."""
    E4 = torch.float8_e4m3fn
    g = torch.Generator(device="cuda").manual_seed(4321)
    a = torch.randn(8192, 8192, generator=g, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(8192, 8192, generator=g, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(16384, 2048, generator=g, device="cuda", dtype=torch.bfloat16)
    d = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    pa, sfa, ta = ops.quantize_nvfp4(a, 1); pb, sfb, tb = ops.quantize_nvfp4(b, 1)
    reps = 60
    nv_ms = time_loop(lambda: ops.gemm_nvfp4(pa, sfa, ta, pb, sfb, tb, out=d), reps=reps)
    flops = 2.0 * 8192 ** 3
    out = {"roofline_nvfp4": roofline_tensor("gemm_pair_kernel<nvfp4> 8192^3", flops, nv_ms, 4.0, NOMINAL_TFLOPS["nvfp4"], reps * nv_ms * 1e-3,
                                             clocks, peaks, traffic=GEMM_DRAM_TRAFFIC.get("nvfp4_square_8192"))}
    am = ops.amax(a)
    n_el = a.numel()
    out["quantize_nvfp4"] = hbm_kernel_record(n_el * 2.5625, lambda: ops.quantize_nvfp4(a, 1, am), peaks, shape="8192x8192",
                                       note="quantize kernel alone (tensor amax given): 2 + 0.5 + 1/16 B per element")
    out["amax"] = hbm_kernel_record(n_el * 2.0, lambda: ops.amax(a), peaks, shape="8192x8192")
    out["quantize_mxfp8"] = hbm_kernel_record(n_el * 3.03125, lambda: ops.quantize_mxfp8(a, 1), peaks, shape="8192x8192")
    out["quantize_fp8"] = hbm_kernel_record(n_el * (3.0 + 4.0 / 8192), lambda: ops.quantize_fp8(a, E4, 1), peaks, shape="8192x8192",
                                     note="per-row FP8 (src/quant/fp8.py:16-32 with dim=-1)")
    nx = x.numel()
    out["quantize_fp8_16384x2048"] = hbm_kernel_record(nx * (3.0 + 4.0 / 2048), lambda: ops.quantize_fp8(x, E4, 1), peaks, shape="16384x2048")
    out["quantize_fp8_both_16384x2048"] = hbm_kernel_record(nx * 4.0, lambda: ops.quantize_fp8_both(x, E4), peaks, shape="16384x2048",
                                                     note="per row and per column from one call; algorithmic bytes: one read, two sets of codes")
    out["quantize_mxfp8_dual_16384x2048"] = hbm_kernel_record(nx * 4.0625, lambda: ops.quantize_mxfp8_dual(x, E4), peaks, shape="16384x2048")
    return out


def run_dense(args, kind, m, n, k, rank, world, local, config):
    """Square / linear-layer workloads: quantize A, quantize B, GEMM.  One GPU: that step.  N GPUs: M sharded over the
    ranks (weak: every rank brings `m` rows; strong: `m` rows in total), B replicated, and the step ends with the
    all-gather of the output shards, fused into the GEMM's epilogue (TMA stores into the peers' gathered buffers over
    NVLink), plus the rendezvous that makes the gathered matrix readable - all inside `value`."""
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from pretrain_b200 import build, ops
    if rank == 0:
        build.build()
    if dist is not None:
        dist.barrier()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def rank_max(*vals):
        if dist is None:
            return vals if len(vals) > 1 else vals[0]
        t = torch.tensor(vals, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist() if len(vals) > 1 else t.item()

    strong = args.scaling == "strong" and world > 1
    m_rank = m // world if strong else m                 # rows of A (and of the output) this rank computes
    if strong and (m % (128 * world)):
        raise SystemExit("--scaling strong needs M to split into 128-row tiles per rank")
    peaks = measured_peaks()
    fmt = {"mxfp8": "mxfp8", "nvfp4": "nvfp4", "fp8": "fp8_e4m3", "int8": "int8"}[kind]
    ratio = {"mxfp8": 2.0, "fp8": 2.0, "int8": 2.0, "nvfp4": 4.0}[kind]
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    a = torch.randn(m_rank, k, generator=g, device="cuda", dtype=torch.bfloat16)
    gb = torch.Generator(device="cuda").manual_seed(99)
    b = torch.randn(n, k, generator=gb, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m_rank, n, device="cuda", dtype=torch.bfloat16)
    compute_step, launches = make_step(kind, a, b, out)
    flops = 2.0 * m_rank * n * k                         # per rank and step
    warm = max(args.warmup, 3)

    gathered = None
    if dist is not None and kind != "int8":
        from pretrain_b200 import dist as D
        gathered = D.GatheredOutput(m_rank, n)
        step = lambda: D.sharded_gemm_fused(a, b, fmt, gathered)      # the product call: quantize x 2, GEMM + gather, rendezvous
    elif kind == "mxfp8":
        step = lambda: ops.linear_mxfp8(a, 1, b, 1, out=out)          # what `_gemm(a, b, "mxfp8", "mxfp8")` runs: one library call
    else:
        step = compute_step

    # ---- headline: blocks of --steps steps until --min-seconds of device time -------------------
    for _ in range(warm):
        step()
    barrier()
    if args.profile:
        torch.cuda.profiler.start()
        torch.cuda.nvtx.range_push("b200q timed region")
    with ClockSampler(local) as clk:
        block_ms = timed_blocks(lambda: [step() for _ in range(args.steps)], args.min_seconds, barrier, dist)
    if args.profile:
        torch.cuda.nvtx.range_pop()
        torch.cuda.profiler.stop()
    ops.device_status()
    clocks = clk.summary()
    timed_region_s = sum(block_ms) * 1e-3
    ms_step = median(block_ms) / args.steps
    value = world * flops / (ms_step * 1e-3) / 1e12

    # ---- the same work as separate launches with CUDA events between them: the quantize / GEMM split, and (N > 1) the
    # step without the gather.  Runs as long as the headline loop, so the GEMM's rate is a sustained one like the headline's. ----
    marks = []
    for _ in range(3):
        compute_step()
    barrier()
    with ClockSampler(local) as clk_split:
        split_ms = timed_blocks(lambda: [compute_step(marks) for _ in range(args.steps)], args.min_seconds, barrier, dist)
    co_ms = median(split_ms) / args.steps
    co_region_s = sum(split_ms) * 1e-3
    split_clocks = clk_split.summary()
    trip = [marks[i:i + 3] for i in range(0, len(marks), 3)]
    quant_ms = sum(q.elapsed_time(g0) for q, g0, _ in trip) / len(trip)
    gemm_ms = sum(g0.elapsed_time(g1) for _, g0, g1 in trip) / len(trip)
    gemm_ms, quant_ms = rank_max(gemm_ms, quant_ms)

    # Short steps are bound by the host's launch rate, not by the GPU: replay the same step from a CUDA graph
    # (what a training loop that cares would do) and report it beside the eager number.
    graph = None
    if co_ms < 0.25 and dist is None:
        try:
            cg = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                compute_step()
                with torch.cuda.graph(cg, stream=side):
                    compute_step()
            torch.cuda.current_stream().wait_stream(side)
            g_ms = time_loop(cg.replay, reps=max(args.steps, 20), warm=3)
            graph = {"ms_per_step": g_ms, "value": world * flops / (g_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                     "note": "the same step replayed from a CUDA graph (no host launch cost)"}
        except Exception as ex:
            graph = {"error": str(ex)[:200]}

    # ---- end to end through the public call, host buffers --------------------------------
    from pretrain_b200.quant.linear import _gemm
    # B is replicated over the ranks: with more than one rank each copies only ITS 1/world of B's rows from its
    # host buffer and the ranks all-gather the rest over NVLink (NCCL), so the host link carries every input
    # byte of the job once per step instead of B once per rank.
    shard_b = dist is not None and n % world == 0
    nb = n // world if shard_b else n
    b_lo = rank * nb if shard_b else 0
    ha, hb = a.cpu().pin_memory(), b[b_lo:b_lo + nb].cpu().pin_memory()
    hout = torch.empty(m_rank, n, dtype=torch.bfloat16).pin_memory()

    # Three streams and two sets of device buffers: step i's host->device copy, step i-1's quantize + GEMM and
    # step i-2's device->host copy overlap (PCIe is full duplex and the copy engines run beside the SMs); every
    # step still copies its own inputs in and its own result out inside the timed region.
    s_in, s_in2, s_c, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    dbuf = [(torch.empty_like(a), torch.empty_like(b), torch.empty(m_rank, n, device="cuda", dtype=torch.bfloat16)) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_in2 = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        j = i & 1
        da, db, dd = dbuf[j]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_c[j])                    # the step that last read these input buffers is done
            da.copy_(ha, non_blocking=True)
            ev_in[j].record()
        with torch.cuda.stream(s_in2):                  # the two operands travel on two streams
            s_in2.wait_event(ev_c[j])
            db[b_lo:b_lo + nb].copy_(hb, non_blocking=True)
            ev_in2[j].record()
        with torch.cuda.stream(s_c):
            s_c.wait_event(ev_in[j])
            s_c.wait_event(ev_in2[j])
            s_c.wait_event(ev_out[j])                   # the result buffer has been read back
            if shard_b:
                dist.all_gather_into_tensor(db, db[b_lo:b_lo + nb])
            dd.copy_(_gemm(da, db.t(), fmt, fmt, torch.bfloat16, rowwise=True))
            ev_c[j].record()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_c[j])
            hout.copy_(dd, non_blocking=True)
            ev_out[j].record()

    def e2e_run(count):
        for st in (s_in, s_in2, s_c, s_out):
            st.wait_stream(torch.cuda.current_stream())
        for i in range(count):
            e2e_step(i)
        for st in (s_in, s_in2, s_c, s_out):
            torch.cuda.current_stream().wait_stream(st)

    e2e_steps = max(4, min(args.steps, 12))
    e2e_run(4)
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_run(e2e_steps)
    t1.record()
    barrier()
    e2e_ms = rank_max(t0.elapsed_time(t1) / e2e_steps)
    e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": ha.numel() * 2 + hb.numel() * 2, "d2h_bytes_per_step": hout.numel() * 2}
    if shard_b:
        e2e["replicated_operand"] = "each rank copies 1/%d of B from host; ncclAllGather over NVLink completes it" % world
    if kind == "mxfp8":
        # The same product with B as a layer's weight: QuantLinear keeps the weight (and its codes, made once) on the
        # device, so a step copies only the activation in and the result out - what src/quant/linear.py:73-76 would
        # re-quantize every call.  Reported beside the main figure, which copies and quantizes both operands every step.
        from pretrain_b200.quant.config import QuantConfig, normalize_quant_rules
        from pretrain_b200.quant.linear import QuantLinear
        rule = normalize_quant_rules(QuantConfig(enabled=True, dtype_recipe="mxfp8"))[0]
        layer = QuantLinear(k, n, False, rule).to("cuda", torch.bfloat16)
        with torch.no_grad():
            layer.weight.copy_(b)
        ev_r = [torch.cuda.Event() for _ in range(2)]

        def resident_step(i):
            j = i & 1
            da, _, dd = dbuf[j]
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_c[j])
                da.copy_(ha, non_blocking=True)
                ev_in[j].record()
            with torch.cuda.stream(s_c):
                s_c.wait_event(ev_in[j])
                s_c.wait_event(ev_out[j])
                with torch.no_grad():
                    dd.copy_(layer(da))
                ev_c[j].record()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c[j])
                hout.copy_(dd, non_blocking=True)
                ev_out[j].record()

        def resident_run(count):
            for st in (s_in, s_c, s_out):
                st.wait_stream(torch.cuda.current_stream())
            for i in range(count):
                resident_step(i)
            for st in (s_in, s_c, s_out):
                torch.cuda.current_stream().wait_stream(st)

        try:
            resident_run(4)
            barrier()
            t0.record()
            resident_run(e2e_steps)
            t1.record()
            barrier()
            r_ms = rank_max(t0.elapsed_time(t1) / e2e_steps)
            e2e["weight_resident"] = {"value": world * flops / (r_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": r_ms,
                                      "h2d_bytes_per_step": ha.numel() * 2, "d2h_bytes_per_step": hout.numel() * 2,
                                      "note": "B held by a QuantLinear as its weight (codes cached on the parameter); only A travels in"}
        except Exception as ex:
            e2e["weight_resident"] = {"error": str(ex)[:200]}

    # ---- the gather in its other forms, beside `value` -----------------------------------------
    allgather = None
    if gathered is not None:
        from pretrain_b200 import dist as D
        link_bytes = (world - 1) * m_rank * n            # elements every rank receives
        reps = 10
        allgather = {"in_value": "bf16 payload, fused into the GEMM epilogue (TMA stores into every rank's gathered buffer), rendezvous included",
                     "ms_per_step": ms_step, "ingress_gbs_per_rank": link_bytes * 2 / (ms_step * 1e-3) / 1e9,
                     "bytes_received_per_rank": link_bytes * 2,
                     "link_bound_ms": link_bytes * 2 / 770e9 * 1e3, "link_note": "770 GB/s per direction per GPU (measured peer copy on this pool)"}

        def timed(fn):
            for _ in range(3):
                fn()
            barrier()
            t0.record()
            for _ in range(reps):
                fn()
            t1.record()
            barrier()
            return rank_max(t0.elapsed_time(t1) / reps)

        full = torch.empty(world * m_rank, n, device="cuda", dtype=torch.bfloat16)

        def nccl_step():
            compute_step()
            dist.all_gather_into_tensor(full, out)

        nccl_ms = timed(nccl_step)
        allgather["nccl"] = {"ms_per_step": nccl_ms, "tflops": world * flops / (nccl_ms * 1e-3) / 1e12,
                             "collective": "ncclAllGather of the bf16 shards after the GEMM"}
        del full
        if kind == "mxfp8" and m_rank % 128 == 0 and n % 128 == 0:
            try:
                gq = D.GatheredOutput(m_rank, n, payload="mxfp8")
                q_ms = timed(lambda: D.sharded_gemm_fused(a, b, fmt, gq))
                qb = link_bytes * 1.03125
                allgather["mxfp8_payload"] = {
                    "ms_per_step": q_ms, "tflops": world * flops / (q_ms * 1e-3) / 1e12, "bytes_received_per_rank": qb,
                    "ingress_gbs_per_rank": qb / (q_ms * 1e-3) / 1e9, "link_bound_ms": qb / 770e9 * 1e3,
                    "what": "the epilogue quantizes each output tile (rounded to bf16 first) to E4M3 codes + E8M0 scale bytes, bit-identical "
                            "to quantizing the gathered bf16 matrix along its columns: the form the next block-scaled GEMM consumes"}
            except Exception as ex:
                allgather["mxfp8_payload"] = {"error": str(ex)[:200]}
        ops.device_status()

    # ---- data-parallel wgrad: dW = sum over ranks of dY_r^T . X_r, reduce-scattered by rows ----
    reduce_scatter = None
    if dist is not None and kind == "mxfp8" and not strong and n % (32 * world) == 0:
        try:
            from pretrain_b200 import dist as D
            e5, e4 = torch.float8_e5m2, torch.float8_e4m3fn
            dy = (1e-2 * torch.randn(m_rank, n, generator=g, device="cuda")).to(torch.bfloat16)
            shard = torch.empty(n // world, k, device="cuda", dtype=torch.bfloat16)

            def nccl_rs_step():
                gt, gtsf = ops.quantize_mxfp8(dy, 0, e5)
                xt, xtsf = ops.quantize_mxfp8(a, 0, e4)
                dist.reduce_scatter_tensor(shard, ops.gemm_mxfp8(gt, gtsf, xt, xtsf, e5, e4))

            sc = D.ScatteredSum(n, k)
            times = []
            for fn in (nccl_rs_step, lambda: D.wgrad_reduce_scatter_fused(dy, a, sc)):
                for _ in range(3):
                    fn()
                barrier()
                t0.record()
                for _ in range(10):
                    fn()
                t1.record()
                barrier()
                times.append(rank_max(t0.elapsed_time(t1) / 10))
            reduce_scatter = {"workload": "wgrad of the same shape per rank (2 transposing quantizations + GEMM), dW summed over ranks",
                              "nccl_ms_per_step": times[0], "nccl_tflops": world * flops / (times[0] * 1e-3) / 1e12,
                              "fused_ms_per_step": times[1], "fused_tflops": world * flops / (times[1] * 1e-3) / 1e12,
                              "bytes_sent_per_rank": (world - 1) * (n // world) * k * 2,
                              "fused": "GEMM epilogue stores each block into its owner's staging slot (symmetric memory, NVLink); "
                                       "one kernel adds the slots"}
        except Exception as ex:
            reduce_scatter = {"error": str(ex)[:200]}

    # ---- expert-parallel MoE (BASELINE config 4: 16384 tokens in all, 64 experts, top-4) beside the GEMM numbers ----
    expert_parallel = None
    if dist is not None and not strong and MOE_EXPERTS % world == 0 and args.workload == "mxfp8_square_8192":
        try:
            expert_parallel = expert_parallel_record(dist, rank, world, barrier, rank_max)
        except Exception as ex:
            expert_parallel = {"error": str(ex)[:300]}

    secondary, incumbent = {}, None
    if world == 1 and args.workload == "mxfp8_square_8192" and not args.headline_only:
        secondary = secondary_kernels(ops, peaks, clocks)
        incumbent = incumbent_scaled_mm(ops, ["mxfp8", "nvfp4", "fp8"], [(8192, 8192, 8192), (8192, 8192, 8192), (16384, 2048, 2048)])

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # fp8 / fp4 tensor peak is not measured directly: the driver's measured bf16 cuBLAS rate times the format's rate
    # ratio - the burst figure when the timed region is shorter than a second, the sustained one otherwise
    roofline = roofline_tensor(f"gemm_pair_kernel<{kind}> / gemm_kernel<{kind}> (chosen by shape)", flops, gemm_ms, ratio, NOMINAL_TFLOPS[kind],
                               co_region_s, split_clocks, peaks, traffic=GEMM_DRAM_TRAFFIC.get(args.workload),
                               timed="CUDA events around the GEMM launch of every step of the separate-launch loop")
    # the quantize kernels of the step against the measured HBM copy bandwidth (algorithmic bytes:
    # bf16 in, codes + scale bytes out; NVFP4 also reads each operand once more for its amax)
    bpe = {"mxfp8": 3.03125, "fp8": 3.0, "int8": 3.0, "nvfp4": 2.0 + 2.5625}[kind]
    quantize = hbm_record((m_rank * k + n * k) * bpe, quant_ms, peaks, note="the quantize launches of every step of the separate-launch loop")
    config = dict(config, M_per_gpu=m_rank, scaling=args.scaling if world > 1 else "single GPU",
                  step=("quantize A, quantize B, GEMM with the bf16 output all-gather in its epilogue, rendezvous" if gathered is not None
                        else ("one b200q_linear_mxfp8 call: A and B quantized by one launch, GEMM launched behind it (programmatic dependent launch)"
                              if kind == "mxfp8" else "quantize A, quantize B, GEMM")))
    line = {"metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": kind,
            "data": "synthetic", "config": config, "clocks": clocks, "timed_region_s": timed_region_s, "timed_blocks": len(block_ms),
            "block_ms": {"median": median(block_ms), "min": min(block_ms), "max": max(block_ms)},
            "e2e": e2e, "gpu_launches": (launches - (1 if kind == "mxfp8" and gathered is None else 0)) * args.steps * len(block_ms), "roofline": roofline, "quantize": quantize}
    line["separate_launches"] = {"ms_per_step": co_ms, "tflops": world * flops / (co_ms * 1e-3) / 1e12, "timed_region_s": co_region_s,
                                 "note": "quantize A, quantize B, GEMM as three library calls with CUDA events between them" +
                                         (" and no gather (N independent shards): the compute-only step" if gathered is not None else "")}
    if gathered is not None:
        line["compute_only"] = line["separate_launches"]
    line.update(secondary)
    if incumbent is not None:
        line["incumbent"] = incumbent
    if graph is not None:
        line["cuda_graph"] = graph
    if allgather is not None:
        line["allgather"] = allgather
    if reduce_scatter is not None:
        line["reduce_scatter"] = reduce_scatter
    if expert_parallel is not None:
        line["expert_parallel"] = expert_parallel
    if world == 1 and not args.no_cpu_baseline:
        cb = run_cpu(kind, m, n, k, 2, 1)
        line["cpu_baseline"] = {k2: cb[k2] for k2 in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def expert_parallel_record(dist, rank, world, barrier, rank_max, total_tokens=16384, d=768, inter=384):
    """BASELINE config 4 as written: 16384 tokens in total, tokens sharded over the ranks, 64 experts split E / N per GPU,
    top-4; forward of the expert path.  Two forms: exchange by NCCL all-to-all, and by the kernels themselves over
    peer-mapped memory.  FLOP = the two grouped GEMMs over all routed rows of the job."""
    from oracle import restate as R
    from pretrain_b200 import dist as D
    e, k = MOE_EXPERTS, MOE_TOPK
    t = total_tokens // world
    x, logits, w_gu, w_d = R.inputs_moe(t, d, e, k, inter, seed=rank)
    top_i, top_w = R.router_topk(logits, k)
    x, top_i, top_w, w_gu, w_d = (v.cuda() for v in (x, top_i, top_w, w_gu, w_d))
    el = e // world
    w1l, w2l = w_gu[rank * el:(rank + 1) * el].contiguous(), w_d[rank * el:(rank + 1) * el].contiguous()
    flops = 2.0 * total_tokens * k * (2 * inter * d + d * inter)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        barrier()
        t0.record()
        for _ in range(reps):
            fn()
        t1.record()
        barrier()
        return rank_max(t0.elapsed_time(t1) / reps)

    rec = {"workload": f"{total_tokens} tokens in total ({t} per rank), hidden {d}, {e} experts ({el} per GPU), top-{k}, intermediate {inter}; forward"}
    with torch.no_grad():
        nccl_ms = timed(lambda: D.expert_parallel_moe(x, top_i, top_w, w1l, w2l, e))
        rec.update(nccl_all_to_all_ms=nccl_ms, nccl_tflops=flops / (nccl_ms * 1e-3) / 1e12)
        ep = D.FusedExpertParallel(t, k, d, e, training=True)     # default capacity: cannot overflow, no host check per call
        fused_ms = timed(lambda: ep.forward(x, top_i, top_w, w1l, w2l))
        rec.update(fused_ms=fused_ms, fused_tflops=flops / (fused_ms * 1e-3) / 1e12,
                   fused="dispatch = gather + MXFP8 kernel storing into the owners' buffers, combine = unpermute kernel loading from "
                         "them (symmetric memory, NVLink); phases ordered by flag barriers in peer memory, index tables by one kernel")
    # forward + backward of the same block (bf16 rows on the wire, the owners' six grouped GEMMs in MXFP8)
    w1p, w2p = torch.nn.Parameter(w1l), torch.nn.Parameter(w2l)
    xg, wg = x.clone().requires_grad_(True), top_w.clone().requires_grad_(True)
    dout = torch.randn(t, d, device="cuda", dtype=torch.bfloat16)

    def train_step():
        out = ep.train(xg, top_i, wg, w1p, w2p)
        torch.autograd.grad(out, (xg, wg, w1p, w2p), dout)

    train_ms = timed(train_step, reps=10)
    rec.update(fused_train_ms=train_ms, fused_train_tflops=3 * flops / (train_ms * 1e-3) / 1e12)
    return rec



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200q", choices=["b200q", "reference"])
    ap.add_argument("--workload", default="mxfp8_square_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1: weak = every rank brings the workload's M rows; strong = the workload's M rows are split over the ranks")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="repeat the --steps-long block until this much device time has been timed; the median block is reported")
    ap.add_argument("--headline-only", action="store_true", help="skip the secondary kernels and the incumbent timings of the default line")
    ap.add_argument("--profile", action="store_true",
                    help="bracket the headline timed region with cudaProfilerStart / cudaProfilerStop and an NVTX range "
                         "(for `ncu --profile-from-start off` / a timeline); numbers printed under a profiler are not bench values")
    args = ap.parse_args()
    kind, m, n, k = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # NCCL only carries the comparators and the plumbing here; without NVLink multicast objects a rank that dies cannot
        # leave its peers with memory bound to one
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    config = {"workload": args.workload, "kind": kind, "M_per_gpu": m, "N": n, "K": k,
              "sharding": "rows of A (M) across ranks, B replicated" if world > 1 else "single GPU",
              "l2": "operands, codes and output of a step total > 126 MB (larger than L2); no flush needed"}

    if args.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(len(os.sched_getaffinity(0)))     # torchrun pins OMP_NUM_THREADS=1
        steps, warm = 1, 0
        if kind in ("moe", "moe_train"):
            cb = cpu_moe_sample(m, n, k)
        elif kind in ("nvfp4_mlp", "fp8_triple", "mxfp8_triple"):
            cb = cpu_composite_sample(kind, m, n, k)
        else:
            cb = run_cpu(kind, m, n, k, args.steps, args.warmup)      # --steps / --warmup honoured (time budget: see run_cpu)
            steps, warm = cb["steps"], cb["warmup"]
        print(json.dumps({"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "TFLOPS", "n_gpus": args.gpus,
                          "steps": steps, "warmup": warm, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "bf16 matmul of fake-quantized operands (CPU)",
                          "data": "synthetic", "config": config,
                          "cpu_baseline": {k2: cb[k2] for k2 in ("value", "unit", "cores", "kind", "sample")},
                          "e2e": {"value": cb["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path for the product arm")
    torch.cuda.set_device(local)
    if kind == "moe":
        return run_moe(args, m, n, k, rank, world, local)
    if kind == "moe_train":
        return run_moe_training(args, m, n, k, rank, world, local)
    if kind in ("nvfp4_mlp", "fp8_triple", "mxfp8_triple"):
        return run_composite(args, kind, m, n, k, rank, world, local)
    return run_dense(args, kind, m, n, k, rank, world, local, config)


if __name__ == "__main__":
    main()
