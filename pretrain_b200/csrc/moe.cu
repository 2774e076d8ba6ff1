// MoE data movement around the ragged grouped GEMM: router back end (score function, top-k,
// src/layers/mlp.py:292-301), permute plan (stable counting sort of the routed (token, slot) pairs
// by expert, in the reference's order, src/layers/mlp.py:446-457), gather into the padded
// expert-sorted layout (optionally fused with MXFP8 quantization), SwiGLU between the two GEMMs
// (src/layers/activation.py:80-81) and its backward, the weighted unpermute
// (src/layers/mlp.py:472-477) and its backward, and the expert-parallel dispatch / combine over
// peer-mapped memory.  Index work is integer and bit-exact; the row movers are HBM-bound: a thread
// owns a run of 32 elements (64 bytes in, two sectors) or a warp owns a row chunk, 16-byte or
// 32-byte accesses.
#include "common.cuh"

#include <atomic>

namespace b200q {
namespace {

constexpr int kPlanThreads = 1024;       // pairs per CTA in the plan kernels
constexpr int kMaxPeers = 8;             // ranks of one NVLink domain
constexpr int kMaxExperts = 256;

// ---- plan, step 1: per-CTA histogram of expert ids -------------------------------------------
__global__ void __launch_bounds__(kPlanThreads)
moe_hist_kernel(const int64_t* __restrict__ top_idx, int64_t n, int E, int32_t* __restrict__ block_counts) {
  pdl_prologue();
  __shared__ int hist[kMaxExperts];
  for (int i = threadIdx.x; i < E; i += kPlanThreads) hist[i] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * kPlanThreads + threadIdx.x;
  if (i < n) {
    const int e = (int)top_idx[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kPlanThreads) block_counts[(int64_t)blockIdx.x * E + e] = hist[e];
}

// ---- plan, step 2 (one CTA): scan over CTAs per expert, then the segment tables -----------------
// block_counts becomes the exclusive prefix over CTAs; offs = cumulative ends of the unpadded
// segments; padded_offs = starts of the 128-row-aligned segments; tile_expert / num_tiles.
__global__ void __launch_bounds__(kMaxExperts)
moe_scan_kernel(int32_t* __restrict__ block_counts, int nblocks, int E, int32_t* __restrict__ offs,
                int32_t* __restrict__ padded_offs, int32_t* __restrict__ tile_expert, int32_t* __restrict__ num_tiles,
                int max_tiles) {
  pdl_prologue();
  __shared__ int count[kMaxExperts];
  __shared__ int pstart[kMaxExperts + 1];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b0 = 0; b0 < nblocks; b0 += 16) {       // 16 independent loads in flight, then the prefix
      int c[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) c[i] = b0 + i < nblocks ? block_counts[(int64_t)(b0 + i) * E + e] : 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (b0 + i < nblocks) block_counts[(int64_t)(b0 + i) * E + e] = run;
        run += c[i];
      }
    }
    count[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int end = 0, p = 0;
    for (int i = 0; i < E; ++i) {
      end += count[i];
      offs[i] = end;
      pstart[i] = p;
      p += (count[i] + 127) & ~127;
    }
    pstart[E] = p;
    *num_tiles = p >> 7;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= E; i += blockDim.x) padded_offs[i] = pstart[i];
  if (e < E)
    for (int t = pstart[e] >> 7; t < (pstart[e + 1] >> 7); ++t) tile_expert[t] = e;
  for (int t = (pstart[E] >> 7) + threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
}

// ---- plan, step 3: stable destination of every pair ----------------------------------------------
// rank inside the CTA = pairs of the same expert in earlier warps + earlier lanes of this warp.
__global__ void __launch_bounds__(kPlanThreads)
moe_scatter_kernel(const int64_t* __restrict__ top_idx, int64_t n, int k, int E, const int32_t* __restrict__ block_excl,
                   const int32_t* __restrict__ padded_offs, int32_t* __restrict__ row_of, int32_t* __restrict__ src_of_row) {
  pdl_prologue();
  extern __shared__ int warp_counts[];      // [32 warps][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += kPlanThreads) warp_counts[i] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * kPlanThreads + threadIdx.x;
  int e = -1;
  if (i < n) {
    e = (int)top_idx[i];
    if (e < 0 || e >= E) e = -1;
  }
  const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
  const int rank_in_warp = __popc(same & ((1u << lane) - 1));
  if (e >= 0 && rank_in_warp == 0) warp_counts[warp * E + e] = __popc(same);
  __syncthreads();
  for (int x = threadIdx.x; x < E; x += kPlanThreads) {     // exclusive prefix over the 32 warps
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = warp_counts[w * E + x];
      warp_counts[w * E + x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (e >= 0) {
    const int dest = padded_offs[e] + block_excl[(int64_t)blockIdx.x * E + e] + warp_counts[warp * E + e] + rank_in_warp;
    row_of[i] = dest;
    src_of_row[dest] = (int32_t)(i / k);
  }
}

// ---- plan, steps 2 + 3 in one launch (up to kFusedPlanBlocks CTAs) ---------------------------------
// Every CTA re-derives what step 2 would hand it from the per-CTA histograms (a few thousand
// integers in L2): the experts' totals, hence the padded segment starts, and its own exclusive
// prefix over the CTAs before it; then it places its pairs like moe_scatter_kernel.  CTA 0 also
// writes the tables (offs, padded_offs, tile_expert, num_tiles) and marks the pad rows of every
// segment with -1, so no separate scan launch and no clearing of src_of_row are needed.
constexpr int kFusedPlanBlocks = 128;

__global__ void __launch_bounds__(kPlanThreads)
moe_scatter_tables_kernel(const int64_t* __restrict__ top_idx, int64_t n, int k, int E, const int32_t* __restrict__ block_counts,
                          int nblocks, int32_t* __restrict__ offs, int32_t* __restrict__ padded_offs,
                          int32_t* __restrict__ row_of, int32_t* __restrict__ src_of_row, int32_t* __restrict__ tile_expert,
                          int32_t* __restrict__ num_tiles, int max_tiles, int64_t padded_rows) {
  pdl_prologue();
  extern __shared__ int warp_counts[];      // [32 warps][E]
  __shared__ int total[kMaxExperts], excl[kMaxExperts], pstart[kMaxExperts + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += kPlanThreads) warp_counts[i] = 0;
  for (int i = threadIdx.x; i < E; i += kPlanThreads) total[i] = excl[i] = 0;
  __syncthreads();
  for (int idx = threadIdx.x; idx < nblocks * E; idx += kPlanThreads) {
    const int b = idx / E, e = idx - b * E;
    const int c = block_counts[idx];
    if (c) {
      atomicAdd(&total[e], c);
      if (b < (int)blockIdx.x) atomicAdd(&excl[e], c);
    }
  }
  const int64_t i = (int64_t)blockIdx.x * kPlanThreads + threadIdx.x;
  int e = -1;
  if (i < n) {
    e = (int)top_idx[i];
    if (e < 0 || e >= E) e = -1;
  }
  const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
  const int rank_in_warp = __popc(same & ((1u << lane) - 1));
  if (e >= 0 && rank_in_warp == 0) warp_counts[warp * E + e] = __popc(same);
  __syncthreads();
  if (warp == 0) {
    // padded segment starts: exclusive scan of the totals rounded up to 128, 32 experts at a time
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int x = e0 + lane < E ? (total[e0 + lane] + 127) & ~127 : 0;
      int inc = x;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += y;
      }
      if (e0 + lane < E) pstart[e0 + lane] = carry + inc - x;
      carry += __shfl_sync(0xFFFFFFFFu, inc, 31);
    }
    if (lane == 0) pstart[E] = carry;
  }
  for (int x = threadIdx.x; x < E; x += kPlanThreads) {     // exclusive prefix over the 32 warps
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = warp_counts[w * E + x];
      warp_counts[w * E + x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (e >= 0) {
    const int dest = pstart[e] + excl[e] + warp_counts[warp * E + e] + rank_in_warp;
    row_of[i] = dest;
    src_of_row[dest] = (int32_t)(i / k);
  }
  // rows past the last segment (the buffer is sized for the worst case): no source either
  for (int64_t r = pstart[E] + (int64_t)blockIdx.x * kPlanThreads + threadIdx.x; r < padded_rows; r += (int64_t)gridDim.x * kPlanThreads)
    src_of_row[r] = -1;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      int end = 0;
      for (int x = 0; x < E; ++x) { end += total[x]; offs[x] = end; }
      *num_tiles = pstart[E] >> 7;
    }
    for (int x = threadIdx.x; x <= E; x += kPlanThreads) padded_offs[x] = pstart[x];
    for (int t = threadIdx.x; t < max_tiles; t += kPlanThreads) {
      // expert of tile t: the segment that contains row 128 t (segments are whole tiles)
      int ex = -1;
      if (t < (pstart[E] >> 7)) {
        int lo = 0, hi = E - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (pstart[mid] <= (t << 7)) lo = mid; else hi = mid - 1;
        }
        ex = lo;   // the last expert that starts at or before the row: empty ones before it share its start
      }
      tile_expert[t] = ex;
    }
    // pad rows at the end of every segment
    for (int x = warp; x < E; x += 32)
      for (int r = pstart[x] + total[x] + lane; r < pstart[x + 1]; r += 32) src_of_row[r] = -1;
  }
}

// ---- plan for rows that are already expert-sorted (grouped_mlp's input convention) ----------------
__global__ void __launch_bounds__(kMaxExperts)
moe_pad_plan_kernel(const int32_t* __restrict__ offs, int E, int32_t* __restrict__ padded_offs,
                    int32_t* __restrict__ tile_expert, int32_t* __restrict__ num_tiles, int max_tiles) {
  pdl_prologue();
  __shared__ int pstart[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int prev = 0, p = 0;
    for (int i = 0; i < E; ++i) {
      const int c = offs[i] - prev;
      prev = offs[i];
      pstart[i] = p;
      p += ((c > 0 ? c : 0) + 127) & ~127;
    }
    pstart[E] = p;
    *num_tiles = p >> 7;
  }
  __syncthreads();
  const int e = threadIdx.x;
  for (int i = threadIdx.x; i <= E; i += blockDim.x) padded_offs[i] = pstart[i];
  if (e < E)
    for (int t = pstart[e] >> 7; t < (pstart[e + 1] >> 7); ++t) tile_expert[t] = e;
  for (int t = (pstart[E] >> 7) + threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
}

// src_of_row[r] = sorted-input row of padded row r, or -1 for pad rows
__global__ void moe_pad_src_kernel(const int32_t* __restrict__ offs, const int32_t* __restrict__ padded_offs,
                                   const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ num_tiles,
                                   int32_t* __restrict__ src_of_row, int64_t padded_rows) {
  pdl_prologue();
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= padded_rows) return;
  int src = -1;
  if ((r >> 7) < *num_tiles) {
    const int e = tile_expert[r >> 7];
    const int start = e > 0 ? offs[e - 1] : 0, cnt = offs[e] - start;
    const int within = (int)(r - padded_offs[e]);
    if (within < cnt) src = start + within;
  }
  src_of_row[r] = src;
}

// ---- gather rows into the padded layout (+ MXFP8) ------------------------------------------------
// Work item = 32 consecutive elements of one padded row (one MX block), owned by one thread and
// dealt round-robin over the grid's threads: 64 bytes in (two sectors), 32 code bytes + one scale
// byte (or the 64 bytes themselves) out.  Pad rows (source -1) become zero rows.
template <int QUANT, bool WIDE, int FMT>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const uint16_t* __restrict__ x, int64_t D, int64_t ld, const int32_t* __restrict__ src_of_row,
                  const int32_t* __restrict__ num_tiles, int64_t padded_rows, uint8_t* __restrict__ out,
                  uint8_t* __restrict__ sf) {
  pdl_prologue();
  int64_t live_rows = (int64_t)(*num_tiles) << 7;
  if (live_rows > padded_rows) live_rows = padded_rows;
  const int runs = (int)(D >> 5);
  const int64_t kt = ((D >> 5) + 3) >> 2;
  for (ItemWalker w((int64_t)blockIdx.x * 256 + threadIdx.x, (int64_t)gridDim.x * 256, runs); w.row < live_rows; w.next()) {
    const int64_t r = w.row;
    const int c = w.chunk << 5;
    const int src = src_of_row[r];
    uint4 v[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (src >= 0) {
      const uint16_t* xp = x + (int64_t)src * ld + c;
      ld_nc_32B<WIDE>(xp, v[0], v[1]);
      ld_nc_32B<WIDE>(xp + 16, v[2], v[3]);
    }
    if (QUANT) {
      uint32_t o[8];
      const int e = mx_quant_block32<FMT>(v, o);
      st_32B<WIDE>(out + r * D + c, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
      sf[sf_swizzled(r, w.chunk, kt)] = (uint8_t)(e + 127);
    } else {
      uint8_t* op = out + (r * D + c) * 2;
      st_32B<WIDE>(op, v[0], v[1]);
      st_32B<WIDE>(op + 32, v[2], v[3]);
    }
  }
}

// ---- SwiGLU (+ MXFP8) between the two grouped GEMMs -------------------------------------------------
// Input rows are [gate (I) | up (I)]; work item = 32 consecutive outputs of one row, one thread.
template <int QUANT, bool WIDE, int FMT>
__global__ void __launch_bounds__(256)
swiglu_kernel(const uint16_t* __restrict__ g, int64_t rows, int64_t I, int64_t ld, uint8_t* __restrict__ out,
              uint8_t* __restrict__ sf) {
  pdl_prologue();
  const int runs = (int)(I >> 5);
  const int64_t kt = ((I >> 5) + 3) >> 2;
  for (ItemWalker w((int64_t)blockIdx.x * 256 + threadIdx.x, (int64_t)gridDim.x * 256, runs); w.row < rows; w.next()) {
    const int64_t r = w.row;
    const int c = w.chunk << 5;
    const uint16_t* gp = g + r * ld + c;
    uint4 vg[4], vu[4], h[4];
    ld_nc_32B<WIDE>(gp, vg[0], vg[1]);
    ld_nc_32B<WIDE>(gp + 16, vg[2], vg[3]);
    ld_nc_32B<WIDE>(gp + I, vu[0], vu[1]);
    ld_nc_32B<WIDE>(gp + I + 16, vu[2], vu[3]);
#pragma unroll
    for (int u = 0; u < 4; ++u) h[u] = swiglu8(vg[u], vu[u]);
    if (QUANT) {
      uint32_t o[8];
      const int e = mx_quant_block32<FMT>(h, o);
      st_32B<WIDE>(out + r * I + c, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
      sf[sf_swizzled(r, w.chunk, kt)] = (uint8_t)(e + 127);
    } else {
      uint8_t* op = out + (r * I + c) * 2;
      st_32B<WIDE>(op, h[0], h[1]);
      st_32B<WIDE>(op + 32, h[2], h[3]);
    }
  }
}

// ---- router back end: score function, top-k, normalised weights, casts, expert histogram ---------
// One warp per token over the fp32 logits of the gate GEMM (src/layers/mlp.py:292-301, :455):
// probs = softmax | sigmoid (fp32), the k largest probs in descending order (equal probs: the
// larger logit first, then the lower expert index), weights = probs[idx] / (sum + 1e-9) when
// normalising, both cast to bf16 (or left in fp32 when the caller's activations are not bf16), plus how
// many tokens chose each expert.  Lane l holds experts
// l, l + 32, ... (E <= 256).
// PER = experts per lane (1, 2, 4 or 8: the smallest that covers E), a template argument so that the
// loops over a lane's experts have no idle iterations.
// BIAS: the k experts are chosen by prob + select_bias[e] (load-balancing bias, selection only); the
// weights are still the probs of the chosen experts.
template <int PER, bool BIAS>
__global__ void __launch_bounds__(256)
moe_router_topk_kernel(const float* __restrict__ logits, int64_t T, int E, int k, int sigmoid, int normalize,
                       int64_t* __restrict__ top_idx, void* __restrict__ top_w, void* __restrict__ probs_out,
                       int32_t* __restrict__ counts, const float* __restrict__ select_bias, int out_fp32) {
  pdl_prologue();
  __shared__ int hist[kMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < E; i += 256) hist[i] = 0;
  __syncthreads();
  constexpr int kRouterMaxPerLane = PER;
  const int per = PER;
  for (int64_t t = (int64_t)blockIdx.x * 8 + warp; t < T; t += (int64_t)gridDim.x * 8) {
    float v[kRouterMaxPerLane], p[kRouterMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      v[j] = (j < per && e < E) ? logits[t * E + e] : -INFINITY;
      m = fmaxf(m, v[j]);
    }
    if (sigmoid) {
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) p[j] = v[j] == -INFINITY ? -1.f : 1.f / (1.f + expf(-v[j]));
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) {
        p[j] = v[j] == -INFINITY ? 0.f : expf(v[j] - m);
        sum += p[j];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) p[j] = v[j] == -INFINITY ? -1.f : p[j] / sum;
    }
    if (probs_out != nullptr) {
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) {
        const int e = j * 32 + lane;
        if (j < per && e < E) {
          if (out_fp32) static_cast<float*>(probs_out)[t * E + e] = p[j];
          else static_cast<uint16_t*>(probs_out)[t * E + e] = __bfloat16_as_ushort(__float2bfloat16_rn(p[j]));
        }
      }
    }
    // selection key: the prob, or prob + bias; absent experts stay below every key
    float key[BIAS ? kRouterMaxPerLane : 1];
    if (BIAS) {
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) {
        const int e = j * 32 + lane;
        key[j] = (j < per && e < E) ? p[j] + select_bias[e] : -INFINITY;
      }
    }
    // k rounds of warp arg-max; a taken entry drops below every key (-2 under the probs and the -1 of absent
    // experts; -infinity under biased keys)
    float wsum = 0.f, mine = 0.f;   // lane j keeps the j-th weight
    int mine_idx = 0;
    for (int r = 0; r < k; ++r) {
      float bp = BIAS ? -INFINITY : -3.f, bv = -INFINITY;
      int be = 0x7FFFFFFF;
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) {
        const int e = j * 32 + lane;
        const float kj = BIAS ? key[j] : p[j];
        if (kj > bp || (kj == bp && (v[j] > bv || (v[j] == bv && e < be)))) { bp = kj; bv = v[j]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float op = __shfl_xor_sync(0xFFFFFFFFu, bp, o), ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
        const int oe = __shfl_xor_sync(0xFFFFFFFFu, be, o);
        if (op > bp || (op == bp && (ov > bv || (ov == bv && oe < be)))) { bp = op; bv = ov; be = oe; }
      }
      float wp = bp;                                   // the weight: the chosen expert's prob
      if (BIAS) {
        float own = 0.f;
#pragma unroll
        for (int j = 0; j < kRouterMaxPerLane; ++j)
          if (j == (be >> 5)) own = p[j];
        wp = __shfl_sync(0xFFFFFFFFu, own, be & 31);
      }
      if ((be & 31) == lane) {                         // selects over the PER registers, no local memory
#pragma unroll
        for (int j = 0; j < kRouterMaxPerLane; ++j)
          if (j == (be >> 5)) {
            if (BIAS) key[j] = -INFINITY; else p[j] = -2.f;
          }
      }
      wsum += wp;
      if (lane == r) { mine = wp; mine_idx = be; }
    }
    if (lane < k) {
      const float w = normalize ? mine / (wsum + 1e-9f) : mine;
      top_idx[t * k + lane] = mine_idx;
      if (out_fp32) static_cast<float*>(top_w)[t * k + lane] = w;
      else static_cast<uint16_t*>(top_w)[t * k + lane] = __bfloat16_as_ushort(__float2bfloat16_rn(w));
      if (counts != nullptr) atomicAdd(&hist[mine_idx], 1);
    }
  }
  __syncthreads();
  if (counts != nullptr)
    for (int i = threadIdx.x; i < E; i += 256)
      if (hist[i]) atomicAdd(&counts[i], hist[i]);
}

// ---- inverse of row_of: the pair that owns every padded row (the array is preset to -1) -------------
__global__ void moe_pair_of_row_kernel(const int32_t* __restrict__ row_of, int64_t n_pairs, int64_t padded_rows,
                                       int32_t* __restrict__ pair_of_row) {
  pdl_prologue();
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  const int r = row_of[p];
  if (r >= 0 && r < padded_rows) pair_of_row[r] = (int32_t)p;
}

// ---- weighted unpermute: out[t] = sum_j w[t,j] * y[row_of[t*k+j]] (fp32 accumulate) ----------------
__global__ void __launch_bounds__(256)
moe_unpermute_kernel(const uint16_t* __restrict__ y, int64_t ldy, const uint16_t* __restrict__ w,
                     const int32_t* __restrict__ row_of, int64_t T, int k, int64_t D, uint16_t* __restrict__ out) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (ItemWalker it((int64_t)blockIdx.x * 8 + warp, (int64_t)gridDim.x * 8, (int)((D + 255) >> 8)); it.row < T; it.next()) {
    const int64_t t = it.row, c = (int64_t)it.chunk * 256 + lane * 8;
    if (c >= D) continue;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int row = row_of[t * k + j];
      const float wj = w != nullptr ? u2f((uint32_t)w[t * k + j] << 16) : 1.f;
      float f[8];
      unpack8(ld_nc_v4(y + (int64_t)row * ldy + c), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(wj, f[i], acc[i]);
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      o[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + t * D + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- expert-parallel dispatch / combine over peer-mapped memory -----------------------------------
// Dispatch: the sender's gather + MXFP8 kernel writes every routed row straight into the padded
// expert-sorted buffer of the rank that owns its expert (plain stores to peer-mapped memory over
// NVLink; nothing is loaded from a peer here).  The sender walks its OWN padded layout (row r ->
// token src_of_row[r], expert tile_expert[r / 128]); row_base[e] is where this rank's rows of
// global expert e start in the owner's buffer, so the destination row keeps the sender's stable
// order inside the expert.
struct PeerBufs {
  uint8_t* codes[kMaxPeers];
  uint8_t* sf[kMaxPeers];
};

__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const uint16_t* __restrict__ x, int64_t D, int64_t ld, const int32_t* __restrict__ src_of_row,
                    const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ padded_offs,
                    const int32_t* __restrict__ num_tiles, int64_t padded_rows, const int32_t* __restrict__ row_base,
                    int experts_per_rank, const PeerBufs peers) {
  pdl_prologue();
  int64_t live_rows = (int64_t)(*num_tiles) << 7;
  if (live_rows > padded_rows) live_rows = padded_rows;
  const int runs = (int)(D >> 5);
  const int64_t kt = ((D >> 5) + 3) >> 2;
  for (ItemWalker w((int64_t)blockIdx.x * 256 + threadIdx.x, (int64_t)gridDim.x * 256, runs); w.row < live_rows; w.next()) {
    const int64_t r = w.row;
    const int src = src_of_row[r];
    if (src < 0) continue;                               // the sender's own pad rows are not sent
    const int e = tile_expert[r >> 7];
    const int dst = e / experts_per_rank;
    const int64_t drow = (int64_t)row_base[e] + (r - padded_offs[e]);
    const int c = w.chunk << 5;
    uint4 v[4];
    const uint16_t* xp = x + (int64_t)src * ld + c;
    ld_nc_32B<false>(xp, v[0], v[1]);
    ld_nc_32B<false>(xp + 16, v[2], v[3]);
    uint32_t o[8];
    const int ex = mx_quant_block32<FMT_E4M3>(v, o);
    st_32B<false>(peers.codes[dst] + drow * D + c, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
    peers.sf[dst][sf_swizzled(drow, w.chunk, kt)] = (uint8_t)(ex + 127);
  }
}

// The receiver clears the pad rows of its own buffer (rows no sender writes): zero codes, scale 2^0.
__global__ void __launch_bounds__(256)
moe_zero_pad_rows_kernel(const int32_t* __restrict__ src_of_row, const int32_t* __restrict__ num_tiles, int64_t padded_rows,
                         int64_t D, uint8_t* __restrict__ codes, uint8_t* __restrict__ sf) {
  pdl_prologue();
  int64_t live_rows = (int64_t)(*num_tiles) << 7;
  if (live_rows > padded_rows) live_rows = padded_rows;
  const int runs = (int)(D >> 5);
  const int64_t kt = ((D >> 5) + 3) >> 2;
  for (ItemWalker w((int64_t)blockIdx.x * 256 + threadIdx.x, (int64_t)gridDim.x * 256, runs); w.row < live_rows; w.next()) {
    if (src_of_row[w.row] >= 0) continue;
    st_32B<false>(codes + w.row * D + (w.chunk << 5), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0));
    sf[sf_swizzled(w.row, w.chunk, kt)] = 127;
  }
}

// Combine: out[t] = sum_j w[t,j] * y_{peer[t,j]}[row[t,j]] with the expert outputs read in place from
// the owners' buffers (plain loads from peer-mapped memory), fp32 accumulation in slot order, one
// rounding - the arithmetic of moe_unpermute_kernel.
struct PeerRows {
  const uint16_t* y[kMaxPeers];
};

__global__ void __launch_bounds__(256)
moe_combine_kernel(const PeerRows peers, int64_t ldy, const uint16_t* __restrict__ w, const int32_t* __restrict__ pair_peer,
                   const int32_t* __restrict__ pair_row, int64_t T, int k, int64_t D, uint16_t* __restrict__ out) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (ItemWalker it((int64_t)blockIdx.x * 8 + warp, (int64_t)gridDim.x * 8, (int)((D + 255) >> 8)); it.row < T; it.next()) {
    const int64_t t = it.row, c = (int64_t)it.chunk * 256 + lane * 8;
    if (c >= D) continue;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const uint16_t* base = peers.y[pair_peer[t * k + j]];
      const float wj = u2f((uint32_t)w[t * k + j] << 16);
      float f[8];
      const uint4 v = *reinterpret_cast<const uint4*>(base + (int64_t)pair_row[t * k + j] * ldy + c);
      unpack8(v, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(wj, f[i], acc[i]);
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      o[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + t * D + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- expert parallelism: index tables, flag barrier, bf16 row scatter, pair dot products ------------------------
// Index tables of one rank, from the gathered per-sender counts: where this rank's rows for every (global) expert
// start inside the owner's padded expert-sorted buffer, the segment ends of the experts it owns, and for every routed
// pair the owner and the row there.  all_offs[r][e] = cumulative count of sender r's pairs up to and including
// expert e (its permute plan's `offs`).  Layout of an owner's buffer: its experts' segments in order, each padded to
// 128 rows, senders in rank order inside a segment, a sender's rows in its own stable order.
// Every CTA rebuilds the small per-expert tables in shared memory (E <= 256, world <= 8); CTA 0 writes them out.
__global__ void __launch_bounds__(256)
moe_ep_index_kernel(const int32_t* __restrict__ all_offs, int world, int rank, int E, int e_local,
                    const int64_t* __restrict__ top_idx, const int32_t* __restrict__ row_of, const int32_t* __restrict__ padded_offs,
                    int64_t n_pairs, int32_t* __restrict__ row_base, int32_t* __restrict__ own_offs,
                    int32_t* __restrict__ pair_peer, int32_t* __restrict__ pair_row) {
  pdl_prologue();
  __shared__ int s_total[kMaxExperts], s_before[kMaxExperts], s_base[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += 256) {
    int tot = 0, before = 0;
    for (int r = 0; r < world; ++r) {
      const int c = all_offs[r * E + e] - (e > 0 ? all_offs[r * E + e - 1] : 0);
      tot += c;
      if (r < rank) before += c;
    }
    s_total[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += 256) {
    int start = 0;
    for (int j = (e / e_local) * e_local; j < e; ++j) start += (s_total[j] + 127) & ~127;
    s_base[e] = start + s_before[e];
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < E; e += 256) row_base[e] = s_base[e];
    for (int j = threadIdx.x; j < e_local; j += 256) {
      int acc = 0;
      for (int i = 0; i <= j; ++i) acc += s_total[rank * e_local + i];
      own_offs[j] = acc;
    }
  }
  for (int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x; p < n_pairs; p += (int64_t)gridDim.x * 256) {
    const int e = (int)top_idx[p];
    pair_peer[p] = e / e_local;
    pair_row[p] = s_base[e] + row_of[p] - padded_offs[e];
  }
}

// Rendezvous of the ranks of one NVLink domain without a collective: every rank writes the epoch into its slot of every
// rank's flag array (peer-mapped memory, release at system scope) and then waits until every slot of its own array has
// reached the epoch (acquire at system scope).  Stream-ordered: the stores of the kernels before it have been performed
// when it starts, the kernels after it start once every rank has arrived.  The wait is bounded (about a second); a rank
// that gives up records status 31 and returns, it never spins forever.
struct PeerFlags {
  int32_t* f[kMaxPeers];
};
constexpr uint32_t kBarrierPolls = 4000000u;

__global__ void peer_barrier_kernel(const PeerFlags flags, int world, int rank, int epoch) {
  pdl_prologue();
  const int lane = threadIdx.x;
  __threadfence_system();
  if (lane < world) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.f[lane] + rank), "r"(epoch) : "memory");
    bool ok = false;
    for (uint32_t i = 0; i < kBarrierPolls && !ok; ++i) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags.f[rank] + lane) : "memory");
      ok = v - epoch >= 0;
      if (!ok && i > 2048u) __nanosleep(200);
    }
    if (!ok) atomicExch(&g_device_status, 31);
  }
  __syncwarp();
  __threadfence_system();
}

// Rows of x (optionally scaled by the pair's routing weight, fp32 multiply, one rounding) stored as bf16 into the
// buffers of the ranks that own the pairs' experts: the transpose of moe_combine_kernel.  Stores only cross NVLink.
struct PeerRowsW {
  uint16_t* y[kMaxPeers];
};

__global__ void __launch_bounds__(256)
moe_scatter_rows_peers_kernel(const uint16_t* __restrict__ x, int64_t ld, const uint16_t* __restrict__ w,
                              const int32_t* __restrict__ pair_peer, const int32_t* __restrict__ pair_row, int64_t n_pairs, int k,
                              int64_t D, const PeerRowsW peers, int64_t ldy) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (ItemWalker it((int64_t)blockIdx.x * 8 + warp, (int64_t)gridDim.x * 8, (int)((D + 255) >> 8)); it.row < n_pairs; it.next()) {
    const int64_t p = it.row, c = (int64_t)it.chunk * 256 + lane * 8;
    if (c >= D) continue;
    uint4 v = ld_nc_v4(x + (p / k) * ld + c);
    if (w != nullptr) {
      const float wj = u2f((uint32_t)w[p] << 16);
      float f[8];
      unpack8(v, f);
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 pk = __floats2bfloat162_rn(wj * f[2 * i], wj * f[2 * i + 1]);
        o[i] = *reinterpret_cast<uint32_t*>(&pk);
      }
      v = make_uint4(o[0], o[1], o[2], o[3]);
    }
    *reinterpret_cast<uint4*>(peers.y[pair_peer[p]] + (int64_t)pair_row[p] * ldy + c) = v;
  }
}

// The receiver clears the rows of its bf16 buffer that no sender writes (the pad rows of every live segment).
__global__ void __launch_bounds__(256)
moe_zero_pad_rows_bf16_kernel(const int32_t* __restrict__ src_of_row, const int32_t* __restrict__ num_tiles, int64_t padded_rows,
                              int64_t D, uint16_t* __restrict__ buf, int64_t ld) {
  pdl_prologue();
  int64_t live_rows = (int64_t)(*num_tiles) << 7;
  if (live_rows > padded_rows) live_rows = padded_rows;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t r = (int64_t)blockIdx.x * 8 + warp; r < live_rows; r += (int64_t)gridDim.x * 8) {
    if (src_of_row[r] >= 0) continue;
    for (int64_t c = lane * 8; c < D; c += 256) *reinterpret_cast<uint4*>(buf + r * ld + c) = make_uint4(0, 0, 0, 0);
  }
}

// dw[p] = <dout[token of p], y_owner[row of p]> in fp32, the expert outputs read in place from their owners.
__global__ void __launch_bounds__(256)
moe_pair_dots_peers_kernel(const uint16_t* __restrict__ dout, int64_t ld, const PeerRows peers, int64_t ldy,
                           const int32_t* __restrict__ pair_peer, const int32_t* __restrict__ pair_row, int64_t n_pairs, int k,
                           int64_t D, float* __restrict__ dw) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t p = (int64_t)blockIdx.x * 8 + warp; p < n_pairs; p += (int64_t)gridDim.x * 8) {
    const uint16_t* yr = peers.y[pair_peer[p]] + (int64_t)pair_row[p] * ldy;
    const uint16_t* dr = dout + (p / k) * ld;
    float dot = 0.f;
    for (int64_t c = lane * 8; c < D; c += 256) {
      float a[8], b[8];
      unpack8(ld_nc_v4(dr + c), a);
      unpack8(*reinterpret_cast<const uint4*>(yr + c), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot = fmaf(a[i], b[i], dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
    if (lane == 0) dw[p] = dot;
  }
}

// ---- backward of SwiGLU: dg = [dh * up * silu'(gate) | dh * silu(gate)] -------------------------
// silu'(x) = s (1 + x (1 - s)), s = 1 / (1 + e^-x); fp32 arithmetic on the bf16 inputs, one rounding.
__global__ void __launch_bounds__(256)
swiglu_backward_kernel(const uint16_t* __restrict__ g, int64_t rows, int64_t I, int64_t ldg, const uint16_t* __restrict__ dh,
                       int64_t lddh, uint16_t* __restrict__ dg, int64_t lddg) {
  pdl_prologue();
  const int runs = (int)(I >> 3);
  for (ItemWalker w((int64_t)blockIdx.x * 256 + threadIdx.x, (int64_t)gridDim.x * 256, runs); w.row < rows; w.next()) {
    const int64_t r = w.row;
    const int c = w.chunk << 3;
    uint4 og4, ou4;
    swiglu_bwd8(ld_nc_v4(g + r * ldg + c), ld_nc_v4(g + r * ldg + I + c), ld_nc_v4(dh + r * lddh + c), og4, ou4);
    *reinterpret_cast<uint4*>(dg + r * lddg + c) = og4;
    *reinterpret_cast<uint4*>(dg + r * lddg + I + c) = ou4;
  }
}

// ---- backward of the weighted unpermute ------------------------------------------------------------
// out[t] = sum_j w[t,j] y[row_of[t,j]]  =>  dy[row_of[t,j]] = w[t,j] dout[t],  dw[t,j] = <dout[t], y[row_of[t,j]]>.
// One warp per routed pair; a second range of warp items zeroes the rows of dy that no pair owns
// (the pad rows of every segment and everything past the last one).
__global__ void __launch_bounds__(256)
moe_unpermute_backward_kernel(const uint16_t* __restrict__ dout, const uint16_t* __restrict__ w, const uint16_t* __restrict__ y,
                              int64_t ldy, const int32_t* __restrict__ row_of, const int32_t* __restrict__ src_of_row,
                              int64_t n_pairs, int k, int64_t D, int64_t padded_rows, uint16_t* __restrict__ dy,
                              float* __restrict__ dw) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t total = n_pairs + padded_rows;
  for (int64_t it = (int64_t)blockIdx.x * 8 + warp; it < total; it += (int64_t)gridDim.x * 8) {
    if (it < n_pairs) {
      const int64_t t = it / k;
      const int row = row_of[it];
      const float wj = u2f((uint32_t)w[it] << 16);
      float dot = 0.f;
      for (int64_t c = lane * 8; c < D; c += 256) {
        float f[8];
        unpack8(ld_nc_v4(dout + t * D + c), f);
        if (y != nullptr) {
          float yy[8];
          unpack8(ld_nc_v4(y + (int64_t)row * ldy + c), yy);
#pragma unroll
          for (int i = 0; i < 8; ++i) dot = fmaf(f[i], yy[i], dot);
        }
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 pk = __floats2bfloat162_rn(wj * f[2 * i], wj * f[2 * i + 1]);
          o[i] = *reinterpret_cast<uint32_t*>(&pk);
        }
        if (dy != nullptr) *reinterpret_cast<uint4*>(dy + (int64_t)row * D + c) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      if (dw != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
        if (lane == 0) dw[it] = dot;
      }
    } else {
      const int64_t r = it - n_pairs;
      if (dy != nullptr && src_of_row[r] < 0)
        for (int64_t c = lane * 8; c < D; c += 256) *reinterpret_cast<uint4*>(dy + r * D + c) = make_uint4(0, 0, 0, 0);
    }
  }
}

// Scratch of b200q_moe_permute_plan_static: the per-CTA expert histograms of the plan kernels
// ([CTAs][E] int32).  It lives in the library image, so every GPU that loads the library holds
// these 1 MiB until the process exits.
constexpr int64_t kStaticPlanInts = 262144;
static __device__ __align__(256) int32_t g_static_plan_scratch[kStaticPlanInts];
constexpr int kMaxDevices = 64;
// device address of the array, per device; filled on first use (every thread that gets there stores the same value)
static std::atomic<int32_t*> g_static_plan_ptr[kMaxDevices] = {};

// The permute plan's launches, shared by the two entry points (workspace from the caller or built in).
int run_permute_plan(const int64_t* top_idx, int64_t n_pairs, int k, int E, int32_t* block_counts, int32_t* offs,
                     int32_t* padded_offs, int32_t* row_of, int32_t* src_of_row, int32_t* tile_expert, int32_t* num_tiles,
                     cudaStream_t st) {
  const int nblocks = (int)((n_pairs + kPlanThreads - 1) / kPlanThreads);
  const int64_t padded_rows = b200q_moe_padded_rows(n_pairs, E);
  launch_pdl(moe_hist_kernel, dim3(nblocks), dim3(kPlanThreads), (size_t)(0), st, top_idx, n_pairs, E, block_counts);
  B200Q_CUDA(cudaGetLastError());
  if (nblocks <= kFusedPlanBlocks) {
    launch_pdl(moe_scatter_tables_kernel, dim3(nblocks), dim3(kPlanThreads), (size_t)(32 * E * sizeof(int)), st, 
        top_idx, n_pairs, k, E, block_counts, nblocks, offs, padded_offs, row_of, src_of_row, tile_expert, num_tiles,
        (int)(padded_rows / 128), padded_rows);
    B200Q_CUDA(cudaGetLastError());
    return B200Q_OK;
  }
  B200Q_CUDA(memset_async(src_of_row, 0xFF, (size_t)padded_rows * sizeof(int32_t), st));   // -1 = pad row
  launch_pdl(moe_scan_kernel, dim3(1), dim3(kMaxExperts), (size_t)(0), st, block_counts, nblocks, E, offs, padded_offs, tile_expert, num_tiles,
                                             (int)(padded_rows / 128));
  B200Q_CUDA(cudaGetLastError());
  launch_pdl(moe_scatter_kernel, dim3(nblocks), dim3(kPlanThreads), (size_t)(32 * E * sizeof(int)), st, top_idx, n_pairs, k, E, block_counts, padded_offs,
                                                                           row_of, src_of_row);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// grid for kernels whose work items belong to single threads (256 per CTA), capped at one wave
inline int thread_item_grid(int64_t items) {
  int64_t want = (items + 255) / 256, cap = (int64_t)kNumSMs * 5;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

inline int row_grid(int64_t items) {
  int64_t want = (items + 7) / 8, cap = (int64_t)kNumSMs * 8;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

int64_t b200q_moe_padded_rows(int64_t n_pairs, int E) {
  if (n_pairs < 0 || E <= 0) return 0;
  // every expert wastes at most 127 rows; round the bound itself up to a tile
  return ((n_pairs + (int64_t)E * 127 + 127) / 128) * 128;
}

int64_t b200q_moe_plan_workspace_bytes(int64_t n_pairs, int E) {
  if (n_pairs < 0 || E <= 0) return 0;
  const int64_t nblocks = (n_pairs + kPlanThreads - 1) / kPlanThreads;
  return (nblocks > 0 ? nblocks : 1) * E * (int64_t)sizeof(int32_t);
}

int b200q_moe_permute_plan(const int64_t* top_idx, int64_t n_pairs, int k, int E, int32_t* offs, int32_t* padded_offs,
                           int32_t* row_of, int32_t* src_of_row, int32_t* tile_expert, int32_t* num_tiles, void* workspace,
                           void* stream) {
  PdlChain pdl_chain;
  if (top_idx == nullptr || offs == nullptr || padded_offs == nullptr || row_of == nullptr || src_of_row == nullptr ||
      tile_expert == nullptr || num_tiles == nullptr || workspace == nullptr || n_pairs <= 0 || k <= 0 || E <= 0)
    return B200Q_ERR_INVALID_ARG;
  if (E > kMaxExperts || n_pairs > INT32_MAX / 2) return B200Q_ERR_SHAPE;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  return run_permute_plan(top_idx, n_pairs, k, E, (int32_t*)workspace, offs, padded_offs, row_of, src_of_row, tile_expert,
                          num_tiles, st);
}

int b200q_moe_pad_plan(const int32_t* offs, int E, int64_t n_rows, int32_t* padded_offs, int32_t* src_of_row,
                       int32_t* tile_expert, int32_t* num_tiles, void* stream) {
  PdlChain pdl_chain;
  if (offs == nullptr || padded_offs == nullptr || src_of_row == nullptr || tile_expert == nullptr || num_tiles == nullptr ||
      E <= 0 || n_rows < 0)
    return B200Q_ERR_INVALID_ARG;
  if (E > kMaxExperts || n_rows > INT32_MAX / 2) return B200Q_ERR_SHAPE;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t padded_rows = b200q_moe_padded_rows(n_rows, E);
  launch_pdl(moe_pad_plan_kernel, dim3(1), dim3(kMaxExperts), (size_t)(0), st, offs, E, padded_offs, tile_expert, num_tiles, (int)(padded_rows / 128));
  B200Q_CUDA(cudaGetLastError());
  launch_pdl(moe_pad_src_kernel, dim3((unsigned)((padded_rows + 255) / 256)), dim3(256), (size_t)(0), st, offs, padded_offs, tile_expert, num_tiles, src_of_row,
                                                                            padded_rows);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_gather(const void* x, int64_t D, int64_t ld, const int32_t* src_of_row, const int32_t* num_tiles,
                     int64_t padded_rows, int quantize, int fmt, void* out, void* sf, void* stream) {
  PdlChain pdl_chain;
  if (x == nullptr || src_of_row == nullptr || num_tiles == nullptr || out == nullptr || D <= 0 || ld < D || padded_rows <= 0 ||
      (quantize && sf == nullptr) || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2))
    return B200Q_ERR_INVALID_ARG;
  if ((D & 31) || (ld & 7) || (padded_rows & 127)) return B200Q_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(out)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (quantize && ((D >> 5) & 3))
    B200Q_CUDA(memset_async(sf, 0, (size_t)b200q_sf_bytes(padded_rows, D >> 5, B200Q_SF_SWIZZLE_128x4), st));
  const bool wide = aligned32(x) && aligned32(out) && (ld & 15) == 0;
  const int grid = thread_item_grid(padded_rows * (D >> 5));
#define B200Q_GO(Q, W, F)                                                                                              \
  launch_pdl(moe_gather_kernel<Q, W, F>, dim3(grid), dim3(256), (size_t)(0), st, (const uint16_t*)x, D, ld, src_of_row, num_tiles, padded_rows, (uint8_t*)out, \
                                                   (uint8_t*)sf)
  if (!quantize) { if (wide) B200Q_GO(0, true, FMT_E4M3); else B200Q_GO(0, false, FMT_E4M3); }
  else if (fmt == B200Q_E4M3) { if (wide) B200Q_GO(1, true, FMT_E4M3); else B200Q_GO(1, false, FMT_E4M3); }
  else { if (wide) B200Q_GO(1, true, FMT_E5M2); else B200Q_GO(1, false, FMT_E5M2); }
#undef B200Q_GO
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_swiglu(const void* g, int64_t rows, int64_t I, int64_t ld, int quantize, int fmt, void* out, void* sf, void* stream) {
  PdlChain pdl_chain;
  if (g == nullptr || out == nullptr || rows <= 0 || I <= 0 || ld < 2 * I || (quantize && sf == nullptr) ||
      (fmt != B200Q_E4M3 && fmt != B200Q_E5M2))
    return B200Q_ERR_INVALID_ARG;
  if ((I & 31) || (ld & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(g) || !aligned16(out)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (quantize && ((rows & 127) || ((I >> 5) & 3)))
    B200Q_CUDA(memset_async(sf, 0, (size_t)b200q_sf_bytes(rows, I >> 5, B200Q_SF_SWIZZLE_128x4), st));
  const bool wide = aligned32(g) && aligned32(out) && (ld & 15) == 0;
  const int grid = thread_item_grid(rows * (I >> 5));
#define B200Q_GO(Q, W, F) launch_pdl(swiglu_kernel<Q, W, F>, dim3(grid), dim3(256), (size_t)(0), st, (const uint16_t*)g, rows, I, ld, (uint8_t*)out, (uint8_t*)sf)
  if (!quantize) { if (wide) B200Q_GO(0, true, FMT_E4M3); else B200Q_GO(0, false, FMT_E4M3); }
  else if (fmt == B200Q_E4M3) { if (wide) B200Q_GO(1, true, FMT_E4M3); else B200Q_GO(1, false, FMT_E4M3); }
  else { if (wide) B200Q_GO(1, true, FMT_E5M2); else B200Q_GO(1, false, FMT_E5M2); }
#undef B200Q_GO
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_dispatch_peers(const void* x, int64_t D, int64_t ld, const int32_t* src_of_row, const int32_t* tile_expert,
                             const int32_t* padded_offs, const int32_t* num_tiles, int64_t padded_rows, const int32_t* row_base,
                             int experts_per_rank, int world, void* const* peer_codes, void* const* peer_sf, void* stream) {
  PdlChain pdl_chain;
  if (x == nullptr || src_of_row == nullptr || tile_expert == nullptr || padded_offs == nullptr || num_tiles == nullptr ||
      row_base == nullptr || peer_codes == nullptr || peer_sf == nullptr || D <= 0 || ld < D || padded_rows <= 0 ||
      experts_per_rank <= 0 || world < 1 || world > kMaxPeers)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (ld & 7) || (padded_rows & 127)) return B200Q_ERR_SHAPE;      // whole scale-factor tiles along D
  if (!aligned16(x)) return B200Q_ERR_ALIGNMENT;
  PeerBufs peers = {};
  for (int i = 0; i < world; ++i) {
    if (peer_codes[i] == nullptr || peer_sf[i] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(peer_codes[i])) return B200Q_ERR_ALIGNMENT;
    peers.codes[i] = (uint8_t*)peer_codes[i];
    peers.sf[i] = (uint8_t*)peer_sf[i];
  }
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_dispatch_kernel, dim3(thread_item_grid(padded_rows * (D >> 5))), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      (const uint16_t*)x, D, ld, src_of_row, tile_expert, padded_offs, num_tiles, padded_rows, row_base, experts_per_rank, peers);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_zero_pad_rows(const int32_t* src_of_row, const int32_t* num_tiles, int64_t padded_rows, int64_t D, void* codes,
                            void* sf, void* stream) {
  PdlChain pdl_chain;
  if (src_of_row == nullptr || num_tiles == nullptr || codes == nullptr || sf == nullptr || padded_rows <= 0 || D <= 0)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (padded_rows & 127)) return B200Q_ERR_SHAPE;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_zero_pad_rows_kernel, dim3(thread_item_grid(padded_rows * (D >> 5))), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      src_of_row, num_tiles, padded_rows, D, (uint8_t*)codes, (uint8_t*)sf);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_combine_peers(void* const* peer_y, int world, int64_t ldy, const void* w, const int32_t* pair_peer,
                            const int32_t* pair_row, int64_t T, int k, int64_t D, void* out, void* stream) {
  PdlChain pdl_chain;
  if (peer_y == nullptr || w == nullptr || pair_peer == nullptr || pair_row == nullptr || out == nullptr || T <= 0 || k <= 0 ||
      D <= 0 || ldy < D || world < 1 || world > kMaxPeers)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 7) || (ldy & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(out)) return B200Q_ERR_ALIGNMENT;
  PeerRows peers = {};
  for (int i = 0; i < world; ++i) {
    if (peer_y[i] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(peer_y[i])) return B200Q_ERR_ALIGNMENT;
    peers.y[i] = (const uint16_t*)peer_y[i];
  }
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_combine_kernel, dim3(row_grid(T * ((D + 255) / 256))), dim3(256), (size_t)(0), (cudaStream_t)stream, peers, ldy, (const uint16_t*)w, pair_peer,
                                                                                      pair_row, T, k, D, (uint16_t*)out);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_ep_index(const int32_t* all_offs, int world, int rank, int E, const int64_t* top_idx, const int32_t* row_of,
                       const int32_t* padded_offs, int64_t n_pairs, int32_t* row_base, int32_t* own_offs, int32_t* pair_peer,
                       int32_t* pair_row, void* stream) {
  PdlChain pdl_chain;
  if (all_offs == nullptr || top_idx == nullptr || row_of == nullptr || padded_offs == nullptr || row_base == nullptr ||
      own_offs == nullptr || pair_peer == nullptr || pair_row == nullptr || n_pairs <= 0 || world < 1 || world > kMaxPeers ||
      rank < 0 || rank >= world || E <= 0)
    return B200Q_ERR_INVALID_ARG;
  if (E > kMaxExperts || E % world) return B200Q_ERR_SHAPE;
  int rc = require_sm100();
  if (rc) return rc;
  const int64_t want = (n_pairs + 255) / 256, cap = (int64_t)kNumSMs * 4;
  launch_pdl(moe_ep_index_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      all_offs, world, rank, E, E / world, top_idx, row_of, padded_offs, n_pairs, row_base, own_offs, pair_peer, pair_row);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_peer_barrier(void* const* flag_ptrs, int world, int rank, int epoch, void* stream) {
  PdlChain pdl_chain;
  if (flag_ptrs == nullptr || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return B200Q_ERR_INVALID_ARG;
  PeerFlags flags = {};
  for (int i = 0; i < world; ++i) {
    if (flag_ptrs[i] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(flag_ptrs[i]) & 3) return B200Q_ERR_ALIGNMENT;
    flags.f[i] = (int32_t*)flag_ptrs[i];
  }
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(peer_barrier_kernel, dim3(1), dim3(32), (size_t)(0), (cudaStream_t)stream, flags, world, rank, epoch);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_scatter_rows_peers(const void* x, int64_t ld, const void* w, const int32_t* pair_peer, const int32_t* pair_row, int64_t T,
                                 int k, int64_t D, void* const* peer_y, int world, int64_t ldy, void* stream) {
  PdlChain pdl_chain;
  if (x == nullptr || pair_peer == nullptr || pair_row == nullptr || peer_y == nullptr || T <= 0 || k <= 0 || D <= 0 || ld < D ||
      ldy < D || world < 1 || world > kMaxPeers)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 7) || (ld & 7) || (ldy & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(x)) return B200Q_ERR_ALIGNMENT;
  PeerRowsW peers = {};
  for (int i = 0; i < world; ++i) {
    if (peer_y[i] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(peer_y[i])) return B200Q_ERR_ALIGNMENT;
    peers.y[i] = (uint16_t*)peer_y[i];
  }
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_scatter_rows_peers_kernel, dim3(row_grid(T * k * ((D + 255) / 256))), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      (const uint16_t*)x, ld, (const uint16_t*)w, pair_peer, pair_row, T * k, k, D, peers, ldy);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_zero_pad_rows_bf16(const int32_t* src_of_row, const int32_t* num_tiles, int64_t padded_rows, int64_t D, void* buf,
                                 int64_t ld, void* stream) {
  PdlChain pdl_chain;
  if (src_of_row == nullptr || num_tiles == nullptr || buf == nullptr || padded_rows <= 0 || D <= 0 || ld < D) return B200Q_ERR_INVALID_ARG;
  if ((D & 7) || (ld & 7) || (padded_rows & 127)) return B200Q_ERR_SHAPE;
  if (!aligned16(buf)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_zero_pad_rows_bf16_kernel, dim3(row_grid(padded_rows)), dim3(256), (size_t)(0), (cudaStream_t)stream, src_of_row, num_tiles, padded_rows, D,
                                                                                        (uint16_t*)buf, ld);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_pair_dots_peers(const void* dout, int64_t ld, void* const* peer_y, int world, int64_t ldy, const int32_t* pair_peer,
                              const int32_t* pair_row, int64_t T, int k, int64_t D, float* dw, void* stream) {
  PdlChain pdl_chain;
  if (dout == nullptr || peer_y == nullptr || pair_peer == nullptr || pair_row == nullptr || dw == nullptr || T <= 0 || k <= 0 ||
      D <= 0 || ld < D || ldy < D || world < 1 || world > kMaxPeers)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 7) || (ld & 7) || (ldy & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(dout)) return B200Q_ERR_ALIGNMENT;
  PeerRows peers = {};
  for (int i = 0; i < world; ++i) {
    if (peer_y[i] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(peer_y[i])) return B200Q_ERR_ALIGNMENT;
    peers.y[i] = (const uint16_t*)peer_y[i];
  }
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_pair_dots_peers_kernel, dim3(row_grid(T * k)), dim3(256), (size_t)(0), (cudaStream_t)stream, (const uint16_t*)dout, ld, peers, ldy, pair_peer, pair_row,
                                                                               T * k, k, D, dw);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_swiglu_backward(const void* g, int64_t rows, int64_t I, int64_t ldg, const void* dh, int64_t lddh, void* dg, int64_t lddg,
                          void* stream) {
  PdlChain pdl_chain;
  if (g == nullptr || dh == nullptr || dg == nullptr || rows <= 0 || I <= 0 || ldg < 2 * I || lddh < I || lddg < 2 * I)
    return B200Q_ERR_INVALID_ARG;
  if ((I & 7) || (ldg & 7) || (lddh & 7) || (lddg & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(g) || !aligned16(dh) || !aligned16(dg)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(swiglu_backward_kernel, dim3(thread_item_grid(rows * (I >> 3))), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      (const uint16_t*)g, rows, I, ldg, (const uint16_t*)dh, lddh, (uint16_t*)dg, lddg);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_unpermute_backward(const void* dout, const void* w, const void* y, int64_t ldy, const int32_t* row_of,
                                 const int32_t* src_of_row, int64_t T, int k, int64_t D, int64_t padded_rows, void* dy, float* dw,
                                 void* stream) {
  PdlChain pdl_chain;
  if (dout == nullptr || w == nullptr || row_of == nullptr || src_of_row == nullptr || (dy == nullptr && dw == nullptr) || T <= 0 ||
      k <= 0 || D <= 0 || padded_rows <= 0 || (y != nullptr && ldy < D) || (dw != nullptr && y == nullptr))
    return B200Q_ERR_INVALID_ARG;
  if ((D & 7) || (y != nullptr && (ldy & 7))) return B200Q_ERR_SHAPE;
  if (!aligned16(dout) || (dy != nullptr && !aligned16(dy)) || (y != nullptr && !aligned16(y))) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_unpermute_backward_kernel, dim3(row_grid(T * k + (dy != nullptr ? padded_rows : 0))), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      (const uint16_t*)dout, (const uint16_t*)w, (const uint16_t*)y, ldy, row_of, src_of_row, T * k, k, D,
      dy != nullptr ? padded_rows : 0, (uint16_t*)dy, dw);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_router_topk(const float* logits, int64_t T, int E, int k, int score_fn, int normalize, int64_t* top_idx,
                          void* top_w, void* probs, int32_t* expert_counts, const float* select_bias, int out_fp32,
                          void* stream) {
  PdlChain pdl_chain;
  if (logits == nullptr || top_idx == nullptr || top_w == nullptr || T <= 0 || E <= 0 || k <= 0 || (score_fn != 0 && score_fn != 1))
    return B200Q_ERR_INVALID_ARG;
  if (E > kMaxExperts || k > 32 || k > E) return B200Q_ERR_SHAPE;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (expert_counts != nullptr) B200Q_CUDA(zero_before_kernel(expert_counts, (size_t)E * sizeof(int32_t), st));
#define B200Q_GO(P)                                                                                                          \
  do {                                                                                                                       \
    if (select_bias != nullptr)                                                                                              \
      launch_pdl(moe_router_topk_kernel<P, true>, dim3(row_grid(T)), dim3(256), (size_t)(0), st, logits, T, E, k, score_fn, normalize, top_idx, top_w, probs,       \
                                                                   expert_counts, select_bias, out_fp32);                    \
    else                                                                                                                     \
      launch_pdl(moe_router_topk_kernel<P, false>, dim3(row_grid(T)), dim3(256), (size_t)(0), st, logits, T, E, k, score_fn, normalize, top_idx, top_w, probs,      \
                                                                    expert_counts, nullptr, out_fp32);                       \
  } while (0)
  if (E <= 32) B200Q_GO(1);
  else if (E <= 64) B200Q_GO(2);
  else if (E <= 128) B200Q_GO(4);
  else B200Q_GO(8);
#undef B200Q_GO
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_pair_of_row(const int32_t* row_of, int64_t n_pairs, int64_t padded_rows, int32_t* pair_of_row, void* stream) {
  PdlChain pdl_chain;
  if (row_of == nullptr || pair_of_row == nullptr || n_pairs <= 0 || padded_rows <= 0 || n_pairs > INT32_MAX) return B200Q_ERR_INVALID_ARG;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  B200Q_CUDA(fill_before_kernel(pair_of_row, 0xff, (size_t)padded_rows * sizeof(int32_t), st));      // -1 everywhere
  launch_pdl(moe_pair_of_row_kernel, dim3((unsigned)((n_pairs + 255) / 256)), dim3(256), (size_t)(0), st, row_of, n_pairs, padded_rows, pair_of_row);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_moe_unpermute(const void* y, int64_t ldy, const void* w, const int32_t* row_of, int64_t T, int k, int64_t D, void* out,
                        void* stream) {
  PdlChain pdl_chain;
  if (y == nullptr || row_of == nullptr || out == nullptr || T <= 0 || k <= 0 || D <= 0 || ldy < D)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 7) || (ldy & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(y) || !aligned16(out)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  launch_pdl(moe_unpermute_kernel, dim3(row_grid(T * ((D + 255) / 256))), dim3(256), (size_t)(0), (cudaStream_t)stream, 
      (const uint16_t*)y, ldy, (const uint16_t*)w, row_of, T, k, D, (uint16_t*)out);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// Same plan as b200q_moe_permute_plan, for callers that cannot hand over a workspace because
// they cannot allocate device memory at this point.  The scratch is a fixed array inside the
// library (g_static_plan_scratch) instead of a caller buffer; nothing is allocated or freed here.
//
// `g_static_plan_scratch` in host code is only a handle: the kernels need the array's address on
// the current device, which cudaGetSymbolAddress returns.  The first call on each device looks
// it up (with that device current) and remembers it, so make that first call outside any stream
// capture.  Limits: ceil(n_pairs / 1024) * E <= 262144 entries, else B200Q_ERR_SHAPE.  The array
// is shared by all calls on a device and keeps what the last call left in it: every entry a call
// reads is first written by that call's own histogram kernel, so nothing has to be cleared, but
// two calls that overlap on the GPU (different streams) race on it — serialize them.
int b200q_moe_permute_plan_static(const int64_t* top_idx, int64_t n_pairs, int k, int E, int32_t* offs,
                                  int32_t* padded_offs, int32_t* row_of, int32_t* src_of_row, int32_t* tile_expert,
                                  int32_t* num_tiles, void* stream) {
  PdlChain pdl_chain;
  if (top_idx == nullptr || offs == nullptr || padded_offs == nullptr || row_of == nullptr || src_of_row == nullptr ||
      tile_expert == nullptr || num_tiles == nullptr || n_pairs <= 0 || k <= 0 || E <= 0)
    return B200Q_ERR_INVALID_ARG;
  if (E > kMaxExperts || n_pairs > INT32_MAX / 2) return B200Q_ERR_SHAPE;
  const int64_t nblocks64 = (n_pairs + kPlanThreads - 1) / kPlanThreads;
  if (nblocks64 * E > kStaticPlanInts) return B200Q_ERR_SHAPE;     // beyond the built-in scratch
  int rc = require_sm100();
  if (rc) return rc;
  int dev = -1;
  B200Q_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200Q_ERR_INVALID_ARG;
  int32_t* ptr = g_static_plan_ptr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    B200Q_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_plan_scratch));
    if (ptr == nullptr) return B200Q_ERR_CUDA;
    g_static_plan_ptr[dev].store(ptr, std::memory_order_release);
  }
  return run_permute_plan(top_idx, n_pairs, k, E, ptr, offs, padded_offs, row_of, src_of_row, tile_expert,
                          num_tiles, (cudaStream_t)stream);
}

// ---- the expert path of the MoE block in one call ----------------------------------------------------
// permute plan -> gather + MXFP8 -> grouped GEMM 1 with SwiGLU + MXFP8 epilogue -> grouped GEMM 2 -> weighted
// unpermute (src/layers/mlp.py:446-477 with grouped_mlp, :55-100, between permute and unpermute), for bias-free
// SwiGLU experts without gradients.  Each step is the entry point of that name; what this call adds is that the
// eight launches are issued back to back by one host call (the Python layer spends more time between two of its
// calls than most of these kernels run) and that every launch after the first may start while its predecessor
// drains.  The workspace holds the plan's tables and the intermediates; nothing in it needs to be initialised.
static inline int64_t ws_align(int64_t v) { return (v + 255) & ~(int64_t)255; }

struct FfnWorkspace {
  int64_t padded_rows, plan, offs, padded_offs, row_of, src_of_row, tile_expert, num_tiles, a, a_sf, h, h_sf, y, total;
};
static FfnWorkspace ffn_workspace(int64_t T, int k, int64_t D, int E, int64_t I) {
  FfnWorkspace w = {};
  const int64_t n_pairs = T * k;
  w.padded_rows = b200q_moe_padded_rows(n_pairs, E);
  int64_t o = 0;
  auto take = [&](int64_t bytes) { const int64_t at = o; o += ws_align(bytes); return at; };
  w.plan = take(b200q_moe_plan_workspace_bytes(n_pairs, E));
  w.offs = take((int64_t)E * 4);
  w.padded_offs = take((int64_t)(E + 1) * 4);
  w.row_of = take(n_pairs * 4);
  w.src_of_row = take(w.padded_rows * 4);
  w.tile_expert = take(w.padded_rows / 128 * 4);
  w.num_tiles = take(4);
  w.a = take(w.padded_rows * D);
  w.a_sf = take(b200q_sf_bytes(w.padded_rows, D / 32, B200Q_SF_SWIZZLE_128x4));
  w.h = take(w.padded_rows * I);
  w.h_sf = take(b200q_sf_bytes(w.padded_rows, I / 32, B200Q_SF_SWIZZLE_128x4));
  w.y = take(w.padded_rows * D * 2);
  w.total = o;
  return w;
}

int64_t b200q_moe_ffn_workspace_bytes(int64_t T, int k, int64_t D, int E, int64_t I) {
  if (T <= 0 || k <= 0 || D <= 0 || E <= 0 || I <= 0) return 0;
  return ffn_workspace(T, k, D, E, I).total;
}

int b200q_moe_ffn_forward(const void* x, int64_t ldx, const int64_t* top_idx, const void* top_w, int64_t T, int k, int64_t D, int E,
                          int64_t I, const void* w1_codes, const void* w1_sf, const void* w2_codes, const void* w2_sf, void* out,
                          int32_t* offs, void* workspace, void* stream) {
  PdlChain pdl_chain;
  if (x == nullptr || top_idx == nullptr || top_w == nullptr || w1_codes == nullptr || w1_sf == nullptr || w2_codes == nullptr ||
      w2_sf == nullptr || out == nullptr || workspace == nullptr || T <= 0 || k <= 0 || D <= 0 || E <= 0 || I <= 0)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (I & 63) || ((2 * I) & 127)) return B200Q_ERR_SHAPE;      // both GEMMs' N % 128, h blocks of 32 per 64 gate/up columns
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return B200Q_ERR_ALIGNMENT;
  const FfnWorkspace w = ffn_workspace(T, k, D, E, I);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* padded_offs = reinterpret_cast<int32_t*>(ws + w.padded_offs);
  int32_t* row_of = reinterpret_cast<int32_t*>(ws + w.row_of);
  int32_t* src_of_row = reinterpret_cast<int32_t*>(ws + w.src_of_row);
  int32_t* tile_expert = reinterpret_cast<int32_t*>(ws + w.tile_expert);
  int32_t* num_tiles = reinterpret_cast<int32_t*>(ws + w.num_tiles);
  int rc = b200q_moe_permute_plan(top_idx, T * k, k, E, offs != nullptr ? offs : reinterpret_cast<int32_t*>(ws + w.offs), padded_offs, row_of,
                                  src_of_row,
                                  tile_expert, num_tiles, ws + w.plan, stream);
  if (rc) return rc;
  if ((rc = b200q_moe_gather(x, D, ldx, src_of_row, num_tiles, w.padded_rows, 1, B200Q_E4M3, ws + w.a, ws + w.a_sf, stream))) return rc;
  if ((rc = b200q_grouped_gemm_mxfp8_swiglu(ws + w.a, B200Q_E4M3, ws + w.a_sf, w1_codes, B200Q_E4M3, w1_sf, tile_expert, num_tiles,
                                            w.padded_rows, E, 2 * I, D, ws + w.h, I, ws + w.h_sf, stream)))
    return rc;
  if ((rc = b200q_grouped_gemm_mxfp8(ws + w.h, B200Q_E4M3, ws + w.h_sf, w2_codes, B200Q_E4M3, w2_sf, tile_expert, num_tiles,
                                     w.padded_rows, E, D, I, ws + w.y, D, stream)))
    return rc;
  return b200q_moe_unpermute(ws + w.y, D, top_w, row_of, T, k, D, out, stream);
}


// ---- the trainable expert path: forward and backward as one call each ---------------------------------
// The sequences of the autograd function of SparseMoEBlock for bias-free SwiGLU experts (the explicit backward of
// src/layers/mlp.py:446-477, which the reference leaves to autograd through torch._grouped_mm), each issued by one host
// call: every kernel after the first of a call may be scheduled while its predecessor drains.  Each step is the entry
// point of that name; results equal the separate calls bit for bit.  The plan comes from b200q_moe_permute_plan.
static int64_t sfb(int64_t rows, int64_t cols) { return ws_align(b200q_sf_bytes(rows, cols / 32, B200Q_SF_SWIZZLE_128x4)); }

int64_t b200q_moe_ffn_train_forward_workspace_bytes(int64_t padded_rows, int64_t D, int64_t I) {
  if (padded_rows <= 0 || D <= 0 || I <= 0) return 0;
  return ws_align(padded_rows * D) + sfb(padded_rows, D) + ws_align(padded_rows * I) + sfb(padded_rows, I);
}

int b200q_moe_ffn_train_forward(const void* x, int64_t ldx, const void* top_w, int64_t T, int k, int64_t D, int E, int64_t I,
                                int64_t padded_rows, const int32_t* row_of, const int32_t* src_of_row, const int32_t* tile_expert,
                                const int32_t* num_tiles, const void* w1r, const void* w1sr, const void* w2r, const void* w2sr,
                                void* ac, void* asc, void* g, void* hc, void* hsc, void* y, void* out, void* workspace, void* stream) {
  PdlChain pdl_chain;
  if (x == nullptr || top_w == nullptr || row_of == nullptr || src_of_row == nullptr || tile_expert == nullptr || num_tiles == nullptr ||
      w1r == nullptr || w1sr == nullptr || w2r == nullptr || w2sr == nullptr || ac == nullptr || asc == nullptr || g == nullptr ||
      hc == nullptr || hsc == nullptr || y == nullptr || out == nullptr || workspace == nullptr || T <= 0 || k <= 0 || E <= 0)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (I & 127) || (padded_rows & 127) || padded_rows <= 0) return B200Q_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return B200Q_ERR_ALIGNMENT;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* ar = ws;
  uint8_t* asr = ar + ws_align(padded_rows * D);
  uint8_t* hr = asr + sfb(padded_rows, D);
  uint8_t* hsr = hr + ws_align(padded_rows * I);
  int rc = b200q_moe_gather_quantize_dual(x, D, ldx, src_of_row, padded_rows, B200Q_E4M3, ar, asr, ac, asc, nullptr, stream);
  if (rc) return rc;
  if ((rc = b200q_grouped_gemm_mxfp8(ar, B200Q_E4M3, asr, w1r, B200Q_E4M3, w1sr, tile_expert, num_tiles, padded_rows, E, 2 * I, D, g, 2 * I,
                                     stream)))
    return rc;
  if ((rc = b200q_swiglu_quantize_dual(g, padded_rows, I, 2 * I, B200Q_E4M3, hr, hsr, hc, hsc, nullptr, stream))) return rc;
  if ((rc = b200q_grouped_gemm_mxfp8(hr, B200Q_E4M3, hsr, w2r, B200Q_E4M3, w2sr, tile_expert, num_tiles, padded_rows, E, D, I, y, D, stream)))
    return rc;
  return b200q_moe_unpermute(y, D, top_w, row_of, T, k, D, out, stream);
}

struct FfnBwdWorkspace { int64_t pair_of_row, dyr, dysr, dyc, dysc, dots, dh, dgr, dgsr, dgc, dgsc, da, total; };
static FfnBwdWorkspace ffn_bwd_workspace(int64_t R, int64_t D, int64_t I) {
  FfnBwdWorkspace w = {};
  int64_t o = 0;
  auto take = [&](int64_t bytes) { const int64_t at = o; o += ws_align(bytes); return at; };
  w.pair_of_row = take(R * 4);
  w.dyr = take(R * D);
  w.dysr = take(sfb(R, D));
  w.dyc = take(D * R);
  w.dysc = take(sfb(D, R));
  w.dots = take(D / 128 * R * 4);
  w.dh = take(R * I * 2);
  w.dgr = take(R * 2 * I);
  w.dgsr = take(sfb(R, 2 * I));
  w.dgc = take(2 * I * R);
  w.dgsc = take(sfb(2 * I, R));
  w.da = take(R * D * 2);
  w.total = o;
  return w;
}

int64_t b200q_moe_ffn_train_backward_workspace_bytes(int64_t padded_rows, int64_t D, int64_t I) {
  if (padded_rows <= 0 || D <= 0 || I <= 0) return 0;
  return ffn_bwd_workspace(padded_rows, D, I).total;
}

int b200q_moe_ffn_train_backward(const void* dout, int64_t lddout, const void* top_w, int64_t T, int k, int64_t D, int E, int64_t I,
                                 int64_t padded_rows, const int32_t* row_of, const int32_t* padded_offs, const int32_t* tile_expert,
                                 const int32_t* num_tiles, const void* y, const void* g, const void* ac, const void* asc, const void* hc,
                                 const void* hsc, const void* w1c, const void* w1sc, const void* w2c, const void* w2sc, void* dx, float* dw,
                                 void* dw1, void* dw2, void* workspace, void* stream) {
  PdlChain pdl_chain;
  if (dout == nullptr || top_w == nullptr || row_of == nullptr || padded_offs == nullptr || tile_expert == nullptr ||
      num_tiles == nullptr || y == nullptr || g == nullptr || ac == nullptr || asc == nullptr || hc == nullptr || hsc == nullptr ||
      w1c == nullptr || w1sc == nullptr || w2c == nullptr || w2sc == nullptr || dx == nullptr || dw == nullptr || dw1 == nullptr ||
      dw2 == nullptr || workspace == nullptr || T <= 0 || k <= 0 || E <= 0)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (I & 127) || (padded_rows & 127) || padded_rows <= 0) return B200Q_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return B200Q_ERR_ALIGNMENT;
  const FfnBwdWorkspace w = ffn_bwd_workspace(padded_rows, D, I);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* pair_of_row = reinterpret_cast<int32_t*>(ws + w.pair_of_row);
  const int64_t n_pairs = T * k;
  int rc = b200q_moe_pair_of_row(row_of, n_pairs, padded_rows, pair_of_row, stream);
  if (rc) return rc;
  // dy = w * dout scattered into the padded layout, both ways in E5M2, and dw = <dout, y>
  if ((rc = b200q_moe_unpermute_backward_quantize_dual(dout, lddout, top_w, pair_of_row, k, padded_rows, D, B200Q_E5M2, ws + w.dyr,
                                                       ws + w.dysr, ws + w.dyc, ws + w.dysc, y, D, row_of, n_pairs,
                                                       reinterpret_cast<float*>(ws + w.dots), dw, stream)))
    return rc;
  if ((rc = b200q_grouped_gemm_mxfp8_dgrad(ws + w.dyr, B200Q_E5M2, ws + w.dysr, w2c, B200Q_E4M3, w2sc, tile_expert, num_tiles, padded_rows, E,
                                           I, D, ws + w.dh, I, stream)))
    return rc;
  if ((rc = b200q_grouped_gemm_mxfp8_wgrad(ws + w.dyc, B200Q_E5M2, ws + w.dysc, hc, B200Q_E4M3, hsc, padded_offs, E, D, I, padded_rows, dw2, I,
                                           stream)))
    return rc;
  if ((rc = b200q_swiglu_backward_quantize_dual(g, padded_rows, I, 2 * I, ws + w.dh, I, B200Q_E5M2, ws + w.dgr, ws + w.dgsr, ws + w.dgc,
                                                ws + w.dgsc, nullptr, stream)))
    return rc;
  if ((rc = b200q_grouped_gemm_mxfp8_dgrad(ws + w.dgr, B200Q_E5M2, ws + w.dgsr, w1c, B200Q_E4M3, w1sc, tile_expert, num_tiles, padded_rows, E,
                                           D, 2 * I, ws + w.da, D, stream)))
    return rc;
  if ((rc = b200q_grouped_gemm_mxfp8_wgrad(ws + w.dgc, B200Q_E5M2, ws + w.dgsc, ac, B200Q_E4M3, asc, padded_offs, E, 2 * I, D, padded_rows, dw1,
                                           D, stream)))
    return rc;
  return b200q_moe_unpermute(ws + w.da, D, nullptr, row_of, T, k, D, dx, stream);
}

// ---- expert-parallel forward after the index tables: one call ------------------------------------------
// zero the pad rows of my receive buffers, dispatch (gather + MXFP8, stored into the owners' buffers), rendezvous, both
// grouped GEMMs over the experts I own (SwiGLU in the first one's epilogue, the second one writing where the peers will
// read), rendezvous, combine (weighted rows loaded from their owners), rendezvous - the steps of
// b200q_moe_zero_pad_rows, b200q_moe_dispatch_peers, b200q_peer_barrier, b200q_grouped_gemm_mxfp8_swiglu,
// b200q_grouped_gemm_mxfp8 and b200q_moe_combine_peers, issued by one host call: per step the host spends more time
// between two calls than most of these kernels run.  The three rendezvous use epochs epoch + 1 .. epoch + 3.
int64_t b200q_moe_ep_forward_workspace_bytes(int64_t own_padded_rows, int64_t I) {
  if (own_padded_rows <= 0 || I <= 0) return 0;
  return ws_align(own_padded_rows * I) + sfb(own_padded_rows, I);
}

int b200q_moe_ep_forward(const void* x, int64_t ldx, const void* top_w, int64_t T, int k, int64_t D, int64_t I, int experts_per_rank,
                         int world, int rank, int epoch, const int32_t* src_of_row, const int32_t* tile_expert,
                         const int32_t* padded_offs, const int32_t* num_tiles, int64_t padded_rows, const int32_t* row_base,
                         const int32_t* pair_peer, const int32_t* pair_row, const int32_t* own_src_of_row,
                         const int32_t* own_tile_expert, const int32_t* own_num_tiles, int64_t own_padded_rows,
                         void* const* peer_codes, void* const* peer_sf, void* const* peer_y, void* const* flag_ptrs,
                         const void* w1_codes, const void* w1_sf, const void* w2_codes, const void* w2_sf, void* out, void* workspace,
                         void* stream) {
  PdlChain pdl_chain;
  if (x == nullptr || top_w == nullptr || src_of_row == nullptr || tile_expert == nullptr || padded_offs == nullptr || num_tiles == nullptr ||
      row_base == nullptr || pair_peer == nullptr || pair_row == nullptr || own_src_of_row == nullptr || own_tile_expert == nullptr ||
      own_num_tiles == nullptr || peer_codes == nullptr || peer_sf == nullptr || peer_y == nullptr || flag_ptrs == nullptr ||
      w1_codes == nullptr || w1_sf == nullptr || w2_codes == nullptr || w2_sf == nullptr || out == nullptr || workspace == nullptr ||
      T <= 0 || k <= 0 || D <= 0 || I <= 0 || padded_rows <= 0 || own_padded_rows <= 0 || experts_per_rank <= 0 || world <= 0 ||
      rank < 0 || rank >= world)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (I & 63) || ((2 * I) & 127) || (own_padded_rows & 127)) return B200Q_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return B200Q_ERR_ALIGNMENT;
  uint8_t* h = static_cast<uint8_t*>(workspace);
  uint8_t* h_sf = h + ws_align(own_padded_rows * I);
  void* my_codes = peer_codes[rank];
  void* my_sf = peer_sf[rank];
  int rc = b200q_moe_zero_pad_rows(own_src_of_row, own_num_tiles, own_padded_rows, D, my_codes, my_sf, stream);
  if (rc) return rc;
  if ((rc = b200q_moe_dispatch_peers(x, D, ldx, src_of_row, tile_expert, padded_offs, num_tiles, padded_rows, row_base, experts_per_rank,
                                     world, peer_codes, peer_sf, stream)))
    return rc;
  if ((rc = b200q_peer_barrier(flag_ptrs, world, rank, epoch + 1, stream))) return rc;
  if ((rc = b200q_grouped_gemm_mxfp8_swiglu(my_codes, B200Q_E4M3, my_sf, w1_codes, B200Q_E4M3, w1_sf, own_tile_expert, own_num_tiles,
                                            own_padded_rows, experts_per_rank, 2 * I, D, h, I, h_sf, stream)))
    return rc;
  if ((rc = b200q_grouped_gemm_mxfp8(h, B200Q_E4M3, h_sf, w2_codes, B200Q_E4M3, w2_sf, own_tile_expert, own_num_tiles, own_padded_rows,
                                     experts_per_rank, D, I, peer_y[rank], D, stream)))
    return rc;
  if ((rc = b200q_peer_barrier(flag_ptrs, world, rank, epoch + 2, stream))) return rc;
  if ((rc = b200q_moe_combine_peers(peer_y, world, D, top_w, pair_peer, pair_row, T, k, D, out, stream))) return rc;
  return b200q_peer_barrier(flag_ptrs, world, rank, epoch + 3, stream);     // nobody overwrites y or the codes while a peer still reads them
}

}  // extern "C"
