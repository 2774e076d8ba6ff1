// Scaled GEMMs on the 5th-generation tensor cores:  D[M,N] (bf16) = A[M,K] . B[N,K]^T
//
//   KIND_F8  : fp8 codes, fp32 scale per row of A and per row of B applied in the epilogue
//              (stands for torch._scaled_mm, src/quant/fp8.py:59-65)
//   KIND_I8  : int8-series codes, tcgen05.mma kind::i8 with 32-bit integer accumulators, the
//              same fp32 row / column scales in the epilogue (stands for torch._int_mm and the
//              scaling after it, src/quant/int8.py:49-53); integer accumulation is exact, so the
//              result equals the reference's bit for bit
//   KIND_MX  : MXFP8, tcgen05.mma kind::mxf8f6f4.block_scale (E8M0 scale per 32 elements)
//   KIND_NV  : NVFP4, tcgen05.mma kind::mxf4nvf4.block_scale.block16 (E4M3 scale per 16
//              elements), fp32 tensor scales applied in the epilogue
// and the ragged grouped form of KIND_MX (stands for torch._grouped_mm, src/layers/mlp.py:89,97),
// where every 128-row tile of A belongs to one expert and B holds the experts' weights stacked.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0    TMA producer: A/B tiles (128-byte-swizzled, K-major) and the scale-factor atoms of
//             each K step into a ring of shared-memory stages, signalled through mbarriers;
//   warp 1    MMA issuer: one thread copies the stage's scale factors to tensor memory
//             (tcgen05.cp), issues the four K=32-byte tcgen05.mma of the stage, and commits to
//             the stage's "empty" barrier; accumulators live in tensor memory;
//   warps 2-5 epilogue: tcgen05.ld the fp32 accumulators (lane = row) 32 columns at a time,
//             scale, round to bf16, stage a 32x32 block in 64-byte-swizzled shared memory and
//             hand it to a TMA store (which also clips the ragged edges).  Two accumulators in
//             tensor memory let the epilogue of tile i overlap the main loop of tile i+1; at
//             width 256 with scale factors they overlap by 32 / 64 columns, which the epilogue
//             reads first.
// No cluster launch and no multicast: the same binary runs under any number of processes.
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <algorithm>

namespace b200q {
namespace {

enum { KIND_F8 = 0, KIND_MX = 1, KIND_NV = 2, KIND_I8 = 3 };
// kinds whose scales are one fp32 per output row and column, applied in the epilogue
__host__ __device__ constexpr bool row_scaled(int kind) { return kind == KIND_F8 || kind == KIND_I8; }

constexpr int BM = 128;
constexpr int BKB = 128;                 // bytes of K per stage (= one 128-byte swizzle row)
constexpr int kGemmThreads = 192;
constexpr int kSmemBudget = 227 * 1024;
constexpr int kSfStageBytes = 2048;             // EPI_MXQ: scale-factor staging, two sets of up to two 512-byte atoms

#include "gemm_epilogue.cuh"

constexpr int cgcd(int a, int b) { return b == 0 ? a : cgcd(b, a % b); }

template <int KIND, int BN_>
struct Cfg {
  static constexpr int BN = BN_;
  // A B tile that does not start on a multiple of 128 rows straddles one more 128-row group of
  // scale factors; NB_ATOMS is the number of groups loaded per K step (enough for any offset).
  static constexpr int MAX_OFF = 128 - cgcd(BN, 128);
  static constexpr int NB_ATOMS = (MAX_OFF + BN + 127) / 128;
  static constexpr int K_ATOMS = KIND == KIND_NV ? 4 : 1;                  // 512-byte SF atoms per K step and row group
  static constexpr int A_BYTES = BM * BKB;
  static constexpr int B_BYTES = BN * BKB;
  static constexpr int SFA_BYTES = row_scaled(KIND) ? 0 : K_ATOMS * 512;
  static constexpr int SFB_BYTES = row_scaled(KIND) ? 0 : NB_ATOMS * K_ATOMS * 512;
  static constexpr int STAGE_BYTES = ((A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + 1023) / 1024) * 1024;
  // Two staging blocks per epilogue warp unless giving one up buys another pipeline stage
  // (NVFP4 at width 256: 4 stages of 54 KB only fit beside 8 KB of staging).
  static constexpr int STAGES_2BUF = (kSmemBudget - 2048 - 2 * kEpiBytes1) / STAGE_BYTES;
  static constexpr int STAGES_1BUF = (kSmemBudget - 2048 - kEpiBytes1) / STAGE_BYTES;
  static constexpr int EPI_BUFS = (STAGES_1BUF > STAGES_2BUF && STAGES_2BUF < 4) ? 1 : 2;
  static constexpr int EPI_BYTES = EPI_BUFS * kEpiBytes1;
  static constexpr int STAGES_RAW = EPI_BUFS == 1 ? STAGES_1BUF : STAGES_2BUF;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SFA_COLS = row_scaled(KIND) ? 0 : 4 * K_ATOMS;
  static constexpr int SFB_COLS = row_scaled(KIND) ? 0 : 4 * K_ATOMS * NB_ATOMS;
  // Two accumulators always.  When two whole ones and the scale factors do not fit in the 512
  // columns (width 256, block-scaled kinds) the second accumulator starts OVL columns early, so
  // the two share OVL columns: the epilogue reads that shared strip of a tile first and only
  // then lets the next tile's MMA (which overwrites it) start; the rest of the tile drains while
  // the next main loop runs.  OVL = scale-factor columns rounded up to an epilogue block.
  static constexpr int SF_COLS = SFA_COLS + SFB_COLS;
  static constexpr bool OVERLAP = 2 * BN + SF_COLS > 512;
  static constexpr int OVL = OVERLAP ? ((2 * BN + SF_COLS - 512 + EPI_COLS - 1) / EPI_COLS) * EPI_COLS : 0;
  static constexpr int ACC1_COL0 = BN - OVL;
  static constexpr int SFA_COL0 = 2 * BN - OVL;
  static constexpr int SFB_COL0 = SFA_COL0 + SFA_COLS;
  static constexpr int TMEM_COLS = 512;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;                     // 1024-aligned
  static constexpr int BAR_OFF = EPI_OFF + EPI_BYTES;   // EPI_BYTES is a multiple of 1024
  static constexpr int SMEM_BYTES = BAR_OFF + 256 /*barriers*/ + 1024 /*alignment slack*/;
  // A B tile may start 64 rows into a 128-row scale-factor group (tensor-memory column offset 2);
  // offsets of 32 or 96 rows (odd column offsets) are misaligned for the MMA's scale operand.
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "tile width: multiple of 64 (also the epilogue block)");
  static_assert(SFB_COL0 + SFB_COLS <= TMEM_COLS, "tensor memory overflow");
  static_assert(STAGES >= 2, "not enough shared memory for a pipeline");
  static_assert(SMEM_BYTES <= kSmemBudget, "shared memory overflow");
};

struct GemmParams {
  const uint8_t* sfa;      // swizzled scale factors of A (block-scaled kinds)
  const uint8_t* sfb;
  const float* scale_a;    // F8: per row of A (or one value); NV: tensor scale of A
  const float* scale_b;
  int a_scalar, b_scalar;
  int a_fmt, b_fmt;
  int64_t M, N, K;         // K in elements; grouped: M = padded rows, N = columns per expert
  int num_m, num_n, num_k; // tiles (grouped: num_m is an upper bound, the true count is *num_tiles)
  int sf_kt;               // 512-byte atoms per row group along K in the SF buffers
  int64_t sfb_groups;      // 128-row groups in the SF buffer of B
  const int32_t* tile_expert;   // grouped: expert of every 128-row tile of A; null otherwise
  const int32_t* num_tiles;     // grouped: device count of row tiles in use
  GluOut glu;                   // EPI_GLU: where the SwiGLU + MXFP8 epilogue writes
  // Grouped backward forms (MXFP8, K % 128 == 0):
  int b_along_k;                // dgrad: B is [N, E*K], expert e's operand at K offset e*K (a transposed weight stack)
  int sf_kt_b;                  // 512-byte atoms per row group along K in B's scale buffer (== sf_kt unless b_along_k)
  const int32_t* ragged_offs;   // wgrad: padded_offs[E+1]; expert e contracts over rows [offs[e], offs[e+1]) of both operands
  int n_experts;                //        and writes rows [e*M, (e+1)*M) of the output
};

// plain output; SwiGLU -> MXFP8 codes; SwiGLU -> bf16 + amax; output quantized to MXFP8 (codes + scale bytes)
enum { EPI_BF16 = 0, EPI_GLU = 1, EPI_GLU_BF16 = 2, EPI_MXQ = 3 };
// Threads per CTA: producer warp, MMA warp and one (bf16 or MXFP8 output) or two (SwiGLU epilogue) groups
// of four epilogue warps.
__host__ __device__ constexpr int gemm_threads(int epi) { return epi == EPI_BF16 || epi == EPI_MXQ ? 192 : 320; }

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m, int& n) {
  constexpr int GM = 16;   // m-blocks per raster group: concurrent CTAs share A and B tiles through L2
  const int per_group = GM * num_n;
  const int g = t / per_group, r = t - g * per_group;
  const int first_m = g * GM;
  const int gm = num_m - first_m < GM ? num_m - first_m : GM;
  m = first_m + r % gm;
  n = r / gm;
}


// Everything the three roles need to know about tile t.
struct Tile {
  int m_blk, n_blk;
  int k0, nk;          // first K step and number of K steps (128 bytes each)
  int sfb_k0;          // first scale atom of B along K
  int64_t brow0;       // first row of the B tile
  int64_t bk0;         // K offset (bytes) of the B operand
  int64_t drow_off;    // row offset of the output tile
  bool zero;           // expert without rows: no K step runs, the epilogue stores zeros
};

template <int BN>
__device__ __forceinline__ Tile get_tile(const GemmParams& p, int t, int num_m) {
  Tile ti;
  int local = t, e = 0;
  if (p.ragged_offs != nullptr) {
    const int per = num_m * p.num_n;
    e = t / per;
    local = t - e * per;
  }
  tile_coords(local, num_m, p.num_n, ti.m_blk, ti.n_blk);
  if (p.tile_expert != nullptr) e = __ldcg(p.tile_expert + ti.m_blk);
  ti.k0 = 0; ti.nk = p.num_k; ti.sfb_k0 = 0; ti.bk0 = 0; ti.drow_off = 0; ti.zero = false;
  ti.brow0 = (int64_t)ti.n_blk * BN;
  if (p.ragged_offs != nullptr) {
    const int r0 = __ldcg(p.ragged_offs + e), r1 = __ldcg(p.ragged_offs + e + 1);
    ti.k0 = r0 >> 7;
    ti.nk = (r1 - r0) >> 7;
    if (ti.nk <= 0) {                      // no rows: nothing is loaded or multiplied (the operands there may hold
      ti.nk = 0;                           // anything, NaN included); the epilogue writes zeros
      ti.zero = true;
    }
    ti.sfb_k0 = 0;
    ti.drow_off = (int64_t)e * p.M;
  } else if (p.b_along_k) {
    ti.bk0 = (int64_t)e * p.K;
    ti.sfb_k0 = e * (int)(p.K >> 7);
  } else {
    ti.brow0 += (int64_t)e * p.N;
  }
  return ti;
}

template <int KIND, int BN, int EPI>
__global__ void __launch_bounds__(gemm_threads(EPI), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ OutMaps outs, const GemmParams p) {
  using C = Cfg<KIND, BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C::BAR_OFF;
  // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem ptr, abort
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + C::BAR_OFF + 8 * (2 * C::STAGES + 4));
  // set by a role whose bounded wait ran out; the others look at it once per tile (not per K step: a shared-memory
  // read after every ring wait costs the issuing threads 30 clocks each) and otherwise run into their own limits
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Grouped forms read the permute plan's tables right away: wait for the kernels before this one first.  The dense
  // forms read nothing of theirs until the roles start, so their set-up below overlaps the previous kernel's tail.
  const bool reads_plan = p.num_tiles != nullptr || p.ragged_offs != nullptr;
  if (reads_plan) grid_dependency_wait();
  int num_m = p.num_m;
  if (p.num_tiles != nullptr) {
    const int live = __ldcg(p.num_tiles);
    num_m = live < num_m ? live : num_m;
  }
  const int total_tiles = num_m * p.num_n * (p.ragged_offs != nullptr ? p.n_experts : 1);

  if (!row_scaled(KIND)) {
    // Scale-factor stage buffers start as zeros so that atoms beyond the end of K (never
    // loaded) multiply the zero-filled operand tail by a finite scale.
    for (int s = 0; s < C::STAGES; ++s) {
      uint32_t* sfz = reinterpret_cast<uint32_t*>(smem_gen + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES);
      for (int i = threadIdx.x; i < (C::SFA_BYTES + C::SFB_BYTES) / 4; i += gemm_threads(EPI)) sfz[i] = 0;
    }
    ptx::fence_proxy_async();
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), gemm_threads(EPI) / 32 - 2); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    for (int g = 0; g < outs.count; ++g) ptx::prefetch_tensormap(&outs.m[g]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (!reads_plan) grid_dependency_wait();      // operands, scales and the output buffer belong to earlier kernels until here

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile ti = get_tile<BN>(p, t, num_m);
        const int m_blk = ti.m_blk;
        const int64_t brow0 = ti.brow0;
        for (int kl = 0; kl < ti.nk; ++kl) {
          const int k = ti.k0 + kl;
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          const uint32_t fb = full_bar(stage);
          uint32_t tx = C::A_BYTES + C::B_BYTES;
          if (!row_scaled(KIND)) {
            // atoms of this K step that exist in the (padded) scale-factor buffers
            const int ka0 = k * C::K_ATOMS;
            const int ka = p.sf_kt - ka0 < C::K_ATOMS ? p.sf_kt - ka0 : C::K_ATOMS;
            tx += (uint32_t)(ka * 512 * (1 + C::NB_ATOMS));
            ptx::mbar_expect_tx(fb, tx);
            const uint32_t ssfa = sb + C::B_BYTES, ssfb = ssfa + C::SFA_BYTES;
            ptx::bulk_load(ssfa, p.sfa + ((int64_t)m_blk * p.sf_kt + ka0) * 512, ka * 512, fb);
            const int64_t g0 = brow0 >> 7;
#pragma unroll
            for (int j = 0; j < C::NB_ATOMS; ++j) {
              const int64_t rg = g0 + j < p.sfb_groups ? g0 + j : g0;     // past the end: any valid group
              ptx::bulk_load(ssfb + j * C::K_ATOMS * 512, p.sfb + (rg * p.sf_kt_b + ti.sfb_k0 + ka0) * 512, ka * 512, fb);
            }
          } else {
            ptx::mbar_expect_tx(fb, tx);
          }
          ptx::tma_load_2d(sa, &tmap_a, k * BKB, m_blk * BM, fb);
          ptx::tma_load_2d(sb, &tmap_b, (int32_t)(k * BKB + ti.bk0), (int32_t)brow0, fb);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 1); }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_iter) {
        const Tile ti = get_tile<BN>(p, t, num_m);
        const int64_t brow0 = ti.brow0;
        const uint32_t sfb_off = (uint32_t)(brow0 & 127) >> 5;   // B tile starts this many 32-row columns into its first SF group
        // Plain double buffering: wait until this accumulator's previous tile has been read.
        // Overlapped: wait until the PREVIOUS tile's epilogue (other accumulator) has read the
        // shared strip; every epilogue warp gets there only after finishing the tile before, which
        // used this accumulator.
        if (C::OVERLAP) {
          if (tile_iter > 0 && (!ptx::mbar_wait(tempty_bar(acc ^ 1), ((tile_iter - 1) >> 1) & 1) || *abort_flag)) { ok = false; break; }
        } else {
          if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1) || *abort_flag) { ok = false; break; }
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc ? C::ACC1_COL0 : 0);
        for (int k = 0; k < ti.nk; ++k) {
          if (!ptx::mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          if (!row_scaled(KIND)) {
            const uint32_t ssfa = sb + C::B_BYTES, ssfb = ssfa + C::SFA_BYTES;
#pragma unroll
            for (int a = 0; a < C::K_ATOMS; ++a) {
              ptx::tmem_cp_32x128b_warpx4(tmem_base + C::SFA_COL0 + 4 * a, ptx::smem_desc_sf(ssfa + a * 512));
#pragma unroll
              for (int j = 0; j < C::NB_ATOMS; ++j)
                ptx::tmem_cp_32x128b_warpx4(tmem_base + C::SFB_COL0 + 4 * (a * C::NB_ATOMS + j),
                                            ptx::smem_desc_sf(ssfb + (j * C::K_ATOMS + a) * 512));
            }
          }
          const uint64_t da = ptx::smem_desc_k_sw128(sa), db = ptx::smem_desc_k_sw128(sb);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t accum = (k | kk) != 0;
            const uint64_t adv = (uint64_t)(kk * 32 >> 4);   // 32 bytes of K per instruction
            if (KIND == KIND_I8) {
              ptx::mma_i8(d_tmem, da + adv, db + adv, ptx::idesc_i8(BM, BN), accum);
            } else if (KIND == KIND_F8) {
              ptx::mma_f8(d_tmem, da + adv, db + adv, ptx::idesc_f8(p.a_fmt, p.b_fmt, BM, BN), accum);
            } else if (KIND == KIND_MX) {
              ptx::mma_mxf8(d_tmem, da + adv, db + adv, ptx::idesc_block_scaled(p.a_fmt, p.b_fmt, 1, BM, BN, kk), accum,
                            tmem_base + C::SFA_COL0, tmem_base + C::SFB_COL0 + sfb_off);
            } else {
              ptx::mma_nvf4(d_tmem, da + adv, db + adv, ptx::idesc_block_scaled(1, 1, 0, BM, BN, 0), accum,
                            tmem_base + C::SFA_COL0 + 4 * kk, tmem_base + C::SFB_COL0 + 4 * C::NB_ATOMS * kk + sfb_off);
            }
          }
          ptx::tc_commit(empty_bar(stage));   // stage reusable once these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit(tfull_bar(acc));       // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 2); }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue ------------------------------------------------
    const int q = warp & 3;                       // tensor-memory lane quarter this warp may read
    const uint32_t epi_s = smem_base + C::EPI_OFF + q * C::EPI_BUFS * EPI_BLOCK_BYTES;
    uint8_t* epi_g = smem_gen + C::EPI_OFF + q * C::EPI_BUFS * EPI_BLOCK_BYTES;
    int buf = 0;
    int acc = 0; uint32_t acc_phase = 0;
    int tile_iter = 0;
    bool ok = true;
    float alpha = 1.f;
    if (KIND == KIND_NV) alpha = __ldcg(p.scale_a) * __ldcg(p.scale_b);
    constexpr int NBLK = BN / EPI_COLS;
    const int64_t m_out = p.ragged_offs != nullptr ? p.M * p.n_experts : p.M;    // rows of the output
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_iter) {
      const Tile ti = get_tile<BN>(p, t, num_m);
      const int m_blk = ti.m_blk, n_blk = ti.n_blk;
      if (!ptx::mbar_wait(tfull_bar(acc), acc_phase) || *abort_flag) { ok = false; break; }
      ptx::tc_fence_after();
      const int64_t row0 = ti.drow_off + (int64_t)m_blk * BM + q * 32, row = row0 + lane;
      const int64_t col0 = (int64_t)n_blk * BN;
      float row_scale = alpha;
      if (row_scaled(KIND)) row_scale = row < p.M ? __ldcg(p.scale_a + (p.a_scalar ? 0 : row)) : 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (acc ? C::ACC1_COL0 : 0);

      // Block order: natural, except that an overlapped accumulator 0 is read from its last
      // block down, because its LAST columns are the strip shared with accumulator 1 (whose
      // shared strip is its first columns).  The accumulator is released for the MMA after the
      // strip has been read (overlapped) or after the last block has been read (otherwise).
      constexpr int RELEASE_AFTER = C::OVERLAP ? C::OVL / EPI_COLS - 1 : NBLK - 1;
      const uint32_t release_bar = tempty_bar(acc);
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(release_bar);
      };
      if constexpr (EPI == EPI_MXQ)
        epilogue_tile_mxq<NBLK, C::EPI_BUFS, RELEASE_AFTER>(taddr, C::OVERLAP && acc == 0, row0, col0, m_out, p.N, alpha, &outs, epi_s,
                                                            epi_g, buf, lane, smem_gen + C::BAR_OFF + 256 + acc * (NBLK / 2) * 512,
                                                            smem_base + C::BAR_OFF + 256 + acc * (NBLK / 2) * 512, q, 1, release);
      else if constexpr (EPI != EPI_BF16)
        // the two warp groups swap block sets from tile to tile, so an odd block count evens out
        epilogue_tile_glu<EPI == EPI_GLU ? GLU_MX : GLU_BF16, NBLK, RELEASE_AFTER, 2>(
            taddr, C::OVERLAP && acc == 0, (((warp - 2) >> 2) + tile_iter) & 1, row, col0, p.M, p.N, alpha, p.glu, release);
      else
        epilogue_tile<row_scaled(KIND), KIND == KIND_I8, NBLK, C::EPI_BUFS, RELEASE_AFTER>(
            taddr, C::OVERLAP && acc == 0, ti.zero, row0, col0, m_out, p.N, row_scale, p.scale_b, p.b_scalar, &outs, epi_s, epi_g, buf,
            lane, release);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (lane == 0) ptx::bulk_wait<0>();           // all stores of this warp have landed
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(&g_device_status, 3); }
  }

  // Teardown.  On the abort path give copies still in flight time to land before the CTA's
  // shared memory is released.
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
              uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return B200Q_ERR_CUDA;
  cuuint64_t gdim[2] = {inner, rows};
  cuuint64_t gstride[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return B200Q_ERR_CUDA; }
  return B200Q_OK;
}

// Output buffers of one launch: [M, N] bf16 each, pitch ldd (the local one first).
struct OutSpec {
  void* ptr[kMaxOutputs];
  int count;
  int64_t scatter_rows;    // > 0: output g is [scatter_rows, N] and receives the rows g * scatter_rows ... of the result
  void* sf[kMaxOutputs];   // MXFP8-quantized output: this rank's first scale-factor tile in output g (ptr[g] are codes)
};
inline OutSpec one_output(void* D) {
  OutSpec o = {};
  o.ptr[0] = D;
  o.count = 1;
  return o;
}
// output maps: bf16 [M, N] pitch ldd, box = 64 columns x 32 rows, 128-byte swizzle
int make_out_maps(OutMaps* om, const OutSpec& outs, int64_t M, int64_t N, int64_t ldd) {
  om->count = outs.count;
  om->scatter_rows = (int)outs.scatter_rows;
  const int64_t map_rows = outs.scatter_rows > 0 ? outs.scatter_rows : M;
  for (int g = 0; g < outs.count; ++g) {
    int rc = encode_2d(&om->m[g], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, outs.ptr[g], N, map_rows, ldd * 2, EPI_COLS, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  for (int g = outs.count; g < kMaxOutputs; ++g) om->m[g] = om->m[0];
  return B200Q_OK;
}

// the same for an MXFP8-quantized output: byte matrices of codes [M, N] pitch ldc, box = 128 columns x 32 rows
int make_code_maps(OutMaps* om, const OutSpec& outs, int64_t M, int64_t N, int64_t ldc) {
  om->count = outs.count;
  om->scatter_rows = 0;
  om->sf_kt = (N / 32 + 3) / 4;
  for (int g = 0; g < outs.count; ++g) {
    int rc = encode_2d(&om->m[g], CU_TENSOR_MAP_DATA_TYPE_UINT8, outs.ptr[g], N, M, ldc, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    om->sf[g] = static_cast<uint8_t*>(outs.sf[g]);
  }
  for (int g = outs.count; g < kMaxOutputs; ++g) { om->m[g] = om->m[0]; om->sf[g] = om->sf[0]; }
  return B200Q_OK;
}

template <int KIND, int BN, int EPI = EPI_BF16>
int launch(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, GemmParams p, cudaStream_t st) {
  using C = Cfg<KIND, BN>;
  const int64_t row_bytes = KIND == KIND_NV ? p.K / 2 : p.K;
  const int64_t b_row_bytes = p.b_along_k ? row_bytes * p.n_experts : row_bytes;      // a transposed weight stack is [N, E*K]
  const int64_t m_out = p.ragged_offs != nullptr ? p.M * p.n_experts : p.M;
  CUtensorMap ma, mb;
  OutMaps md = {};
  int rc;
  // operands: byte matrices [rows, row_bytes], box = 128 bytes x tile rows, 128-byte swizzle
  if ((rc = encode_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, row_bytes, p.M, row_bytes, BKB, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, b_row_bytes, b_rows, b_row_bytes, BKB, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (EPI == EPI_MXQ) {
    if ((rc = make_code_maps(&md, D, m_out, p.N, ldd))) return rc;
  } else if (EPI != EPI_BF16) {
    md.count = 0; md.scatter_rows = 0;                       // no TMA-stored output: the epilogue writes its results itself
    for (int g = 0; g < kMaxOutputs; ++g) md.m[g] = ma;
  } else if ((rc = make_out_maps(&md, D, m_out, p.N, ldd))) {
    return rc;
  }
  p.num_m = (int)((p.M + BM - 1) / BM);
  p.num_n = (int)((p.N + BN - 1) / BN);
  p.num_k = (int)((row_bytes + BKB - 1) / BKB);
  const int64_t nblk = KIND == KIND_MX ? p.K / 32 : p.K / 16;
  p.sf_kt = (int)((nblk + 3) / 4);
  p.sf_kt_b = p.b_along_k ? p.sf_kt * p.n_experts : p.sf_kt;
  p.sfb_groups = (b_rows + 127) / 128;
  // the quantized-output epilogue stages its scale-factor atoms behind the barriers (two sets of BN / 128 atoms)
  constexpr int SMEM = C::SMEM_BYTES + (EPI == EPI_MXQ ? kSfStageBytes : 0);
  static_assert(SMEM <= kSmemBudget, "shared memory overflow");
  B200Q_CUDA(ensure_dynamic_smem(gemm_kernel<KIND, BN, EPI>, SMEM));
  const int64_t tiles = (int64_t)p.num_m * p.num_n * (p.ragged_offs != nullptr ? p.n_experts : 1);
  const int grid = (int)(tiles < kNumSMs ? tiles : kNumSMs);
  B200Q_CUDA(launch_pdl(gemm_kernel<KIND, BN, EPI>, dim3(grid), dim3(gemm_threads(EPI)), SMEM, st, ma, mb, md, p));
  return B200Q_OK;
}

int g_force_bn = 0;   // test hook: 0 = choose by shape

// Tile width by a small cost model (cycles per tile x waves): the main loop is bound by the
// tensor pipe (2*BN cycles per K step) or by the operand bytes the SM pulls from L2 per K step,
// (128+BN)*128, at ~45 B/clk per SM when all SMs load at once (about 12 TB/s in total, fitted to
// grouped and small dense shapes: the widest tile won or tied on every one of them); the
// epilogue hides behind the next main loop only when two accumulators fit in tensor memory
// (every width but 256).
template <int KIND>
int choose_bn(int64_t M, int64_t N, int64_t row_bytes, int64_t groups = 1) {
  const int cands[3] = {256, 192, 128};
  const int64_t num_k = (row_bytes + BKB - 1) / BKB, num_m = groups * ((M + BM - 1) / BM);
  double best = 1e30;
  int best_bn = 256;
  for (int bn : cands) {
    const int64_t tiles = num_m * ((N + bn - 1) / bn);
    const int64_t waves = (tiles + kNumSMs - 1) / kNumSMs;
    const double kstep = std::max(2.0 * bn, (128.0 + bn) * 128.0 / 45.0);
    const double mainloop = num_k * kstep + 600.0, epi = 300.0 + (bn / 32) * 220.0;
    // the epilogue hides behind the next main loop; at width 256 with scale factors the MMA
    // still waits for the first epilogue block(s) of the previous tile
    const double per_tile = std::max(mainloop + (bn == 256 && !row_scaled(KIND) ? 500.0 : 0.0), epi);
    const double cost = waves * per_tile;
    if (cost < best * 0.995) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

// CTA-pair form of the dense GEMMs (gemm_2cta.cu, same translation unit)
bool pair_eligible(int64_t M, int64_t N, int64_t row_bytes, bool grouped);
template <int KIND, int EPI = 0>
int launch_pair(const void* A, const void* B, const OutSpec& D, int64_t ldd, const GemmParams& gp, cudaStream_t st);
// ... and of the grouped MXFP8 forms
bool pair_grouped_eligible(const GemmParams& gp);
template <int EPI>
int launch_pair_grouped(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& gp,
                        cudaStream_t st);

// B-stationary form of the grouped fprop / dgrad GEMMs for short K (gemm_bstat.cu, same translation unit)
constexpr int kBstatNotApplicable = -1000;
template <int EPI>
int try_bstat(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& p, cudaStream_t st);
// Row-stationary pair form of the same GEMMs (gemm_rowstat.cu, same translation unit)
constexpr int kRowstatNotApplicable = -1001;
template <int EPI>
int try_rowstat(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& p, cudaStream_t st);

template <int KIND>
int dispatch(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& p, cudaStream_t st) {
  if (pair_eligible(p.M, p.N, KIND == KIND_NV ? p.K / 2 : p.K, p.tile_expert != nullptr)) return launch_pair<KIND>(A, B, D, ldd, p, st);
  const int bn = g_force_bn ? g_force_bn : choose_bn<KIND>(p.M, p.N, KIND == KIND_NV ? p.K / 2 : p.K);
  switch (bn) {
    case 128: return launch<KIND, 128>(A, B, D, ldd, b_rows, p, st);
    case 192: return launch<KIND, 192>(A, B, D, ldd, b_rows, p, st);
    case 256: return launch<KIND, 256>(A, B, D, ldd, b_rows, p, st);
    default: return B200Q_ERR_INVALID_ARG;
  }
}

// MXFP8 GEMM with the SwiGLU + MXFP8 epilogue (one-CTA kernel; every tile width is a whole number
// of 64-column epilogue blocks).
int dispatch_glu(const void* A, const void* B, int64_t b_rows, const GemmParams& p, cudaStream_t st) {
  if (pair_eligible(p.M, p.N, p.K, p.tile_expert != nullptr)) return launch_pair<KIND_MX, EPI_GLU>(A, B, OutSpec{}, 0, p, st);
  const int bn = g_force_bn ? g_force_bn : choose_bn<KIND_MX>(p.M, p.N, p.K);
  const OutSpec none = {};
  switch (bn) {
    case 128: return launch<KIND_MX, 128, EPI_GLU>(A, B, none, 0, b_rows, p, st);
    case 192: return launch<KIND_MX, 192, EPI_GLU>(A, B, none, 0, b_rows, p, st);
    case 256: return launch<KIND_MX, 256, EPI_GLU>(A, B, none, 0, b_rows, p, st);
    default: return B200Q_ERR_INVALID_ARG;
  }
}

// MXFP8 GEMM whose output leaves as MXFP8 codes + scale bytes (tile widths with an even number of 64-column blocks).
int dispatch_mxq(const void* A, const void* B, const OutSpec& D, int64_t ldc, const GemmParams& p, cudaStream_t st) {
  if (pair_eligible(p.M, p.N, p.K, false)) return launch_pair<KIND_MX, EPI_MXQ>(A, B, D, ldc, p, st);
  int bn = g_force_bn ? g_force_bn : choose_bn<KIND_MX>(p.M, p.N, p.K);
  if (bn == 192) bn = 256;
  switch (bn) {
    case 128: return launch<KIND_MX, 128, EPI_MXQ>(A, B, D, ldc, p.N, p, st);
    case 256: return launch<KIND_MX, 256, EPI_MXQ>(A, B, D, ldc, p.N, p, st);
    default: return B200Q_ERR_INVALID_ARG;
  }
}

// NVFP4 GEMM with the SwiGLU -> bf16 + amax epilogue.
int dispatch_glu_nv(const void* A, const void* B, int64_t b_rows, const GemmParams& p, cudaStream_t st) {
  if (pair_eligible(p.M, p.N, p.K / 2, false)) return launch_pair<KIND_NV, EPI_GLU_BF16>(A, B, OutSpec{}, 0, p, st);
  const int bn = g_force_bn ? g_force_bn : choose_bn<KIND_NV>(p.M, p.N, p.K / 2);
  const OutSpec none = {};
  switch (bn) {
    case 128: return launch<KIND_NV, 128, EPI_GLU_BF16>(A, B, none, 0, b_rows, p, st);
    case 192: return launch<KIND_NV, 192, EPI_GLU_BF16>(A, B, none, 0, b_rows, p, st);
    case 256: return launch<KIND_NV, 256, EPI_GLU_BF16>(A, B, none, 0, b_rows, p, st);
    default: return B200Q_ERR_INVALID_ARG;
  }
}

// Argument checks and the zeroing of scale-factor pad bytes shared by the two SwiGLU entry points.
int prepare_glu(GemmParams* p, const void* A, const void* sfA, const void* B, const void* sfB, int a_fmt, int b_fmt, int64_t M,
                int64_t N, int64_t K, void* H, int64_t ldh, void* sfH, bool zero_pads, cudaStream_t st) {
  if (A == nullptr || B == nullptr || sfA == nullptr || sfB == nullptr || H == nullptr || sfH == nullptr || M <= 0 || N <= 0 ||
      K <= 0 || ldh < N / 2 || ((a_fmt | b_fmt) & ~1))
    return B200Q_ERR_INVALID_ARG;
  if ((K & 31) || (N & 63) || (ldh & 15)) return B200Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(B) || !aligned16(H) || !aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  const int64_t hblk = N / 64;
  if (zero_pads && ((M & 127) || (hblk & 3)))
    B200Q_CUDA(memset_async(sfH, 0, (size_t)b200q_sf_bytes(M, hblk, B200Q_SF_SWIZZLE_128x4), st));
  *p = GemmParams{};
  p->sfa = (const uint8_t*)sfA; p->sfb = (const uint8_t*)sfB; p->a_fmt = a_fmt; p->b_fmt = b_fmt;
  p->M = M; p->N = N; p->K = K;
  p->glu.codes = (uint8_t*)H; p->glu.ldh = ldh; p->glu.sf = (uint8_t*)sfH; p->glu.kt = (hblk + 3) / 4;
  p->glu.wide = aligned32(H) && (ldh & 31) == 0;
  return B200Q_OK;
}

// Destination list of a fused GEMM + all-gather: rows [rank*M, rank*M + M) of every rank's gathered
// buffer, the local one first, then the peers starting with the next rank (so that at any moment
// the ranks write to different peers).
int gathered_outputs(OutSpec* o, void* const* d_all, int world, int rank, int64_t M, int64_t ldd) {
  if (d_all == nullptr || world < 1 || world > kMaxOutputs || rank < 0 || rank >= world) return B200Q_ERR_INVALID_ARG;
  *o = OutSpec{};
  o->count = world;
  for (int i = 0; i < world; ++i) {
    void* base = d_all[(rank + i) % world];
    if (base == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(base)) return B200Q_ERR_ALIGNMENT;
    o->ptr[i] = static_cast<uint8_t*>(base) + (size_t)rank * M * ldd * 2;
  }
  return B200Q_OK;
}

// Outputs of a GEMM whose result is summed over the ranks and scattered by rows: output g is this rank's slot
// (rank-th block of rows_per_owner rows) in the staging buffer of rank g, which owns rows [g * rows_per_owner, ...).
int scattered_outputs(OutSpec* o, void* const* stage_all, int world, int rank, int64_t M, int64_t ldd) {
  if (stage_all == nullptr || world < 1 || world > kMaxOutputs || rank < 0 || rank >= world) return B200Q_ERR_INVALID_ARG;
  if (M % world || (M / world) % 32) return B200Q_ERR_SHAPE;
  *o = OutSpec{};
  o->count = world;
  o->scatter_rows = M / world;
  for (int g = 0; g < world; ++g) {
    if (stage_all[g] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(stage_all[g])) return B200Q_ERR_ALIGNMENT;
    o->ptr[g] = static_cast<uint8_t*>(stage_all[g]) + (size_t)rank * o->scatter_rows * ldd * 2;
  }
  return B200Q_OK;
}

// out[r, c] = bf16(sum over the slots of float(stage[slot][r][c])), slots in order
__global__ void __launch_bounds__(256)
sum_slots_kernel(const uint16_t* __restrict__ stage, int slots, int64_t rows, int64_t cols, int64_t ld, uint16_t* __restrict__ out,
                 int64_t ldo) {
  const int64_t chunks = cols >> 3, total = rows * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks, c = (i - r * chunks) << 3;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < slots; ++s) {
      float f[8];
      unpack8(ld_nc_v4(stage + ((int64_t)s * rows + r) * ld + c), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    *reinterpret_cast<uint4*>(out + r * ldo + c) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

int check_gemm(const void* A, const void* B, const void* D, int64_t M, int64_t N, int64_t K, int64_t ldd, int kmult) {
  if (A == nullptr || B == nullptr || D == nullptr || M <= 0 || N <= 0 || K <= 0 || ldd < N) return B200Q_ERR_INVALID_ARG;
  if ((K % kmult) || (N & 7) || (ldd & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(B) || !aligned16(D)) return B200Q_ERR_ALIGNMENT;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_SHAPE;
  return require_sm100();
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

// Test hook: what every bounded wait of the kernels does when it runs out, on a wait that cannot succeed: one thread
// waits on an mbarrier that nobody ever arrives on, with a limit of `iterations` polls (a few milliseconds at most);
// when the limit is reached it records status 21 in the device status word and the kernel returns normally.  The host
// then sees B200Q_ERR_DEVICE_TIMEOUT from b200q_device_status() and the context stays usable.
}  // extern "C"
namespace b200q { namespace {
__global__ void expire_wait_kernel(int iterations) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x != 0) return;
  const uint32_t b = ptx::smem_u32(&bar);
  ptx::mbar_init(b, 1);
  ptx::fence_barrier_init();
  bool done = false;
  for (int i = 0; i < iterations && !done; ++i) {
    done = ptx::mbar_try_wait(b, 0);
    if (!done) __nanosleep(64);
  }
  if (!done) atomicExch(&g_device_status, 21);
}
} }  // namespace b200q::{anonymous}
extern "C" {
int b200q_debug_expire_wait(int iterations, void* stream) {
  PdlChain pdl_chain;
  if (iterations < 1 || iterations > 100000) return B200Q_ERR_INVALID_ARG;
  int rc = require_sm100();
  if (rc) return rc;
  expire_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(iterations);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// Test hook: force the N tile width (128, 192 or 256; 0 restores the choice by shape).
int b200q_debug_set_gemm_bn(int bn) {
  if (bn != 0 && bn != 128 && bn != 192 && bn != 256) return B200Q_ERR_INVALID_ARG;
  g_force_bn = bn;
  return B200Q_OK;
}

int b200q_gemm_fp8(const void* A, int a_fmt, const void* B, int b_fmt, const float* scale_a, int a_scale_is_scalar,
                   const float* scale_b, int b_scale_is_scalar, int64_t M, int64_t N, int64_t K, void* D, int64_t ldd,
                   void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(A, B, D, M, N, K, ldd, 16);
  if (rc) return rc;
  if (scale_a == nullptr || scale_b == nullptr || (a_fmt | b_fmt) & ~1) return B200Q_ERR_INVALID_ARG;
  GemmParams p = {};
  p.scale_a = scale_a; p.scale_b = scale_b; p.a_scalar = a_scale_is_scalar; p.b_scalar = b_scale_is_scalar;
  p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_F8>(A, B, one_output(D), ldd, N, p, (cudaStream_t)stream);
}

int b200q_gemm_int8(const void* A, const void* B, const float* scale_a, int a_scale_is_scalar, const float* scale_b,
                    int b_scale_is_scalar, int64_t M, int64_t N, int64_t K, void* D, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(A, B, D, M, N, K, ldd, 16);
  if (rc) return rc;
  if (scale_a == nullptr || scale_b == nullptr) return B200Q_ERR_INVALID_ARG;
  GemmParams p = {};
  p.scale_a = scale_a; p.scale_b = scale_b; p.a_scalar = a_scale_is_scalar; p.b_scalar = b_scale_is_scalar;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_I8>(A, B, one_output(D), ldd, N, p, (cudaStream_t)stream);
}

int b200q_gemm_mxfp8(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB, int64_t M,
                     int64_t N, int64_t K, void* D, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(A, B, D, M, N, K, ldd, 32);
  if (rc) return rc;
  if (sfA == nullptr || sfB == nullptr || (a_fmt | b_fmt) & ~1) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_MX>(A, B, one_output(D), ldd, N, p, (cudaStream_t)stream);
}

// ---- the `_gemm` seam for MXFP8 in one call ---------------------------------------------------------------------
static inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

int64_t b200q_linear_mxfp8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return align256(M * K) + align256(b200q_sf_bytes(M, K / 32, B200Q_SF_SWIZZLE_128x4)) + align256(N * K) +
         align256(b200q_sf_bytes(N, K / 32, B200Q_SF_SWIZZLE_128x4));
}

int b200q_linear_mxfp8(const void* a, int64_t a_rows, int64_t a_cols, int64_t lda, int a_axis, int a_fmt, const void* b,
                       int64_t b_rows, int64_t b_cols, int64_t ldb, int b_axis, int b_fmt, void* D, int64_t ldd, void* workspace,
                       void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(a, a_rows, a_cols, lda);
  if (rc) return rc;
  if ((rc = check_matrix(b, b_rows, b_cols, ldb))) return rc;
  if (D == nullptr || workspace == nullptr || (a_axis != 0 && a_axis != 1) || (b_axis != 0 && b_axis != 1) || ((a_fmt | b_fmt) & ~1))
    return B200Q_ERR_INVALID_ARG;
  const int64_t M = a_axis == 1 ? a_rows : a_cols, K = a_axis == 1 ? a_cols : a_rows;
  const int64_t N = b_axis == 1 ? b_rows : b_cols, Kb = b_axis == 1 ? b_cols : b_rows;
  if (K != Kb || ldd < N) return B200Q_ERR_INVALID_ARG;
  if ((K & 31) || (N & 7) || (ldd & 7)) return B200Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(D) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int swz = B200Q_SF_SWIZZLE_128x4;
  uint8_t* ca = static_cast<uint8_t*>(workspace);
  uint8_t* sfa = ca + align256(M * K);
  uint8_t* cb = sfa + align256(b200q_sf_bytes(M, K / 32, swz));
  uint8_t* sfb = cb + align256(N * K);
  if ((rc = zero_sf_pads(sfa, M, K / 32, swz, st))) return rc;
  if ((rc = zero_sf_pads(sfb, N, K / 32, swz, st))) return rc;
  const uint16_t* xa = static_cast<const uint16_t*>(a);
  const uint16_t* xb = static_cast<const uint16_t*>(b);
  if (a_axis == 1 && b_axis == 1 && a_fmt == b_fmt) {
    // both operands have K contiguous (fprop of a linear layer): one launch quantizes the two of them
    // the GEMM is launched directly behind this kernel, with the attribute: the quantizer may let it set up early
    const RowQuantJob ja = {xa, a_rows, a_cols, lda, ca, sfa, nullptr, pdl_enabled() ? 1 : 0}, jb = {xb, b_rows, b_cols, ldb, cb, sfb, nullptr, 0};
    launch_rowwise_block<MODE_MX>(ja, jb, a_fmt, swz, nullptr, nullptr, st);
  } else {
    if (a_axis == 1) launch_rowwise_block<MODE_MX>(xa, a_rows, a_cols, lda, a_fmt, ca, sfa, swz, nullptr, nullptr, st);
    else launch_transpose<MODE_MX>(xa, a_rows, a_cols, lda, a_fmt, ca, sfa, swz, nullptr, nullptr, nullptr, st);
    if (b_axis == 1) launch_rowwise_block<MODE_MX>(xb, b_rows, b_cols, ldb, b_fmt, cb, sfb, swz, nullptr, nullptr, st);
    else launch_transpose<MODE_MX>(xb, b_rows, b_cols, ldb, b_fmt, cb, sfb, swz, nullptr, nullptr, nullptr, st);
  }
  B200Q_CUDA(cudaGetLastError());
  GemmParams p = {};
  p.sfa = sfa; p.sfb = sfb; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_MX>(ca, cb, one_output(D), ldd, N, p, st);
}

int b200q_gemm_nvfp4(const void* A, const void* sfA, const void* B, const void* sfB, const float* tsA, const float* tsB,
                     int64_t M, int64_t N, int64_t K, void* D, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(A, B, D, M, N, K, ldd, 32);
  if (rc) return rc;
  if (sfA == nullptr || sfB == nullptr || tsA == nullptr || tsB == nullptr) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.scale_a = tsA; p.scale_b = tsB;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_NV>(A, B, one_output(D), ldd, N, p, (cudaStream_t)stream);
}

int b200q_grouped_gemm_mxfp8(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB,
                             const int32_t* tile_expert, const int32_t* num_tiles, int64_t padded_rows, int E, int64_t N,
                             int64_t K, void* D, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(A, B, D, padded_rows, N, K, ldd, 32);
  if (rc) return rc;
  if (sfA == nullptr || sfB == nullptr || tile_expert == nullptr || num_tiles == nullptr || E <= 0 || (a_fmt | b_fmt) & ~1)
    return B200Q_ERR_INVALID_ARG;
  // N % 128: expert e's rows of B start at e*N, which must be the start of a 128-row scale-factor group
  if ((padded_rows & 127) || (N & 127) || (int64_t)E * N > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = padded_rows; p.N = N; p.K = K; p.tile_expert = tile_expert; p.num_tiles = num_tiles; p.n_experts = E;
  rc = try_rowstat<EPI_BF16>(A, B, one_output(D), ldd, (int64_t)E * N, p, (cudaStream_t)stream);
  if (rc != kRowstatNotApplicable) return rc;
  rc = try_bstat<EPI_BF16>(A, B, one_output(D), ldd, (int64_t)E * N, p, (cudaStream_t)stream);
  if (rc != kBstatNotApplicable) return rc;
  if (pair_grouped_eligible(p)) return launch_pair_grouped<EPI_BF16>(A, B, one_output(D), ldd, (int64_t)E * N, p, (cudaStream_t)stream);
  return dispatch<KIND_MX>(A, B, one_output(D), ldd, (int64_t)E * N, p, (cudaStream_t)stream);
}

int b200q_gemm_mxfp8_swiglu(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB, int64_t M,
                            int64_t N, int64_t K, void* H, int64_t ldh, void* sfH, void* stream) {
  PdlChain pdl_chain;
  GemmParams p;
  int rc = prepare_glu(&p, A, sfA, B, sfB, a_fmt, b_fmt, M, N, K, H, ldh, sfH, true, (cudaStream_t)stream);
  if (rc) return rc;
  return dispatch_glu(A, B, N, p, (cudaStream_t)stream);
}

int b200q_grouped_gemm_mxfp8_swiglu(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB,
                                    const int32_t* tile_expert, const int32_t* num_tiles, int64_t padded_rows, int E, int64_t N,
                                    int64_t K, void* H, int64_t ldh, void* sfH, void* stream) {
  PdlChain pdl_chain;
  if (tile_expert == nullptr || num_tiles == nullptr || E <= 0) return B200Q_ERR_INVALID_ARG;
  if ((padded_rows & 127) || (N & 127) || (int64_t)E * N > INT32_MAX) return B200Q_ERR_SHAPE;
  GemmParams p;
  int rc = prepare_glu(&p, A, sfA, B, sfB, a_fmt, b_fmt, padded_rows, N, K, H, ldh, sfH, true, (cudaStream_t)stream);
  if (rc) return rc;
  p.tile_expert = tile_expert; p.num_tiles = num_tiles; p.n_experts = E;
  rc = try_rowstat<EPI_GLU>(A, B, OutSpec{}, 0, (int64_t)E * N, p, (cudaStream_t)stream);
  if (rc != kRowstatNotApplicable) return rc;
  rc = try_bstat<EPI_GLU>(A, B, OutSpec{}, 0, (int64_t)E * N, p, (cudaStream_t)stream);
  if (rc != kBstatNotApplicable) return rc;
  if (pair_grouped_eligible(p)) return launch_pair_grouped<EPI_GLU>(A, B, OutSpec{}, 0, (int64_t)E * N, p, (cudaStream_t)stream);
  return dispatch_glu(A, B, (int64_t)E * N, p, (cudaStream_t)stream);
}

int b200q_gemm_nvfp4_swiglu(const void* A, const void* sfA, const void* B, const void* sfB, const float* tsA, const float* tsB,
                            int64_t M, int64_t N, int64_t K, void* H, int64_t ldh, float* amax_out, void* stream) {
  PdlChain pdl_chain;
  if (A == nullptr || B == nullptr || sfA == nullptr || sfB == nullptr || tsA == nullptr || tsB == nullptr || H == nullptr ||
      amax_out == nullptr || M <= 0 || N <= 0 || K <= 0 || ldh < N / 2)
    return B200Q_ERR_INVALID_ARG;
  if ((K & 31) || (N & 63) || (ldh & 7)) return B200Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(B) || !aligned16(H) || !aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  B200Q_CUDA(zero_before_kernel(amax_out, sizeof(float), st));
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.scale_a = tsA; p.scale_b = tsB;
  p.M = M; p.N = N; p.K = K;
  p.glu.codes = (uint8_t*)H; p.glu.ldh = ldh * 2; p.glu.amax = amax_out;
  p.glu.wide = aligned32(H) && ((ldh * 2) & 31) == 0;
  return dispatch_glu_nv(A, B, N, p, st);
}

// the grouped backward forms: CTA pairs when the shape allows, else the one-CTA kernel with the tile width of the cost model
static int dispatch_one_cta_mx(const void* A, const void* B, void* D, int64_t ldd, int64_t b_rows, const GemmParams& p,
                               cudaStream_t st) {
  int rc = try_rowstat<EPI_BF16>(A, B, one_output(D), ldd, b_rows, p, st);          // dgrad with a short K; never the ragged wgrad
  if (rc != kRowstatNotApplicable) return rc;
  rc = try_bstat<EPI_BF16>(A, B, one_output(D), ldd, b_rows, p, st);
  if (rc != kBstatNotApplicable) return rc;
  if (pair_grouped_eligible(p)) return launch_pair_grouped<EPI_BF16>(A, B, one_output(D), ldd, b_rows, p, st);
  // ragged form: every expert has its own output tiles and (on average) its share of the K range
  const int64_t groups = p.ragged_offs ? p.n_experts : 1;
  const int bn = g_force_bn ? g_force_bn : choose_bn<KIND_MX>(p.M, p.N, p.K / groups, groups);
  switch (bn) {
    case 128: return launch<KIND_MX, 128>(A, B, one_output(D), ldd, b_rows, p, st);
    case 192: return launch<KIND_MX, 192>(A, B, one_output(D), ldd, b_rows, p, st);
    case 256: return launch<KIND_MX, 256>(A, B, one_output(D), ldd, b_rows, p, st);
    default: return B200Q_ERR_INVALID_ARG;
  }
}

int b200q_grouped_gemm_mxfp8_dgrad(const void* A, int a_fmt, const void* sfA, const void* Bt, int b_fmt, const void* sfBt,
                                   const int32_t* tile_expert, const int32_t* num_tiles, int64_t padded_rows, int E, int64_t N,
                                   int64_t K, void* D, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(A, Bt, D, padded_rows, N, K, ldd, 128);
  if (rc) return rc;
  if (sfA == nullptr || sfBt == nullptr || tile_expert == nullptr || num_tiles == nullptr || E <= 0 || (a_fmt | b_fmt) & ~1)
    return B200Q_ERR_INVALID_ARG;
  if ((padded_rows & 127) || (int64_t)E * K > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(sfA) || !aligned16(sfBt)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfBt; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = padded_rows; p.N = N; p.K = K; p.tile_expert = tile_expert; p.num_tiles = num_tiles;
  p.b_along_k = 1; p.n_experts = E;
  return dispatch_one_cta_mx(A, Bt, D, ldd, N, p, (cudaStream_t)stream);
}

int b200q_grouped_gemm_mxfp8_wgrad(const void* At, int a_fmt, const void* sfAt, const void* Bt, int b_fmt, const void* sfBt,
                                   const int32_t* padded_offs, int E, int64_t M, int64_t N, int64_t padded_rows, void* D,
                                   int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  int rc = check_gemm(At, Bt, D, M, N, padded_rows, ldd, 128);
  if (rc) return rc;
  if (sfAt == nullptr || sfBt == nullptr || padded_offs == nullptr || E <= 0 || (a_fmt | b_fmt) & ~1) return B200Q_ERR_INVALID_ARG;
  if ((M & 127) || (int64_t)E * M > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(sfAt) || !aligned16(sfBt)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfAt; p.sfb = (const uint8_t*)sfBt; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = M; p.N = N; p.K = padded_rows; p.ragged_offs = padded_offs; p.n_experts = E;
  return dispatch_one_cta_mx(At, Bt, D, ldd, N, p, (cudaStream_t)stream);
}

int b200q_gemm_fp8_allgather(const void* A, int a_fmt, const void* B, int b_fmt, const float* scale_a, int a_scale_is_scalar,
                             const float* scale_b, int b_scale_is_scalar, int64_t M, int64_t N, int64_t K, void* const* D_all,
                             int world, int rank, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  OutSpec outs;
  int rc = gathered_outputs(&outs, D_all, world, rank, M, ldd);
  if (rc) return rc;
  if ((rc = check_gemm(A, B, outs.ptr[0], M, N, K, ldd, 16))) return rc;
  if (scale_a == nullptr || scale_b == nullptr || (a_fmt | b_fmt) & ~1) return B200Q_ERR_INVALID_ARG;
  GemmParams p = {};
  p.scale_a = scale_a; p.scale_b = scale_b; p.a_scalar = a_scale_is_scalar; p.b_scalar = b_scale_is_scalar;
  p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_F8>(A, B, outs, ldd, N, p, (cudaStream_t)stream);
}

int b200q_gemm_mxfp8_allgather(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB, int64_t M,
                               int64_t N, int64_t K, void* const* D_all, int world, int rank, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  OutSpec outs;
  int rc = gathered_outputs(&outs, D_all, world, rank, M, ldd);
  if (rc) return rc;
  if ((rc = check_gemm(A, B, outs.ptr[0], M, N, K, ldd, 32))) return rc;
  if (sfA == nullptr || sfB == nullptr || (a_fmt | b_fmt) & ~1) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_MX>(A, B, outs, ldd, N, p, (cudaStream_t)stream);
}

int b200q_gemm_mxfp8_allgather_mxfp8(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB, int64_t M,
                                     int64_t N, int64_t K, void* const* C_all, void* const* SF_all, int world, int rank,
                                     int64_t ldc, void* stream) {
  PdlChain pdl_chain;
  if (A == nullptr || B == nullptr || sfA == nullptr || sfB == nullptr || C_all == nullptr || SF_all == nullptr || M <= 0 || N <= 0 ||
      K <= 0 || ldc < N || world < 1 || world > kMaxOutputs || rank < 0 || rank >= world || ((a_fmt | b_fmt) & ~1))
    return B200Q_ERR_INVALID_ARG;
  // whole 128-row scale-factor tiles per rank, whole 128-column chunks (4 scale bytes) per row
  if ((M & 127) || (N & 127) || (K & 31) || (ldc & 15)) return B200Q_ERR_SHAPE;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || (int64_t)world * M > INT32_MAX) return B200Q_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(B) || !aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  OutSpec outs = {};
  outs.count = world;
  const int64_t sf_kt = (N / 32 + 3) / 4;
  for (int i = 0; i < world; ++i) {                     // the local copy first, then the peers starting with the next rank
    const int g = (rank + i) % world;
    if (C_all[g] == nullptr || SF_all[g] == nullptr) return B200Q_ERR_INVALID_ARG;
    if (!aligned16(C_all[g]) || !aligned16(SF_all[g])) return B200Q_ERR_ALIGNMENT;
    outs.ptr[i] = static_cast<uint8_t*>(C_all[g]) + (size_t)rank * M * ldc;
    outs.sf[i] = static_cast<uint8_t*>(SF_all[g]) + (size_t)rank * (M / 128) * sf_kt * 512;
  }
  int rc = require_sm100();
  if (rc) return rc;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = M; p.N = N; p.K = K;
  return dispatch_mxq(A, B, outs, ldc, p, (cudaStream_t)stream);
}

int b200q_gemm_mxfp8_scatter(const void* A, int a_fmt, const void* sfA, const void* B, int b_fmt, const void* sfB, int64_t M,
                             int64_t N, int64_t K, void* const* stage_all, int world, int rank, int64_t ldd, void* stream) {
  PdlChain pdl_chain;
  OutSpec outs;
  int rc = scattered_outputs(&outs, stage_all, world, rank, M, ldd);
  if (rc) return rc;
  if ((rc = check_gemm(A, B, outs.ptr[0], M, N, K, ldd, 32))) return rc;
  if (sfA == nullptr || sfB == nullptr || (a_fmt | b_fmt) & ~1) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_MX>(A, B, outs, ldd, N, p, (cudaStream_t)stream);
}

int b200q_sum_slots(const void* stage, int slots, int64_t rows, int64_t cols, int64_t ld, void* out, int64_t ldo, void* stream) {
  PdlChain pdl_chain;
  if (stage == nullptr || out == nullptr || slots < 1 || rows <= 0 || cols <= 0 || ld < cols || ldo < cols) return B200Q_ERR_INVALID_ARG;
  if ((cols & 7) || (ld & 7) || (ldo & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(stage) || !aligned16(out)) return B200Q_ERR_ALIGNMENT;
  int rc = require_sm100();
  if (rc) return rc;
  const int64_t want = (rows * (cols >> 3) + 255) / 256, cap = (int64_t)kNumSMs * 8;
  sum_slots_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, (cudaStream_t)stream>>>(
      (const uint16_t*)stage, slots, rows, cols, ld, (uint16_t*)out, ldo);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_gemm_nvfp4_allgather(const void* A, const void* sfA, const void* B, const void* sfB, const float* tsA, const float* tsB,
                               int64_t M, int64_t N, int64_t K, void* const* D_all, int world, int rank, int64_t ldd,
                               void* stream) {
  PdlChain pdl_chain;
  OutSpec outs;
  int rc = gathered_outputs(&outs, D_all, world, rank, M, ldd);
  if (rc) return rc;
  if ((rc = check_gemm(A, B, outs.ptr[0], M, N, K, ldd, 32))) return rc;
  if (sfA == nullptr || sfB == nullptr || tsA == nullptr || tsB == nullptr) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(sfA) || !aligned16(sfB)) return B200Q_ERR_ALIGNMENT;
  GemmParams p = {};
  p.sfa = (const uint8_t*)sfA; p.sfb = (const uint8_t*)sfB; p.scale_a = tsA; p.scale_b = tsB;
  p.M = M; p.N = N; p.K = K;
  return dispatch<KIND_NV>(A, B, outs, ldd, N, p, (cudaStream_t)stream);
}

}  // extern "C"
