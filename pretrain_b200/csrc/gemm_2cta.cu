// The dense GEMMs of gemm.cu on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster share one
// 256-row x 256-column output tile.  Each CTA stages only its own 128 rows of A and its own 128
// rows of B per K step (32 KB instead of the 48 KB a lone CTA needs for 128 x 256), which cuts the
// L2 -> shared-memory traffic and the shared-memory reads per FLOP by a third and leaves room for
// a deeper ring.  The leader CTA (cluster rank 0) issues the MMAs for the pair; each CTA keeps its
// 128 accumulator rows in its own tensor memory and runs its own epilogue.
//
// Differences from the one-CTA kernel, all of them about who signals whom:
//   * every TMA load (operands and scale-factor atoms, the latter through a 2-D view of the
//     scale buffers, 256 bytes per row) counts its bytes on the LEADER's "full" barrier, on which
//     both producers also arrive;
//   * the leader's tcgen05.commit arrives on the "empty" / "accumulator full" barriers of both CTAs;
//   * the peer's epilogue warps arrive remotely on the leader's "accumulator free" barrier;
//   * the pair synchronizes as a cluster after barrier set-up and before tear-down.
// No TMA multicast is used.
//
// GROUPED: the three ragged MoE forms of gemm.cu (rows of A grouped by expert; the transposed weight
// stack along K; per-expert K ranges) on the same pairs.  Expert segments are whole 128-row tiles,
// not 256-row ones, so the pair tiles are formed INSIDE each expert: expert e with n tiles gets
// ceil(n / 2) pair tiles, and when n is odd the second CTA of the last pair has no rows of its own -
// it still stages its half of B (the first CTA's MMA reads it) but stores nothing.  Every CTA builds
// the (first tile, pair-tile prefix) table of the experts in shared memory from tile_expert at start.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200q {
namespace {

namespace pair {

constexpr int PBN = 256;                          // columns of the pair's tile
constexpr int HALF_N = PBN / 2;                   // B rows each CTA stages

constexpr int kPairMaxExperts = 256;
constexpr int kGroupTableBytes = 2 * (kPairMaxExperts + 1) * 4 + 248;     // first tile + pair prefix per expert, 256-aligned

template <int KIND, bool GROUPED = false>
struct PCfg {
  static constexpr int K_ATOMS = KIND == KIND_NV ? 4 : 1;
  static constexpr int A_BYTES = BM * BKB, B_BYTES = HALF_N * BKB;
  static constexpr int SFA_BYTES = row_scaled(KIND) ? 0 : K_ATOMS * 512;
  static constexpr int SFB_BYTES = row_scaled(KIND) ? 0 : 2 * K_ATOMS * 512;       // both halves of B's columns
  static constexpr int TX_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;      // per CTA and K step
  static constexpr int STAGE_BYTES = ((TX_BYTES + 1023) / 1024) * 1024;
  static constexpr int EPI_BYTES = 2 * kEpiBytes1;
  static constexpr int GRP_BYTES = GROUPED ? kGroupTableBytes : 0;
  static constexpr int STAGES_RAW = (kSmemBudget - 2048 - GRP_BYTES - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SFA_COLS = row_scaled(KIND) ? 0 : 4 * K_ATOMS;
  static constexpr int SFB_COLS = row_scaled(KIND) ? 0 : 8 * K_ATOMS;
  static constexpr int SF_COLS = SFA_COLS + SFB_COLS;
  static constexpr bool OVERLAP = SF_COLS > 0;     // two 256-column accumulators + scale columns > 512
  static constexpr int OVL = OVERLAP ? ((SF_COLS + EPI_COLS - 1) / EPI_COLS) * EPI_COLS : 0;
  static constexpr int ACC1_COL0 = PBN - OVL;
  static constexpr int SFA_COL0 = 2 * PBN - OVL;
  static constexpr int SFB_COL0 = SFA_COL0 + SFA_COLS;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = EPI_OFF + EPI_BYTES;
  static constexpr int GRP_OFF = BAR_OFF + 256;
  static constexpr int SMEM_BYTES = BAR_OFF + 256 + GRP_BYTES + 1024;
  static_assert(SFB_COL0 + SFB_COLS <= 512, "tensor memory overflow");
  static_assert(SMEM_BYTES <= kSmemBudget, "shared memory overflow");
};

struct PairParams {
  const float* scale_a;
  const float* scale_b;
  int a_scalar, b_scalar, a_fmt, b_fmt;
  int64_t M, N;
  int num_mp, num_n, num_k;      // pair tiles (256 rows), column tiles, K steps
  int sf_kt;                     // 512-byte scale atoms per 128-row group along K
  GluOut glu;                    // SwiGLU epilogues: where they write
  // GROUPED only (see GemmParams): M = padded rows (fprop, dgrad) or rows per expert (wgrad); N per expert
  const int32_t* tile_expert;    // fprop / dgrad: expert of every 128-row tile of A
  const int32_t* num_tiles;      //                128-row tiles in use (device)
  int num_m128;                  //                upper bound of that count
  const int32_t* ragged_offs;    // wgrad: K range of every expert
  int n_experts;
  int b_along_k;                 // dgrad: B is [N, E*K]
  int sf_kt_b;                   // scale atoms per row group of B
  int64_t K;                     // contraction length per expert (bytes), dgrad's K offset unit
  int raster_gm;                 // dense form: pair-tile rows per raster group
};

// Everything the roles of one CTA need to know about pair tile t.
struct PTile {
  int row0;            // this CTA's first row of A
  int n_blk;
  int k0, nk;          // first K step, number of K steps
  int brow0;           // this CTA's first row of B
  int bgroup;          // first 128-row scale group of the pair's B tile
  int bk0;             // K offset of B (bytes)
  int sfb_k0;          // first scale atom of B along K
  int64_t drow_off;    // row offset of the output
  bool zero;           // expert without rows (wgrad): no K step runs, the epilogue stores zeros
  bool live;           // this CTA owns output rows
};

// Raster: groups of GM pair-tile rows, inside a group the row index runs fastest.  The pairs that are resident together
// then share GM tiles of A and about 74 / GM tiles of B through L2, and over a whole group A is read from DRAM once
// and B once per group: the larger GM, the fewer re-reads of B, as long as the group's rows of A stay in L2.
__device__ __forceinline__ void pair_tile_coords(int t, int num_mp, int num_n, int& mp, int& n, int GM = 8) {
  const int per_group = GM * num_n;
  const int g = t / per_group, r = t - g * per_group;
  const int first = g * GM;
  const int gm = num_mp - first < GM ? num_mp - first : GM;
  mp = first + r % gm;
  n = r / gm;
}

template <bool GROUPED>
__device__ __forceinline__ PTile get_ptile(const PairParams& p, int t, int total_pt, int cta, const int* g_first, const int* g_pairs) {
  PTile ti;
  ti.k0 = 0; ti.nk = p.num_k; ti.bk0 = 0; ti.sfb_k0 = 0; ti.drow_off = 0; ti.zero = false;
  int mp;
  if (!GROUPED) {
    pair_tile_coords(t, p.num_mp, p.num_n, mp, ti.n_blk, p.raster_gm);
    ti.row0 = mp * 256 + cta * BM;
    ti.live = true;                                   // rows beyond M are clipped by the epilogue
    ti.brow0 = ti.n_blk * PBN + cta * HALF_N;
    ti.bgroup = ti.n_blk * 2;
  } else if (p.ragged_offs != nullptr) {
    const int per = p.num_mp * p.num_n;
    const int e = t / per;
    pair_tile_coords(t - e * per, p.num_mp, p.num_n, mp, ti.n_blk);
    ti.row0 = mp * 256 + cta * BM;
    ti.live = ti.row0 < p.M;
    ti.brow0 = ti.n_blk * PBN + cta * HALF_N;
    ti.bgroup = ti.n_blk * 2;
    const int r0 = __ldcg(p.ragged_offs + e), r1 = __ldcg(p.ragged_offs + e + 1);
    ti.k0 = r0 >> 7;
    ti.nk = (r1 - r0) >> 7;
    if (ti.nk <= 0) {                                 // no rows: nothing is loaded or multiplied, zeros are stored
      ti.nk = 0;
      ti.zero = true;
    }
    ti.drow_off = (int64_t)e * p.M;
  } else {
    int pt;
    pair_tile_coords(t, total_pt, p.num_n, pt, ti.n_blk);
    int lo = 0, hi = p.n_experts - 1;                 // last expert whose first pair tile is <= pt
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (g_pairs[mid] <= pt) lo = mid; else hi = mid - 1;
    }
    const int e = lo, tile0 = g_first[e] + 2 * (pt - g_pairs[e]);
    ti.row0 = (tile0 + cta) * BM;
    ti.live = cta == 0 || tile0 + 1 < g_first[e + 1];
    ti.brow0 = ti.n_blk * PBN + cta * HALF_N;
    ti.bgroup = ti.n_blk * 2;
    if (p.b_along_k) {
      ti.bk0 = (int)(e * p.K);
      ti.sfb_k0 = e * p.sf_kt;
    } else {
      ti.brow0 += e * (int)p.N;
      ti.bgroup += (int)((e * p.N) >> 7);
    }
  }
  return ti;
}

// The (first tile, pair-tile prefix) table of the experts, built by all THREADS threads of a CTA in shared memory:
// g_first[e] = first 128-row tile of expert e (an expert without tiles starts where the next one does; entry E = tiles in
// use), g_pairs[e] = pair tiles of the experts before e (entry E = their total).  Returns the tiles in use.
template <int THREADS>
__device__ __forceinline__ int build_expert_pairs(const int32_t* tile_expert, const int32_t* num_tiles, int num_m128, int n_experts,
                                                  int* g_first, int* g_pairs) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int live_tiles = __ldcg(num_tiles);
  live_tiles = live_tiles < num_m128 ? live_tiles : num_m128;
  for (int e = threadIdx.x; e <= n_experts; e += THREADS) g_first[e] = e == n_experts ? live_tiles : 0x7fffffff;
  __syncthreads();
  for (int t = threadIdx.x; t < live_tiles; t += THREADS) {
    const int e = __ldcg(tile_expert + t), prev = t > 0 ? __ldcg(tile_expert + t - 1) : -1;
    if (e != prev && e >= 0 && e < n_experts) g_first[e] = t;
  }
  __syncthreads();
  if (warp == 0) {
    // suffix minimum (an expert without tiles starts where the next one does), pair-tile counts, their prefix sums
    constexpr int PER = kPairMaxExperts / 32;
    const int E = n_experts, base = lane * PER;
    int v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = base + i < E ? g_first[base + i] : live_tiles;
#pragma unroll
    for (int i = PER - 2; i >= 0; --i) v[i] = v[i] < v[i + 1] ? v[i] : v[i + 1];
    int suf = v[0];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_down_sync(0xffffffffu, suf, o);
      if (lane + o < 32 && x < suf) suf = x;
    }
    int later = __shfl_down_sync(0xffffffffu, suf, 1);       // minimum over all later lanes
    if (lane == 31) later = live_tiles;
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = v[i] < later ? v[i] : later;
    int next0 = __shfl_down_sync(0xffffffffu, v[0], 1);
    if (lane == 31) next0 = live_tiles;
    int cnt[PER], sum = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int end = i + 1 < PER ? v[i + 1] : next0;
      cnt[i] = base + i < E ? (end - v[i] + 1) >> 1 : 0;
      sum += cnt[i];
    }
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += x;
    }
    int run = inc - sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (base + i < E) { g_first[base + i] = v[i]; g_pairs[base + i] = run; }
      run += cnt[i];
    }
    if (lane == 31) g_pairs[E] = inc;
  }
  __syncthreads();
  return live_tiles;
}

}  // namespace pair

template <int KIND, int EPI, bool GROUPED = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm_threads(EPI), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                 const __grid_constant__ OutMaps outs, const pair::PairParams p) {
  using C = pair::PCfg<KIND, GROUPED>;
  constexpr int BN = pair::PBN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // used in the leader only
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };        // one per CTA
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + a); };    // one per CTA
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + 2 + a); };   // used in the leader only
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + C::BAR_OFF + 8 * (2 * C::STAGES + 4));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = ptx::cluster_ctarank();       // 0 = leader
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  int* g_first = reinterpret_cast<int*>(smem_gen + C::GRP_OFF);        // GROUPED: first 128-row tile of every expert (+ end)
  int* g_pairs = g_first + pair::kPairMaxExperts + 1;                   //          pair tiles before every expert (+ total)
  const bool by_expert = GROUPED && p.tile_expert != nullptr;
  if (GROUPED) grid_dependency_wait();            // the grouped forms read the permute plan's tables right away
  if (by_expert) pair::build_expert_pairs<gemm_threads(EPI)>(p.tile_expert, p.num_tiles, p.num_m128, p.n_experts, g_first, g_pairs);
  const int total_pt = by_expert ? g_pairs[p.n_experts] : 0;
  const int total_tiles = by_expert ? total_pt * p.num_n
                                    : p.num_mp * p.num_n * (GROUPED && p.ragged_offs != nullptr ? p.n_experts : 1);

  if (threadIdx.x == 0) {
    // full: one arrival (with its byte count) per producer of the pair; empty / accumulator-full: the
    // leader's commit; accumulator-free: every epilogue warp (4 or 8) of each CTA
    for (int s = 0; s < C::STAGES; ++s) { ptx::mbar_init(full_bar(s), 2); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), 2 * (gemm_threads(EPI) / 32 - 2)); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    for (int g = 0; g < outs.count; ++g) ptx::prefetch_tensormap(&outs.m[g]);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();            // both CTAs' barriers exist before anyone signals the peer
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (!GROUPED) grid_dependency_wait();           // operands, scales and the output buffer belong to earlier kernels until here

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ---------------------------------
    if (ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        const pair::PTile ti = pair::get_ptile<GROUPED>(p, t, total_pt, (int)cta, g_first, g_pairs);
        const int row0 = ti.row0;                                    // this CTA's rows of A
        const int brow0 = ti.brow0;                                  // this CTA's rows of B
        for (int kl = 0; kl < ti.nk; ++kl) {
          const int k = ti.k0 + kl;
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          const uint32_t fb = full_bar(stage) & ptx::kLeaderMask;    // the leader's barrier, from either CTA
          ptx::mbar_expect_tx_cluster(fb, C::TX_BYTES);
          ptx::tma_load_2d_pair(sa, &tmap_a, k * BKB, row0, fb);
          ptx::tma_load_2d_pair(sb, &tmap_b, k * BKB + ti.bk0, brow0, fb);
          if (!row_scaled(KIND)) {
            // scale buffers viewed as rows of 256 bytes: a 512-byte atom is 2 rows, the K_ATOMS atoms of
            // one K step and row group are contiguous
            const uint32_t ssfa = sb + C::B_BYTES, ssfb = ssfa + C::SFA_BYTES;
            const int sf_kt = p.sf_kt, sf_kt_b = GROUPED ? p.sf_kt_b : p.sf_kt;
            ptx::tma_load_2d_pair(ssfa, &tmap_sfa, 0, 2 * ((row0 >> 7) * sf_kt + k * C::K_ATOMS), fb);
#pragma unroll
            for (int j = 0; j < 2; ++j)
              ptx::tma_load_2d_pair(ssfb + j * C::K_ATOMS * 512, &tmap_sfb, 0,
                                    2 * ((ti.bgroup + j) * sf_kt_b + ti.sfb_k0 + k * C::K_ATOMS), fb);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 11); }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------
    if (cta == 0 && ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++tile_iter) {
        if (C::OVERLAP) {
          if (tile_iter > 0 && (!ptx::mbar_wait(tempty_bar(acc ^ 1), ((tile_iter - 1) >> 1) & 1) || *abort_flag)) { ok = false; break; }
        } else {
          if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1) || *abort_flag) { ok = false; break; }
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc ? C::ACC1_COL0 : 0);
        // only the ragged form has a K range per tile; the others need no tile lookup here
        const int nk = GROUPED && p.ragged_offs != nullptr ? pair::get_ptile<GROUPED>(p, t, total_pt, 0, g_first, g_pairs).nk : p.num_k;
        for (int k = 0; k < nk; ++k) {
          if (!ptx::mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          if (!row_scaled(KIND)) {
            const uint32_t ssfa = sb + C::B_BYTES, ssfb = ssfa + C::SFA_BYTES;
#pragma unroll
            for (int a = 0; a < C::K_ATOMS; ++a) {
              ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + C::SFA_COL0 + 4 * a, ptx::smem_desc_sf(ssfa + a * 512));
#pragma unroll
              for (int j = 0; j < 2; ++j)
                ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + C::SFB_COL0 + 4 * (a * 2 + j),
                                                 ptx::smem_desc_sf(ssfb + (j * C::K_ATOMS + a) * 512));
            }
          }
          const uint64_t da = ptx::smem_desc_k_sw128(sa), db = ptx::smem_desc_k_sw128(sb);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t accum = (k | kk) != 0;
            const uint64_t adv = (uint64_t)(kk * 32 >> 4);
            if (KIND == KIND_I8) {
              ptx::mma_i8_pair(d_tmem, da + adv, db + adv, ptx::idesc_i8(256, BN), accum);
            } else if (KIND == KIND_F8) {
              ptx::mma_f8_pair(d_tmem, da + adv, db + adv, ptx::idesc_f8(p.a_fmt, p.b_fmt, 256, BN), accum);
            } else if (KIND == KIND_MX) {
              ptx::mma_mxf8_pair(d_tmem, da + adv, db + adv, ptx::idesc_block_scaled(p.a_fmt, p.b_fmt, 1, 256, BN, kk), accum,
                                 tmem_base + C::SFA_COL0, tmem_base + C::SFB_COL0);
            } else {
              ptx::mma_nvf4_pair(d_tmem, da + adv, db + adv, ptx::idesc_block_scaled(1, 1, 0, 256, BN, 0), accum,
                                 tmem_base + C::SFA_COL0 + 4 * kk, tmem_base + C::SFB_COL0 + 8 * kk);
            }
          }
          ptx::tc_commit_pair(empty_bar(stage));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit_pair(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 12); }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (both CTAs, own 128 rows) ------------------------
    const int q = warp & 3;
    const uint32_t epi_s = smem_base + C::EPI_OFF + q * 2 * EPI_BLOCK_BYTES;
    uint8_t* epi_g = smem_gen + C::EPI_OFF + q * 2 * EPI_BLOCK_BYTES;
    int buf = 0;
    int acc = 0; uint32_t acc_phase = 0;
    int tile_iter = 0;
    bool ok = true;
    float alpha = 1.f;
    if (KIND == KIND_NV) alpha = __ldcg(p.scale_a) * __ldcg(p.scale_b);
    constexpr int NBLK = BN / EPI_COLS;
    for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++tile_iter) {
      const pair::PTile ti = pair::get_ptile<GROUPED>(p, t, total_pt, (int)cta, g_first, g_pairs);
      if (!ptx::mbar_wait(tfull_bar(acc), acc_phase) || *abort_flag) { ok = false; break; }
      ptx::tc_fence_after();
      const int64_t row0 = ti.drow_off + ti.row0 + q * 32, row = row0 + lane;
      const int64_t col0 = (int64_t)ti.n_blk * BN;
      // rows this CTA may store: none for the idle half of an expert's odd last pair
      const int64_t m_lim = !ti.live ? 0 : (GROUPED && p.ragged_offs != nullptr ? ti.drow_off + p.M : p.M);
      float row_scale = alpha;
      if (row_scaled(KIND)) row_scale = row < p.M ? __ldcg(p.scale_a + (p.a_scalar ? 0 : row)) : 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (acc ? C::ACC1_COL0 : 0);

      constexpr int RELEASE_AFTER = C::OVERLAP ? C::OVL / EPI_COLS - 1 : NBLK - 1;
      const uint32_t release_bar = tempty_bar(acc) & ptx::kLeaderMask;       // the leader's barrier, from either CTA
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(release_bar);
      };
      if constexpr (EPI == EPI_MXQ)
        epilogue_tile_mxq<NBLK, 2, RELEASE_AFTER>(taddr, C::OVERLAP && acc == 0, row0, col0, m_lim, p.N, alpha, &outs, epi_s, epi_g, buf,
                                                  lane, smem_gen + C::BAR_OFF + 256 + acc * (NBLK / 2) * 512,
                                                  smem_base + C::BAR_OFF + 256 + acc * (NBLK / 2) * 512, q, 1, release);
      else if constexpr (EPI != EPI_BF16)
        epilogue_tile_glu<EPI == EPI_GLU ? GLU_MX : GLU_BF16, NBLK, RELEASE_AFTER, 2>(
            taddr, C::OVERLAP && acc == 0, (((warp - 2) >> 2) + tile_iter) & 1, row, col0, m_lim, p.N, alpha, p.glu, release);
      else
        epilogue_tile<row_scaled(KIND), KIND == KIND_I8, NBLK, 2, RELEASE_AFTER>(
            taddr, C::OVERLAP && acc == 0, ti.zero, row0, col0, m_lim, p.N, row_scale, p.scale_b, p.b_scalar, &outs, epi_s, epi_g, buf,
            lane, release);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (lane == 0) ptx::bulk_wait<0>();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(&g_device_status, 13); }
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();            // neither CTA leaves while the other may still touch its memory
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, 512);
  }
}

int g_pair_mode = 0;   // test hook: 0 = choose by shape, 1 = always (when eligible), -1 = never

// Pair tiles pay off when there are enough 256 x 256 tiles to occupy the 74 CTA pairs for a few waves.
bool pair_eligible(int64_t M, int64_t N, int64_t row_bytes, bool grouped) {
  if (grouped || g_pair_mode < 0) return false;
  if (g_pair_mode > 0) return true;
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
  (void)row_bytes;
  return tiles >= kNumSMs / 2;     // measured faster than the one-CTA kernel from K = 384 up once the pairs are busy
}

// Pair-tile rows per raster group: as many as keep the group's rows of A (GM x 256 x row_bytes) within 32 MB, a quarter
// of L2, between 4 and 32.  B200Q_RASTER_GM overrides it (experiments).
int pair_raster_gm(int64_t row_bytes) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("B200Q_RASTER_GM");
    forced = e != nullptr ? atoi(e) : 0;
  }
  if (forced > 0) return forced;
  int64_t gm = ((int64_t)32 << 20) / (256 * (row_bytes > 0 ? row_bytes : 1));
  return (int)(gm < 4 ? 4 : (gm > 32 ? 32 : gm));
}

template <int KIND, int EPI>
int launch_pair(const void* A, const void* B, const OutSpec& D, int64_t ldd, const GemmParams& gp, cudaStream_t st) {
  using C = pair::PCfg<KIND>;
  const int64_t row_bytes = KIND == KIND_NV ? gp.K / 2 : gp.K;
  CUtensorMap ma, mb, msa, msb;
  OutMaps md = {};
  int rc;
  if ((rc = encode_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, row_bytes, gp.M, row_bytes, BKB, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, row_bytes, gp.N, row_bytes, BKB, pair::HALF_N, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (EPI == EPI_MXQ) {
    if ((rc = make_code_maps(&md, D, gp.M, gp.N, ldd))) return rc;
  } else if (EPI != EPI_BF16) {
    md.count = 0; md.scatter_rows = 0;                       // the SwiGLU epilogues write their results themselves
    for (int g = 0; g < kMaxOutputs; ++g) md.m[g] = ma;
  } else if ((rc = make_out_maps(&md, D, gp.M, gp.N, ldd))) {
    return rc;
  }
  int sf_kt = 0;
  if (!row_scaled(KIND)) {
    // scale buffers as rows of 256 bytes (two rows per 512-byte atom); box = the atoms of one K step
    const int64_t nblk = KIND == KIND_MX ? gp.K / 32 : gp.K / 16;
    sf_kt = (int)((nblk + 3) / 4);
    const uint64_t rows_a = (uint64_t)((gp.M + 127) / 128) * sf_kt * 2, rows_b = (uint64_t)((gp.N + 127) / 128) * sf_kt * 2;
    if ((rc = encode_2d(&msa, CU_TENSOR_MAP_DATA_TYPE_UINT8, gp.sfa, 256, rows_a, 256, 256, 2 * C::K_ATOMS, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if ((rc = encode_2d(&msb, CU_TENSOR_MAP_DATA_TYPE_UINT8, gp.sfb, 256, rows_b, 256, 256, 2 * C::K_ATOMS, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  } else {
    msa = ma; msb = mb;   // unused
  }
  pair::PairParams p = {};
  p.scale_a = gp.scale_a; p.scale_b = gp.scale_b; p.a_scalar = gp.a_scalar; p.b_scalar = gp.b_scalar;
  p.a_fmt = gp.a_fmt; p.b_fmt = gp.b_fmt; p.M = gp.M; p.N = gp.N;
  p.num_mp = (int)((gp.M + 255) / 256);
  p.num_n = (int)((gp.N + pair::PBN - 1) / pair::PBN);
  p.num_k = (int)((row_bytes + BKB - 1) / BKB);
  p.sf_kt = sf_kt;
  p.glu = gp.glu;
  p.raster_gm = pair_raster_gm(row_bytes);
  // the quantized-output epilogue stages its scale-factor atoms behind the barriers
  constexpr int SMEM = C::SMEM_BYTES + (EPI == EPI_MXQ ? kSfStageBytes : 0);
  static_assert(SMEM <= kSmemBudget, "shared memory overflow");
  B200Q_CUDA(ensure_dynamic_smem(gemm_pair_kernel<KIND, EPI>, SMEM));
  const int tiles = p.num_mp * p.num_n, pairs = tiles < kNumSMs / 2 ? tiles : kNumSMs / 2;
  B200Q_CUDA(launch_pdl(gemm_pair_kernel<KIND, EPI>, dim3(2 * pairs), dim3(gemm_threads(EPI)), SMEM, st, ma, mb, msa, msb, md, p));
  return B200Q_OK;
}

// The grouped MXFP8 forms on pairs.  gp as for the one-CTA kernel: tile_expert / num_tiles (fprop, and dgrad
// with b_along_k) or ragged_offs (wgrad); b_rows = rows of the B matrix as stored.
// Opt-in (b200q_debug_set_gemm_pair(1)): at T = 16384, E = 64, k = 4, D = 768 the pairs move a third
// fewer operand bytes but lose it again to the idle halves of odd experts (6 % more tiles), the
// table build at the start of every CTA and the per-tile expert search: 54 / 46 us against 54 / 40 us
// for the one-CTA kernel on the two forward GEMMs (the dense pair kernel on the same shapes: 46 / 34 us).
// The wgrad form has neither table nor idle halves and still only ties (44 / 32 us against 46 / 32 us).
bool pair_grouped_eligible(const GemmParams& gp) {
  // a forced tile width (test hook) means the one-CTA kernel
  if (g_pair_mode <= 0 || g_force_bn != 0 || gp.n_experts > pair::kPairMaxExperts || (gp.K & 127)) return false;
  if (gp.ragged_offs != nullptr) return (gp.M & 127) == 0;
  return gp.tile_expert != nullptr && (gp.N & 127) == 0;     // an expert's B rows start on a scale-group boundary
}

template <int EPI>
int launch_pair_grouped(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& gp,
                        cudaStream_t st) {
  using C = pair::PCfg<KIND_MX, true>;
  const bool ragged = gp.ragged_offs != nullptr;
  const int64_t row_bytes = gp.K;                                              // per expert for the dgrad form
  const int64_t b_row_bytes = gp.b_along_k ? row_bytes * gp.n_experts : row_bytes;
  const int64_t m_out = ragged ? gp.M * gp.n_experts : gp.M;
  CUtensorMap ma, mb, msa, msb;
  OutMaps md = {};
  int rc;
  if ((rc = encode_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, row_bytes, gp.M, row_bytes, BKB, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, b_row_bytes, b_rows, b_row_bytes, BKB, pair::HALF_N, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (EPI != EPI_BF16) {
    md.count = 0; md.scatter_rows = 0;
    for (int g = 0; g < kMaxOutputs; ++g) md.m[g] = ma;
  } else if ((rc = make_out_maps(&md, D, m_out, gp.N, ldd))) {
    return rc;
  }
  const int sf_kt = (int)(row_bytes / 128), sf_kt_b = gp.b_along_k ? sf_kt * gp.n_experts : sf_kt;
  const uint64_t rows_a = (uint64_t)((gp.M + 127) / 128) * sf_kt * 2, rows_b = (uint64_t)((b_rows + 127) / 128) * sf_kt_b * 2;
  if ((rc = encode_2d(&msa, CU_TENSOR_MAP_DATA_TYPE_UINT8, gp.sfa, 256, rows_a, 256, 256, 2, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  if ((rc = encode_2d(&msb, CU_TENSOR_MAP_DATA_TYPE_UINT8, gp.sfb, 256, rows_b, 256, 256, 2, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  pair::PairParams p = {};
  p.a_fmt = gp.a_fmt; p.b_fmt = gp.b_fmt; p.M = gp.M; p.N = gp.N;
  p.num_mp = (int)((gp.M + 255) / 256);
  p.num_n = (int)((gp.N + pair::PBN - 1) / pair::PBN);
  p.num_k = (int)(row_bytes / BKB);
  p.sf_kt = sf_kt; p.sf_kt_b = sf_kt_b;
  p.glu = gp.glu;
  p.tile_expert = gp.tile_expert; p.num_tiles = gp.num_tiles; p.num_m128 = (int)((gp.M + 127) / 128);
  p.ragged_offs = gp.ragged_offs; p.n_experts = gp.n_experts; p.b_along_k = gp.b_along_k; p.K = gp.K;
  B200Q_CUDA(ensure_dynamic_smem(gemm_pair_kernel<KIND_MX, EPI, true>, C::SMEM_BYTES));
  // the pair-tile count of the expert forms is only known on the device: every pair of the GPU starts
  const int64_t tiles = ragged ? (int64_t)p.num_mp * p.num_n * gp.n_experts : (int64_t)(p.num_m128 + 1) / 2 * p.num_n;
  const int pairs = (int)(tiles < kNumSMs / 2 ? tiles : kNumSMs / 2);
  B200Q_CUDA(launch_pdl(gemm_pair_kernel<KIND_MX, EPI, true>, dim3(2 * pairs), dim3(gemm_threads(EPI)), C::SMEM_BYTES, st, ma, mb, msa, msb, md, p));
  return B200Q_OK;
}

}  // namespace
}  // namespace b200q

extern "C" {
// Test hook: 1 = run eligible dense GEMMs on CTA pairs, -1 = never, 0 = choose by shape.
int b200q_debug_set_gemm_pair(int mode) {
  b200q::g_pair_mode = mode > 0 ? 1 : (mode < 0 ? -1 : 0);
  return B200Q_OK;
}
}
