// Grouped MXFP8 GEMM on CTA pairs with the rows of A held in shared memory ("row-stationary"), for the expert GEMMs of a
// MoE layer whose contraction dimension is short (K <= 768: src/layers/mlp.py:89,97 at hidden sizes of a few hundred).
//
// With 3 .. 6 K steps per tile the tensor pipe of the general kernels is 25 - 38 % busy: a 128 x 256 tile at K = 768
// moves 288 KB (one CTA) or 192 KB (pair) of operands for 3072 clocks of MMA, and the ring holds at most one tile.  Here
// a pair of CTAs takes a contiguous range of (pair tile, column block) with the column block running fastest and keeps
// its 256 rows of A (codes and scale factors, all K steps, 128 rows per CTA) in shared memory for the whole run of column
// blocks.  Only the halves of the B tiles stream through the ring (12 or 16 KB stages, more than a tile deep), and A is
// read from L2 exactly once.  The stationary rows are reloaded chunk by chunk: K step k of the next run's rows is fetched
// as soon as the last tile of the old run is done with step k (one "free" / "full" barrier pair per K step), so the
// reload runs behind the last tile's main loop instead of after it.
//
// What it buys, measured at 69632 x 768 x 768 over 64 experts (B200): in a steady loop of the one kernel the SwiGLU form
// takes 44.6 us against 46.4 us for the general kernel and the bf16 forms tie; inside the MoE block (gather + quantize
// before it) it is 1 us SLOWER (53.4 against 52.4 us), so it is an opt-in, kept for the record and covered by the same
// tests as the other forms.  Timelines (clock64 per role, tile and K step) and runs with parts switched off show why a
// kernel that moves a third of the operand bytes gains nothing:
//   * with the MMAs, the epilogue arithmetic and the stores all removed the kernel still takes 38 us, and just as long
//     when every load is pointed at one and the same small tile: the floor is not set by the memory system;
//   * the thread that issues the MMAs needs about 500 clocks per K step for waiting on the "full" barrier (300, on a
//     barrier that completed long before), three scale-factor copies into tensor memory and the commit (230), before any
//     MMA - as long as the four MMAs of a 256 x 192 (384 clocks) or 256 x 256 (512 clocks) step run.  The dense kernels
//     hide the same cost behind 64 K steps per tile; here a tile has six;
//   * about 13 us are the start of the kernel: 3 us of set-up (table of the experts' pair tiles, barriers, tensor memory),
//     then every SM fills 200 KB of shared memory at once and the first tile completes after 22000 clocks;
//   * the SwiGLU epilogue's stores (16 bytes per lane to 32 rows per instruction) add 7 - 9 us in every kernel form.
// Running the producer and MMA loops with the whole warp (one elected lane issuing) instead of one thread measured slower.
//
// Roles, pair protocol (who signals whom) and epilogues are those of gemm_pair_kernel; two epilogue warps share each
// tensor-memory lane quarter for every output form.  Forms: fprop (B rows e*N + n) and dgrad (B = transposed weight
// stack, expert e at K offset e*K); outputs bf16 (TMA store) or SwiGLU + MXFP8 (direct stores).  No TMA multicast.
#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200q {
namespace {

namespace rowstat {

constexpr int kThreads = 320;                   // producer warp, MMA warp, eight epilogue warps
constexpr int kEpiWarps = kThreads / 32 - 2;
constexpr int kMaxStages = 8;
constexpr int kMaxNk = 6;                       // K <= 768
// ring stage: this CTA's half of the B tile + the two scale atoms the tile's columns touch
template <int BN> __host__ __device__ constexpr int b_stage() { return BN / 2 * BKB + 1024; }
constexpr int kBarBytes = 512;

struct Layout {
  int nk;            // K steps (128 bytes each)
  int stages;        // ring stages for B
  int sfa_off;       // offsets from the 1024-aligned base; the rows of A start at 0
  int ring_off;
  int epi_off;
  int bar_off;
  int grp_off;
  int smem_bytes;
};

// Tile width 192 leaves room for two whole accumulators beside the scale columns (2 * 192 + 12 <= 512), so a main loop
// never waits for the epilogue of the tile before it; at 256 the accumulators share a 64-column strip that the previous
// tile's epilogue has to read first (about 1500 clocks per tile in the timeline).  The two widths measure the same.
template <int BN, int EPI, int EBUFS>
inline bool make_layout(int64_t K, Layout* L) {
  constexpr int B_STAGE = b_stage<BN>();
  const int nk = (int)(K / BKB);
  if (K % BKB || nk < 1 || nk > kMaxNk) return false;
  const int a_bytes = nk * BM * BKB;
  const int sfa_bytes = ((nk * 512 + 1023) / 1024) * 1024;
  const int epi_bytes = EPI == EPI_BF16 ? EBUFS * kEpiWarps * EPI_BLOCK_BYTES : 0;
  const int grp_bytes = ((pair::kGroupTableBytes + 255) / 256) * 256;
  const int fixed = 1024 /*alignment slack*/ + a_bytes + sfa_bytes + epi_bytes + kBarBytes + grp_bytes;
  int stages = (kSmemBudget - fixed) / B_STAGE;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 4) return false;
  L->nk = nk;
  L->stages = stages;
  L->sfa_off = a_bytes;
  L->ring_off = a_bytes + sfa_bytes;
  L->epi_off = L->ring_off + stages * B_STAGE;
  L->bar_off = L->epi_off + epi_bytes;
  L->grp_off = L->bar_off + kBarBytes;
  L->smem_bytes = fixed + stages * B_STAGE;
  return true;
}

template <int BN>
struct TCfg {                                     // tensor-memory columns
  static constexpr bool OVERLAP = 2 * BN + 12 > 512;
  static constexpr int OVL = OVERLAP ? 64 : 0;
  static constexpr int ACC1_COL0 = BN - OVL;
  static constexpr int SFA_COL0 = 2 * BN - OVL;
  static constexpr int SFB_COL0 = SFA_COL0 + 4;
  static_assert(SFB_COL0 + 8 <= 512, "tensor memory overflow");
};

// What the roles of one CTA need to know about a run (one pair tile: 256 rows of one expert, 128 per CTA).
struct Run {
  int row0;          // this CTA's first row of A
  bool live;         // this CTA owns output rows (not the idle half of an expert's odd last pair)
  int brow_e;        // B row offset of the expert (fprop) or 0
  int bgroup_e;      // scale-group offset of the expert (fprop) or 0
  int bk0;           // K offset of B in bytes (dgrad) or 0
  int sfb_k0;        // first scale atom of B along K (dgrad) or 0
};

__device__ __forceinline__ Run get_run(const pair::PairParams& p, int pt, int cta, const int* g_first, const int* g_pairs) {
  int lo = 0, hi = p.n_experts - 1;                   // last expert whose first pair tile is <= pt
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (g_pairs[mid] <= pt) lo = mid; else hi = mid - 1;
  }
  const int e = lo, tile0 = g_first[e] + 2 * (pt - g_pairs[e]);
  Run r;
  r.row0 = (tile0 + cta) * BM;
  r.live = cta == 0 || tile0 + 1 < g_first[e + 1];
  r.brow_e = 0; r.bgroup_e = 0; r.bk0 = 0; r.sfb_k0 = 0;
  if (p.b_along_k) {
    r.bk0 = (int)(e * p.K);
    r.sfb_k0 = e * p.sf_kt;
  } else {
    r.brow_e = e * (int)p.N;
    r.bgroup_e = (int)((e * p.N) >> 7);
  }
  return r;
}

// The walk over the pair's contiguous range of (pair tile, column block), column block fastest.  (Handing whole pair tiles
// round-robin to the pairs instead, so that neighbouring pairs ask for the same tiles of B at the same time, measured 7 %
// slower at 64 experts x 768 x 768.)
struct Walk {
  int num_n, pt, n;
  int left;
  bool first;        // first tile of the range
  __device__ __forceinline__ void start(int total_pt, int num_n_, int pair_id, int num_pairs) {
    const int total = total_pt * num_n_;
    const int u0 = (int)((int64_t)total * pair_id / num_pairs), u1 = (int)((int64_t)total * (pair_id + 1) / num_pairs);
    num_n = num_n_; pt = u0 / num_n_; n = u0 - pt * num_n_; left = u1 - u0; first = true;
  }
  __device__ __forceinline__ void step() { if (++n == num_n) { n = 0; ++pt; } --left; first = false; }
  __device__ __forceinline__ bool first_of_run() const { return first || n == 0; }
  __device__ __forceinline__ bool last_of_run() const { return left == 1 || n == num_n - 1; }
};

}  // namespace rowstat

template <int BN, int EPI, int EBUFS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(rowstat::kThreads, 1)
gemm_rowstat_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                    const __grid_constant__ OutMaps outs, const pair::PairParams p, const rowstat::Layout L) {
  using C = rowstat::TCfg<BN>;
  constexpr int HALF_N = BN / 2, B_STAGE = rowstat::b_stage<BN>();
  constexpr int A_STEP = BM * BKB;
  constexpr uint32_t B_TX = HALF_N * BKB + 1024, A_TX = A_STEP + 512;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L.bar_off;
  constexpr int S = rowstat::kMaxStages, NK = rowstat::kMaxNk;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // used in the leader only
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };                // one per CTA
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };            // one per CTA
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };       // used in the leader only
  auto afull_bar = [&](int k) { return bar_base + 8u * (2 * S + 4 + k); };        // used in the leader only
  auto afree_bar = [&](int k) { return bar_base + 8u * (2 * S + 4 + NK + k); };   // one per CTA
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L.bar_off + 8 * (2 * S + 4 + 2 * NK));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = ptx::cluster_ctarank();       // 0 = leader
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  int* g_first = reinterpret_cast<int*>(smem_gen + L.grp_off);          // first 128-row tile of every expert (+ end)
  int* g_pairs = g_first + pair::kPairMaxExperts + 1;                    // pair tiles before every expert (+ total)

  if (threadIdx.x == 0) {
    // full / A full: one arrival (with its byte count) per producer of the pair; empty / A free / accumulator full: the
    // leader's commit; accumulator free: every epilogue warp of each CTA
    for (int s = 0; s < L.stages; ++s) { ptx::mbar_init(full_bar(s), 2); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), 2 * rowstat::kEpiWarps); }
    for (int k = 0; k < L.nk; ++k) { ptx::mbar_init(afull_bar(k), 2); ptx::mbar_init(afree_bar(k), 1); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_sfa);
    ptx::prefetch_tensormap(&tmap_sfb);
    for (int g = 0; g < outs.count; ++g) ptx::prefetch_tensormap(&outs.m[g]);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish_pair();
  }
  grid_dependency_wait();                          // the permute plan's tables are read next
  pair::build_expert_pairs<rowstat::kThreads>(p.tile_expert, p.num_tiles, p.num_m128, p.n_experts, g_first, g_pairs);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();            // both CTAs' barriers exist before anyone signals the peer
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_pt = g_pairs[p.n_experts];

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ---------------------------------
    if (ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      uint32_t runs = 0;
      bool ok = true;
      rowstat::Run r = {};
      rowstat::Walk w;
      for (w.start(total_pt, p.num_n, pair_id, num_pairs); w.left > 0 && ok; w.step()) {
        const bool new_run = w.first_of_run();
        if (new_run) r = rowstat::get_run(p, w.pt, (int)cta, g_first, g_pairs);
        const int brow0 = r.brow_e + w.n * BN + (int)cta * HALF_N, bgroup = r.bgroup_e + ((w.n * BN) >> 7);
        for (int k = 0; k < L.nk; ++k) {
          if (new_run) {
            // K step k of the rows: free once the last tile of the previous run has multiplied it
            if (runs > 0 && (!ptx::mbar_wait(afree_bar(k), (runs - 1) & 1) || *abort_flag)) { ok = false; break; }
            const uint32_t ab = afull_bar(k) & ptx::kLeaderMask;
            ptx::mbar_expect_tx_cluster(ab, A_TX);
            ptx::tma_load_2d_pair(smem_base + k * A_STEP, &tmap_a, k * BKB, r.row0, ab);
            ptx::tma_load_2d_pair(smem_base + L.sfa_off + k * 512, &tmap_sfa, 0, 2 * ((r.row0 >> 7) * p.sf_kt + k), ab);
          }
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1)) { ok = false; break; }
          const uint32_t sb = smem_base + L.ring_off + stage * B_STAGE, ssfb = sb + HALF_N * BKB;
          const uint32_t fb = full_bar(stage) & ptx::kLeaderMask;    // the leader's barrier, from either CTA
          ptx::mbar_expect_tx_cluster(fb, B_TX);
          ptx::tma_load_2d_pair(sb, &tmap_b, k * BKB + r.bk0, brow0, fb);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            ptx::tma_load_2d_pair(ssfb + j * 512, &tmap_sfb, 0, 2 * ((bgroup + j) * p.sf_kt_b + r.sfb_k0 + k), fb);
          if (++stage == L.stages) { stage = 0; phase ^= 1; }
        }
        if (new_run) ++runs;
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 51); }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------
    if (cta == 0 && ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t tile_iter = 0;
      uint32_t runs = 0;
      bool ok = true;
      rowstat::Walk w;
      for (w.start(total_pt, p.num_n, pair_id, num_pairs); w.left > 0 && ok; w.step(), ++tile_iter) {
        if (C::OVERLAP) {
          // the accumulators overlap: tile t may start once tile t - 1 has handed back the shared strip
          if (tile_iter > 0 && (!ptx::mbar_wait(tempty_bar(acc ^ 1), ((tile_iter - 1) >> 1) & 1) || *abort_flag)) { ok = false; break; }
        } else {
          if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1) || *abort_flag) { ok = false; break; }
        }
        // the tile's columns start this many 32-row columns into their first scale group (0 or 2)
        const uint32_t sfb_col = (uint32_t)((w.n * BN) & 127) >> 5;
        const bool new_run = w.first_of_run(), last = w.last_of_run();
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc ? C::ACC1_COL0 : 0);
        for (int k = 0; k < L.nk; ++k) {
          if (new_run && (!ptx::mbar_wait(afull_bar(k), runs & 1) || *abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + k * A_STEP, sb = smem_base + L.ring_off + stage * B_STAGE;
          const uint32_t ssfb = sb + HALF_N * BKB;
          ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + C::SFA_COL0, ptx::smem_desc_sf(smem_base + L.sfa_off + k * 512));
#pragma unroll
          for (int j = 0; j < 2; ++j) ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + C::SFB_COL0 + 4 * j, ptx::smem_desc_sf(ssfb + j * 512));
          const uint64_t da = ptx::smem_desc_k_sw128(sa), db = ptx::smem_desc_k_sw128(sb);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adv = (uint64_t)(kk * 32 >> 4);
            ptx::mma_mxf8_pair(d_tmem, da + adv, db + adv, ptx::idesc_block_scaled(p.a_fmt, p.b_fmt, 1, 256, BN, kk), (k | kk) != 0,
                               tmem_base + C::SFA_COL0, tmem_base + C::SFB_COL0 + sfb_col);
          }
          ptx::tc_commit_pair(empty_bar(stage));
          if (last) ptx::tc_commit_pair(afree_bar(k));
          if (++stage == L.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit_pair(tfull_bar(acc));
        if (new_run) ++runs;
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 52); }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (both CTAs, own 128 rows) ------------------------
    const int q = warp & 3, grp = (warp - 2) >> 2;
    const uint32_t epi_s = smem_base + L.epi_off + (warp - 2) * EBUFS * EPI_BLOCK_BYTES;
    uint8_t* epi_g = smem_gen + L.epi_off + (warp - 2) * EBUFS * EPI_BLOCK_BYTES;
    int buf = 0;
    int acc = 0; uint32_t acc_phase = 0;
    int tile_iter = 0;
    bool ok = true;
    constexpr int NBLK = BN / EPI_COLS;
    rowstat::Run r = {};
    rowstat::Walk w;
    for (w.start(total_pt, p.num_n, pair_id, num_pairs); w.left > 0 && ok; w.step(), ++tile_iter) {
      if (w.first_of_run()) r = rowstat::get_run(p, w.pt, (int)cta, g_first, g_pairs);
      if (!ptx::mbar_wait(tfull_bar(acc), acc_phase) || *abort_flag) { ok = false; break; }
      ptx::tc_fence_after();
      const int64_t row0 = (int64_t)r.row0 + q * 32, row = row0 + lane;
      const int64_t col0 = (int64_t)w.n * BN;
      const int64_t m_lim = r.live ? p.M : 0;       // rows this CTA may store
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (acc ? C::ACC1_COL0 : 0);
      const uint32_t release_bar = tempty_bar(acc) & ptx::kLeaderMask;       // the leader's barrier, from either CTA
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(release_bar);
      };
      const bool rev = C::OVERLAP && acc == 0;      // overlapping accumulators: number 0 shares its LAST columns with number 1
      if constexpr (EPI == EPI_GLU) {
        constexpr int RELEASE_AFTER = C::OVERLAP ? C::OVL / EPI_COLS - 1 : NBLK - 1;
        epilogue_tile_glu<GLU_MX, NBLK, RELEASE_AFTER, 2>(taddr, rev, (grp + tile_iter) & 1, row, col0, m_lim, p.N, 1.f, p.glu, release);
      } else {
        // The two warps of a lane quarter split the tile's 64-column blocks into a first and a second share (the larger one
        // changes hands from tile to tile when the count is odd).  With overlapping accumulators the share that holds the
        // strip the next main loop overwrites walks from that end, and both hand the accumulator back after their first
        // block; without, each hands it back after its last.
        constexpr int NB0 = (NBLK + 1) / 2, NB1 = NBLK - NB0;
        const bool first_share = NB0 == NB1 ? grp == 0 : ((grp + tile_iter) & 1) == 0;
        if (first_share)
          epilogue_tile<false, false, NB0, EBUFS, C::OVERLAP ? 0 : NB0 - 1>(taddr, rev, false, row0, col0, m_lim, p.N, 1.f, nullptr, 0, &outs, epi_s,
                                                                          epi_g, buf, lane, release);
        else
          epilogue_tile<false, false, NB1, EBUFS, C::OVERLAP ? 0 : NB1 - 1>(taddr + NB0 * EPI_COLS, rev, false, row0, col0 + NB0 * EPI_COLS, m_lim,
                                                                          p.N, 1.f, nullptr, 0, &outs, epi_s, epi_g, buf, lane, release);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (lane == 0) ptx::bulk_wait<0>();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(&g_device_status, 53); }
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

int g_rowstat_bn = 0;     // experiments (B200Q_ROWSTAT_BN): only this tile width
int g_rowstat_mode = 0;   // test hook: 0 = the row-stationary form when the shape allows and is large enough, 1 = whenever it allows, -1 = never

template <int BN, int EPI, int EBUFS>
int launch_rowstat(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& gp, const rowstat::Layout& L,
                   cudaStream_t st) {
  const int64_t row_bytes = gp.K;                                              // per expert for the dgrad form
  const int64_t b_row_bytes = gp.b_along_k ? row_bytes * gp.n_experts : row_bytes;
  CUtensorMap ma, mb, msa, msb;
  OutMaps md = {};
  int rc;
  if ((rc = encode_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, row_bytes, gp.M, row_bytes, BKB, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, b_row_bytes, b_rows, b_row_bytes, BKB, BN / 2, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (EPI != EPI_BF16) {
    md.count = 0; md.scatter_rows = 0;
    for (int g = 0; g < kMaxOutputs; ++g) md.m[g] = ma;
  } else if ((rc = make_out_maps(&md, D, gp.M, gp.N, ldd))) {
    return rc;
  }
  const int sf_kt = (int)(row_bytes / 128), sf_kt_b = gp.b_along_k ? sf_kt * gp.n_experts : sf_kt;
  const uint64_t rows_a = (uint64_t)((gp.M + 127) / 128) * sf_kt * 2, rows_b = (uint64_t)((b_rows + 127) / 128) * sf_kt_b * 2;
  if ((rc = encode_2d(&msa, CU_TENSOR_MAP_DATA_TYPE_UINT8, gp.sfa, 256, rows_a, 256, 256, 2, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  if ((rc = encode_2d(&msb, CU_TENSOR_MAP_DATA_TYPE_UINT8, gp.sfb, 256, rows_b, 256, 256, 2, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  pair::PairParams p = {};
  p.a_fmt = gp.a_fmt; p.b_fmt = gp.b_fmt; p.M = gp.M; p.N = gp.N;
  p.num_mp = (int)((gp.M + 255) / 256);
  p.num_n = (int)((gp.N + BN - 1) / BN);
  p.num_k = L.nk;
  p.sf_kt = sf_kt; p.sf_kt_b = sf_kt_b;
  p.glu = gp.glu;
  p.tile_expert = gp.tile_expert; p.num_tiles = gp.num_tiles; p.num_m128 = (int)((gp.M + 127) / 128);
  p.ragged_offs = nullptr; p.n_experts = gp.n_experts; p.b_along_k = gp.b_along_k; p.K = gp.K;
  // the layout's size varies with K: allow the whole budget once instead of following each launch's size
  B200Q_CUDA(ensure_dynamic_smem(gemm_rowstat_kernel<BN, EPI, EBUFS>, kSmemBudget));
  // the pair-tile count is only known on the device: every pair of the GPU starts (a pair without tiles leaves at once)
  const int64_t tiles = (int64_t)(p.num_m128 + 1) / 2 * p.num_n;
  const int pairs = (int)(tiles < kNumSMs / 2 ? tiles : kNumSMs / 2);
  B200Q_CUDA(launch_pdl(gemm_rowstat_kernel<BN, EPI, EBUFS>, dim3(2 * pairs), dim3(rowstat::kThreads), (size_t)L.smem_bytes, st, ma, mb, msa, msb, md,
                        p, L));
  return B200Q_OK;
}

// The row-stationary form for a grouped fprop / dgrad GEMM when its shape allows: K a multiple of 128 and at most 768,
// N a multiple of 128 (an expert's rows of B start on a scale-group boundary), at most 256 experts.  Returns
// kRowstatNotApplicable when it does not apply (the caller then takes the general kernel).
template <int EPI>
int try_rowstat(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& p, cudaStream_t st) {
  static bool env_read = false;
  if (!env_read) {                                 // B200Q_ROWSTAT=-1 / 0 / 1 sets the initial mode (experiments)
    env_read = true;
    const char* e = getenv("B200Q_ROWSTAT");
    if (e != nullptr) g_rowstat_mode = atoi(e) < 0 ? -1 : (atoi(e) > 0 ? 1 : 0);
    e = getenv("B200Q_ROWSTAT_BN");
    if (e != nullptr) g_rowstat_bn = atoi(e);
  }
  if (g_rowstat_mode < 0 || g_force_bn != 0 || g_pair_mode > 0) return kRowstatNotApplicable;
  if (p.tile_expert == nullptr || p.num_tiles == nullptr || p.ragged_offs != nullptr || (p.K & 127) || p.K > rowstat::kMaxNk * BKB ||
      (p.N & 127) || p.n_experts > pair::kPairMaxExperts)
    return kRowstatNotApplicable;
  // Opt-in only (b200q_debug_set_gemm_rowstat(1) / B200Q_ROWSTAT=1): see the account at the top of this file - a tie with
  // the general kernel inside the MoE block, where the kernels before it leave other things in L2 than a steady loop does.
  if (g_rowstat_mode == 0) return kRowstatNotApplicable;
  int rc = kRowstatNotApplicable;
  auto attempt = [&](auto bn_tag) {
    constexpr int BN = decltype(bn_tag)::value;
    rowstat::Layout L;
    if constexpr (EPI == EPI_BF16) {
      // two staging blocks per epilogue warp when the ring still holds two tiles' worth of B beside them, else one
      if (rowstat::make_layout<BN, EPI, 2>(p.K, &L) && L.stages >= 2 * L.nk) { rc = launch_rowstat<BN, EPI, 2>(A, B, D, ldd, b_rows, p, L, st); return true; }
      if (rowstat::make_layout<BN, EPI, 1>(p.K, &L)) { rc = launch_rowstat<BN, EPI, 1>(A, B, D, ldd, b_rows, p, L, st); return true; }
    } else {
      if (rowstat::make_layout<BN, EPI, 2>(p.K, &L)) { rc = launch_rowstat<BN, EPI, 2>(A, B, D, ldd, b_rows, p, L, st); return true; }
    }
    return false;
  };
  const int only = g_rowstat_bn;
  if ((only == 0 || only == 192) && p.N % 192 == 0 && attempt(std::integral_constant<int, 192>{})) return rc;
  if ((only == 0 || only == 256) && attempt(std::integral_constant<int, 256>{})) return rc;
  return kRowstatNotApplicable;
}

}  // namespace
}  // namespace b200q

extern "C" {
// Test hook: -1 = the grouped GEMMs never take the row-stationary pair kernel, 1 = whenever the shape allows (small problems
// too), 0 = by shape and size (the default).
int b200q_debug_set_gemm_rowstat(int mode) {
  b200q::g_rowstat_mode = mode < 0 ? -1 : (mode > 0 ? 1 : 0);
  return B200Q_OK;
}
}
