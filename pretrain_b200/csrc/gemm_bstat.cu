// Ragged grouped MXFP8 GEMM with the weight tile held in shared memory ("B-stationary"), for the expert GEMMs of a MoE
// layer whose contraction dimension is short (K <= 768: src/layers/mlp.py:89,97 at hidden sizes of a few hundred).
//
// With K = 384 .. 768 a 128 x BN output tile has only 3 .. 6 K steps, and the kernel of gemm.cu pulls (128 + BN) * K
// operand bytes from L2 for every tile, besides storing the tile; the tensor pipe is 25 - 38 % busy.  The rows of A are
// sorted by expert, so consecutive 128-row tiles of one column block use the SAME [BN, K] tile of B: here a CTA takes a
// contiguous range of (column block, row tile) pairs with the row tile running fastest, loads B (codes and scale factors,
// all K steps) once per run of tiles that share it, and streams only A through the ring.  Per tile that is 128 * K bytes
// in, a third to a quarter of before.
//
// What it buys, measured at 69632 rows, 64 experts (B200, steady loop): K = 384, N = 768 to bf16: 36.9 us against 40.4 us
// for the general kernel; at K = 768 it loses (the stationary tile leaves a ring of four stages for six K steps, and
// every tile then waits once for a load: 2000 - 4500 clocks under load).  It is therefore taken by default for the
// bf16-output forms with K <= 384 only; gemm_rowstat.cu has the account of what bounds these GEMMs.
//
// Roles, barriers and epilogues are those of gemm_kernel (gemm.cu): producer warp, MMA warp, epilogue warps; TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma with block scales, two accumulators in tensor memory.  New: a "B full" /
// "B free" barrier pair around the stationary tile (single-buffered: at a run boundary the MMAs of the old run drain before
// the new tile lands, while the ring already prefetches the new run's A tiles), a ring stage that holds A and its scale
// factors only, and a stage count that depends on K at run time.  Forms: fprop (B rows e*N + n) and dgrad (B = transposed
// weight stack, expert e at K offset e*K), outputs bf16 (TMA store) or SwiGLU + MXFP8 (direct stores).
#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200q {
namespace {

namespace bstat {

constexpr int kMaxStages = 8;
// producer warp, MMA warp, eight epilogue warps: two per tensor-memory lane quarter for every output form.  With 3 .. 6 K
// steps per tile a main loop is as short as one warp's walk over its 32 rows of the tile, so the epilogue, not the MMA, sets
// the pace unless two warps share each quarter (measured at K = 384, width 256: 3300 clocks per tile with four warps, against
// 1540 clocks of MMA).
constexpr int kThreads = 320;
constexpr int kEpiWarps = kThreads / 32 - 2;
constexpr int kMaxK = 768;                     // bytes of K a stationary tile may hold (6 K steps)
constexpr int A_STAGE = BM * BKB + 1024;       // A tile + its 512-byte scale atom, padded to keep 1024-byte alignment

struct Layout {
  int nk;            // K steps (128 bytes each)
  int stages;        // ring stages for A
  int sfb_off;       // offsets from the 1024-aligned base
  int ring_off;
  int epi_off;
  int bar_off;
  int smem_bytes;
};

// EBUFS: staging blocks per epilogue warp for the bf16 output (two overlap a block's TMA store with the next block's
// conversion; one leaves room for a wider stationary tile)
template <int BN, int EPI, int EBUFS>
inline bool make_layout(int64_t K, Layout* L) {
  using C = Cfg<KIND_MX, BN>;
  const int nk = (int)(K / BKB);
  if (K % BKB || nk < 1 || nk * BKB > kMaxK) return false;
  const int b_bytes = nk * BN * BKB;
  const int sfb_bytes = ((nk * C::NB_ATOMS * 512 + 1023) / 1024) * 1024;
  const int epi_bytes = EPI == EPI_BF16 ? EBUFS * kEpiWarps * EPI_BLOCK_BYTES : 0;
  const int fixed = 1024 /*alignment slack*/ + b_bytes + sfb_bytes + epi_bytes + 256 /*barriers*/;
  int stages = (kSmemBudget - fixed) / A_STAGE;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 3) return false;
  L->nk = nk;
  L->stages = stages;
  L->sfb_off = b_bytes;
  L->ring_off = b_bytes + sfb_bytes;
  L->epi_off = L->ring_off + stages * A_STAGE;
  L->bar_off = L->epi_off + epi_bytes;
  L->smem_bytes = fixed + stages * A_STAGE;
  return true;
}

}  // namespace bstat

template <int BN, int EPI, int EBUFS>
__global__ void __launch_bounds__(bstat::kThreads, 1)
gemm_bstat_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ OutMaps outs, const GemmParams p, const bstat::Layout L) {
  using C = Cfg<KIND_MX, BN>;
  constexpr int B_STEP = BN * BKB;                 // bytes of B per K step
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L.bar_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (bstat::kMaxStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * bstat::kMaxStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * bstat::kMaxStages + 2 + a); };
  const uint32_t bfull_bar = bar_base + 8u * (2 * bstat::kMaxStages + 4), bfree_bar = bfull_bar + 8u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L.bar_off + 8 * (2 * bstat::kMaxStages + 6));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dependency_wait();                          // the permute plan's tables are read right away
  int num_m = p.num_m;
  {
    const int live = __ldcg(p.num_tiles);
    num_m = live < num_m ? live : num_m;
  }
  // this CTA's contiguous range of (column block, row tile) pairs, row tile fastest
  const int64_t total = (int64_t)num_m * p.num_n;
  const int64_t t_begin = total * blockIdx.x / gridDim.x, t_end = total * (blockIdx.x + 1) / gridDim.x;

  {
    // scale-factor areas start as zeros (atoms beyond the end of K are never loaded)
    uint32_t* z = reinterpret_cast<uint32_t*>(smem_gen + L.sfb_off);
    for (int i = threadIdx.x; i < (L.ring_off - L.sfb_off) / 4; i += bstat::kThreads) z[i] = 0;
    for (int s = 0; s < L.stages; ++s) {
      uint32_t* zs = reinterpret_cast<uint32_t*>(smem_gen + L.ring_off + s * bstat::A_STAGE + BM * BKB);
      for (int i = threadIdx.x; i < 1024 / 4; i += bstat::kThreads) zs[i] = 0;
    }
    ptx::fence_proxy_async();
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < L.stages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), bstat::kEpiWarps); }
    ptx::mbar_init(bfull_bar, 1);
    ptx::mbar_init(bfree_bar, 1);
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

  // The walk over this CTA's pairs, kept by each role for itself.  The expert of a row tile comes from a table in global
  // memory; the entries of the next two tiles are fetched ahead, so that no role ever waits for that load between tiles.
  struct Walk {
    const int32_t* te; int num_m;
    int n_blk, m_blk, e;      // current pair and its expert
    int n1, m1, e1;           // the following pair (valid while left > 1)
    int n2, m2, e2;           // and the one after it (valid while left > 2)
    int64_t left;             // pairs from the current one to the end of the range
    __device__ __forceinline__ void next_of(int n, int m, int& no, int& mo) const { mo = m + 1; no = n; if (mo == num_m) { mo = 0; ++no; } }
    __device__ __forceinline__ void start(const int32_t* table, int num_m_, int64_t t0, int64_t t1) {
      te = table; num_m = num_m_; left = t1 - t0;
      n_blk = (int)(t0 / num_m_); m_blk = (int)(t0 - (int64_t)n_blk * num_m_);
      next_of(n_blk, m_blk, n1, m1);
      next_of(n1, m1, n2, m2);
      e = left > 0 ? __ldcg(te + m_blk) : -1;
      e1 = left > 1 ? __ldcg(te + m1) : -1;
      e2 = left > 2 ? __ldcg(te + m2) : -1;
    }
    __device__ __forceinline__ void step() {
      n_blk = n1; m_blk = m1; e = e1;
      n1 = n2; m1 = m2; e1 = e2;
      --left;
      next_of(n1, m1, n2, m2);
      e2 = left > 2 ? __ldcg(te + m2) : -1;
    }
    // the following pair exists and uses the same tile of B
    __device__ __forceinline__ bool next_shares_b() const { return left > 1 && n1 == n_blk && e1 == e; }
  };
  // which B tile a pair needs: rows of B, K offset, scale-atom offset
  struct BTile { int64_t brow0; int64_t bk0; int sfb_k0; };
  auto b_tile = [&](int n_blk, int e) {
    BTile b;
    b.brow0 = (int64_t)n_blk * BN;
    b.bk0 = 0; b.sfb_k0 = 0;
    if (p.b_along_k) { b.bk0 = (int64_t)e * p.K; b.sfb_k0 = e * (int)(p.K >> 7); }
    else b.brow0 += (int64_t)e * p.N;
    return b;
  };

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      uint32_t runs = 0;
      bool new_run = true;
      bool ok = true;
      Walk w;
      for (w.start(p.tile_expert, num_m, t_begin, t_end); w.left > 0 && ok; w.step()) {
        const int m_blk = w.m_blk;
        if (new_run) {
          // the stationary tile may be overwritten once every MMA of the previous run has read it
          if (runs > 0 && (!ptx::mbar_wait(bfree_bar, (runs - 1) & 1) || *abort_flag)) { ok = false; break; }
          const BTile b = b_tile(w.n_blk, w.e);
          ptx::mbar_expect_tx(bfull_bar, (uint32_t)(L.nk * (B_STEP + C::NB_ATOMS * 512)));
          const int64_t g0 = b.brow0 >> 7;
          for (int k = 0; k < L.nk; ++k) {
            ptx::tma_load_2d(smem_base + k * B_STEP, &tmap_b, (int32_t)(k * BKB + b.bk0), (int32_t)b.brow0, bfull_bar);
#pragma unroll
            for (int j = 0; j < C::NB_ATOMS; ++j) {
              const int64_t rg = g0 + j < p.sfb_groups ? g0 + j : g0;     // past the end: any valid group
              ptx::bulk_load(smem_base + L.sfb_off + (k * C::NB_ATOMS + j) * 512, p.sfb + (rg * p.sf_kt_b + b.sfb_k0 + k) * 512, 512,
                             bfull_bar);
            }
          }
          ++runs;
        }
        new_run = !w.next_shares_b();
        for (int k = 0; k < L.nk; ++k) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1)) { ok = false; break; }
          const uint32_t sa = smem_base + L.ring_off + stage * bstat::A_STAGE, fb = full_bar(stage);
          ptx::mbar_expect_tx(fb, BM * BKB + 512);
          ptx::bulk_load(sa + BM * BKB, p.sfa + ((int64_t)m_blk * p.sf_kt + k) * 512, 512, fb);
          ptx::tma_load_2d(sa, &tmap_a, k * BKB, m_blk * BM, fb);
          if (++stage == L.stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 41); }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------
    if (ptx::elect_one()) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t tile_iter = 0;
      uint32_t runs = 0;
      bool new_run = true;
      bool ok = true;
      Walk w;
      for (w.start(p.tile_expert, num_m, t_begin, t_end); w.left > 0 && ok; w.step(), ++tile_iter) {
        // the B tile starts this many 32-row columns into its first scale-factor group
        const uint32_t sfb_col = (uint32_t)(b_tile(w.n_blk, w.e).brow0 & 127) >> 5;
        if (C::OVERLAP) {
          if (tile_iter > 0 && (!ptx::mbar_wait(tempty_bar(acc ^ 1), ((tile_iter - 1) >> 1) & 1) || *abort_flag)) { ok = false; break; }
        } else {
          if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1) || *abort_flag) { ok = false; break; }
        }
        if (new_run) {
          if (!ptx::mbar_wait(bfull_bar, runs & 1) || *abort_flag) { ok = false; break; }
          ++runs;
        }
        const bool last_of_run = !w.next_shares_b();
        new_run = last_of_run;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc ? C::ACC1_COL0 : 0);
        for (int k = 0; k < L.nk; ++k) {
          if (!ptx::mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + L.ring_off + stage * bstat::A_STAGE;
          ptx::tmem_cp_32x128b_warpx4(tmem_base + C::SFA_COL0, ptx::smem_desc_sf(sa + BM * BKB));
#pragma unroll
          for (int j = 0; j < C::NB_ATOMS; ++j)
            ptx::tmem_cp_32x128b_warpx4(tmem_base + C::SFB_COL0 + 4 * j, ptx::smem_desc_sf(smem_base + L.sfb_off + (k * C::NB_ATOMS + j) * 512));
          const uint64_t da = ptx::smem_desc_k_sw128(sa), db = ptx::smem_desc_k_sw128(smem_base + k * B_STEP);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adv = (uint64_t)(kk * 32 >> 4);
            ptx::mma_mxf8(d_tmem, da + adv, db + adv, ptx::idesc_block_scaled(p.a_fmt, p.b_fmt, 1, BM, BN, kk), (k | kk) != 0,
                          tmem_base + C::SFA_COL0, tmem_base + C::SFB_COL0 + sfb_col);
          }
          ptx::tc_commit(empty_bar(stage));
          if (++stage == L.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit(tfull_bar(acc));
        // last tile of a run (the next pair needs another B tile, or there is none): B is free once these MMAs are done
        if (last_of_run) ptx::tc_commit(bfree_bar);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(&g_device_status, 42); }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue ------------------------------------------------
    const int q = warp & 3, grp = (warp - 2) >> 2;
    const uint32_t epi_s = smem_base + L.epi_off + (warp - 2) * EBUFS * EPI_BLOCK_BYTES;
    uint8_t* epi_g = smem_gen + L.epi_off + (warp - 2) * EBUFS * EPI_BLOCK_BYTES;
    int buf = 0;
    int acc = 0; uint32_t acc_phase = 0;
    int tile_iter = 0;
    bool ok = true;
    constexpr int NBLK = BN / EPI_COLS;
    int n_blk = (int)(t_begin / num_m), m_blk = (int)(t_begin - (int64_t)n_blk * num_m);
    for (int64_t t = t_begin; t < t_end && ok; ++t, ++tile_iter) {
      if (!ptx::mbar_wait(tfull_bar(acc), acc_phase) || *abort_flag) { ok = false; break; }
      ptx::tc_fence_after();
      const int64_t row0 = (int64_t)m_blk * BM + q * 32, row = row0 + lane;
      const int64_t col0 = (int64_t)n_blk * BN;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (acc ? C::ACC1_COL0 : 0);
      const uint32_t release_bar = tempty_bar(acc);
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(release_bar);
      };
      if constexpr (EPI == EPI_GLU) {
        constexpr int RELEASE_AFTER = C::OVERLAP ? C::OVL / EPI_COLS - 1 : NBLK - 1;
        epilogue_tile_glu<GLU_MX, NBLK, RELEASE_AFTER, 2>(taddr, C::OVERLAP && acc == 0, (grp + tile_iter) & 1, row, col0, p.M, p.N, 1.f, p.glu,
                                                          release);
      } else {
        // The two warps of a lane quarter split the tile's 64-column blocks into a first and a second share (the larger one
        // changes hands from tile to tile when the count is odd).  With overlapping accumulators the strip that the next
        // main loop overwrites is the tile's last block for accumulator 0 and its first for accumulator 1: the share that
        // holds it walks from that end and hands the accumulator back after its first block; so does the other share, which
        // holds nothing of the strip.
        constexpr int NB0 = (NBLK + 1) / 2, NB1 = NBLK - NB0;
        const bool rev = C::OVERLAP && acc == 0;
        const bool first_share = NB0 == NB1 ? grp == 0 : ((grp + tile_iter) & 1) == 0;
        if (first_share)
          epilogue_tile<false, false, NB0, EBUFS, C::OVERLAP ? 0 : NB0 - 1>(taddr, rev, false, row0, col0, p.M, p.N, 1.f, nullptr, 0, &outs, epi_s,
                                                                          epi_g, buf, lane, release);
        else
          epilogue_tile<false, false, NB1, EBUFS, C::OVERLAP ? 0 : NB1 - 1>(taddr + NB0 * EPI_COLS, rev, false, row0, col0 + NB0 * EPI_COLS, p.M, p.N,
                                                                          1.f, nullptr, 0, &outs, epi_s, epi_g, buf, lane, release);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (++m_blk == num_m) { m_blk = 0; ++n_blk; }
    }
    if (lane == 0) ptx::bulk_wait<0>();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(&g_device_status, 43); }
  }

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

int g_bstat_bn = 0;     // experiments (B200Q_BSTAT_BN): only this tile width
int g_bstat_ebufs = 0;  // experiments (B200Q_BSTAT_EBUFS): staging blocks per epilogue warp, 0 = by the rule in try_bstat
int g_bstat_mode = 0;   // test hook: 0 = the stationary form when the shape allows and is large enough, 1 = whenever it allows, -1 = never

template <int BN, int EPI, int EBUFS>
int launch_bstat(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, GemmParams p, const bstat::Layout& L,
                 cudaStream_t st) {
  const int64_t row_bytes = p.K;
  const int64_t b_row_bytes = p.b_along_k ? row_bytes * p.n_experts : row_bytes;
  CUtensorMap ma, mb;
  OutMaps md = {};
  int rc;
  if ((rc = encode_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, row_bytes, p.M, row_bytes, BKB, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = encode_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, b_row_bytes, b_rows, b_row_bytes, BKB, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (EPI != EPI_BF16) {
    md.count = 0; md.scatter_rows = 0;
    for (int g = 0; g < kMaxOutputs; ++g) md.m[g] = ma;
  } else if ((rc = make_out_maps(&md, D, p.M, p.N, ldd))) {
    return rc;
  }
  p.num_m = (int)((p.M + BM - 1) / BM);
  p.num_n = (int)((p.N + BN - 1) / BN);
  p.num_k = L.nk;
  p.sf_kt = (int)((p.K / 32 + 3) / 4);
  p.sf_kt_b = p.b_along_k ? p.sf_kt * p.n_experts : p.sf_kt;
  p.sfb_groups = (b_rows + 127) / 128;
  // the layout's size varies with K: allow the whole budget once instead of following each launch's size
  B200Q_CUDA(ensure_dynamic_smem(gemm_bstat_kernel<BN, EPI, EBUFS>, kSmemBudget));
  const int64_t tiles = (int64_t)p.num_m * p.num_n;
  const int grid = (int)(tiles < kNumSMs ? tiles : kNumSMs);
  B200Q_CUDA(launch_pdl(gemm_bstat_kernel<BN, EPI, EBUFS>, dim3(grid), dim3(bstat::kThreads), (size_t)L.smem_bytes, st, ma, mb, md, p, L));
  return B200Q_OK;
}

// The stationary form for a grouped fprop / dgrad GEMM when its shape allows: K a multiple of 128 and at most 768, and a
// tile width whose B tile leaves room for at least three ring stages.  Returns kBstatNotApplicable when it does not apply
// (the caller then takes the general kernel).
template <int EPI>
int try_bstat(const void* A, const void* B, const OutSpec& D, int64_t ldd, int64_t b_rows, const GemmParams& p, cudaStream_t st) {
  static bool env_read = false;
  if (!env_read) {                                 // B200Q_BSTAT=-1 / 0 / 1 sets the initial mode (experiments)
    env_read = true;
    const char* e = getenv("B200Q_BSTAT");
    if (e != nullptr) g_bstat_mode = atoi(e) < 0 ? -1 : (atoi(e) > 0 ? 1 : 0);
    e = getenv("B200Q_BSTAT_BN");
    if (e != nullptr) g_bstat_bn = atoi(e);
    e = getenv("B200Q_BSTAT_EBUFS");
    if (e != nullptr) g_bstat_ebufs = atoi(e) == 1 ? 1 : (atoi(e) == 2 ? 2 : 0);
  }
  if (g_bstat_mode < 0 || g_force_bn != 0 || g_pair_mode > 0) return kBstatNotApplicable;
  if (p.tile_expert == nullptr || p.num_tiles == nullptr || p.ragged_offs != nullptr || (p.K & 127) || p.K > bstat::kMaxK)
    return kBstatNotApplicable;
  if (g_bstat_mode == 0 && p.M < 16 * BM) return kBstatNotApplicable;      // a handful of tiles: nothing to reuse
  // By default only where it measured faster than the general kernel (65536 x 768 rows, 64 experts): the bf16-output forms
  // with K <= 384, whose ring then holds two tiles of A (37 us against 40 us at K = 384, N = 768).  At K = 768 the ring
  // is shorter than one tile and every tile waits once for a load (dgrad 51 us against 49 us); the SwiGLU form is taken
  // by the row-stationary pair kernel.
  if (g_bstat_mode == 0 && (EPI == EPI_GLU || p.K > 384)) return kBstatNotApplicable;
  // The widest stationary tile that leaves room for three ring stages.  bf16 output: two staging blocks per epilogue warp
  // when the ring still holds two tiles' worth of A beside them, else one (the ring's depth hides the load latency; a
  // second staging block only overlaps a 4 KB store with the next block's conversion).
  int rc = kBstatNotApplicable;
  auto attempt = [&](auto bn_tag) {
    constexpr int BN = decltype(bn_tag)::value;
    bstat::Layout L2;
    if constexpr (EPI == EPI_BF16) {
      bstat::Layout L1;
      const bool ok2 = bstat::make_layout<BN, EPI, 2>(p.K, &L2), ok1 = bstat::make_layout<BN, EPI, 1>(p.K, &L1);
      const int want = g_bstat_ebufs;
      if (ok2 && (want == 2 || (want == 0 && L2.stages >= 2 * L2.nk) || !ok1)) { rc = launch_bstat<BN, EPI, 2>(A, B, D, ldd, b_rows, p, L2, st); return true; }
      if (ok1) { rc = launch_bstat<BN, EPI, 1>(A, B, D, ldd, b_rows, p, L1, st); return true; }
      return false;
    } else {
      if (!bstat::make_layout<BN, EPI, 2>(p.K, &L2)) return false;
      rc = launch_bstat<BN, EPI, 2>(A, B, D, ldd, b_rows, p, L2, st);
      return true;
    }
  };
  const int only = g_bstat_bn;
  // 192 before 256 when it divides N: two whole accumulators fit in tensor memory, and it measured 1 - 2 % faster
  if ((only == 0 || only == 192) && p.N % 192 == 0 && attempt(std::integral_constant<int, 192>{})) return rc;
  if ((only == 0 || only == 256) && p.N % 256 == 0 && attempt(std::integral_constant<int, 256>{})) return rc;
  if ((only == 0 || only == 192) && p.N % 64 == 0 && attempt(std::integral_constant<int, 192>{})) return rc;
  if ((only == 0 || only == 128) && attempt(std::integral_constant<int, 128>{})) return rc;
  return kBstatNotApplicable;
}

}  // namespace
}  // namespace b200q

extern "C" {
// Test hook: -1 = the grouped GEMMs never take the B-stationary kernel, 1 = whenever the shape allows (small problems too),
// 0 = by shape and size (the default).
int b200q_debug_set_gemm_bstat(int mode) {
  b200q::g_bstat_mode = mode < 0 ? -1 : (mode > 0 ? 1 : 0);
  return B200Q_OK;
}
}
