// Epilogue of one output tile, shared by the one-CTA and the CTA-pair GEMM kernels.  A warp owns
// 32 accumulator rows (its tensor-memory lane quarter) and walks the tile in blocks of 64 columns:
// tcgen05.ld (two 32-column loads, the next block's loads in flight while this one is converted)
// -> scale -> bf16 -> 32 x 128-byte rows in 128-byte-swizzled shared memory -> one TMA store,
// which also clips rows / columns beyond the matrix.  Included inside namespace b200q::{anonymous}.
#pragma once

constexpr int EPI_COLS = 64;                         // columns per epilogue block (128 bytes of bf16)
constexpr int EPI_BLOCK_BYTES = 32 * EPI_COLS * 2;   // 4 KB staging block
constexpr int kEpiBytes1 = 4 * EPI_BLOCK_BYTES;      // one staging block per epilogue warp

// Where a tile's blocks are stored: this GPU's output and, for the fused GEMM + all-gather, the
// same rows of every peer's copy of the gathered output (peer-mapped device memory, written by
// TMA stores over NVLink; stores only — nothing is ever loaded from a peer).
constexpr int kMaxOutputs = 8;
struct OutMaps {
  CUtensorMap m[kMaxOutputs];
  int count;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  ptx::tmem_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
  ptx::tmem_ld32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
}

// KIND_F8 (= 0) multiplies by a scale per output column; the other kinds only by `row_scale`.
// `rev` walks the blocks from the last to the first (used when the tile's LAST columns are the ones
// to hand back first); `release` is called once, after block number RELEASE_AFTER (in walking
// order) has been read from tensor memory.
template <bool COL_SCALE, int NBLK, int EPI_BUFS, int RELEASE_AFTER, class Release>
__device__ __forceinline__ void epilogue_tile(uint32_t taddr, bool rev, int64_t row0, int64_t col0, int64_t M, int64_t N,
                                              float row_scale, const float* __restrict__ scale_b, int b_scalar,
                                              const OutMaps* outs, uint32_t epi_s, uint8_t* epi_g, int& buf, int lane,
                                              Release release) {
  auto emit = [&](int c, const uint32_t (&r)[64]) {
    const int64_t colg = col0 + c * EPI_COLS;
    float sb0 = 1.f, sb1 = 1.f;
    if (COL_SCALE) {
      if (b_scalar) {
        sb0 = sb1 = __ldg(scale_b);
      } else {
        sb0 = colg + lane < N ? __ldg(scale_b + colg + lane) : 0.f;
        sb1 = colg + 32 + lane < N ? __ldg(scale_b + colg + 32 + lane) : 0.f;
      }
    }
    uint32_t o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float lo = u2f(r[2 * i]) * row_scale, hi = u2f(r[2 * i + 1]) * row_scale;
      if (COL_SCALE) {
        lo *= __shfl_sync(0xFFFFFFFFu, i < 16 ? sb0 : sb1, (2 * i) & 31);
        hi *= __shfl_sync(0xFFFFFFFFu, i < 16 ? sb0 : sb1, (2 * i + 1) & 31);
      }
      o[i] = pack_bf16(lo, hi);
    }
    if (lane == 0) ptx::bulk_wait_read<EPI_BUFS - 1>();   // the store that last read this buffer is done with it
    __syncwarp();
    uint8_t* dst = epi_g + buf * EPI_BLOCK_BYTES + lane * 128;
    const int sw = lane & 7;                              // 128-byte swizzle: 16-byte chunk j of row r sits at j ^ (r & 7)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<uint4*>(dst + ((j ^ sw) << 4)) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
    ptx::fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      for (int g = 0; g < outs->count; ++g)
        ptx::tma_store_2d(&outs->m[g], (int32_t)colg, (int32_t)row0, epi_s + buf * EPI_BLOCK_BYTES);
      ptx::bulk_commit();
    }
    buf = (buf + 1) % EPI_BUFS;
  };

  uint32_t ra[64], rb[64];
  tmem_ld64(taddr + (rev ? NBLK - 1 : 0) * EPI_COLS, ra);
#pragma unroll
  for (int i = 0; i < NBLK; ++i) {
    const int c = rev ? NBLK - 1 - i : i;
    ptx::tmem_ld_wait();
    if (i == RELEASE_AFTER) release();
    if (i + 1 < NBLK) {
      const int cn = rev ? c - 1 : c + 1;
      if (i & 1) tmem_ld64(taddr + cn * EPI_COLS, ra);
      else tmem_ld64(taddr + cn * EPI_COLS, rb);
    }
    if (col0 + c * EPI_COLS < N && row0 < M) {            // warp-uniform
      if (i & 1) emit(c, rb);
      else emit(c, ra);
    }
  }
}
