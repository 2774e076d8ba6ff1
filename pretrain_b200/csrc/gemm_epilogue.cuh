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
// Scatter form (GEMM + reduce-scatter): output g holds only the rows [g * scatter_rows, (g + 1) * scatter_rows) of
// the result - this rank's slot in the staging buffer of the rank that owns those rows - so every block goes to
// exactly one output, the owner of its rows.
constexpr int kMaxOutputs = 8;
struct OutMaps {
  CUtensorMap m[kMaxOutputs];
  int count;
  int scatter_rows;    // 0: every output receives every block; else a multiple of 32
  // MXFP8-quantized output (epilogue_tile_mxq): the maps above are byte matrices of codes, and sf[g] is where this
  // rank's rows start in output g's 128x4-tiled scale-factor buffer, which has sf_kt K-tiles per row tile
  uint8_t* sf[kMaxOutputs];
  int64_t sf_kt;
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
// ACC_INT: the accumulators are 32-bit integers (kind::i8); they are converted to fp32 with
// round-to-nearest, then scaled by the row's and the column's scale in that order.
// `zero` (warp-uniform): the accumulator was never written (a tile without K steps); zeros are stored
// whatever tensor memory holds.
template <bool COL_SCALE, bool ACC_INT, int NBLK, int EPI_BUFS, int RELEASE_AFTER, class Release>
__device__ __forceinline__ void epilogue_tile(uint32_t taddr, bool rev, bool zero, int64_t row0, int64_t col0, int64_t M, int64_t N,
                                              float row_scale, const float* __restrict__ scale_b, int b_scalar,
                                              const OutMaps* outs, uint32_t epi_s, uint8_t* epi_g, int& buf, int lane,
                                              Release release) {
  auto emit = [&](int c, const uint32_t (&r)[64]) {
    const int64_t colg = col0 + c * EPI_COLS;
    float sb0 = 1.f, sb1 = 1.f;
    if (COL_SCALE) {
      if (b_scalar) {
        sb0 = sb1 = __ldcg(scale_b);
      } else {
        sb0 = colg + lane < N ? __ldcg(scale_b + colg + lane) : 0.f;
        sb1 = colg + 32 + lane < N ? __ldcg(scale_b + colg + 32 + lane) : 0.f;
      }
    }
    uint32_t o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float lo = (ACC_INT ? __int2float_rn((int)r[2 * i]) : u2f(r[2 * i])) * row_scale;
      float hi = (ACC_INT ? __int2float_rn((int)r[2 * i + 1]) : u2f(r[2 * i + 1])) * row_scale;
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
      if (outs->scatter_rows > 0) {
        const int owner = (int)(row0 / outs->scatter_rows);
        ptx::tma_store_2d(&outs->m[owner], (int32_t)colg, (int32_t)(row0 - (int64_t)owner * outs->scatter_rows),
                          epi_s + buf * EPI_BLOCK_BYTES);
      } else {
        for (int g = 0; g < outs->count; ++g)
          ptx::tma_store_2d(&outs->m[g], (int32_t)colg, (int32_t)row0, epi_s + buf * EPI_BLOCK_BYTES);
      }
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
    if (zero) {
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        if (i & 1) rb[j] = 0;
        else ra[j] = 0;
      }
    }
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

// ---- MXFP8-quantized output ------------------------------------------------------------------------
// The tile leaves the kernel as what the NEXT block-scaled GEMM wants for its A operand: every
// accumulator is scaled, rounded to bf16 (the GEMM's output dtype) and then quantized exactly as
// b200q_quantize_mxfp8(axis = 1) would quantize that bf16 matrix - E4M3 codes, one E8M0 scale per 32
// columns - so 1.03 bytes per element leave the SM instead of 2.  A thread owns a row, so it owns whole
// 32-column blocks.  Two 64-column blocks make one 128-byte row of codes in the (128-byte-swizzled)
// staging block, stored by TMA to every output.  The four scale bytes of a row and a 128-column chunk are
// one aligned 32-bit word of the 128x4-tiled layout, and the 128 rows of the tile times one chunk are exactly
// one 512-byte atom of it: the four epilogue warps (one lane quarter each) put their words into a staging
// atom in shared memory, meet at a named barrier once per tile, and one lane sends every atom to every
// output with ONE bulk store - 512 bytes per store instead of 128 four-byte stores, which matters when the
// outputs are peers' buffers across NVLink (a four-byte remote store costs a whole packet).
// NBLK must be even; rows [row0, row0 + 32) and columns [col0, col0 + 64 * NBLK); row0 - 32 * q is a multiple of 128.
// sfst_g / sfst_s: this tile's staging atoms (NBLK / 2 x 512 bytes; the caller alternates two sets by
// accumulator); q: the warp's lane quarter; bar_id: a named barrier of the four epilogue warps.
template <int NBLK, int EPI_BUFS, int RELEASE_AFTER, class Release>
__device__ __forceinline__ void epilogue_tile_mxq(uint32_t taddr, bool rev, int64_t row0, int64_t col0, int64_t M, int64_t N,
                                                  float alpha, const OutMaps* outs, uint32_t epi_s, uint8_t* epi_g, int& buf,
                                                  int lane, uint8_t* sfst_g, uint32_t sfst_s, int q, int bar_id, Release release) {
  static_assert(NBLK % 2 == 0, "the quantized-output epilogue stores 128-column chunks");
  uint32_t sfw = 0;                                        // the chunk's four scale bytes, lowest block first
  auto emit = [&](int c, const uint32_t (&r)[64]) {
    const int half = c & 1;
    if (half == (rev ? 1 : 0)) {                           // first half of a chunk in walking order: claim the staging block
      if (lane == 0) ptx::bulk_wait_read<EPI_BUFS - 1>();
      __syncwarp();
      sfw = 0;
    }
    uint8_t* dst = epi_g + buf * EPI_BLOCK_BYTES + lane * 128;
    const int sw = lane & 7;
#pragma unroll
    for (int b = 0; b < 2; ++b) {                          // the two 32-column blocks of this 64-column block
      uint4 h[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i0 = 32 * b + 8 * u;
        h[u] = make_uint4(pack_bf16(u2f(r[i0]) * alpha, u2f(r[i0 + 1]) * alpha), pack_bf16(u2f(r[i0 + 2]) * alpha, u2f(r[i0 + 3]) * alpha),
                          pack_bf16(u2f(r[i0 + 4]) * alpha, u2f(r[i0 + 5]) * alpha), pack_bf16(u2f(r[i0 + 6]) * alpha, u2f(r[i0 + 7]) * alpha));
      }
      uint32_t o[8];
      const int e = mx_quant_block32<FMT_E4M3>(h, o);
      sfw |= (uint32_t)((e + 127) & 0xFF) << (8 * (2 * half + b));
      const int j0 = 4 * half + 2 * b;                      // 16-byte chunk of the 128-byte row
      *reinterpret_cast<uint4*>(dst + (((j0) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4*>(dst + (((j0 + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
    if (half == (rev ? 0 : 1)) {                           // chunk complete
      const int64_t colg = col0 + (int64_t)(c >> 1) * 128;
      // this row's word of the chunk's atom: (row % 32) * 16 + (row / 32 % 4) * 4
      *reinterpret_cast<uint32_t*>(sfst_g + (c >> 1) * 512 + lane * 16 + q * 4) = sfw;
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        for (int g = 0; g < outs->count; ++g)
          ptx::tma_store_2d(&outs->m[g], (int32_t)colg, (int32_t)row0, epi_s + buf * EPI_BLOCK_BYTES);
        ptx::bulk_commit();
      }
      buf = (buf + 1) % EPI_BUFS;
    }
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
    if (col0 + (int64_t)(c >> 1) * 128 < N && row0 < M) {  // warp-uniform; N % 128 == 0, so a chunk is in range or not as a whole
      if (i & 1) emit(c, rb);
      else emit(c, ra);
    }
  }
  // The staging atoms of the tile before the previous one are about to be rewritten by the other warps: the bulk store that
  // read them must be done (at most the newest group - this tile's last codes - may still be reading).  Then all four
  // lane quarters meet: every word of this tile's atoms is in place (every warp executes this, in range or not).
  if (q == 0 && lane == 0) ptx::bulk_wait_read<1>();
  ptx::named_bar_sync(bar_id, 128);
  if (q == 0 && lane == 0 && row0 < M) {
    const int64_t tile_row = row0;                          // q == 0: the tile's first row, a multiple of 128
#pragma unroll
    for (int j = 0; j < NBLK / 2; ++j) {
      const int64_t colg = col0 + (int64_t)j * 128;
      if (colg < N) {
        const int64_t off = sf_swizzled(tile_row, (int)(colg >> 5), outs->sf_kt);     // the atom's first byte
        for (int g = 0; g < outs->count; ++g) ptx::bulk_store(outs->sf[g] + off, sfst_s + j * 512, 512);
      }
    }
    ptx::bulk_commit();
  }
}

// ---- SwiGLU epilogues ------------------------------------------------------------------------------
// For a GEMM whose B rows come in the order "32 gate rows, then the 32 up rows of the same 32
// outputs": every 64-column accumulator block holds gate[0..32) | up[0..32) of one 32-wide block
// of h = silu(gate) * up, and a thread (one accumulator row) holds that whole block.  The thread
// rounds the scaled accumulators to bf16 (the reference's GEMM output dtype) and applies the same
// SwiGLU arithmetic as the stand-alone kernel; the bf16 [M, 2I] intermediate never exists.  Then
//   GLU_MX   : the block is exactly one MXFP8 block along the next GEMM's contraction dimension:
//              quantize, write 32 code bytes and one scale byte;
//   GLU_BF16 : write the 32 bf16 values and fold them into the tensor's absolute maximum (what an
//              NVFP4 quantization of h needs before it can start), one atomic per warp and tile.
enum { GLU_MX = 0, GLU_BF16 = 1 };

struct GluOut {
  uint8_t* codes;   // GLU_MX: [M, N/2] E4M3 codes; GLU_BF16: [M, N/2] bf16; pitch ldh BYTES
  int64_t ldh;
  uint8_t* sf;      // GLU_MX: 128x4-tiled E8M0 scale factors over (M, N/64)
  int64_t kt;       // K-tiles per row tile of that layout
  float* amax;      // GLU_BF16: max |h| over the tensor (zeroed before the launch)
  int wide;         // codes and ldh are 32-byte aligned: a lane's 32 bytes go out as one 256-bit store (a whole sector)
};

// Two warps share each tensor-memory lane quarter here (the arithmetic per block is long):
// warp group `grp` of NGRP takes the blocks whose walking index i has i % NGRP == grp, and hands
// the accumulator back once ITS blocks among the first RELEASE_AFTER + 1 have been read.
template <int OUT, int NBLK, int RELEASE_AFTER, int NGRP, class Release>
__device__ __forceinline__ void epilogue_tile_glu(uint32_t taddr, bool rev, int grp, int64_t row, int64_t col0, int64_t M,
                                                  int64_t N, float alpha, const GluOut& out, Release release) {
  uint32_t hmax = 0;   // packed |bf16| maxima of this thread's h values (GLU_BF16)
  auto emit = [&](int c, const uint32_t (&r)[64]) {
    uint4 h[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint4 vg = make_uint4(pack_bf16(u2f(r[8 * u]) * alpha, u2f(r[8 * u + 1]) * alpha),
                                  pack_bf16(u2f(r[8 * u + 2]) * alpha, u2f(r[8 * u + 3]) * alpha),
                                  pack_bf16(u2f(r[8 * u + 4]) * alpha, u2f(r[8 * u + 5]) * alpha),
                                  pack_bf16(u2f(r[8 * u + 6]) * alpha, u2f(r[8 * u + 7]) * alpha));
      const uint4 vu = make_uint4(pack_bf16(u2f(r[32 + 8 * u]) * alpha, u2f(r[33 + 8 * u]) * alpha),
                                  pack_bf16(u2f(r[34 + 8 * u]) * alpha, u2f(r[35 + 8 * u]) * alpha),
                                  pack_bf16(u2f(r[36 + 8 * u]) * alpha, u2f(r[37 + 8 * u]) * alpha),
                                  pack_bf16(u2f(r[38 + 8 * u]) * alpha, u2f(r[39 + 8 * u]) * alpha));
      h[u] = swiglu8(vg, vu);
    }
    const int64_t hb = (col0 + c * EPI_COLS) >> 6;   // 32-wide block of h along the row
    if (OUT == GLU_MX) {
      uint32_t o[8];
      const int e = mx_quant_block32<FMT_E4M3>(h, o);
      if (row < M) {
        uint8_t* dst = out.codes + row * out.ldh + hb * 32;
        if (out.wide) st_32B<true>(dst, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
        else st_32B<false>(dst, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
        out.sf[sf_swizzled(row, (int)hb, out.kt)] = (uint8_t)(e + 127);
      }
    } else if (row < M) {
      uint8_t* dst = out.codes + row * out.ldh + hb * 64;
      if (out.wide) { st_32B<true>(dst, h[0], h[1]); st_32B<true>(dst + 32, h[2], h[3]); }
      else { st_32B<false>(dst, h[0], h[1]); st_32B<false>(dst + 32, h[2], h[3]); }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        hmax = absmax_raw_bf16x2(hmax, absmax_raw_bf16x2(h[u].x, h[u].y));
        hmax = absmax_raw_bf16x2(hmax, absmax_raw_bf16x2(h[u].z, h[u].w));
      }
    }
  };

  // last walking index <= RELEASE_AFTER that belongs to this group (-1: none)
  const int my_last = RELEASE_AFTER - ((RELEASE_AFTER - grp) % NGRP + NGRP) % NGRP;
  if (my_last < 0) release();
  uint32_t r[64];
  // not unrolled: one copy of the (long) block body keeps the epilogue inside the instruction cache
#pragma unroll 1
  for (int i = 0; i < NBLK; ++i) {
    if (i % NGRP != grp) continue;                        // warp-uniform
    const int c = rev ? NBLK - 1 - i : i;
    const bool valid = col0 + c * EPI_COLS < N;           // warp-uniform
    if (valid) {
      tmem_ld64(taddr + c * EPI_COLS, r);
      ptx::tmem_ld_wait();
    }
    if (i == my_last) release();
    if (valid) emit(c, r);
  }
  if (OUT == GLU_BF16) {
    float a = absmax_halves(hmax);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmax_nan(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
    // a >= 0 or NaN: the unsigned order of the bits is the float order, with NaN above everything
    if ((threadIdx.x & 31) == 0 && !(a <= 0.f)) atomicMax(reinterpret_cast<unsigned int*>(out.amax), f2u(a));
  }
}
