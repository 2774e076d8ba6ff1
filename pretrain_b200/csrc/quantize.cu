// Quantize kernels: amax, FP8 and the int8 series (per-row / per-column / per-tensor fp32
// scales), MXFP8 (32-element blocks, E8M0 scales) and NVFP4 (16-element blocks, E4M3 scales +
// fp32 tensor scale), each in a row-wise form (contraction dimension contiguous in the input)
// and a transposing form (contraction dimension = input rows; output written transposed), plus
// the forms that produce both directions of one tensor (MXFP8 in one read, FP8 in two).
//
// All of them are HBM-bound streaming kernels: 16- or 32-byte loads with several in flight per
// thread, block maxima inside one thread (block-scaled formats) or warp-shuffle reductions
// (row maxima), hardware fp8 / fp4 conversion instructions, 8- to 32-byte stores.  Arithmetic is
// the bit-exact core in numeric.cuh (reference formulas: src/quant/fp8.py:16-32,
// src/quant/int8.py:9-19).
#include "common.cuh"

namespace b200q {

int require_sm100() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_ok = 0;
  int dev = -1;
  B200Q_CUDA(cudaGetDevice(&dev));
  if (dev != cached_dev) {
    int major = 0;
    B200Q_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    cached_dev = dev;
    cached_ok = (major == 10);
  }
  return cached_ok ? B200Q_OK : B200Q_ERR_NOT_SM100;
}

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmax_nan(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));   // a NaN reaches every lane
  return v;
}

// ------------------------------------------------------------------------------------------
// amax over a matrix
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) amax_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols,
                                                        int64_t ld, float* __restrict__ amax) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t m = 0;
  // work item = (row, 1024-column chunk); items are dealt round-robin to all warps of the grid
  const int chunks = (int)((cols + 1023) >> 10), ncols = (int)cols;
  for (ItemWalker w((int64_t)blockIdx.x * kWarps + warp, (int64_t)gridDim.x * kWarps, chunks); w.row < rows; w.next()) {
    const int c0 = w.chunk << 10;
    const uint16_t* xr = x + w.row * ld + c0;
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = u * 256 + lane * 8;
      v[u] = c0 + c < ncols ? ld_nc_v4(xr + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(v[u].x, v[u].y));
      m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(v[u].z, v[u].w));
    }
  }
  float a = warp_max(absmax_halves(m));
  __shared__ float s[kWarps];
  if (lane == 0) s[warp] = a;
  __syncthreads();
  if (warp == 0) {
    a = warp_max(lane < kWarps ? s[lane] : 0.f);
    // a >= 0 or NaN: the unsigned order of the bits is the float order, with NaN above everything
    if (lane == 0) atomicMax(reinterpret_cast<unsigned int*>(amax), f2u(a));
  }
}

// ------------------------------------------------------------------------------------------
// Row-wise block quantizers (MXFP8 / NVFP4).  The work item is a run of 32 consecutive elements
// of a row (one MX block, or two NV blocks) and belongs to ONE thread: block maximum, scale and
// scale-factor store happen once per block with no shuffles.  Items are dealt round-robin to
// the threads of the grid, so the lanes of a warp read consecutive 64-byte runs (two 32-byte
// sectors each, as 256-bit loads when the pitch allows) whatever the row length, and write 32
// (MX) or 16 (NV) contiguous code bytes.
// ------------------------------------------------------------------------------------------
enum { MODE_MX = 0, MODE_NV = 1, MODE_FP8 = 2 };

// One matrix to quantize row-wise: bf16 [rows, cols] pitch ld -> codes [rows, cols] (+ scale factors), input row r
// written as output row dst_row[r] when a map is given.
struct RowQuantJob {
  const uint16_t* x;
  int64_t rows, cols, ld;
  uint8_t* codes;
  uint8_t* sf;
  const int32_t* dst_row;
  int trigger_early;     // (first job only) an attributed kernel that waits is launched directly behind this one
};

// Up to two matrices per launch (MXFP8 only; second.rows == 0: one matrix): both operands of a GEMM quantized by one
// grid, each thread taking its round-robin share of the first matrix's runs and then of the second's.
template <int MODE, bool WIDE, int FMT>
__global__ void __launch_bounds__(kThreads)
rowwise_block_quant_kernel(const RowQuantJob first, const RowQuantJob second, int swz,
                           const float* __restrict__ tensor_amax, float* __restrict__ tensor_scale_out) {
  if (first.trigger_early) grid_launch_dependents();   // the whole grid is resident: the GEMM behind this kernel may set up now
  pdl_prologue();
  constexpr int BS = MODE == MODE_MX ? 32 : 16;
  float s_t = 0.f, rcp_st = 0.f;
  if (MODE == MODE_NV) {
    s_t = nv_tensor_scale(*tensor_amax);
    rcp_st = rcp_rn(s_t);
    if (blockIdx.x == 0 && threadIdx.x == 0) *tensor_scale_out = s_t;
  }
#pragma unroll 1
  for (int t = 0; t < 2; ++t) {
    const RowQuantJob& job = t == 0 ? first : second;
    if (job.rows == 0) continue;
    const uint16_t* __restrict__ x = job.x;
    uint8_t* __restrict__ codes = job.codes;
    uint8_t* __restrict__ sf = job.sf;
    const int32_t* __restrict__ dst_row = job.dst_row;
    const int64_t rows = job.rows, cols = job.cols, ld = job.ld;
    const int64_t nblk = cols / BS;
    const int runs = (int)(cols >> 5);            // 32-element runs per row
    const int64_t kt = (nblk + 3) >> 2;
    // NVFP4 keeps the NEXT item's 64 bytes in flight while it works on this one (its arithmetic per byte is several
    // times MXFP8's, and without this a warp alternates between waiting and computing): 36.9 -> 35.2 us on an
    // 8192 x 8192 operand, 33.2 us with the pair of scale bytes stored as one 16-bit word.  MXFP8 gains nothing from it.
    constexpr bool kAhead = MODE == MODE_NV;
    ItemWalker w((int64_t)blockIdx.x * kThreads + threadIdx.x, (int64_t)gridDim.x * kThreads, runs);
    uint4 v[4];
    auto load = [&](uint4 (&d)[4]) {
      const uint16_t* xp = x + w.row * ld + (w.chunk << 5);
      ld_nc_32B<WIDE>(xp, d[0], d[1]);
      ld_nc_32B<WIDE>(xp + 16, d[2], d[3]);
    };
    if (kAhead && w.row < rows) load(v);
    while (w.row < rows) {
      const int64_t in_row = w.row;
      const int chunk = w.chunk, c = chunk << 5;
      uint4 nxt[4];
      if (kAhead) {
        w.next();
        if (w.row < rows) load(nxt);
      } else {
        load(v);
        w.next();
      }
      const int64_t row = dst_row ? (int64_t)__ldcg(dst_row + in_row) : in_row;   // output row (codes and scale factors)
      if (MODE == MODE_MX) {
        uint32_t o[8];
        const int e = mx_quant_block32<FMT>(v, o);
        st_32B<WIDE>(codes + row * cols + c, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
        sf[swz ? sf_swizzled(row, chunk, kt) : row * nblk + chunk] = (uint8_t)(e + 127);
      } else {
        uint32_t o[4];
        uint32_t sq2 = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float a = fmax_nan(absmax8(v[2 * h]), absmax8(v[2 * h + 1]));
          const uint8_t sq = nv_block_scale_fast(a, s_t, rcp_st);
          const float eff = mul_rn(e4m3_to_float(sq), s_t);
          const QuotScale qs = quot_scale(eff, rcp_rn(eff));
          sq2 |= (uint32_t)sq << (8 * h);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float f[8];
            quot8_for_cast(v[2 * h + q], qs, f);
            uint32_t tt = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) tt |= (uint32_t)cvt_e2m1x2(f[2 * i], f[2 * i + 1]) << (8 * i);
            o[2 * h + q] = sq != 0 ? tt : 0u;
          }
        }
        *reinterpret_cast<uint4*>(codes + ((row * cols + c) >> 1)) = make_uint4(o[0], o[1], o[2], o[3]);
        const int kb = 2 * chunk;   // even: the pair of scale bytes is adjacent in both layouts
        uint8_t* sp = sf + (swz ? sf_swizzled(row, kb, kt) : row * nblk + kb);
        if ((reinterpret_cast<uintptr_t>(sp) & 1) == 0) {     // one store instead of two: each costs the warp 16 sectors
          *reinterpret_cast<uint16_t*>(sp) = (uint16_t)sq2;
        } else {
          sp[0] = (uint8_t)sq2;
          sp[1] = (uint8_t)(sq2 >> 8);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = nxt[i];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Row-wise FP8 with one fp32 scale per row (or one for the tensor).  `wpr` warps (1, 2, 4 or 8)
// share a row and keep it in registers between the amax pass and the conversion pass (NVEC
// 16-byte vectors per lane; partial maxima meet in shared memory).  NVEC == 0 re-reads the row
// (it is still in L2) for rows too long for that.
// ------------------------------------------------------------------------------------------
// COLMAX: the same pass also reduces |x| down the columns (for the per-column scales of the transposed
// copy of the same tensor): every thread keeps the maxima of its columns over the rows it visits, the
// CTA merges its row groups in shared memory and writes one row of partial maxima (packed bf16) per CTA.
template <int NVEC, int FMT, bool COLMAX = false>
__global__ void __launch_bounds__(kThreads)
rowwise_fp8_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                   uint8_t* __restrict__ codes, float* __restrict__ scales, const float* __restrict__ tensor_amax,
                   float* __restrict__ tensor_scale_out, int wpr, float qmax, unsigned int* __restrict__ col_partials = nullptr) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int fmt = FMT;
  const int grp = warp / wpr, wig = warp - grp * wpr, rpc = kWarps / wpr;
  __shared__ float smax[2][kWarps];
  extern __shared__ unsigned int colmax_s[];            // COLMAX: [row groups of the CTA][cols / 2] packed bf16 pairs
  uint32_t cm[COLMAX && NVEC > 0 ? NVEC * 4 : 1] = {};
  int it = 0;
  for (int64_t base = (int64_t)blockIdx.x * rpc; base < rows; base += (int64_t)gridDim.x * rpc, ++it) {
    const int64_t row = base + grp;
    const bool live = row < rows;
    const uint16_t* xr = x + (live ? row : 0) * ld;
    uint4 v[NVEC > 0 ? NVEC : 1];
    uint32_t m = 0;
    if (NVEC > 0) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        int64_t c = (int64_t)((i * wpr + wig) * 32 + lane) * 8;
        v[i] = (live && c < cols) ? ld_nc_v4(xr + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(v[i].x, v[i].y));
        m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(v[i].z, v[i].w));
        if (COLMAX) {                                   // signs cleared when the maxima are parked below
          cm[4 * i] = absmax_raw_bf16x2(cm[4 * i], v[i].x);
          cm[4 * i + 1] = absmax_raw_bf16x2(cm[4 * i + 1], v[i].y);
          cm[4 * i + 2] = absmax_raw_bf16x2(cm[4 * i + 2], v[i].z);
          cm[4 * i + 3] = absmax_raw_bf16x2(cm[4 * i + 3], v[i].w);
        }
      }
    } else if (tensor_amax == nullptr && live) {
      for (int64_t c = (wig * 32 + lane) * 8; c < cols; c += 256 * wpr) {
        uint4 t = ld_nc_v4(xr + c);
        m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(t.x, t.y));
        m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(t.z, t.w));
      }
    }
    float amax = warp_max(absmax_halves(m));
    if (wpr > 1) {
      if (lane == 0) smax[it & 1][warp] = amax;
      __syncthreads();
      for (int j = 0; j < wpr; ++j) amax = fmax_nan(amax, smax[it & 1][grp * wpr + j]);
    }
    if (tensor_amax) amax = *tensor_amax;
    const float scale = scale_from_amax(amax, fmt, qmax);
    const float rcp = rcp_rn(scale);
    if (lane == 0 && wig == 0 && live) {
      if (tensor_amax == nullptr) scales[row] = scale;
      else if (row == 0) *tensor_scale_out = scale;
    }
    uint8_t* cr = codes + (live ? row : 0) * cols;
    if (NVEC > 0) {
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        int64_t c = (int64_t)((i * wpr + wig) * 32 + lane) * 8;
        float f[8];
        unpack8(v[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = quot_for_cast(f[j], scale, rcp);
        uint2 o;
        o.x = cvt_codes_x4(f[0], f[1], f[2], f[3], fmt, qmax);
        o.y = cvt_codes_x4(f[4], f[5], f[6], f[7], fmt, qmax);
        if (live && c < cols) *reinterpret_cast<uint2*>(cr + c) = o;
      }
    } else if (live) {
      for (int64_t c = (wig * 32 + lane) * 8; c < cols; c += 256 * wpr) {
        float f[8];
        unpack8(ld_nc_v4(xr + c), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = quot_for_cast(f[j], scale, rcp);
        uint2 o;
        o.x = cvt_codes_x4(f[0], f[1], f[2], f[3], fmt, qmax);
        o.y = cvt_codes_x4(f[4], f[5], f[6], f[7], fmt, qmax);
        *reinterpret_cast<uint2*>(cr + c) = o;
      }
    }
  }
  if (COLMAX && NVEC > 0) {
    const int64_t half = cols >> 1;                    // words per row group
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int64_t c = (int64_t)((i * wpr + wig) * 32 + lane) * 8;
      if (c < cols)
        *reinterpret_cast<uint4*>(&colmax_s[grp * half + (c >> 1)]) =
            make_uint4(abs_bf16x2(cm[4 * i]), abs_bf16x2(cm[4 * i + 1]), abs_bf16x2(cm[4 * i + 2]), abs_bf16x2(cm[4 * i + 3]));
    }
    __syncthreads();
    for (int64_t wi = threadIdx.x; wi < half; wi += kThreads) {
      uint32_t m = colmax_s[wi];
      for (int g2 = 1; g2 < rpc; ++g2) m = absmax_bf16x2(m, colmax_s[g2 * half + wi]);
      col_partials[(int64_t)blockIdx.x * half + wi] = m;
    }
  }
}

// scales[c] = scale(max over the CTAs' partial column maxima)
constexpr int kRedWords = 8, kRedSlices = 128;        // a CTA: 8 packed column pairs (one 32-byte sector per row) x 128 row slices
__global__ void __launch_bounds__(kRedWords * kRedSlices)
col_partials_to_scale_kernel(const unsigned int* __restrict__ partials, int nparts, int64_t cols, int fmt, float qmax,
                             float* __restrict__ scales) {
  pdl_prologue();
  // few loads per thread (nparts / 128), many CTAs: the reduction is a chain of load latencies, not of bytes
  __shared__ uint32_t red[kRedSlices][kRedWords + 1];
  const int tx = threadIdx.x & (kRedWords - 1), ty = threadIdx.x / kRedWords;
  const int64_t wi = (int64_t)blockIdx.x * kRedWords + tx, half = cols >> 1;
  uint32_t m = 0;
  if (wi < half)
    for (int p = ty; p < nparts; p += kRedSlices) m = absmax_bf16x2(m, partials[(int64_t)p * half + wi]);
  red[ty][tx] = m;
  __syncthreads();
  if (ty < 8) {                                        // 128 slices -> 8 -> 1
    for (int j = ty + 8; j < kRedSlices; j += 8) m = absmax_bf16x2(m, red[j][tx]);
    red[ty][tx] = m;
  }
  __syncthreads();
  if (ty == 0 && wi < half) {
#pragma unroll
    for (int j = 1; j < 8; ++j) m = absmax_bf16x2(m, red[j][tx]);
    scales[2 * wi] = scale_from_amax(bf16lo(m), fmt, qmax);
    scales[2 * wi + 1] = scale_from_amax(bf16hi(m), fmt, qmax);
  }
}

// ------------------------------------------------------------------------------------------
// Per-column amax (for FP8 scales that run along the rows), then amax -> scale in place.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
col_amax_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols, int64_t ld, unsigned int* __restrict__ amax_bits) {
  pdl_prologue();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = ((int64_t)blockIdx.x * 32 + tx) * 8;
  uint32_t m[4] = {0, 0, 0, 0};
  if (c < cols) {
    for (int64_t r0 = (int64_t)blockIdx.y * kWarps * 4 + ty; r0 < rows; r0 += (int64_t)gridDim.y * kWarps * 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int64_t r = r0 + u * kWarps;
        v[u] = r < rows ? ld_nc_v4(x + r * ld + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        m[0] = absmax_raw_bf16x2(m[0], v[u].x); m[1] = absmax_raw_bf16x2(m[1], v[u].y);
        m[2] = absmax_raw_bf16x2(m[2], v[u].z); m[3] = absmax_raw_bf16x2(m[3], v[u].w);
      }
    }
  }
  __shared__ uint32_t s[kWarps][32][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[ty][tx][i] = abs_bf16x2(m[i]);
  __syncthreads();
  if (ty == 0 && c < cols) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t a = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) a = absmax_bf16x2(a, s[w][tx][i]);
      atomicMax(amax_bits + c + 2 * i, f2u(bf16lo(a)));
      atomicMax(amax_bits + c + 2 * i + 1, f2u(bf16hi(a)));
    }
  }
}

__global__ void amax_to_scale_kernel(float* __restrict__ scales, int64_t n, int fmt, float qmax) {
  pdl_prologue();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scales[i] = scale_from_amax(scales[i], fmt, qmax);
}

// ------------------------------------------------------------------------------------------
// Transposing quantizers: scales run along the input rows; codes are written transposed.
// A CTA stages a 128-row x 64-column bf16 tile in shared memory (16-byte coalesced loads, four
// in flight per thread); each thread then owns one column and a run of 32 rows, and the code
// tile goes back out through shared memory as 128-byte (64-byte for FP4) row segments.
// ------------------------------------------------------------------------------------------
constexpr int kTR = 128, kTC = 64;

template <int MODE, int FMT>
__global__ void __launch_bounds__(kThreads)
transpose_quant_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                       uint8_t* __restrict__ codes, uint8_t* __restrict__ sf, int swz,
                       const float* __restrict__ col_scales, const float* __restrict__ tensor_amax,
                       float* __restrict__ tensor_scale_out, float qmax) {
  pdl_prologue();
  __shared__ __align__(16) uint16_t tin[kTR * kTC];
  constexpr int OUT_PITCH = (MODE == MODE_NV ? kTR / 2 : kTR) + 16;
  __shared__ __align__(16) uint8_t tout[kTC * OUT_PITCH];
  constexpr int fmt = FMT;
  const int tid = threadIdx.x;
  const int64_t c0 = (int64_t)blockIdx.x * kTC, r0 = (int64_t)blockIdx.y * kTR;

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = i * kThreads + tid, r = id >> 3, ch = id & 7;
    const int64_t gr = r0 + r, gc = c0 + ch * 8;
    uint4 v = (gr < rows && gc < cols) ? ld_nc_v4(x + gr * ld + gc) : make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(&tin[r * kTC + ch * 8]) = v;
  }
  float s_t = 0.f, t_scale = 0.f, rcp_st = 0.f;
  if (MODE == MODE_NV) {
    s_t = nv_tensor_scale(*tensor_amax);
    rcp_st = rcp_rn(s_t);
    if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) *tensor_scale_out = s_t;
  }
  if (MODE == MODE_FP8 && tensor_amax != nullptr) {
    t_scale = scale_from_amax(*tensor_amax, fmt, qmax);
    if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) *tensor_scale_out = t_scale;
  }
  __syncthreads();

  const int c = tid & 63, j = tid >> 6;
  const int64_t gc = c0 + c, gr = r0 + 32 * j;
  float f[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = u2f((uint32_t)tin[(32 * j + i) * kTC + c] << 16);

  if (MODE == MODE_MX) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) a = fmax_nan(a, fabsf(f[i]));
    const int e = mx_scale_exp(a, fmt);
    const float inv = mx_inv_scale(e);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = cvt_fp8x4(f[4 * i] * inv, f[4 * i + 1] * inv, f[4 * i + 2] * inv, f[4 * i + 3] * inv, fmt);
    uint4* dst = reinterpret_cast<uint4*>(&tout[c * OUT_PITCH + 32 * j]);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    if (gc < cols && gr < rows) sf[sf_offset(gc, gr >> 5, rows >> 5, swz)] = (uint8_t)(e + 127);
  } else if (MODE == MODE_NV) {
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) a = fmax_nan(a, fabsf(f[16 * h + i]));
      const uint8_t sq = nv_block_scale_fast(a, s_t, rcp_st);
      const float eff = mul_rn(e4m3_to_float(sq), s_t);
      const float rcp = rcp_rn(eff);
      o[2 * h] = o[2 * h + 1] = 0;
      if (sq != 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint32_t b = cvt_e2m1x2(quot_for_cast(f[16 * h + 2 * i], eff, rcp), quot_for_cast(f[16 * h + 2 * i + 1], eff, rcp));
          o[2 * h + (i >> 2)] |= b << (8 * (i & 3));
        }
      }
      if (gc < cols && gr + 16 * h < rows) sf[sf_offset(gc, (gr >> 4) + h, rows >> 4, swz)] = sq;
    }
    *reinterpret_cast<uint4*>(&tout[c * OUT_PITCH + 16 * j]) = make_uint4(o[0], o[1], o[2], o[3]);
  } else {
    const float scale = tensor_amax ? t_scale : (gc < cols ? col_scales[gc] : 1.f);
    const float rcp = rcp_rn(scale);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      o[i] = cvt_codes_x4(quot_for_cast(f[4 * i], scale, rcp), quot_for_cast(f[4 * i + 1], scale, rcp),
                          quot_for_cast(f[4 * i + 2], scale, rcp), quot_for_cast(f[4 * i + 3], scale, rcp), fmt, qmax);
    uint4* dst = reinterpret_cast<uint4*>(&tout[c * OUT_PITCH + 32 * j]);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  __syncthreads();

  if (MODE == MODE_NV) {
    const int oc = tid >> 2, ch = tid & 3;
    if (c0 + oc < cols && r0 + ch * 32 < rows)
      *reinterpret_cast<uint4*>(codes + (c0 + oc) * (rows >> 1) + (r0 >> 1) + ch * 16) =
          *reinterpret_cast<const uint4*>(&tout[oc * OUT_PITCH + ch * 16]);
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int id = i * kThreads + tid, oc = id >> 3, ch = id & 7;
      if (c0 + oc < cols && r0 + ch * 16 < rows)
        *reinterpret_cast<uint4*>(codes + (c0 + oc) * rows + r0 + ch * 16) =
            *reinterpret_cast<const uint4*>(&tout[oc * OUT_PITCH + ch * 16]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// MXFP8 in both directions from one read of the input: row-wise codes/scales (blocks along the
// columns) for the GEMM that contracts over the columns, and transposed codes/scales (blocks
// along the rows) for the GEMM that contracts over the rows - what a linear layer needs of an
// activation (fprop + wgrad), of a weight (fprop + dgrad) and of an output gradient (dgrad +
// wgrad).  Results equal the two single-direction kernels byte for byte.
//
// A CTA takes a 128 x 128 tile.  Phase 1: every thread loads two runs of 32 consecutive elements
// of a row (64 bytes each), quantizes them row-wise straight from registers and parks the
// bf16 values in shared memory (row pitch 272 bytes: 16-byte stores without bank conflicts).
// Phase 2: a thread owns TWO adjacent columns and 32 rows: 32 four-byte shared-memory loads give
// it both columns as packed bf16 pairs, the block maxima come from packed max instructions, and
// the codes go to a staging tile (which reuses the input tile's memory once every thread holds
// its columns in registers).  Phase 3 writes that tile out as 128-byte rows of the transposed
// matrix.
// ------------------------------------------------------------------------------------------
constexpr int kDT = 128;                    // tile edge
constexpr int kDPitch = kDT * 2 + 16;       // bytes per staged input row
constexpr int kDOutPitch = kDT + 16;        // bytes per staged output row (= input column)
constexpr int kDualSmem = kDT * kDPitch;     // the output staging tile reuses the input tile's memory

// Steps the tile kernels share.  A thread's two columns x 32 rows of codes go to the staging tile
// (row = column of the input), then the tile leaves as 128-byte rows of the transposed matrix.
__device__ __forceinline__ void tile_park_columns(uint8_t* tout, int cp, int j, const uint32_t (&o0)[8], const uint32_t (&o1)[8]) {
  uint4* d0 = reinterpret_cast<uint4*>(tout + (2 * cp) * kDOutPitch + 32 * j);
  uint4* d1 = reinterpret_cast<uint4*>(tout + (2 * cp + 1) * kDOutPitch + 32 * j);
  d0[0] = make_uint4(o0[0], o0[1], o0[2], o0[3]); d0[1] = make_uint4(o0[4], o0[5], o0[6], o0[7]);
  d1[0] = make_uint4(o1[0], o1[1], o1[2], o1[3]); d1[1] = make_uint4(o1[4], o1[5], o1[6], o1[7]);
}
// `first_col` = the tile's first column in the output, `c0` / `width` = its position and limit in the part it belongs to
__device__ __forceinline__ void tile_store_transposed(const uint8_t* tout, int tid, int64_t first_col, int64_t c0, int64_t width,
                                                      int64_t r0, int64_t rows, uint8_t* __restrict__ codes_c) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = i * kThreads + tid, oc = id >> 3, ch = id & 7;
    if (c0 + oc < width && r0 + ch * 16 < rows)
      *reinterpret_cast<uint4*>(codes_c + (first_col + oc) * rows + r0 + ch * 16) =
          *reinterpret_cast<const uint4*>(tout + oc * kDOutPitch + ch * 16);
  }
}

// Where the tile kernel gets its values from: a matrix in memory, or one of the element-wise steps of
// the MoE expert path computed on the fly, so that the bf16 tensor between that step and its two
// MXFP8 copies never exists.
enum { SRC_PLAIN = 0, SRC_GATHER = 1, SRC_SCALED_GATHER = 2, SRC_SWIGLU = 3, SRC_SWIGLU_BWD = 4 };
struct TileSrc {
  const uint16_t* x;       // PLAIN / GATHER: the matrix; SCALED_GATHER: dout [T, cols]; SWIGLU(_BWD): g = [gate | up] [rows, 2I]
  int64_t ld;
  const int32_t* index;    // GATHER: source row of every output row (-1: zero row); SCALED_GATHER: routed pair of every row (-1: zero row)
  const uint16_t* w;       // SCALED_GATHER: routing weight of every pair (bf16)
  int k;                   //                slots per token (token = pair / k)
  const uint16_t* dh;      // SWIGLU_BWD: gradient of h [rows, I]
  int64_t lddh;
  int64_t I;               // SWIGLU: cols == I; SWIGLU_BWD: cols == 2 I (gate half, then up half)
  const uint16_t* y;       // SCALED_GATHER, optional: expert outputs [rows, cols]; <dout[token], y[row]> per row and
  int64_t ldy;             //                column tile goes to dot_partial[column tile][row] (the routing weights' gradient)
  float* dot_partial;
  const int32_t* live_tiles;   // optional (device): only the first *live_tiles 128-row tiles are processed (the rows of the
                               // padded expert-sorted layout that are in use); the outputs past them are left untouched
};

template <int SRC, bool WIDE>
__device__ __forceinline__ void load_run(const TileSrc& s, int64_t gr, int64_t gc, uint4 (&v)[4], float& dot) {
  if (SRC == SRC_PLAIN) {
    const uint16_t* xp = s.x + gr * s.ld + gc;
    ld_nc_32B<WIDE>(xp, v[0], v[1]);
    ld_nc_32B<WIDE>(xp + 16, v[2], v[3]);
  } else if (SRC == SRC_GATHER) {
    const int src = s.index[gr];
    if (src >= 0) {
      const uint16_t* xp = s.x + (int64_t)src * s.ld + gc;
      ld_nc_32B<WIDE>(xp, v[0], v[1]);
      ld_nc_32B<WIDE>(xp + 16, v[2], v[3]);
    }
  } else if (SRC == SRC_SCALED_GATHER) {
    const int pair = s.index[gr];
    if (pair >= 0) {
      const float wj = u2f((uint32_t)s.w[pair] << 16);
      const uint16_t* xp = s.x + (int64_t)(pair / s.k) * s.ld + gc;
      uint4 t[4], ty[4] = {};
      ld_nc_32B<WIDE>(xp, t[0], t[1]);
      ld_nc_32B<WIDE>(xp + 16, t[2], t[3]);
      if (s.y != nullptr) {
        const uint16_t* yp = s.y + gr * s.ldy + gc;
        ld_nc_32B<WIDE>(yp, ty[0], ty[1]);
        ld_nc_32B<WIDE>(yp + 16, ty[2], ty[3]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8], fy[8];
        unpack8(t[u], f);
        unpack8(ty[u], fy);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(f[i], fy[i], dot);
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 pk = __floats2bfloat162_rn(wj * f[2 * i], wj * f[2 * i + 1]);
          o[i] = *reinterpret_cast<uint32_t*>(&pk);
        }
        v[u] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else if (SRC == SRC_SWIGLU) {
    const uint16_t* gp = s.x + gr * s.ld + gc;
    uint4 vg[4], vu[4];
    ld_nc_32B<WIDE>(gp, vg[0], vg[1]);
    ld_nc_32B<WIDE>(gp + 16, vg[2], vg[3]);
    ld_nc_32B<WIDE>(gp + s.I, vu[0], vu[1]);
    ld_nc_32B<WIDE>(gp + s.I + 16, vu[2], vu[3]);
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = swiglu8(vg[u], vu[u]);
  }
}

// SWIGLU_BWD: one evaluation of the backward gives the run of the gate half (columns lc .. lc+31)
// and the run of the up half (columns I + lc ..) together.
template <bool WIDE>
__device__ __forceinline__ void load_run_swiglu_bwd(const TileSrc& s, int64_t gr, int64_t lc, uint4 (&dgate)[4], uint4 (&dup)[4]) {
  const uint16_t* gp = s.x + gr * s.ld + lc;
  const uint16_t* dp = s.dh + gr * s.lddh + lc;
  uint4 vg[4], vu[4], vd[4];
  ld_nc_32B<WIDE>(gp, vg[0], vg[1]);
  ld_nc_32B<WIDE>(gp + 16, vg[2], vg[3]);
  ld_nc_32B<WIDE>(gp + s.I, vu[0], vu[1]);
  ld_nc_32B<WIDE>(gp + s.I + 16, vu[2], vu[3]);
  ld_nc_32B<WIDE>(dp, vd[0], vd[1]);
  ld_nc_32B<WIDE>(dp + 16, vd[2], vd[3]);
#pragma unroll
  for (int u = 0; u < 4; ++u) swiglu_bwd8(vg[u], vu[u], vd[u], dgate[u], dup[u]);
}

// SWIGLU_BWD tiles come in pairs: the CTA at column tile c takes columns [c, c + 128) of the gate half
// and of the up half (two staged tiles), so the backward is evaluated once per element.
template <int SRC> __host__ __device__ constexpr int tile_parts() { return SRC == SRC_SWIGLU_BWD ? 2 : 1; }

template <int FMT, bool WIDE, int SRC = SRC_PLAIN>
__global__ void __launch_bounds__(kThreads)
mx_tile_quant_kernel(const TileSrc src, int64_t rows, int64_t cols, uint8_t* __restrict__ codes_r,
                     uint8_t* __restrict__ sf_r, uint8_t* __restrict__ codes_c, uint8_t* __restrict__ sf_c, int swz) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t dual_smem[];
  constexpr int NT = tile_parts<SRC>();
  // part t covers columns [t * width + c0, ...) below (t + 1) * width of the output matrix
  const int64_t width = NT == 2 ? src.I : cols;
  const int tid = threadIdx.x;
  const int64_t c0 = (int64_t)blockIdx.x * kDT, r0 = (int64_t)blockIdx.y * kDT;
  if (src.live_tiles != nullptr && r0 >= ((int64_t)__ldcg(src.live_tiles) << 7)) return;      // CTA-uniform: kDT == 128
  const int64_t nblk_r = cols >> 5, kt_r = (nblk_r + 3) >> 2;

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int item = i * kThreads + tid, r = item >> 2, q = item & 3;     // 4 runs of 32 per tile row
    const int64_t gr = r0 + r, lc = c0 + q * 32;
    const bool live = gr < rows && lc < width;                            // width % 32 == 0: a run is whole or absent
    uint4 v[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int u = 0; u < 4; ++u) v[t][u] = make_uint4(0, 0, 0, 0);
    float dot = 0.f;
    if (live) {
      if constexpr (NT == 2) load_run_swiglu_bwd<WIDE>(src, gr, lc, v[0], v[1]);
      else load_run<SRC, WIDE>(src, gr, lc, v[0], dot);
    }
    if constexpr (SRC == SRC_SCALED_GATHER) {
      if (src.dot_partial != nullptr) {                 // the four lanes q = 0..3 of a row are neighbours
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        if (q == 0 && gr < rows) src.dot_partial[(int64_t)blockIdx.x * rows + gr] = dot;
      }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      uint4* dst = reinterpret_cast<uint4*>(dual_smem + t * kDualSmem + r * kDPitch + q * 64);
      dst[0] = v[t][0]; dst[1] = v[t][1]; dst[2] = v[t][2]; dst[3] = v[t][3];
      if (live) {
        const int64_t gc = t * width + lc;
        uint32_t o[8];
        const int e = mx_quant_block32<FMT>(v[t], o);
        st_32B<WIDE>(codes_r + gr * cols + gc, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
        sf_r[swz ? sf_swizzled(gr, (int)(gc >> 5), kt_r) : gr * nblk_r + (gc >> 5)] = (uint8_t)(e + 127);
      }
    }
  }
  __syncthreads();

#pragma unroll
  for (int t = 0; t < NT; ++t) {
    uint8_t* tin = dual_smem + t * kDualSmem;
    uint8_t* tout = tin;                              // written only after every thread has read its columns (barrier below)
    const int cp = tid & 63, j = tid >> 6;            // column pair, block of 32 rows
    const uint32_t* col = reinterpret_cast<const uint32_t*>(tin + (32 * j) * kDPitch) + cp;
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = col[i * (kDPitch / 4)];
    __syncthreads();                            // all column reads done: the tile may be overwritten
    uint32_t m = absmax_raw_bf16x2(w[0], w[1]);
#pragma unroll
    for (int i = 2; i < 32; ++i) m = absmax_raw_bf16x2(m, w[i]);
    m = abs_bf16x2(m);
    const int e0 = mx_scale_exp(bf16lo(m), FMT), e1 = mx_scale_exp(bf16hi(m), FMT);
    const uint32_t inv2 = mx_inv_scale_bf16x2(e0, e1);        // one packed multiply scales both columns
    uint32_t o0[8], o1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t a = mul_bf16x2(w[4 * i], inv2), b = mul_bf16x2(w[4 * i + 1], inv2), c = mul_bf16x2(w[4 * i + 2], inv2),
                     d = mul_bf16x2(w[4 * i + 3], inv2);
      o0[i] = cvt_fp8x4(bf16lo(a), bf16lo(b), bf16lo(c), bf16lo(d), FMT);
      o1[i] = cvt_fp8x4(bf16hi(a), bf16hi(b), bf16hi(c), bf16hi(d), FMT);
    }
    tile_park_columns(tout, cp, j, o0, o1);
    const int64_t lc = c0 + 2 * cp, gc = t * width + lc, gr = r0 + 32 * j;
    if (gr < rows) {
      if (lc < width) sf_c[sf_offset(gc, gr >> 5, rows >> 5, swz)] = (uint8_t)(e0 + 127);
      if (lc + 1 < width) sf_c[sf_offset(gc + 1, gr >> 5, rows >> 5, swz)] = (uint8_t)(e1 + 127);
    }
  }
  __syncthreads();

#pragma unroll
  for (int t = 0; t < NT; ++t) tile_store_transposed(dual_smem + t * kDualSmem, tid, t * width + c0, c0, width, r0, rows, codes_c);
}

// dw[pair] = sum over the column tiles of the partial dot products of the pair's row (0 for a dropped pair).
__global__ void dot_partials_to_pairs_kernel(const float* __restrict__ partial, int parts, int64_t rows,
                                             const int32_t* __restrict__ row_of, int64_t n_pairs, float* __restrict__ dw) {
  pdl_prologue();
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  const int r = row_of[p];
  float acc = 0.f;
  if (r >= 0)
    for (int c = 0; c < parts; ++c) acc += partial[(int64_t)c * rows + r];
  dw[p] = acc;
}

template <int SRC>
int launch_mx_tile_quant(const TileSrc& src, bool aligned_src, int64_t rows, int64_t cols, int fmt, uint8_t* codes_r, uint8_t* sf_r,
                         uint8_t* codes_c, uint8_t* sf_c, int swz, cudaStream_t st) {
  const bool wide = aligned_src && aligned32(codes_r);
  constexpr int NT = tile_parts<SRC>();
  dim3 grid((unsigned)((cols / NT + kDT - 1) / kDT), (unsigned)((rows + kDT - 1) / kDT));
#define B200Q_GO(F, W)                                                                                                  \
  do {                                                                                                                  \
    auto kernel = mx_tile_quant_kernel<F, W, SRC>;                                                                      \
    B200Q_CUDA(ensure_dynamic_smem(kernel, NT * kDualSmem));                                                           \
    launch_pdl(kernel, dim3(grid), dim3(kThreads), (size_t)(NT * kDualSmem), st, src, rows, cols, codes_r, sf_r, codes_c, sf_c, swz);                 \
  } while (0)
  if (fmt == FMT_E4M3) { if (wide) B200Q_GO(FMT_E4M3, true); else B200Q_GO(FMT_E4M3, false); }
  else { if (wide) B200Q_GO(FMT_E5M2, true); else B200Q_GO(FMT_E5M2, false); }
#undef B200Q_GO
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// ------------------------------------------------------------------------------------------
// Per-column FP8 / int8 codes (transposed output) given the column scales.  The scales are known, so no thread needs to
// own a column: a 128 x 128 tile per CTA, warp w takes the tile's columns [16 w, 16 w + 16) (32 bytes of every row),
// lane l its rows 4 l .. 4 l + 3 straight from global memory (four 32-byte loads in flight per thread; the eight warps
// together read whole 256-byte row segments).  The four codes a thread makes for one column are one 32-bit word of that
// column's row in the staging tile (lanes = consecutive words: no bank conflicts), and the tile leaves as 128-byte rows
// of the transposed matrix.  One pass through shared memory and one barrier, where staging the input as well took
// three passes and three barriers.  The arithmetic is the scaled-FP8 one (division by the fp32 scale: hoisted reciprocal
// + one correction); a column's scale and reciprocal are made by one lane and handed round by shuffles.
// rows % 32 == 0, cols % 32 == 0; other shapes use transpose_quant_kernel.
// ------------------------------------------------------------------------------------------
constexpr int kColTileSmem = kDT * kDOutPitch;
template <int FMT, bool WIDE>
__global__ void __launch_bounds__(kThreads)
fp8_col_tile_quant_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                          const float* __restrict__ col_scales, uint8_t* __restrict__ codes_c, float qmax) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t dual_smem[];
  uint8_t* tout = dual_smem;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * kDT, r0 = (int64_t)blockIdx.y * kDT;
  const int64_t gc = c0 + 16 * warp, gr = r0 + 4 * lane;
  const bool live = gc < cols && gr < rows;          // whole groups of 16 columns and of 4 rows are in or out

  uint4 v[4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i][0] = v[i][1] = make_uint4(0, 0, 0, 0);
    if (live) ld_nc_32B<WIDE>(x + (gr + i) * ld + gc, v[i][0], v[i][1]);
  }
  const int64_t my_col = gc + (lane & 15);
  const float my_scale = my_col < cols ? __ldcg(col_scales + my_col) : 1.f;
  const float my_rcp = rcp_rn(my_scale);
  uint32_t* dst = reinterpret_cast<uint32_t*>(tout + (16 * warp) * kDOutPitch) + lane;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float sc = __shfl_sync(0xffffffffu, my_scale, j), rc = __shfl_sync(0xffffffffu, my_rcp, j);
    float q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4& h = v[i][j >> 3];
      const uint32_t word = ((j >> 1) & 3) == 0 ? h.x : ((j >> 1) & 3) == 1 ? h.y : ((j >> 1) & 3) == 2 ? h.z : h.w;
      q[i] = quot_for_cast((j & 1) ? bf16hi(word) : bf16lo(word), sc, rc);
    }
    dst[j * (kDOutPitch / 4)] = cvt_codes_x4(q[0], q[1], q[2], q[3], FMT, qmax);
  }
  __syncthreads();

  tile_store_transposed(tout, tid, c0, c0, cols, r0, rows, codes_c);
}

inline bool rows_32B_aligned(const void* p, int64_t ld) { return aligned32(p) && (ld & 15) == 0; }

int check_matrix(const void* x, int64_t rows, int64_t cols, int64_t ld) {
  if (x == nullptr || rows <= 0 || cols <= 0 || ld < cols) return B200Q_ERR_INVALID_ARG;
  if ((cols & 7) || (ld & 7)) return B200Q_ERR_SHAPE;
  if (!aligned16(x)) return B200Q_ERR_ALIGNMENT;
  return B200Q_OK;
}

// Grid for the item-based row-wise kernels: exactly one resident wave (as many CTAs of 256
// threads per SM as the kernel's registers allow); the items are dealt round-robin, so every
// warp gets the same share and there is no tail wave.  `per_cta` = items one CTA takes per pass.
template <typename Kernel>
int rowwise_grid(Kernel kernel, int64_t items, int per_cta) {
  const int per_sm = blocks_per_sm(kernel, kThreads, 4);
  const int64_t want = (items + per_cta - 1) / per_cta, cap = (int64_t)kNumSMs * per_sm;
  return (int)(want < cap ? want : cap);
}

int zero_sf_pads(void* sf, int64_t outer, int64_t nblk, int layout, cudaStream_t st) {
  if (layout == B200Q_SF_SWIZZLE_128x4 && ((outer & 127) || (nblk & 3)))
    B200Q_CUDA(memset_async(sf, 0, (size_t)b200q_sf_bytes(outer, nblk, layout), st));
  return B200Q_OK;
}

// Launch helpers: the kernels take the fp8 format and the load width as template arguments.
template <int MODE, bool WIDE, int FMT>
void launch_rowwise_block(const RowQuantJob& j0, const RowQuantJob& j1, int swz, const float* tensor_amax, float* tensor_scale_out,
                          cudaStream_t st) {
  auto kernel = rowwise_block_quant_kernel<MODE, WIDE, FMT>;
  const int64_t items = j0.rows * (j0.cols / 32) + j1.rows * (j1.cols / 32);
  launch_pdl(kernel, dim3(rowwise_grid(kernel, items, kThreads)), dim3(kThreads), (size_t)(0), st, j0, j1, swz, tensor_amax, tensor_scale_out);
}
// 256-bit loads and stores need 32-byte aligned rows on both sides
inline bool job_is_wide(const RowQuantJob& j) { return j.rows == 0 || (aligned32(j.x) && aligned32(j.codes) && (j.ld & 15) == 0); }
template <int MODE>
void launch_rowwise_block(const RowQuantJob& j0, const RowQuantJob& j1, int fmt, int swz, const float* tensor_amax,
                          float* tensor_scale_out, cudaStream_t st) {
  const bool wide = job_is_wide(j0) && job_is_wide(j1);
#define B200Q_GO(W, F) launch_rowwise_block<MODE, W, F>(j0, j1, swz, tensor_amax, tensor_scale_out, st)
  if (MODE == MODE_NV || fmt == FMT_E4M3) { if (wide) B200Q_GO(true, FMT_E4M3); else B200Q_GO(false, FMT_E4M3); }
  else { if (wide) B200Q_GO(true, FMT_E5M2); else B200Q_GO(false, FMT_E5M2); }
#undef B200Q_GO
}
template <int MODE>
void launch_rowwise_block(const uint16_t* x, int64_t rows, int64_t cols, int64_t ld, int fmt, uint8_t* codes, uint8_t* sf,
                          int swz, const float* tensor_amax, float* tensor_scale_out, cudaStream_t st,
                          const int32_t* dst_row = nullptr) {
  const RowQuantJob j0 = {x, rows, cols, ld, codes, sf, dst_row}, none = {};
  launch_rowwise_block<MODE>(j0, none, fmt, swz, tensor_amax, tensor_scale_out, st);
}
template <int MODE>
void launch_transpose(const uint16_t* x, int64_t rows, int64_t cols, int64_t ld, int fmt, uint8_t* codes, uint8_t* sf, int swz,
                      const float* col_scales, const float* tensor_amax, float* tensor_scale_out, cudaStream_t st,
                      float qmax = 0.f) {
  dim3 grid((unsigned)((cols + kTC - 1) / kTC), (unsigned)((rows + kTR - 1) / kTR));
  if (MODE == MODE_FP8 && fmt == FMT_I8)
    launch_pdl(transpose_quant_kernel<MODE_FP8, FMT_I8>, dim3(grid), dim3(kThreads), (size_t)(0), st, x, rows, cols, ld, codes, sf, swz, col_scales, tensor_amax, tensor_scale_out, qmax);
  else if (MODE == MODE_NV || fmt == FMT_E4M3)
    launch_pdl(transpose_quant_kernel<MODE, FMT_E4M3>, dim3(grid), dim3(kThreads), (size_t)(0), st, x, rows, cols, ld, codes, sf, swz, col_scales, tensor_amax, tensor_scale_out, qmax);
  else
    launch_pdl(transpose_quant_kernel<MODE, FMT_E5M2>, dim3(grid), dim3(kThreads), (size_t)(0), st, x, rows, cols, ld, codes, sf, swz, col_scales, tensor_amax, tensor_scale_out, qmax);
}

// Per-column codes from given column scales: the tile kernel on whole 32 x 32 blocks, else the general transposing kernel.
void launch_fp8_cols(const uint16_t* x, int64_t rows, int64_t cols, int64_t ld, int fmt, uint8_t* codes, const float* col_scales,
                     cudaStream_t st, float qmax = 0.f) {
  if ((rows & 31) || (cols & 31)) {
    launch_transpose<MODE_FP8>(x, rows, cols, ld, fmt, codes, nullptr, 0, col_scales, nullptr, nullptr, st, qmax);
    return;
  }
  dim3 grid((unsigned)((cols + kDT - 1) / kDT), (unsigned)((rows + kDT - 1) / kDT));
  const bool wide = rows_32B_aligned(x, ld);
#define B200Q_TILE(F)                                                                                                        \
  do {                                                                                                                       \
    if (wide) launch_pdl(fp8_col_tile_quant_kernel<F, true>, dim3(grid), dim3(kThreads), (size_t)(kColTileSmem), st, x, rows, cols, ld, col_scales, codes, qmax);      \
    else launch_pdl(fp8_col_tile_quant_kernel<F, false>, dim3(grid), dim3(kThreads), (size_t)(kColTileSmem), st, x, rows, cols, ld, col_scales, codes, qmax);          \
  } while (0)
  if (fmt == FMT_I8) B200Q_TILE(FMT_I8);
  else if (fmt == FMT_E4M3) B200Q_TILE(FMT_E4M3);
  else B200Q_TILE(FMT_E5M2);
#undef B200Q_TILE
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

const char* b200q_status_string(int status) {
  switch (status) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_INVALID_ARG: return "invalid argument";
    case B200Q_ERR_SHAPE: return "unsupported shape (size is not a multiple the kernel requires)";
    case B200Q_ERR_ALIGNMENT: return "pointer or pitch is not 16-byte aligned";
    case B200Q_ERR_CUDA: return "CUDA call failed";
    case B200Q_ERR_NOT_SM100: return "device is not sm_100 (B200)";
    case B200Q_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    default: return "unknown status";
  }
}

int b200q_last_cuda_error(void) { return g_last_cuda_error; }

int b200q_device_status(void) {
  int v = 0, zero = 0;
  B200Q_CUDA(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
  if (v != 0) {
    B200Q_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    return B200Q_ERR_DEVICE_TIMEOUT;
  }
  return B200Q_OK;
}

int64_t b200q_sf_bytes(int64_t outer, int64_t nblk, int sf_layout) {
  if (outer < 0 || nblk < 0) return 0;
  if (sf_layout == B200Q_SF_SWIZZLE_128x4) return ((outer + 127) / 128) * ((nblk + 3) / 4) * 512;
  return outer * nblk;
}

int b200q_amax(const void* x, int64_t rows, int64_t cols, int64_t ld, float* amax, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (amax == nullptr) return B200Q_ERR_INVALID_ARG;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  B200Q_CUDA(zero_before_kernel(amax, sizeof(float), st));
  launch_pdl(amax_kernel, dim3(rowwise_grid(amax_kernel, rows * ((cols + 1023) / 1024), kWarps)), dim3(kThreads), (size_t)(0), st, (const uint16_t*)x, rows, cols, ld, amax);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

static int launch_rowwise_fp8(const uint16_t* x, int64_t rows, int64_t cols, int64_t ld, int fmt, uint8_t* codes,
                              float* scales, const float* tensor_amax, float* tensor_scale_out, cudaStream_t st,
                              float qmax = 0.f) {
  // warps per row: enough that a lane keeps at most 4 vectors (32 elements), up to the whole CTA
  const int64_t nv = cols / 8;
  int wpr = 1;
  while (wpr < kWarps && nv > (int64_t)wpr * 32 * 4) wpr *= 2;
  const int64_t nvec = (nv + wpr * 32 - 1) / (wpr * 32);
  const int64_t rpc = kWarps / wpr, want = (rows + rpc - 1) / rpc, cap = (int64_t)kNumSMs * 8;
  const int grid = (int)(want < cap ? want : cap);
#define B200Q_LAUNCH(NV)                                                                                                   \
  do {                                                                                                                     \
    if (fmt == FMT_E4M3)                                                                                                   \
      launch_pdl(rowwise_fp8_kernel<NV, FMT_E4M3>, dim3(grid), dim3(kThreads), (size_t)(0), st, x, rows, cols, ld, codes, scales, tensor_amax, tensor_scale_out, wpr, qmax, nullptr); \
    else if (fmt == FMT_E5M2)                                                                                              \
      launch_pdl(rowwise_fp8_kernel<NV, FMT_E5M2>, dim3(grid), dim3(kThreads), (size_t)(0), st, x, rows, cols, ld, codes, scales, tensor_amax, tensor_scale_out, wpr, qmax, nullptr); \
    else                                                                                                                   \
      launch_pdl(rowwise_fp8_kernel<NV, FMT_I8>, dim3(grid), dim3(kThreads), (size_t)(0), st, x, rows, cols, ld, codes, scales, tensor_amax, tensor_scale_out, wpr, qmax, nullptr); \
  } while (0)
  if (nvec <= 1) B200Q_LAUNCH(1);
  else if (nvec <= 2) B200Q_LAUNCH(2);
  else if (nvec <= 4) B200Q_LAUNCH(4);
  else if (nvec <= 8) B200Q_LAUNCH(8);
  else if (nvec <= 16) B200Q_LAUNCH(16);
  else B200Q_LAUNCH(0);
#undef B200Q_LAUNCH
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_fp8(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, int fmt, void* codes,
                       float* scales, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || scales == nullptr || (axis != 0 && axis != 1) || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (axis == 1) return launch_rowwise_fp8((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, scales, nullptr, nullptr, st);
  if (rows & 15) return B200Q_ERR_SHAPE;
  B200Q_CUDA(zero_before_kernel(scales, (size_t)cols * sizeof(float), st));
  {
    dim3 grid((unsigned)((cols / 8 + 31) / 32), 1);
    int64_t ymax = (rows + kWarps * 4 - 1) / (kWarps * 4);
    int64_t want = (int64_t)kNumSMs * 4 / grid.x + 1;
    grid.y = (unsigned)(want < ymax ? want : ymax);
    launch_pdl(col_amax_kernel, dim3(grid), dim3(kThreads), (size_t)(0), st, (const uint16_t*)x, rows, cols, ld, (unsigned int*)scales);
    B200Q_CUDA(cudaGetLastError());
  }
  launch_pdl(amax_to_scale_kernel, dim3((unsigned)((cols + 255) / 256)), dim3(256), (size_t)(0), st, scales, cols, fmt, 0.f);
  B200Q_CUDA(cudaGetLastError());
  launch_fp8_cols((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, scales, st);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// Rows of partial column maxima the COLMAX pass writes (one per CTA of a grid that is capped at this)
constexpr int kColmaxParts = kNumSMs * 8;

int64_t b200q_quantize_fp8_both_workspace_bytes(int64_t cols) { return cols > 0 ? (int64_t)kColmaxParts * cols * 2 : 0; }

int b200q_quantize_fp8_both(const void* x, int64_t rows, int64_t cols, int64_t ld, int fmt, void* codes_row, float* scales_row,
                            void* codes_col, float* scales_col, void* workspace, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes_row == nullptr || scales_row == nullptr || codes_col == nullptr || scales_col == nullptr || workspace == nullptr ||
      (fmt != B200Q_E4M3 && fmt != B200Q_E5M2))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes_row) || !aligned16(codes_col)) return B200Q_ERR_ALIGNMENT;
  if ((rows & 15) || cols > 8192) return B200Q_ERR_SHAPE;       // the column maxima of a CTA live in 32 KB of shared memory
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const uint16_t* xp = (const uint16_t*)x;
  unsigned int* parts = (unsigned int*)workspace;
  // pass 1: row-wise codes and scales + partial column maxima
  const int64_t nv = cols / 8;
  int wpr = 1;
  while (wpr < kWarps && nv > (int64_t)wpr * 32 * 4) wpr *= 2;
  const int64_t nvec = (nv + wpr * 32 - 1) / (wpr * 32);
  const int64_t rpc = kWarps / wpr, want = (rows + rpc - 1) / rpc;
  // one resident wave of the COLMAX kernel (64 registers: four CTAs per SM): half the partial rows to reduce afterwards
  const int64_t wave = (int64_t)kNumSMs * 4;
  const int grid = (int)(want < wave ? want : wave);
  const size_t smem = (size_t)rpc * cols * 2;          // packed bf16 column maxima of every row group
#define B200Q_GO(NV, F)                                                                                                      \
  launch_pdl(rowwise_fp8_kernel<NV, F, true>, dim3(grid), dim3(kThreads), (size_t)(smem), st, xp, rows, cols, ld, (uint8_t*)codes_row, scales_row, nullptr, nullptr, \
                                                                wpr, 0.f, parts)
#define B200Q_PICK(NV) do { if (fmt == FMT_E4M3) B200Q_GO(NV, FMT_E4M3); else B200Q_GO(NV, FMT_E5M2); } while (0)
  if (nvec <= 1) B200Q_PICK(1);
  else if (nvec <= 2) B200Q_PICK(2);
  else if (nvec <= 4) B200Q_PICK(4);
  else B200Q_PICK(8);                                            // cols <= 8192: at most 4 vectors per lane with 8 warps per row
#undef B200Q_PICK
#undef B200Q_GO
  B200Q_CUDA(cudaGetLastError());
  // pass 2: column scales, then the transposed codes
  launch_pdl(col_partials_to_scale_kernel, dim3((unsigned)((cols / 2 + kRedWords - 1) / kRedWords)), dim3(kRedWords * kRedSlices), (size_t)(0), st, parts, grid, cols, fmt,
                                                                                                                0.f, scales_col);
  B200Q_CUDA(cudaGetLastError());
  launch_fp8_cols(xp, rows, cols, ld, fmt, (uint8_t*)codes_col, scales_col, st);     // the second read comes mostly from L2
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// int8 series: the FP8 kernels with integer rounding and qmax = 2^(bits-1) - 1 (src/quant/int8.py:9-19)
int b200q_quantize_int8(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, int qmax, void* codes, float* scales,
                        void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || scales == nullptr || (axis != 0 && axis != 1) || qmax < 1 || qmax > 127) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (axis == 1)
    return launch_rowwise_fp8((const uint16_t*)x, rows, cols, ld, FMT_I8, (uint8_t*)codes, scales, nullptr, nullptr, st, (float)qmax);
  if (rows & 15) return B200Q_ERR_SHAPE;
  B200Q_CUDA(zero_before_kernel(scales, (size_t)cols * sizeof(float), st));
  {
    dim3 grid((unsigned)((cols / 8 + 31) / 32), 1);
    int64_t ymax = (rows + kWarps * 4 - 1) / (kWarps * 4);
    int64_t want = (int64_t)kNumSMs * 4 / grid.x + 1;
    grid.y = (unsigned)(want < ymax ? want : ymax);
    launch_pdl(col_amax_kernel, dim3(grid), dim3(kThreads), (size_t)(0), st, (const uint16_t*)x, rows, cols, ld, (unsigned int*)scales);
    B200Q_CUDA(cudaGetLastError());
  }
  launch_pdl(amax_to_scale_kernel, dim3((unsigned)((cols + 255) / 256)), dim3(256), (size_t)(0), st, scales, cols, FMT_I8, (float)qmax);
  B200Q_CUDA(cudaGetLastError());
  launch_fp8_cols((const uint16_t*)x, rows, cols, ld, FMT_I8, (uint8_t*)codes, scales, st, (float)qmax);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_int8_tensorwise(const void* x, int64_t rows, int64_t cols, int64_t ld, int transpose, int qmax,
                                   const float* tensor_amax, void* codes, float* scale_out, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || tensor_amax == nullptr || scale_out == nullptr || qmax < 1 || qmax > 127) return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (!transpose)
    return launch_rowwise_fp8((const uint16_t*)x, rows, cols, ld, FMT_I8, (uint8_t*)codes, nullptr, tensor_amax, scale_out, st,
                              (float)qmax);
  if (rows & 15) return B200Q_ERR_SHAPE;
  launch_transpose<MODE_FP8>((const uint16_t*)x, rows, cols, ld, FMT_I8, (uint8_t*)codes, nullptr, 0, nullptr, tensor_amax, scale_out, st,
                             (float)qmax);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_fp8_tensorwise(const void* x, int64_t rows, int64_t cols, int64_t ld, int transpose, int fmt,
                                  const float* tensor_amax, void* codes, float* scale_out, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || tensor_amax == nullptr || scale_out == nullptr || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (!transpose)
    return launch_rowwise_fp8((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, nullptr, tensor_amax, scale_out, st);
  if (rows & 15) return B200Q_ERR_SHAPE;
  launch_transpose<MODE_FP8>((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, nullptr, 0, nullptr, tensor_amax, scale_out, st);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, int fmt, void* codes,
                         void* sf, int sf_layout, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || sf == nullptr || (axis != 0 && axis != 1) || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2) ||
      (sf_layout != B200Q_SF_NATURAL && sf_layout != B200Q_SF_SWIZZLE_128x4))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  const int64_t contraction = axis == 1 ? cols : rows, outer = axis == 1 ? rows : cols;
  if (contraction & 31) return B200Q_ERR_SHAPE;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = zero_sf_pads(sf, outer, contraction / 32, sf_layout, st))) return rc;
  if (axis == 1)
    launch_rowwise_block<MODE_MX>((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, (uint8_t*)sf, sf_layout, nullptr, nullptr, st);
  else
    launch_transpose<MODE_MX>((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, (uint8_t*)sf, sf_layout, nullptr, nullptr, nullptr, st);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_mxfp8_dual(const void* x, int64_t rows, int64_t cols, int64_t ld, int fmt, void* codes_row, void* sf_row,
                              void* codes_col, void* sf_col, int sf_layout, const int32_t* num_tiles, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes_row == nullptr || sf_row == nullptr || codes_col == nullptr || sf_col == nullptr ||
      (fmt != B200Q_E4M3 && fmt != B200Q_E5M2) || (sf_layout != B200Q_SF_NATURAL && sf_layout != B200Q_SF_SWIZZLE_128x4))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes_row) || !aligned16(codes_col)) return B200Q_ERR_ALIGNMENT;
  if ((rows & 31) || (cols & 31)) return B200Q_ERR_SHAPE;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = zero_sf_pads(sf_row, rows, cols / 32, sf_layout, st))) return rc;
  if ((rc = zero_sf_pads(sf_col, cols, rows / 32, sf_layout, st))) return rc;
  TileSrc src = {};
  src.x = (const uint16_t*)x; src.ld = ld; src.live_tiles = num_tiles;
  return launch_mx_tile_quant<SRC_PLAIN>(src, rows_32B_aligned(x, ld), rows, cols, fmt, (uint8_t*)codes_row, (uint8_t*)sf_row,
                                         (uint8_t*)codes_col, (uint8_t*)sf_col, sf_layout, st);
}

// ---- the element-wise steps of the MoE expert path, fused with the both-directions quantizer ----
static int check_dual_out(void* codes_row, void* sf_row, void* codes_col, void* sf_col, int fmt) {
  if (codes_row == nullptr || sf_row == nullptr || codes_col == nullptr || sf_col == nullptr || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes_row) || !aligned16(codes_col)) return B200Q_ERR_ALIGNMENT;
  return B200Q_OK;
}

int b200q_moe_gather_quantize_dual(const void* x, int64_t D, int64_t ld, const int32_t* src_of_row, int64_t padded_rows, int fmt,
                                   void* codes_row, void* sf_row, void* codes_col, void* sf_col, const int32_t* num_tiles,
                                   void* stream) {
  PdlChain pdl_chain;
  int rc = check_dual_out(codes_row, sf_row, codes_col, sf_col, fmt);
  if (rc) return rc;
  if (x == nullptr || src_of_row == nullptr || D <= 0 || ld < D || padded_rows <= 0) return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (ld & 7) || (padded_rows & 127)) return B200Q_ERR_SHAPE;
  if (!aligned16(x)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  TileSrc src = {};
  src.x = (const uint16_t*)x; src.ld = ld; src.index = src_of_row; src.live_tiles = num_tiles;
  return launch_mx_tile_quant<SRC_GATHER>(src, rows_32B_aligned(x, ld), padded_rows, D, fmt, (uint8_t*)codes_row, (uint8_t*)sf_row,
                                          (uint8_t*)codes_col, (uint8_t*)sf_col, B200Q_SF_SWIZZLE_128x4, (cudaStream_t)stream);
}

int b200q_moe_unpermute_backward_quantize_dual(const void* dout, int64_t ld, const void* w, const int32_t* pair_of_row, int k,
                                               int64_t padded_rows, int64_t D, int fmt, void* codes_row, void* sf_row,
                                               void* codes_col, void* sf_col, const void* y, int64_t ldy,
                                               const int32_t* row_of, int64_t n_pairs, float* dot_workspace, float* dw,
                                               void* stream) {
  PdlChain pdl_chain;
  int rc = check_dual_out(codes_row, sf_row, codes_col, sf_col, fmt);
  if (rc) return rc;
  if (dout == nullptr || w == nullptr || pair_of_row == nullptr || k <= 0 || D <= 0 || ld < D || padded_rows <= 0)
    return B200Q_ERR_INVALID_ARG;
  if ((D & 127) || (ld & 7) || (padded_rows & 127)) return B200Q_ERR_SHAPE;
  if (!aligned16(dout)) return B200Q_ERR_ALIGNMENT;
  if (dw != nullptr) {
    if (y == nullptr || row_of == nullptr || dot_workspace == nullptr || n_pairs <= 0 || ldy < D) return B200Q_ERR_INVALID_ARG;
    if (ldy & 7) return B200Q_ERR_SHAPE;
    if (!aligned16(y)) return B200Q_ERR_ALIGNMENT;
  }
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  TileSrc src = {};
  src.x = (const uint16_t*)dout; src.ld = ld; src.index = pair_of_row; src.w = (const uint16_t*)w; src.k = k;
  bool wide = rows_32B_aligned(dout, ld);
  if (dw != nullptr) {
    src.y = (const uint16_t*)y; src.ldy = ldy; src.dot_partial = dot_workspace;
    wide = wide && rows_32B_aligned(y, ldy);
  }
  rc = launch_mx_tile_quant<SRC_SCALED_GATHER>(src, wide, padded_rows, D, fmt, (uint8_t*)codes_row, (uint8_t*)sf_row,
                                               (uint8_t*)codes_col, (uint8_t*)sf_col, B200Q_SF_SWIZZLE_128x4, st);
  if (rc || dw == nullptr) return rc;
  launch_pdl(dot_partials_to_pairs_kernel, dim3((unsigned)((n_pairs + kThreads - 1) / kThreads)), dim3(kThreads), (size_t)(0), st, 
      dot_workspace, (int)(D / kDT), padded_rows, row_of, n_pairs, dw);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_swiglu_quantize_dual(const void* g, int64_t rows, int64_t I, int64_t ldg, int fmt, void* codes_row, void* sf_row,
                               void* codes_col, void* sf_col, const int32_t* num_tiles, void* stream) {
  PdlChain pdl_chain;
  int rc = check_dual_out(codes_row, sf_row, codes_col, sf_col, fmt);
  if (rc) return rc;
  if (g == nullptr || rows <= 0 || I <= 0 || ldg < 2 * I) return B200Q_ERR_INVALID_ARG;
  if ((I & 127) || (ldg & 7) || (rows & 127)) return B200Q_ERR_SHAPE;
  if (!aligned16(g)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  TileSrc src = {};
  src.x = (const uint16_t*)g; src.ld = ldg; src.I = I; src.live_tiles = num_tiles;
  return launch_mx_tile_quant<SRC_SWIGLU>(src, rows_32B_aligned(g, ldg) && (I & 15) == 0, rows, I, fmt, (uint8_t*)codes_row,
                                          (uint8_t*)sf_row, (uint8_t*)codes_col, (uint8_t*)sf_col, B200Q_SF_SWIZZLE_128x4,
                                          (cudaStream_t)stream);
}

int b200q_swiglu_backward_quantize_dual(const void* g, int64_t rows, int64_t I, int64_t ldg, const void* dh, int64_t lddh, int fmt,
                                        void* codes_row, void* sf_row, void* codes_col, void* sf_col, const int32_t* num_tiles,
                                        void* stream) {
  PdlChain pdl_chain;
  int rc = check_dual_out(codes_row, sf_row, codes_col, sf_col, fmt);
  if (rc) return rc;
  if (g == nullptr || dh == nullptr || rows <= 0 || I <= 0 || ldg < 2 * I || lddh < I) return B200Q_ERR_INVALID_ARG;
  if ((I & 63) || (ldg & 7) || (lddh & 7) || (rows & 127)) return B200Q_ERR_SHAPE;       // 2 I % 128 == 0: whole scale tiles
  if (!aligned16(g) || !aligned16(dh)) return B200Q_ERR_ALIGNMENT;
  if ((rc = require_sm100())) return rc;
  TileSrc src = {};
  src.x = (const uint16_t*)g; src.ld = ldg; src.I = I; src.dh = (const uint16_t*)dh; src.lddh = lddh; src.live_tiles = num_tiles;
  return launch_mx_tile_quant<SRC_SWIGLU_BWD>(src, rows_32B_aligned(g, ldg) && rows_32B_aligned(dh, lddh) && (I & 15) == 0, rows, 2 * I,
                                              fmt, (uint8_t*)codes_row, (uint8_t*)sf_row, (uint8_t*)codes_col, (uint8_t*)sf_col,
                                              B200Q_SF_SWIZZLE_128x4, (cudaStream_t)stream);
}

int b200q_quantize_mxfp8_rowmap(const void* x, int64_t rows, int64_t cols, int64_t ld, int fmt, const int32_t* dst_row,
                                void* codes, void* sf, int sf_layout, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || sf == nullptr || dst_row == nullptr || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2) ||
      (sf_layout != B200Q_SF_NATURAL && sf_layout != B200Q_SF_SWIZZLE_128x4))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  if ((cols & 31) || rows > INT32_MAX) return B200Q_ERR_SHAPE;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = zero_sf_pads(sf, rows, cols / 32, sf_layout, st))) return rc;
  launch_rowwise_block<MODE_MX>((const uint16_t*)x, rows, cols, ld, fmt, (uint8_t*)codes, (uint8_t*)sf, sf_layout, nullptr, nullptr, st,
                                dst_row);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// Two matrices along their rows in ONE launch (same format and layout; each with an optional output-row map): the two
// weight stacks of an expert FFN, or any two operands of one step.  Equal to two b200q_quantize_mxfp8(_rowmap) calls.
int b200q_quantize_mxfp8_pair(const void* x0, int64_t rows0, int64_t cols0, int64_t ld0, const int32_t* dst_row0, void* codes0,
                              void* sf0, const void* x1, int64_t rows1, int64_t cols1, int64_t ld1, const int32_t* dst_row1,
                              void* codes1, void* sf1, int fmt, int sf_layout, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x0, rows0, cols0, ld0);
  if (rc) return rc;
  if ((rc = check_matrix(x1, rows1, cols1, ld1))) return rc;
  if (codes0 == nullptr || sf0 == nullptr || codes1 == nullptr || sf1 == nullptr || (fmt != B200Q_E4M3 && fmt != B200Q_E5M2) ||
      (sf_layout != B200Q_SF_NATURAL && sf_layout != B200Q_SF_SWIZZLE_128x4))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes0) || !aligned16(codes1)) return B200Q_ERR_ALIGNMENT;
  if ((cols0 & 31) || (cols1 & 31) || rows0 > INT32_MAX || rows1 > INT32_MAX) return B200Q_ERR_SHAPE;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = zero_sf_pads(sf0, rows0, cols0 / 32, sf_layout, st))) return rc;
  if ((rc = zero_sf_pads(sf1, rows1, cols1 / 32, sf_layout, st))) return rc;
  const RowQuantJob j0 = {(const uint16_t*)x0, rows0, cols0, ld0, (uint8_t*)codes0, (uint8_t*)sf0, dst_row0, 0};
  const RowQuantJob j1 = {(const uint16_t*)x1, rows1, cols1, ld1, (uint8_t*)codes1, (uint8_t*)sf1, dst_row1, 0};
  launch_rowwise_block<MODE_MX>(j0, j1, fmt, sf_layout, nullptr, nullptr, st);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_nvfp4_rowmap(const void* x, int64_t rows, int64_t cols, int64_t ld, const float* tensor_amax,
                                const int32_t* dst_row, void* codes, void* sf, int sf_layout, float* tensor_scale_out,
                                void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || sf == nullptr || tensor_amax == nullptr || tensor_scale_out == nullptr || dst_row == nullptr ||
      (sf_layout != B200Q_SF_NATURAL && sf_layout != B200Q_SF_SWIZZLE_128x4))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  if ((cols & 31) || rows > INT32_MAX) return B200Q_ERR_SHAPE;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = zero_sf_pads(sf, rows, cols / 16, sf_layout, st))) return rc;
  launch_rowwise_block<MODE_NV>((const uint16_t*)x, rows, cols, ld, 0, (uint8_t*)codes, (uint8_t*)sf, sf_layout, tensor_amax,
                                tensor_scale_out, st, dst_row);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

int b200q_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int64_t ld, int axis, const float* tensor_amax,
                         void* codes, void* sf, int sf_layout, float* tensor_scale_out, void* stream) {
  PdlChain pdl_chain;
  int rc = check_matrix(x, rows, cols, ld);
  if (rc) return rc;
  if (codes == nullptr || sf == nullptr || tensor_amax == nullptr || tensor_scale_out == nullptr ||
      (axis != 0 && axis != 1) || (sf_layout != B200Q_SF_NATURAL && sf_layout != B200Q_SF_SWIZZLE_128x4))
    return B200Q_ERR_INVALID_ARG;
  if (!aligned16(codes)) return B200Q_ERR_ALIGNMENT;
  const int64_t contraction = axis == 1 ? cols : rows, outer = axis == 1 ? rows : cols;
  if (contraction & 31) return B200Q_ERR_SHAPE;
  if ((rc = require_sm100())) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = zero_sf_pads(sf, outer, contraction / 16, sf_layout, st))) return rc;
  if (axis == 1)
    launch_rowwise_block<MODE_NV>((const uint16_t*)x, rows, cols, ld, 0, (uint8_t*)codes, (uint8_t*)sf, sf_layout, tensor_amax, tensor_scale_out, st);
  else
    launch_transpose<MODE_NV>((const uint16_t*)x, rows, cols, ld, 0, (uint8_t*)codes, (uint8_t*)sf, sf_layout, nullptr, tensor_amax, tensor_scale_out, st);
  B200Q_CUDA(cudaGetLastError());
  return B200Q_OK;
}

}  // extern "C"
