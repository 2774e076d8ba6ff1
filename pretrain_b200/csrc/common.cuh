// Shared host/device helpers of the library: status plumbing, argument checks,
// vector loads, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/b200q.h"
#include "numeric.cuh"

namespace b200q {

constexpr int kNumSMs = 148;

// The library is built as one translation unit (b200q_lib.cu), so these are single objects.
// Last failing CUDA error on this host thread.
static thread_local int g_last_cuda_error = 0;
// Device status word set by kernels whose bounded waits expire.
static __device__ int g_device_status = 0;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return B200Q_ERR_CUDA;
}
#define B200Q_CUDA(call)                                      \
  do {                                                        \
    cudaError_t _e = (call);                                  \
    if (_e != cudaSuccess) return ::b200q::cuda_fail(_e);     \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Checks the current device is sm_10x (cached per device).
int require_sm100();

// Per-launch runtime queries that never change for a (kernel, device) pair, remembered per host thread:
// the opt-in to more than 48 KB of dynamic shared memory and the occupancy of a kernel at a block size.
struct KernelFact { const void* fn; int dev; int key; int value; };
inline KernelFact* kernel_fact(const void* fn, int dev, int key) {
  static thread_local KernelFact facts[128];
  static thread_local int n = 0;
  for (int i = 0; i < n; ++i)
    if (facts[i].fn == fn && facts[i].dev == dev && facts[i].key == key) return &facts[i];
  KernelFact* f = &facts[n < 128 ? n++ : 127];       // a full table recycles its last slot
  *f = KernelFact{fn, dev, key, -1};
  return f;
}
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  KernelFact* f = kernel_fact(reinterpret_cast<const void*>(kernel), dev, -bytes);
  if (f->value == 1) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) f->value = 1;
  return e;
}
template <typename Kernel>
inline int blocks_per_sm(Kernel kernel, int threads, int fallback) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fallback;
  KernelFact* f = kernel_fact(reinterpret_cast<const void*>(kernel), dev, threads);
  if (f->value < 1) {
    int per_sm = 0;
    f->value = (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) == cudaSuccess && per_sm >= 1) ? per_sm : fallback;
  }
  return f->value;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization is scheduled as soon as the kernel before it
// in the stream has "triggered": explicitly, once every CTA has executed grid_launch_dependents() or exited, or implicitly
// when it completes.  What the later kernel does before grid_dependency_wait() - CTA set-up, barrier initialisation,
// tensor-memory allocation, descriptor prefetch - overlaps the earlier kernel's tail; grid_dependency_wait() returns once
// the earlier kernel has completed and its memory operations are visible (without the attribute it returns at once).
//
// Two rules, both learnt from wrong results on B200 / CUDA 12.9:
//  * After a kernel has triggered EXPLICITLY, not only an attributed kernel but also a copy or memset enqueued behind it
//    starts before it is complete, and so does whatever follows that copy (a gather kernel that triggered at its start,
//    then the next entry point's cudaMemsetAsync and GEMM: the GEMM read half-written rows; a quantizer behind torch's
//    clone() read the old contents in 27 - 30 of 30 runs).  So a kernel triggers early only where the entry point that
//    launches it puts an attributed kernel, which waits, directly behind it; everywhere else the trigger is the implicit
//    one at completion, which is safe with anything behind it.
//  * The attribute is given only to a kernel that directly follows another kernel of the same entry point: what the
//    caller enqueued before an entry point is unknown, and a memset inside one restarts the chain (memset_async).
// Every kernel of the library executes grid_dependency_wait() before it touches memory (pdl_prologue(); the GEMMs after
// their set-up), so a follower gains the launch latency and its set-up time, never correctness risk; and because a
// follower may run while its predecessor still writes, no load of possibly-produced data is non-coherent (.nc / __ldg).
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() { grid_dependency_wait(); }

// B200Q_PDL=0 in the environment turns the attribute off.
inline int pdl_mode() {                 // 0: never, 1: followers inside an entry point, 2: every launch (experiments only)
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200Q_PDL");
    v = e == nullptr ? 1 : (e[0] == '0' ? 0 : (e[0] == '2' ? 2 : 1));
  }
  return v;
}
inline bool pdl_enabled() { return pdl_mode() != 0; }
// kernels launched so far in the entry point's chain; -1 = no chain open (every launch is plain)
inline thread_local int t_pdl_chain = -1;
struct PdlChain {                       // opened at the top of every entry point
  bool outer;
  PdlChain() : outer(t_pdl_chain < 0) { if (outer) t_pdl_chain = 0; }
  ~PdlChain() { if (outer) t_pdl_chain = -1; }
  PdlChain(const PdlChain&) = delete;
  PdlChain& operator=(const PdlChain&) = delete;
};
inline cudaError_t memset_async(void* p, int value, size_t bytes, cudaStream_t st) {
  if (t_pdl_chain > 0) t_pdl_chain = 0;         // the next kernel follows a memset, not a kernel
  return cudaMemsetAsync(p, value, bytes, st);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mode() == 2 || (t_pdl_chain > 0 && pdl_mode() == 1)) ? 1 : 0;
  if (t_pdl_chain >= 0) ++t_pdl_chain;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// A few words zeroed by a kernel instead of cudaMemsetAsync, for an entry point whose next launch is a kernel that
// accumulates into them with atomics (a tensor maximum, column maxima, expert counts).  A memset node costs the
// stream two dependency bubbles (about 3 us around a 4-byte memset in front of an 18 us kernel); this kernel joins the entry
// point's launch chain instead, and triggers its dependents at once - allowed by the first rule above, because every
// caller launches an attributed kernel, which waits, directly behind it - so that kernel's CTAs are resident and
// waiting by the time the words are zero.
static __global__ void fill_words_kernel(uint32_t* __restrict__ p, int64_t n, uint32_t word, int trigger_early) {
  if (trigger_early) grid_launch_dependents();
  grid_dependency_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = word;
}
// `bytes` set to `value` (a byte, as for memset) ahead of a kernel launch of the same entry point: the caller MUST launch a
// kernel next.  Up to 1 MiB; larger or unaligned ranges go to cudaMemsetAsync.
inline cudaError_t fill_before_kernel(void* p, int value, size_t bytes, cudaStream_t st) {
  if ((bytes & 3) || (reinterpret_cast<uintptr_t>(p) & 3) || bytes > (1u << 20)) return memset_async(p, value, bytes, st);
  const int64_t n = (int64_t)(bytes >> 2);
  const int grid = (int)((n + 255) / 256 < 64 ? (n + 255) / 256 : 64);
  const uint32_t word = 0x01010101u * (uint32_t)(value & 0xFF);
  return launch_pdl(fill_words_kernel, dim3(grid), dim3(256), (size_t)0, st, reinterpret_cast<uint32_t*>(p), n, word, pdl_mode() == 1 ? 1 : 0);
}
inline cudaError_t zero_before_kernel(void* p, size_t bytes, cudaStream_t st) { return fill_before_kernel(p, 0, bytes, st); }

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// 32 bytes per lane: one 256-bit load when the address allows it (WIDE), else two 128-bit
// loads that keep the line in L1 between them (the pair covers one 32-byte sector).
template <bool WIDE>
__device__ __forceinline__ void ld_nc_32B(const void* p, uint4& a, uint4& b) {
  if (WIDE) {
    asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
  } else {
    asm volatile("ld.global.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p));
    asm volatile("ld.global.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(static_cast<const char*>(p) + 16));
  }
}
template <bool WIDE>
__device__ __forceinline__ void st_32B(void* p, const uint4& a, const uint4& b) {
  if (WIDE) {
    asm volatile("st.global.v8.u32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                 :: "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w), "l"(p) : "memory");
  } else {
    reinterpret_cast<uint4*>(p)[0] = a;
    reinterpret_cast<uint4*>(p)[1] = b;
  }
}
__host__ __device__ inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }

// max(|a|, |b|) of two packed bf16 pairs in ONE instruction; the sign bits of the result are
// unspecified (the xor of the operands' signs): chain freely, then clear them with abs_bf16x2.
// Exact (comparisons only).  A NaN operand wins (.NaN), as in torch's amax / max, which is what the
// reference reduces with (src/quant/fp8.py:26-29): a NaN anywhere in a group reaches the group's scale.
__device__ __forceinline__ uint32_t absmax_raw_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// fp32 maximum that returns NaN when either operand is NaN (fmaxf would drop it)
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t m) { return m & 0x7fff7fffu; }
// |bf16x2| max of two packed words, as packed non-negative bf16x2.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t v) { return abs_bf16x2(absmax_raw_bf16x2(acc, v)); }
// max magnitude over the two halves of a packed word -> float
__device__ __forceinline__ float absmax_halves(uint32_t m) { return fmax_nan(fabsf(bf16lo(m)), fabsf(bf16hi(m))); }
// max over the 8 bf16 of a uint4 -> float
__device__ __forceinline__ float absmax8(uint4 v) {
  return absmax_halves(absmax_raw_bf16x2(absmax_raw_bf16x2(v.x, v.y), absmax_raw_bf16x2(v.z, v.w)));
}

// bf16 x 8 in a 16-byte word -> floats (exact)
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}

// quot_for_cast() for the two bf16 of a word at once on the packed fp32 pair instructions (sm_100): the same three
// IEEE operations per lane - q = x r, e = b q - x, q' = q - e r - at half the issue slots.  The pair is unpacked
// NEGATED (one shift-add and one logic operation, like the plain unpack), and the reciprocal is passed negated, so that
// q = (-x)(-r), e = b q + (-x) and q' = e (-r) + q need no sign change of their own.  Pays only in a kernel that is
// bound by instruction issue (the NVFP4 row quantizer once its loads run ahead); the FP8 kernels did not change.
struct QuotScale {
  uint64_t b2, nr2;      // (b, b) and (-r, -r)
};
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ QuotScale quot_scale(float b, float r) {
  QuotScale s;
  s.b2 = pack_f32x2(__float_as_uint(b), __float_as_uint(b));
  s.nr2 = pack_f32x2(__float_as_uint(-r), __float_as_uint(-r));
  return s;
}
__device__ __forceinline__ void quot2_for_cast(uint32_t w, const QuotScale& s, float& q_lo, float& q_hi) {
  const uint64_t na = pack_f32x2(neg_bf16lo_bits(w), neg_bf16hi_bits(w));     // per lane: quot_for_cast_negated()
  uint64_t q, e;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q) : "l"(na), "l"(s.nr2));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(e) : "l"(s.b2), "l"(q), "l"(na));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(e), "l"(s.nr2), "l"(q));
  uint32_t lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(q));
  q_lo = __uint_as_float(lo);
  q_hi = __uint_as_float(hi);
}
__device__ __forceinline__ void quot8_for_cast(const uint4& v, const QuotScale& s, float (&q)[8]) {
  quot2_for_cast(v.x, s, q[0], q[1]);
  quot2_for_cast(v.y, s, q[2], q[3]);
  quot2_for_cast(v.z, s, q[4], q[5]);
  quot2_for_cast(v.w, s, q[6], q[7]);
}

// Packed bf16 pair (2^-e_lo, 2^-e_hi) for block exponents in [-39, 126], and the packed product.  Scaling a
// bf16 value by a power of two is exact in bf16 unless the result falls below 2^-126, far under the
// smallest fp8 subnormal, where it rounds to a (signed) zero code either way - so the packed multiply
// gives the codes of the fp32 multiply at half the instructions.  kMxNanExp (a block that holds a NaN)
// gives a NaN multiplier: every code of that block becomes NaN.
__device__ __forceinline__ uint32_t mx_inv_scale_bf16(int e) { return e == kMxNanExp ? 0x7FC0u : (uint32_t)(127 - e) << 7; }
__device__ __forceinline__ uint32_t mx_inv_scale_bf16x2(int e_lo, int e_hi) {
  return mx_inv_scale_bf16(e_lo) | (mx_inv_scale_bf16(e_hi) << 16);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// two floats rounded to nearest-even bf16, `lo` in the low half
__device__ __forceinline__ uint32_t pack_bf16_rn(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// One MXFP8 block held by one thread: 32 bf16 in four 16-byte words -> 32 code bytes in o[0..7];
// returns the block's unbiased scale exponent.
template <int FMT>
__device__ __forceinline__ int mx_quant_block32(const uint4 (&v)[4], uint32_t (&o)[8]) {
  uint32_t m = absmax_raw_bf16x2(absmax_raw_bf16x2(v[0].x, v[0].y), absmax_raw_bf16x2(v[0].z, v[0].w));
#pragma unroll
  for (int u = 1; u < 4; ++u) {
    m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(v[u].x, v[u].y));
    m = absmax_raw_bf16x2(m, absmax_raw_bf16x2(v[u].z, v[u].w));
  }
  const int e = mx_scale_exp(absmax_halves(m), FMT);
  const uint32_t inv2 = mx_inv_scale_bf16x2(e, e);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint32_t a = mul_bf16x2(v[u].x, inv2), b = mul_bf16x2(v[u].y, inv2), c = mul_bf16x2(v[u].z, inv2),
                   d = mul_bf16x2(v[u].w, inv2);
    o[2 * u] = cvt_fp8x4(bf16lo(a), bf16hi(a), bf16lo(b), bf16hi(b), FMT);
    o[2 * u + 1] = cvt_fp8x4(bf16lo(c), bf16hi(c), bf16lo(d), bf16hi(d), FMT);
  }
  return e;
}

// h = bf16(bf16(silu(gate)) * up) for 8 (gate, up) pairs packed as bf16: the roundings of the
// reference's bf16 tensor ops.  silu(x) = x * (1 / (1 + e^-x)) with the hardware exponential and
// reciprocal: within 2 fp32 ulp, far inside the bf16 rounding that follows.  Both roundings are packed
// instructions: one conversion rounds two silu values to bf16, and the bf16 x bf16 product (exact in
// fp32, 16 significant bits) is rounded once by the packed multiply, as the fp32 multiply + conversion
// would.  That leaves the exponential and the reciprocal as the only work for the special-function
// unit, which bounds this arithmetic (a scalar float -> bf16 conversion runs there too).
// 1 / (1 + e^-x) in exactly five instructions' worth of arithmetic with silu below: the flush-to-zero forms of the
// hardware exponential and reciprocal need none of the range fix-ups that the compiler wraps around __expf / __fdividef
// (a third of this arithmetic's instructions), and give the same bits wherever those are specified: e^-x below 2^-126
// vanishes against the 1 either way, and a denominator above 2^126 gives a zero quotient in both.
__device__ __forceinline__ float sigmoid_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return r;
}

__device__ __forceinline__ uint4 swiglu8(const uint4& vg, const uint4& vu) {
  float a[8];
  unpack8(vg, a);
  const uint32_t u[4] = {vu.x, vu.y, vu.z, vu.w};
  uint32_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float s0 = a[2 * i] * sigmoid_fast(a[2 * i]);
    const float s1 = a[2 * i + 1] * sigmoid_fast(a[2 * i + 1]);
    h[i] = mul_bf16x2(pack_bf16_rn(s0, s1), u[i]);
  }
  return make_uint4(h[0], h[1], h[2], h[3]);
}

// Backward of swiglu8 for 8 (gate, up, dh) triples: d_gate = dh * up * silu'(gate), d_up = dh * silu(gate),
// silu'(x) = s (1 + x (1 - s)), s = 1 / (1 + e^-x); fp32 arithmetic, one rounding to bf16.
__device__ __forceinline__ void swiglu_bwd8(const uint4& vg, const uint4& vu, const uint4& vd, uint4& dgate, uint4& dup) {
  float a[8], b[8], d[8];
  unpack8(vg, a);
  unpack8(vu, b);
  unpack8(vd, d);
  uint32_t og[4], ou[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float pg[2], pu[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float x = a[2 * i + j];
      const float sg = sigmoid_fast(x);
      pu[j] = d[2 * i + j] * x * sg;
      pg[j] = d[2 * i + j] * b[2 * i + j] * sg * (1.f + x * (1.f - sg));
    }
    __nv_bfloat162 qg = __floats2bfloat162_rn(pg[0], pg[1]), qu = __floats2bfloat162_rn(pu[0], pu[1]);
    og[i] = *reinterpret_cast<uint32_t*>(&qg);
    ou[i] = *reinterpret_cast<uint32_t*>(&qu);
  }
  dgate = make_uint4(og[0], og[1], og[2], og[3]);
  dup = make_uint4(ou[0], ou[1], ou[2], ou[3]);
}

// Byte offset of the scale factor of (row, block kb) in the 128x4-tiled layout; kt = K-tiles per row tile.
__device__ __forceinline__ int64_t sf_swizzled(int64_t row, int kb, int64_t kt) {
  return ((row >> 7) * kt + (kb >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3);
}

// Walks (row, chunk) work items that are dealt round-robin over the warps (or the threads) of the
// grid, without a division inside the loop: item = first, first + stride, ...; row = item / chunks.
struct ItemWalker {
  int64_t row, row_step;
  int chunk, chunks, chunk_step;
  __device__ __forceinline__ ItemWalker(int64_t first, int64_t stride, int chunks_) : chunks(chunks_) {
    row = first / chunks_;
    chunk = (int)(first - row * chunks_);
    row_step = stride / chunks_;
    chunk_step = (int)(stride - row_step * chunks_);
  }
  __device__ __forceinline__ void next() {
    row += row_step;
    chunk += chunk_step;
    if (chunk >= chunks) { chunk -= chunks; ++row; }
  }
};

}  // namespace b200q
