// Bit-exact numeric core of the quantizers, shared by every kernel.
//
// Every function is __host__ __device__: the device build uses the hardware
// conversion instructions (cvt.rn.satfinite.{e4m3x2,e5m2x2,e2m1x2}.f32), the host
// build uses the toolkit's software emulation of the same instructions, so the
// arithmetic can be verified on a CPU against the oracle value by value.
//
// Formulas follow quantize_fp8 of the reference (src/quant/fp8.py:16-32):
//   scale = max(amax / qmax, 1e-12);  codes = cast(clamp(x / scale, +-qmax))
// with IEEE fp32 divisions, extended to block granularity for MXFP8 / NVFP4.
#pragma once

#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define B200Q_HD __host__ __device__ __forceinline__
#else
#define B200Q_HD inline
#endif

namespace b200q {

enum Fp8Fmt : int { FMT_E4M3 = 0, FMT_E5M2 = 1, FMT_I8 = 2 };   // FMT_I8: the int8 series (qmax is a run-time value)

constexpr float kEps = 1e-12f;            // src/quant/fp8.py:6
constexpr int kMxFloorExp = -39;          // 2^-39 is the smallest power of two >= 1e-12
constexpr int kMxNanExp = 128;            // block maximum is NaN: scale byte 128 + 127 = 0xFF, the E8M0 NaN
constexpr float kE2M1Max = 6.0f;
constexpr float kNvTensorDiv = 2688.0f;   // 448 * 6

B200Q_HD uint32_t f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
B200Q_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f; memcpy(&f, &u, 4); return f;
#endif
}

B200Q_HD float fp8_max(int fmt) { return fmt == FMT_E4M3 ? 448.0f : 57344.0f; }

// bf16 pair packed in a 32-bit word -> two floats (exact).
B200Q_HD float bf16lo(uint32_t w) { return u2f(w << 16); }
B200Q_HD float bf16hi(uint32_t w) { return u2f(w & 0xFFFF0000u); }

// IEEE round-to-nearest fp32 division and reciprocal.
B200Q_HD float div_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(a, b);
#else
  return a / b;
#endif
}
B200Q_HD float rcp_rn(float b) {
#if defined(__CUDA_ARCH__)
  return __frcp_rn(b);
#else
  return 1.0f / b;
#endif
}
B200Q_HD float fma_rn(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
  return __fmaf_rn(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}
B200Q_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  volatile float r = a * b; return r;
#endif
}

// a / b with the reciprocal r = RN(1/b) hoisted out of the inner loop: one multiply
// and two fused residual corrections.  For the operand ranges the quantizers produce
// (|a/b| <= ~2^10 and the result either a normal fp32 or far below the smallest fp8 /
// fp4 subnormal) this returns the correctly rounded quotient; the host check compares
// it with the IEEE division over every (bf16 value, bf16-derived scale) pair.
B200Q_HD float div_by_rcp(float a, float b, float r) {
  float q = mul_rn(a, r);
  float e = fma_rn(-b, q, a);
  q = fma_rn(e, r, q);
  e = fma_rn(-b, q, a);
  q = fma_rn(e, r, q);
  // b > 0, so the quotient carries a's sign; the corrections lose it on a zero result
  return u2f((f2u(q) & 0x7FFFFFFFu) | (f2u(a) & 0x80000000u));
}

// a / b for a value that is about to be narrowed to fp8 or fp4: one multiply and ONE
// residual correction.  The result is within one fp32 ulp of the quotient, which is not
// always the correctly rounded fp32 value, but the narrow cast of it equals the narrow cast
// of the IEEE quotient: the host check walks every (bf16 x, bf16-derived scale) pair for
// both fp8 formats, and for fp4 every bf16 x next to a rounding boundary of every
// (block scale byte, tensor scale) product.  Only a bf16 input makes this safe: its 8-bit
// significand keeps quotients away from the narrow formats' ties unless they sit on them.
B200Q_HD float quot_for_cast(float a, float b, float r) {
  float q = mul_rn(a, r);
  // residual with its sign flipped, so that a = -0 (q = -0, e = +0) ends as -0 + -0 = -0 and a
  // zero quotient keeps a's sign without a fix-up; for every other input it is the same value
  float e = fma_rn(b, q, -a);
  return fma_rn(e, -r, q);   // negate the reciprocal, not e: no compiler may fold that into e's fma
}

// The same quotient from the NEGATED operand and the negated reciprocal, which is how the packed fp32 pair form in
// common.cuh computes it: q = (-a)(-r), e = b q + (-a), q' = e (-r) + q are the three operations above with the
// signs moved into the operands, so the bits are the same (the host check walks every bf16 a, unpacked negated from
// either half of a word as the kernel does, against quot_for_cast).
B200Q_HD float quot_for_cast_negated(float na, float b, float nr) {
  float q = mul_rn(na, nr);
  float e = fma_rn(b, q, na);
  return fma_rn(e, nr, q);
}
// bits of -x for the bf16 x in the low / high half of a word
B200Q_HD uint32_t neg_bf16lo_bits(uint32_t w) { return (w << 16) + 0x80000000u; }
B200Q_HD uint32_t neg_bf16hi_bits(uint32_t w) { return (w & 0xFFFF0000u) ^ 0x80000000u; }

// scale = max(amax / qmax, 1e-12)   (src/quant/fp8.py:30)
B200Q_HD float fp8_scale_from_amax(float amax, int fmt) {
  float s = div_rn(amax, fp8_max(fmt));
  return s < kEps ? kEps : s;   // NaN compares false and passes through like clamp_min
}

// Two floats -> two fp8 codes (x.x in the low byte), RNE with saturation to +-qmax,
// which equals clamp(+-qmax) followed by torch's RNE cast (src/quant/fp8.py:31).
B200Q_HD uint16_t cvt_fp8x2(float lo, float hi, int fmt) {
  float2 v; v.x = lo; v.y = hi;
  return (uint16_t)__nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, fmt == FMT_E4M3 ? __NV_E4M3 : __NV_E5M2);
}
B200Q_HD uint32_t cvt_fp8x4(float a, float b, float c, float d, int fmt) {
  return (uint32_t)cvt_fp8x2(a, b, fmt) | ((uint32_t)cvt_fp8x2(c, d, fmt) << 16);
}
B200Q_HD uint8_t cvt_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
// E4M3 byte -> float (exact)
B200Q_HD float e4m3_to_float(uint8_t b) {
  uint32_t sign = (uint32_t)(b & 0x80) << 24;
  uint32_t ex = (b >> 3) & 0xF, man = b & 7;
  if (ex == 0) return u2f(f2u((float)man * 0.001953125f) | sign);   // subnormal: man * 2^-9
  if (ex == 15 && man == 7) return u2f(0x7FC00000u | sign);
  return u2f(sign | ((ex + 120u) << 23) | (man << 20));
}
// Two floats -> packed E2M1 pair (lo in the low nibble), RNE, saturating at +-6.
B200Q_HD uint8_t cvt_e2m1x2(float lo, float hi) {
  float2 v; v.x = lo; v.y = hi;
  return (uint8_t)__nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest);
}

// ---- int8 series (src/quant/int8.py:9-19) ---------------------------------------------------------
// scale = max(amax / qmax, 1e-12); codes = clamp(round_half_even(x / scale), +-qmax) as int8.
B200Q_HD float int_scale_from_amax(float amax, float qmax) {
  float s = div_rn(amax, qmax);
  return s < kEps ? kEps : s;
}
B200Q_HD uint32_t cvt_i8(float q, float qmax) {
#if defined(__CUDA_ARCH__)
  float r = rintf(q);
#else
  float r = nearbyintf(q);
#endif
  r = r < -qmax ? -qmax : (r > qmax ? qmax : r);
  return (uint32_t)(int)r & 0xFFu;
}
// Four of them packed, lowest address first.  Clamping before the rounding gives the same integer
// (the bounds are integers and rounding is monotone); on the device that is two min/max, one
// convert and half a saturating pack per value.
B200Q_HD uint32_t cvt_i8x4(float a, float b, float c, float d, float qmax) {
#if defined(__CUDA_ARCH__)
  const int ia = __float2int_rn(fminf(fmaxf(a, -qmax), qmax)), ib = __float2int_rn(fminf(fmaxf(b, -qmax), qmax));
  const int ic = __float2int_rn(fminf(fmaxf(c, -qmax), qmax)), id = __float2int_rn(fminf(fmaxf(d, -qmax), qmax));
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(id), "r"(ic), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(ib), "r"(ia), "r"(hi));
  return out;
#else
  return cvt_i8(a, qmax) | (cvt_i8(b, qmax) << 8) | (cvt_i8(c, qmax) << 16) | (cvt_i8(d, qmax) << 24);
#endif
}
// Scale and four packed codes for any of the per-row / per-column / per-tensor formats; `fmt` is a
// compile-time constant at every call site, so the branch folds.
B200Q_HD float scale_from_amax(float amax, int fmt, float qmax) {
  return fmt == FMT_I8 ? int_scale_from_amax(amax, qmax) : fp8_scale_from_amax(amax, fmt);
}
B200Q_HD uint32_t cvt_codes_x4(float a, float b, float c, float d, int fmt, float qmax) {
  if (fmt == FMT_I8) return cvt_i8x4(a, b, c, d, qmax);
  return cvt_fp8x4(a, b, c, d, fmt);
}

// ---- MXFP8 block scale -------------------------------------------------------------
// Unbiased exponent e of the smallest power of two >= max(amax / qmax, 1e-12).
// amax = m * 2^E, qmax = 1.75 * 2^P  =>  e = E - P + (m > 1.75), floored at -39.
// A NaN maximum (some element of the block is NaN) gives kMxNanExp: the scale "max(NaN / qmax, 1e-12)" of the
// reference's formula is NaN, which E8M0 stores as 0xFF, and every code of the block is NaN.
B200Q_HD int mx_scale_exp(float amax, int fmt) {
  uint32_t u = f2u(amax) & 0x7FFFFFFFu;
  if (u > 0x7F800000u) return kMxNanExp;
  int e = (int)(u >> 23) - 127 - (fmt == FMT_E4M3 ? 8 : 15) + ((u & 0x7FFFFFu) > 0x600000u ? 1 : 0);
  e = e < kMxFloorExp ? kMxFloorExp : e;
  return e > 127 ? 127 : e;
}
// exact 2^-e for e in [-39, 126]; NaN for kMxNanExp
B200Q_HD float mx_inv_scale(int e) { return e == kMxNanExp ? u2f(0x7FC00000u) : u2f((uint32_t)(127 - e) << 23); }

// ---- NVFP4 two-level scale -----------------------------------------------------------
B200Q_HD float nv_tensor_scale(float amax_tensor) {
  float s = div_rn(amax_tensor, kNvTensorDiv);
  return s < kEps ? kEps : s;
}
// Block scale byte sq = e4m3_rne(min(max(amax_b / 6, 1e-12) / s_t, 448)).
B200Q_HD uint8_t nv_block_scale(float amax_block, float s_t) {
  float d = div_rn(amax_block, kE2M1Max);
  d = d < kEps ? kEps : d;
  float r = div_rn(d, s_t);
  r = r > 448.0f ? 448.0f : r;
  return cvt_e4m3(r);
}

// The same value with both divisions done by hoisted reciprocals: rcp6 = RN(1/6) and
// rcp_st = RN(1/s_t).  Equal to nv_block_scale() for every bf16 block maximum (the host
// check walks all of them): quotients that could differ are fp32 subnormals, which either
// fall under the 1e-12 floor or round to the scale byte 0 both ways.
B200Q_HD uint8_t nv_block_scale_fast(float amax_block, float s_t, float rcp_st) {
  float d = div_by_rcp(amax_block, kE2M1Max, 0.16666667163372039794921875f);
  d = d < kEps ? kEps : d;
  float r = div_by_rcp(d, s_t, rcp_st);
  r = r > 448.0f ? 448.0f : r;
  return cvt_e4m3(r);
}

// Scale-factor byte offset in the 128x4-tiled layout the tensor core's scale copy reads:
// rows padded to 128, blocks to 4, each tile 512 contiguous bytes, K-tile fastest.
B200Q_HD int64_t sf_offset(int64_t r, int64_t kb, int64_t nblk, int swizzled) {
  if (!swizzled) return r * nblk + kb;
  int64_t kt = (nblk + 3) >> 2;
  return ((r >> 7) * kt + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3);
}

}  // namespace b200q
