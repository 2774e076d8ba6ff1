// Host build of the quantizers' numeric core (pretrain_b200/csrc/numeric.cuh), driven
// serially, so that tests can compare the exact arithmetic the CUDA kernels use with the
// oracle on a machine without a GPU.  Test infrastructure: never linked into the library.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../pretrain_b200/csrc/numeric.cuh"

using namespace b200q;

static inline float bf(uint16_t b) { return u2f((uint32_t)b << 16); }

extern "C" {

// Every positive finite bf16 amax, every bf16 |x| <= amax: the two-correction division must
// equal the IEEE division at fp32 level, and the one-correction quotient the kernels feed
// to the narrow cast must give the same fp8 code.
// out[0] = code mismatches of quot_for_cast, out[1] = fp32 mismatches of div_by_rcp whose
// quotient is >= 2^-20, out[2] = pairs
void hc_div_exhaustive_fp8(int fmt, int amax_stride, int64_t* out) {
  int64_t bad_code = 0, bad_f32 = 0, n = 0;
  for (uint32_t ab = 1; ab < 0x7F80u; ab += amax_stride) {
    float amax = bf((uint16_t)ab);
    float scale = fp8_scale_from_amax(amax, fmt);
    float r = rcp_rn(scale);
    for (uint32_t xb = 0; xb <= ab; ++xb) {
      float x = bf((uint16_t)xb);
      float q0 = x / scale;
      float q1 = div_by_rcp(x, scale, r);
      ++n;
      if (f2u(q0) != f2u(q1) && fabsf(q0) >= 9.5367431640625e-07f) ++bad_f32;
      float q2 = quot_for_cast(x, scale, r);
      if (cvt_fp8x2(q0, -q0, fmt) != cvt_fp8x2(q2, -q2, fmt)) ++bad_code;
    }
  }
  out[0] = bad_code; out[1] = bad_f32; out[2] = n;
}

// Random (x, eff) pairs in the NVFP4 operating range: codes from the hoisted-reciprocal
// division against codes from the IEEE division.
void hc_div_random_fp4(int64_t count, uint64_t seed, int64_t* out) {
  int64_t bad_code = 0, bad_f32 = 0;
  uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
  for (int64_t i = 0; i < count; ++i) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    uint32_t eb = (uint32_t)(s >> 33);
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    uint16_t xb = (uint16_t)(s >> 40) & 0x7FFF;
    // eff: random mantissa, exponent within [-45, 40]
    int ee = (int)(eb >> 23 & 0xFF) % 86 - 45;
    float eff = u2f(((uint32_t)(ee + 127) << 23) | (eb & 0x7FFFFFu));
    float x = bf(xb);
    if (!(x <= eff * 8.0f)) x = eff * (float)(xb & 7);
    float r = rcp_rn(eff);
    float q0 = x / eff, q1 = div_by_rcp(x, eff, r), q2 = quot_for_cast(x, eff, r);
    if (f2u(q0) != f2u(q1) && fabsf(q0) >= 9.5367431640625e-07f) ++bad_f32;
    if (cvt_e2m1x2(q0, -q0) != cvt_e2m1x2(q2, -q2)) ++bad_code;
  }
  out[0] = bad_code; out[1] = bad_f32;
}

// The packed-pair form of the quotient (common.cuh: quot2_for_cast) works on operands unpacked NEGATED from the two
// halves of a word.  Every bf16 bit pattern in either half, `n_scales` scales (bf16-derived FP8 scales and random
// fp32 ones): same bits as quot_for_cast on the plainly unpacked value (NaN for NaN).  out[0] = mismatches, out[1] = cases
void hc_negated_quotient(int n_scales, uint64_t seed, int64_t* out) {
  int64_t bad = 0, n = 0;
  uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
  for (int i = 0; i < n_scales; ++i) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    float b;
    if (i & 1) {
      const int ee = (int)((s >> 40) % 86) - 45;
      b = u2f(((uint32_t)(ee + 127) << 23) | (uint32_t)((s >> 8) & 0x7FFFFFu));
    } else {
      b = fp8_scale_from_amax(bf((uint16_t)(1 + (s >> 33) % 0x7F7Fu)), i & 2 ? FMT_E5M2 : FMT_E4M3);
    }
    const float r = rcp_rn(b);
    for (uint32_t xb = 0; xb < 0x10000u; ++xb) {
      const uint32_t other = (uint32_t)(s >> 13) & 0xFFFFu;
      const uint32_t w_lo = xb | (other << 16), w_hi = (xb << 16) | other;
      const float x = u2f(xb << 16);
      const float want = quot_for_cast(x, b, r);
      const float got_lo = quot_for_cast_negated(u2f(neg_bf16lo_bits(w_lo)), b, -r);
      const float got_hi = quot_for_cast_negated(u2f(neg_bf16hi_bits(w_hi)), b, -r);
      ++n;
      if (want != want) { if (got_lo == got_lo || got_hi == got_hi) ++bad; continue; }
      if (f2u(want) != f2u(got_lo) || f2u(want) != f2u(got_hi)) ++bad;
    }
  }
  out[0] = bad; out[1] = n;
}

// The fp4 cast can only differ where the quotient is within an fp32 ulp of a rounding
// boundary of E2M1, so walk exactly those: for every block scale byte and every `stride`-th
// tensor scale derived from a bf16 maximum (plus `extra` random fp32 tensor scales), the
// bf16 inputs nearest to boundary * eff.  out[0] = code mismatches, out[1] = cases
void hc_quot_fp4_boundaries(int stride, int64_t extra, uint64_t seed, int64_t* out) {
  static const float kBoundary[8] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f, 6.0f};
  int64_t bad = 0, n = 0;
  auto walk = [&](float eff) {
    if (!(eff > 0.f) || isinf(eff)) return;
    float r = rcp_rn(eff);
    for (int bi = 0; bi < 8; ++bi) {
      uint32_t tb = f2u(kBoundary[bi] * eff) >> 16;
      for (int d = -3; d <= 3; ++d) {
        int xb = (int)tb + d;
        if (xb < 0 || xb >= 0x7F80) continue;
        float x = bf((uint16_t)xb);
        float q0 = x / eff, q2 = quot_for_cast(x, eff, r);
        ++n;
        if (cvt_e2m1x2(q0, -q0) != cvt_e2m1x2(q2, -q2)) ++bad;
      }
    }
  };
  for (uint32_t ab = 1; ab < 0x7F80u; ab += stride) {
    float s_t = nv_tensor_scale(bf((uint16_t)ab));
    for (int sq = 1; sq < 127; ++sq) walk(mul_rn(e4m3_to_float((uint8_t)sq), s_t));
  }
  uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
  for (int64_t i = 0; i < extra; ++i) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    uint32_t u = (uint32_t)(s >> 32);
    float s_t = u2f(((127u - 45u + (u >> 23) % 90u) << 23) | (u & 0x7FFFFFu));
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    walk(mul_rn(e4m3_to_float((uint8_t)(1 + (s >> 40) % 126)), s_t));
  }
  out[0] = bad; out[1] = n;
}

// codes [rows, cols], scales [rows]: per-row FP8 quantization as the kernel does it.
void hc_quant_fp8_rows(const uint16_t* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, float* scales) {
  for (int64_t r = 0; r < rows; ++r) {
    float amax = 0.f;
    for (int64_t c = 0; c < cols; ++c) amax = fmaxf(amax, fabsf(bf(x[r * cols + c])));
    float scale = fp8_scale_from_amax(amax, fmt);
    float rcp = rcp_rn(scale);
    scales[r] = scale;
    for (int64_t c = 0; c < cols; c += 2) {
      uint16_t p = cvt_fp8x2(quot_for_cast(bf(x[r * cols + c]), scale, rcp),
                             quot_for_cast(bf(x[r * cols + c + 1]), scale, rcp), fmt);
      codes[r * cols + c] = (uint8_t)p; codes[r * cols + c + 1] = (uint8_t)(p >> 8);
    }
  }
}

void hc_quant_mxfp8_rows(const uint16_t* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* sf) {
  int64_t nblk = cols / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < nblk; ++b) {
      const uint16_t* p = x + r * cols + b * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(bf(p[i])));
      int e = mx_scale_exp(amax, fmt);
      float inv = mx_inv_scale(e);
      sf[r * nblk + b] = (uint8_t)(e + 127);
      for (int i = 0; i < 32; i += 2) {
        uint16_t c2 = cvt_fp8x2(bf(p[i]) * inv, bf(p[i + 1]) * inv, fmt);
        codes[r * cols + b * 32 + i] = (uint8_t)c2; codes[r * cols + b * 32 + i + 1] = (uint8_t)(c2 >> 8);
      }
    }
}

void hc_quant_nvfp4_rows(const uint16_t* x, int64_t rows, int64_t cols, float tensor_amax, uint8_t* packed,
                         uint8_t* sf, float* tensor_scale) {
  int64_t nblk = cols / 16;
  float s_t = nv_tensor_scale(tensor_amax);
  *tensor_scale = s_t;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < nblk; ++b) {
      const uint16_t* p = x + r * cols + b * 16;
      float amax = 0.f;
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(bf(p[i])));
      uint8_t sq = nv_block_scale_fast(amax, s_t, rcp_rn(s_t));
      sf[r * nblk + b] = sq;
      float eff = e4m3_to_float(sq) * s_t;
      float rcp = rcp_rn(eff);
      for (int i = 0; i < 16; i += 2) {
        uint8_t c = sq == 0 ? 0 : cvt_e2m1x2(quot_for_cast(bf(p[i]), eff, rcp), quot_for_cast(bf(p[i + 1]), eff, rcp));
        packed[r * (cols / 2) + b * 8 + i / 2] = c;
      }
    }
}

// Every bf16 block maximum against every `stride`-th bf16 tensor maximum >= it: the
// hoisted-reciprocal block scale must equal the one computed with IEEE divisions.
void hc_nv_block_scale_exhaustive(int stride, int64_t* out) {
  int64_t bad = 0, n = 0;
  for (uint32_t tb = 1; tb < 0x7F80u; tb += stride) {
    float s_t = nv_tensor_scale(bf((uint16_t)tb));
    float rcp_st = rcp_rn(s_t);
    for (uint32_t ab = 0; ab <= tb; ++ab) {
      float a = bf((uint16_t)ab);
      ++n;
      if (nv_block_scale(a, s_t) != nv_block_scale_fast(a, s_t, rcp_st)) ++bad;
    }
  }
  out[0] = bad; out[1] = n;
}

void hc_e4m3_decode_table(float* out256) {
  for (int i = 0; i < 256; ++i) out256[i] = e4m3_to_float((uint8_t)i);
}

int64_t hc_sf_offset(int64_t r, int64_t kb, int64_t nblk, int swizzled) { return sf_offset(r, kb, nblk, swizzled); }

}  // extern "C"
