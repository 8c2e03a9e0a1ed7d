// Element-level arithmetic of the dynamic quantiser, shared by every kernel that quantises a row
// (quant.cu, dit_block.cu).  Bit-for-bit the reference's eager arithmetic
// (dax/quant/nn/dynamic/functional.py:124-135, dax/quant/nn/quantized/functional.py:11-20).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace dax {

// Two 16-bit floats in one 32-bit word (element 0 in the low half) <-> two fp32, and the packed |.|-max: one
// instruction per element or per pair instead of an extract-and-convert sequence per element.
template <bool BF16>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
  if constexpr (BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2_rn(float lo, float hi) {  // round to nearest even
  uint32_t r;
  if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// acc = max(acc, |w|) on both halves; acc starts at 0.  A NaN element is ignored, as fmaxf does.
template <bool BF16>
__device__ __forceinline__ uint32_t absmax2(uint32_t acc, uint32_t w) {
  uint32_t r;
  const uint32_t a = w & 0x7fff7fffu;
  if constexpr (BF16) asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(acc), "r"(a));
  else asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(acc), "r"(a));
  return r;
}

// x / s rounded to nearest, for a divisor whose correctly rounded reciprocal r = RN(1 / s) is at hand
// (one per row): q0 = RN(x r), then one residual correction.  Both steps are fused multiply-adds, so the result
// is the correctly rounded quotient wherever neither step leaves the normal range; quotients that small or
// that large quantise to zero or saturate either way.  Requires s > 0.
__device__ __forceinline__ float div_rn_by(float x, float s, float r) {
  const float q0 = __fmul_rn(x, r);
  const float q = __fmaf_rn(__fmaf_rn(-q0, s, x), r, q0);
  // s > 0, so the quotient carries the sign of x; the correction step alone would turn -0 into +0
  return __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(x) & 0x80000000u));
}

// Four values -> four codes packed into 32 bits (element 0 in the low byte).
//   INT8: clamp(rint(x * inv_scale), -128, 127): one multiply and one saturating round-to-nearest-even conversion
//   FP8 : round_nearest_even_to_fp8(clamp(x / scale)): the saturating conversion clamps to the largest finite code
template <int QDT>
__device__ __forceinline__ uint32_t quant_four(float a, float b, float c, float d, float scale, float inv_scale) {
  if constexpr (QDT == DAX_I8) {
    int32_t qa, qb, qc, qd;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qa) : "f"(__fmul_rn(a, inv_scale)));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qb) : "f"(__fmul_rn(b, inv_scale)));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qc) : "f"(__fmul_rn(c, inv_scale)));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qd) : "f"(__fmul_rn(d, inv_scale)));
    uint32_t lo, hi, w;
    asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(qa), "r"(qb));
    asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(qc), "r"(qd));
    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(w) : "r"(lo), "r"(hi));
    return w;
  } else {
    const float qa = div_rn_by(a, scale, inv_scale), qb = div_rn_by(b, scale, inv_scale);
    const float qc = div_rn_by(c, scale, inv_scale), qd = div_rn_by(d, scale, inv_scale);
    uint16_t lo, hi;
    if constexpr (QDT == DAX_E4M3) {
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(qb), "f"(qa));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(qd), "f"(qc));
    } else {
      asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(qb), "f"(qa));
      asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(qd), "f"(qc));
    }
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  }
}

// ---- packed fp32 pairs (one 64-bit register, two lanes of arithmetic per instruction) ----------------------
// The row kernels are bound by instruction issue before they are bound by HBM; add / mul / fma on pairs halve
// the arithmetic instructions.  Each lane of a pair is rounded exactly like the scalar instruction.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ uint64_t f2_splat(float v) { return f2_pack(v, v); }
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
template <bool BF16>
__device__ __forceinline__ uint64_t f2_from16(uint32_t w) {  // two 16-bit floats -> pair
  float lo, hi;
  unpack2<BF16>(w, lo, hi);
  return f2_pack(lo, hi);
}
template <bool BF16>
__device__ __forceinline__ uint32_t f2_to16_rn(uint64_t p) {
  float lo, hi;
  f2_unpack(p, lo, hi);
  return pack2_rn<BF16>(lo, hi);
}

// Four 16-bit values (two packed words, element 0 in the low half of w0) -> four codes, the arithmetic of
// quant_four on pairs: for FP8 the quotient is q0 = RN(x r) corrected once, e = x - q0 s, q = q0 + e r, and the
// sign of x is put back on the CODE (the correction alone turns -0 into +0): the high byte of each 16-bit input
// carries its sign, one byte permute collects the four of them.
template <bool BF16, int QDT>
__device__ __forceinline__ uint32_t quant_four16(uint32_t w0, uint32_t w1, uint64_t neg_scale2, uint64_t inv2) {
  const uint64_t x0 = f2_from16<BF16>(w0), x1 = f2_from16<BF16>(w1);
  if constexpr (QDT == DAX_I8) {
    float a, b, c, d;
    f2_unpack(f2_mul(x0, inv2), a, b);
    f2_unpack(f2_mul(x1, inv2), c, d);
    int32_t qa, qb, qc, qd;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qa) : "f"(a));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qb) : "f"(b));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qc) : "f"(c));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(qd) : "f"(d));
    uint32_t lo, hi, w;
    asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(qa), "r"(qb));
    asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(qc), "r"(qd));
    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(w) : "r"(lo), "r"(hi));
    return w;
  } else {
    const uint64_t q0 = f2_mul(x0, inv2), q1 = f2_mul(x1, inv2);
    float a, b, c, d;
    f2_unpack(f2_fma(f2_fma(q0, neg_scale2, x0), inv2, q0), a, b);
    f2_unpack(f2_fma(f2_fma(q1, neg_scale2, x1), inv2, q1), c, d);
    uint16_t lo, hi;
    if constexpr (QDT == DAX_E4M3) {
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    } else {
      asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
      asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    }
    uint32_t codes, signs;
    asm("mov.b32 %0, {%1, %2};" : "=r"(codes) : "h"(lo), "h"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7531;" : "=r"(signs) : "r"(w0), "r"(w1));  // the high byte of each input
    return (codes & 0x7f7f7f7fu) | (signs & 0x80808080u);
  }
}

template <int QDT>
__device__ __forceinline__ constexpr float quant_max() {
  return QDT == DAX_I8 ? 127.f : (QDT == DAX_E4M3 ? 448.f : 57344.f);
}

// scale = round_to_input_dtype(amax / qmax), floored at fp32 eps; `round_trip` rounds to the input dtype
// The quotient amax / qmax is correctly rounded either way; the short form (div_rn_by with the constant
// reciprocal) is three instructions instead of a division routine that every thread of a row would run.  It is
// exact wherever it stays in the normal range: above it (an infinite or NaN amax) the full division runs, below
// it the result is under the floor anyway.
template <int QDT, typename RoundTrip>
__device__ __forceinline__ float quant_scale(float amax, RoundTrip round_trip) {
  constexpr float qmax = quant_max<QDT>();
  constexpr float rq = 1.0f / qmax;  // correctly rounded by the host compiler
  const float quot = amax <= 3.0e38f ? div_rn_by(amax, qmax, rq) : __fdiv_rn(amax, qmax);
  return fmaxf(round_trip(quot), 1.1920928955078125e-07f);
}
// 1 / scale, correctly rounded (the same value as a full division of 1.0f by scale)
__device__ __forceinline__ float quant_inv_scale(float scale) { return __frcp_rn(scale); }

}  // namespace dax
