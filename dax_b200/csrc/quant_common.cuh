// Element-level arithmetic of the dynamic quantiser, shared by every kernel that quantises a row
// (quant.cu, dit_block.cu).  Bit-for-bit the reference's eager arithmetic
// (dax/quant/nn/dynamic/functional.py:124-135, dax/quant/nn/quantized/functional.py:11-20).
#pragma once
#include "common.cuh"

namespace dax {

template <int QDT>
__device__ __forceinline__ uint8_t quant_one(float x, float scale, float inv_scale) {
  if constexpr (QDT == DAX_I8) {
    float r = rintf(__fmul_rn(x, inv_scale));
    r = fminf(fmaxf(r, -128.f), 127.f);
    return static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(r)));
  } else if constexpr (QDT == DAX_E4M3) {
    float r = __fdiv_rn(x, scale);
    r = fminf(fmaxf(r, -448.f), 448.f);
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3));
  } else {
    float r = __fdiv_rn(x, scale);
    r = fminf(fmaxf(r, -57344.f), 57344.f);
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E5M2));
  }
}

template <int QDT>
__device__ __forceinline__ constexpr float quant_max() {
  return QDT == DAX_I8 ? 127.f : (QDT == DAX_E4M3 ? 448.f : 57344.f);
}

// scale = round_to_input_dtype(amax / qmax), floored at fp32 eps; `round_trip` rounds to the input dtype
template <int QDT, typename RoundTrip>
__device__ __forceinline__ float quant_scale(float amax, RoundTrip round_trip) {
  return fmaxf(round_trip(__fdiv_rn(amax, quant_max<QDT>())), 1.1920928955078125e-07f);
}

}  // namespace dax
