// LayerNorm + adaLN modulation (+ per-token quantisation) for the parts of a Wan DiT block around the
// attention: the normalised, modulated activations feed a quantised linear, so the kernel can emit the
// INT8 / FP8 codes and scales directly and the separate quantiser pass (and its HBM round trip) goes away.
//
// HBM-bound: 2 bytes read per element, 2 written (bf16 output) and/or 1 written (codes).  One CTA per
// token row; the row lives in registers (128-bit loads); mean and centred variance are two CTA
// reductions in fp32, the absmax of the rounded outputs a third.
//   y = round_dtype( LN(x) [* w + b] [* (1 + scale) + shift] )          LN: eps inside the square root
//   (q, s) = dynamic per-token quantisation of y, arithmetic of quant_common.cuh
#include "quant_common.cuh"

namespace dax {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 4;  // rows up to 8192 elements

struct alignas(16) V8 { uint16_t v[8]; };

template <bool BF16> __device__ __forceinline__ float to_f(uint16_t u) {
  if constexpr (BF16) return __bfloat162float(__ushort_as_bfloat16(u));
  else return __half2float(__ushort_as_half(u));
}
template <bool BF16> __device__ __forceinline__ uint16_t from_f(float f) {
  if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  else return __half_as_ushort(__float2half_rn(f));
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();  // red may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int k = 0; k < kThreads / 32; ++k) t += red[k];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int k = 1; k < kThreads / 32; ++k) t = fmaxf(t, red[k]);
  return t;
}

// QDT < 0: no quantised output
template <bool BF16, int QDT>
__global__ void __launch_bounds__(kThreads)
ln_modulate_quant_kernel(const uint16_t* __restrict__ x, int64_t D, int64_t ldx, const float* __restrict__ w,
                         const float* __restrict__ b, const float* __restrict__ shift,
                         const float* __restrict__ scale, float eps, uint16_t* __restrict__ y, int64_t ldy,
                         uint8_t* __restrict__ q, float* __restrict__ qscale) {
  __shared__ float red[kThreads / 32];
  const int64_t t = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t nvec = D / 8;
  float f[kMaxVec][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t vi = tid + static_cast<int64_t>(i) * kThreads;
    if (vi < nvec) {
      const V8 raw = *reinterpret_cast<const V8*>(x + t * ldx + vi * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[i][j] = to_f<BF16>(raw.v[j]);
        sum += f[i][j];
      }
    }
  }
  const float mean = block_sum(sum, red) / static_cast<float>(D);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t vi = tid + static_cast<int64_t>(i) * kThreads;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[i][j] -= mean;
        sq = fmaf(f[i][j], f[i][j], sq);
      }
    }
  }
  const float rstd = rsqrtf(block_sum(sq, red) / static_cast<float>(D) + eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t vi = tid + static_cast<int64_t>(i) * kThreads;
    if (vi < nvec) {
      const int64_t n = vi * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = f[i][j] * rstd;
        if (w != nullptr) v = fmaf(v, w[n + j], b != nullptr ? b[n + j] : 0.f);
        if (scale != nullptr) v = fmaf(v, 1.f + scale[n + j], shift[n + j]);
        v = to_f<BF16>(from_f<BF16>(v));  // the tensor the reference materialises in the activation dtype
        f[i][j] = v;
        amax = fmaxf(amax, fabsf(v));
      }
      if (y != nullptr) {
        V8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = from_f<BF16>(f[i][j]);
        *reinterpret_cast<V8*>(y + t * ldy + n) = o;
      }
    }
  }
  if constexpr (QDT >= 0) {
    amax = block_max(amax, red);
    const float s = quant_scale<QDT>(amax, [](float v) { return to_f<BF16>(from_f<BF16>(v)); });
    const float inv = __fdiv_rn(1.0f, s);
    if (tid == 0) qscale[t] = s;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int64_t vi = tid + static_cast<int64_t>(i) * kThreads;
      if (vi < nvec) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          w0 |= static_cast<uint32_t>(quant_one<QDT>(f[i][j], s, inv)) << (8 * j);
          w1 |= static_cast<uint32_t>(quant_one<QDT>(f[i][4 + j], s, inv)) << (8 * j);
        }
        *reinterpret_cast<uint2*>(q + t * D + vi * 8) = make_uint2(w0, w1);
      }
    }
  }
}

template <bool BF16>
int dispatch(int q_dtype, bool want_q, unsigned s, cudaStream_t st, const uint16_t* x, int64_t D, int64_t ldx,
             const float* w, const float* b, const float* shift, const float* scale, float eps, uint16_t* y,
             int64_t ldy, uint8_t* q, float* qscale) {
  if (!want_q) {
    ln_modulate_quant_kernel<BF16, -1><<<s, kThreads, 0, st>>>(x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  } else if (q_dtype == DAX_I8) {
    ln_modulate_quant_kernel<BF16, DAX_I8><<<s, kThreads, 0, st>>>(x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  } else if (q_dtype == DAX_E4M3) {
    ln_modulate_quant_kernel<BF16, DAX_E4M3><<<s, kThreads, 0, st>>>(x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  } else if (q_dtype == DAX_E5M2) {
    ln_modulate_quant_kernel<BF16, DAX_E5M2><<<s, kThreads, 0, st>>>(x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  } else {
    return fail(DAX_ERR_UNSUPPORTED, "layernorm_modulate_quant: q_dtype %d is not I8/E4M3/E5M2", q_dtype);
  }
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

}  // namespace
}  // namespace dax

extern "C" int dax_layernorm_modulate_quant(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx,
                                            const float* ln_weight, const float* ln_bias, const float* shift,
                                            const float* scale, float eps, void* y, int64_t ldy, void* q,
                                            int q_dtype, float* qscale, void* stream) {
  using namespace dax;
  DAX_REQUIRE(s >= 0 && D > 0, DAX_ERR_INVALID, "layernorm_modulate_quant: bad shape s=%lld D=%lld", (long long)s, (long long)D);
  if (s == 0) return DAX_OK;
  DAX_REQUIRE(x != nullptr && (y != nullptr || q != nullptr), DAX_ERR_INVALID, "layernorm_modulate_quant: null pointer");
  DAX_REQUIRE(dtype == DAX_BF16 || dtype == DAX_F16, DAX_ERR_UNSUPPORTED, "layernorm_modulate_quant: dtype %d is not BF16/F16", dtype);
  DAX_REQUIRE(D % 8 == 0 && D <= 8 * kThreads * kMaxVec, DAX_ERR_UNSUPPORTED,
              "layernorm_modulate_quant: D=%lld must be a multiple of 8 and at most %d", (long long)D, 8 * kThreads * kMaxVec);
  DAX_REQUIRE((shift == nullptr) == (scale == nullptr), DAX_ERR_INVALID, "layernorm_modulate_quant: shift and scale come together");
  DAX_REQUIRE(ln_bias == nullptr || ln_weight != nullptr, DAX_ERR_INVALID, "layernorm_modulate_quant: bias needs weight");
  DAX_REQUIRE(q == nullptr || qscale != nullptr, DAX_ERR_INVALID, "layernorm_modulate_quant: q needs qscale");
  DAX_REQUIRE(ldx % 8 == 0 && ldy % 8 == 0 && aligned16(x) && (y == nullptr || aligned16(y)) && (q == nullptr || aligned16(q)),
              DAX_ERR_ALIGN, "layernorm_modulate_quant: pointers 16-byte aligned, leading dimensions multiples of 8");
  DAX_REQUIRE(s < (1ll << 31), DAX_ERR_UNSUPPORTED, "layernorm_modulate_quant: s too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  uint16_t* yp = static_cast<uint16_t*>(y);
  uint8_t* qp = static_cast<uint8_t*>(q);
  if (dtype == DAX_BF16)
    return dispatch<true>(q_dtype, q != nullptr, static_cast<unsigned>(s), st, xp, D, ldx, ln_weight, ln_bias, shift, scale, eps, yp, ldy, qp, qscale);
  return dispatch<false>(q_dtype, q != nullptr, static_cast<unsigned>(s), st, xp, D, ldx, ln_weight, ln_bias, shift, scale, eps, yp, ldy, qp, qscale);
}
