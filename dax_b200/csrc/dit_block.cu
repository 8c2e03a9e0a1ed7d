// LayerNorm + adaLN modulation (+ per-token quantisation) for the parts of a Wan DiT block around the
// attention: the normalised, modulated activations feed a quantised linear, so the kernel can emit the
// INT8 / FP8 codes and scales directly and the separate quantiser pass (and its HBM round trip) goes away.
//
// HBM-bound: 2 bytes read per element, 2 written (bf16 output) and/or 1 written (codes).  One WARP owns a token
// row: the row lives in the warp's registers (128-bit loads, all issued before the first use), mean, centred
// variance and the absmax of the rounded outputs are warp shuffles, so no row ever waits at a CTA barrier and the
// eight warps of a CTA (and the CTAs sharing an SM) hide one another's memory latency.
//   y = round_dtype( LN(x) [* w + b] [* (1 + scale) + shift] )          LN: eps inside the square root
//   (q, s) = dynamic per-token quantisation of y, arithmetic of quant_common.cuh
#include <algorithm>

#include "quant_common.cuh"

namespace dax {
namespace {

constexpr int kMaxVec = 32;  // 16-byte vectors per lane: rows up to 32 * 32 * 8 = 8192 elements

struct alignas(16) V8 { uint32_t w[4]; };  // eight 16-bit elements, two per word

template <bool BF16> __device__ __forceinline__ float to_f(uint16_t u) {
  if constexpr (BF16) return __bfloat162float(__ushort_as_bfloat16(u));
  else return __half2float(__ushort_as_half(u));
}
template <bool BF16> __device__ __forceinline__ uint16_t from_f(float f) {
  if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  else return __half_as_ushort(__float2half_rn(f));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// QDT < 0: no quantised output.  NV = 16-byte vectors per lane (rows of up to NV * 256 elements); vector i of lane l
// covers elements [8 (l + 32 i), +8), so a warp's loads and stores are contiguous 512-byte runs.
// Long rows (more than 12 vectors = 48 packed registers per lane) run with 4 warps per CTA and three CTAs per SM so
// that the row and the pass temporaries fit the register budget without spilling; shorter rows with 8 warps.
template <int NV> struct LnThreads { static constexpr int value = NV <= 12 ? 256 : 128; };

template <bool BF16, int QDT, int NV>
__global__ void __launch_bounds__(LnThreads<NV>::value, NV <= 8 ? 3 : (NV <= 12 ? 2 : 3))
ln_modulate_quant_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t D, int64_t ldx, const float* __restrict__ w,
                         const float* __restrict__ b, const float* __restrict__ shift,
                         const float* __restrict__ scale, float eps, uint16_t* __restrict__ y, int64_t ldy,
                         uint8_t* __restrict__ q, float* __restrict__ qscale) {
  // The per-column vectors (fp32) are four times the bytes of a bf16 row: they are staged in shared memory once
  // per CTA, as mul0/add0 (LayerNorm weight and bias) and mul1/add1 (1 + scale, shift), and read from there
  // for every row.
  extern __shared__ float4 vec_smem[];
  float* mul0 = reinterpret_cast<float*>(vec_smem);
  float* add0 = mul0 + (w != nullptr ? D : 0);
  float* mul1 = add0 + (w != nullptr ? D : 0);
  float* add1 = mul1 + (scale != nullptr ? D : 0);
  constexpr int kThreads = LnThreads<NV>::value, kWarps = kThreads / 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvec = static_cast<int>(D / 8);
  for (int64_t n = tid; n < D; n += kThreads) {
    if (w != nullptr) {
      mul0[n] = w[n];
      add0[n] = b != nullptr ? b[n] : 0.f;
    }
    if (scale != nullptr) {
      mul1[n] = 1.f + scale[n];
      add1[n] = shift[n];
    }
  }
  __syncthreads();
  const float inv_d = 1.f / static_cast<float>(D);
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * kWarps + warp; t < rows; t += static_cast<int64_t>(gridDim.x) * kWarps) {
    V8 raw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < nvec) raw[i] = *reinterpret_cast<const V8*>(x + t * ldx + static_cast<int64_t>(lane + 32 * i) * 8);
    // The row stays packed (16-bit) in registers and is widened again in each pass.
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < nvec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float lo, hi;
          unpack2<BF16>(raw[i].w[k], lo, hi);
          sum += lo;
          sum += hi;
        }
      }
    const float mean = warp_sum(sum) * inv_d;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < nvec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float lo, hi;
          unpack2<BF16>(raw[i].w[k], lo, hi);
          lo -= mean;
          hi -= mean;
          sq = fmaf(lo, lo, sq);
          sq = fmaf(hi, hi, sq);
        }
      }
    const float rstd = rsqrtf(warp_sum(sq) * inv_d + eps);
    uint32_t amax2 = 0u;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < nvec) {
        const int64_t n = static_cast<int64_t>(lane + 32 * i) * 8;
        float m0[8], a0[8], m1[8], a1[8];
        if (w != nullptr) {
          *reinterpret_cast<float4*>(&m0[0]) = *reinterpret_cast<const float4*>(mul0 + n);
          *reinterpret_cast<float4*>(&m0[4]) = *reinterpret_cast<const float4*>(mul0 + n + 4);
          *reinterpret_cast<float4*>(&a0[0]) = *reinterpret_cast<const float4*>(add0 + n);
          *reinterpret_cast<float4*>(&a0[4]) = *reinterpret_cast<const float4*>(add0 + n + 4);
        }
        if (scale != nullptr) {
          *reinterpret_cast<float4*>(&m1[0]) = *reinterpret_cast<const float4*>(mul1 + n);
          *reinterpret_cast<float4*>(&m1[4]) = *reinterpret_cast<const float4*>(mul1 + n + 4);
          *reinterpret_cast<float4*>(&a1[0]) = *reinterpret_cast<const float4*>(add1 + n);
          *reinterpret_cast<float4*>(&a1[4]) = *reinterpret_cast<const float4*>(add1 + n + 4);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float v[2];
          unpack2<BF16>(raw[i].w[k], v[0], v[1]);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int j = 2 * k + h;
            v[h] = (v[h] - mean) * rstd;
            if (w != nullptr) v[h] = fmaf(v[h], m0[j], a0[j]);
            if (scale != nullptr) v[h] = fmaf(v[h], m1[j], a1[j]);
          }
          // the tensor the reference materialises in the activation dtype; it replaces the input in registers
          raw[i].w[k] = pack2_rn<BF16>(v[0], v[1]);
          amax2 = absmax2<BF16>(amax2, raw[i].w[k]);
        }
        if (y != nullptr) *reinterpret_cast<V8*>(y + t * ldy + n) = raw[i];
      }
    if constexpr (QDT >= 0) {
      float alo, ahi;
      unpack2<BF16>(amax2, alo, ahi);
      const float amax = warp_max(fmaxf(alo, ahi));
      const float s = quant_scale<QDT>(amax, [](float v) { return to_f<BF16>(from_f<BF16>(v)); });
      const float inv = __fdiv_rn(1.0f, s);
      if (lane == 0) qscale[t] = s;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (lane + 32 * i < nvec) {
          float f[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) unpack2<BF16>(raw[i].w[k], f[2 * k], f[2 * k + 1]);
          const uint32_t w0 = quant_four<QDT>(f[0], f[1], f[2], f[3], s, inv);
          const uint32_t w1 = quant_four<QDT>(f[4], f[5], f[6], f[7], s, inv);
          *reinterpret_cast<uint2*>(q + t * D + static_cast<int64_t>(lane + 32 * i) * 8) = make_uint2(w0, w1);
        }
    }
  }
}

template <bool BF16, int QDT, int NV>
int launch(int64_t s, cudaStream_t st, const uint16_t* x, int64_t D, int64_t ldx, const float* w, const float* b,
           const float* shift, const float* scale, float eps, uint16_t* y, int64_t ldy, uint8_t* q, float* qscale) {
  // as many CTAs as fit on the GPU at once; each warp strides over the rows
  constexpr int kThreads = LnThreads<NV>::value, kWarps = kThreads / 32;
  int per_sm = 0;
  const size_t smem = static_cast<size_t>(D) * sizeof(float) * ((w != nullptr ? 2 : 0) + (scale != nullptr ? 2 : 0));
  if (smem > 48 * 1024)
    DAX_CUDA(cudaFuncSetAttribute(ln_modulate_quant_kernel<BF16, QDT, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
  DAX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ln_modulate_quant_kernel<BF16, QDT, NV>, kThreads, smem));
  const int64_t want = (s + kWarps - 1) / kWarps;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(want, static_cast<int64_t>(sm_count()) * std::max(per_sm, 1)));
  ln_modulate_quant_kernel<BF16, QDT, NV><<<grid, kThreads, smem, st>>>(x, s, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

template <bool BF16, int QDT>
int dispatch_nv(int64_t s, cudaStream_t st, const uint16_t* x, int64_t D, int64_t ldx, const float* w, const float* b,
                const float* shift, const float* scale, float eps, uint16_t* y, int64_t ldy, uint8_t* q, float* qscale) {
  const int64_t nv = (D / 8 + 31) / 32;
#define DAX_LN_CASE(N) if (nv <= N) return launch<BF16, QDT, N>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale)
  DAX_LN_CASE(1);
  DAX_LN_CASE(2);
  DAX_LN_CASE(4);
  DAX_LN_CASE(6);
  DAX_LN_CASE(8);
  DAX_LN_CASE(12);
  DAX_LN_CASE(16);
  DAX_LN_CASE(20);
  DAX_LN_CASE(24);
#undef DAX_LN_CASE
  return launch<BF16, QDT, kMaxVec>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
}

template <bool BF16>
int dispatch(int q_dtype, bool want_q, int64_t s, cudaStream_t st, const uint16_t* x, int64_t D, int64_t ldx,
             const float* w, const float* b, const float* shift, const float* scale, float eps, uint16_t* y,
             int64_t ldy, uint8_t* q, float* qscale) {
  if (!want_q) return dispatch_nv<BF16, -1>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  if (q_dtype == DAX_I8) return dispatch_nv<BF16, DAX_I8>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  if (q_dtype == DAX_E4M3) return dispatch_nv<BF16, DAX_E4M3>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  if (q_dtype == DAX_E5M2) return dispatch_nv<BF16, DAX_E5M2>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  return fail(DAX_ERR_UNSUPPORTED, "layernorm_modulate_quant: q_dtype %d is not I8/E4M3/E5M2", q_dtype);
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
  DAX_REQUIRE(D % 8 == 0 && D <= 8 * 32 * kMaxVec, DAX_ERR_UNSUPPORTED,
              "layernorm_modulate_quant: D=%lld must be a multiple of 8 and at most %d", (long long)D, 8 * 32 * kMaxVec);
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
    return dispatch<true>(q_dtype, q != nullptr, s, st, xp, D, ldx, ln_weight, ln_bias, shift, scale, eps, yp, ldy, qp, qscale);
  return dispatch<false>(q_dtype, q != nullptr, s, st, xp, D, ldx, ln_weight, ln_bias, shift, scale, eps, yp, ldy, qp, qscale);
}
