// Prepare step of the quantised attention: turns bf16/bf16 Q, K, V (any batch/head/token strides,
// channels contiguous) into the operand arrays of the forward kernel (layout in attn_common.cuh).
// HBM-bound: every input element is read twice at most (statistics pass + quantise pass for K and
// V, once for Q) and written once at 1 or 2 bytes.
//
//   1. colstats      partial per-channel sums of K and maxima of |V| over blocks of 512 tokens
//   2. colstats_fin  K mean and V scale per (batch, head, channel); fixed summation order
//   3. quant_q       per token: q * (sm_scale * log2 e) -> INT8 with a per-token scale (or bf16)
//   4. quant_k       per block of 128 tokens: (k - mean) -> INT8 with one scale per block (or bf16)
//   5. quant_v       per block of 128 tokens: v / scale[channel] -> FP8 e4m3 (or bf16), transposed
// Subtracting the K mean leaves softmax unchanged (it shifts every score of a row by the same
// amount) and removes the channel offset that would otherwise eat the INT8 range.
#include <type_traits>

#include "attn_common.cuh"

namespace dax {
namespace {

struct Strides { int64_t b, h, t; };

template <bool BF16>
__device__ __forceinline__ float ld16(const uint16_t u) {
  if constexpr (BF16) return __bfloat162float(__ushort_as_bfloat16(u));
  else return __half2float(__ushort_as_half(u));
}

struct alignas(16) V8 { uint16_t v[8]; };

// grid (chunks, BH), 256 threads: 16 channel groups of 8 x 16 token lanes.
template <bool BF16>
__global__ void __launch_bounds__(256)
colstats_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v, Strides ks, Strides vs, int heads,
                int64_t Sk, float* __restrict__ part, int64_t chunks) {
  __shared__ float red[2][16][128];
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int cg = threadIdx.x & 15, tl = threadIdx.x >> 4;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * kStatChunk;
  const int64_t t1 = min(t0 + kStatChunk, Sk);
  const uint16_t* kb = k + b * ks.b + h * ks.h + cg * 8;
  const uint16_t* vb = v + b * vs.b + h * vs.h + cg * 8;
  float sum[8], mx[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { sum[j] = 0.f; mx[j] = 0.f; }
  for (int64_t t = t0 + tl; t < t1; t += 16) {
    const V8 kv = *reinterpret_cast<const V8*>(kb + t * ks.t);
    const V8 vv = *reinterpret_cast<const V8*>(vb + t * vs.t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sum[j] += ld16<BF16>(kv.v[j]);
      mx[j] = fmaxf(mx[j], fabsf(ld16<BF16>(vv.v[j])));
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { red[0][tl][cg * 8 + j] = sum[j]; red[1][tl][cg * 8 + j] = mx[j]; }
  __syncthreads();
  if (threadIdx.x < 128) {
    float s = 0.f, m = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { s += red[0][i][threadIdx.x]; m = fmaxf(m, red[1][i][threadIdx.x]); }
    float* dst = part + (static_cast<int64_t>(bh) * chunks + blockIdx.x) * 256;
    dst[threadIdx.x] = s;
    dst[128 + threadIdx.x] = m;
  }
}

// grid BH, 128 threads
__global__ void colstats_fin_kernel(const float* __restrict__ part, int64_t chunks, int64_t Sk, int fp8_v,
                                    float* __restrict__ k_mean, float* __restrict__ v_scale) {
  const int bh = blockIdx.x, c = threadIdx.x;
  float s = 0.f, m = 0.f;
  for (int64_t i = 0; i < chunks; ++i) {
    const float* src = part + (static_cast<int64_t>(bh) * chunks + i) * 256;
    s += src[c];
    m = fmaxf(m, src[128 + c]);
  }
  k_mean[bh * 128 + c] = s / static_cast<float>(Sk);
  v_scale[bh * 128 + c] = fp8_v ? fmaxf(m / 448.f, 1e-30f) : 1.f;
}

// grid (Sq_pad / 8, BH), 256 threads: one warp per token, a lane owns 4 channels.
template <bool BF16, bool I8>
__global__ void __launch_bounds__(256)
quant_q_kernel(const uint16_t* __restrict__ q, Strides qs, int heads, int64_t Sq, int64_t Sq_pad, float cscale,
               void* __restrict__ qo, float* __restrict__ q_scale) {
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (t >= Sq_pad) return;
  float f[4] = {0.f, 0.f, 0.f, 0.f};
  if (t < Sq) {
    const uint2 raw = *reinterpret_cast<const uint2*>(q + b * qs.b + h * qs.h + t * qs.t + lane * 4);
    f[0] = ld16<BF16>(raw.x & 0xffff); f[1] = ld16<BF16>(raw.x >> 16);
    f[2] = ld16<BF16>(raw.y & 0xffff); f[3] = ld16<BF16>(raw.y >> 16);
  }
  const int64_t row = static_cast<int64_t>(bh) * Sq_pad + t;
  if constexpr (I8) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[j] *= cscale; amax = fmaxf(amax, fabsf(f[j])); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = fmaxf(amax / 127.f, 1e-30f);
    const float inv = 1.f / sc;
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int qi = max(-127, min(127, __float2int_rn(f[j] * inv)));
      w |= (static_cast<uint32_t>(qi) & 0xffu) << (8 * j);
    }
    reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(qo) + row * 128)[lane] = w;
    if (lane == 0) q_scale[row] = sc;
  } else {
    uint2 w;
    w.x = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[0]))) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[1]))) << 16);
    w.y = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[2]))) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[3]))) << 16);
    reinterpret_cast<uint2*>(static_cast<uint16_t*>(qo) + row * 128)[lane] = w;
    if (lane == 0) q_scale[row] = cscale;
  }
}

// grid (Sk_pad / 128, BH), 256 threads: thread = (token = tid / 2, half row of 64 channels).
template <bool BF16, bool I8>
__global__ void __launch_bounds__(256)
quant_k_kernel(const uint16_t* __restrict__ k, Strides ks, int heads, int64_t Sk, int64_t Sk_pad,
               const float* __restrict__ k_mean, void* __restrict__ ko, float* __restrict__ k_scale) {
  __shared__ float red[8];
  __shared__ float mean_s[128];
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 128 + (threadIdx.x >> 1);
  const int c0 = (threadIdx.x & 1) * 64;
  if (threadIdx.x < 128) mean_s[threadIdx.x] = k_mean[bh * 128 + threadIdx.x];
  __syncthreads();
  float f[64];
  float amax = 0.f;
  if (t < Sk) {
    const uint16_t* src = k + b * ks.b + h * ks.h + t * ks.t + c0;
#pragma unroll
    for (int vi = 0; vi < 8; ++vi) {
      const V8 raw = *reinterpret_cast<const V8*>(src + vi * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = ld16<BF16>(raw.v[j]) - mean_s[c0 + vi * 8 + j];
        f[vi * 8 + j] = x;
        amax = fmaxf(amax, fabsf(x));
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j) f[j] = 0.f;
  }
  const int64_t row = static_cast<int64_t>(bh) * Sk_pad + t;
  if constexpr (I8) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    const float sc = fmaxf(amax / 127.f, 1e-30f);
    const float inv = 1.f / sc;
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(ko) + row * 128 + c0);
#pragma unroll
    for (int vi = 0; vi < 4; ++vi) {
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        w[q] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int qi = max(-127, min(127, __float2int_rn(f[vi * 16 + q * 4 + j] * inv)));
          w[q] |= (static_cast<uint32_t>(qi) & 0xffu) << (8 * j);
        }
      }
      dst[vi] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (threadIdx.x == 0) k_scale[static_cast<int64_t>(bh) * (Sk_pad / 128) + blockIdx.x] = sc;
  } else {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(ko) + row * 128 + c0);
#pragma unroll
    for (int vi = 0; vi < 8; ++vi) {
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        w[q] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[vi * 8 + 2 * q]))) |
               (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[vi * 8 + 2 * q + 1]))) << 16);
      dst[vi] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (threadIdx.x == 0) k_scale[static_cast<int64_t>(bh) * (Sk_pad / 128) + blockIdx.x] = 1.f;
  }
}

// grid (Sk_pad / 128, BH), 256 threads.  Reads a [128 tokens x 128 channels] tile row-wise, writes it
// transposed: vt[bh, channel, token].  The transpose goes through shared memory with a padded pitch.
template <bool BF16, bool F8>
__global__ void __launch_bounds__(256)
quant_v_kernel(const uint16_t* __restrict__ v, Strides vs, int heads, int64_t Sk, int64_t Sk_pad,
               const float* __restrict__ v_scale, void* __restrict__ vo) {
  using OutT = typename std::conditional<F8, uint8_t, uint16_t>::type;
  constexpr int PITCH = 128 + (F8 ? 4 : 2);  // elements; keeps 4-byte alignment and spreads banks
  __shared__ OutT tile[128 * PITCH];         // [channel][token]
  __shared__ float inv_s[128];
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * 128;
  if (threadIdx.x < 128) inv_s[threadIdx.x] = 1.f / v_scale[bh * 128 + threadIdx.x];
  __syncthreads();
  {
    const int cg = threadIdx.x & 15;  // 8 channels
    for (int tl = threadIdx.x >> 4; tl < 128; tl += 16) {
      const int64_t t = tok0 + tl;
      V8 raw;
      if (t < Sk) raw = *reinterpret_cast<const V8*>(v + b * vs.b + h * vs.h + t * vs.t + cg * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = cg * 8 + j;
        const float x = t < Sk ? ld16<BF16>(raw.v[j]) * inv_s[c] : 0.f;
        if constexpr (F8) tile[c * PITCH + tl] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
        else tile[c * PITCH + tl] = __bfloat16_as_ushort(__float2bfloat16_rn(x));
      }
    }
  }
  __syncthreads();
  {
    // each warp writes whole channel rows: 128 tokens = 128 B (fp8) or 256 B (bf16)
    const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
    for (int c = wrp; c < 128; c += 8) {
      OutT* dst = static_cast<OutT*>(vo) + (static_cast<int64_t>(bh) * 128 + c) * Sk_pad + tok0;
      if constexpr (F8) {
        reinterpret_cast<uint32_t*>(dst)[lane] = *reinterpret_cast<const uint32_t*>(&tile[c * PITCH + lane * 4]);
      } else {
        reinterpret_cast<uint32_t*>(dst)[lane] = *reinterpret_cast<const uint32_t*>(&tile[c * PITCH + lane * 2]);
        reinterpret_cast<uint32_t*>(dst)[32 + lane] = *reinterpret_cast<const uint32_t*>(&tile[c * PITCH + 64 + lane * 2]);
      }
    }
  }
}

template <bool BF16>
int run_prepare(const void* q, const void* k, const void* v, int64_t B, int64_t heads, int64_t Sq, int64_t Sk,
                Strides qs, Strides ks, Strides vs, float sm_scale, int mode, const AttnWorkspace& ws, cudaStream_t st) {
  const int64_t BH = B * heads;
  const uint16_t* qp = static_cast<const uint16_t*>(q);
  const uint16_t* kp = static_cast<const uint16_t*>(k);
  const uint16_t* vp = static_cast<const uint16_t*>(v);
  const bool qk_i8 = attn_qk_bytes(mode) == 1, v_f8 = attn_pv_bytes(mode) == 1;
  const float cscale = sm_scale * 1.4426950408889634f;
  const unsigned bh = static_cast<unsigned>(BH);
  colstats_kernel<BF16><<<dim3(static_cast<unsigned>(ws.chunks), bh), 256, 0, st>>>(kp, vp, ks, vs, static_cast<int>(heads), Sk, ws.part, ws.chunks);
  colstats_fin_kernel<<<bh, 128, 0, st>>>(ws.part, ws.chunks, Sk, v_f8 ? 1 : 0, ws.k_mean, ws.v_scale);
  const dim3 gq(static_cast<unsigned>(ws.Sq_pad / 8), bh), gk(static_cast<unsigned>(ws.Sk_pad / 128), bh);
  if (qk_i8) {
    quant_q_kernel<BF16, true><<<gq, 256, 0, st>>>(qp, qs, static_cast<int>(heads), Sq, ws.Sq_pad, cscale, ws.q, ws.q_scale);
    quant_k_kernel<BF16, true><<<gk, 256, 0, st>>>(kp, ks, static_cast<int>(heads), Sk, ws.Sk_pad, ws.k_mean, ws.k, ws.k_scale);
  } else {
    quant_q_kernel<BF16, false><<<gq, 256, 0, st>>>(qp, qs, static_cast<int>(heads), Sq, ws.Sq_pad, cscale, ws.q, ws.q_scale);
    quant_k_kernel<BF16, false><<<gk, 256, 0, st>>>(kp, ks, static_cast<int>(heads), Sk, ws.Sk_pad, ws.k_mean, ws.k, ws.k_scale);
  }
  if (v_f8) quant_v_kernel<BF16, true><<<gk, 256, 0, st>>>(vp, vs, static_cast<int>(heads), Sk, ws.Sk_pad, ws.v_scale, ws.vt);
  else quant_v_kernel<BF16, false><<<gk, 256, 0, st>>>(vp, vs, static_cast<int>(heads), Sk, ws.Sk_pad, ws.v_scale, ws.vt);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

bool strides_ok(const int64_t* s) { return s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0 && s[2] >= 128; }

}  // namespace
}  // namespace dax

extern "C" size_t dax_attn_workspace_bytes(int64_t B, int64_t heads, int64_t Sq, int64_t Sk, int mode) {
  dax::AttnWorkspace ws;
  if (dax::attn_workspace_layout(B, heads, Sq, Sk, mode, nullptr, 0, &ws) != DAX_OK) return 0;
  return ws.bytes;
}

extern "C" int dax_attn_prepare(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                                int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3],
                                int64_t v_strides[3], float sm_scale, int mode, void* workspace,
                                size_t workspace_bytes, void* stream) {
  using namespace dax;
  DAX_REQUIRE(q && k && v && workspace && q_strides && k_strides && v_strides, DAX_ERR_INVALID, "attn_prepare: null pointer");
  DAX_REQUIRE(dtype == DAX_BF16 || dtype == DAX_F16, DAX_ERR_UNSUPPORTED, "attn_prepare: dtype %d is not BF16/F16", dtype);
  AttnWorkspace ws;
  int rc = attn_workspace_layout(B, heads, Sq, Sk, mode, workspace, workspace_bytes, &ws);
  if (rc != DAX_OK) return rc;
  DAX_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && strides_ok(q_strides) && strides_ok(k_strides) && strides_ok(v_strides),
              DAX_ERR_ALIGN, "attn_prepare: q, k, v must be 16-byte aligned with strides that are multiples of 8 elements");
  DAX_REQUIRE(sm_scale > 0.f, DAX_ERR_INVALID, "attn_prepare: sm_scale must be positive");
  const Strides qs{q_strides[0], q_strides[1], q_strides[2]};
  const Strides ks{k_strides[0], k_strides[1], k_strides[2]};
  const Strides vs{v_strides[0], v_strides[1], v_strides[2]};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == DAX_BF16) return run_prepare<true>(q, k, v, B, heads, Sq, Sk, qs, ks, vs, sm_scale, mode, ws, st);
  return run_prepare<false>(q, k, v, B, heads, Sq, Sk, qs, ks, vs, sm_scale, mode, ws, st);
}
