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
#include "quant_common.cuh"

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
  uint32_t mx2[4] = {0u, 0u, 0u, 0u};  // packed running maxima of |V|
#pragma unroll
  for (int j = 0; j < 8; ++j) sum[j] = 0.f;
  for (int64_t t = t0 + tl; t < t1; t += 16) {
    const uint4 kv = *reinterpret_cast<const uint4*>(kb + t * ks.t);
    const uint4 vv = *reinterpret_cast<const uint4*>(vb + t * vs.t);
    const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float lo, hi;
      unpack2<BF16>(kw[q], lo, hi);
      sum[2 * q] += lo;
      sum[2 * q + 1] += hi;
      mx2[q] = absmax2<BF16>(mx2[q], vw[q]);
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) unpack2<BF16>(mx2[q], mx[2 * q], mx[2 * q + 1]);
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

// grid (Sq_pad / 64, BH), 256 threads: a warp owns 8 consecutive tokens, a lane 4 channels of each.  All eight
// loads of a lane are issued before the first token is reduced.
template <bool BF16, bool I8>
__global__ void __launch_bounds__(256)
quant_q_kernel(const uint16_t* __restrict__ q, Strides qs, int heads, int64_t Sq, int64_t Sq_pad, float cscale,
               void* __restrict__ qo, float* __restrict__ q_scale) {
  constexpr int TPW = 8;  // tokens per warp
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int lane = threadIdx.x & 31;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * 64 + (threadIdx.x >> 5) * TPW;
  const uint16_t* src = q + b * qs.b + h * qs.h + lane * 4;
  uint2 raw[TPW];
#pragma unroll
  for (int i = 0; i < TPW; ++i)
    raw[i] = t0 + i < Sq ? *reinterpret_cast<const uint2*>(src + (t0 + i) * qs.t) : make_uint2(0u, 0u);
#pragma unroll
  for (int i = 0; i < TPW; ++i) {
    const int64_t t = t0 + i;
    if (t >= Sq_pad) break;
    float f[4];
    unpack2<BF16>(raw[i].x, f[0], f[1]);
    unpack2<BF16>(raw[i].y, f[2], f[3]);
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
      // 16-bit scores: Q goes through unscaled, as bf16 (the scale is applied to the scores)
      uint2 w;
      w.x = pack2_rn<true>(f[0], f[1]);
      w.y = pack2_rn<true>(f[2], f[3]);
      reinterpret_cast<uint2*>(static_cast<uint16_t*>(qo) + row * 128)[lane] = w;
      if (lane == 0) q_scale[row] = cscale;
    }
  }
}

// grid (Sk_pad / 128, BH), 256 threads: thread = (8 channels, tokens tl, tl + 16, ..., tl + 112), so that a
// warp's 16-byte loads cover two whole 256-byte token rows.
template <bool BF16, bool I8>
__global__ void __launch_bounds__(256)
quant_k_kernel(const uint16_t* __restrict__ k, Strides ks, int heads, int64_t Sk, int64_t Sk_pad,
               const float* __restrict__ k_mean, void* __restrict__ ko, float* __restrict__ k_scale) {
  __shared__ float red[8];
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int cg = threadIdx.x & 15, tl = threadIdx.x >> 4;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * 128;
  const uint16_t* src = k + b * ks.b + h * ks.h + cg * 8;
  uint4 raw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t t = tok0 + tl + 16 * i;
    raw[i] = t < Sk ? *reinterpret_cast<const uint4*>(src + t * ks.t) : make_uint4(0u, 0u, 0u, 0u);
  }
  float mean[8];
  *reinterpret_cast<float4*>(&mean[0]) = *reinterpret_cast<const float4*>(k_mean + bh * 128 + cg * 8);
  *reinterpret_cast<float4*>(&mean[4]) = *reinterpret_cast<const float4*>(k_mean + bh * 128 + cg * 8 + 4);
  float f[8][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool live = tok0 + tl + 16 * i < Sk;
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float lo, hi;
      unpack2<BF16>(w[q], lo, hi);
      f[i][2 * q] = live ? lo - mean[2 * q] : 0.f;
      f[i][2 * q + 1] = live ? hi - mean[2 * q + 1] : 0.f;
      amax = fmaxf(amax, fmaxf(fabsf(f[i][2 * q]), fabsf(f[i][2 * q + 1])));
    }
  }
  const int64_t row0 = static_cast<int64_t>(bh) * Sk_pad + tok0 + tl;
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
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t w[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        w[q] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int qi = max(-127, min(127, __float2int_rn(f[i][q * 4 + j] * inv)));
          w[q] |= (static_cast<uint32_t>(qi) & 0xffu) << (8 * j);
        }
      }
      *reinterpret_cast<uint2*>(static_cast<uint8_t*>(ko) + (row0 + 16 * i) * 128 + cg * 8) = make_uint2(w[0], w[1]);
    }
    if (threadIdx.x == 0) k_scale[static_cast<int64_t>(bh) * (Sk_pad / 128) + blockIdx.x] = sc;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint4 w;
      w.x = pack2_rn<true>(f[i][0], f[i][1]);
      w.y = pack2_rn<true>(f[i][2], f[i][3]);
      w.z = pack2_rn<true>(f[i][4], f[i][5]);
      w.w = pack2_rn<true>(f[i][6], f[i][7]);
      *reinterpret_cast<uint4*>(static_cast<uint16_t*>(ko) + (row0 + 16 * i) * 128 + cg * 8) = w;
    }
    if (threadIdx.x == 0) k_scale[static_cast<int64_t>(bh) * (Sk_pad / 128) + blockIdx.x] = 1.f;
  }
}

// grid (Sk_pad / 128, BH), 256 threads.  Reads a [128 tokens x 128 channels] tile row-wise, writes it
// transposed: vt[bh, channel, token].  Thread = (8 channels, 8 consecutive tokens): it converts its 8 x 8 block,
// gathers the 8 tokens of each channel into one 8- or 16-byte shared-memory store, and the warps then copy whole
// channel rows out.
template <bool BF16, bool F8>
__global__ void __launch_bounds__(256)
quant_v_kernel(const uint16_t* __restrict__ v, Strides vs, int heads, int64_t Sk, int64_t Sk_pad,
               const float* __restrict__ v_scale, void* __restrict__ vo) {
  using OutT = typename std::conditional<F8, uint8_t, uint16_t>::type;
  constexpr int PITCH = 128 + 16 / static_cast<int>(sizeof(OutT));  // elements: rows 16 bytes apart in the banks
  __shared__ __align__(16) OutT tile[128 * PITCH];                  // [channel][token]
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * 128;
  const int cg = threadIdx.x & 15, tq = threadIdx.x >> 4;
  const uint16_t* src = v + b * vs.b + h * vs.h + cg * 8;
  uint4 raw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t t = tok0 + tq * 8 + i;
    raw[i] = t < Sk ? *reinterpret_cast<const uint4*>(src + t * vs.t) : make_uint4(0u, 0u, 0u, 0u);
  }
  float inv[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) inv[j] = 1.f / v_scale[bh * 128 + cg * 8 + j];
  float x[8][8];  // [token][channel]
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float lo, hi;
      unpack2<BF16>(w[q], lo, hi);
      x[i][2 * q] = lo * inv[2 * q];
      x[i][2 * q + 1] = hi * inv[2 * q + 1];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    OutT* dst = &tile[(cg * 8 + j) * PITCH + tq * 8];
    if constexpr (F8) {
      uint16_t p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(p[i]) : "f"(x[2 * i + 1][j]), "f"(x[2 * i][j]));
      *reinterpret_cast<uint2*>(dst) = make_uint2(static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 16),
                                                  static_cast<uint32_t>(p[2]) | (static_cast<uint32_t>(p[3]) << 16));
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack2_rn<true>(x[0][j], x[1][j]), pack2_rn<true>(x[2][j], x[3][j]),
                                                  pack2_rn<true>(x[4][j], x[5][j]), pack2_rn<true>(x[6][j], x[7][j]));
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
        reinterpret_cast<uint2*>(dst)[lane] = *reinterpret_cast<const uint2*>(&tile[c * PITCH + lane * 4]);
      }
    }
  }
}

template <bool BF16>
int run_prepare(const void* q, const void* k, const void* v, int64_t B, int64_t heads, int64_t Sq, int64_t Sk,
                Strides qs, Strides ks, Strides vs, float sm_scale, int mode, int parts, const AttnWorkspace& ws,
                cudaStream_t st) {
  const int64_t BH = B * heads;
  const uint16_t* qp = static_cast<const uint16_t*>(q);
  const uint16_t* kp = static_cast<const uint16_t*>(k);
  const uint16_t* vp = static_cast<const uint16_t*>(v);
  const bool qk_i8 = attn_qk_bytes(mode) == 1, v_f8 = attn_pv_bytes(mode) == 1;
  const float cscale = sm_scale * 1.4426950408889634f;
  const unsigned bh = static_cast<unsigned>(BH);
  const dim3 gq(static_cast<unsigned>((ws.Sq_pad + 63) / 64), bh), gk(static_cast<unsigned>(ws.Sk_pad / 128), bh);
  if (parts & DAX_ATTN_PREPARE_KV) {
    colstats_kernel<BF16><<<dim3(static_cast<unsigned>(ws.chunks), bh), 256, 0, st>>>(kp, vp, ks, vs, static_cast<int>(heads), Sk, ws.part, ws.chunks);
    colstats_fin_kernel<<<bh, 128, 0, st>>>(ws.part, ws.chunks, Sk, v_f8 ? 1 : 0, ws.k_mean, ws.v_scale);
    if (qk_i8) quant_k_kernel<BF16, true><<<gk, 256, 0, st>>>(kp, ks, static_cast<int>(heads), Sk, ws.Sk_pad, ws.k_mean, ws.k, ws.k_scale);
    else quant_k_kernel<BF16, false><<<gk, 256, 0, st>>>(kp, ks, static_cast<int>(heads), Sk, ws.Sk_pad, ws.k_mean, ws.k, ws.k_scale);
    if (v_f8) quant_v_kernel<BF16, true><<<gk, 256, 0, st>>>(vp, vs, static_cast<int>(heads), Sk, ws.Sk_pad, ws.v_scale, ws.vt);
    else quant_v_kernel<BF16, false><<<gk, 256, 0, st>>>(vp, vs, static_cast<int>(heads), Sk, ws.Sk_pad, ws.v_scale, ws.vt);
  }
  if (parts & DAX_ATTN_PREPARE_Q) {
    if (qk_i8) quant_q_kernel<BF16, true><<<gq, 256, 0, st>>>(qp, qs, static_cast<int>(heads), Sq, ws.Sq_pad, cscale, ws.q, ws.q_scale);
    else quant_q_kernel<BF16, false><<<gq, 256, 0, st>>>(qp, qs, static_cast<int>(heads), Sq, ws.Sq_pad, cscale, ws.q, ws.q_scale);
  }
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

extern "C" int dax_attn_prepare_parts(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                                      int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3],
                                      int64_t v_strides[3], float sm_scale, int mode, int parts, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  using namespace dax;
  DAX_REQUIRE(parts >= 1 && parts <= 3, DAX_ERR_INVALID, "attn_prepare: parts must be a combination of KV (1) and Q (2)");
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
  if (dtype == DAX_BF16) return run_prepare<true>(q, k, v, B, heads, Sq, Sk, qs, ks, vs, sm_scale, mode, parts, ws, st);
  return run_prepare<false>(q, k, v, B, heads, Sq, Sk, qs, ks, vs, sm_scale, mode, parts, ws, st);
}

extern "C" int dax_attn_prepare(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                                int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3],
                                int64_t v_strides[3], float sm_scale, int mode, void* workspace,
                                size_t workspace_bytes, void* stream) {
  return dax_attn_prepare_parts(q, k, v, dtype, B, heads, Sq, Sk, q_strides, k_strides, v_strides, sm_scale, mode,
                                DAX_ATTN_PREPARE_KV | DAX_ATTN_PREPARE_Q, workspace, workspace_bytes, stream);
}
