// RMSNorm over the full hidden dimension + 3-D rotary embedding + pack into the exchange layout,
// one pass over HBM (2 bytes read + 2 bytes written per element; the rotary tables and the norm
// weight stay in L2).
//
// One CTA per token row.  The row is read once into registers with 128-bit loads.  The sum of
// squares either comes from the per-column-tile partial sums the projection GEMM's epilogue wrote
// (summed in tile order, so the result does not depend on scheduling) or is reduced here.
// The normalised value is rounded to the tensor dtype before the rotation, like the tensor the
// reference materialises between its RMSNorm module and apply_rotary_emb
// (dax/adapters/wan/attn_adapter.py:108-109,164-173); the rotation itself runs in fp32 on
// interleaved pairs (x[2i], x[2i+1]) * (cos_i + j sin_i) and is rounded once.
#include "common.cuh"

namespace dax {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 4;  // 8-element vectors per thread: rows up to 8192 elements

struct alignas(16) V8 {
  uint16_t v[8];
};

template <bool BF16>
__device__ __forceinline__ float to_f(uint16_t u) {
  if constexpr (BF16) return __bfloat162float(__ushort_as_bfloat16(u));
  else return __half2float(__ushort_as_half(u));
}
template <bool BF16>
__device__ __forceinline__ uint16_t from_f(float f) {
  if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  else return __half_as_ushort(__float2half_rn(f));
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads)
rmsnorm_rope_pack_kernel(const uint16_t* __restrict__ x, int64_t s, int64_t D, int64_t ldx,
                         const float* __restrict__ row_sumsq, int64_t n_partials, int do_norm,
                         const uint16_t* __restrict__ w, float eps, const float* __restrict__ rope_cos,
                         const float* __restrict__ rope_sin, int64_t token_offset, uint16_t* __restrict__ out,
                         int64_t ldo, int64_t col_group, int64_t group_stride) {
  __shared__ float red[kThreads / 32];
  const int64_t t = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t nvec = D / 8;

  V8 regs[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t vi = tid + static_cast<int64_t>(i) * kThreads;
    if (vi < nvec) {
      regs[i] = *reinterpret_cast<const V8*>(x + t * ldx + vi * 8);
      if (do_norm && row_sumsq == nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = to_f<BF16>(regs[i].v[j]);
          ss = fmaf(f, f, ss);
        }
      }
    }
  }
  float rstd = 1.f;
  if (do_norm) {
    if (row_sumsq != nullptr) {
      ss = 0.f;
      for (int64_t j = 0; j < n_partials; ++j) ss += row_sumsq[t * n_partials + j];
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((tid & 31) == 0) red[tid >> 5] = ss;
      __syncthreads();
      ss = 0.f;
#pragma unroll
      for (int k = 0; k < kThreads / 32; ++k) ss += red[k];
    }
    rstd = rsqrtf(ss / static_cast<float>(D) + eps);
  }

  const bool rope = rope_cos != nullptr;
  const int64_t gtok = token_offset + t;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t vi = tid + static_cast<int64_t>(i) * kThreads;
    if (vi < nvec) {
      const int64_t n = vi * 8;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = to_f<BF16>(regs[i].v[j]);
      if (do_norm) {
        V8 wv;
        if (w != nullptr) wv = *reinterpret_cast<const V8*>(w + n);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float y = f[j] * rstd;
          if (w != nullptr) y *= to_f<BF16>(wv.v[j]);
          f[j] = to_f<BF16>(from_f<BF16>(y));
        }
      }
      if (rope) {
        const int pair0 = static_cast<int>((n & 127) >> 1);  // 4 consecutive pairs of one head
        const float4 c4 = *reinterpret_cast<const float4*>(rope_cos + gtok * 64 + pair0);
        const float4 s4 = *reinterpret_cast<const float4*>(rope_sin + gtok * 64 + pair0);
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w};
        const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = f[2 * j], b = f[2 * j + 1];
          f[2 * j] = a * cs[j] - b * sn[j];
          f[2 * j + 1] = a * sn[j] + b * cs[j];
        }
      }
      V8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] = from_f<BF16>(f[j]);
      const int64_t g = n / col_group;
      *reinterpret_cast<V8*>(out + g * group_stride + t * ldo + (n - g * col_group)) = o;
    }
  }
}

}  // namespace
}  // namespace dax

extern "C" int dax_rmsnorm_rope_pack(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx,
                                     const float* row_sumsq, int64_t n_partials, int do_norm,
                                     const void* norm_weight, float eps, const float* rope_cos,
                                     const float* rope_sin, int64_t token_offset, void* out, int64_t ldo,
                                     int64_t col_group, int64_t group_stride, void* stream) {
  using namespace dax;
  DAX_REQUIRE(s >= 0 && D > 0, DAX_ERR_INVALID, "rmsnorm_rope_pack: bad shape s=%lld D=%lld", (long long)s, (long long)D);
  if (s == 0) return DAX_OK;
  DAX_REQUIRE(x && out, DAX_ERR_INVALID, "rmsnorm_rope_pack: null pointer");
  DAX_REQUIRE(dtype == DAX_BF16 || dtype == DAX_F16, DAX_ERR_UNSUPPORTED, "rmsnorm_rope_pack: dtype %d is not BF16/F16", dtype);
  DAX_REQUIRE(D % 128 == 0 && D <= 8 * kThreads * kMaxVec, DAX_ERR_UNSUPPORTED,
              "rmsnorm_rope_pack: D=%lld must be a multiple of 128 and at most %d", (long long)D, 8 * kThreads * kMaxVec);
  DAX_REQUIRE(col_group > 0 && D % col_group == 0 && col_group % 8 == 0, DAX_ERR_ALIGN,
              "rmsnorm_rope_pack: col_group=%lld must divide D and be a multiple of 8", (long long)col_group);
  DAX_REQUIRE(ldx % 8 == 0 && ldo % 8 == 0 && group_stride % 8 == 0, DAX_ERR_ALIGN,
              "rmsnorm_rope_pack: ldx, ldo, group_stride must be multiples of 8 elements");
  DAX_REQUIRE(aligned16(x) && aligned16(out) && (norm_weight == nullptr || aligned16(norm_weight)) &&
                  (rope_cos == nullptr || (aligned16(rope_cos) && aligned16(rope_sin))),
              DAX_ERR_ALIGN, "rmsnorm_rope_pack: pointers must be 16-byte aligned");
  DAX_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr), DAX_ERR_INVALID, "rmsnorm_rope_pack: cos/sin must come together");
  DAX_REQUIRE(row_sumsq == nullptr || n_partials > 0, DAX_ERR_INVALID, "rmsnorm_rope_pack: n_partials must be positive");
  DAX_REQUIRE(s < (1ll << 31), DAX_ERR_UNSUPPORTED, "rmsnorm_rope_pack: s too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const uint16_t* wp = static_cast<const uint16_t*>(norm_weight);
  uint16_t* op = static_cast<uint16_t*>(out);
  if (dtype == DAX_BF16)
    rmsnorm_rope_pack_kernel<true><<<static_cast<unsigned>(s), kThreads, 0, st>>>(
        xp, s, D, ldx, row_sumsq, n_partials, do_norm, wp, eps, rope_cos, rope_sin, token_offset, op, ldo, col_group, group_stride);
  else
    rmsnorm_rope_pack_kernel<false><<<static_cast<unsigned>(s), kThreads, 0, st>>>(
        xp, s, D, ldx, row_sumsq, n_partials, do_norm, wp, eps, rope_cos, rope_sin, token_offset, op, ldo, col_group, group_stride);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}
