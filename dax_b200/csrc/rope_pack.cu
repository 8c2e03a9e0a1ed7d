// RMSNorm over the full hidden dimension + 3-D rotary embedding + pack into the exchange layout,
// one pass over HBM (2 bytes read + 2 bytes written per element; the rotary tables and the norm
// weight stay in L2).
//
// CTAs stride over the token rows.  A row is read once: it travels through a ring of rows in shared memory
// (cp.async, 16 bytes per thread and vector; every thread reads back only what it copied itself, so no barrier
// is involved) with the next rows' copies in flight while the current row is normalised and rotated.  The sum of
// squares either comes from the per-column-tile partial sums the projection GEMM's epilogue wrote
// (summed in tile order, so the result does not depend on scheduling) or is reduced here.
// The normalised value is rounded to the tensor dtype before the rotation, like the tensor the
// reference materialises between its RMSNorm module and apply_rotary_emb
// (dax/adapters/wan/attn_adapter.py:108-109,164-173); the rotation itself runs in fp32 on
// interleaved pairs (x[2i], x[2i+1]) * (cos_i + j sin_i) and is rounded once.
#include <algorithm>

#include "quant_common.cuh"

namespace dax {
namespace {

constexpr int kMaxVec = 4;       // 8-element vectors per thread
constexpr int kMaxThreads = 320;  // rows up to 8 * 320 * 4 elements

struct alignas(16) V8 {
  uint32_t w[4];  // eight 16-bit elements, two per word
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

// What a thread needs of one row besides its vectors: its four rotary pairs (the same for every vector of the
// thread, because the thread's vectors lie a multiple of 128 elements apart) and its share of the GEMM's partial
// sums of squares.  These come from L2 and are loaded one row ahead; the vectors come from HBM and travel through a
// ring of kStages rows in shared memory, each thread copying (cp.async) and reading back its own 16-byte pieces, so
// that no barrier is needed and the bytes in flight do not cost registers.
struct RowSide {
  float4 c, sn;
  float part[2];
};

template <int NV>
struct StagesFor {
  static constexpr int value = NV <= 2 ? 4 : 3;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// T threads per CTA, NV 16-byte vectors per thread; FULL: the row is exactly T * NV vectors (no predicates)
template <bool BF16, int NV, int T, bool FULL>
__global__ void __launch_bounds__(T, NV <= 3 ? 3 : 2)
rmsnorm_rope_pack_kernel(const uint16_t* __restrict__ x, int64_t s, int64_t D, int64_t ldx,
                         const float* __restrict__ row_sumsq, int64_t n_partials, int do_norm,
                         const uint16_t* __restrict__ w, float eps, const float* __restrict__ rope_cos,
                         const float* __restrict__ rope_sin, int64_t token_offset, uint16_t* __restrict__ out,
                         int64_t ldo, int64_t col_group, int64_t group_stride, const GroupTable tab) {
  static_assert((T * 8) % 128 == 0, "a thread's vectors must lie a multiple of one head apart");
  constexpr int kStages = StagesFor<NV>::value;
  extern __shared__ __align__(16) uint8_t ring_raw[];
  V8* ring = reinterpret_cast<V8*>(ring_raw);  // [kStages][NV][T]
  __shared__ float red[2][T / 32];
  const int tid = threadIdx.x, lane = tid & 31;
  const int nvec = static_cast<int>(D / 8);
  const bool rope = rope_cos != nullptr;
  const bool partials = do_norm && row_sumsq != nullptr;
  const int pair0 = (tid * 8 & 127) >> 1;  // 4 consecutive pairs of one head

  // per-thread constants of the row layout: output offset of each vector and the norm weight
  int64_t out_off[NV];
  V8 wv[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t n = static_cast<int64_t>(tid + i * T) * 8;
    const int64_t g = n / col_group;
    out_off[i] = (tab.n > 0 ? tab.off[g < kMaxGroups ? g : 0] : g * group_stride) + (n - g * col_group);
    if (do_norm && w != nullptr && (FULL || tid + i * T < nvec)) wv[i] = *reinterpret_cast<const V8*>(w + n);
  }
  auto fetch_row = [&](int64_t row, int slot) {
    if (row < s) {
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (FULL || tid + i * T < nvec)
          cp_async16(ring + (slot * NV + i) * T + tid, x + row * ldx + static_cast<int64_t>(tid + i * T) * 8);
    }
    cp_async_commit();  // one group per row, empty past the end, so that the group count stays uniform
  };
  auto load_side = [&](int64_t row, RowSide& r) {
    if (rope) {
      r.c = *reinterpret_cast<const float4*>(rope_cos + (token_offset + row) * 64 + pair0);
      r.sn = *reinterpret_cast<const float4*>(rope_sin + (token_offset + row) * 64 + pair0);
    }
    if (partials) {
      // the GEMM's per-tile partial sums: lane j holds partials j and j + 32
      r.part[0] = lane < n_partials ? row_sumsq[row * n_partials + lane] : 0.f;
      r.part[1] = lane + 32 < n_partials ? row_sumsq[row * n_partials + lane + 32] : 0.f;
    }
  };
  RowSide cur, nxt;
  int64_t t = blockIdx.x;
  const int64_t step = gridDim.x;
#pragma unroll
  for (int k = 0; k < kStages - 1; ++k) fetch_row(t + k * step, k);
  if (t < s) load_side(t, cur);
  // CTAs stride over the rows with the next kStages - 1 rows in flight
  for (int it = 0; t < s; t += step, ++it) {
    fetch_row(t + (kStages - 1) * step, (it + kStages - 1) % kStages);
    if (t + step < s) load_side(t + step, nxt);
    cp_async_wait<kStages - 1>();  // this thread's pieces of row t have landed
    V8 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (FULL || tid + i * T < nvec) v[i] = ring[((it % kStages) * NV + i) * T + tid];
    float rstd = 1.f;
    if (do_norm) {
      float ss;
      if (partials) {
        // added in an order fixed by the lane number alone
        ss = cur.part[0] + cur.part[1];
        for (int64_t j = lane + 64; j < n_partials; j += 32) ss += row_sumsq[t * n_partials + j];  // very wide rows only
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      } else {
        ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
          if (FULL || tid + i * T < nvec) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float lo, hi;
              unpack2<BF16>(v[i].w[k], lo, hi);
              ss = fmaf(lo, lo, ss);
              ss = fmaf(hi, hi, ss);
            }
          }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float* r = red[it & 1];  // two buffers: one barrier per row
        if (lane == 0) r[tid >> 5] = ss;
        __syncthreads();
        ss = 0.f;
#pragma unroll
        for (int k = 0; k < T / 32; ++k) ss += r[k];
      }
      rstd = rsqrtf(ss / static_cast<float>(D) + eps);
    }
    const uint64_t rstd2 = f2_splat(rstd);
    const float cs[4] = {cur.c.x, cur.c.y, cur.c.z, cur.c.w};
    const float sn[4] = {cur.sn.x, cur.sn.y, cur.sn.z, cur.sn.w};
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (FULL || tid + i * T < nvec) {
        float f[8];
        if (do_norm) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t p = f2_mul(f2_from16<BF16>(v[i].w[k]), rstd2);
            if (w != nullptr) p = f2_mul(p, f2_from16<BF16>(wv[i].w[k]));
            // rounded to the tensor dtype, as the reference's RMSNorm module returns it
            unpack2<BF16>(f2_to16_rn<BF16>(p), f[2 * k], f[2 * k + 1]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) unpack2<BF16>(v[i].w[k], f[2 * k], f[2 * k + 1]);
        }
        if (rope) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = f[2 * j], b = f[2 * j + 1];
            f[2 * j] = a * cs[j] - b * sn[j];
            f[2 * j + 1] = a * sn[j] + b * cs[j];
          }
        }
        V8 o;
#pragma unroll
        for (int k = 0; k < 4; ++k) o.w[k] = pack2_rn<BF16>(f[2 * k], f[2 * k + 1]);
        *reinterpret_cast<V8*>(out + out_off[i] + t * ldo) = o;
      }
    }
    cur = nxt;
  }
}

template <bool BF16, int NV, int T, bool FULL, typename... Args>
int launch(int64_t s, cudaStream_t st, Args... args) {
  int per_sm = 0;
  constexpr size_t smem = static_cast<size_t>(StagesFor<NV>::value) * NV * T * sizeof(V8);
  if (smem > 40 * 1024)
    DAX_CUDA(cudaFuncSetAttribute(rmsnorm_rope_pack_kernel<BF16, NV, T, FULL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
  DAX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rmsnorm_rope_pack_kernel<BF16, NV, T, FULL>, T, smem));
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(s, static_cast<int64_t>(sm_count()) * std::max(per_sm, 1)));
  rmsnorm_rope_pack_kernel<BF16, NV, T, FULL><<<grid, T, smem, st>>>(args...);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

template <bool BF16, typename... Args>
int dispatch(int64_t s, int64_t D, cudaStream_t st, Args... args) {
  const int64_t nvec = D / 8;
  // rows that fill every thread of the CTA exactly run without predicates (5120 = 320 threads x 2 vectors x 8)
  if (nvec == 320 * 2) return launch<BF16, 2, 320, true>(s, st, args...);
  if (nvec == 256 * 1) return launch<BF16, 1, 256, true>(s, st, args...);
  if (nvec == 256 * 2) return launch<BF16, 2, 256, true>(s, st, args...);
  if (nvec == 256 * 4) return launch<BF16, 4, 256, true>(s, st, args...);
  const int64_t nv = (nvec + 255) / 256;
  if (nv <= 1) return launch<BF16, 1, 256, false>(s, st, args...);
  if (nv <= 2) return launch<BF16, 2, 256, false>(s, st, args...);
  if (nv <= 3) return launch<BF16, 3, 256, false>(s, st, args...);
  if (nv <= 4) return launch<BF16, 4, 256, false>(s, st, args...);
  return launch<BF16, kMaxVec, kMaxThreads, false>(s, st, args...);
}

}  // namespace
}  // namespace dax

namespace dax {
namespace {
int rope_pack_entry(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx, const float* row_sumsq,
                    int64_t n_partials, int do_norm, const void* norm_weight, float eps, const float* rope_cos,
                    const float* rope_sin, int64_t token_offset, void* out, int64_t ldo, int64_t col_group,
                    int64_t group_stride, const GroupTable& tab, void* stream) {
  DAX_REQUIRE(s >= 0 && D > 0, DAX_ERR_INVALID, "rmsnorm_rope_pack: bad shape s=%lld D=%lld", (long long)s, (long long)D);
  if (s == 0) return DAX_OK;
  DAX_REQUIRE(x && out, DAX_ERR_INVALID, "rmsnorm_rope_pack: null pointer");
  DAX_REQUIRE(dtype == DAX_BF16 || dtype == DAX_F16, DAX_ERR_UNSUPPORTED, "rmsnorm_rope_pack: dtype %d is not BF16/F16", dtype);
  DAX_REQUIRE(D % 128 == 0 && D <= 8 * kMaxThreads * kMaxVec, DAX_ERR_UNSUPPORTED,
              "rmsnorm_rope_pack: D=%lld must be a multiple of 128 and at most %d", (long long)D, 8 * kMaxThreads * kMaxVec);
  DAX_REQUIRE(col_group > 0 && D % col_group == 0 && col_group % 8 == 0, DAX_ERR_ALIGN,
              "rmsnorm_rope_pack: col_group=%lld must divide D and be a multiple of 8", (long long)col_group);
  DAX_REQUIRE(tab.n == 0 || tab.n == D / col_group, DAX_ERR_INVALID,
              "rmsnorm_rope_pack: %d group pointers for %lld column groups", tab.n, (long long)(D / col_group));
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
    return dispatch<true>(s, D, st, xp, s, D, ldx, row_sumsq, n_partials, do_norm, wp, eps, rope_cos, rope_sin, token_offset,
                          op, ldo, col_group, group_stride, tab);
  return dispatch<false>(s, D, st, xp, s, D, ldx, row_sumsq, n_partials, do_norm, wp, eps, rope_cos, rope_sin, token_offset,
                         op, ldo, col_group, group_stride, tab);
}
}  // namespace
}  // namespace dax

extern "C" int dax_rmsnorm_rope_pack(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx,
                                     const float* row_sumsq, int64_t n_partials, int do_norm,
                                     const void* norm_weight, float eps, const float* rope_cos,
                                     const float* rope_sin, int64_t token_offset, void* out, int64_t ldo,
                                     int64_t col_group, int64_t group_stride, void* stream) {
  dax::GroupTable tab{};
  return dax::rope_pack_entry(x, dtype, s, D, ldx, row_sumsq, n_partials, do_norm, norm_weight, eps, rope_cos, rope_sin,
                              token_offset, out, ldo, col_group, group_stride, tab, stream);
}

extern "C" int dax_rmsnorm_rope_pack_scatter(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx,
                                             const float* row_sumsq, int64_t n_partials, int do_norm,
                                             const void* norm_weight, float eps, const float* rope_cos,
                                             const float* rope_sin, int64_t token_offset, void* const* group_out,
                                             int64_t n_groups, int64_t ldo, int64_t col_group, void* stream) {
  dax::GroupTable tab{};
  void* base = nullptr;
  int rc = dax::make_group_table(group_out, n_groups, 2, &tab, &base);
  if (rc != DAX_OK) return rc;
  return dax::rope_pack_entry(x, dtype, s, D, ldx, row_sumsq, n_partials, do_norm, norm_weight, eps, rope_cos, rope_sin,
                              token_offset, base, ldo, col_group, 0, tab, stream);
}
