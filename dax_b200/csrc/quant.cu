// Per-token dynamic activation quantiser (absmax -> scale -> INT8 / FP8), one pass over HBM.
//
// HBM-bound: 2 (or 4) bytes read and 1 byte written per element plus 4 bytes per row.  A row is
// read once with 128-bit loads into registers, reduced, and quantised from registers.  Short rows go one per
// warp; rows of 257..2048 vectors go to CTAs that stride over the rows with the next row's loads already in
// flight while the current row is reduced and converted (6.6-6.7 TB/s at 75,600 x 5120 / 13,824 on a B200);
// longer rows are re-read from L2 for the second pass.
//
// Arithmetic follows the reference bit for bit (dax/quant/nn/dynamic/functional.py:124-135 and
// dax/quant/nn/quantized/functional.py:11-20, evaluated eagerly):
//   amax  = max |x|                       (exact in any precision)
//   scale = round_to_input_dtype(amax / qmax), floored at fp32 eps, widened to fp32
//   INT8: q = clamp(rint(x * (1.0f / scale)), -128, 127)    (multiply by the reciprocal)
//   FP8 : q = round_nearest_even_to_fp8(clamp(x / scale))   (true division, see div_rn_by)
// All fp32 operations are IEEE round-to-nearest (intrinsics, or the packed-pair instructions of quant_common.cuh,
// whose lanes round like the scalar ones) so that the compiler cannot contract or approximate them.
#include <algorithm>

#include "quant_common.cuh"

namespace dax {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 8;  // 16-byte vectors cached per thread

template <typename T> struct VecTraits;
template <> struct VecTraits<__nv_bfloat16> {
  static constexpr int N = 8;
  static constexpr bool IS16 = true, BF16 = true;
  __device__ static float round_trip(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
};
template <> struct VecTraits<__half> {
  static constexpr int N = 8;
  static constexpr bool IS16 = true, BF16 = false;
  __device__ static float round_trip(float f) { return __half2float(__float2half_rn(f)); }
};
template <> struct VecTraits<float> {
  static constexpr int N = 4;
  static constexpr bool IS16 = false, BF16 = false;
  __device__ static float round_trip(float f) { return f; }
};

// 16 bytes of a row: 8 sixteen-bit elements (two per word) or 4 fp32 elements
template <typename T>
struct alignas(16) Vec {
  uint32_t w[4];
};

// Running |.|-maximum of a thread: packed for 16-bit inputs (exact: the maximum of bf16 values is a bf16 value)
template <typename T>
struct AbsMax {
  uint32_t packed = 0u;
  float f = 0.f;
  __device__ __forceinline__ void add(const Vec<T>& t) {
    using V = VecTraits<T>;
    if constexpr (V::IS16) {
#pragma unroll
      for (int k = 0; k < 4; ++k) packed = absmax2<V::BF16>(packed, t.w[k]);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) f = fmaxf(f, fabsf(__uint_as_float(t.w[k])));
    }
  }
  __device__ __forceinline__ float value() const {
    using V = VecTraits<T>;
    if constexpr (V::IS16) {
      float lo, hi;
      unpack2<V::BF16>(packed, lo, hi);
      return fmaxf(lo, hi);
    } else {
      return f;
    }
  }
};

// One 16-byte vector of inputs -> N codes.
template <typename T, int QDT>
__device__ __forceinline__ void emit_vec(const Vec<T>& t, float s, float inv, uint8_t* dst) {
  using V = VecTraits<T>;
  if constexpr (V::IS16) {
    const uint64_t neg_s2 = f2_splat(-s), inv2 = f2_splat(inv);
    const uint32_t w0 = quant_four16<V::BF16, QDT>(t.w[0], t.w[1], neg_s2, inv2);
    const uint32_t w1 = quant_four16<V::BF16, QDT>(t.w[2], t.w[3], neg_s2, inv2);
    *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
  } else {
    *reinterpret_cast<uint32_t*>(dst) = quant_four<QDT>(__uint_as_float(t.w[0]), __uint_as_float(t.w[1]),
                                                        __uint_as_float(t.w[2]), __uint_as_float(t.w[3]), s, inv);
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// TPR threads cooperate on one row; a CTA of kThreads handles kThreads / TPR rows.
template <typename T, int QDT, int TPR>
__global__ void __launch_bounds__(kThreads)
quant_rowwise_kernel(const T* __restrict__ x, int64_t M, int64_t K, int64_t ldx, int64_t col_group,
                     int64_t group_stride, uint8_t* __restrict__ q, float* __restrict__ scale) {
  constexpr int N = VecTraits<T>::N;
  constexpr int RPB = kThreads / TPR;
  __shared__ float red[kThreads / 32];

  const int tid = threadIdx.x;
  const int sub = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPB + tid / TPR;
  const bool live = row < M;
  const int64_t nvec = K / N;
  const bool cached = nvec <= static_cast<int64_t>(TPR) * kMaxVec;

  Vec<T> regs[kMaxVec];
  AbsMax<T> am;
  auto src = [&](int64_t vi) -> const Vec<T>* {
    const int64_t n = vi * N;
    const int64_t g = n / col_group;
    return reinterpret_cast<const Vec<T>*>(x + g * group_stride + row * ldx + (n - g * col_group));
  };
  if (live) {
    if (cached) {
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int64_t vi = sub + static_cast<int64_t>(i) * TPR;
        if (vi < nvec) {
          regs[i] = *src(vi);
          am.add(regs[i]);
        }
      }
    } else {
      for (int64_t vi = sub; vi < nvec; vi += TPR) {
        am.add(*src(vi));
      }
    }
  }
  float amax = warp_max(am.value());
  if constexpr (TPR > 32) {
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, red[w]);
  }
  if (!live) return;

  const float s = quant_scale<QDT>(amax, [](float v) { return VecTraits<T>::round_trip(v); });
  const float inv = quant_inv_scale(s);
  if (sub == 0) scale[row] = s;

  uint8_t* qrow = q + row * K;
  auto emit = [&](const Vec<T>& t, int64_t vi) {
    emit_vec<T, QDT>(t, s, inv, qrow + vi * N);
  };
  if (cached) {
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int64_t vi = sub + static_cast<int64_t>(i) * TPR;
      if (vi < nvec) emit(regs[i], vi);
    }
  } else {
    for (int64_t vi = sub; vi < nvec; vi += TPR) emit(*src(vi), vi);
  }
}

// Rows of 257..2048 vectors: CTAs stride over the rows and hold two rows in registers, the one being
// quantised and the next one, whose loads are issued before the reduction of the current row: the reduction,
// the barrier and the conversions run under the next row's memory latency.  NV = vectors per thread.
template <typename T, int QDT, int NV>
__global__ void __launch_bounds__(kThreads)
quant_rows_pipelined_kernel(const T* __restrict__ x, int64_t M, int64_t K, int64_t ldx, int64_t col_group,
                            int64_t group_stride, uint8_t* __restrict__ q, float* __restrict__ scale) {
  constexpr int N = VecTraits<T>::N;
  __shared__ float red[2][kThreads / 32];
  const int tid = threadIdx.x;
  const int nvec = static_cast<int>(K / N);
  // element offset of each of this thread's vectors inside a row (column-group addressing), fixed for all rows
  int64_t off[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t n = static_cast<int64_t>(tid + i * kThreads) * N;
    const int64_t g = n / col_group;
    off[i] = g * group_stride + (n - g * col_group);
  }
  auto load_row = [&](int64_t row, Vec<T> (&buf)[NV]) {
    const T* base = x + row * ldx;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (tid + i * kThreads < nvec) buf[i] = *reinterpret_cast<const Vec<T>*>(base + off[i]);
  };
  Vec<T> cur[NV], nxt[NV];
  int64_t row = blockIdx.x;
  if (row < M) load_row(row, cur);
  for (int it = 0; row < M; row += gridDim.x, ++it) {
    if (row + gridDim.x < M) load_row(row + gridDim.x, nxt);
    AbsMax<T> am;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (tid + i * kThreads < nvec) am.add(cur[i]);
    float amax = warp_max(am.value());
    float* r = red[it & 1];  // two buffers: one barrier per row is enough
    if ((tid & 31) == 0) r[tid >> 5] = amax;
    __syncthreads();
    amax = r[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, r[w]);
    const float s = quant_scale<QDT>(amax, [](float v) { return VecTraits<T>::round_trip(v); });
    const float inv = quant_inv_scale(s);
    if (tid == 0) scale[row] = s;
    uint8_t* qrow = q + row * K;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (tid + i * kThreads < nvec) emit_vec<T, QDT>(cur[i], s, inv, qrow + static_cast<int64_t>(tid + i * kThreads) * N);
#pragma unroll
    for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
  }
}

template <typename T, int QDT, int NV>
int launch_pipelined(const void* x, int64_t M, int64_t K, int64_t ldx, int64_t col_group, int64_t group_stride, void* q,
                     float* scale, cudaStream_t st) {
  int per_sm = 0;
  DAX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_rows_pipelined_kernel<T, QDT, NV>, kThreads, 0));
  const int64_t blocks = std::min<int64_t>(M, static_cast<int64_t>(sm_count()) * std::max(per_sm, 1));
  quant_rows_pipelined_kernel<T, QDT, NV><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
      static_cast<const T*>(x), M, K, ldx, col_group, group_stride, static_cast<uint8_t*>(q), scale);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

template <typename T, int QDT>
int launch(const void* x, int64_t M, int64_t K, int64_t ldx, int64_t col_group, int64_t group_stride, void* q,
           float* scale, cudaStream_t st) {
  const int64_t nvec = K / VecTraits<T>::N;
  if (nvec > 32 * kMaxVec && nvec <= kThreads * kMaxVec) {
    const int nv = static_cast<int>((nvec + kThreads - 1) / kThreads);
    if (nv <= 2) return launch_pipelined<T, QDT, 2>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    if (nv <= 3) return launch_pipelined<T, QDT, 3>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    if (nv <= 4) return launch_pipelined<T, QDT, 4>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    if (nv <= 6) return launch_pipelined<T, QDT, 6>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    return launch_pipelined<T, QDT, 8>(x, M, K, ldx, col_group, group_stride, q, scale, st);
  }
  if (nvec <= 32 * kMaxVec) {
    constexpr int RPB = kThreads / 32;
    const int64_t blocks = (M + RPB - 1) / RPB;
    quant_rowwise_kernel<T, QDT, 32><<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(
        static_cast<const T*>(x), M, K, ldx, col_group, group_stride, static_cast<uint8_t*>(q), scale);
  } else {
    quant_rowwise_kernel<T, QDT, kThreads><<<static_cast<unsigned>(M), kThreads, 0, st>>>(
        static_cast<const T*>(x), M, K, ldx, col_group, group_stride, static_cast<uint8_t*>(q), scale);
  }
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

template <typename T>
int dispatch_q(int q_dtype, const void* x, int64_t M, int64_t K, int64_t ldx, int64_t col_group,
               int64_t group_stride, void* q, float* scale, cudaStream_t st) {
  switch (q_dtype) {
    case DAX_I8: return launch<T, DAX_I8>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    case DAX_E4M3: return launch<T, DAX_E4M3>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    case DAX_E5M2: return launch<T, DAX_E5M2>(x, M, K, ldx, col_group, group_stride, q, scale, st);
    default: return fail(DAX_ERR_UNSUPPORTED, "quant_rowwise: q_dtype %d is not I8/E4M3/E5M2", q_dtype);
  }
}

}  // namespace
}  // namespace dax

extern "C" int dax_quant_rowwise(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int64_t col_group,
                                 int64_t group_stride, void* q, int q_dtype, float* scale, void* stream) {
  using namespace dax;
  DAX_REQUIRE(M >= 0 && K > 0, DAX_ERR_INVALID, "quant_rowwise: bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (M == 0) return DAX_OK;
  DAX_REQUIRE(x && q && scale, DAX_ERR_INVALID, "quant_rowwise: null pointer");
  DAX_REQUIRE(M < (1ll << 31), DAX_ERR_UNSUPPORTED, "quant_rowwise: M=%lld too large", (long long)M);
  DAX_REQUIRE(K % 16 == 0, DAX_ERR_ALIGN, "quant_rowwise: K=%lld must be a multiple of 16", (long long)K);
  DAX_REQUIRE(col_group > 0 && col_group % 16 == 0 && K % col_group == 0, DAX_ERR_ALIGN,
              "quant_rowwise: col_group=%lld must be a multiple of 16 that divides K", (long long)col_group);
  DAX_REQUIRE(ldx % 8 == 0 && group_stride % 8 == 0, DAX_ERR_ALIGN,
              "quant_rowwise: ldx and group_stride must be multiples of 8 elements");
  DAX_REQUIRE(aligned16(x) && aligned16(q), DAX_ERR_ALIGN, "quant_rowwise: x and q must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case DAX_BF16: return dispatch_q<__nv_bfloat16>(q_dtype, x, M, K, ldx, col_group, group_stride, q, scale, st);
    case DAX_F16: return dispatch_q<__half>(q_dtype, x, M, K, ldx, col_group, group_stride, q, scale, st);
    case DAX_F32: return dispatch_q<float>(q_dtype, x, M, K, ldx, col_group, group_stride, q, scale, st);
    default: return fail(DAX_ERR_UNSUPPORTED, "quant_rowwise: x_dtype %d is not BF16/F16/F32", x_dtype);
  }
}
