// LayerNorm + adaLN modulation (+ per-token quantisation) for the parts of a Wan DiT block around the
// attention: the normalised, modulated activations feed a quantised linear, so the kernel can emit the
// INT8 / FP8 codes and scales directly and the separate quantiser pass (and its HBM round trip) goes away.
//
// 2 bytes read per element, 2 written (16-bit output) and/or 1 written (codes).  Two kernels:
//  - rows whose width fills a CTA exactly (the model widths: 5120, 4096, 3072, 2048, 1536, 1024): one CTA of a few
//    warps per row, the row widened to fp32 once, arithmetic on fp32 pairs (ln_rows_cta_kernel below);
//  - any other width: one WARP owns a row, which lives packed in the warp's registers; mean, centred variance and
//    the absmax of the rounded outputs are warp shuffles (ln_modulate_quant_kernel).
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
__global__ void __launch_bounds__(LnThreads<NV>::value, NV <= 6 ? 3 : (NV <= 12 ? 2 : (NV <= 24 ? 3 : 2)))
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
      const float inv = quant_inv_scale(s);
      if (lane == 0) qscale[t] = s;
      const uint64_t neg_s2 = f2_splat(-s), inv2 = f2_splat(inv);
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (lane + 32 * i < nvec) {
          const uint32_t w0 = quant_four16<BF16, QDT>(raw[i].w[0], raw[i].w[1], neg_s2, inv2);
          const uint32_t w1 = quant_four16<BF16, QDT>(raw[i].w[2], raw[i].w[3], neg_s2, inv2);
          *reinterpret_cast<uint2*>(q + t * D + static_cast<int64_t>(lane + 32 * i) * 8) = make_uint2(w0, w1);
        }
    }
  }
}

// ---- rows that fill a CTA exactly: one CTA per row, T threads x NV vectors = D / 8 --------------------------------
// Bound by instruction issue before HBM, so the design counts instructions.  The rows travel through a ring of kRing
// rows in shared memory, each thread copying (cp.async) and reading back its own 16-byte pieces: the bytes in flight
// cost neither registers nor barriers.  A row is widened to fp32 once and stays in registers through the four steps
// (sum, centred sum of squares, normalise + round + absmax, quantise); the arithmetic runs on fp32 pairs.  Few
// threads per row (4-6 warps, 32-40 elements per thread) keep the per-row cost of the three CTA-wide reductions and
// of the scale small per element; several CTAs per SM hide one another's barriers.  The per-column coefficients are
// read from global memory for every row (they stay in L1: the rows themselves bypass it).
constexpr int kRing = 2;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// acc = max(|acc|, |w|) per half, sign bits left undefined (the caller clears them at the end): one instruction
template <bool BF16>
__device__ __forceinline__ uint32_t absmax2_lazy(uint32_t acc, uint32_t w) {
  uint32_t r;
  if constexpr (BF16) asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(acc), "r"(w));
  else asm("max.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(r) : "r"(acc), "r"(w));
  return r;
}

template <bool BF16, int QDT, int T, int NV, int MINB, int CR>
__global__ void __launch_bounds__(T, MINB)
ln_rows_cta_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t D, int64_t ldx, const float* __restrict__ w,
                   const float* __restrict__ b, const float* __restrict__ shift, const float* __restrict__ scale,
                   float eps, uint16_t* __restrict__ y, int64_t ldy, uint8_t* __restrict__ q, float* __restrict__ qscale) {
  constexpr int kWarps = T / 32;
  extern __shared__ __align__(16) uint8_t ring_raw[];
  V8* ring = reinterpret_cast<V8*>(ring_raw);  // [kRing][NV][T]
  float4* coef = reinterpret_cast<float4*>(ring_raw + sizeof(V8) * kRing * NV * T) + threadIdx.x;  // [NV - CR][4][T]
  __shared__ float2 red2[2][2][kWarps];  // [moments | centred sum of squares][iteration parity][warp]
  __shared__ uint32_t redm[2][kWarps];   // absmax, as bit patterns
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // this thread's columns: vector i covers elements [8 (tid + i T), +8) of the row
  const uint16_t* x_t = x + tid * 8;
  uint16_t* y_t = y != nullptr ? y + tid * 8 : nullptr;
  uint8_t* q_t = q != nullptr ? q + tid * 8 : nullptr;
  const float* w_t = w != nullptr ? w + tid * 8 : nullptr;
  const float* b_t = b != nullptr ? b + tid * 8 : nullptr;
  const float* sc_t = scale != nullptr ? scale + tid * 8 : nullptr;
  const float* sh_t = shift != nullptr ? shift + tid * 8 : nullptr;
  V8* ring_t = ring + tid;

  auto fetch_row = [&](int64_t row, int slot) {
    if (row < rows) {
#pragma unroll
      for (int i = 0; i < NV; ++i) cp_async16(ring_t + (slot * NV + i) * T, x_t + row * ldx + i * T * 8);
    }
    cp_async_commit();  // one group per row, empty past the end, so that the group count stays uniform
  };
  // CTA-wide sums of a pair of values; two result buffers, so one barrier is enough
  auto cta_sum2 = [&](float& a, float& c, int which, int it) {
    a = warp_sum(a);
    c = warp_sum(c);
    float2* r = red2[which][it & 1];
    if (lane == 0) r[warp] = make_float2(a, c);
    __syncthreads();
    a = r[0].x;
    c = r[0].y;
#pragma unroll
    for (int k = 1; k < kWarps; ++k) {
      a += r[k].x;
      c += r[k].y;
    }
  };

  const float inv_d = 1.f / static_cast<float>(D);
  // Per-column coefficients, folded into one multiplier and one addend per column:
  // (n w + b) (1 + scale) + shift = n [w (1 + scale)] + [b (1 + scale) + shift].  Those of the thread's first CR
  // vectors stay in registers for the whole kernel, the others in shared memory (read back once per row): reading
  // all of them through the L1 / shared-memory data path for every row would make that path the bound.
  uint64_t mulc[CR > 0 ? CR : 1][4], addc[CR > 0 ? CR : 1][4];
  const bool affine = w != nullptr || scale != nullptr;
  if (affine) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float m[8], a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = i * T * 8 + j;
        const float w0 = w != nullptr ? w_t[n] : 1.f, b0 = (w != nullptr && b != nullptr) ? b_t[n] : 0.f;
        const float m1 = scale != nullptr ? 1.f + sc_t[n] : 1.f, a1 = scale != nullptr ? sh_t[n] : 0.f;
        m[j] = w0 * m1;
        a[j] = fmaf(b0, m1, a1);
      }
      if (i < CR) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          mulc[i < CR ? i : 0][k] = f2_pack(m[2 * k], m[2 * k + 1]);
          addc[i < CR ? i : 0][k] = f2_pack(a[2 * k], a[2 * k + 1]);
        }
      } else {
        // the other vectors' coefficients: shared memory, in the order this thread reads them back (no barrier)
        coef[((i - CR) * 4 + 0) * T] = make_float4(m[0], m[1], m[2], m[3]);
        coef[((i - CR) * 4 + 1) * T] = make_float4(m[4], m[5], m[6], m[7]);
        coef[((i - CR) * 4 + 2) * T] = make_float4(a[0], a[1], a[2], a[3]);
        coef[((i - CR) * 4 + 3) * T] = make_float4(a[4], a[5], a[6], a[7]);
      }
    }
  }
  int64_t t = blockIdx.x;
  const int64_t step = gridDim.x;
#pragma unroll
  for (int k = 0; k < kRing - 1; ++k) fetch_row(t + k * step, k);
  for (int it = 0; t < rows; t += step, ++it) {
    fetch_row(t + (kRing - 1) * step, (it + kRing - 1) % kRing);
    cp_async_wait<kRing - 1>();  // this thread's pieces of row t have landed
    // both moments in one pass and one reduction
    uint64_t f[NV][4];
    uint64_t acc = f2_splat(0.f), acc_sq = f2_splat(0.f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const V8 raw = ring_t[((it % kRing) * NV + i) * T];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        f[i][k] = f2_from16<BF16>(raw.w[k]);
        acc = f2_add(acc, f[i][k]);
        acc_sq = f2_fma(f[i][k], f[i][k], acc_sq);
      }
    }
    float lo, hi, qlo, qhi;
    f2_unpack(acc, lo, hi);
    f2_unpack(acc_sq, qlo, qhi);
    float sum = lo + hi, sumsq = qlo + qhi;
    cta_sum2(sum, sumsq, 0, it);
    const float mean = div_rn_by(sum, static_cast<float>(D), inv_d);  // the correctly rounded quotient: a constant row gives itself
    float var = fmaf(-mean, mean, sumsq * inv_d);
    // E[x^2] - mean^2 loses digits when the mean dwarfs the spread: such a row (every thread sees the same two
    // numbers, so the branch is uniform) gets the centred sum of squares instead
    if (!(var * 64.f > mean * mean)) {
      const uint64_t neg_mean2 = f2_splat(-mean);
      uint64_t c2 = f2_splat(0.f);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t dlt = f2_add(f[i][k], neg_mean2);
          c2 = f2_fma(dlt, dlt, c2);
        }
      f2_unpack(c2, lo, hi);
      float centred = lo + hi, unused = 0.f;
      cta_sum2(centred, unused, 1, it);
      var = centred * inv_d;
    }
    const float rstd = rsqrtf(var + eps);
    const uint64_t rstd2 = f2_splat(rstd), shift2 = f2_splat(-mean * rstd);
    uint32_t amax2 = 0u;
    V8 out[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {  // four columns at a time
        uint64_t v0 = f2_fma(f[i][2 * h], rstd2, shift2), v1 = f2_fma(f[i][2 * h + 1], rstd2, shift2);
        if (i < CR) {
          if (affine) {
            v0 = f2_fma(v0, mulc[i < CR ? i : 0][2 * h], addc[i < CR ? i : 0][2 * h]);
            v1 = f2_fma(v1, mulc[i < CR ? i : 0][2 * h + 1], addc[i < CR ? i : 0][2 * h + 1]);
          }
        } else if (affine) {
          const float4 m = coef[((i - CR) * 4 + h) * T];
          const float4 a = coef[((i - CR) * 4 + 2 + h) * T];
          v0 = f2_fma(v0, f2_pack(m.x, m.y), f2_pack(a.x, a.y));
          v1 = f2_fma(v1, f2_pack(m.z, m.w), f2_pack(a.z, a.w));
        }
        // the tensor the reference materialises in the activation dtype
        out[i].w[2 * h] = f2_to16_rn<BF16>(v0);
        out[i].w[2 * h + 1] = f2_to16_rn<BF16>(v1);
        amax2 = absmax2_lazy<BF16>(absmax2_lazy<BF16>(amax2, out[i].w[2 * h]), out[i].w[2 * h + 1]);
      }
      if (y != nullptr) *reinterpret_cast<V8*>(y_t + t * ldy + i * T * 8) = out[i];
    }
    if constexpr (QDT >= 0) {
      // non-negative floats order like their bit patterns: the maximum is an integer reduction
      float alo, ahi;
      unpack2<BF16>(amax2 & 0x7fff7fffu, alo, ahi);
      const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(alo, ahi)));
      uint32_t* r = redm[it & 1];
      if (lane == 0) r[warp] = wmax;
      __syncthreads();
      uint32_t cmax = r[0];
#pragma unroll
      for (int k = 1; k < kWarps; ++k) cmax = max(cmax, r[k]);
      const float s = quant_scale<QDT>(__uint_as_float(cmax), [](float v) { return to_f<BF16>(from_f<BF16>(v)); });
      const float inv = quant_inv_scale(s);
      if (tid == 0) qscale[t] = s;
      const uint64_t neg_s2 = f2_splat(-s), inv2 = f2_splat(inv);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const uint32_t c0 = quant_four16<BF16, QDT>(out[i].w[0], out[i].w[1], neg_s2, inv2);
        const uint32_t c1 = quant_four16<BF16, QDT>(out[i].w[2], out[i].w[3], neg_s2, inv2);
        *reinterpret_cast<uint2*>(q_t + t * D + i * T * 8) = make_uint2(c0, c1);
      }
    }
  }
}

template <bool BF16, int QDT, int T, int NV, int MINB, int CR>
int launch_cta_rows(int64_t s, cudaStream_t st, const uint16_t* x, int64_t D, int64_t ldx, const float* w, const float* b,
                    const float* shift, const float* scale, float eps, uint16_t* y, int64_t ldy, uint8_t* q, float* qscale) {
  int per_sm = 0;
  constexpr size_t smem = static_cast<size_t>(kRing) * NV * T * sizeof(V8) + static_cast<size_t>(NV - CR) * 4 * T * sizeof(float4);
  if (smem > 40 * 1024)
    DAX_CUDA(cudaFuncSetAttribute(ln_rows_cta_kernel<BF16, QDT, T, NV, MINB, CR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
  DAX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ln_rows_cta_kernel<BF16, QDT, T, NV, MINB, CR>, T, smem));
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(s, static_cast<int64_t>(sm_count()) * std::max(per_sm, 1)));
  ln_rows_cta_kernel<BF16, QDT, T, NV, MINB, CR><<<grid, T, smem, st>>>(x, s, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
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
  // rows that fill a CTA exactly take the CTA-per-row kernel (5120 = 160 threads x 4 vectors x 8); per width: threads,
  // vectors per thread, CTAs per SM the register allocation is held to, vectors whose coefficients live in registers
#define DAX_LN_CTA(T, NV, MINB, CR) \
  if (D == 8 * (T) * (NV)) \
  return launch_cta_rows<BF16, QDT, T, NV, MINB, CR>(s, st, x, D, ldx, w, b, shift, scale, eps, y, ldy, q, qscale)
  DAX_LN_CTA(160, 4, 4, 1);   // 5120
  DAX_LN_CTA(128, 4, 4, 2);   // 4096
  DAX_LN_CTA(128, 3, 5, 2);   // 3072
  DAX_LN_CTA(128, 2, 6, 2);   // 2048
  DAX_LN_CTA(96, 2, 8, 2);    // 1536
  DAX_LN_CTA(128, 1, 8, 1);   // 1024
#undef DAX_LN_CTA
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
