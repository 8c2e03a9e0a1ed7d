// INT8 / FP8 GEMM with fused de-quantisation for the dynamic linears:
//     out[t, n] = cast( (acc[t, n] * sx[t]) * sw[n] ) + bias[n],   acc = qx . qw^T
//
// Tensor-core bound (2*M*N*K operations on the 8-bit tcgen05 pipe).  One persistent CTA per SM,
// warp-specialised:
//   warp 0      TMA producer: 128x128-byte tiles of qx and 256x128-byte tiles of qw into a 4-stage
//               shared-memory ring (128-byte swizzle, no multicast)
//   warp 1      MMA issuer: tcgen05.mma kind::i8 / kind::f8f6f4, 128x256 accumulator in tensor memory,
//               two accumulator buffers (2 x 256 columns) so the epilogue of tile i overlaps the
//               main loop of tile i+1
//   warps 2..9  epilogue (two warps per TMEM lane quarter, one per 128-column half of the tile):
//               tcgen05.ld 32 columns at a time, de-quantise with scales staged in shared memory, add
//               bias, round, optional per-row sum of squares per 128-column block, 16-byte stores
// Tiles are visited column-block-fastest so that the CTAs of one wave share the same rows of qx
// in L2 while the (much smaller) weight matrix stays L2-resident.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace dax {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BKB = 128;  // bytes (= elements) of K per stage: one 128-byte swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BKB;
constexpr int B_BYTES = BN * BKB;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 320;     // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int EPI_THREADS = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + 8 * 3 * 128 * 4 /*per-warp sw, bias, gate*/;

struct GemmParams {
  const float* sx;
  const float* sw;
  const void* bias;
  void* out;
  float* row_sumsq;
  void* acc_dump;
  int* status;
  int64_t M, N, K, ldo, out_col_group, out_group_stride;
  GroupTable groups;  // n > 0: slab g of the output sits at out + groups.off[g] (scattered, e.g. in peer memory)
  int m_tiles, n_tiles, k_blocks;
  int bias_dtype;
  // optional post-operations on the rounded linear output y (16-bit outputs only):
  //   act == 1: y = gelu_tanh(y);   resid != null: y = resid[t, n] + gate[n] * y   (fp32, then rounded)
  int act;
  const void* resid;
  int64_t ldr;
  const float* gate;
};

__device__ __forceinline__ float load_as_float(const void* p, int dt, int64_t i) {
  if (dt == DAX_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dt == DAX_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return static_cast<const float*>(p)[i];
}

// Round a pair to the output dtype; returns the packed 16-bit pair and leaves the rounded values in a, b.
template <int OUT>
__device__ __forceinline__ uint32_t round_pair(float& a, float& b) {
  if constexpr (OUT == DAX_BF16) {
    uint32_t pk;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk) : "f"(b), "f"(a));
    a = __uint_as_float(pk << 16);
    b = __uint_as_float(pk & 0xffff0000u);
    return pk;
  } else if constexpr (OUT == DAX_F16) {
    uint32_t pk;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(pk) : "f"(b), "f"(a));
    const __half2 h = *reinterpret_cast<__half2*>(&pk);
    a = __low2float(h);
    b = __high2float(h);
    return pk;
  } else {
    return 0;
  }
}

// GELU, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), hardware tanh approximation
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.f + t);
}

template <int KIND, int OUT, bool POST>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_dequant_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p, const uint32_t idesc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                  // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;        // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES; // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;     // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* scale_stage = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);  // [8 warps][sw 128 | bias 128 | gate 128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], EPI_THREADS / 32);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int m0 = (tile / p.n_tiles) * BM;
        const int n0 = (tile % p.n_tiles) * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, &full[s], kb * BKB, m0);
          tma_load_2d(b_dst, &map_b, &full[s], kb * BKB, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local_tile) {
        const uint32_t buf = local_tile & 1u;
        const uint32_t use = local_tile >> 1;  // how often this buffer has been used before
        if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = make_desc_k_sw128(a_addr);
          const uint64_t db = make_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k) {
            // advancing K by 32 bytes inside the 128-byte swizzle row = +2 in the encoded address
            umma_ss<KIND>(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // warp -> TMEM lane quarter (warp % 4, fixed by the hardware) and column half of the 256-wide tile
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local_tile) {
      const uint32_t buf = local_tile & 1u;
      const uint32_t use = local_tile >> 1;
      const int n_blk = tile % p.n_tiles;
      const int64_t m0 = static_cast<int64_t>(tile / p.n_tiles) * BM;
      const int64_t n0 = static_cast<int64_t>(n_blk) * BN;
      // stage the weight scales and bias (as fp32) of this warp's 128 columns in its own slice of
      // shared memory: no cross-warp synchronisation, so no warp can be left waiting at a barrier
      float* swp_w = scale_stage + (warp - 2) * 384;
      float* bp_w = swp_w + 128;
      float* gp_w = swp_w + 256;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int cl = lane + 32 * i;
        const int64_t col = n0 + half * (BN / 2) + cl;
        const bool col_ok = col < p.N;
        swp_w[cl] = col_ok ? __ldg(p.sw + col) : 0.f;
        bp_w[cl] = (col_ok && p.bias != nullptr) ? load_as_float(p.bias, p.bias_dtype, col) : 0.f;
        if constexpr (POST) gp_w[cl] = (col_ok && p.gate != nullptr) ? __ldg(p.gate + col) : 1.f;
      }
      __syncwarp();
      if (!mbar_wait(&acc_full[buf], use & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int64_t row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const float sx = row_ok ? p.sx[row] : 0.f;
      const bool has_bias = p.bias != nullptr;
      const bool want_ss = p.row_sumsq != nullptr;
      float sumsq = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        const int cl = half * (BN / 2) + c * 32;  // column inside the tile
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + cl, r);
        tmem_wait_ld();
        const int64_t col0 = n0 + cl;
        if (col0 >= p.N) continue;
        if (p.acc_dump != nullptr && row_ok) {
          uint32_t* dump = static_cast<uint32_t*>(p.acc_dump) + row * p.N + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) dump[j] = r[j];
        }
        const float* swp = swp_w + c * 32;
        const float* bp = bp_w + c * 32;
        uint32_t packed[16];
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float a0, a1;
          if constexpr (KIND == KIND_I8) {
            a0 = __int2float_rn(static_cast<int>(r[j]));
            a1 = __int2float_rn(static_cast<int>(r[j + 1]));
          } else {
            a0 = __uint_as_float(r[j]);
            a1 = __uint_as_float(r[j + 1]);
          }
          float t0 = __fmul_rn(__fmul_rn(a0, sx), swp[j]);
          float t1 = __fmul_rn(__fmul_rn(a1, sx), swp[j + 1]);
          if constexpr (KIND == KIND_I8) {
            // reference order: cast to the output dtype, then add the bias in the output dtype
            packed[j / 2] = round_pair<OUT>(t0, t1);
            if (has_bias) {
              t0 = __fadd_rn(t0, bp[j]);
              t1 = __fadd_rn(t1, bp[j + 1]);
              packed[j / 2] = round_pair<OUT>(t0, t1);
            }
          } else {
            // scaled-matmul semantics: the bias joins in fp32, one rounding
            t0 = __fadd_rn(t0, bp[j]);
            t1 = __fadd_rn(t1, bp[j + 1]);
            packed[j / 2] = round_pair<OUT>(t0, t1);
          }
          if (want_ss) sumsq = fmaf(t1, t1, fmaf(t0, t0, sumsq));
          if constexpr (POST) {
            if (p.act == 1) {
              t0 = gelu_tanh(t0);
              t1 = gelu_tanh(t1);
              packed[j / 2] = round_pair<OUT>(t0, t1);
            }
            if (p.resid != nullptr && row_ok && col0 + j < p.N) {
              const uint32_t rr = *reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(p.resid) + row * p.ldr + col0 + j);
              float r0, r1;
              if constexpr (OUT == DAX_BF16) {
                r0 = __uint_as_float(rr << 16);
                r1 = __uint_as_float(rr & 0xffff0000u);
              } else {
                const __half2 h = *reinterpret_cast<const __half2*>(&rr);
                r0 = __low2float(h);
                r1 = __high2float(h);
              }
              t0 = fmaf(gp_w[c * 32 + j], t0, r0);
              t1 = fmaf(gp_w[c * 32 + j + 1], t1, r1);
              packed[j / 2] = round_pair<OUT>(t0, t1);
            }
          }
          if constexpr (OUT == DAX_F32) { v[j] = t0; v[j + 1] = t1; }
        }
        if (row_ok) {
          const int64_t g = col0 / p.out_col_group;
          const int64_t off = (p.groups.n > 0 ? p.groups.off[g < kMaxGroups ? g : 0] : g * p.out_group_stride) + row * p.ldo +
                              (col0 - g * p.out_col_group);
          if constexpr (OUT == DAX_F32) {
            float* o = static_cast<float*>(p.out) + off;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (col0 + j < p.N) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            uint16_t* o = static_cast<uint16_t*>(p.out) + off;
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              if (col0 + j < p.N)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(packed[j / 2], packed[j / 2 + 1], packed[j / 2 + 2], packed[j / 2 + 3]);
          }
        }
      }
      // all TMEM reads of this buffer are complete (wait::ld above): hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (want_ss && row_ok) p.row_sumsq[row * (2 * p.n_tiles) + 2 * n_blk + half] = sumsq;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, DAX_ERR_TIMEOUT);
}

template <int KIND, int OUT, bool POST>
int launch_gemm_post(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, uint32_t idesc, int grid,
                     cudaStream_t st) {
  DAX_CUDA(cudaFuncSetAttribute(gemm_dequant_kernel<KIND, OUT, POST>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  gemm_dequant_kernel<KIND, OUT, POST><<<grid, GEMM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, p, idesc);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

template <int KIND, int OUT>
int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, uint32_t idesc, int grid,
                cudaStream_t st) {
  if constexpr (OUT != DAX_F32) {
    if (p.act != 0 || p.resid != nullptr) return launch_gemm_post<KIND, OUT, true>(map_a, map_b, p, idesc, grid, st);
  }
  return launch_gemm_post<KIND, OUT, false>(map_a, map_b, p, idesc, grid, st);
}

template <int KIND>
int launch_gemm_out(int out_dtype, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p,
                    uint32_t idesc, int grid, cudaStream_t st) {
  if (out_dtype == DAX_BF16) return launch_gemm<KIND, DAX_BF16>(map_a, map_b, p, idesc, grid, st);
  if (out_dtype == DAX_F16) return launch_gemm<KIND, DAX_F16>(map_a, map_b, p, idesc, grid, st);
  return launch_gemm<KIND, DAX_F32>(map_a, map_b, p, idesc, grid, st);
}

bool is_f8(int dt) { return dt == DAX_E4M3 || dt == DAX_E5M2; }

}  // namespace
}  // namespace dax

extern "C" int dax_gemm_dequant(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype,
                                const float* sw, const void* bias, int bias_dtype, void* out, int out_dtype,
                                int64_t M, int64_t N, int64_t K, int64_t ldo, int64_t out_col_group,
                                int64_t out_group_stride, float* row_sumsq, void* acc_dump, void* stream) {
  return dax_gemm_dequant_ex(qx, a_dtype, sx, qw, b_dtype, sw, bias, bias_dtype, out, out_dtype, M, N, K, ldo,
                             out_col_group, out_group_stride, row_sumsq, acc_dump, 0, nullptr, 0, nullptr, stream);
}

namespace dax {
namespace {
int gemm_entry(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype, const float* sw,
               const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldo,
               int64_t out_col_group, int64_t out_group_stride, const GroupTable& groups, float* row_sumsq,
               void* acc_dump, int act, const void* resid, int64_t ldr, const float* gate, void* stream) {
  DAX_REQUIRE(act == 0 || act == 1, DAX_ERR_UNSUPPORTED, "gemm_dequant: unknown activation %d", act);
  DAX_REQUIRE((act == 0 && resid == nullptr) || out_dtype != DAX_F32, DAX_ERR_UNSUPPORTED,
              "gemm_dequant: activation / residual epilogues need a 16-bit output dtype");
  DAX_REQUIRE(resid == nullptr || (ldr % 2 == 0 && (reinterpret_cast<uintptr_t>(resid) & 3u) == 0), DAX_ERR_ALIGN,
              "gemm_dequant: resid must be 4-byte aligned with an even leading dimension");
  DAX_REQUIRE(gate == nullptr || resid != nullptr, DAX_ERR_INVALID, "gemm_dequant: gate needs resid");
  DAX_REQUIRE(M >= 0 && N > 0 && K > 0, DAX_ERR_INVALID, "gemm_dequant: bad shape M=%lld N=%lld K=%lld",
              (long long)M, (long long)N, (long long)K);
  if (M == 0) return DAX_OK;
  DAX_REQUIRE(qx && sx && qw && sw && out, DAX_ERR_INVALID, "gemm_dequant: null pointer");
  const bool i8 = a_dtype == DAX_I8 && b_dtype == DAX_I8;
  const bool f8 = is_f8(a_dtype) && is_f8(b_dtype);
  DAX_REQUIRE(i8 || f8, DAX_ERR_UNSUPPORTED, "gemm_dequant: operand dtypes (%d, %d) must be both I8 or both FP8",
              a_dtype, b_dtype);
  DAX_REQUIRE(out_dtype == DAX_BF16 || out_dtype == DAX_F16 || out_dtype == DAX_F32, DAX_ERR_UNSUPPORTED,
              "gemm_dequant: out_dtype %d is not BF16/F16/F32", out_dtype);
  DAX_REQUIRE(bias == nullptr || bias_dtype == DAX_BF16 || bias_dtype == DAX_F16 || bias_dtype == DAX_F32,
              DAX_ERR_UNSUPPORTED, "gemm_dequant: bias_dtype %d is not BF16/F16/F32", bias_dtype);
  DAX_REQUIRE(K % 16 == 0, DAX_ERR_ALIGN, "gemm_dequant: K=%lld must be a multiple of 16", (long long)K);
  DAX_REQUIRE(N % 8 == 0, DAX_ERR_ALIGN, "gemm_dequant: N=%lld must be a multiple of 8", (long long)N);
  DAX_REQUIRE(out_col_group > 0 && N % out_col_group == 0 && (out_col_group == N || out_col_group % 32 == 0),
              DAX_ERR_ALIGN, "gemm_dequant: out_col_group=%lld must divide N and be a multiple of 32",
              (long long)out_col_group);
  DAX_REQUIRE(ldo % 8 == 0 && out_group_stride % 8 == 0, DAX_ERR_ALIGN,
              "gemm_dequant: ldo and out_group_stride must be multiples of 8 elements");
  DAX_REQUIRE(aligned16(qx) && aligned16(qw) && aligned16(out), DAX_ERR_ALIGN,
              "gemm_dequant: qx, qw and out must be 16-byte aligned");
  DAX_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), DAX_ERR_UNSUPPORTED, "gemm_dequant: size overflow");
  DAX_REQUIRE(groups.n == 0 || groups.n == N / out_col_group, DAX_ERR_INVALID,
              "gemm_dequant: %d group pointers for %lld column groups", groups.n, (long long)(N / out_col_group));

  CUtensorMap map_a, map_b;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t strides[2] = {1, static_cast<uint64_t>(K)};
    uint32_t box[2] = {BKB, BM};
    int rc = make_tma_map(&map_a, qx, 1, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t strides[2] = {1, static_cast<uint64_t>(K)};
    uint32_t box[2] = {BKB, BN};
    int rc = make_tma_map(&map_b, qw, 1, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }

  GemmParams p;
  p.sx = sx; p.sw = sw; p.bias = bias; p.out = out; p.row_sumsq = row_sumsq; p.acc_dump = acc_dump;
  p.status = device_status_ptr();
  DAX_REQUIRE(p.status != nullptr, DAX_ERR_CUDA, "gemm_dequant: cannot resolve the device status word");
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.out_col_group = out_col_group; p.out_group_stride = out_group_stride;
  p.groups = groups;
  p.m_tiles = static_cast<int>((M + BM - 1) / BM);
  p.n_tiles = static_cast<int>((N + BN - 1) / BN);
  p.k_blocks = static_cast<int>((K + BKB - 1) / BKB);
  p.bias_dtype = bias_dtype;
  p.act = act; p.resid = resid; p.ldr = ldr; p.gate = gate;
  const int64_t total = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  DAX_REQUIRE(total < (1ll << 31), DAX_ERR_UNSUPPORTED, "gemm_dequant: too many tiles");
  const int grid = static_cast<int>(total < sm_count() ? total : sm_count());
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (i8) {
    const uint32_t idesc = make_idesc(/*c=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, BM, BN);
    return launch_gemm_out<KIND_I8>(out_dtype, map_a, map_b, p, idesc, grid, st);
  }
  const uint32_t idesc = make_idesc(/*c=f32*/ 1, a_dtype == DAX_E5M2 ? 1 : 0, b_dtype == DAX_E5M2 ? 1 : 0, BM, BN);
  return launch_gemm_out<KIND_F8>(out_dtype, map_a, map_b, p, idesc, grid, st);
}
}  // namespace
}  // namespace dax

extern "C" int dax_gemm_dequant_ex(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype,
                                   const float* sw, const void* bias, int bias_dtype, void* out, int out_dtype,
                                   int64_t M, int64_t N, int64_t K, int64_t ldo, int64_t out_col_group,
                                   int64_t out_group_stride, float* row_sumsq, void* acc_dump, int act,
                                   const void* resid, int64_t ldr, const float* gate, void* stream) {
  dax::GroupTable none{};
  return dax::gemm_entry(qx, a_dtype, sx, qw, b_dtype, sw, bias, bias_dtype, out, out_dtype, M, N, K, ldo, out_col_group,
                         out_group_stride, none, row_sumsq, acc_dump, act, resid, ldr, gate, stream);
}

extern "C" int dax_gemm_dequant_scatter(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype,
                                        const float* sw, const void* bias, int bias_dtype, void* const* group_out,
                                        int64_t n_groups, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldo,
                                        int64_t out_col_group, void* stream) {
  dax::GroupTable tab{};
  void* base = nullptr;
  const int eb = dax::dtype_bytes(out_dtype);
  if (eb != 2 && eb != 4) return dax::fail(DAX_ERR_UNSUPPORTED, "gemm_dequant_scatter: out_dtype %d is not BF16/F16/F32", out_dtype);
  int rc = dax::make_group_table(group_out, n_groups, eb, &tab, &base);
  if (rc != DAX_OK) return rc;
  return dax::gemm_entry(qx, a_dtype, sx, qw, b_dtype, sw, bias, bias_dtype, base, out_dtype, M, N, K, ldo, out_col_group, 0,
                         tab, nullptr, nullptr, 0, nullptr, 0, nullptr, stream);
}
