// Non-causal flash attention for head_dim 128 with 16-bit operands (bf16 Q.K^T, bf16 P.V) in which the
// probabilities never touch shared memory: the softmax warps write P back into TENSOR MEMORY, over the
// score tile they have just read, and P.V is issued with its A operand in tensor memory.
//
// A CTA owns 256 query rows of one (batch, head) as two 128-row tiles X = 0, 1 and runs 12 warps:
//   warps 0..3    softmax of tile 0: one thread = one query row x all 128 key columns of the tile (row maximum and
//                 row sum stay inside the thread: no shuffle, no shared-memory exchange)
//   warps 4..7    the same for tile 1
//   warp  8       TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... through a ring of five 32 KB slots
//   warp  9, 10   MMA issuers: warp 9 every Q.K^T, warp 10 every P.V (the warp runs the loop, one elected lane issues)
//   warp  11      owns the tensor-memory allocation
// The softmax warps raise their register budget with setmaxnreg (a row of 128 fp32 scores lives in registers), the
// other four warps lower theirs.
//
// Tensor memory (512 columns): S [0,128) (ONE score buffer, used by the two tiles in turn)  P_0 [128,192)
// P_1 [192,256) (bf16, 64 columns each)  O_0 [256,384)  O_1 [384,512).  Per KV tile j and query tile X:
//     S = Q_X.K_j^T  ->  the softmax warps of X copy S into registers and release it at once (s_free), so the other
//                        tile's Q.K^T follows immediately;  row maximum, exponentials, P_X(j) -> tensor memory
//                    ->  O_X += P_X(j).V_j   (pv_done)
// The score buffer is busy only from the issue of a Q.K^T to the moment its 128 columns are in registers (about 800
// clocks), twice per period, so sharing it costs nothing, and because P has columns of its own no product ever waits
// for the softmax of its own tile: the exponential unit and the tensor pipe both run continuously.
// Shared memory holds only Q (64 KB) and the K/V ring (160 KB).
//
// Operands come from the workspace written by the prepare step (attn_prep.cu) exactly as for the kernels in attn.cu.
#include <climits>

#include "attn_common.cuh"
#include "sm100_ptx.cuh"

namespace dax {
namespace {

constexpr int BOX_BYTES = 128 * 128;     // one [128 rows x 128 B] box
constexpr int TILE_BYTES = 2 * BOX_BYTES;  // a [128 x 128] tile of 16-bit elements: two boxes of 64 columns
constexpr int NSLOT = 5;                 // K/V ring
constexpr int THREADS = 384;
constexpr int PRODUCER_WARP = 8, ISSUER_WARP0 = 9, TMEM_WARP = 11;
constexpr float TAU = 8.f;               // lazy rescale: P <= 2^8, far inside the bf16 range

constexpr int OFF_Q = 0;
constexpr int OFF_RING = OFF_Q + 2 * TILE_BYTES;
constexpr int OFF_BAR = OFF_RING + NSLOT * TILE_BYTES;
constexpr int SMEM_TOTAL = OFF_BAR + 256 + 1024 /*alignment slack*/;

__device__ __forceinline__ void reg_alloc_216() { asm volatile("setmaxnreg.inc.sync.aligned.u32 216;"); }
__device__ __forceinline__ void reg_dealloc_72() { asm volatile("setmaxnreg.dec.sync.aligned.u32 72;"); }

// D[tmem] (+)= A[tmem] * B[smem]^T, kind::f16, issued by ONE thread.  A: 128 lanes x (K/2) columns, two 16-bit
// elements of consecutive K per 32-bit cell.
__device__ __forceinline__ void umma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two fp32 values -> bf16x2 by keeping the upper halves (one byte-permute for two elements; the rounding
// conversions run on the unit the exponentials already saturate).  Truncation lowers every P by 2^-9 on average;
// the epilogue multiplies O by (1 + 2^-9) to centre it.
__device__ __forceinline__ uint32_t pack_bf16x2_trunc(float a, float b) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(r) : "r"(__float_as_uint(a)), "r"(__float_as_uint(b)));
  return r;
}

// DIRECT: Q, K and V are read in place from [BH, S, 128] tensors (3-D TMA maps, rows past the end read as zero);
// V is then a [keys x channels] tile, i.e. the B operand of P.V with N (channels) contiguous: MN-major descriptor.
template <bool DIRECT>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_tmem_p_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* q_full = bars;                  // [1]
  uint64_t* kv_full = bars + 1;             // [NSLOT]
  uint64_t* kv_empty = kv_full + NSLOT;     // [NSLOT] released by two MMA commits (one per query tile)
  uint64_t* s_full = kv_empty + NSLOT;      // [2]  MMA -> softmax of X: S holds Q_X.K_j^T
  uint64_t* s_free = s_full + 2;            // [1]  softmax -> MMA: S is in registers (uses alternate: tile 0, tile 1, ...)
  uint64_t* p_full = s_free + 1;            // [2]  softmax -> MMA: P_X(j) is in tensor memory, O_X rescaled
  uint64_t* pv_done = p_full + 2;           // [2]  MMA -> softmax: P_X(j).V_j complete, P_X and O_X are at rest
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int range = blockIdx.x / p.tiles_per_range;
  const int q0 = p.q_begin + range * p.range_stride + (blockIdx.x % p.tiles_per_range) * 256;
  const int q_stop = min(p.q_end + range * p.range_stride, p.Sq);
  const int n_kv = p.Sk_pad / 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 2);
    }
    mbar_init(s_free, 4);          // one arrival per softmax warp of the tile that read S
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp of the tile
      mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == TMEM_WARP) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= PRODUCER_WARP) {
    reg_dealloc_72();
    if (warp == PRODUCER_WARP) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
        const int q_row = bh * p.Sq_pad + q0;
        for (int x = 0; x < 2; ++x)
          for (int sub = 0; sub < 2; ++sub) {
            uint8_t* dst = smem + OFF_Q + x * TILE_BYTES + sub * BOX_BYTES;
            if constexpr (DIRECT) tma_load_3d(dst, &map_q, q_full, sub * 64, q0 + x * 128, bh);
            else tma_load_2d(dst, &map_q, q_full, sub * 64, q_row + x * 128);
          }
        for (int seq = 0; seq < 2 * n_kv; ++seq) {
          const int j = seq >> 1;
          const uint32_t s = seq % NSLOT, ph = (seq / NSLOT) & 1u;
          if (!mbar_wait(&kv_empty[s], ph ^ 1u, abort_flag)) break;
          mbar_arrive_expect_tx(&kv_full[s], TILE_BYTES);
          uint8_t* dst = smem + OFF_RING + s * TILE_BYTES;
          if constexpr (DIRECT) {  // K_j, V_j : [128 tokens x 128 channels], two boxes of 64 channels
            for (int sub = 0; sub < 2; ++sub)
              tma_load_3d(dst + sub * BOX_BYTES, (seq & 1) == 0 ? &map_k : &map_v, &kv_full[s], sub * 64, j * 128, bh);
          } else if ((seq & 1) == 0) {  // K_j : [128 tokens x 128 channels]
            for (int sub = 0; sub < 2; ++sub)
              tma_load_2d(dst + sub * BOX_BYTES, &map_k, &kv_full[s], sub * 64, bh * p.Sk_pad + j * 128);
          } else {               // V_j^T : [128 channels x 128 tokens]
            for (int sub = 0; sub < 2; ++sub)
              tma_load_2d(dst + sub * BOX_BYTES, &map_v, &kv_full[s], j * 128 + sub * 64, bh * 128);
          }
        }
      }
    } else if (warp < TMEM_WARP) {
      // ---------------------------------------------------------------- MMA issuers
      // The whole warp runs the loops (uniform control flow, every lane polls the barriers); one elected lane
      // issues the tensor-core instructions and the commits.
      {
        const bool leader = elect_one();
        // f32 accumulators, M = N = 128.  Q.K^T multiplies the input format by itself; P is always bf16; in direct mode
        // the B operand of P.V (V as stored: channels contiguous) is MN-major (bit 16)
        const uint32_t fmt = DIRECT ? static_cast<uint32_t>(p.in_fmt) : 1u;
        const uint32_t idesc_qk = make_idesc(1, fmt, fmt, 128, 128);
        const uint32_t idesc_pv = make_idesc(1, 1, fmt, 128, 128) | (DIRECT ? (1u << 16) : 0u);
        const uint32_t q_base = smem_u32(smem + OFF_Q);
        const uint32_t ring = smem_u32(smem + OFF_RING);
        const uint32_t s_tm = tmem_base;
        // S = Q_x . K_j^T : 8 steps of 16 channels; box `sub` holds channels [64 sub, 64 sub + 64).  Use number
        // u = 2 j + x of the shared score buffer: it must have been read by the previous user.
        auto issue_qk = [&](int x, int j) -> bool {
          const uint32_t seq = 2 * j, slot = seq % NSLOT, ph = (seq / NSLOT) & 1u;
          const int u = 2 * j + x;
          if (!mbar_wait(&kv_full[slot], ph, abort_flag)) return false;
          if (u > 0 && !mbar_wait(s_free, (u - 1) & 1u, abort_flag)) return false;
          tc_fence_after_sync();
          const uint64_t q_desc = make_desc_k_sw128(q_base + x * TILE_BYTES);
          const uint64_t k_desc = make_desc_k_sw128(ring + slot * TILE_BYTES);
          if (leader) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint64_t adv = static_cast<uint64_t>((i >> 2) * (BOX_BYTES >> 4) + 2 * (i & 3));
              umma_ss<KIND_F16>(s_tm, q_desc + adv, k_desc + adv, idesc_qk, i != 0 ? 1u : 0u);
            }
            umma_commit(&s_full[x]);
            umma_commit(&kv_empty[slot]);
          }
          __syncwarp();
          return true;
        };
        // O_x += P_x(j) . V_j : 8 steps of 16 keys; A from tensor memory (8 columns per step), box `sub` of V^T
        // holds keys [64 sub, 64 sub + 64)
        auto issue_pv = [&](int x, int j) -> bool {
          const uint32_t seq = 2 * j + 1, slot = seq % NSLOT, ph = (seq / NSLOT) & 1u;
          if (!mbar_wait(&kv_full[slot], ph, abort_flag)) return false;
          if (!mbar_wait(&p_full[x], j & 1u, abort_flag)) return false;
          tc_fence_after_sync();
          const uint64_t v_desc = DIRECT ? make_desc_mn_sw128(ring + slot * TILE_BYTES, BOX_BYTES)
                                         : make_desc_k_sw128(ring + slot * TILE_BYTES);
          const uint32_t p_tm = tmem_base + 128 + x * 64;
          const uint32_t o_tm = tmem_base + 256 + x * 128;
          if (leader) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              // 16 keys further: K-major V^T = 32 bytes along the row (second box after 64 keys); MN-major V = 16 rows
              const uint64_t adv = DIRECT ? static_cast<uint64_t>(i * ((16 * 128) >> 4))
                                          : static_cast<uint64_t>((i >> 2) * (BOX_BYTES >> 4) + 2 * (i & 3));
              umma_ts_f16(o_tm, p_tm + 8 * i, v_desc + adv, idesc_pv, (j > 0 || i != 0) ? 1u : 0u);
            }
            umma_commit(&pv_done[x]);
            umma_commit(&kv_empty[slot]);
          }
          __syncwarp();
          return true;
        };
        // warp 9 issues every Q.K^T (tile 0, tile 1, tile 0, ... through the shared score buffer), warp 10 every P.V
        if (warp == ISSUER_WARP0) {
          bool ok = mbar_wait(q_full, 0, abort_flag);
          for (int j = 0; ok && j < n_kv; ++j) ok = issue_qk(0, j) && issue_qk(1, j);
        } else {
          bool ok = true;
          for (int j = 0; ok && j < n_kv; ++j) ok = issue_pv(0, j) && issue_pv(1, j);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    reg_alloc_216();
    const int x = warp >> 2;            // query tile
    const int quarter = warp & 3;       // TMEM lanes [32*quarter, +32)
    const int r = quarter * 32 + lane;  // row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base;
    const uint32_t p_tmem = tmem_base + lane_base + 128 + x * 64;
    const uint32_t o_tmem = tmem_base + lane_base + 256 + x * 128;
    const int q_row = q0 + x * 128 + r;
    // 16-bit scores are unscaled: the per-row factor (softmax scale * log2 e) multiplies them here
    const float cmul = DIRECT ? p.direct_cmul
                              : (q_row < p.Sq ? p.q_scale[static_cast<int64_t>(bh) * p.Sq_pad + q_row] : 1.f);
    float m = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&s_full[x], j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t sv[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&sv[32 * c]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);  // S is in registers: the other tile's Q.K^T may overwrite it
      const int valid = p.Sk - j * 128;  // columns >= valid are padding (only in the last tile)
      if (valid < 128) {
#pragma unroll
        for (int i = 0; i < 128; ++i) sv[i] = i < valid ? sv[i] : 0xFF800000u;  // -inf: never the maximum, exp = 0
      }
      float fmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 128; i += 2)
        fmx[(i >> 1) & 3] = fmax3(fmx[(i >> 1) & 3], __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
      const float mx = fmaxf(fmax3(fmx[0], fmx[1], fmx[2]), fmx[3]) * cmul;  // cmul > 0
      const float m_new = (mx > m + TAU) ? mx : m;
      const float alpha = ex2(m - m_new);  // m = -inf on the first tile -> 0
      const float off = -m_new;

      // P_X and O_X are at rest once P_X(j-1).V_{j-1} has completed (normally long ago)
      if (j > 0) {
        if (!mbar_wait(&pv_done[x], (j - 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
      }
      // correction: O_X *= alpha when a row of this warp moved its maximum
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tmem_ld32(o_tmem + 32 * c, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st32(o_tmem + 32 * c, ov);
        }
      }

      // p_i = 2^(s_i * cmul - m_new), packed to bf16 pairs, to tensor memory
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int hseg = 0; hseg < 2; ++hseg) {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int i = 64 * hseg + 2 * c;
          const float e0 = ex2(fmaf(__uint_as_float(sv[i]), cmul, off));
          const float e1 = ex2(fmaf(__uint_as_float(sv[i + 1]), cmul, off));
          sum[c & 3] += e0;
          sum[(c + 2) & 3] += e1;
          pk[c] = pack_bf16x2_trunc(e0, e1);
        }
        tmem_st32(p_tmem + 32 * hseg, pk);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
      l = fmaf(l, alpha, (sum[0] + sum[1]) + (sum[2] + sum[3]));
      m = m_new;
    }

    if (ok && mbar_wait(&pv_done[x], (n_kv - 1) & 1u, abort_flag)) {
      tc_fence_after_sync();
      const float inv_l = 1.001953125f / l;  // bf16 P was truncated, not rounded: centre the result
      const bool store = q_row < q_stop;
      const int b = bh / p.heads, h = bh % p.heads;
      uint16_t* orow = static_cast<uint16_t*>(p.o) + attn_out_offset(p, b, h, q_row);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t ov[32];
        tmem_ld32(o_tmem + c * 32, ov);
        tmem_wait_ld();
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float a = __uint_as_float(ov[i + 2 * q]) * inv_l;
              const float bb = __uint_as_float(ov[i + 2 * q + 1]) * inv_l;
              if (p.out_bf16) {
                w[q] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(a))) |
                       (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(bb))) << 16);
              } else {
                w[q] = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(a))) |
                       (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(bb))) << 16);
              }
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == TMEM_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, DAX_ERR_TIMEOUT);
}

}  // namespace

int launch_attn_fwd_tmem_p(const AttnWorkspace& ws, const AttnParams& p, int64_t BH, cudaStream_t st) {
  CUtensorMap map_q, map_k, map_v;
  {
    uint64_t dims[2] = {128, static_cast<uint64_t>(BH) * ws.Sq_pad};
    uint64_t strides[2] = {2, 256};
    uint32_t box[2] = {64, 128};
    int rc = make_tma_map(&map_q, ws.q, 2, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  {
    uint64_t dims[2] = {128, static_cast<uint64_t>(BH) * ws.Sk_pad};
    uint64_t strides[2] = {2, 256};
    uint32_t box[2] = {64, 128};
    int rc = make_tma_map(&map_k, ws.k, 2, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(ws.Sk_pad), static_cast<uint64_t>(BH) * 128};
    uint64_t strides[2] = {2, static_cast<uint64_t>(ws.Sk_pad) * 2};
    uint32_t box[2] = {64, 128};
    int rc = make_tma_map(&map_v, ws.vt, 2, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  dim3 grid(static_cast<unsigned>(p.n_ranges * p.tiles_per_range), static_cast<unsigned>(BH));
  DAX_CUDA(cudaFuncSetAttribute(attn_fwd_tmem_p_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
  attn_fwd_tmem_p_kernel<false><<<grid, THREADS, SMEM_TOTAL, st>>>(map_q, map_k, map_v, p);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

int launch_attn_fwd_tmem_p_direct(const void* q, const void* k, const void* v, int64_t q_sh, int64_t q_st, int64_t k_sh,
                                  int64_t k_st, int64_t v_sh, int64_t v_st, const AttnParams& p, int64_t BH, cudaStream_t st) {
  CUtensorMap maps[3];
  const void* base[3] = {q, k, v};
  const int64_t sh[3] = {q_sh, k_sh, v_sh}, stt[3] = {q_st, k_st, v_st};
  const int64_t rows[3] = {p.Sq, p.Sk, p.Sk};
  for (int i = 0; i < 3; ++i) {
    uint64_t dims[3] = {128, static_cast<uint64_t>(rows[i]), static_cast<uint64_t>(BH)};
    uint64_t strides[3] = {2, static_cast<uint64_t>(stt[i]) * 2, static_cast<uint64_t>(sh[i]) * 2};
    uint32_t box[3] = {64, 128, 1};
    int rc = make_tma_map(&maps[i], base[i], 2, 3, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  dim3 grid(static_cast<unsigned>(p.n_ranges * p.tiles_per_range), static_cast<unsigned>(BH));
  DAX_CUDA(cudaFuncSetAttribute(attn_fwd_tmem_p_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
  attn_fwd_tmem_p_kernel<true><<<grid, THREADS, SMEM_TOTAL, st>>>(maps[0], maps[1], maps[2], p);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

}  // namespace dax

