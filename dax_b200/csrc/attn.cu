// Quantised non-causal flash attention for head_dim 128 on tcgen05 / TMEM / TMA.
//
// Two precisions of the two contractions (template parameters, chosen per call):
//   INT8 Q.K^T (kind::i8, int32 accumulators)  + FP8 e4m3 P.V (kind::f8f6f4, fp32 accumulators)
//   fp16 Q.K^T (kind::f16, fp32 accumulators)  + fp16 P.V
// A CTA owns 256 query rows of one (batch, head): two 128-row tiles X = 0, 1 that ping-pong so
// that the tensor pipe works on one tile while the softmax warps work on the other.
//
//   warps 0..3   softmax + correction + epilogue of tile 0 (thread = one query row)
//   warps 4..7   the same for tile 1
//   warp  8      TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... through a ring
//   warp  9      MMA issuer (one thread)
//
// Tensor memory (512 columns): S_0 [0,128)  S_1 [128,256)  O_0 [256,384)  O_1 [384,512).
// Per KV tile j and query tile X:   S_X = Q_X . K_j^T   ->  softmax warps read S_X, keep the running
// row maximum m and sum l (base-2 domain), write P_X to shared memory in the K-major 128-byte
// swizzled layout the MMA reads, rescale O_X in tensor memory when m moved  ->  O_X += P_X . V_j.
// A tcgen05.commit completes only after every earlier MMA of the issuing thread, so the arrival of
// S_X(j+1) also tells the softmax warps that P_X . V_j is done: P_X may be overwritten and O_X rescaled.
//
// Operands come from the workspace written by the prepare step (attn_prep.cu): every tile is a set
// of [128 rows x 128 bytes] boxes, so one shared-memory descriptor form serves Q, K, P and V^T.
#include <climits>

#include "attn_common.cuh"
#include "sm100_ptx.cuh"

namespace dax {
namespace {

constexpr int ATT_THREADS = 320;
constexpr int BOX_BYTES = 128 * 128;  // one [128 x 128 B] box

template <int MODE> struct AttnCfg;
template <> struct AttnCfg<DAX_ATTN_QK_I8_PV_F8> {
  static constexpr int QK_KIND = KIND_I8, PV_KIND = KIND_F8;
  static constexpr int EQ = 1, EP = 1;       // bytes per element of Q/K and of P/V
  static constexpr int NSLOT = 8;
  static constexpr float TAU = 0.f;          // P is scaled to the e4m3 range: the row max must be exact
  static constexpr float PBIAS = 8.8073549f; // log2(448): P in (0, 448]
};
template <> struct AttnCfg<DAX_ATTN_QK_F16_PV_F16> {
  static constexpr int QK_KIND = KIND_F16, PV_KIND = KIND_F16;
  static constexpr int EQ = 2, EP = 2;
  static constexpr int NSLOT = 3;
  static constexpr float TAU = 8.f;          // lazy rescale: P <= 2^8 fits fp16 easily
  static constexpr float PBIAS = 0.f;
};

template <int MODE>
struct Smem {
  using C = AttnCfg<MODE>;
  static constexpr int Q_TILE = BOX_BYTES * C::EQ;
  static constexpr int P_TILE = BOX_BYTES * C::EP;
  static constexpr int SLOT = BOX_BYTES * (C::EQ > C::EP ? C::EQ : C::EP);
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_P = OFF_Q + 2 * Q_TILE;
  static constexpr int OFF_RING = OFF_P + 2 * P_TILE;
  static constexpr int OFF_BAR = OFF_RING + C::NSLOT * SLOT;
  static constexpr int OFF_VSCALE = OFF_BAR + 256;
  static constexpr int TOTAL = OFF_VSCALE + 512 + 1024 /*alignment slack*/;
};

struct AttnParams {
  const float* q_scale;  // [BH, Sq_pad]
  const float* k_scale;  // [BH, Sk_pad/128]
  const float* v_scale;  // [BH, 128]
  void* o;
  int* status;
  int64_t o_sb, o_sh, o_st;  // element strides of o: batch, head, token
  int heads;
  int Sq, Sk, Sq_pad, Sk_pad;
  int q_begin, q_end;      // first query range
  int n_ranges, range_stride, tiles_per_range;
  int out_bf16;
};

// K-major descriptor pair advance: `sub` selects the 16 KB box, `k` the 32-byte step inside it.
__device__ __forceinline__ uint64_t desc_at(uint32_t tile_addr, int sub, int k) {
  return make_desc_k_sw128(tile_addr + sub * BOX_BYTES) + 2 * k;
}

template <int KIND, int E>
__device__ __forceinline__ void mma_tile(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                         bool accumulate) {
#pragma unroll
  for (int sub = 0; sub < E; ++sub) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      umma_ss<KIND>(d_tmem, desc_at(a_addr, sub, k), desc_at(b_addr, sub, k), idesc,
                    (accumulate || sub != 0 || k != 0) ? 1u : 0u);
    }
  }
}

__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Row maximum of the scaled scores.  The scale is positive, so for integer accumulators the maximum
// is taken on the integers and scaled once.
template <int MODE, bool FULL>
__device__ __forceinline__ float row_max(const uint32_t (&sv)[128], float cmul, int valid) {
  using C = AttnCfg<MODE>;
  if constexpr (C::QK_KIND == KIND_I8) {
    int imax[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
#pragma unroll
    for (int i = 0; i < 128; ++i)
      if (FULL || i < valid) imax[i & 3] = max(imax[i & 3], static_cast<int>(sv[i]));
    return static_cast<float>(max(max(imax[0], imax[1]), max(imax[2], imax[3]))) * cmul;
  } else {
    float fmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 128; ++i)
      if (FULL || i < valid) fmx[i & 3] = fmaxf(fmx[i & 3], __uint_as_float(sv[i]));
    return fmaxf(fmaxf(fmx[0], fmx[1]), fmaxf(fmx[2], fmx[3])) * cmul;
  }
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// p_i = 2^(s_i * cmul + off) for the row held in sv; converts to the P format, writes the row into
// the K-major 128-byte-swizzled P tile and returns the fp32 row sum (four independent partial sums
// keep the add chain short).
template <int MODE, bool FULL>
__device__ __forceinline__ float exp_and_store(const uint32_t (&sv)[128], float cmul, float off, int valid,
                                               uint8_t* p_tile, int r) {
  using C = AttnCfg<MODE>;
  // int -> float by the 1.5 * 2^23 bias trick (|acc| <= 127*127*128 < 2^22), folded into the FMA
  const float off2 = fmaf(-12582912.f, cmul, off);
  auto pv = [&](int i) -> float {
    float v;
    if constexpr (C::QK_KIND == KIND_I8) v = ex2(fmaf(__uint_as_float(sv[i] + 0x4B400000u), cmul, off2));
    else v = ex2(fmaf(__uint_as_float(sv[i]), cmul, off));
    return (FULL || i < valid) ? v : 0.f;
  };
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  if constexpr (C::EP == 1) {
#pragma unroll
    for (int ck = 0; ck < 8; ++ck) {
      float e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        e[i] = pv(16 * ck + i);
        sum[i & 3] += e[i];
      }
      uint4 w;
      w.x = pack_e4m3x4(e[0], e[1], e[2], e[3]);
      w.y = pack_e4m3x4(e[4], e[5], e[6], e[7]);
      w.z = pack_e4m3x4(e[8], e[9], e[10], e[11]);
      w.w = pack_e4m3x4(e[12], e[13], e[14], e[15]);
      *reinterpret_cast<uint4*>(p_tile + r * 128 + ((ck ^ (r & 7)) << 4)) = w;
    }
  } else {
#pragma unroll
    for (int ck = 0; ck < 16; ++ck) {
      float e[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        e[i] = pv(8 * ck + i);
        sum[i & 3] += e[i];
      }
      uint4 w;
      w.x = pack_f16x2(e[0], e[1]);
      w.y = pack_f16x2(e[2], e[3]);
      w.z = pack_f16x2(e[4], e[5]);
      w.w = pack_f16x2(e[6], e[7]);
      *reinterpret_cast<uint4*>(p_tile + (ck >> 3) * BOX_BYTES + r * 128 + (((ck & 7) ^ (r & 7)) << 4)) = w;
    }
  }
  return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

template <int MODE>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  using C = AttnCfg<MODE>;
  using L = Smem<MODE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* kv_full = bars + 1;                  // [NSLOT]
  uint64_t* kv_empty = kv_full + C::NSLOT;       // [NSLOT]
  uint64_t* s_full = kv_empty + C::NSLOT;        // [2]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_full + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* vscale_s = reinterpret_cast<float*>(smem + L::OFF_VSCALE);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int range = blockIdx.x / p.tiles_per_range;
  const int q0 = p.q_begin + range * p.range_stride + (blockIdx.x % p.tiles_per_range) * 256;
  const int q_stop = min(p.q_end + range * p.range_stride, p.Sq);
  const int n_kv = p.Sk_pad / 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::NSLOT; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 128) vscale_s[threadIdx.x] = p.v_scale[static_cast<int64_t>(bh) * 128 + threadIdx.x];
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_arrive_expect_tx(q_full, 2 * L::Q_TILE);
      const int q_row = bh * p.Sq_pad + q0;
      for (int x = 0; x < 2; ++x)
        for (int sub = 0; sub < C::EQ; ++sub)
          tma_load_2d(smem + L::OFF_Q + x * L::Q_TILE + sub * BOX_BYTES, &map_q, q_full, sub * 64, q_row + x * 128);
      uint32_t seq = 0;
      bool ok = true;
      for (int j = 0; ok && j < n_kv; ++j) {
        {  // K_j : [128 tokens x 128 channels]
          const uint32_t s = seq % C::NSLOT, ph = (seq / C::NSLOT) & 1u;
          if (!mbar_wait(&kv_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&kv_full[s], BOX_BYTES * C::EQ);
          for (int sub = 0; sub < C::EQ; ++sub)
            tma_load_2d(smem + L::OFF_RING + s * L::SLOT + sub * BOX_BYTES, &map_k, &kv_full[s], sub * 64,
                        bh * p.Sk_pad + j * 128);
          ++seq;
        }
        {  // V_j^T : [128 channels x 128 tokens]
          const uint32_t s = seq % C::NSLOT, ph = (seq / C::NSLOT) & 1u;
          if (!mbar_wait(&kv_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&kv_full[s], BOX_BYTES * C::EP);
          for (int sub = 0; sub < C::EP; ++sub)
            tma_load_2d(smem + L::OFF_RING + s * L::SLOT + sub * BOX_BYTES, &map_v, &kv_full[s],
                        j * 128 + sub * 64, bh * 128);
          ++seq;
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = C::QK_KIND == KIND_I8 ? make_idesc(2, 1, 1, 128, 128) : make_idesc(1, 0, 0, 128, 128);
      constexpr uint32_t idesc_pv = make_idesc(1, 0, 0, 128, 128);  // e4m3 x e4m3 or f16 x f16 -> f32
      const uint32_t q_addr = smem_u32(smem + L::OFF_Q);
      const uint32_t p_addr = smem_u32(smem + L::OFF_P);
      const uint32_t ring = smem_u32(smem + L::OFF_RING);
      auto slot_of = [](uint32_t seq) { return seq % C::NSLOT; };
      auto phase_of = [](uint32_t seq) { return (seq / C::NSLOT) & 1u; };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&kv_full[slot_of(0)], phase_of(0), abort_flag);
      if (ok) {
        tc_fence_after_sync();
        for (int x = 0; x < 2; ++x) {
          mma_tile<C::QK_KIND, C::EQ>(tmem_base + x * 128, q_addr + x * L::Q_TILE, ring + slot_of(0) * L::SLOT, idesc_qk, false);
          umma_commit(&s_full[x]);
        }
        umma_commit(&kv_empty[slot_of(0)]);
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const uint32_t seq_v = 2 * j + 1, seq_k = 2 * j + 2;
        const bool more = j + 1 < n_kv;
        if (!mbar_wait(&kv_full[slot_of(seq_v)], phase_of(seq_v), abort_flag)) { ok = false; break; }
        if (more && !mbar_wait(&kv_full[slot_of(seq_k)], phase_of(seq_k), abort_flag)) { ok = false; break; }
        for (int x = 0; x < 2; ++x) {
          if (!mbar_wait(&p_full[x], j & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          mma_tile<C::PV_KIND, C::EP>(tmem_base + 256 + x * 128, p_addr + x * L::P_TILE, ring + slot_of(seq_v) * L::SLOT,
                                      idesc_pv, j > 0);
          if (more)
            mma_tile<C::QK_KIND, C::EQ>(tmem_base + x * 128, q_addr + x * L::Q_TILE, ring + slot_of(seq_k) * L::SLOT,
                                        idesc_qk, false);
          umma_commit(&s_full[x]);
        }
        if (!ok) break;
        umma_commit(&kv_empty[slot_of(seq_v)]);
        if (more) umma_commit(&kv_empty[slot_of(seq_k)]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int x = warp >> 2;          // query tile of this warpgroup
    const int quarter = warp & 3;     // TMEM lanes [32*quarter, +32)
    const int r = quarter * 32 + lane;  // row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + x * 128;
    const uint32_t o_tmem = tmem_base + lane_base + 256 + x * 128;
    uint8_t* p_tile = smem + L::OFF_P + x * L::P_TILE;
    const int q_row = q0 + x * 128 + r;
    const float sq = q_row < p.Sq ? p.q_scale[static_cast<int64_t>(bh) * p.Sq_pad + q_row] : 1.f;
    const float* ks = p.k_scale + static_cast<int64_t>(bh) * n_kv;
    float m = -INFINITY, l = 0.f;
    float ks_next = ks[0];
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const float kscale = ks_next;
      if (j + 1 < n_kv) ks_next = ks[j + 1];
      if (!mbar_wait(&s_full[x], j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t sv[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[c * 32]));
      tmem_wait_ld();

      const float cmul = sq * kscale;
      const int valid = p.Sk - j * 128;  // columns >= valid are padding (only in the last tile)
      const bool full = valid >= 128;
      const float mx = full ? row_max<MODE, true>(sv, cmul, valid) : row_max<MODE, false>(sv, cmul, valid);
      const float m_new = (mx > m + C::TAU) ? mx : m;
      const float alpha = ex2(m - m_new);  // m = -inf on the first tile -> 0
      const float off = C::PBIAS - m_new;
      const float sum = full ? exp_and_store<MODE, true>(sv, cmul, off, valid, p_tile, r)
                             : exp_and_store<MODE, false>(sv, cmul, off, valid, p_tile, r);
      l = fmaf(l, alpha, sum);
      m = m_new;

      // correction: O_X *= alpha when any row of this warp moved its maximum (P_X . V_{j-1} is complete)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tmem_ld32(o_tmem + c * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st32(o_tmem + c * 32, ov);
        }
        tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&p_full[x]);
    }

    if (ok && mbar_wait(&s_full[x], n_kv & 1u, abort_flag)) {
      tc_fence_after_sync();
      const float inv_l = 1.f / l;
      const bool store = q_row < q_stop;
      const int b = bh / p.heads, h = bh % p.heads;
      uint16_t* orow = static_cast<uint16_t*>(p.o) + b * p.o_sb + h * p.o_sh + static_cast<int64_t>(q_row) * p.o_st;
#pragma unroll
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
              const float a = __uint_as_float(ov[i + 2 * q]) * vscale_s[c * 32 + i + 2 * q] * inv_l;
              const float bb = __uint_as_float(ov[i + 2 * q + 1]) * vscale_s[c * 32 + i + 2 * q + 1] * inv_l;
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
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, DAX_ERR_TIMEOUT);
}

template <int MODE>
int launch_fwd(const AttnWorkspace& ws, const AttnParams& p, int64_t BH, cudaStream_t st) {
  using C = AttnCfg<MODE>;
  using L = Smem<MODE>;
  CUtensorMap map_q, map_k, map_v;
  const uint32_t inner = 128 / C::EQ;  // elements per 128-byte row
  {
    uint64_t dims[2] = {128, static_cast<uint64_t>(BH) * ws.Sq_pad};
    uint64_t strides[2] = {static_cast<uint64_t>(C::EQ), 128ull * C::EQ};
    uint32_t box[2] = {inner, 128};
    int rc = make_tma_map(&map_q, ws.q, C::EQ, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  {
    uint64_t dims[2] = {128, static_cast<uint64_t>(BH) * ws.Sk_pad};
    uint64_t strides[2] = {static_cast<uint64_t>(C::EQ), 128ull * C::EQ};
    uint32_t box[2] = {inner, 128};
    int rc = make_tma_map(&map_k, ws.k, C::EQ, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(ws.Sk_pad), static_cast<uint64_t>(BH) * 128};
    uint64_t strides[2] = {static_cast<uint64_t>(C::EP), static_cast<uint64_t>(ws.Sk_pad) * C::EP};
    uint32_t box[2] = {static_cast<uint32_t>(128 / C::EP), 128};
    int rc = make_tma_map(&map_v, ws.vt, C::EP, 2, dims, strides, box);
    if (rc != DAX_OK) return rc;
  }
  DAX_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  dim3 grid(static_cast<unsigned>(p.n_ranges * p.tiles_per_range), static_cast<unsigned>(BH));
  attn_fwd_kernel<MODE><<<grid, ATT_THREADS, L::TOTAL, st>>>(map_q, map_k, map_v, p);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

}  // namespace
}  // namespace dax

extern "C" int dax_attn_forward(void* o, int dtype, int64_t B, int64_t heads, int64_t Sq, int64_t Sk,
                                int64_t o_strides[3], int64_t q_begin, int64_t q_end, int64_t n_ranges,
                                int64_t range_stride, int mode, void* workspace, size_t workspace_bytes,
                                void* stream) {
  using namespace dax;
  DAX_REQUIRE(o && workspace && o_strides, DAX_ERR_INVALID, "attn_forward: null pointer");
  DAX_REQUIRE(dtype == DAX_BF16 || dtype == DAX_F16, DAX_ERR_UNSUPPORTED, "attn_forward: dtype %d is not BF16/F16", dtype);
  AttnWorkspace ws;
  int rc = attn_workspace_layout(B, heads, Sq, Sk, mode, workspace, workspace_bytes, &ws);
  if (rc != DAX_OK) return rc;
  DAX_REQUIRE(q_begin >= 0 && q_begin <= q_end && q_end <= Sq, DAX_ERR_INVALID,
              "attn_forward: bad query range [%lld, %lld) for Sq=%lld", (long long)q_begin, (long long)q_end, (long long)Sq);
  DAX_REQUIRE(n_ranges >= 1 && (n_ranges == 1 || range_stride >= q_end - q_begin) &&
                  q_end + (n_ranges - 1) * range_stride <= Sq,
              DAX_ERR_INVALID, "attn_forward: %lld ranges of stride %lld do not fit Sq=%lld", (long long)n_ranges,
              (long long)range_stride, (long long)Sq);
  if (q_begin == q_end) return DAX_OK;
  DAX_REQUIRE(aligned16(o) && o_strides[0] % 8 == 0 && o_strides[1] % 8 == 0 && o_strides[2] % 8 == 0, DAX_ERR_ALIGN,
              "attn_forward: o must be 16-byte aligned with strides that are multiples of 8 elements");
  AttnParams p;
  p.q_scale = ws.q_scale; p.k_scale = ws.k_scale; p.v_scale = ws.v_scale;
  p.o = o;
  p.status = device_status_ptr();
  DAX_REQUIRE(p.status != nullptr, DAX_ERR_CUDA, "attn_forward: cannot resolve the device status word");
  p.o_sb = o_strides[0]; p.o_sh = o_strides[1]; p.o_st = o_strides[2];
  p.heads = static_cast<int>(heads);
  p.Sq = static_cast<int>(Sq); p.Sk = static_cast<int>(Sk);
  p.Sq_pad = static_cast<int>(ws.Sq_pad); p.Sk_pad = static_cast<int>(ws.Sk_pad);
  p.q_begin = static_cast<int>(q_begin); p.q_end = static_cast<int>(q_end);
  p.n_ranges = static_cast<int>(n_ranges); p.range_stride = static_cast<int>(range_stride);
  p.tiles_per_range = static_cast<int>((q_end - q_begin + 255) / 256);
  p.out_bf16 = dtype == DAX_BF16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mode == DAX_ATTN_QK_I8_PV_F8) return launch_fwd<DAX_ATTN_QK_I8_PV_F8>(ws, p, B * heads, st);
  return launch_fwd<DAX_ATTN_QK_F16_PV_F16>(ws, p, B * heads, st);
}
