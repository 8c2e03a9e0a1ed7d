// Quantised non-causal flash attention for head_dim 128 on tcgen05 / TMEM / TMA.
//
// The two modes with INT8 scores (template parameter, chosen per call):
//   INT8 Q.K^T (kind::i8, int32 accumulators)  + FP8 e4m3 P.V (kind::f8f6f4, fp32 accumulators)
//   INT8 Q.K^T                                 + bf16 P.V   (V unquantised; P -> bf16 by truncation)
// (the mode with bf16 scores, bf16 Q.K^T + bf16 P.V, is the kernel in attn_tmem.cu)
// A CTA owns 256 query rows of one (batch, head): two 128-row tiles X = 0, 1 that ping-pong so
// that the tensor pipe works on one tile while the softmax warps work on the other.
//
//   warps 0..7    softmax + correction + epilogue of tile 0: thread = one query row x 64 key columns
//                 (warps w and w+4 share the rows of TMEM lane quarter w%4 and split the columns)
//   warps 8..15   the same for tile 1
//   warp  16      TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... through a ring
//   warps 17..    MMA issuers, one thread each: two (one per tile: Q.K^T of the next KV tile, then P.V of this
//                 one) or, with 16-bit P.V, three (Q.K^T of both tiles; P.V of tile 0; P.V of tile 1), see AttnCfg
// Four softmax warps per scheduler instead of two: the softmax is a chain of dependent fixed-latency
// operations around a 16-per-clock exp unit, and only more resident warps hide that latency.  The two
// threads of a row agree on the row maximum through a sequence-stamped shared-memory slot (no CTA or
// named barrier, every poll is bounded) and add their partial row sums once at the end.
//
// Tensor memory (512 columns): S_0 [0,128)  S_1 [128,256)  O_0 [256,384)  O_1 [384,512).
// Per KV tile j and query tile X:   S_X = Q_X . K_j^T   ->  softmax warps read S_X, keep the running
// row maximum m and sum l (base-2 domain), write P_X to shared memory in the K-major 128-byte
// swizzled layout the MMA reads, rescale O_X in tensor memory when m moved  ->  O_X += P_X . V_j.
// The softmax warps copy S_X into registers first and release it at once (s_free), so Q_X . K_{j+1}^T
// runs while they are still exponentiating tile j: they never wait for a score tile.  P_X and O_X are
// reused only after P_X . V_{j-1} has completed (pv_done), which by then it normally has.
//
// Operands come from the workspace written by the prepare step (attn_prep.cu): every tile is a set
// of [128 rows x 128 bytes] boxes, so one shared-memory descriptor form serves Q, K, P and V^T.
#include <climits>

#include "attn_common.cuh"
#include "sm100_ptx.cuh"

namespace dax {
namespace {

constexpr int PRODUCER_WARP = 16;
constexpr int SOFTMAX_WARPS = 16;
constexpr int BOX_BYTES = 128 * 128;  // one [128 x 128 B] box

template <int MODE> struct AttnCfg;
template <> struct AttnCfg<DAX_ATTN_QK_I8_PV_F8> {
  static constexpr int QK_KIND = KIND_I8, PV_KIND = KIND_F8;
  static constexpr int EQ = 1, EP = 1;       // bytes per element of Q/K and of P/V
  static constexpr int NSLOT = 8;            // 8 x 16 KB: four (K, V) pairs in flight
  static constexpr int ISSUERS = 2;
  static constexpr float TAU = 0.f;          // P is scaled to the e4m3 range: the row max must be exact
  static constexpr float PBIAS = 8.8073549f; // log2(448): P in (0, 448]
};
template <> struct AttnCfg<DAX_ATTN_QK_I8_PV_BF16> {
  static constexpr int QK_KIND = KIND_I8, PV_KIND = KIND_F16;
  static constexpr int EQ = 1, EP = 2;
  static constexpr int NSLOT = 3;            // 3 x 32 KB (K tiles use half a slot): Q 32 KB + P 64 KB + ring 96 KB
  static constexpr int ISSUERS = 3;
  static constexpr float TAU = 8.f;
  static constexpr float PBIAS = 0.f;
};

// 16 softmax warps, the producer warp, the issuer warps: at most 20 warps, i.e. five per scheduler, which
// is what leaves 96 registers per thread
template <int MODE>
constexpr int att_threads() { return 32 * (SOFTMAX_WARPS + 1 + AttnCfg<MODE>::ISSUERS); }
// The kernel is always compiled for the register budget of 640 threads (96 per thread, which is also what it
// uses).  With the bound at 608 threads the compiler still uses 96 registers but schedules the softmax loop
// differently, and the INT8/FP8 kernel ran 15 % slower.
constexpr int ATT_BOUND_THREADS = 640;

template <int MODE>
struct Smem {
  using C = AttnCfg<MODE>;
  static constexpr int Q_TILE = BOX_BYTES * C::EQ;
  static constexpr int P_TILE = BOX_BYTES * C::EP;
  static constexpr int SLOT = BOX_BYTES * (C::EQ > C::EP ? C::EQ : C::EP);
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_P = OFF_Q + 2 * Q_TILE;
  static constexpr int OFF_RING = OFF_P + 2 * P_TILE;
  static constexpr int OFF_BIAS = OFF_RING + C::NSLOT * SLOT;  // constant tile that seeds the score accumulators
  static constexpr int OFF_BAR = OFF_BIAS + (C::QK_KIND == KIND_I8 ? BOX_BYTES : 0);
  static constexpr int OFF_VSCALE = OFF_BAR + 256;
  static constexpr int OFF_XCHG = OFF_VSCALE + 512;           // [2 tiles][2 parities][2 halves][128 rows] x 8 B
  static constexpr int TOTAL = OFF_XCHG + 2 * 2 * 2 * 128 * 8 + 1024 /*alignment slack*/;
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

// Two fp32 values -> bf16x2 by keeping the upper halves (one byte-permute for two elements; the
// rounding conversion instructions run on the 16-per-clock unit the exponentials already saturate).
// Truncation lowers every P by 2^-9 on average; the epilogue multiplies O by (1 + 2^-9) to centre it.
__device__ __forceinline__ uint32_t pack_bf16x2_trunc(float a, float b) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(r) : "r"(__float_as_uint(a)), "r"(__float_as_uint(b)));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// Integer score accumulators start from the bit pattern of 1.5 * 2^23 (see the MMA issuer), so that the
// register a thread reads IS the float 12582912 + acc: no conversion instruction per element.
constexpr float kAccBias = 12582912.f;

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Columns >= valid of the last KV tile are padding: give them the score -inf, which is never the row maximum
// and whose exponential is exactly zero whatever the (positive) scale; read as a biased integer accumulator
// the same bit pattern behaves identically, because the scores only ever go through max and one FMA.
// Only the last KV tile of a ragged sequence takes this path, so the hot loop carries one copy of the
// max / exponential code and no per-column predicate.
__device__ __forceinline__ void mask_padding64(uint32_t (&sv)[64], int valid) {
#pragma unroll
  for (int i = 0; i < 64; ++i) sv[i] = i < valid ? sv[i] : 0xFF800000u;
}

// Maximum of the scaled scores over the 64 columns a thread owns.  The scale is positive, so the maximum is
// taken on the raw accumulators (two columns per instruction) and scaled once.
template <int MODE>
__device__ __forceinline__ float row_max64(const uint32_t (&sv)[64], float cmul) {
  using C = AttnCfg<MODE>;
  float fmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < 64; i += 2)
    fmx[(i >> 1) & 3] = fmax3(fmx[(i >> 1) & 3], __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
  const float mx = fmaxf(fmax3(fmx[0], fmx[1], fmx[2]), fmx[3]);
  if constexpr (C::QK_KIND == KIND_I8) return (mx - kAccBias) * cmul;
  else return mx * cmul;
}

// p_i = 2^(s_i * cmul + off) for the 64 columns held in sv (columns 64*half .. 64*half+63 of the tile);
// converts to the P format, writes them into the K-major 128-byte-swizzled P tile and returns the
// fp32 partial row sum (four independent partial sums keep the add chain short).
template <int MODE>
__device__ __forceinline__ float exp_and_store64(const uint32_t (&sv)[64], float cmul, float off, uint8_t* p_tile,
                                                 int r, int half) {
  using C = AttnCfg<MODE>;
  // integer accumulators arrive as 12582912 + acc (|acc| <= 127*127*128 < 2^22): the bias folds into the FMA
  const float off2 = C::QK_KIND == KIND_I8 ? fmaf(-kAccBias, cmul, off) : off;
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  auto pv = [&](int i) -> float {
    const float e = ex2(fmaf(__uint_as_float(sv[i]), cmul, off2));
    sum[i & 3] += e;
    return e;
  };
  if constexpr (C::EP == 1) {
    // one row of the P tile is 128 bytes: this thread owns 16-byte chunks 4*half .. 4*half+3
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      // sixteen exponentials per 16-byte store: converting and storing in these batches interleaves the
      // conversions with the next batch's exponentials (all 64 at once was 15 % slower)
      float e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = pv(16 * c + i);
      uint4 w;
      w.x = pack_e4m3x4(e[0], e[1], e[2], e[3]);
      w.y = pack_e4m3x4(e[4], e[5], e[6], e[7]);
      w.z = pack_e4m3x4(e[8], e[9], e[10], e[11]);
      w.w = pack_e4m3x4(e[12], e[13], e[14], e[15]);
      const int ck = 4 * half + c;
      *reinterpret_cast<uint4*>(p_tile + r * 128 + ((ck ^ (r & 7)) << 4)) = w;
    }
  } else {
    // bf16 P: two 16 KB boxes of 64 key columns each; this thread owns one full 128-byte row of box `half`
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float e[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) e[i] = pv(8 * c + i);
      uint4 w;
      w.x = pack_bf16x2_trunc(e[0], e[1]);
      w.y = pack_bf16x2_trunc(e[2], e[3]);
      w.z = pack_bf16x2_trunc(e[4], e[5]);
      w.w = pack_bf16x2_trunc(e[6], e[7]);
      *reinterpret_cast<uint4*>(p_tile + half * BOX_BYTES + r * 128 + ((c ^ (r & 7)) << 4)) = w;
    }
  }
  return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

// Sequence-stamped exchange slot between the two threads of a row: {value, sequence number}.
__device__ __forceinline__ void xchg_write(uint2* slot, float v, uint32_t seq) {
  asm volatile("st.volatile.shared.v2.u32 [%0], {%1, %2};" ::"r"(smem_u32(slot)), "r"(__float_as_uint(v)), "r"(seq)
               : "memory");
}
__device__ __forceinline__ bool xchg_read(const uint2* slot, uint32_t seq, float& v, volatile uint32_t* abort_flag) {
  const uint32_t addr = smem_u32(slot);
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t a, b;
    asm volatile("ld.volatile.shared.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr) : "memory");
    if (b == seq) {
      v = __uint_as_float(a);
      return true;
    }
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

template <int MODE>
__global__ void __launch_bounds__(ATT_BOUND_THREADS, 1)
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
  uint64_t* p_full = s_full + 2;                 // [2]  softmax -> MMA: P_X written, O_X rescaled
  uint64_t* s_free = p_full + 2;                 // [2]  softmax -> MMA: S_X is in registers, may be overwritten
  uint64_t* pv_done = s_free + 2;                // [2]  MMA -> softmax: P_X . V_j complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* vscale_s = reinterpret_cast<float*>(smem + L::OFF_VSCALE);
  uint2* xchg = reinterpret_cast<uint2*>(smem + L::OFF_XCHG);

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
      mbar_init(&kv_empty[i], 2);  // released by two MMA commits (one per query tile)
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);   // one arrival per softmax warp of the tile
      mbar_init(&s_free[i], 8);   // likewise
      mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 128) vscale_s[threadIdx.x] = p.v_scale[static_cast<int64_t>(bh) * 128 + threadIdx.x];
  for (int i = threadIdx.x; i < 2 * 2 * 2 * 128; i += blockDim.x) xchg[i] = make_uint2(0u, 0u);
  if constexpr (C::QK_KIND == KIND_I8) {
    // [128 rows x 128 B] box, bf16, 128-byte swizzle: K elements 0..2 of every row are 2048, the rest 0, so that
    // tile . tile^T = 3 * 2048^2 = 12582912 = 1.5 * 2^23 in every accumulator (logical chunk 0 of row r sits in
    // physical chunk r & 7)
    uint4* bias = reinterpret_cast<uint4*>(smem + L::OFF_BIAS);
    for (int i = threadIdx.x; i < BOX_BYTES / 16; i += blockDim.x) {
      const int r = i >> 3, ck = i & 7;
      bias[i] = ck == (r & 7) ? make_uint4(0x45004500u, 0x00004500u, 0u, 0u) : make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
  }
  if (warp == SOFTMAX_WARPS) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == PRODUCER_WARP) {
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
  } else if (warp > SOFTMAX_WARPS && warp <= SOFTMAX_WARPS + C::ISSUERS) {
    // ---------------------------------------------------------------- MMA issuers (one thread each)
    // One thread cannot issue faster than one tcgen05.mma per ~100 clocks whatever the shape, while the pipe
    // retires a 128x128x32 step in 64; two or more threads together reach the pipe's rate.
    // Two issuers (8-bit Q.K^T): one per query tile, so that a tile never waits behind the other tile's
    // barriers.  For its tile the events come in a fixed order: S(j) copied to registers -> Q.K^T(j+1) may
    // overwrite it; then P(j) written -> P.V(j); then S(j+1) copied, and so on.
    // Three issuers (16-bit Q.K^T, eight steps per product, the tensor pipe is the busiest unit): one for
    // Q.K^T of both tiles, one per tile for P.V.
    if (lane == 0) {
      const int role = warp - (SOFTMAX_WARPS + 1);
      // s8 x s8 -> s32, or bf16 x bf16 -> f32;  e4m3 x e4m3 -> f32, or bf16 x bf16 -> f32
      constexpr uint32_t idesc_qk = C::QK_KIND == KIND_I8 ? make_idesc(2, 1, 1, 128, 128) : make_idesc(1, 1, 1, 128, 128);
      constexpr uint32_t idesc_pv = C::PV_KIND == KIND_F8 ? make_idesc(1, 0, 0, 128, 128) : make_idesc(1, 1, 1, 128, 128);
      const uint32_t q_addr = smem_u32(smem + L::OFF_Q);
      const uint32_t p_addr = smem_u32(smem + L::OFF_P);
      const uint32_t ring = smem_u32(smem + L::OFF_RING);
      const uint64_t bias_desc = make_desc_k_sw128(smem_u32(smem + L::OFF_BIAS));
      (void)bias_desc;
      auto issue_qk = [&](int j, int x) -> bool {  // S_x(j) = Q_x . K_j^T
        const uint32_t seq_k = 2 * j, slot = seq_k % C::NSLOT, ph = (seq_k / C::NSLOT) & 1u;
        const uint32_t s_tm = tmem_base + x * 128;
        if (!mbar_wait(&kv_full[slot], ph, abort_flag)) return false;
        // S_x(j-1) has been copied to registers by all eight warps of the tile
        if (j > 0 && !mbar_wait(&s_free[x], (j - 1) & 1u, abort_flag)) return false;
        tc_fence_after_sync();
        if constexpr (C::QK_KIND == KIND_I8) {
          // one bf16 K=16 instruction writes the float 12582912 into every accumulator; the integer
          // instructions then add the dot products to that bit pattern
          umma_ss<KIND_F16>(s_tm, bias_desc, bias_desc, make_idesc(1, 1, 1, 128, 128), 0u);
        }
        mma_tile<C::QK_KIND, C::EQ>(s_tm, q_addr + x * L::Q_TILE, ring + slot * L::SLOT, idesc_qk, C::QK_KIND == KIND_I8);
        umma_commit(&s_full[x]);
        umma_commit(&kv_empty[slot]);  // two arrivals free the slot: one per tile
        return true;
      };
      auto issue_pv = [&](int j, int x) -> bool {  // O_x += P_x . V_j
        const uint32_t seq_v = 2 * j + 1, slot = seq_v % C::NSLOT, ph = (seq_v / C::NSLOT) & 1u;
        if (!mbar_wait(&kv_full[slot], ph, abort_flag)) return false;
        if (!mbar_wait(&p_full[x], j & 1u, abort_flag)) return false;
        tc_fence_after_sync();
        mma_tile<C::PV_KIND, C::EP>(tmem_base + 256 + x * 128, p_addr + x * L::P_TILE, ring + slot * L::SLOT, idesc_pv, j > 0);
        umma_commit(&pv_done[x]);
        umma_commit(&kv_empty[slot]);  // the other tile's P.V supplies the second arrival
        return true;
      };
      if constexpr (C::ISSUERS == 2) {
        const int x = role;
        bool ok = mbar_wait(q_full, 0, abort_flag) && issue_qk(0, x);
        for (int j = 0; ok && j < n_kv; ++j) ok = (j + 1 >= n_kv || issue_qk(j + 1, x)) && issue_pv(j, x);
      } else if (role == 0) {
        bool ok = mbar_wait(q_full, 0, abort_flag);
        for (int j = 0; ok && j < n_kv; ++j) ok = issue_qk(j, 0) && issue_qk(j, 1);
      } else {
        bool ok = true;
        for (int j = 0; ok && j < n_kv; ++j) ok = issue_pv(j, role - 1);
      }
    }
  } else if (warp < SOFTMAX_WARPS) {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int x = warp >> 3;            // query tile
    const int quarter = warp & 3;       // TMEM lanes [32*quarter, +32)
    const int half = (warp >> 2) & 1;   // key columns [64*half, +64) of every tile; O channels likewise
    const int r = quarter * 32 + lane;  // row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + x * 128 + half * 64;
    const uint32_t o_tmem = tmem_base + lane_base + 256 + x * 128 + half * 64;
    uint8_t* p_tile = smem + L::OFF_P + x * L::P_TILE;
    // exchange slots: [tile][parity][half][row]
    auto slot = [&](int parity, int hf) { return xchg + ((x * 2 + parity) * 2 + hf) * 128 + r; };
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
      uint32_t sv[64];
      tmem_ld32(s_tmem, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld32(s_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[x]);  // S_X is in registers: Q.K^T of the next tile may start

      const float cmul = sq * kscale;
      const int valid = p.Sk - j * 128 - half * 64;  // columns >= valid are padding (only in the last tile)
      if (valid < 64) mask_padding64(sv, valid);
      const float pm = row_max64<MODE>(sv, cmul);
      xchg_write(slot(j & 1, half), pm, static_cast<uint32_t>(j + 1));
      float pm2;
      if (!xchg_read(slot(j & 1, half ^ 1), static_cast<uint32_t>(j + 1), pm2, abort_flag)) { ok = false; break; }
      const float mx = fmaxf(pm, pm2);
      const float m_new = (mx > m + C::TAU) ? mx : m;
      const float alpha = ex2(m - m_new);  // m = -inf on the first tile -> 0
      const float off = C::PBIAS - m_new;
      // P_X and O_X are free once P_X . V_{j-1} has completed
      if (j > 0) {
        if (!mbar_wait(&pv_done[x], (j - 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
      }
      const float sum = exp_and_store64<MODE>(sv, cmul, off, p_tile, r, half);
      l = fmaf(l, alpha, sum);
      m = m_new;

      // correction: O_X *= alpha when any row of this warp moved its maximum (P_X . V_{j-1} is complete)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        uint32_t ov[64];
        tmem_ld32(o_tmem, *reinterpret_cast<uint32_t(*)[32]>(&ov[0]));
        tmem_ld32(o_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&ov[32]));
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 64; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
        tmem_st32(o_tmem, *reinterpret_cast<uint32_t(*)[32]>(&ov[0]));
        tmem_st32(o_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&ov[32]));
        tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }

    if (ok && mbar_wait(&pv_done[x], (n_kv - 1) & 1u, abort_flag)) {
      tc_fence_after_sync();
      // the two threads of a row hold partial sums of the same row: add them
      xchg_write(slot(n_kv & 1, half), l, static_cast<uint32_t>(n_kv + 1));
      float l2 = 0.f;
      if (xchg_read(slot(n_kv & 1, half ^ 1), static_cast<uint32_t>(n_kv + 1), l2, abort_flag)) {
        // bf16 P was truncated, not rounded: centre the result (see pack_bf16x2_trunc)
        const float inv_l = (C::EP == 2 ? 1.001953125f : 1.f) / (l + l2);
        const bool store = q_row < q_stop;
        const int b = bh / p.heads, h = bh % p.heads;
        uint16_t* orow = static_cast<uint16_t*>(p.o) + attn_out_offset(p, b, h, q_row) + half * 64;
        const float* vs = vscale_s + half * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t ov[32];
          tmem_ld32(o_tmem + c * 32, ov);
          tmem_wait_ld();
          if (store) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float a = __uint_as_float(ov[i + 2 * q]) * vs[c * 32 + i + 2 * q] * inv_l;
                const float bb = __uint_as_float(ov[i + 2 * q + 1]) * vs[c * 32 + i + 2 * q + 1] * inv_l;
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
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == SOFTMAX_WARPS) {
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
  static_assert(att_threads<MODE>() <= ATT_BOUND_THREADS, "more warps than the register budget allows");
  attn_fwd_kernel<MODE><<<grid, att_threads<MODE>(), L::TOTAL, st>>>(map_q, map_k, map_v, p);
  DAX_CUDA(cudaGetLastError());
  return DAX_OK;
}

}  // namespace
}  // namespace dax

namespace dax {
namespace {
int attn_forward_entry(void* o, int dtype, int64_t B, int64_t heads, int64_t Sq, int64_t Sk, const int64_t o_strides[3],
                       int64_t q_begin, int64_t q_end, int64_t n_ranges, int64_t range_stride, const GroupTable& dest,
                       int64_t rows_per_dest, int mode, void* workspace, size_t workspace_bytes, void* stream) {
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
  DAX_REQUIRE(dest.n == 0 || (B == 1 && rows_per_dest > 0 && static_cast<int64_t>(dest.n) * rows_per_dest >= Sq),
              DAX_ERR_INVALID, "attn_forward: %d destinations of %lld rows do not cover Sq=%lld (batch must be 1)", dest.n,
              (long long)rows_per_dest, (long long)Sq);
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
  p.dest = dest;
  p.rows_per_dest = static_cast<int>(rows_per_dest > 0 ? rows_per_dest : 1);
  p.direct_cmul = 0.f;
  p.in_fmt = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mode == DAX_ATTN_QK_I8_PV_F8) return launch_fwd<DAX_ATTN_QK_I8_PV_F8>(ws, p, B * heads, st);
  if (mode == DAX_ATTN_QK_I8_PV_BF16) return launch_fwd<DAX_ATTN_QK_I8_PV_BF16>(ws, p, B * heads, st);
  return launch_attn_fwd_tmem_p(ws, p, B * heads, st);  // bf16 Q.K^T + bf16 P.V: attn_tmem.cu
}
}  // namespace
}  // namespace dax

extern "C" int dax_attn_forward(void* o, int dtype, int64_t B, int64_t heads, int64_t Sq, int64_t Sk,
                                int64_t o_strides[3], int64_t q_begin, int64_t q_end, int64_t n_ranges,
                                int64_t range_stride, int mode, void* workspace, size_t workspace_bytes,
                                void* stream) {
  dax::GroupTable none{};
  return dax::attn_forward_entry(o, dtype, B, heads, Sq, Sk, o_strides, q_begin, q_end, n_ranges, range_stride, none, 0,
                                 mode, workspace, workspace_bytes, stream);
}

extern "C" int dax_attn_forward_scatter(void* const* o_dest, int64_t n_dest, int64_t rows_per_dest, int dtype,
                                        int64_t heads, int64_t Sq, int64_t Sk, int64_t head_stride,
                                        int64_t token_stride, int64_t q_begin, int64_t q_end, int mode,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  dax::GroupTable tab{};
  void* base = nullptr;
  int rc = dax::make_group_table(o_dest, n_dest, 2, &tab, &base);
  if (rc != DAX_OK) return rc;
  int64_t strides[3] = {0, head_stride, token_stride};
  return dax::attn_forward_entry(base, dtype, 1, heads, Sq, Sk, strides, q_begin, q_end, 1, 0, tab, rows_per_dest, mode,
                                 workspace, workspace_bytes, stream);
}

extern "C" int dax_attn_forward_direct(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                                       int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3],
                                       int64_t v_strides[3], float sm_scale, void* o, int64_t o_strides[3],
                                       void* const* o_dest, int64_t n_dest, int64_t rows_per_dest, int64_t q_begin,
                                       int64_t q_end, int64_t n_ranges, int64_t range_stride, void* stream) {
  using namespace dax;
  DAX_REQUIRE(q && k && v && q_strides && k_strides && v_strides && o_strides, DAX_ERR_INVALID, "attn_forward_direct: null pointer");
  // bf16 only: P is produced as bf16 (truncation), and both operands of one kind::f16 product take the same format here;
  // sequences of at least one tile, so that no tensor-map box is larger than the tensor it reads
  DAX_REQUIRE(dtype == DAX_BF16, DAX_ERR_UNSUPPORTED, "attn_forward_direct: dtype %d is not BF16 (use dax_attn_prepare + dax_attn_forward)", dtype);
  DAX_REQUIRE(Sq >= 128 && Sk >= 128, DAX_ERR_UNSUPPORTED,
              "attn_forward_direct: Sq=%lld, Sk=%lld: sequences shorter than 128 go through dax_attn_prepare + dax_attn_forward",
              (long long)Sq, (long long)Sk);
  DAX_REQUIRE(B > 0 && heads > 0 && Sq > 0 && Sk > 0 && B * heads <= 65535 && Sq < (1ll << 31) - 256 && Sk < (1ll << 31) - 128,
              DAX_ERR_INVALID, "attn_forward_direct: bad shape B=%lld heads=%lld Sq=%lld Sk=%lld", (long long)B,
              (long long)heads, (long long)Sq, (long long)Sk);
  DAX_REQUIRE(sm_scale > 0.f, DAX_ERR_INVALID, "attn_forward_direct: sm_scale must be positive");
  const int64_t* ss[3] = {q_strides, k_strides, v_strides};
  const void* ptrs[3] = {q, k, v};
  for (int i = 0; i < 3; ++i) {
    DAX_REQUIRE(aligned16(ptrs[i]) && ss[i][1] % 8 == 0 && ss[i][2] % 8 == 0 && ss[i][2] >= 128 && ss[i][1] > 0, DAX_ERR_ALIGN,
                "attn_forward_direct: q, k, v must be 16-byte aligned with head / token strides that are multiples of 8 elements");
    // the 3-D tensor map flattens (batch, head) into one dimension of stride = head stride
    DAX_REQUIRE(B == 1 || ss[i][0] == heads * ss[i][1], DAX_ERR_UNSUPPORTED,
                "attn_forward_direct: batch stride must equal heads x head stride (or batch 1)");
  }
  DAX_REQUIRE(q_begin >= 0 && q_begin <= q_end && q_end <= Sq, DAX_ERR_INVALID,
              "attn_forward_direct: bad query range [%lld, %lld) for Sq=%lld", (long long)q_begin, (long long)q_end, (long long)Sq);
  DAX_REQUIRE(n_ranges >= 1 && (n_ranges == 1 || range_stride >= q_end - q_begin) && q_end + (n_ranges - 1) * range_stride <= Sq,
              DAX_ERR_INVALID, "attn_forward_direct: %lld ranges of stride %lld do not fit Sq=%lld", (long long)n_ranges,
              (long long)range_stride, (long long)Sq);
  GroupTable dest{};
  void* base = o;
  if (n_dest > 0) {
    int rc = make_group_table(o_dest, n_dest, 2, &dest, &base);
    if (rc != DAX_OK) return rc;
    DAX_REQUIRE(B == 1 && rows_per_dest > 0 && n_dest * rows_per_dest >= Sq && n_ranges == 1, DAX_ERR_INVALID,
                "attn_forward_direct: %lld destinations of %lld rows do not cover Sq=%lld (batch 1, one range)", (long long)n_dest,
                (long long)rows_per_dest, (long long)Sq);
  }
  DAX_REQUIRE(base != nullptr && aligned16(base) && o_strides[0] % 8 == 0 && o_strides[1] % 8 == 0 && o_strides[2] % 8 == 0,
              DAX_ERR_ALIGN, "attn_forward_direct: o must be 16-byte aligned with strides that are multiples of 8 elements");
  if (q_begin == q_end) return DAX_OK;
  AttnParams p{};
  p.o = base;
  p.status = device_status_ptr();
  DAX_REQUIRE(p.status != nullptr, DAX_ERR_CUDA, "attn_forward_direct: cannot resolve the device status word");
  p.o_sb = o_strides[0]; p.o_sh = o_strides[1]; p.o_st = o_strides[2];
  p.heads = static_cast<int>(heads);
  p.Sq = static_cast<int>(Sq); p.Sk = static_cast<int>(Sk);
  p.Sq_pad = static_cast<int>(round_up(Sq, 256)); p.Sk_pad = static_cast<int>(round_up(Sk, 128));
  p.q_begin = static_cast<int>(q_begin); p.q_end = static_cast<int>(q_end);
  p.n_ranges = static_cast<int>(n_ranges); p.range_stride = static_cast<int>(range_stride);
  p.tiles_per_range = static_cast<int>((q_end - q_begin + 255) / 256);
  p.out_bf16 = dtype == DAX_BF16;
  p.dest = dest;
  p.rows_per_dest = static_cast<int>(rows_per_dest > 0 ? rows_per_dest : 1);
  p.direct_cmul = sm_scale * 1.4426950408889634f;
  p.in_fmt = 1;
  return launch_attn_fwd_tmem_p_direct(q, k, v, q_strides[1], q_strides[2], k_strides[1], k_strides[2], v_strides[1],
                                       v_strides[2], p, B * heads, static_cast<cudaStream_t>(stream));
}
