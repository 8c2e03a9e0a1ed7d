// Workspace shared by the two attention steps (prepare and forward).  The caller owns the memory;
// this header only fixes where each array lives inside it.
//
//   q      [BH, Sq_pad, 128]   INT8 or bf16, softmax scale * log2(e) folded in (INT8: per-token scale)
//   k      [BH, Sk_pad, 128]   INT8 or bf16, per-(batch, head, channel) sequence mean removed
//   vt     [BH, 128, Sk_pad]   FP8 e4m3 or bf16, transposed so that tokens are contiguous
//   q_scale[BH, Sq_pad]  k_scale[BH, Sk_pad/128]  v_scale[BH, 128]      fp32
//   k_mean [BH, 128]           fp32
//   part   [BH, chunks, 2, 128] fp32 partial column sums of K and column maxima of |V|
// Sq_pad is Sq rounded up to 256 (one CTA of the forward kernel owns 256 query rows), Sk_pad is Sk
// rounded up to 128; the prepare step zero-fills the padding.
#pragma once
#include "common.cuh"

namespace dax {

constexpr int64_t kStatChunk = 512;  // tokens per partial-statistics block

struct AttnWorkspace {
  void* q;
  void* k;
  void* vt;
  float* q_scale;
  float* k_scale;
  float* v_scale;
  float* k_mean;
  float* part;
  int64_t Sq_pad, Sk_pad, chunks;
  size_t bytes;
};

// Arguments of the forward kernels.
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
  // scattered output (dest.n > 0): query row q belongs to destination q / rows_per_dest and is written at
  // o + dest.off[q / rows_per_dest] + (q % rows_per_dest) * o_st + head * o_sh  (the head->sequence exchange of the
  // sequence-parallel attention written by the kernel itself, each destination being another GPU's buffer)
  GroupTable dest;
  int rows_per_dest;
  // direct mode of the bf16 kernel (operands read in place, no prepare step): score multiplier
  // softmax_scale * log2(e), and the 16-bit format of Q / K / V (1 = bf16, 0 = f16)
  float direct_cmul;
  int in_fmt;
};

// Address of output row q_row of (batch b, head h), element units.
__device__ __forceinline__ int64_t attn_out_offset(const AttnParams& p, int b, int h, int q_row) {
  if (p.dest.n > 0) {
    const int d = q_row / p.rows_per_dest;
    return p.dest.off[d < kMaxGroups ? d : 0] + static_cast<int64_t>(q_row - d * p.rows_per_dest) * p.o_st + h * p.o_sh;
  }
  return b * p.o_sb + h * p.o_sh + static_cast<int64_t>(q_row) * p.o_st;
}

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// bytes per element of the Q/K operands and of the P/V operands for a mode
inline int attn_qk_bytes(int mode) { return mode == DAX_ATTN_QK_BF16_PV_BF16 ? 2 : 1; }
inline int attn_pv_bytes(int mode) { return mode == DAX_ATTN_QK_I8_PV_F8 ? 1 : 2; }

// Fills `ws`; with base == nullptr only the size is computed.
inline int attn_workspace_layout(int64_t B, int64_t heads, int64_t Sq, int64_t Sk, int mode, void* base,
                                 size_t available, AttnWorkspace* ws) {
  DAX_REQUIRE(B > 0 && heads > 0 && Sq > 0 && Sk > 0, DAX_ERR_INVALID, "attention: bad shape B=%lld heads=%lld Sq=%lld Sk=%lld",
              (long long)B, (long long)heads, (long long)Sq, (long long)Sk);
  DAX_REQUIRE(mode == DAX_ATTN_QK_I8_PV_F8 || mode == DAX_ATTN_QK_BF16_PV_BF16 || mode == DAX_ATTN_QK_I8_PV_BF16,
              DAX_ERR_UNSUPPORTED, "attention: unknown mode %d", mode);
  const int64_t BH = B * heads;
  DAX_REQUIRE(BH <= 65535, DAX_ERR_UNSUPPORTED, "attention: batch*heads=%lld exceeds 65535", (long long)BH);
  const int eq = attn_qk_bytes(mode), ev = attn_pv_bytes(mode);
  ws->Sq_pad = round_up(Sq, 256);
  ws->Sk_pad = round_up(Sk, 128);
  ws->chunks = (Sk + kStatChunk - 1) / kStatChunk;
  DAX_REQUIRE(BH * ws->Sq_pad < (1ll << 31) && BH * ws->Sk_pad < (1ll << 31), DAX_ERR_UNSUPPORTED,
              "attention: batch*heads*sequence exceeds 2^31 rows");
  size_t off = 0;
  auto take = [&](size_t n) {
    size_t o = off;
    off += (n + 1023) / 1024 * 1024;
    return o;
  };
  uint8_t* b = static_cast<uint8_t*>(base);
  const size_t o_q = take(static_cast<size_t>(BH) * ws->Sq_pad * 128 * eq);
  const size_t o_k = take(static_cast<size_t>(BH) * ws->Sk_pad * 128 * eq);
  const size_t o_v = take(static_cast<size_t>(BH) * ws->Sk_pad * 128 * ev);
  const size_t o_qs = take(static_cast<size_t>(BH) * ws->Sq_pad * 4);
  const size_t o_ks = take(static_cast<size_t>(BH) * (ws->Sk_pad / 128) * 4);
  const size_t o_vs = take(static_cast<size_t>(BH) * 128 * 4);
  const size_t o_km = take(static_cast<size_t>(BH) * 128 * 4);
  const size_t o_pt = take(static_cast<size_t>(BH) * ws->chunks * 2 * 128 * 4);
  ws->bytes = off;
  if (base != nullptr) {
    DAX_REQUIRE((reinterpret_cast<uintptr_t>(base) & 1023u) == 0, DAX_ERR_ALIGN, "attention: workspace must be 1024-byte aligned");
    DAX_REQUIRE(available >= off, DAX_ERR_INVALID, "attention: workspace of %zu bytes is smaller than the %zu required", available, off);
    ws->q = b + o_q; ws->k = b + o_k; ws->vt = b + o_v;
    ws->q_scale = reinterpret_cast<float*>(b + o_qs);
    ws->k_scale = reinterpret_cast<float*>(b + o_ks);
    ws->v_scale = reinterpret_cast<float*>(b + o_vs);
    ws->k_mean = reinterpret_cast<float*>(b + o_km);
    ws->part = reinterpret_cast<float*>(b + o_pt);
  }
  return DAX_OK;
}

// bf16 Q.K^T + bf16 P.V with the probabilities kept in tensor memory (attn_tmem.cu)
int launch_attn_fwd_tmem_p(const AttnWorkspace& ws, const AttnParams& p, int64_t BH, cudaStream_t st);
// the same kernel reading Q, K, V in place: [BH, S, 128] with element strides (head, token), channels contiguous
int launch_attn_fwd_tmem_p_direct(const void* q, const void* k, const void* v, int64_t q_sh, int64_t q_st, int64_t k_sh,
                                  int64_t k_st, int64_t v_sh, int64_t v_st, const AttnParams& p, int64_t BH, cudaStream_t st);

}  // namespace dax
