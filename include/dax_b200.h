/*
 * dax_b200 — C ABI of the B200 (sm_100a) kernels behind DAX's Ulysses self-attention hot path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host".  The library never
 *     allocates or frees device memory and keeps no pointer after a call returns (the one
 *     documented exception owns a fixed file-scope buffer instead of allocating).
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises.
 *   - Every function returns a dax_status; dax_last_error() gives the message of the calling
 *     thread's last failure.  Shape / alignment / dtype problems are reported BEFORE any launch.
 *   - A kernel whose bounded device-side wait ran out raises the device status word, readable
 *     with dax_device_status() (that call synchronises).
 *   - Reference locations are given as path:line inside the RiseAI-Sys/DAX project.
 */
#ifndef DAX_B200_H_
#define DAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  DAX_OK = 0,
  DAX_ERR_INVALID = 1,     /* bad shape / null pointer / inconsistent arguments            */
  DAX_ERR_ALIGN = 2,       /* pointer or leading dimension not aligned as documented        */
  DAX_ERR_UNSUPPORTED = 3, /* dtype combination or size outside what the kernels implement  */
  DAX_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed                           */
  DAX_ERR_TIMEOUT = 5      /* device status: a bounded wait inside a kernel ran out         */
} dax_status;

typedef enum {
  DAX_BF16 = 0,
  DAX_F16 = 1,
  DAX_F32 = 2,
  DAX_I8 = 3,
  DAX_E4M3 = 4, /* float8_e4m3fn */
  DAX_E5M2 = 5
} dax_dtype;

/* Precision of the two tensor-core contractions of the attention kernel. */
typedef enum {
  DAX_ATTN_QK_I8_PV_F8 = 0,     /* INT8 Q.K^T, FP8(e4m3) P.V  — the SageAttention2-style mode                */
  DAX_ATTN_QK_BF16_PV_BF16 = 1, /* bf16 Q.K^T, bf16 P.V       — high-accuracy mode                           */
  DAX_ATTN_QK_I8_PV_BF16 = 2    /* INT8 Q.K^T, bf16 P.V       — V unquantised; P becomes bf16 by truncation,
                                    which costs the softmax warps less than the conversion to FP8        */
} dax_attn_mode;

int dax_version(void);
const char* dax_last_error(void);

/* Reads (and clears) the device status word of the current device: DAX_OK or DAX_ERR_TIMEOUT.
 * Synchronises the device.  `host_status` is a host pointer. */
int dax_device_status(int* host_status);

/* ---------------------------------------------------------------------------------------------
 * Per-token dynamic activation quantiser.
 * Replaces dax/quant/nn/dynamic/functional.py:54-148 (_dynamic_quantize_func, per_token_symmetric)
 * with dax/quant/nn/quantized/functional.py:11-20 (quantize_to_fp8 / quantize_to_int8).
 *
 * x is a logical [M, K] matrix of x_dtype (BF16 / F16 / F32).  Element (t, n) lives at
 *     x + (n / col_group) * group_stride + t * ldx + (n % col_group)        (in elements)
 * so that a matrix whose column groups sit in separate slabs (the receive buffer of the
 * head->sequence exchange, [P, s, h*d]) is read in place; pass col_group = K, group_stride = 0
 * for a plain row-major matrix.  q is [M, K] row-major of q_dtype (I8 / E4M3 / E5M2), scale is
 * [M] fp32.  Bit-exact with the reference: absmax and absmax/qmax in the input dtype, floor at
 * fp32 eps, INT8 = clamp(rint(x * (1/scale))), FP8 = round-to-nearest-even(x / scale).
 * K and col_group must be multiples of 16; x, q 16-byte aligned; ldx, group_stride multiples of 8.
 * ------------------------------------------------------------------------------------------- */
int dax_quant_rowwise(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int64_t col_group,
                      int64_t group_stride, void* q, int q_dtype, float* scale, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Quantised GEMM with fused de-quantisation:  out = cast((acc(qx . qw^T) * sx) * sw) + bias.
 * INT8 replaces dax/quant/nn/dynamic/linear.py:218-228 (int32 aten.mm, two fp32 scale multiplies
 * in that order, cast to the output dtype, bias added in the output dtype) — bit-exact.
 * FP8 replaces dax/quant/nn/dynamic/linear.py:155-173 (torch._scaled_mm, row-wise scales, fp32
 * accumulation, bias inside, one rounding to the output dtype).
 *
 *   qx [M, K] row-major, a_dtype I8 | E4M3 | E5M2      sx [M] fp32
 *   qw [N, K] row-major, b_dtype I8 | E4M3 | E5M2      sw [N] fp32
 *   bias [N] of bias_dtype (BF16/F16/F32) or NULL
 *   out: element (t, n) at out + (n / out_col_group) * out_group_stride + t * ldo + (n % out_col_group)
 *        of out_dtype (BF16/F16/F32); out_col_group = N, out_group_stride = 0 for a plain matrix.
 *        With out_col_group = h*d and out_group_stride = s*h*d the projection writes straight into
 *        the send buffer [P, s, h, d] of the sequence->head exchange
 *        (dax/parallel/patches/wanx2_1_t2v_opt/layer.py:35-42,113-120).
 *   row_sumsq: optional [M, 2*ceil(N/256)] fp32; slot (t, j) receives the sum of squares of the
 *        rounded outputs of row t in columns [128 j, 128 j + 128) (feeds the RMSNorm that follows a
 *        Q/K projection).
 *   acc_dump: optional [M, N] int32 (INT8) / fp32 (FP8) raw accumulators, for parity tests.
 * K % 16 == 0, N % 8 == 0, out_col_group % 32 == 0 (or == N), pointers 16-byte aligned.
 * The reference's float fallback for M <= 16 (linear.py:186-202) does not exist here.
 * ------------------------------------------------------------------------------------------- */
int dax_gemm_dequant(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype,
                     const float* sw, const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M,
                     int64_t N, int64_t K, int64_t ldo, int64_t out_col_group, int64_t out_group_stride,
                     float* row_sumsq, void* acc_dump, void* stream);

/* dax_gemm_dequant with an epilogue for the rest of the DiT block (16-bit outputs only).  With y the
 * rounded linear output:  act = 1: y <- gelu_tanh(y) (the FFN's first linear);  resid != NULL:
 * out[t, n] = resid[t, n] + gate[n] * y (fp32, rounded once; gate NULL = 1): the gated residual that
 * follows the O projection and the FFN's second linear in a Wan block.  resid is [M, N] (ldr) of out_dtype
 * and may alias out.  Everything else as dax_gemm_dequant. */
int dax_gemm_dequant_ex(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype,
                        const float* sw, const void* bias, int bias_dtype, void* out, int out_dtype, int64_t M,
                        int64_t N, int64_t K, int64_t ldo, int64_t out_col_group, int64_t out_group_stride,
                        float* row_sumsq, void* acc_dump, int act, const void* resid, int64_t ldr,
                        const float* gate, void* stream);

/* dax_gemm_dequant whose output column groups sit at unrelated addresses: group g (columns [g * out_col_group,
 * (g + 1) * out_col_group)) of row t is written at group_out[g] + t * ldo.  group_out is a HOST array of n_groups =
 * N / out_col_group (at most 8) device pointers, each 16-byte aligned.  A pointer may be the peer mapping of another
 * GPU's buffer: the V projection of the sequence-parallel block then writes each rank's head group straight into that
 * rank's receive buffer, which is the sequence->head exchange of
 * dax/parallel/patches/wanx2_1_t2v_opt/layer.py:181-222 done by the producing kernel (plain stores over NVLink, no
 * collective call, no pack / unpack copy). */
int dax_gemm_dequant_scatter(const void* qx, int a_dtype, const float* sx, const void* qw, int b_dtype,
                             const float* sw, const void* bias, int bias_dtype, void* const* group_out,
                             int64_t n_groups, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldo,
                             int64_t out_col_group, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One-call dynamic quantised linear = dax_quant_rowwise followed by dax_gemm_dequant, i.e. the whole of
 * dax.quant.nn.dynamic.Linear.forward (dax/quant/nn/dynamic/linear.py:143-228) for a plain row-major
 * x [M, K] (ldx) and out [M, N] (ldo).  The quantised activations and their scales sit in `workspace`
 * (256-byte aligned, at least dax_linear_dynamic_workspace_bytes(M, K)) between the two launches.
 * act_dtype: I8 with I8 weights, E4M3 / E5M2 with FP8 weights (w_dtype).
 * ------------------------------------------------------------------------------------------- */
size_t dax_linear_dynamic_workspace_bytes(int64_t M, int64_t K);

int dax_linear_dynamic(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* qw, int w_dtype,
                       int act_dtype, const float* sw, const void* bias, int bias_dtype, void* out, int out_dtype,
                       int64_t N, int64_t ldo, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * dax_linear_dynamic for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Some hosts of this library hand it nothing but their input and output buffers and are
 * not allowed to call cudaMalloc on the path that runs the layer: a serving runtime whose memory pool
 * is carved up at start-up, a binding from another language that owns no CUDA allocator, code that
 * runs where an allocation would stall every stream of the device.  For them the quantised
 * activations and scales go to a fixed buffer that is part of the library image instead of a
 * workspace argument.
 *   - Limit: dax_linear_dynamic_workspace_bytes(M, K) <= DAX_LINEAR_STATIC_SCRATCH_BYTES (8 MiB; e.g.
 *     the 512 x 4096 text-context projections, or 1024 rows of a 5120-wide layer).  Larger problems
 *     are rejected with DAX_ERR_UNSUPPORTED and a message; nothing is launched.
 *   - Cost: every GPU that loads the library keeps those 8 MiB until the process exits.
 *   - The first call on each device looks up the buffer's device address (no allocation); make that
 *     first call before starting any stream capture.
 *   - All calls on a device share the one buffer.  Calls that may run at the same time on the GPU
 *     (different streams) race on it: keep them on one stream or order them with events.  The buffer
 *     keeps the previous call's bytes; the entry point never relies on its contents.
 *   - The call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
 * Arguments as dax_linear_dynamic, without the workspace.
 * ------------------------------------------------------------------------------------------- */
#define DAX_LINEAR_STATIC_SCRATCH_BYTES (8u << 20)

int dax_linear_dynamic_static(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* qw,
                              int w_dtype, int act_dtype, const float* sw, const void* bias, int bias_dtype,
                              void* out, int out_dtype, int64_t N, int64_t ldo, void* stream);

/* ---------------------------------------------------------------------------------------------
 * RMSNorm over the full hidden dimension + 3-D rotary embedding + pack into the exchange layout.
 * Replaces the norm_q / norm_k call sites (dax/adapters/wan/attn_adapter.py:82-85,108-109,121-122),
 * apply_rotary_emb (attn_adapter.py:164-173; the reference rotates after the exchange, which is
 * the same per-token, per-head operation) and the pack copy of the exchange
 * (dax/parallel/patches/wanx2_1_t2v_opt/layer.py:113-120).
 *
 *   x [s, D] row-major (ldx), dtype BF16/F16; D = heads * 128.
 *   row_sumsq: NULL (the kernel reduces each row itself) or [s, n_partials] fp32 partial sums of
 *              squares written by dax_gemm_dequant; norm_weight [D] of x's dtype or NULL (no norm:
 *              pass NULL weight and do_norm = 0).
 *   rope_cos, rope_sin: [S_total, 64] fp32 tables (row = global token index), or NULL for no
 *              rotation; token_offset = global index of local token 0.
 *   out: element (t, n) at out + (n / col_group) * group_stride + t * ldo + (n % col_group).
 * ------------------------------------------------------------------------------------------- */
int dax_rmsnorm_rope_pack(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx, const float* row_sumsq,
                          int64_t n_partials, int do_norm, const void* norm_weight, float eps,
                          const float* rope_cos, const float* rope_sin, int64_t token_offset, void* out,
                          int64_t ldo, int64_t col_group, int64_t group_stride, void* stream);

/* dax_rmsnorm_rope_pack with scattered output groups (see dax_gemm_dequant_scatter): column group g of row t goes
 * to group_out[g] + t * ldo; the Q and K halves of the same exchange
 * (dax/adapters/wan/attn_adapter.py:112-130 -> layer.py:181-222). */
int dax_rmsnorm_rope_pack_scatter(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx, const float* row_sumsq,
                                  int64_t n_partials, int do_norm, const void* norm_weight, float eps,
                                  const float* rope_cos, const float* rope_sin, int64_t token_offset,
                                  void* const* group_out, int64_t n_groups, int64_t ldo, int64_t col_group,
                                  void* stream);

/* ---------------------------------------------------------------------------------------------
 * LayerNorm + adaLN modulation (+ per-token quantisation): the step in front of every quantised linear
 * of a Wan DiT block outside the attention itself (the block is diffusers code called from
 * dax/adapters/wan/transformer_adapter.py:127-134; the quantiser it absorbs is
 * dax/quant/nn/dynamic/functional.py:54-148).
 *   y = round_dtype( LN(x; eps) [* ln_weight + ln_bias] [* (1 + scale) + shift] )      per token row
 *   (q, qscale) = per-token dynamic quantisation of y (bit-exact with dax_quant_rowwise applied to y)
 * x [s, D] (ldx) BF16/F16; ln_weight, ln_bias, shift, scale: [D] fp32 or NULL; y [s, D] (ldy) or NULL;
 * q [s, D] of q_dtype + qscale [s] or NULL (at least one output).  D % 8 == 0, D <= 8192.
 * ------------------------------------------------------------------------------------------- */
int dax_layernorm_modulate_quant(const void* x, int dtype, int64_t s, int64_t D, int64_t ldx,
                                 const float* ln_weight, const float* ln_bias, const float* shift,
                                 const float* scale, float eps, void* y, int64_t ldy, void* q, int q_dtype,
                                 float* qscale, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Quantised non-causal attention (replaces the attention dispatch at
 * dax/adapters/wan/attn_adapter.py:198-229, i.e. sageattn_qk_int8_pv_fp8_cuda_sm90 / SDPA).
 *
 * q, k, v, o: [B, heads, S, 128] addressed by element strides (batch, head, token); the last
 * dimension is contiguous; dtype BF16 or F16.  Sq may differ from Sk.
 * Two steps share a caller-provided workspace (dax_attn_workspace_bytes):
 *   dax_attn_prepare   K: per-(batch, head, channel) mean over the sequence removed, then INT8 per
 *                      block of 128 tokens (or bf16); Q: softmax scale folded in, INT8 per token (or
 *                      bf16); V: FP8 e4m3 with a per-channel scale, stored transposed (or bf16).
 *   dax_attn_forward   flash-style pass over the prepared operands for the query rows
 *                      [q_begin + r*range_stride, q_end + r*range_stride), r = 0 .. n_ranges-1
 *                      (one call per O-path micro-batch: the i-th slice of every destination rank's
 *                      token block, dax/parallel/patches/wanx2_1_t2v_opt/micro_batch_layer.py:14-29);
 *                      n_ranges = 1, q_begin = 0, q_end = Sq for all queries.
 * sm_scale: softmax scale (1/sqrt(128) in the reference).
 * ------------------------------------------------------------------------------------------- */
size_t dax_attn_workspace_bytes(int64_t B, int64_t heads, int64_t Sq, int64_t Sk, int mode);

int dax_attn_prepare(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                     int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3], int64_t v_strides[3],
                     float sm_scale, int mode, void* workspace, size_t workspace_bytes, void* stream);

/* dax_attn_prepare in two parts, for callers whose K and V are complete before Q is (the sequence-parallel block:
 * the K / V statistics and operand passes run while the last Q rows are still in flight between the GPUs):
 * DAX_ATTN_PREPARE_KV = statistics + K + V operands, DAX_ATTN_PREPARE_Q = Q operands; q may be NULL-free but is not
 * read by the KV part, k and v are not read by the Q part. */
#define DAX_ATTN_PREPARE_KV 1
#define DAX_ATTN_PREPARE_Q 2
int dax_attn_prepare_parts(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                           int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3], int64_t v_strides[3],
                           float sm_scale, int mode, int parts, void* workspace, size_t workspace_bytes, void* stream);

int dax_attn_forward(void* o, int dtype, int64_t B, int64_t heads, int64_t Sq, int64_t Sk, int64_t o_strides[3],
                     int64_t q_begin, int64_t q_end, int64_t n_ranges, int64_t range_stride, int mode,
                     void* workspace, size_t workspace_bytes, void* stream);

/* One contiguous device-to-device copy on `stream`, carried out by the GPU's copy engines (no SM is used, so it
 * runs beside compute kernels).  dst or src may be the peer mapping of another GPU's buffer: this is the transport of
 * the Q / K / V half of the sequence->head exchange when it overlaps the next projection (the slab a rank produced
 * for rank p, [s, h*d] contiguous, goes to rows [rank*s, (rank+1)*s) of rank p's receive buffer); it stands where
 * the reference calls all_to_all_single (dax/parallel/patches/wanx2_1_t2v_opt/layer.py:123-132). */
int dax_peer_copy(void* dst, const void* src, size_t bytes, void* stream);

/* dax_attn_forward (batch 1) whose result rows are scattered by destination: query row q belongs to destination
 * q / rows_per_dest and is written, for head h, at  o_dest[q / rows_per_dest] + (q % rows_per_dest) * token_stride +
 * h * head_stride  (elements).  o_dest is a HOST array of n_dest (at most 8) device pointers.  With destination d =
 * rank d's receive buffer (peer mapping) this is the head->sequence exchange in front of the O projection
 * (dax/adapters/wan/attn_adapter.py:241-300, layer.py:13-29) written by the attention kernel's own epilogue. */
int dax_attn_forward_scatter(void* const* o_dest, int64_t n_dest, int64_t rows_per_dest, int dtype, int64_t heads,
                             int64_t Sq, int64_t Sk, int64_t head_stride, int64_t token_stride, int64_t q_begin,
                             int64_t q_end, int mode, void* workspace, size_t workspace_bytes, void* stream);

/* The 16-bit attention (bf16 Q.K^T and P.V, the mode that stays within rel-L2 1e-2 of fp32 SDPA) in ONE call,
 * reading q, k, v in place: no prepare step, no workspace.  dtype BF16 only, Sq and Sk at least 128 (anything else:
 * DAX_ERR_UNSUPPORTED, use dax_attn_prepare + dax_attn_forward).  The kernel's TMA maps address the [B, heads, S, 128] views
 * directly (batch stride = heads x head stride, or B = 1), V is consumed as stored (its tile is the MN-major operand of
 * P.V), K is not mean-smoothed (smoothing serves the INT8 range; softmax is invariant to it).  Replaces the dispatch at
 * dax/adapters/wan/attn_adapter.py:198-229 like dax_attn_forward.  Output either to o (strides as in dax_attn_forward,
 * with query ranges) or, with n_dest > 0, scattered by destination as in dax_attn_forward_scatter (o_strides[1] /
 * o_strides[2] = head / token stride inside a destination; o may be NULL). */
int dax_attn_forward_direct(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t heads,
                            int64_t Sq, int64_t Sk, int64_t q_strides[3], int64_t k_strides[3], int64_t v_strides[3],
                            float sm_scale, void* o, int64_t o_strides[3], void* const* o_dest, int64_t n_dest,
                            int64_t rows_per_dest, int64_t q_begin, int64_t q_end, int64_t n_ranges,
                            int64_t range_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DAX_B200_H_ */
