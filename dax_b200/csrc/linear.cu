// One-call dynamic quantised linear: per-token quantiser followed by the tcgen05 GEMM with the
// de-quantisation epilogue, the two launches of dax.quant.nn.dynamic.Linear.forward
// (dax/quant/nn/dynamic/linear.py:143-228).  The quantised activations and their scales live in a
// workspace between the two launches: [M*K bytes, padded to 256][M floats].
#include "common.cuh"

namespace dax {

inline size_t linear_ws_q_bytes(int64_t M, int64_t K) {
  return (static_cast<size_t>(M) * static_cast<size_t>(K) + 255) / 256 * 256;
}

int linear_dynamic_impl(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* qw, int w_dtype,
                        int act_dtype, const float* sw, const void* bias, int bias_dtype, void* out, int out_dtype,
                        int64_t N, int64_t ldo, void* workspace, void* stream) {
  uint8_t* qx = static_cast<uint8_t*>(workspace);
  float* sx = reinterpret_cast<float*>(qx + linear_ws_q_bytes(M, K));
  int rc = dax_quant_rowwise(x, x_dtype, M, K, ldx, K, 0, qx, act_dtype, sx, stream);
  if (rc != DAX_OK) return rc;
  return dax_gemm_dequant(qx, act_dtype, sx, qw, w_dtype, sw, bias, bias_dtype, out, out_dtype, M, N, K, ldo, N, 0,
                          nullptr, nullptr, stream);
}

}  // namespace dax

extern "C" size_t dax_linear_dynamic_workspace_bytes(int64_t M, int64_t K) {
  if (M < 0 || K <= 0) return 0;
  return dax::linear_ws_q_bytes(M, K) + static_cast<size_t>(M) * sizeof(float);
}

extern "C" int dax_linear_dynamic(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* qw,
                                  int w_dtype, int act_dtype, const float* sw, const void* bias, int bias_dtype,
                                  void* out, int out_dtype, int64_t N, int64_t ldo, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  using namespace dax;
  DAX_REQUIRE(M >= 0 && K > 0 && N > 0, DAX_ERR_INVALID, "linear_dynamic: bad shape M=%lld N=%lld K=%lld", (long long)M,
              (long long)N, (long long)K);
  if (M == 0) return DAX_OK;
  DAX_REQUIRE(workspace != nullptr, DAX_ERR_INVALID, "linear_dynamic: workspace is null");
  DAX_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, DAX_ERR_ALIGN, "linear_dynamic: workspace must be 256-byte aligned");
  DAX_REQUIRE(workspace_bytes >= dax_linear_dynamic_workspace_bytes(M, K), DAX_ERR_INVALID,
              "linear_dynamic: workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
              dax_linear_dynamic_workspace_bytes(M, K));
  return linear_dynamic_impl(x, x_dtype, M, K, ldx, qw, w_dtype, act_dtype, sw, bias, bias_dtype, out, out_dtype, N, ldo,
                             workspace, stream);
}
