// One-call dynamic quantised linear: per-token quantiser followed by the tcgen05 GEMM with the
// de-quantisation epilogue, the two launches of dax.quant.nn.dynamic.Linear.forward
// (dax/quant/nn/dynamic/linear.py:143-228).  The quantised activations and their scales live in a
// workspace between the two launches: [M*K bytes, padded to 256][M floats].
#include "common.cuh"

#include <mutex>

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

// ---------------------------------------------------------------------------------------------
// Variant for callers that must not allocate device memory
// ---------------------------------------------------------------------------------------------
namespace dax {
namespace {

// The quantised activations and scales of dax_linear_dynamic_static live here instead of in a
// caller-provided workspace.  The array is part of the loaded module: every GPU that loads the
// library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_linear_static_scratch[DAX_LINEAR_STATIC_SCRATCH_BYTES];

// Device address of the array for the current device.  In host code the array's name is only a
// handle for the runtime, not a pointer a kernel could use, so the address is looked up once per
// device (with that device current) and cached.
int linear_static_scratch(void** out) {
  static std::mutex mu;
  static void* table[64] = {nullptr};
  int dev = 0;
  DAX_CUDA(cudaGetDevice(&dev));
  DAX_REQUIRE(dev >= 0 && dev < 64, DAX_ERR_UNSUPPORTED, "linear_dynamic_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] == nullptr) {
    void* p = nullptr;
    DAX_CUDA(cudaGetSymbolAddress(&p, g_linear_static_scratch));
    DAX_REQUIRE(p != nullptr, DAX_ERR_CUDA, "linear_dynamic_static: the scratch array has no device address");
    table[dev] = p;
  }
  *out = table[dev];
  return DAX_OK;
}

}  // namespace
}  // namespace dax

extern "C" int dax_linear_dynamic_static(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* qw,
                                         int w_dtype, int act_dtype, const float* sw, const void* bias,
                                         int bias_dtype, void* out, int out_dtype, int64_t N, int64_t ldo,
                                         void* stream) {
  using namespace dax;
  DAX_REQUIRE(M >= 0 && K > 0 && N > 0, DAX_ERR_INVALID, "linear_dynamic_static: bad shape M=%lld N=%lld K=%lld",
              (long long)M, (long long)N, (long long)K);
  const size_t need = dax_linear_dynamic_workspace_bytes(M, K);
  DAX_REQUIRE(need <= static_cast<size_t>(DAX_LINEAR_STATIC_SCRATCH_BYTES), DAX_ERR_UNSUPPORTED,
              "linear_dynamic_static: M=%lld x K=%lld needs %zu bytes of scratch, the built-in buffer holds %zu; "
              "use dax_linear_dynamic with your own workspace for larger problems",
              (long long)M, (long long)K, need, static_cast<size_t>(DAX_LINEAR_STATIC_SCRATCH_BYTES));
  if (M == 0) return DAX_OK;
  void* scratch = nullptr;
  int rc = linear_static_scratch(&scratch);
  if (rc != DAX_OK) return rc;
  // Nothing in the scratch has to start at zero: the quantiser writes all M*K codes and all M scales
  // before the GEMM reads them, so whatever an earlier call left behind is never observed.
  return linear_dynamic_impl(x, x_dtype, M, K, ldx, qw, w_dtype, act_dtype, sw, bias, bias_dtype, out, out_dtype, N, ldo,
                             scratch, stream);
}
