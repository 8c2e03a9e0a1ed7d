// Library-wide C entry points and host plumbing: version, error string, device status word,
// TMA descriptor creation through the driver entry point (no link-time dependency on libcuda).
#include "common.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace dax {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

__device__ int g_device_status = 0;

int* device_status_ptr() {
  // one address per device; devices are few, a small table under a mutex is enough
  static std::mutex mu;
  static int* table[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!table[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    table[dev] = static_cast<int*>(p);
  }
  return table[dev];
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

int make_tma_map(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box) {
  auto fn = encode_fn();
  DAX_REQUIRE(fn != nullptr, DAX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  DAX_REQUIRE(aligned16(base), DAX_ERR_ALIGN, "TMA base address must be 16-byte aligned");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      DAX_REQUIRE(strides_bytes[i] % 16 == 0, DAX_ERR_ALIGN, "TMA stride %d (%llu B) must be a multiple of 16",
                  i, (unsigned long long)strides_bytes[i]);
      gstr[i - 1] = strides_bytes[i];
    }
  }
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  CUresult r = fn(map, dt, rank, const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DAX_REQUIRE(r == CUDA_SUCCESS, DAX_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DAX_OK;
}

}  // namespace dax

extern "C" {

int dax_version(void) { return 100; }

const char* dax_last_error(void) { return dax::error_buffer(); }

int dax_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
  DAX_REQUIRE(dst != nullptr && src != nullptr, DAX_ERR_INVALID, "peer_copy: null pointer");
  if (bytes == 0) return DAX_OK;
  DAX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return DAX_OK;
}

int dax_device_status(int* host_status) {
  DAX_REQUIRE(host_status != nullptr, DAX_ERR_INVALID, "host_status is null");
  int* p = dax::device_status_ptr();
  DAX_REQUIRE(p != nullptr, DAX_ERR_CUDA, "cannot resolve the device status word");
  DAX_CUDA(cudaDeviceSynchronize());
  DAX_CUDA(cudaMemcpy(host_status, p, sizeof(int), cudaMemcpyDeviceToHost));
  DAX_CUDA(cudaMemset(p, 0, sizeof(int)));
  return DAX_OK;
}

}  // extern "C"
