// Host-side plumbing shared by every translation unit of the library: status codes, the
// thread-local error string, argument checks, the device status word and TMA descriptor creation.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../../include/dax_b200.h"

namespace dax {

// ---- error reporting ------------------------------------------------------------------------
char* error_buffer();  // thread-local, 512 bytes (defined in capi.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define DAX_REQUIRE(cond, code, ...) \
  do {                               \
    if (!(cond)) return ::dax::fail((code), __VA_ARGS__); \
  } while (0)

#define DAX_CUDA(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess)                                                                         \
      return ::dax::fail(DAX_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));            \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_bytes(int dt) {
  switch (dt) {
    case DAX_BF16: case DAX_F16: return 2;
    case DAX_F32: return 4;
    case DAX_I8: case DAX_E4M3: case DAX_E5M2: return 1;
    default: return 0;
  }
}

// ---- scattered column groups ------------------------------------------------------------------
// Several kernels write a [rows, N] matrix as column groups of `col_group` columns that live in separate slabs:
// element (t, n) goes to  out + off[n / col_group] + t * ld + (n % col_group)  (element units).  With n == 0 the
// slabs are equally spaced (off[g] = g * group_stride, any number of groups); with n > 0 the table gives the
// offset of every slab relative to `out`, which lets a slab sit anywhere in the address space, in particular in
// the memory of another GPU of the node (peer mapping): that is how the sequence<->head exchange of the
// sequence-parallel attention is written by the producing kernels themselves.
constexpr int kMaxGroups = 8;
struct GroupTable {
  int64_t off[kMaxGroups];
  int n;
};

// Fills `tab` (and the base pointer) from a host array of `n` device pointers; elem_bytes = size of one element.
inline int make_group_table(void* const* ptrs, int64_t n, int elem_bytes, GroupTable* tab, void** base) {
  DAX_REQUIRE(ptrs != nullptr && n >= 1 && n <= kMaxGroups, DAX_ERR_INVALID,
              "scatter: between 1 and %d group pointers are needed (got %lld)", kMaxGroups, (long long)n);
  for (int64_t g = 0; g < n; ++g) {
    DAX_REQUIRE(ptrs[g] != nullptr && aligned16(ptrs[g]), DAX_ERR_ALIGN, "scatter: group pointer %lld is null or not 16-byte aligned", (long long)g);
    tab->off[g] = (reinterpret_cast<intptr_t>(ptrs[g]) - reinterpret_cast<intptr_t>(ptrs[0])) / elem_bytes;
  }
  for (int64_t g = n; g < kMaxGroups; ++g) tab->off[g] = 0;
  tab->n = static_cast<int>(n);
  *base = ptrs[0];
  return DAX_OK;
}

// ---- device status word ---------------------------------------------------------------------
// Kernels store an error code into this word when a bounded wait gives up.  The word is a
// file-scope __device__ variable of capi.cu; kernels of other translation units get its address
// as an argument.  Returns nullptr if the address cannot be resolved.
int* device_status_ptr();

// ---- TMA descriptors ------------------------------------------------------------------------
// 2-D / 3-D tiled map over 1- or 2-byte elements with the 128-byte swizzle.  dims/strides in
// elements / bytes, innermost first (strides[0] is implied by the element size).
int make_tma_map(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box);

int sm_count();

}  // namespace dax
