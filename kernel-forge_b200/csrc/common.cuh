// Shared host-side helpers of the kfb200 library: status codes, per-thread error text,
// argument checks.  No torch, no exceptions across the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/kfb200.h"

namespace kfb {

// Per-thread message buffer behind kfb_last_error().
char* error_buffer();
constexpr int kErrorBufferBytes = 512;

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), kErrorBufferBytes, fmt, ap);
  va_end(ap);
  return code;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device id).
int sm_count();
// KFB_OK when the current device is compute capability 10.x.
int require_sm100();

#define KFB_CUDA_TRY(expr)                                                                  \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess)                                                                  \
      return ::kfb::fail(KFB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                         __FILE__, __LINE__);                                               \
  } while (0)

// Programmatic dependent launch.  A kernel launched with the attribute may become resident while the kernel in front
// of it in the stream is still running; it must call pdl_wait() before it touches anything that kernel wrote (or
// still reads), and it releases its own successor with pdl_launch_dependents().  Every kernel of this library that
// can be part of a decode step waits first and releases its successor right after, so at most two grids overlap and
// the order of all memory operations is that of the plain stream.  Both instructions are no-ops in a kernel that
// was launched without the attribute.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif
// Whether launches carry the attribute (kfb_set_programmatic_launch; off by default).
bool pdl_enabled();

template <class... KArgs, class... Args>
int launch_kernel(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) return fail(KFB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return KFB_OK;
}

#define KFB_LAUNCH_CHECK(what)                                                              \
  do {                                                                                      \
    cudaError_t _e = cudaGetLastError();                                                    \
    if (_e != cudaSuccess)                                                                  \
      return ::kfb::fail(KFB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(_e)); \
  } while (0)

}  // namespace kfb

// ---- per-device status word and TMA tensor maps (api.cu) ------------------------------------
#include <cuda.h>
namespace kfb {
// Device address of the status word kernels write when a bounded wait expires (0 = fine).
// The first call on a device resolves the symbol address; returns nullptr on failure.
unsigned int* device_status_word();
// Tiled 4-D tensor map with 128-byte swizzle over a 16-bit element tensor.
// dims[0] is the innermost (dense) extent; strides_bytes[i] is the stride of dims[i+1].
int make_tmap_4d_sw128(CUtensorMap* out, const void* base, int dtype, const uint64_t dims[4],
                       const uint64_t strides_bytes[3], const uint32_t box[4]);
// Tiled 2-D tensor map over 32-bit elements (the packed INT4 words), without swizzle or with the 128-byte swizzle
// (box_inner <= 32 elements then).
int make_tmap_2d_plain(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                       uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128 = false);
}  // namespace kfb
