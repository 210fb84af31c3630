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

#define KFB_LAUNCH_CHECK(what)                                                              \
  do {                                                                                      \
    cudaError_t _e = cudaGetLastError();                                                    \
    if (_e != cudaSuccess)                                                                  \
      return ::kfb::fail(KFB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(_e)); \
  } while (0)

}  // namespace kfb
