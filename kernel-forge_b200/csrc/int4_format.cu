// INT4 weight format on the GPU: quantise+pack, pack, unpack, dequantise.
//
// Bit-exact with the torch implementation of the reference (kernelforge/quantize.py:61-114):
// every step is an IEEE fp32 operation (division, rint = round-half-to-even, one RN to fp16),
// so no fast-math flag may be applied to this file.  The kernels stream the weight once
// (HBM-bound: 4 B read + 0.52 B written per weight for fp32 input).
#include "common.cuh"

namespace kfb {
namespace {

// nibble position (bits 4p..4p+3) of k-offset o inside its 8-weight word:
// positions 0..7 hold offsets 0,2,4,6,1,3,5,7 (kernelforge/quantize.py:34).
__device__ __forceinline__ int nibble_pos(int o) { return (o >> 1) + ((o & 1) << 2); }

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One warp quantises 128 consecutive k of one row per step: lane l owns k = 4l .. 4l+3.
// For G = 128 the warp is one group; for G = 64 each half-warp is one group.
// Grid-stride over the N * K/128 warp-steps.
template <typename T, int G>
__global__ void __launch_bounds__(256) quantize_pack_kernel(const T* __restrict__ w, int32_t* __restrict__ packed,
                                                            __half* __restrict__ scales, int N, int K) {
  const int lane = threadIdx.x & 31;
  const long long steps_per_row = (K + 127) / 128;  // K % 128 == 64 is possible when G = 64
  const long long total = (long long)N * steps_per_row;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long step = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); step < total; step += warps) {
    const long long row = step / steps_per_row;
    const int k0 = (int)(step - row * steps_per_row) * 128;
    const bool live = k0 + 4 * lane < K;  // a whole group is live or not (G divides K)
    const T* src = w + row * K + k0 + 4 * lane;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = live ? to_f32<T>(src[i]) : 0.0f;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    constexpr int kWidth = G / 4;  // lanes per group: 32 or 16
#pragma unroll
    for (int off = kWidth / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    // scale = fp16(max(absmax / 7, smallest normal fp16)); exactly 1 for an all-zero group
    float s = fmaxf(__fdiv_rn(amax, 7.0f), 6.103515625e-05f);
    __half sh = __float2half_rn(s);
    if (amax == 0.0f) sh = __float2half_rn(1.0f);
    const float s32 = __half2float(sh);
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float q = rintf(__fdiv_rn(v[i], s32));
      q = fminf(fmaxf(q, -8.0f), 7.0f);
      const uint32_t u = (uint32_t)((int)q + 8) & 0xFu;
      const int o = (lane & 1) * 4 + i;  // k offset inside the 8-weight word
      word |= u << (4 * nibble_pos(o));
    }
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    if (live && (lane & 1) == 0) packed[row * (K / 8) + k0 / 8 + (lane >> 1)] = (int32_t)word;
    if (live && (lane & (kWidth - 1)) == 0) scales[row * (K / G) + k0 / G + lane / kWidth] = sh;
  }
}

// One thread per packed word.
__global__ void __launch_bounds__(256) unpack_kernel(const uint32_t* __restrict__ packed, int8_t* __restrict__ q,
                                                     long long words) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words;
       i += (long long)gridDim.x * blockDim.x) {
    const uint32_t w = packed[i];
    uint32_t lo = 0, hi = 0;  // bytes k0..k3, k4..k7
#pragma unroll
    for (int o = 0; o < 8; ++o) {
      const uint32_t b = (((w >> (4 * nibble_pos(o))) & 0xFu) - 8u) & 0xFFu;
      if (o < 4) lo |= b << (8 * o); else hi |= b << (8 * (o - 4));
    }
    reinterpret_cast<uint2*>(q)[i] = make_uint2(lo, hi);
  }
}

__global__ void __launch_bounds__(256) pack_kernel(const int8_t* __restrict__ q, uint32_t* __restrict__ packed,
                                                   long long words) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words;
       i += (long long)gridDim.x * blockDim.x) {
    const uint2 b = reinterpret_cast<const uint2*>(q)[i];
    uint32_t w = 0;
#pragma unroll
    for (int o = 0; o < 8; ++o) {
      const uint32_t byte = ((o < 4 ? b.x : b.y) >> (8 * (o & 3))) & 0xFFu;
      w |= ((byte + 8u) & 0xFu) << (4 * nibble_pos(o));
    }
    packed[i] = w;
  }
}

// One thread per packed word; writes 8 consecutive outputs.
template <typename OutT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint32_t* __restrict__ packed,
                                                         const __half* __restrict__ scales, OutT* __restrict__ out,
                                                         int N, int K, int G) {
  const long long words = (long long)N * (K / 8);
  const int wpr = K / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / wpr;
    const int j = (int)(i - row * wpr);
    const uint32_t w = packed[i];
    const __half sh = scales[row * (K / G) + (j * 8) / G];
    __align__(16) OutT vals[8];
#pragma unroll
    for (int o = 0; o < 8; ++o) {
      const int qv = (int)((w >> (4 * nibble_pos(o))) & 0xFu) - 8;
      if constexpr (sizeof(OutT) == 2) {
        vals[o] = __hmul(__int2half_rn(qv), sh);  // one fp16 multiply, as the reference's fp16 path
      } else {
        vals[o] = __fmul_rn((float)qv, __half2float(sh));
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + row * K + (long long)j * 8);
    const uint4* srcv = reinterpret_cast<const uint4*>(vals);
#pragma unroll
    for (int t = 0; t < (int)(sizeof(OutT) * 8 / 16); ++t) dst[t] = srcv[t];
  }
}

int check_format_args(const void* a, const void* b, int N, int K) {
  if (N < 1 || K < 8 || (K % 8) != 0) return fail(KFB_ERR_INVALID, "need N >= 1 and K a positive multiple of 8, got N=%d K=%d", N, K);
  if (!a || !b) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(a) || !aligned16(b)) return fail(KFB_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  return KFB_OK;
}

int grid_for(long long items, int per_block) {
  long long blocks = (items + per_block - 1) / per_block;
  long long cap = (long long)sm_count() * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace kfb

using namespace kfb;

extern "C" int kfb_quantize_pack(const void* w, int w_dtype, int N, int K, int group, void* packed, void* scales,
                                 void* stream) {
  if (int rc = require_sm100()) return rc;
  if (group != 64 && group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", group);
  if (N < 1 || K < group || K % group) return fail(KFB_ERR_INVALID, "K=%d is not a multiple of group_size=%d", K, group);
  if (!w || !packed || !scales) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(w) || !aligned16(packed)) return fail(KFB_ERR_ALIGNMENT, "w and packed must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const long long steps = (long long)N * ((K + 127) / 128);
  const int grid = grid_for(steps, 8);
#define KFB_Q(T, G) quantize_pack_kernel<T, G><<<grid, 256, 0, s>>>((const T*)w, (int32_t*)packed, (__half*)scales, N, K)
  if (w_dtype == KFB_F32) { if (group == 128) KFB_Q(float, 128); else KFB_Q(float, 64); }
  else if (w_dtype == KFB_F16) { if (group == 128) KFB_Q(__half, 128); else KFB_Q(__half, 64); }
  else if (w_dtype == KFB_BF16) { if (group == 128) KFB_Q(__nv_bfloat16, 128); else KFB_Q(__nv_bfloat16, 64); }
  else return fail(KFB_ERR_INVALID, "w_dtype must be KFB_F16, KFB_BF16 or KFB_F32");
#undef KFB_Q
  KFB_LAUNCH_CHECK("quantize_pack_kernel");
  return KFB_OK;
}

extern "C" int kfb_unpack_int4(const void* packed, int N, int K, void* q_out, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_format_args(packed, q_out, N, K)) return rc;
  const long long words = (long long)N * (K / 8);
  unpack_kernel<<<grid_for(words, 256), 256, 0, (cudaStream_t)stream>>>((const uint32_t*)packed, (int8_t*)q_out, words);
  KFB_LAUNCH_CHECK("unpack_kernel");
  return KFB_OK;
}

extern "C" int kfb_pack_int4(const void* q, int N, int K, void* packed, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_format_args(q, packed, N, K)) return rc;
  const long long words = (long long)N * (K / 8);
  pack_kernel<<<grid_for(words, 256), 256, 0, (cudaStream_t)stream>>>((const int8_t*)q, (uint32_t*)packed, words);
  KFB_LAUNCH_CHECK("pack_kernel");
  return KFB_OK;
}

extern "C" int kfb_dequantize(const void* packed, const void* scales, int N, int K, int group, void* out,
                              int out_dtype, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_format_args(packed, out, N, K)) return rc;
  if (group != 64 && group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", group);
  if (K % group) return fail(KFB_ERR_INVALID, "K=%d is not a multiple of group_size=%d", K, group);
  if (!scales) return fail(KFB_ERR_INVALID, "null pointer");
  const long long words = (long long)N * (K / 8);
  const int grid = grid_for(words, 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == KFB_F16)
    dequantize_kernel<__half><<<grid, 256, 0, s>>>((const uint32_t*)packed, (const __half*)scales, (__half*)out, N, K, group);
  else if (out_dtype == KFB_F32)
    dequantize_kernel<float><<<grid, 256, 0, s>>>((const uint32_t*)packed, (const __half*)scales, (float*)out, N, K, group);
  else
    return fail(KFB_ERR_INVALID, "out_dtype must be KFB_F16 or KFB_F32");
  KFB_LAUNCH_CHECK("dequantize_kernel");
  return KFB_OK;
}
