// Small fused kernels around the two hot paths in a decode step of a Llama-architecture model.
//
// The reference leaves these operations to Hugging Face / torch (RMSNorm, rotary embedding, KV-cache
// write, SiLU * up, residual add: kernelforge/modules.py swaps only the linears and the attention
// function), which costs ~45 tiny kernels per layer.  At batch 1 a decode step is launch-bound (631 MB
// per token are 0.1 ms of HBM time), so the step is cut to 11 kernels per layer with three fused
// element-wise kernels.  All three are HBM / latency trivial; they exist to remove launches.
//
// Rounding follows what the torch formulation does in fp16 models, so results track the unfused path:
//   add_rmsnorm : s = fp16(x + r);  y = fp16( fp16(s * rsqrt(mean(s^2) + eps)) * w )
//   rope        : fp16( t * cos + rotate_half(t) * sin ) computed in FP32
//   silu_mul    : fp16( fp16(silu(g)) * u )
#include "common.cuh"

namespace kfb {
namespace fused {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// One CTA (256 threads) per row.  hidden % 8 == 0, hidden <= 256 * 8 * kMaxVec.
constexpr int kRmsThreads = 256;
constexpr int kMaxVec = 4;  // 16-byte vectors per thread => hidden <= 8192

__global__ void __launch_bounds__(kRmsThreads)
add_rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ res, const __half* __restrict__ w,
                   __half* __restrict__ y, __half* __restrict__ sum_out, int hidden, float eps) {
  __shared__ float warp_part[kRmsThreads / 32];
  const int nvec = hidden / 8;
  // The norm weight is a constant of the model (and cold in HBM: every layer has its own): it is requested before the
  // wait for the kernel in front, so its round trip overlaps that kernel's tail instead of following the reduction.
  uint4 wreg[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kRmsThreads;
    if (v < nvec) wreg[i] = reinterpret_cast<const uint4*>(w)[v];
  }
  pdl_wait();
  pdl_launch_dependents();
  const size_t base = (size_t)blockIdx.x * hidden;
  __half2 vals[kMaxVec][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kRmsThreads;
    if (v < nvec) {
      uint4 a = reinterpret_cast<const uint4*>(x + base)[v];
      __half2* ah = reinterpret_cast<__half2*>(&a);
      if (res) {
        uint4 b = reinterpret_cast<const uint4*>(res + base)[v];
        const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
        for (int j = 0; j < 4; ++j) ah[j] = __hadd2(ah[j], bh[j]);
        if (sum_out) reinterpret_cast<uint4*>(sum_out + base)[v] = a;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        vals[i][j] = ah[j];
        const float2 f = __half22float2(ah[j]);
        ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kRmsThreads / 32; ++i) tot += warp_part[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kRmsThreads;
    if (v < nvec) {
      const __half2* wh = reinterpret_cast<const __half2*>(&wreg[i]);
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(vals[i][j]);
        oh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
      }
      reinterpret_cast<uint4*>(y + base)[v] = o;
    }
  }
}

constexpr unsigned int kStatusRopePosition = 0x701;  // rope_kv_write: position outside [0, Lmax)

// grid (H + 2 Hk, B), D / 2 threads.  qkv: [B, (H + 2 Hk) * D] = q heads, k heads, v heads.
__global__ void rope_kv_write_kernel(const __half* __restrict__ qkv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const long long* __restrict__ pos_ptr,
                                     __half* __restrict__ q_out, __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                     int H, int Hk, int D, int Lmax, unsigned int* status) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x, half = D / 2;
  pdl_wait();
  pdl_launch_dependents();
  const long long pos = pos_ptr[0];
  // The position comes from device memory (a graph replay advances it), so it is checked here: a position outside
  // the cache / the rotary tables writes nothing and reads nothing, and leaves a code in the device status word.
  if (pos < 0 || pos >= Lmax) {
    if (threadIdx.x == 0 && head == 0 && b == 0) atomicCAS(status, 0u, kStatusRopePosition);
    return;
  }
  const __half* src = qkv + ((size_t)b * (H + 2 * Hk) + head) * D;
  if (head < H + Hk) {
    const float lo = __half2float(src[d]), hi = __half2float(src[d + half]);
    const float c0 = cos_t[pos * D + d], s0 = sin_t[pos * D + d];
    const float c1 = cos_t[pos * D + d + half], s1 = sin_t[pos * D + d + half];
    // separate FP32 roundings of both products and of the sum (no contraction), like the torch formulation
    // t * cos + rotate_half(t) * sin; the GEMV epilogue that replaces this kernel at batch <= 2 does the same
    const __half rlo = __float2half_rn(__fsub_rn(__fmul_rn(lo, c0), __fmul_rn(hi, s0)));
    const __half rhi = __float2half_rn(__fadd_rn(__fmul_rn(hi, c1), __fmul_rn(lo, s1)));
    __half* dst = head < H ? q_out + ((size_t)b * H + head) * D
                           : k_cache + (((size_t)b * Hk + (head - H)) * Lmax + pos) * D;
    dst[d] = rlo;
    dst[d + half] = rhi;
  } else {
    __half* dst = v_cache + (((size_t)b * Hk + (head - H - Hk)) * Lmax + pos) * D;
    dst[d] = src[d];
    dst[d + half] = src[d + half];
  }
}

// gu: [rows, 2 * inter] (gate | up) -> out [rows, inter]
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ out, int rows, int inter) {
  const int per_row = inter / 2;  // half2 per row
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)rows * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i - r * per_row);
    const __half2 g = reinterpret_cast<const __half2*>(gu + r * 2 * inter)[c];
    const __half2 u = reinterpret_cast<const __half2*>(gu + r * 2 * inter + inter)[c];
    const float2 gf = __half22float2(g);
    const __half2 s = __floats2half2_rn(gf.x / (1.0f + __expf(-gf.x)), gf.y / (1.0f + __expf(-gf.y)));
    reinterpret_cast<__half2*>(out + r * inter)[c] = __hmul2(s, u);
  }
}

}  // namespace
}  // namespace fused
}  // namespace kfb

using namespace kfb;

extern "C" int kfb_add_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* sum_out, int rows,
                               int hidden, float eps, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (rows < 1 || hidden < 8 || hidden % 8 || hidden > fused::kRmsThreads * 8 * fused::kMaxVec)
    return fail(KFB_ERR_INVALID, "add_rmsnorm needs rows >= 1 and hidden a multiple of 8 up to %d, got %d x %d",
                fused::kRmsThreads * 8 * fused::kMaxVec, rows, hidden);
  if (!x || !weight || !y) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || (residual && !aligned16(residual)) || (sum_out && !aligned16(sum_out)))
    return fail(KFB_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  return launch_kernel("add_rmsnorm_kernel", fused::add_rmsnorm_kernel, dim3(rows), dim3(fused::kRmsThreads), 0,
                       (cudaStream_t)stream, pdl_enabled(), (const __half*)x, (const __half*)residual, (const __half*)weight,
                       (__half*)y, (__half*)sum_out, hidden, eps);
}

extern "C" int kfb_rope_kv_write(const void* qkv, const void* cos_table, const void* sin_table, const void* pos_dev,
                                 void* q_out, void* k_cache, void* v_cache, int B, int H, int Hk, int D, int Lmax,
                                 void* stream) {
  if (int rc = require_sm100()) return rc;
  if (B < 1 || H < 1 || Hk < 1 || Lmax < 1 || (D != 64 && D != 128) || B > 65535)
    return fail(KFB_ERR_INVALID, "rope_kv_write: bad shape B=%d H=%d Hk=%d D=%d Lmax=%d", B, H, Hk, D, Lmax);
  if (!qkv || !cos_table || !sin_table || !pos_dev || !q_out || !k_cache || !v_cache) return fail(KFB_ERR_INVALID, "null pointer");
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  return launch_kernel("rope_kv_write_kernel", fused::rope_kv_write_kernel, dim3(H + 2 * Hk, B), dim3(D / 2), 0,
                       (cudaStream_t)stream, pdl_enabled(), (const __half*)qkv, (const float*)cos_table,
                       (const float*)sin_table, (const long long*)pos_dev, (__half*)q_out, (__half*)k_cache,
                       (__half*)v_cache, H, Hk, D, Lmax, status);
}

extern "C" int kfb_silu_mul(const void* gate_up, void* out, int rows, int inter, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (rows < 1 || inter < 2 || inter % 2) return fail(KFB_ERR_INVALID, "silu_mul needs rows >= 1 and an even width, got %d x %d", rows, inter);
  if (!gate_up || !out) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(gate_up) || !aligned16(out)) return fail(KFB_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  const long long total = (long long)rows * (inter / 2);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return launch_kernel("silu_mul_kernel", fused::silu_mul_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream,
                       pdl_enabled(), (const __half*)gate_up, (__half*)out, rows, inter);
}
