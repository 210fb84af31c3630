// Epilogues shared by the M <= 8 INT4 GEMV kernels (the CUDA-core kernel of int4_gemv.cu, the fragment-order kernel of
// int4_gemv_frag.cu): what happens to a pair of adjacent result rows before it is stored.
#pragma once

#include "common.cuh"

namespace kfb {
namespace gemv {

// Pair epilogues: the weight rows were laid out (by the caller, once, when the model was built -- a private row order of
// the public packed format; rows are quantised independently, so any row order is exact) so that rows 2p and 2p + 1
// belong together, and the kernel turns each pair of results into what the next kernel of a decode step needs:
//   kEpiSiluPair  rows (gate_p, up_p): writes act[m, p] = fp16(fp16(silu(g)) * u), y is [M, N / 2]
//                 (replaces the separate SiLU * up kernel; same roundings);
//   kEpiRopeKv    the fused q / k / v projection of one decode position: pairs (d, d + D/2) of a q or k head are rotated
//                 (rotate-half convention, FP32, one rounding) and written to q_out / row `pos` of the K cache; v pairs
//                 (d, d + 1) go to row `pos` of the V cache (replaces the separate RoPE + cache-write kernel).
enum Epilogue : int { kEpiNone = 0, kEpiSiluPair = 1, kEpiRopeKv = 2 };

struct RopeKv {
  const float* cos_t;       // [Lmax, D]
  const float* sin_t;
  const long long* pos;     // device scalar: the position being written
  __half* q_out;            // [M, H, D]
  __half* k_cache;          // [M, Hk, Lmax, D]
  __half* v_cache;
  int H, Hk, D, Lmax;
  unsigned int* status;
};

struct Fusion {
  const __half* norm_w;    // kXformRmsNorm: [K]
  float eps;
  const __half* bias;      // [N] or nullptr
  const __half* residual;  // [M, N] or nullptr
  int epi;                 // Epilogue
  RopeKv rope;
};

constexpr unsigned int kStatusRopePosition = 0x701;  // the position read on the device lies outside [0, Lmax)

// One rounding of the FP32 sum to fp16, then the optional bias and residual as fp16 additions.
__device__ __forceinline__ __half finish(float acc, const Fusion& fu, int m, int n, int N) {
  __half v = __float2half_rn(acc);
  if (fu.bias) v = __hadd(v, fu.bias[n]);
  if (fu.residual) v = __hadd(v, fu.residual[(size_t)m * N + n]);
  return v;
}

// Stores the results of rows n (even) and n + 1 of batch row m.
template <int EPI>
__device__ __forceinline__ void store_pair(float a0, float a1, const Fusion& fu, __half* __restrict__ y, int m, int n, int N) {
  if constexpr (EPI == kEpiNone) {
    y[(size_t)m * N + n] = finish(a0, fu, m, n, N);
    if (n + 1 < N) y[(size_t)m * N + n + 1] = finish(a1, fu, m, n + 1, N);
    return;
  }
  const float g = __half2float(__float2half_rn(a0)), u = __half2float(__float2half_rn(a1));   // what the unfused path reads back
  if constexpr (EPI == kEpiSiluPair) {
    y[(size_t)m * (N / 2) + (n >> 1)] = __hmul(__float2half_rn(g / (1.0f + __expf(-g))), __float2half_rn(u));
    return;
  }
  const RopeKv& rp = fu.rope;
  const long long pos = rp.pos[0];
  if (pos < 0 || pos >= rp.Lmax) {   // nothing is read or written for a position outside the cache
    if (n == 0 && m == 0) atomicCAS(rp.status, 0u, kStatusRopePosition);
    return;
  }
  const int half = rp.D / 2, p = n >> 1;
  const int q_pairs = rp.H * half, k_pairs = rp.Hk * half;
  if (p < q_pairs + k_pairs) {
    const int head = p < q_pairs ? p / half : (p - q_pairs) / half;
    const int j = p < q_pairs ? p % half : (p - q_pairs) % half;
    const float c0 = rp.cos_t[pos * rp.D + j], s0 = rp.sin_t[pos * rp.D + j];
    const float c1 = rp.cos_t[pos * rp.D + j + half], s1 = rp.sin_t[pos * rp.D + j + half];
    // the roundings of the separate RoPE kernel: both products and the sum rounded on their own
    const __half rlo = __float2half_rn(__fsub_rn(__fmul_rn(g, c0), __fmul_rn(u, s0)));
    const __half rhi = __float2half_rn(__fadd_rn(__fmul_rn(u, c1), __fmul_rn(g, s1)));
    __half* dst = p < q_pairs ? rp.q_out + ((size_t)m * rp.H + head) * rp.D
                              : rp.k_cache + (((size_t)m * rp.Hk + head) * rp.Lmax + pos) * rp.D;
    dst[j] = rlo;
    dst[j + half] = rhi;
  } else {
    const int pv = p - q_pairs - k_pairs, head = pv / half, j = pv % half;
    __half* dst = rp.v_cache + (((size_t)m * rp.Hk + head) * rp.Lmax + pos) * rp.D;
    dst[2 * j] = __float2half_rn(a0);
    dst[2 * j + 1] = __float2half_rn(a1);
  }
}

}  // namespace gemv
}  // namespace kfb
