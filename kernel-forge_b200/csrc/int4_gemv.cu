// INT4 weight-only GEMV for M = 1..8 on sm_100a:  y[m, n] = sum_k x[m, k] * q[n, k] * s[n, k / G].
//
// Replaces dequant_gemv_kernel of the reference (csrc/gemm/dequant_gemv_kernel.cuh:38-109).
// The kernel is HBM-bound (0.516 B per weight at G = 128) and uses no tensor cores:
//   * a lane streams one 16-byte chunk (32 weights) of each of its R rows per step with
//     L1-bypassing 128-bit loads; consecutive lanes read consecutive chunks, so a warp step
//     covers 512 contiguous bytes of every row it owns;
//   * nibbles are turned into exact fp16 integers with the magic-number trick the packed
//     layout was designed for (kernelforge/quantize.py:18-23, csrc/gemm/int4.cuh:20-27):
//     (w & 0x000F000F) | 0x6400 6400 = 1024 + u, (w & 0x00F000F0) | 0x64006400 = 1024 + 16u,
//     one HSUB2 / HFMA2 each gives the pair (q[2i], q[2i+1]) -- 1 shift + 4 LOP3 + 4 half2 ops
//     per 8 weights;
//   * products are accumulated in FP32 with the sm_100 mixed-precision FMA
//     (fma.rn.f32.f16: fp16 x fp16 + fp32, the product is exact), the per-group scale is
//     applied in FP32 once per 32-weight chunk (32 divides G), then a warp-shuffle reduction
//     and ONE rounding to fp16.  For M >= 3: an FP32 dot product of the exact dequantised weights.
//     For M <= 2 the kernel is issue-bound on B200 (INT and half2 ops issue at half the FP32 rate),
//     so there the half2 conversions are skipped: the masked 1024+u / 1024+16u forms feed the FMA
//     directly and the offsets are subtracted per chunk using sums of x shared by all rows.  The
//     accumulator then carries the offsets (up to ~1e3 |x| per weight) until the subtraction; the
//     FMA rounds to nearest, so this costs a little precision (within the stated bounds, checked
//     with one-signed activations too) but no bias.
// K can be split across the warps of a CTA (fixed-order shared-memory reduce: deterministic).
#include "common.cuh"
#include "int4_gemv_mma.cuh"
#include "int4_epilogue.cuh"

#include <cstdlib>

namespace kfb {
namespace gemv {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ldg_cached(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// 8 packed weights -> 4 half2 (q[2i], q[2i+1]), exact integers in [-8, 7].
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t (&q)[4]) {
  constexpr uint32_t kMagic = 0x64006400u;                     // half2(1024, 1024)
  const __half2 k1032 = u32_as_h2(0x64086408u);                // half2(1032, 1032)
  const __half2 kSixteenth = u32_as_h2(0x2C002C00u);           // half2(1/16, 1/16)
  const __half2 kMinus72 = u32_as_h2(0xD480D480u);             // half2(-72, -72)
  const uint32_t h = w >> 8;
  q[0] = h2_as_u32(__hsub2(u32_as_h2((w & 0x000F000Fu) | kMagic), k1032));               // (1024+u) - 1032
  q[1] = h2_as_u32(__hfma2(u32_as_h2((w & 0x00F000F0u) | kMagic), kSixteenth, kMinus72));  // (1024+16u)/16 - 72
  q[2] = h2_as_u32(__hsub2(u32_as_h2((h & 0x000F000Fu) | kMagic), k1032));
  q[3] = h2_as_u32(__hfma2(u32_as_h2((h & 0x00F000F0u) | kMagic), kSixteenth, kMinus72));
}

// acc += a.lo * b.lo + a.hi * b.hi with fp16 inputs and an FP32 accumulator (exact products).
__device__ __forceinline__ float dot2_acc(uint32_t a, uint32_t b, float acc) {
  asm("{\n\t"
      ".reg .b16 al, ah, bl, bh;\n\t"
      "mov.b32 {al, ah}, %1;\n\t"
      "mov.b32 {bl, bh}, %2;\n\t"
      "fma.rn.f32.f16 %0, al, bl, %0;\n\t"
      "fma.rn.f32.f16 %0, ah, bh, %0;\n\t"
      "}"
      : "+f"(acc)
      : "r"(a), "r"(b));
  return acc;
}

// Same with the activation pair already split into two 16-bit registers (done once per chunk and
// shared by all rows of the warp instead of once per row).
__device__ __forceinline__ float dot2_acc_split(uint32_t a, unsigned short bl, unsigned short bh, float acc) {
  asm("{\n\t"
      ".reg .b16 al, ah;\n\t"
      "mov.b32 {al, ah}, %1;\n\t"
      "fma.rn.f32.f16 %0, al, %2, %0;\n\t"
      "fma.rn.f32.f16 %0, ah, %3, %0;\n\t"
      "}"
      : "+f"(acc)
      : "r"(a), "h"(bl), "h"(bh));
  return acc;
}

// FP32 dot product of one unpacked 16-byte weight chunk (16 half2) with 32 activations.
__device__ __forceinline__ float dot32(const uint32_t (&q)[16], const uint4 (&xv)[4]) {
  float p0 = 0.f, p1 = 0.f;  // two chains for ILP
  const uint32_t* xs = reinterpret_cast<const uint32_t*>(xv);
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    p0 = dot2_acc(q[i], xs[i], p0);
    p1 = dot2_acc(q[i + 1], xs[i + 1], p1);
  }
  return p0 + p1;
}

__device__ __forceinline__ void unpack32(const uint4& wv, uint32_t (&q)[16]) {
  uint32_t t[4];
  unpack8(wv.x, t); q[0] = t[0]; q[1] = t[1]; q[2] = t[2]; q[3] = t[3];
  unpack8(wv.y, t); q[4] = t[0]; q[5] = t[1]; q[6] = t[2]; q[7] = t[3];
  unpack8(wv.z, t); q[8] = t[0]; q[9] = t[1]; q[10] = t[2]; q[11] = t[3];
  unpack8(wv.w, t); q[12] = t[0]; q[13] = t[1]; q[14] = t[2]; q[15] = t[3];
}

// What the kernel does to its activations before the product, and to its result after it (decode-step fusions; the
// reference leaves all of these to separate torch kernels, kernelforge/modules.py:51-68, kernelforge/ops.py:300-301).
//   kXformNone     x is used as given
//   kXformRmsNorm  x is the residual stream s; the product uses fp16(fp16(s * rsqrt(mean(s^2) + eps)) * norm_w)
//   kXformSiluMul  x is [M, 2 K] = gate | up; the product uses fp16(fp16(silu(gate)) * up)
// Epilogue (any transform): y = fp16(acc), then + bias[n], then + residual[m, n], each an fp16 addition like the
// separate torch kernels it replaces.
enum Xform : int { kXformNone = 0, kXformRmsNorm = 1, kXformSiluMul = 2 };

// M: activation rows; R: weight rows per warp; G: group size; XF: the transform above (a transformed x is built once
// per CTA in shared memory, M * K halfs, and the main loop reads it from there).
// `ksplit_log2`: 2^ksplit_log2 warps of a CTA share one row tile and split its K chunks.
template <int M, int R, int G, int XF = kXformNone, int EPI = kEpiNone>
__global__ void __launch_bounds__(kThreads)
int4_gemv_kernel(const __half* __restrict__ x, const uint4* __restrict__ packed, const __half* __restrict__ scales,
                 __half* __restrict__ y, int N, int K, int ksplit_log2, const Fusion fu) {
  __shared__ float red[kWarps][M * R];
  // XF != 0: the transformed activations.  The four 16-byte vectors of a 32-activation chunk are stored KC vectors apart
  // (vector v = 4 c + j sits at j * KC + c), so that lanes, which walk consecutive chunks c, read consecutive vectors:
  // in the natural order a warp's 16-byte loads were 64 bytes apart, a four-way bank conflict on every load.
  extern __shared__ uint4 xs_raw[];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksplit = 1 << ksplit_log2;
  const int tile = blockIdx.x * (kWarps >> ksplit_log2) + (warp >> ksplit_log2);
  const int kpart = warp & (ksplit - 1);
  const int r0 = tile * R;
  const int KC = K >> 5;  // 16-byte chunks per packed row
  const int SG = K / G;   // scales per row
  constexpr int kChunksPerGroup = G / 32;

  float acc[M][R];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[m][r] = 0.f;

  // Weights and scales are constants: the first two chunks of every lane are fetched BEFORE waiting for the kernel in
  // front (programmatic dependent launch: this grid is already resident while that kernel finishes, so its launch
  // latency and the first DRAM round trip are hidden); x (and y, in the epilogue) are touched only after the wait.
  // The dependents of this grid are released right after its own wait has returned, so at most two grids overlap.
  const uint4* wrow[R];
  const __half* srow[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int row = min(r0 + r, N - 1);  // rows past N are computed on a clamped row and never stored
    wrow[r] = packed + (size_t)row * KC;
    srow[r] = scales + (size_t)row * SG;
  }
  const int stride = 32 * ksplit;
  const int c_first = r0 < N ? kpart * 32 + lane : KC;   // a tile past N does nothing
  uint4 wbuf[2][R];
  float sbuf[2][R];
  auto fetch = [&](int slot, int c) {
    if (c < KC) {
#pragma unroll
      for (int r = 0; r < R; ++r) wbuf[slot][r] = ldg_stream(wrow[r] + c);
#pragma unroll
      for (int r = 0; r < R; ++r) sbuf[slot][r] = __half2float(srow[r][c / kChunksPerGroup]);
    }
  };
  fetch(0, c_first);
  fetch(1, c_first + stride);
  if constexpr (XF == kXformNone) pdl_wait();   // (with a transform the wait opens the prologue below)
  if constexpr (XF != kXformNone) {
    pdl_wait();   // x is the previous kernel's output
    const int nvec = K / 8;
    if constexpr (XF == kXformRmsNorm) {
      __shared__ float part[M][kWarps];
      constexpr int kMaxVec = 4;   // K <= 256 * 8 * 4
      uint4 keep[M][kMaxVec];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxVec; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nvec) {
            keep[m][i] = reinterpret_cast<const uint4*>(x + (size_t)m * K)[v];
            const __half2* h = reinterpret_cast<const __half2*>(&keep[m][i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(h[j]);
              ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
            }
          }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if ((threadIdx.x & 31) == 0) part[m][threadIdx.x >> 5] = ss;
      }
      __syncthreads();
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) tot += part[m][i];
        const float inv = rsqrtf(tot / (float)K + fu.eps);
#pragma unroll
        for (int i = 0; i < kMaxVec; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nvec) {
            const uint4 wv = reinterpret_cast<const uint4*>(fu.norm_w)[v];
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
            const __half2* h = reinterpret_cast<const __half2*>(&keep[m][i]);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(h[j]);
              oh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
            }
            xs_raw[(size_t)m * nvec + (v & 3) * KC + (v >> 2)] = o;   // chunk-major: see the main loop
          }
        }
      }
    } else {
#pragma unroll
      for (int m = 0; m < M; ++m)
        for (int v = threadIdx.x; v < nvec; v += kThreads) {
          const uint4 gv = reinterpret_cast<const uint4*>(x + (size_t)m * 2 * K)[v];
          const uint4 uv = reinterpret_cast<const uint4*>(x + (size_t)m * 2 * K + K)[v];
          const __half2* gh = reinterpret_cast<const __half2*>(&gv);
          const __half2* uh = reinterpret_cast<const __half2*>(&uv);
          uint4 o;
          __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = __half22float2(gh[j]);
            oh[j] = __hmul2(__floats2half2_rn(gf.x / (1.0f + __expf(-gf.x)), gf.y / (1.0f + __expf(-gf.y))), uh[j]);
          }
          xs_raw[(size_t)m * nvec + (v & 3) * KC + (v >> 2)] = o;   // chunk-major: see the main loop
        }
    }
    __syncthreads();
  }
  pdl_launch_dependents();

  auto process = [&](const uint4 (&wv)[R], const float (&sc)[R], int c) {
      const uint4* xc = reinterpret_cast<const uint4*>(x) + (size_t)c * 4;
    if constexpr (M <= 2) {
      // Decode path.  The kernel is issue-bound, so the nibbles are NOT converted to q: the masked
      // forms A = 1024 + u (nibble pairs 0, 2) and B = 1024 + 16u (pairs 1, 3) go straight into the
      // FP32 mixed-precision FMA (products of two 11-bit significands are exact in FP32) and the
      // offsets are removed per 32-weight chunk with the class sums of x, shared by all R rows:
      //   sum q x = (sum_A (1024+u) x - 1032 SxA) + (sum_B (1024+16u) x / 16 - 72 SxB).
      uint4 xv[M][4];
      unsigned short xl[M][16], xh[M][16];
      float sxa[M], sxb[M];
#pragma unroll
      for (int m = 0; m < M; ++m) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (XF != kXformNone) xv[m][j] = xs_raw[(size_t)m * (K / 8) + (size_t)j * KC + c];
          else xv[m][j] = ldg_cached(xc + (size_t)m * (K / 8) + j);
        }
        const uint32_t* xs = reinterpret_cast<const uint32_t*>(xv[m]);
#pragma unroll
        for (int i = 0; i < 16; ++i) asm("mov.b32 {%0, %1}, %2;" : "=h"(xl[m][i]), "=h"(xh[m][i]) : "r"(xs[i]));
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          a = dot2_acc_split(0x3C003C00u, xl[m][i], xh[m][i], a);      // half2(1, 1)
          b = dot2_acc_split(0x3C003C00u, xl[m][i + 1], xh[m][i + 1], b);
        }
        sxa[m] = a * -1032.0f;
        sxb[m] = b * -72.0f;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t wr[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float pa = 0.f, pb = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            constexpr uint32_t kMagic = 0x64006400u;
            const uint32_t w = wr[j], h = w >> 8;
            pa = dot2_acc_split((w & 0x000F000Fu) | kMagic, xl[m][4 * j + 0], xh[m][4 * j + 0], pa);
            pb = dot2_acc_split((w & 0x00F000F0u) | kMagic, xl[m][4 * j + 1], xh[m][4 * j + 1], pb);
            pa = dot2_acc_split((h & 0x000F000Fu) | kMagic, xl[m][4 * j + 2], xh[m][4 * j + 2], pa);
            pb = dot2_acc_split((h & 0x00F000F0u) | kMagic, xl[m][4 * j + 3], xh[m][4 * j + 3], pb);
          }
          acc[m][r] = fmaf(sc[r], (pa + sxa[m]) + fmaf(pb, 0.0625f, sxb[m]), acc[m][r]);
        }
      }
    } else {
      // weights resident (unpacked once), activations streamed per m
      uint32_t q[R][16];
#pragma unroll
      for (int r = 0; r < R; ++r) unpack32(wv[r], q[r]);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        uint4 xv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (XF != kXformNone) xv[j] = xs_raw[(size_t)m * (K / 8) + (size_t)j * KC + c];
          else xv[j] = ldg_cached(xc + (size_t)m * (K / 8) + j);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) acc[m][r] = fmaf(sc[r], dot32(q[r], xv), acc[m][r]);
      }
    }
  };
  for (int c = c_first; c < KC; c += 2 * stride) {
    process(wbuf[0], sbuf[0], c);
    fetch(0, c + 2 * stride);
    if (c + stride < KC) {
      process(wbuf[1], sbuf[1], c + stride);
      fetch(1, c + 3 * stride);
    }
  }

#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float v = acc[m][r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      acc[m][r] = v;
    }

  if (ksplit_log2 == 0) {
    if (lane == 0 && r0 < N) {
#pragma unroll
      for (int m = 0; m < M; ++m)
        if constexpr (R == 1) {
          y[(size_t)m * N + r0] = finish(acc[m][0], fu, m, r0, N);
        } else {
#pragma unroll
          for (int r = 0; r < R; r += 2)
            if (r0 + r < N) store_pair<EPI>(acc[m][r], acc[m][r + 1], fu, y, m, r0 + r, N);
        }
    }
    return;
  }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r) red[warp][m * R + r] = acc[m][r];
  }
  __syncthreads();
  if (kpart == 0) {   // warp-uniform
    const bool live = lane < M * R && r0 < N;
    const int m = lane / R, r = lane % R;
    float v = 0.f;
    if (live)
      for (int p = 0; p < ksplit; ++p) v += red[warp + p][lane];  // fixed order
    if constexpr (R == 1) {
      if (live) y[(size_t)m * N + r0] = finish(v, fu, m, r0, N);
    } else {
      const float partner = __shfl_xor_sync(0xffffffffu, v, 1);   // row r ^ 1 of the same batch row (R is even)
      if (live && (r & 1) == 0 && r0 + r < N) store_pair<EPI>(v, partner, fu, y, m, r0 + r, N);
    }
  }
}

template <int M, int R, int G, int XF = kXformNone, int EPI = kEpiNone>
int launch(const void* x, const void* packed, const void* scales, void* y, int N, int K, int ksplit_log2, int flags,
           cudaStream_t stream, const Fusion& fu = Fusion{}) {
  const int tiles = ceil_div(N, R);
  const int grid = ceil_div(tiles, kWarps >> ksplit_log2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = XF != kXformNone ? (size_t)M * K * sizeof(__half) : 0;
  cfg.stream = stream;
  if (cfg.dynamicSmemBytes > 48 * 1024) {
    static bool configured[64] = {false};
    int dev = 0;
    KFB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      KFB_CUDA_TRY(cudaFuncSetAttribute(int4_gemv_kernel<M, R, G, XF, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      configured[dev] = true;
    }
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ((flags & 1) || pdl_enabled()) ? 1 : 0;
  KFB_CUDA_TRY(cudaLaunchKernelEx(&cfg, int4_gemv_kernel<M, R, G, XF, EPI>, (const __half*)x, (const uint4*)packed,
                                  (const __half*)scales, (__half*)y, N, K, ksplit_log2, fu));
  return KFB_OK;
}

template <int M, int G, int XF = kXformNone, int EPI = kEpiNone>
int pick_rows(const void* x, const void* packed, const void* scales, void* y, int N, int K, int flags,
              cudaStream_t stream, const Fusion& fu = Fusion{}) {
  // K split inside the CTA: aim at about two 16-byte chunks per lane, never less than one.
  const int KC = K / 32;
  int ksplit_log2 = 0;
  while (ksplit_log2 < 3 && KC / (32 << ksplit_log2) >= 4) ++ksplit_log2;
  // Rows per warp: as many as the register budget allows while the grid still fills the SMs.
  const int sms = sm_count();
  constexpr int kMaxR = (M == 1) ? 8 : (M == 2) ? 4 : 2;
  int R = kMaxR;
  while (R > 1 && ceil_div(ceil_div(N, R), kWarps >> ksplit_log2) < 2 * sms) R >>= 1;
  if (EPI != kEpiNone && R < 2) R = 2;   // a pair of rows must sit in one warp
  if constexpr (kMaxR == 8) {
    if (R == 8) return launch<M, 8, G, XF, EPI>(x, packed, scales, y, N, K, ksplit_log2, flags, stream, fu);
  }
  if constexpr (kMaxR >= 4) {
    if (R == 4) return launch<M, 4, G, XF, EPI>(x, packed, scales, y, N, K, ksplit_log2, flags, stream, fu);
  }
  if (R == 2) return launch<M, 2, G, XF, EPI>(x, packed, scales, y, N, K, ksplit_log2, flags, stream, fu);
  if constexpr (EPI == kEpiNone) return launch<M, 1, G, XF>(x, packed, scales, y, N, K, ksplit_log2, flags, stream, fu);
  return fail(KFB_ERR_INVALID, "a pair epilogue needs two rows per warp");
}

// The fused entry: M <= 2 only (the batch sizes at which this kernel is the one the dispatcher uses anyway).
template <int G, int M, int EPI>
int pick_xform(const void* x, const void* packed, const void* scales, void* y, int N, int K, int xform, int flags,
               cudaStream_t stream, const Fusion& fu) {
  if (xform == kXformRmsNorm) return pick_rows<M, G, kXformRmsNorm, EPI>(x, packed, scales, y, N, K, flags, stream, fu);
  if constexpr (EPI == kEpiNone) {
    if (xform == kXformSiluMul) return pick_rows<M, G, kXformSiluMul, EPI>(x, packed, scales, y, N, K, flags, stream, fu);
  } else {
    if (xform == kXformSiluMul) return fail(KFB_ERR_UNSUPPORTED, "the pair epilogues take no SiLU * up prologue");
  }
  return pick_rows<M, G, kXformNone, EPI>(x, packed, scales, y, N, K, flags, stream, fu);
}

template <int G>
int pick_fused(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, int xform, int flags,
               cudaStream_t stream, const Fusion& fu) {
  if (M == 1) {
    if (fu.epi == kEpiSiluPair) return pick_xform<G, 1, kEpiSiluPair>(x, packed, scales, y, N, K, xform, flags, stream, fu);
    if (fu.epi == kEpiRopeKv) return pick_xform<G, 1, kEpiRopeKv>(x, packed, scales, y, N, K, xform, flags, stream, fu);
    return pick_xform<G, 1, kEpiNone>(x, packed, scales, y, N, K, xform, flags, stream, fu);
  }
  if (fu.epi == kEpiSiluPair) return pick_xform<G, 2, kEpiSiluPair>(x, packed, scales, y, N, K, xform, flags, stream, fu);
  if (fu.epi == kEpiRopeKv) return pick_xform<G, 2, kEpiRopeKv>(x, packed, scales, y, N, K, xform, flags, stream, fu);
  return pick_xform<G, 2, kEpiNone>(x, packed, scales, y, N, K, xform, flags, stream, fu);
}

template <int G>
int pick_m(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, int flags,
           cudaStream_t stream) {
  switch (M) {
    case 1: return pick_rows<1, G>(x, packed, scales, y, N, K, flags, stream);
    case 2: return pick_rows<2, G>(x, packed, scales, y, N, K, flags, stream);
    case 3: return pick_rows<3, G>(x, packed, scales, y, N, K, flags, stream);
    case 4: return pick_rows<4, G>(x, packed, scales, y, N, K, flags, stream);
    case 5: return pick_rows<5, G>(x, packed, scales, y, N, K, flags, stream);
    case 6: return pick_rows<6, G>(x, packed, scales, y, N, K, flags, stream);
    case 7: return pick_rows<7, G>(x, packed, scales, y, N, K, flags, stream);
    default: return pick_rows<8, G>(x, packed, scales, y, N, K, flags, stream);
  }
}

}  // namespace gemv
}  // namespace kfb

using namespace kfb;

namespace {

int gemv_entry(const char* what, int max_m, const void* x, const void* packed, const void* scales, void* y, int M, int N, int K,
               int group, int flags, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (M < 1 || M > max_m) return fail(KFB_ERR_INVALID, "%s handles M in [1, %d], got M=%d", what, max_m, M);
  if (group != 64 && group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", group);
  if (N < 1 || K < group || K % group) return fail(KFB_ERR_INVALID, "K=%d is not a multiple of group_size=%d", K, group);
  if (!x || !packed || !scales || !y) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(x) || !aligned16(packed)) return fail(KFB_ERR_ALIGNMENT, "x and packed must be 16-byte aligned");
  if ((flags & ~7) || (flags & 6) == 6) return fail(KFB_ERR_INVALID, "unknown flags 0x%x", flags);
  cudaStream_t s = (cudaStream_t)stream;
  // Two kernels: the mma.sync formulation (int4_gemv_mma.cuh) and the CUDA-core one of this file, which is
  // issue-bound on B200 and whose time grows with M.  Measured under a CUDA graph on L2-cold weights (us, CUDA core /
  // mma):  5632x2048  M=1 4.2/5.0  M=2 5.9/5.4  M=4 9.2/6.3  M=8 16.1/7.7;   8960x1536  5.3/5.4  7.8/5.7  11.6/6.0
  // 20.2/7.0;   11264x2048  6.3/9.0  8.9/9.7  16.2/10.5  25.7/12.3;   2048x5632  6.1/5.3  8.8/5.9  14.2/6.7  32.0/9.0;
  // 32000x2048  13.3/12.6  18.2/13.7  36.4/15.2  68.4/18.3;   128256x4096  76/62  132/64  273/67  521/80.  So: M = 1 takes
  // the CUDA-core kernel unless N is large enough for the persistent streaming kernel, M >= 2 takes mma.  Flag bit 1
  // forces the CUDA-core kernel (M <= 8), flag bit 2 the mma one; K too long for the class sums to fit in shared
  // memory also goes to the CUDA-core kernel.
  const bool fits = group == 128 ? gemv_mma::fits<128>(M, K) : gemv_mma::fits<64>(M, K);
  const bool prefer_mma = (flags & 4) || (!(flags & 2) && (M >= 2 || gemv_mma::uses_stream_kernel(N)));
  if (fits && (M > 8 || prefer_mma))
    return group == 128 ? gemv_mma::launch<128>(x, packed, scales, y, M, N, K, (flags & 1) != 0, s)
                        : gemv_mma::launch<64>(x, packed, scales, y, M, N, K, (flags & 1) != 0, s);
  if (M > 8) return fail(KFB_ERR_UNSUPPORTED, "%s: K=%d is too long for M=%d (class sums exceed shared memory)", what, K, M);
  return group == 128 ? gemv::pick_m<128>(x, packed, scales, y, M, N, K, flags, s)
                      : gemv::pick_m<64>(x, packed, scales, y, M, N, K, flags, s);
}

}  // namespace

extern "C" int kfb_int4_gemv(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K,
                             int group, int flags, void* stream) {
  return gemv_entry("int4_gemv", 8, x, packed, scales, y, M, N, K, group, flags, stream);
}

namespace {

int fused_common(const char* what, const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, int group,
                 int xform, int flags, void* stream, const gemv::Fusion& fu) {
  if (int rc = require_sm100()) return rc;
  if (M < 1 || M > 2) return fail(KFB_ERR_UNSUPPORTED, "%s handles M in [1, 2], got M=%d", what, M);
  if (group != 64 && group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", group);
  if (N < 1 || K < group || K % group) return fail(KFB_ERR_INVALID, "K=%d is not a multiple of group_size=%d", K, group);
  if (xform < 0 || xform > 2) return fail(KFB_ERR_INVALID, "unknown activation transform %d", xform);
  if (xform != gemv::kXformNone && K > 8192) return fail(KFB_ERR_UNSUPPORTED, "fused transforms handle K <= 8192, got %d", K);
  if (xform == gemv::kXformRmsNorm && !fu.norm_w) return fail(KFB_ERR_INVALID, "the RMSNorm transform needs its weight");
  if (!x || !packed || !scales) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(x) || !aligned16(packed) || (fu.norm_w && !aligned16(fu.norm_w)))
    return fail(KFB_ERR_ALIGNMENT, "x, packed and the norm weight must be 16-byte aligned");
  if (flags & ~1) return fail(KFB_ERR_INVALID, "unknown flags 0x%x", flags);
  cudaStream_t s = (cudaStream_t)stream;
  return group == 128 ? gemv::pick_fused<128>(x, packed, scales, y, M, N, K, xform, flags, s, fu)
                      : gemv::pick_fused<64>(x, packed, scales, y, M, N, K, xform, flags, s, fu);
}

}  // namespace

extern "C" int kfb_int4_gemv_fused(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, int group,
                                   int xform, const void* norm_weight, float eps, const void* bias, const void* residual,
                                   int flags, void* stream) {
  if (!y) return fail(KFB_ERR_INVALID, "null pointer");
  gemv::Fusion fu = {};
  fu.norm_w = static_cast<const __half*>(norm_weight);
  fu.eps = eps;
  fu.bias = static_cast<const __half*>(bias);
  fu.residual = static_cast<const __half*>(residual);
  return fused_common("int4_gemv_fused", x, packed, scales, y, M, N, K, group, xform, flags, stream, fu);
}

extern "C" int kfb_int4_gemv_silu_pair(const void* x, const void* packed, const void* scales, void* act_out, int M, int N, int K,
                                       int group, int xform, const void* norm_weight, float eps, int flags, void* stream) {
  if (!act_out) return fail(KFB_ERR_INVALID, "null pointer");
  if (N % 2) return fail(KFB_ERR_INVALID, "int4_gemv_silu_pair needs an even number of rows (gate, up interleaved), got N=%d", N);
  gemv::Fusion fu = {};
  fu.norm_w = static_cast<const __half*>(norm_weight);
  fu.eps = eps;
  fu.epi = gemv::kEpiSiluPair;
  return fused_common("int4_gemv_silu_pair", x, packed, scales, act_out, M, N, K, group, xform, flags, stream, fu);
}

extern "C" int kfb_int4_gemv_rope_kv(const void* x, const void* packed, const void* scales, int M, int K, int group, int xform,
                                     const void* norm_weight, float eps, const void* cos_table, const void* sin_table,
                                     const void* pos_dev, void* q_out, void* k_cache, void* v_cache, int H, int Hk, int D,
                                     int Lmax, int flags, void* stream) {
  if (H < 1 || Hk < 1 || Lmax < 1 || (D != 64 && D != 128))
    return fail(KFB_ERR_INVALID, "int4_gemv_rope_kv: bad shape H=%d Hk=%d D=%d Lmax=%d", H, Hk, D, Lmax);
  if (!cos_table || !sin_table || !pos_dev || !q_out || !k_cache || !v_cache) return fail(KFB_ERR_INVALID, "null pointer");
  gemv::Fusion fu = {};
  fu.norm_w = static_cast<const __half*>(norm_weight);
  fu.eps = eps;
  fu.epi = gemv::kEpiRopeKv;
  fu.rope.cos_t = static_cast<const float*>(cos_table);
  fu.rope.sin_t = static_cast<const float*>(sin_table);
  fu.rope.pos = static_cast<const long long*>(pos_dev);
  fu.rope.q_out = static_cast<__half*>(q_out);
  fu.rope.k_cache = static_cast<__half*>(k_cache);
  fu.rope.v_cache = static_cast<__half*>(v_cache);
  fu.rope.H = H; fu.rope.Hk = Hk; fu.rope.D = D; fu.rope.Lmax = Lmax;
  fu.rope.status = device_status_word();
  if (!fu.rope.status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  // y is not written by this epilogue: q_out stands in for the pointer checks of the common path
  return fused_common("int4_gemv_rope_kv", x, packed, scales, q_out, M, (H + 2 * Hk) * D, K, group, xform, flags, stream, fu);
}

extern "C" int kfb_int4_small_batch(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K,
                                    int group, int flags, void* stream) {
  return gemv_entry("int4_small_batch", gemv_mma::kMaxM, x, packed, scales, y, M, N, K, group, flags, stream);
}

#ifdef KFB_TRACE
// Tuning aid of -DKFB_TRACE builds (not part of the public header): device buffer of 4 words per warp of the
// streaming kernel (3 timestamps in ns, SM id).
extern "C" void kfb_debug_set_gemv_trace(void* device_buffer) {
  kfb::gemv_mma::g_trace = static_cast<unsigned long long*>(device_buffer);
}
#endif
