// INT4 GEMV (M = 1..8) with the dot products on mma.sync fragments.
//
// Why this exists: on B200 the CUDA-core GEMV (int4_gemv.cu) is issue-bound, not HBM-bound -- logic/shift ops
// issue at half the FP32 rate, so unpack + one FMA per weight + operand extraction cost ~3 issue slots per weight
// against a budget of 2.8 at the full HBM rate (ncu: issue slots 63 % busy, ALU pipe 57 %, DRAM 41 %).  Here the
// multiply-accumulate of 16 rows x 16 k x 8 batch columns is ONE instruction, which leaves the unpack (5 logic ops per
// 8 weights) as the only per-weight work: ~1.6 issue slots per weight.  The weight stream is unchanged: 128-bit
// L1-bypassing loads of the packed rows, nothing staged through shared memory.
//
// Arithmetic.  The nibbles are NOT converted to q.  The masked forms A = 1024 + u (nibble pairs 0 and 2 of a word)
// and B = 1024 + 16u (pairs 1 and 3) are exact fp16 values and go straight into the MMA (fp16 x fp16 products are
// exact, FP32 accumulation); class-A and class-B values go to different MMAs, and per scale group
//     sum_k q x = (accA - 1032 * SxA) + (accB / 16 - 72 * SxB),
// with SxA / SxB the sums of the activations multiplied by class-A / class-B weights in that group (they depend on x
// only and are computed once per CTA).  The group scale is applied in FP32, one rounding to fp16 at the end.
//
// Fragment use (m16n8k16, A = weights row-major 16 rows x 16 k, B = activations, 8 columns = batch rows):
//   lane = 4 g + t.  The lane streams rows g and g + 8 of the tile; per round (one scale group of 128 k, or 64 k when
//   G = 64) it loads G/32 packed words of each row, its k range being 32 t .. 32 t + 31 (16 t .. when G = 64) of the
//   group.  For word j: a0/a1 = pair 0 of rows g / g+8, a2/a3 = pair 2  -> MMA (j, A);  pairs 1 and 3 -> MMA (j, B).
//   The k positions an MMA multiplies are whatever the four lanes t = 0..3 put in the same fragment slots, so the B
//   fragment of lane (g, t) is simply the same pairs of x[m = g] at this lane's k range -- any consistent assignment
//   of k to fragment slots gives the same dot product.
#pragma once

#include "common.cuh"

namespace kfb {
namespace gemv_mma {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kTileRows = 16;

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
  uint2 v;
  asm("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma16816_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// G: scale group size (128 or 64).  Rounds of G k; `ksplit` warps of a CTA share a row tile and take rounds
// kpart, kpart + ksplit, ...  Shared memory: class sums of x for every round, then the cross-warp reduction.
template <int G>
__global__ void __launch_bounds__(kThreads)
int4_gemv_mma_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ packed, const __half* __restrict__ scales,
                     __half* __restrict__ y, int M, int N, int K, int ksplit_log2) {
  constexpr int W = G / 32;            // packed words per lane per row per round
  constexpr int kLaneK = G / 4;        // k per lane per round (32 or 16)
  extern __shared__ float smem_f[];
  const int rounds = K / G;
  float* sx = smem_f;                          // [rounds][8 columns][2 classes], pre-multiplied by -1032 / -72
  float* red = smem_f + rounds * 16;           // [kWarps][32 lanes][4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // ---- class sums of the activations, once per CTA.  Four lanes share one (round, batch row): each sums a quarter
  // of the group (whole packed words: pairs 0, 2 of a word are class A, pairs 1, 3 class B), then a quad reduction.
  for (int i = threadIdx.x; i < rounds * 16; i += kThreads)
    if (((i >> 1) & 7) >= M) sx[i] = 0.f;
  {
    const int q = threadIdx.x & 3, items = rounds * M;
    for (int base = 0; base < items; base += kThreads / 4) {
      const int item = base + (threadIdx.x >> 2);
      const bool live = item < items;
      const int rd = live ? item / M : 0, m = live ? item - rd * M : 0;
      const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)rd * G + q * (G / 4));
      float sa = 0.f, sb = 0.f;
      if (live) {
#pragma unroll
        for (int i = 0; i < G / 32; ++i) {
          const uint4 v = xr[i];
          const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
          const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
          const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
          const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
          sa += (p0.x + p0.y) + (p2.x + p2.y);
          sb += (p1.x + p1.y) + (p3.x + p3.y);
        }
      }
      sa += __shfl_xor_sync(0xffffffffu, sa, 1);
      sb += __shfl_xor_sync(0xffffffffu, sb, 1);
      sa += __shfl_xor_sync(0xffffffffu, sa, 2);
      sb += __shfl_xor_sync(0xffffffffu, sb, 2);
      if (live && q == 0) {
        sx[(rd * 8 + m) * 2 + 0] = sa * -1032.0f;
        sx[(rd * 8 + m) * 2 + 1] = sb * -72.0f;
      }
    }
  }
  __syncthreads();

  const int ksplit = 1 << ksplit_log2;
  const int tile = blockIdx.x * (kWarps >> ksplit_log2) + (warp >> ksplit_log2);
  const int kpart = warp & (ksplit - 1);
  const int row_lo = min(tile * kTileRows + g, N - 1);      // rows past N: clamped loads, never stored
  const int row_hi = min(tile * kTileRows + g + 8, N - 1);
  const int words_per_row = K / 8;
  const uint32_t* plo = packed + (size_t)row_lo * words_per_row + t * W;
  const uint32_t* phi = packed + (size_t)row_hi * words_per_row + t * W;
  const __half* slo = scales + (size_t)row_lo * rounds;
  const __half* shi = scales + (size_t)row_hi * rounds;
  const __half* xrow = x + (size_t)min(g, M - 1) * K + t * kLaneK;   // column g of the B operand (zero when g >= M)
  const bool col_live = g < M;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};   // rows g, g+8 x columns 2t, 2t+1
  if (tile * kTileRows < N) {
    // weights and scales of the next round are in flight while the current round is multiplied
    auto load_round = [&](int rd, uint32_t (&lo)[W], uint32_t (&hi)[W], float& sl, float& sh) {
      if constexpr (W == 4) {
        const uint4 a = ldg_stream16(plo + (size_t)rd * (G / 8));
        const uint4 b = ldg_stream16(phi + (size_t)rd * (G / 8));
        lo[0] = a.x; lo[1] = a.y; lo[2] = a.z; lo[3] = a.w;
        hi[0] = b.x; hi[1] = b.y; hi[2] = b.z; hi[3] = b.w;
      } else {
        const uint2 a = ldg_stream8(plo + (size_t)rd * (G / 8));
        const uint2 b = ldg_stream8(phi + (size_t)rd * (G / 8));
        lo[0] = a.x; lo[1] = a.y;
        hi[0] = b.x; hi[1] = b.y;
      }
      sl = __half2float(slo[rd]);
      sh = __half2float(shi[rd]);
    };
    uint32_t wlo[W], whi[W], nlo[W], nhi[W];
    float s_lo = 0.f, s_hi = 0.f, ns_lo = 0.f, ns_hi = 0.f;
    if (kpart < rounds) load_round(kpart, wlo, whi, s_lo, s_hi);
    for (int rd = kpart; rd < rounds; rd += ksplit) {
      const bool more = rd + ksplit < rounds;
      if (more) load_round(rd + ksplit, nlo, nhi, ns_lo, ns_hi);
      uint32_t xs[W * 4];
      {
        const uint4* xp = reinterpret_cast<const uint4*>(xrow + (size_t)rd * G);
#pragma unroll
        for (int i = 0; i < W; ++i) {
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (col_live) v = xp[i];
          xs[4 * i + 0] = v.x; xs[4 * i + 1] = v.y; xs[4 * i + 2] = v.z; xs[4 * i + 3] = v.w;
        }
      }
      float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};
      constexpr uint32_t kMagic = 0x64006400u;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const uint32_t lo = wlo[j], hi = whi[j], lo8 = lo >> 8, hi8 = hi >> 8;
        // xs[4j + p] holds the activation pair multiplied by nibble pair p of word j
        mma16816_f16(ca, (lo & 0x000F000Fu) | kMagic, (hi & 0x000F000Fu) | kMagic, (lo8 & 0x000F000Fu) | kMagic,
                     (hi8 & 0x000F000Fu) | kMagic, xs[4 * j + 0], xs[4 * j + 2]);
        mma16816_f16(cb, (lo & 0x00F000F0u) | kMagic, (hi & 0x00F000F0u) | kMagic, (lo8 & 0x00F000F0u) | kMagic,
                     (hi8 & 0x00F000F0u) | kMagic, xs[4 * j + 1], xs[4 * j + 3]);
      }
      // remove the offsets of the unsigned forms and apply the group scale
      const float2 c0 = *reinterpret_cast<const float2*>(sx + (rd * 8 + 2 * t) * 2);       // column 2t: (A, B) terms
      const float2 c1 = *reinterpret_cast<const float2*>(sx + (rd * 8 + 2 * t + 1) * 2);   // column 2t+1
      acc[0] = fmaf(s_lo, (ca[0] + c0.x) + fmaf(cb[0], 0.0625f, c0.y), acc[0]);
      acc[1] = fmaf(s_lo, (ca[1] + c1.x) + fmaf(cb[1], 0.0625f, c1.y), acc[1]);
      acc[2] = fmaf(s_hi, (ca[2] + c0.x) + fmaf(cb[2], 0.0625f, c0.y), acc[2]);
      acc[3] = fmaf(s_hi, (ca[3] + c1.x) + fmaf(cb[3], 0.0625f, c1.y), acc[3]);
      if (more) {
#pragma unroll
        for (int j = 0; j < W; ++j) { wlo[j] = nlo[j]; whi[j] = nhi[j]; }
        s_lo = ns_lo;
        s_hi = ns_hi;
      }
    }
  }

  if (ksplit_log2 != 0) {
    __syncthreads();
    float4* mine = reinterpret_cast<float4*>(red + (warp * 32 + lane) * 4);
    *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (kpart != 0) return;
    for (int p = 1; p < ksplit; ++p) {  // fixed order
      const float4 o = *reinterpret_cast<const float4*>(red + ((warp + p) * 32 + lane) * 4);
      acc[0] += o.x; acc[1] += o.y; acc[2] += o.z; acc[3] += o.w;
    }
  }
  const int r0 = tile * kTileRows + g, r1 = r0 + 8, m0 = 2 * t, m1 = 2 * t + 1;
  if (m0 < M) {
    if (r0 < N) y[(size_t)m0 * N + r0] = __float2half_rn(acc[0]);
    if (r1 < N) y[(size_t)m0 * N + r1] = __float2half_rn(acc[2]);
  }
  if (m1 < M) {
    if (r0 < N) y[(size_t)m1 * N + r0] = __float2half_rn(acc[1]);
    if (r1 < N) y[(size_t)m1 * N + r1] = __float2half_rn(acc[3]);
  }
}

template <int G>
int launch(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, cudaStream_t stream) {
  const int rounds = K / G;
  const int tiles = ceil_div(N, kTileRows);
  // split K over the warps of a CTA until the grid offers about 16 warps per SM (never more warps than rounds)
  int ksplit_log2 = 0;
  const long long want = 16LL * sm_count();
  while (ksplit_log2 < 3 && (long long)tiles * (1 << ksplit_log2) < want && (2 << ksplit_log2) <= rounds) ++ksplit_log2;
  const int grid = ceil_div(tiles, kWarps >> ksplit_log2);
  const size_t smem = (size_t)(rounds * 16 + kWarps * 32 * 4) * sizeof(float);
  if (smem > 48 * 1024) return fail(KFB_ERR_UNSUPPORTED, "K=%d needs %zu bytes of shared memory for the class sums", K, smem);
  int4_gemv_mma_kernel<G><<<grid, kThreads, smem, stream>>>((const __half*)x, (const uint32_t*)packed, (const __half*)scales,
                                                           (__half*)y, M, N, K, ksplit_log2);
  KFB_LAUNCH_CHECK("int4_gemv_mma_kernel");
  return KFB_OK;
}

}  // namespace gemv_mma
}  // namespace kfb
