// INT4 GEMV (M = 1..8) with the dot products on mma.sync fragments.
//
// Why this exists: on B200 the CUDA-core GEMV (int4_gemv.cu) is issue-bound, not HBM-bound -- logic/shift ops
// issue at half the FP32 rate, so unpack + one FMA per weight + operand extraction cost ~3 issue slots per weight
// against a budget of 2.8 at the full HBM rate (ncu: issue slots 63 % busy, ALU pipe 57 %, DRAM 41 %).  Here the
// multiply-accumulate of 16 rows x 16 k x 8 batch columns is ONE instruction, which leaves the unpack (5 logic ops per
// 8 weights) as the only per-weight work: ~0.6 issue slots per weight, the same for every M up to 8.
//
// With the issue limit gone the kernel is bound by how many bytes each SM keeps in flight, so the weight stream goes
// through a shared-memory ring filled by cp.async (16 bytes per lane per row per round, L1 bypassed, 128-byte L2
// fetch): kStages rounds per warp are outstanding at any time, ~170 KB per SM.  A lane consumes exactly the 16-byte
// pieces it requested itself, so the ring is private to the lane (no barrier, no bank conflict) -- it is a register
// file extension for loads in flight, not a data exchange.
//
// The second limit is the integer pipe (logic and shift instructions issue at half rate on B200): the first version
// of this kernel spent 110 such instructions per round where the unpack needs 40, the rest being address arithmetic
// and predication.  So the round loop is unrolled by the ring depth with the K split a template parameter -- every
// global, shared and ring address of a round is then a pointer plus an immediate -- accumulators start from the zero
// register instead of being cleared, and batch columns past M read a valid row instead of being zero-filled (a
// column of the MMA result depends on its own column of the activations only, and those columns are never stored).
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
constexpr int kStages = 8;             // rounds in flight per warp = unroll factor of the round loop

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// d = a * b + c, m16n8k16, fp16 operands, FP32 accumulation
__device__ __forceinline__ void mma16816_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1, const float* c) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__host__ __device__ constexpr size_t ring_bytes() { return (size_t)kWarps * kStages * 2 * 32 * 16; }
inline size_t smem_bytes(int rounds) { return (size_t)(rounds * 16 + kWarps * 32 * 4) * sizeof(float) + ring_bytes(); }

// G: scale group size (128 or 64).  Rounds of G k.  KS = 1 << KSL warps of a CTA share a row tile and take rounds
// kpart, kpart + KS, ...  Shared memory: class sums of x for every round, the cross-warp reduction, the ring.
template <int G, int KSL>
__global__ void __launch_bounds__(kThreads, 3)
int4_gemv_mma_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ packed, const __half* __restrict__ scales,
                     __half* __restrict__ y, int M, int N, int K) {
  constexpr int W = G / 32;            // packed words per lane per row per round
  constexpr int kLaneK = G / 4;        // k per lane per round (32 or 16)
  constexpr int KS = 1 << KSL;
  constexpr int kWStep = KS * (G / 8);   // words between two rounds of this warp
  constexpr int kXStep = KS * G;         // activations
  constexpr int kSxStep = KS * 16;       // class-sum floats
  constexpr uint32_t kSlot = 2 * 32 * 16;  // ring bytes per round
  extern __shared__ __align__(16) float smem_f[];
  const int rounds = K / G;
  float* sx = smem_f;                          // [rounds][8 columns][2 classes], pre-multiplied by -1032 / -72
  float* red = smem_f + rounds * 16;           // [kWarps][32 lanes][4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // this lane's ring slots: [stage][row lo / hi] 16 bytes each; consecutive lanes are 16 bytes apart
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(red + kWarps * 32 * 4) + (uint32_t)(warp * kStages * 2 * 32 + lane) * 16u;

  const int tile = blockIdx.x * (kWarps >> KSL) + (warp >> KSL);
  const int kpart = warp & (KS - 1);
  const int row_lo = min(tile * kTileRows + g, N - 1);      // rows past N: clamped loads, never stored
  const int row_hi = min(tile * kTileRows + g + 8, N - 1);
  const int words_per_row = K / 8;
  // everything below points at round kpart and advances by kStages rounds of this warp per loop trip
  const uint32_t* pw_lo = packed + (size_t)row_lo * words_per_row + t * W + kpart * (G / 8);
  const uint32_t* pw_hi = packed + (size_t)row_hi * words_per_row + t * W + kpart * (G / 8);
  const __half* ps_lo = scales + (size_t)row_lo * rounds + kpart;
  const __half* ps_hi = scales + (size_t)row_hi * rounds + kpart;
  const __half* px = x + (size_t)min(g, M - 1) * K + t * kLaneK + kpart * G;   // column g of the B operand
  const float* psx = sx + kpart * 16 + t * 4;                                  // columns 2t, 2t+1: (A, B, A, B)
  // rounds of this warp: rd(i) = kpart + i * KS, i < n_i (none for a tile past N)
  const int n_i = tile * kTileRows < N ? (rounds - kpart + KS - 1) >> KSL : 0;

  // the weight stream starts before anything else: the class sums below run under its latency
#pragma unroll
  for (int u = 0; u < kStages; ++u) {
    if (u < n_i) {
      if constexpr (W == 4) {
        cp_async16(ring + u * kSlot, pw_lo + u * kWStep);
        cp_async16(ring + u * kSlot + 32 * 16, pw_hi + u * kWStep);
      } else {
        cp_async8(ring + u * kSlot, pw_lo + u * kWStep);
        cp_async8(ring + u * kSlot + 32 * 16, pw_hi + u * kWStep);
      }
    }
    cp_async_commit();   // always: group i <-> round i
  }

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

  float acc[4] = {0.f, 0.f, 0.f, 0.f};   // rows g, g+8 x columns 2t, 2t+1
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i0 = 0; i0 < n_i; i0 += kStages) {
#pragma unroll
    for (int u = 0; u < kStages; ++u) {
      if (i0 + u < n_i) {   // warp-uniform
        const float s_lo = __half2float(ps_lo[u * KS]), s_hi = __half2float(ps_hi[u * KS]);
        uint32_t xs[W * 4];
#pragma unroll
        for (int j = 0; j < W; ++j) {
          const uint4 v = *reinterpret_cast<const uint4*>(px + u * kXStep + j * 8);
          xs[4 * j + 0] = v.x; xs[4 * j + 1] = v.y; xs[4 * j + 2] = v.z; xs[4 * j + 3] = v.w;
        }
        cp_async_wait<kStages - 1>();   // round i0 + u has landed (this lane's own copies)
        uint32_t wlo[W], whi[W];
        if constexpr (W == 4) {
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wlo[0]), "=r"(wlo[1]), "=r"(wlo[2]), "=r"(wlo[3]) : "r"(ring + u * kSlot));
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(whi[0]), "=r"(whi[1]), "=r"(whi[2]), "=r"(whi[3]) : "r"(ring + u * kSlot + 32 * 16));
        } else {
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(wlo[0]), "=r"(wlo[1]) : "r"(ring + u * kSlot));
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(whi[0]), "=r"(whi[1]) : "r"(ring + u * kSlot + 32 * 16));
        }
        float ca[4], cb[4];
        constexpr uint32_t kMagic = 0x64006400u;
#pragma unroll
        for (int j = 0; j < W; ++j) {
          const uint32_t lo = wlo[j], hi = whi[j], lo8 = lo >> 8, hi8 = hi >> 8;
          // xs[4j + p] holds the activation pair multiplied by nibble pair p of word j
          mma16816_f16(ca, (lo & 0x000F000Fu) | kMagic, (hi & 0x000F000Fu) | kMagic, (lo8 & 0x000F000Fu) | kMagic,
                       (hi8 & 0x000F000Fu) | kMagic, xs[4 * j + 0], xs[4 * j + 2], j == 0 ? zero : ca);
          mma16816_f16(cb, (lo & 0x00F000F0u) | kMagic, (hi & 0x00F000F0u) | kMagic, (lo8 & 0x00F000F0u) | kMagic,
                       (hi8 & 0x00F000F0u) | kMagic, xs[4 * j + 1], xs[4 * j + 3], j == 0 ? zero : cb);
        }
        // the slot is free again (its words sit in the MMA operands): request the round kStages ahead
        if (i0 + kStages + u < n_i) {
          if constexpr (W == 4) {
            cp_async16(ring + u * kSlot, pw_lo + (kStages + u) * kWStep);
            cp_async16(ring + u * kSlot + 32 * 16, pw_hi + (kStages + u) * kWStep);
          } else {
            cp_async8(ring + u * kSlot, pw_lo + (kStages + u) * kWStep);
            cp_async8(ring + u * kSlot + 32 * 16, pw_hi + (kStages + u) * kWStep);
          }
        }
        cp_async_commit();
        // remove the offsets of the unsigned forms and apply the group scale
        const float4 c = *reinterpret_cast<const float4*>(psx + u * kSxStep);   // column 2t: (A, B), column 2t+1: (A, B)
        acc[0] = fmaf(s_lo, (ca[0] + c.x) + fmaf(cb[0], 0.0625f, c.y), acc[0]);
        acc[1] = fmaf(s_lo, (ca[1] + c.z) + fmaf(cb[1], 0.0625f, c.w), acc[1]);
        acc[2] = fmaf(s_hi, (ca[2] + c.x) + fmaf(cb[2], 0.0625f, c.y), acc[2]);
        acc[3] = fmaf(s_hi, (ca[3] + c.z) + fmaf(cb[3], 0.0625f, c.w), acc[3]);
      }
    }
    pw_lo += kStages * kWStep;
    pw_hi += kStages * kWStep;
    ps_lo += kStages * KS;
    ps_hi += kStages * KS;
    px += kStages * kXStep;
    psx += kStages * kSxStep;
  }
  cp_async_wait<0>();

  if constexpr (KSL != 0) {
    __syncthreads();
    float4* mine = reinterpret_cast<float4*>(red + (warp * 32 + lane) * 4);
    *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (kpart != 0) return;
    for (int p = 1; p < KS; ++p) {  // fixed order
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

template <int G, int KSL>
int launch_ks(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, int grid, size_t smem,
              cudaStream_t stream) {
  static bool attr_done[64] = {};   // per device: opt in to more than 48 KB of dynamic shared memory
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !attr_done[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(int4_gemv_mma_kernel<G, KSL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev] = true;
  }
  int4_gemv_mma_kernel<G, KSL><<<grid, kThreads, smem, stream>>>((const __half*)x, (const uint32_t*)packed, (const __half*)scales,
                                                                 (__half*)y, M, N, K);
  KFB_LAUNCH_CHECK("int4_gemv_mma_kernel");
  return KFB_OK;
}

template <int G>
int launch(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, cudaStream_t stream) {
  const int rounds = K / G;
  const int tiles = ceil_div(N, kTileRows);
  // split K over the warps of a CTA until the grid offers about 16 warps per SM (never more warps than rounds)
  int ksl = 0;
  const long long want = 16LL * sm_count();
  while (ksl < 3 && (long long)tiles * (1 << ksl) < want && (2 << ksl) <= rounds) ++ksl;
  const int grid = ceil_div(tiles, kWarps >> ksl);
  const size_t smem = smem_bytes(rounds);
  if (smem > 200 * 1024) return fail(KFB_ERR_UNSUPPORTED, "K=%d needs %zu bytes of shared memory for the class sums", K, smem);
  switch (ksl) {
    case 0: return launch_ks<G, 0>(x, packed, scales, y, M, N, K, grid, smem, stream);
    case 1: return launch_ks<G, 1>(x, packed, scales, y, M, N, K, grid, smem, stream);
    case 2: return launch_ks<G, 2>(x, packed, scales, y, M, N, K, grid, smem, stream);
    default: return launch_ks<G, 3>(x, packed, scales, y, M, N, K, grid, smem, stream);
  }
}

}  // namespace gemv_mma
}  // namespace kfb
