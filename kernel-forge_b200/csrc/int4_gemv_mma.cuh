// INT4 GEMV (M = 1..8, and up to 32 batch rows through the small-batch entry) with the dot products on mma.sync
// fragments.
//
// Why this exists: on B200 the CUDA-core GEMV (int4_gemv.cu) is issue-bound, not HBM-bound -- logic/shift ops
// issue at half the FP32 rate, so unpack + one FMA per weight + operand extraction cost ~3 issue slots per weight
// against a budget of 2.8 at the full HBM rate (ncu: issue slots 63 % busy, ALU pipe 57 %, DRAM 41 %).  Here the
// multiply-accumulate of 16 rows x 16 k x 8 batch columns is ONE instruction, which leaves the unpack (5 logic ops per
// 8 weights) as the only per-weight work: ~0.6 issue slots per weight, the same for every M up to 8.
//
// What limits the kernel after that, in the order it was measured (ncu, N = 180224, K = 2048):
//  1. bytes in flight per SM -> the weight stream is staged through shared memory, several rounds ahead per warp;
//  2. the integer pipe (logic and shift instructions issue at half rate on B200): address arithmetic and predication
//     cost more than the unpack itself -> everything inside a chunk is addressed as pointer + immediate, accumulators
//     start from the zero register, batch columns past M read a valid row instead of being zero-filled (a column of
//     the MMA result depends on its own column of the activations only, and those columns are never stored);
//  3. the L1 tag stage (one 128-byte line per clock per SM): per-lane 16-byte loads of 16 different rows touch 8
//     lines per instruction -> the weights are fetched by the TMA unit instead (no LSU involvement), scales are
//     loaded a chunk at a time as one vector per row, and a warp may own two MMA row tiles that share every
//     activation fragment;
//  4. the request rate of the TMA unit: untiled bulk copies of 256 bytes (one per row) stop at ~2.5 TB/s, i.e. one
//     request per ~29 clocks per SM -> one tiled copy (tensor map over the packed matrix, box = R rows x 128 bytes)
//     per warp and chunk, 2 or 4 KB per request;
//  5. tail and prologue: with one CTA per 256 rows the last wave of CTAs is partly empty (2.4 waves at N = 180224:
//     21 % of the time) and every CTA waits ~2 us at the barrier behind the class sums -> for large N the kernel
//     is persistent (one CTA of 16 warps per SM, class sums once), the tiles are split evenly over the CTAs, the warps
//     of a CTA take pairs of tiles and finally single tiles from a shared-memory counter, and a warp's ring keeps
//     streaming across tile boundaries;
//  6. the memory system: with all of that the SMs wait for data (~5 us of queueing at 8-12 KB in flight per warp);
//     two stages per warp instead of three are faster (less queueing, more L1 left for the activations).  What is
//     left at N = 180224 is ~10 us of launch, class sums, ramp and tail per launch (72 % of the copy peak; 88 % on
//     763 MB);
//  7. the activations: read through L1 every round they make the kernel slower the larger M is (the ring leaves L1
//     little room) -> for M >= 2 the persistent kernel copies x to shared memory once, in fragment order, and M = 8
//     then runs at the speed of M = 1 (87 % of the copy peak on 763 MB).
//
// Shared-memory stage of a warp: R = 16 or 32 rows x 128 bytes (2 rounds of G = 128, 4 of G = 64), written by the TMA
// with the 128-byte swizzle (16-byte piece j of row r sits at piece j ^ (r & 7)).  Fragment row slot g of a tile
// holds matrix row p(g) = 4 (g & 1) + (g >> 1) (and p(g) + 8): the eight lanes of one 128-bit shared load then read
// rows q and q + 4, whose swizzled pieces lie in opposite 64-byte halves, so every load covers all 32 banks.  One
// lane issues the copy; a stage is re-issued by the same warp after __syncwarp(), so there is no consumer ->
// producer barrier.  Rows past N and bytes past K/2 are zero-filled by the TMA.
//
// Arithmetic.  Masking a word in place gives exact fp16 values with the nibble in the mantissa: pairs 0 and 2 of a
// word (k offsets 0,1 / 4,5) as (w & 0x000F000F) | 0x7400.. = 16384 + 16 u, pairs 1 and 3 (k offsets 2,3 / 6,7) as
// (w & 0x00F000F0) | 0x6400.. = 1024 + 16 u.  Both carry 16 u, so all of them go into the same accumulator (fp16 x fp16
// products are exact, FP32 accumulation).  The first form sits 128 times above its signal (16384 against 16 u ~ 128):
// left in, a one-signed x (post-ReLU inputs, a large mean) drives the accumulator to ~1e6 |x| and the truncating FP32
// accumulation of the tensor core shows as a systematic bias of ~4e-4 of the result (measured).  So that form is
// turned into 16 q = 16 (u - 8) with one half2 subtraction (exact); the second form, 8 times above its signal, stays.
// Per scale group
//     sum_k q x = acc / 16 - 72 * SxB,
// with SxB the sum of the activations that meet pairs 1,3 in that group (it depends on x only and is computed once
// per CTA).  The group scale is applied in FP32, one rounding to fp16 at the end.  An MMA takes pairs (0, 1) or (2, 3) of one word, so its B operand is two consecutive registers of the
// 16-byte activation vector.
//
// Fragment use (m16n8k16, A = weights row-major 16 rows x 16 k, B = activations, 8 columns = batch rows):
//   lane = 4 g + t.  The lane consumes rows g and g + 8 of a tile; per round (one scale group of 128 k, or 64 k when
//   G = 64) it reads G/32 packed words of each row, its k range being 32 t .. 32 t + 31 (16 t .. when G = 64) of the
//   group.  For word j: a0/a1 = pair 0 of the two rows, a2/a3 = pair 1 -> first MMA;  pairs 2 and 3 -> second MMA.
//   The k positions an MMA multiplies are whatever the four lanes t = 0..3 put in the same fragment slots, so the B
//   fragment of lane (g, t) is simply the same pairs of x[m = g] at this lane's k range -- any consistent assignment
//   of k to fragment slots gives the same dot product.
#pragma once

#include "common.cuh"
#include "sm100.cuh"

#include <type_traits>

namespace kfb {
namespace gemv_mma {

using namespace kfb::sm100;

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kTileRows = 16;
constexpr int kChunkBytes = 128;       // bytes of one weight row per stage (the span of the 128-byte swizzle)
constexpr uint32_t kWaitStage = 0x501; // status code of an expired wait

// d = a * b + c, m16n8k16, fp16 operands, FP32 accumulation
__device__ __forceinline__ void mma16816_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1, const float* c) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// (a & mask) | magic as ONE logic instruction.  Written with literal constants the compiler emits two (a LOP3 takes a
// single immediate), which doubled the integer-pipe load of the unpack; the constants therefore arrive as a kernel
// argument and stay in registers.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(magic));
  return d;
}

// (16384 + 16 u) - 16512 = 16 (u - 8) = 16 q on both halves, exact in fp16.  One half2 subtraction on the FMA pipe,
// which this kernel leaves idle (its limit is the integer pipe).
__device__ __forceinline__ uint32_t sub_offset_a(uint32_t a) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(0x74087408u));
  return d;
}

// Bounded wait for a stage.  Unlike sm100::mbar_wait it sleeps between polls: several chunks are in flight per warp,
// so a late wake-up costs nothing, while a polling warp would take issue slots and integer-pipe cycles from the warps
// that have data.
__device__ __forceinline__ bool wait_stage(uint64_t* bar, uint32_t parity, const AbortCtx& ctx) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    __nanosleep(100);
    if ((++spins & 255u) == 0) {
      if (*ctx.cta_word != 0) return false;
      if (globaltimer_ns() - t0 > kWaitTimeoutNs) {
        *ctx.cta_word = kWaitStage;
        atomicCAS(ctx.device_word, 0u, kWaitStage);
        return false;
      }
    }
  }
  return true;
}

// Shared memory of a CTA: (ring, 1024-byte aligned: kWarps x S stages of RT row tiles) | mbarriers | abort word |
// class sums.  The split-K reduction reuses the ring.
__host__ __device__ constexpr uint32_t stage_bytes(int RT) { return (uint32_t)(kTileRows * RT * kChunkBytes); }
__host__ __device__ constexpr size_t sx_offset(int RT, int S) { return (size_t)kWarps * S * stage_bytes(RT) + kWarps * S * 8 + 16; }
inline size_t smem_bytes(int RT, int S, int rounds, int NB) { return 1024 + sx_offset(RT, S) + (size_t)rounds * 8 * NB * sizeof(float); }

// What a lane needs to find its words and its activations; the same for every tile.
// NB: blocks of 8 batch columns (M <= 8 NB); every block is one more MMA on the same unpacked weight fragment.
template <int G, int NB = 1>
struct LaneMap {
  static constexpr int W = G / 32;                   // packed words per lane per row per round
  static constexpr int C = kChunkBytes / (G / 2);    // rounds per chunk (2 or 4)
  int g, t, pg;         // lane = 4 g + t; fragment row slot g holds matrix rows pg + 8 k of the warp's rows
  uint32_t off[C];      // position of this lane's words of round u inside a stage (row pg, swizzled 16-byte piece)
  const __half* xrow[NB];   // column 8 nb + g of the B operand (a valid row when >= M), at this lane's k offset
  // optional copy of x in shared memory in fragment order (NB = 1): unit ((round * W + j) * Mp + m) * 4 + t holds the 16
  // bytes lane (m, t) needs for word j of that round, so the 32 lanes of a load read consecutive units
  const uint4* xs_lane = nullptr;
  int xs_shift = 0;         // log2(4 * Mp): units per (round, word)
  __device__ __forceinline__ LaneMap(int lane, const __half* x, int M, int K) {
    g = lane >> 2;
    t = lane & 3;
    pg = ((g & 1) << 2) | (g >> 1);
#pragma unroll
    for (int u = 0; u < C; ++u) {
      const uint32_t byte = (uint32_t)u * (G / 2) + (uint32_t)t * (W * 4);
      off[u] = (uint32_t)pg * kChunkBytes + ((((byte >> 4) ^ (uint32_t)pg) << 4) | (byte & 15u));
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) xrow[nb] = x + (size_t)min(8 * nb + g, M - 1) * K + t * (G / 4);
  }
};

// Class sums of the activations, once per CTA: sx[round][column < 8 NB] = -72 SxB.  Four lanes share one (round,
// batch row): each sums a quarter of the group (whole packed words: pairs 1, 3 of a word meet the 1024 + 16 u form),
// then a quad reduction.  Ends with the CTA barrier.
template <int G, int NB>
__device__ __forceinline__ void class_sums(const __half* __restrict__ x, int M, int K, float* sx) {
  const int rounds = K / G;
  for (int i = threadIdx.x; i < rounds * 8 * NB; i += blockDim.x)
    if ((i & (8 * NB - 1)) >= M) sx[i] = 0.f;
  const int q = threadIdx.x & 3, items = rounds * M;
  for (int base = 0; base < items; base += blockDim.x / 4) {
    const int item = base + (threadIdx.x >> 2);
    const bool live = item < items;
    const int rd = live ? item / M : 0, m = live ? item - rd * M : 0;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)rd * G + q * (G / 4));
    float sb = 0.f;
    if (live) {
#pragma unroll
      for (int i = 0; i < G / 32; ++i) {
        const uint4 v = xr[i];
        const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        sb += (p1.x + p1.y) + (p3.x + p3.y);
      }
    }
    sb += __shfl_xor_sync(0xffffffffu, sb, 1);
    sb += __shfl_xor_sync(0xffffffffu, sb, 2);
    if (live && q == 0) sx[rd * 8 * NB + m] = sb * -72.0f;
  }
  __syncthreads();
}

// Group scales of one chunk for this lane's 2 T rows, raw fp16 bits: sc[k][u / 2] holds rounds u (low half), u + 1.
// `vec`: every chunk is full and the scale rows are aligned, so a chunk's scales are one vector load per row.
template <int G, int T>
__device__ __forceinline__ void load_scales(const __half* const (&srow)[2 * T], int r0, int nr, int vec,
                                            uint32_t (&sc)[2 * T][LaneMap<G>::C / 2]) {
  constexpr int C = LaneMap<G>::C;
  if (vec) {
#pragma unroll
    for (int k = 0; k < 2 * T; ++k) {
      if constexpr (C == 2) {
        sc[k][0] = *reinterpret_cast<const uint32_t*>(srow[k] + r0);
      } else {
        const uint2 v = *reinterpret_cast<const uint2*>(srow[k] + r0);
        sc[k][0] = v.x; sc[k][1] = v.y;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 2 * T; ++k)
#pragma unroll
      for (int u = 0; u < C; u += 2) {
        const uint32_t a = u < nr ? (uint32_t)__half_as_ushort(srow[k][r0 + u]) : 0u;
        const uint32_t b = u + 1 < nr ? (uint32_t)__half_as_ushort(srow[k][r0 + u + 1]) : 0u;
        sc[k][u / 2] = a | (b << 16);
      }
  }
}

// One chunk (C rounds) of T row tiles out of the stage at shared address `st` (already complete).  `refill` runs once
// every shared load of the stage has delivered, i.e. as early as the stage may be handed back to the TMA.
template <int G, int T, int RG, int NB, bool XS = false, class Refill>
__device__ __forceinline__ void chunk_compute(const LaneMap<G, NB>& lm, uint32_t st, const float* sx, int r0, int nr,
                                              const uint32_t (&sc)[2 * T][LaneMap<G>::C / 2], const uint4& unpack,
                                              float (&acc)[T][NB][4], Refill&& refill) {
  constexpr int W = LaneMap<G>::W, C = LaneMap<G>::C;
  static_assert(C % RG == 0, "rounds per chunk must be a multiple of the round group");
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t kMaskA = unpack.x, kMaskB = unpack.y, kMagicA = unpack.z, kMagicB = unpack.w;
  // Rounds are computed RG (1 or 2) at a time.  Rounds past the end of K (last chunk only; their weights are TMA zero
  // fill and their scales zero) read the activations of the chunk's first round instead of running past x.
#pragma unroll
  for (int h = 0; h < C; h += RG) {
    int xoff[RG];      // element offset of the round in a row of x
    float2 cs[RG][NB]; // corrections of columns 8 nb + 2t, + 1
    uint32_t w[RG][2 * T][W];
#pragma unroll
    for (int v = 0; v < RG; ++v) {
      const int ue = h + v < nr ? h + v : 0;
      xoff[v] = (r0 + ue) * G;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
        cs[v][nb] = *reinterpret_cast<const float2*>(sx + (r0 + ue) * (8 * NB) + 8 * nb + lm.t * 2);
#pragma unroll
      for (int k = 0; k < 2 * T; ++k) {
        const uint32_t a = st + lm.off[h + v] + k * 8 * kChunkBytes;
        if constexpr (W == 4)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[v][k][0]), "=r"(w[v][k][1]), "=r"(w[v][k][2]), "=r"(w[v][k][3]) : "r"(a));
        else
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[v][k][0]), "=r"(w[v][k][1]) : "r"(a));
      }
    }
    // kAcc accumulators per (round, tile, column block).  The MMAs are issued word by word and half word by half
    // word across all of those, so that two MMAs on the same accumulator are RG * T * NB * kAcc MMAs apart (asm
    // volatile keeps this order).  A weight fragment is unpacked once and multiplied with every column block.
    constexpr int kAcc = T * RG * NB >= 4 ? 1 : 2;
    float ca[RG][T][NB][kAcc][4];
#pragma unroll
    for (int j = 0; j < W; ++j) {
      uint4 xv[RG][NB];   // .x .y .z .w: the activation pairs multiplied by nibble pairs 0..3 of word j
#pragma unroll
      for (int v = 0; v < RG; ++v)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          if constexpr (XS) xv[v][nb] = lm.xs_lane[(size_t)((xoff[v] / G) * W + j) << lm.xs_shift];
          else xv[v][nb] = *reinterpret_cast<const uint4*>(lm.xrow[nb] + xoff[v] + j * 8);
        }
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int v = 0; v < RG; ++v)
#pragma unroll
          for (int tt = 0; tt < T; ++tt) {
            const uint32_t lo = w[v][2 * tt][j] >> (8 * half), hi = w[v][2 * tt + 1][j] >> (8 * half);
            const uint32_t a0 = sub_offset_a(and_or(lo, kMaskA, kMagicA)), a1 = sub_offset_a(and_or(hi, kMaskA, kMagicA));
            const uint32_t a2 = and_or(lo, kMaskB, kMagicB), a3 = and_or(hi, kMaskB, kMagicB);
            const bool first = j == 0 && half < kAcc;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              float(&c)[4] = ca[v][tt][nb][half % kAcc];
              mma16816_f16(c, a0, a1, a2, a3, half ? xv[v][nb].z : xv[v][nb].x, half ? xv[v][nb].w : xv[v][nb].y, first ? zero : c);
            }
          }
      if (j == 0 && h + RG >= C) refill();   // each shared load's first word has just been consumed
    }
    // remove the offsets of the unsigned forms and apply the group scale
#pragma unroll
    for (int v = 0; v < RG; ++v)
#pragma unroll
      for (int tt = 0; tt < T; ++tt) {
        const int u = h + v;
        const __half2 s2lo = *reinterpret_cast<const __half2*>(&sc[2 * tt][u / 2]);
        const __half2 s2hi = *reinterpret_cast<const __half2*>(&sc[2 * tt + 1][u / 2]);
        const float s_lo = (u & 1) ? __high2float(s2lo) : __low2float(s2lo);
        const float s_hi = (u & 1) ? __high2float(s2hi) : __low2float(s2hi);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float d[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) d[e] = kAcc == 2 ? ca[v][tt][nb][0][e] + ca[v][tt][nb][kAcc - 1][e] : ca[v][tt][nb][0][e];
          acc[tt][nb][0] = fmaf(s_lo, fmaf(d[0], 0.0625f, cs[v][nb].x), acc[tt][nb][0]);
          acc[tt][nb][1] = fmaf(s_lo, fmaf(d[1], 0.0625f, cs[v][nb].y), acc[tt][nb][1]);
          acc[tt][nb][2] = fmaf(s_hi, fmaf(d[2], 0.0625f, cs[v][nb].x), acc[tt][nb][2]);
          acc[tt][nb][3] = fmaf(s_hi, fmaf(d[3], 0.0625f, cs[v][nb].y), acc[tt][nb][3]);
        }
      }
  }
}

// Stores rows row0 + pg, row0 + pg + 8 of columns col0 + 2t, + 1 (acc = {row lo col 2t, row lo col 2t+1, row hi ...}).
__device__ __forceinline__ void store_tile(__half* __restrict__ y, const float (&acc)[4], int row0, int col0, int pg, int t, int M,
                                           int N) {
  const int ra = row0 + pg, rb = ra + 8, m0 = col0 + 2 * t, m1 = m0 + 1;
  if (m0 < M) {
    if (ra < N) y[(size_t)m0 * N + ra] = __float2half_rn(acc[0]);
    if (rb < N) y[(size_t)m0 * N + rb] = __float2half_rn(acc[2]);
  }
  if (m1 < M) {
    if (ra < N) y[(size_t)m1 * N + ra] = __float2half_rn(acc[1]);
    if (rb < N) y[(size_t)m1 * N + rb] = __float2half_rn(acc[3]);
  }
}

__device__ __forceinline__ void linger_after_abort(volatile uint32_t* abort_word) {
  if (*abort_word != 0) {   // a wait expired: give the copies still in flight time to land before the CTA retires
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Kernel for small and medium N: one 16-row tile per warp, KS = 1 << KSL warps of a CTA share a tile and take chunks
// kpart, kpart + KS, ... ; partial sums meet in shared memory in a fixed order.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kSplitStages = 4;   // 8 KB in flight per warp

template <int G, int KSL, int NB>
__global__ void __launch_bounds__(kThreads, 2)
int4_gemv_mma_split_kernel(const __half* __restrict__ x, const __grid_constant__ CUtensorMap wmap16,
                           const __half* __restrict__ scales, __half* __restrict__ y, int M, int N, int K, int vec_scales,
                           unsigned int* status, const uint4 unpack) {
  constexpr int C = LaneMap<G>::C, KS = 1 << KSL, S = kSplitStages;
  constexpr uint32_t kStage = stage_bytes(1);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // the swizzle pattern is 1024-byte periodic
  const int rounds = K / G;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kWarps * S * kStage);
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(bars + kWarps * S);
  float* sx = reinterpret_cast<float*>(smem + sx_offset(1, S));
  float* red = reinterpret_cast<float*>(smem);   // [kWarps][32 lanes][NB][4], after the main loop
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int tile = blockIdx.x * (kWarps >> KSL) + (warp >> KSL);
  const int kpart = warp & (KS - 1);
  const int row0 = tile * kTileRows;
  // chunks of this warp: c(i) = kpart + i * KS, i < n_c (none for a tile past N)
  const int n_chunks = (rounds + C - 1) / C;
  const int n_c = row0 < N ? (n_chunks - kpart + KS - 1) >> KSL : 0;

  uint64_t* my_bars = bars + warp * S;
  const uint32_t my_ring = smem_u32(smem) + (uint32_t)warp * S * kStage;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(&my_bars[s], 1);
    fence_mbar_init();
  }
  if (threadIdx.x == 0) *abort_word = 0;
  __syncwarp();

  auto issue = [&](int i) {   // one tiled copy: 16 rows x 128 bytes of chunk c(i)
    if (lane == 0) {
      const int c = kpart + (i << KSL), st = i % S;
      mbar_arrive_expect_tx(&my_bars[st], kStage);
      tma_load_2d(smem + (size_t)(warp * S + st) * kStage, &wmap16, &my_bars[st], c * (kChunkBytes / 4), row0);
    }
  };
  // the weight stream starts before anything else: the class sums below run under its latency
#pragma unroll
  for (int i = 0; i < S; ++i)
    if (i < n_c) issue(i);
  pdl_wait();   // the kernel before this one has finished: x may be its output, y may be its input
  pdl_launch_dependents();

  class_sums<G, NB>(x, M, K, sx);

  const AbortCtx ctx{abort_word, status};
  const LaneMap<G, NB> lm(lane, x, M, K);
  float acc[1][NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) acc[0][nb][0] = acc[0][nb][1] = acc[0][nb][2] = acc[0][nb][3] = 0.f;
  const __half* srow[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) srow[k] = scales + (size_t)min(row0 + lm.pg + 8 * k, N - 1) * rounds;

  for (int i = 0; i < n_c; ++i) {
    const int r0 = (kpart + (i << KSL)) * C, nr = min(C, rounds - r0);
    uint32_t sc[2][C / 2];
    load_scales<G, 1>(srow, r0, nr, vec_scales, sc);
    if (!__all_sync(0xffffffffu, wait_stage(&my_bars[i % S], (uint32_t)(i / S) & 1u, ctx))) break;
    chunk_compute<G, 1, (NB <= 2 ? 2 : 1), NB>(lm, my_ring + (uint32_t)(i % S) * kStage, sx, r0, nr, sc, unpack, acc, [&] {
      __syncwarp();
      if (i + S < n_c) issue(i + S);
    });
  }
  linger_after_abort(abort_word);

  if constexpr (KSL != 0) {
    __syncthreads();   // all warps are past their last stage: the ring becomes the reduction buffer
    float4* mine = reinterpret_cast<float4*>(red + (size_t)(warp * 32 + lane) * NB * 4);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) mine[nb] = make_float4(acc[0][nb][0], acc[0][nb][1], acc[0][nb][2], acc[0][nb][3]);
    __syncthreads();
    if (kpart != 0) return;
    for (int p = 1; p < KS; ++p) {  // fixed order
      const float4* o = reinterpret_cast<const float4*>(red + (size_t)((warp + p) * 32 + lane) * NB * 4);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        acc[0][nb][0] += o[nb].x; acc[0][nb][1] += o[nb].y; acc[0][nb][2] += o[nb].z; acc[0][nb][3] += o[nb].w;
      }
    }
  }
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) store_tile(y, acc[0][nb], row0, 8 * nb, lm.pg, lm.t, M, N);
}

// ---------------------------------------------------------------------------------------------------------------
// Kernel for large N: persistent, NW warps per CTA.  The 16-row tiles are split evenly over the CTAs (contiguous
// ranges); inside a CTA the warps take work units from a shared-memory counter: first pairs of tiles (one 32-row copy
// per chunk, activation fragments shared by both tiles), at the end single tiles, so that the warps of a CTA finish
// within one single-tile time of each other whatever service each of them got from the memory system.  A warp's ring
// runs ahead across unit boundaries: the producer side takes the next unit as soon as it has requested the last
// chunk of the current one and passes it to the consumer side through a small queue.
// ---------------------------------------------------------------------------------------------------------------
template <int NW, int S_ = 3>
struct StreamSmem {   // offsets from the 1024-byte aligned base
  static constexpr int S = S_;                                  // 4 KB in flight per warp and stage
  static constexpr uint32_t kStage = stage_bytes(2);
  static constexpr size_t bars = (size_t)NW * S * kStage;       // uint64_t[NW * S]
  static constexpr size_t abort_word = bars + (size_t)NW * S * 8;
  static constexpr size_t counter = abort_word + 4;             // next unit of the CTA
  static constexpr size_t queue = abort_word + 16;              // int[NW][4]: units taken by a warp's producer side
  static constexpr size_t sx = queue + (size_t)NW * 16;
  static size_t bytes(int rounds, int NB, size_t xs_bytes = 0) { return 1024 + sx + (size_t)rounds * 8 * NB * sizeof(float) + xs_bytes; }
};

// XS: the activations are copied to shared memory in fragment order once per CTA (Mp = M rounded up to a power of two
// columns); without it every round reads them through L1, which makes the kernel slower the larger M is.
template <int G, int RG, int NW, int MINB, int NS, int NB, bool XS = false>
__global__ void __launch_bounds__(NW * 32, MINB)
int4_gemv_mma_stream_kernel(const __half* __restrict__ x, const __grid_constant__ CUtensorMap wmap32,
                            const __grid_constant__ CUtensorMap wmap16, const __half* __restrict__ scales,
                            __half* __restrict__ y, int M, int N, int K, int vec_scales, unsigned int* status,
                            const uint4 unpack, unsigned long long* trace, int mp_log2) {
  static_assert(!XS || NB == 1, "the shared-memory copy of x is laid out for one column block");
  using L = StreamSmem<NW, NS>;
  constexpr int C = LaneMap<G>::C, S = L::S;
  constexpr uint32_t kStage = L::kStage;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int rounds = K / G;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bars);
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem + L::abort_word);
  int* counter = reinterpret_cast<int*>(smem + L::counter);
  float* sx = reinterpret_cast<float*>(smem + L::sx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* my_queue = reinterpret_cast<volatile int*>(smem + L::queue) + warp * 4;
  // optional timeline for tuning: per warp (start, class sums done, end) in ns and the SM id
#ifdef KFB_TRACE
  unsigned long long* tr = trace != nullptr && lane == 0 ? trace + (size_t)(blockIdx.x * NW + warp) * 4 : nullptr;
#else
  constexpr unsigned long long* tr = nullptr;
#endif
  if (tr) {
    uint32_t smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    tr[0] = globaltimer_ns();
    tr[3] = smid;
  }

  // this CTA's range of 16-row tiles: tiles / grid each, the remainder spread evenly over the grid
  const int tiles = (N + kTileRows - 1) / kTileRows;
  const int base = tiles / (int)gridDim.x, extra = tiles - base * (int)gridDim.x;
  const int ex0 = (int)(((long long)blockIdx.x * extra) / gridDim.x), ex1 = (int)(((long long)(blockIdx.x + 1) * extra) / gridDim.x);
  const int first = blockIdx.x * base + ex0, count = base + (ex1 - ex0);
  // units: n_pairs pairs, then n_single single tiles (about one per warp, parity adjusted)
  const int n_single = min(count, NW + ((count - NW) & 1));
  const int n_pairs = (count - n_single) >> 1, n_units = n_pairs + n_single;
  auto unit_tile = [&](int u) { return first + (u < n_pairs ? 2 * u : 2 * n_pairs + (u - n_pairs)); };
  const int n_chunks = (rounds + C - 1) / C;

  uint64_t* my_bars = bars + warp * S;
  const uint32_t my_ring = smem_u32(smem) + (uint32_t)warp * S * kStage;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(&my_bars[s], 1);
    fence_mbar_init();
  }
  if (threadIdx.x == 0) {
    *abort_word = 0;
    *counter = NW;   // units 0 .. NW-1 are the warps' first units
  }
  __syncthreads();

  // producer side: the unit being requested, its next chunk, copies requested so far, units taken so far
  int p_unit = warp, p_chunk = 0, p_count = 0, p_taken = 1;
  if (lane == 0) my_queue[0] = p_unit;
  auto issue_next = [&]() {
    if (p_unit >= n_units) return;
    if (lane == 0) {
      const int st = p_count % S;
      const bool single = p_unit >= n_pairs;
      mbar_arrive_expect_tx(&my_bars[st], single ? stage_bytes(1) : kStage);
      tma_load_2d(smem + (size_t)(warp * S + st) * kStage, single ? &wmap16 : &wmap32, &my_bars[st], p_chunk * (kChunkBytes / 4),
                  unit_tile(p_unit) * kTileRows);
    }
    ++p_count;
    if (++p_chunk == n_chunks) {   // take the next unit of the CTA
      p_chunk = 0;
      int u = 0;
      if (lane == 0) {
        u = atomicAdd(counter, 1);
        my_queue[p_taken & 3] = u;
      }
      p_unit = __shfl_sync(0xffffffffu, u, 0);
      ++p_taken;
    }
  };
#pragma unroll
  for (int i = 0; i < S; ++i) issue_next();
  pdl_wait();   // the kernel before this one has finished: x may be its output, y may be its input
  pdl_launch_dependents();

  uint4* xs = reinterpret_cast<uint4*>(sx + (size_t)rounds * 8 * NB);   // 16-byte aligned: rounds * 32 NB bytes after sx
  if constexpr (XS) {
    constexpr int W = LaneMap<G>::W;
    const int units = (rounds * W) << (2 + mp_log2);
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
      const int t4 = u & 3, m = (u >> 2) & ((1 << mp_log2) - 1), jj = u >> (2 + mp_log2);
      const int rd = jj / W, j = jj - rd * W;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < M) v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)rd * G + t4 * (G / 4) + j * 8);
      xs[u] = v;
    }
  }
  class_sums<G, NB>(x, M, K, sx);   // ends with the CTA barrier, which also publishes xs
  if (tr) tr[1] = globaltimer_ns();

  const AbortCtx ctx{abort_word, status};
  LaneMap<G, NB> lm(lane, x, M, K);
  if constexpr (XS) {
    lm.xs_shift = 2 + mp_log2;
    lm.xs_lane = xs + ((lm.g & ((1 << mp_log2) - 1)) << 2) + lm.t;
  }
  int q = 0;   // copies consumed
  bool ok = true;
  auto run_unit = [&](auto tag, int row0) {
    constexpr int T = decltype(tag)::value;
    float acc[T][NB][4];
#pragma unroll
    for (int tt = 0; tt < T; ++tt)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) acc[tt][nb][0] = acc[tt][nb][1] = acc[tt][nb][2] = acc[tt][nb][3] = 0.f;
    const __half* srow[2 * T];
#pragma unroll
    for (int k = 0; k < 2 * T; ++k) srow[k] = scales + (size_t)min(row0 + lm.pg + 8 * k, N - 1) * rounds;
    for (int ci = 0; ci < n_chunks; ++ci, ++q) {
      const int r0 = ci * C, nr = min(C, rounds - r0);
      uint32_t sc[2 * T][C / 2];
      load_scales<G, T>(srow, r0, nr, vec_scales, sc);   // before the wait: overlaps it
      if (!__all_sync(0xffffffffu, wait_stage(&my_bars[q % S], (uint32_t)(q / S) & 1u, ctx))) { ok = false; return; }
      chunk_compute<G, T, RG, NB, XS>(lm, my_ring + (uint32_t)(q % S) * kStage, sx, r0, nr, sc, unpack, acc, [&] {
        __syncwarp();
        issue_next();
      });
    }
#pragma unroll
    for (int tt = 0; tt < T; ++tt)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) store_tile(y, acc[tt][nb], row0 + tt * kTileRows, 8 * nb, lm.pg, lm.t, M, N);
  };
  for (int taken = 0; ok; ++taken) {
    // the producer side is at least one chunk ahead, so the queue entry exists (same warp: __syncwarp orders it)
    __syncwarp();
    const int u = my_queue[taken & 3];
    if (u >= n_units) break;
    const int row0 = unit_tile(u) * kTileRows;
    if (u < n_pairs) run_unit(std::integral_constant<int, 2>{}, row0);
    else run_unit(std::integral_constant<int, 1>{}, row0);
  }
  if (tr) tr[2] = globaltimer_ns();
  linger_after_abort(abort_word);
}

// ---------------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------------
template <auto kernel>
int opt_in_shared_memory() {   // once per kernel instantiation and device: more than 48 KB of dynamic smem
  static bool done[64] = {};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !done[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    done[dev] = true;
  }
  return KFB_OK;
}

#ifdef KFB_TRACE
inline unsigned long long* g_trace = nullptr;   // tuning aid, set through kfb_debug_set_gemv_trace
#else
constexpr unsigned long long* g_trace = nullptr;
#endif

template <class... KArgs, class... Args>
int launch_ex(void (*kernel)(KArgs...), int grid, int threads, size_t smem, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl || pdl_enabled()) ? 1 : 0;
  KFB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
  return KFB_OK;
}

constexpr int kMaxM = 32;   // 4 column blocks

// N from which the persistent kernel is used: every warp of its grid (16 per SM) gets at least two 16-row tiles.
inline bool uses_stream_kernel(int N) { return ceil_div(N, kTileRows) >= 2 * 16 * sm_count(); }

inline int column_blocks(int M) { return M <= 8 ? 1 : M <= 16 ? 2 : 4; }

template <int G>
inline bool fits(int M, int K) {
  const int nb = column_blocks(M);
  const size_t a = smem_bytes(1, kSplitStages, K / G, nb), b = StreamSmem<16, 2>::bytes(K / G, nb);
  return (a > b ? a : b) <= 227u * 1024u;
}

struct Call {
  const void* x; const void* scales; void* y;
  int M, N, K, vec;
  unsigned int* status;
  uint4 unpack;
  bool pdl;
  cudaStream_t stream;
};

template <int G, int KSL, int NB>
int launch_split(const Call& c, const CUtensorMap& wmap16, int grid) {
  if (int rc = opt_in_shared_memory<int4_gemv_mma_split_kernel<G, KSL, NB>>()) return rc;
  return launch_ex(int4_gemv_mma_split_kernel<G, KSL, NB>, grid, kThreads, smem_bytes(1, kSplitStages, c.K / G, NB), c.stream, c.pdl,
                   (const __half*)c.x, wmap16, (const __half*)c.scales, (__half*)c.y, c.M, c.N, c.K, c.vec, c.status, c.unpack);
}

template <int G, int RG, int NW, int NS, int NB, bool XS = false>
int launch_stream(const Call& c, const CUtensorMap& wmap32, const CUtensorMap& wmap16, int mp_log2 = 0) {
  if (int rc = opt_in_shared_memory<int4_gemv_mma_stream_kernel<G, RG, NW, 1, NS, NB, XS>>()) return rc;
  const size_t xs_bytes = XS ? ((size_t)c.K * 2) << mp_log2 : 0;
  return launch_ex(int4_gemv_mma_stream_kernel<G, RG, NW, 1, NS, NB, XS>, sm_count(), NW * 32,
                   StreamSmem<NW, NS>::bytes(c.K / G, NB, xs_bytes), c.stream, c.pdl, (const __half*)c.x, wmap32, wmap16,
                   (const __half*)c.scales, (__half*)c.y, c.M, c.N, c.K, c.vec, c.status, c.unpack, g_trace, mp_log2);
}

template <int G, int NB>
int launch_nb(const Call& c, const void* packed) {
  constexpr int C = kChunkBytes / (G / 2);
  const int N = c.N, K = c.K;
  const int rounds = K / G, n_chunks = ceil_div(rounds, C), tiles = ceil_div(N, kTileRows);
  // packed matrix as [N rows][K / 8 words]; box = 16 (or 32) rows x 32 words, 128-byte swizzle
  CUtensorMap wmap16;
  if (int rc = make_tmap_2d_plain(&wmap16, packed, /*elem_bytes=*/4, (uint64_t)K / 8, (uint64_t)N, (uint64_t)K / 2, kChunkBytes / 4,
                                  kTileRows, /*swizzle128=*/true))
    return rc;
  if (uses_stream_kernel(N)) {   // every warp of the persistent grid gets at least two tiles
    CUtensorMap wmap32;
    if (int rc = make_tmap_2d_plain(&wmap32, packed, 4, (uint64_t)K / 8, (uint64_t)N, (uint64_t)K / 2, kChunkBytes / 4,
                                    2 * kTileRows, true))
      return rc;
    // Two stages (8 KB in flight per warp, 128 KB per SM) measured faster than three: the memory system is saturated
    // either way and the shared memory not taken by the ring is L1 for the activations (N = 180224, K = 2048:
    // 41.7 vs 45.5 us at M = 1, 48.6 vs 54.4 us at M = 8).  Registers: 512 threads leave 128 per thread, enough
    // for two rounds at a time with one column block, one round with two; four column blocks run with 8 warps.
    if constexpr (NB == 1) {
      // M >= 2: activations from a fragment-ordered shared-memory copy when it fits next to the ring (64 KB).  Through
      // L1 the kernel slows down with M (N = 720896, K = 2048: 133 us at M = 1, 151 us at M = 8); with the copy M = 8
      // takes 135 us.
      const int mp_log2 = c.M <= 1 ? 0 : c.M <= 2 ? 1 : c.M <= 4 ? 2 : 3;
      if (c.M >= 2 && (((size_t)K * 2) << mp_log2) <= 64 * 1024)
        return launch_stream<G, 2, 16, 2, 1, true>(c, wmap32, wmap16, mp_log2);
      return launch_stream<G, 2, 16, 2, 1>(c, wmap32, wmap16);
    }
    else if constexpr (NB == 2) return launch_stream<G, 1, 16, 2, 2>(c, wmap32, wmap16);
    else return launch_stream<G, 1, 8, 3, 4>(c, wmap32, wmap16);
  }
  // split K over the warps of a CTA as far as the grid still fits in one wave (two CTAs per SM are resident) and every
  // warp keeps at least one chunk: a second, partly filled wave costs more than the extra parallelism brings
  // (5632 x 2048: 352 CTAs with K split 8 ways took 5.9 us, 176 CTAs with 4 ways fit one wave)
  int ksl = 0;
  while (ksl < 3 && ceil_div(tiles, kWarps >> (ksl + 1)) <= 2 * sm_count() && (2 << ksl) <= n_chunks) ++ksl;
  const int grid = ceil_div(tiles, kWarps >> ksl);
  switch (ksl) {
    case 0: return launch_split<G, 0, NB>(c, wmap16, grid);
    case 1: return launch_split<G, 1, NB>(c, wmap16, grid);
    case 2: return launch_split<G, 2, NB>(c, wmap16, grid);
    default: return launch_split<G, 3, NB>(c, wmap16, grid);
  }
}

template <int G>
int launch(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K, bool pdl, cudaStream_t stream) {
  constexpr int C = kChunkBytes / (G / 2);
  Call c;
  c.x = x; c.scales = scales; c.y = y; c.M = M; c.N = N; c.K = K;
  c.vec = ((K / G) % C == 0) && aligned16(scales);
  c.unpack = make_uint4(0x000F000Fu, 0x00F000F0u, 0x74007400u, 0x64006400u);
  c.status = device_status_word();
  c.pdl = pdl;
  c.stream = stream;
  if (!c.status) return KFB_ERR_CUDA;
  switch (column_blocks(M)) {
    case 1: return launch_nb<G, 1>(c, packed);
    case 2: return launch_nb<G, 2>(c, packed);
    default: return launch_nb<G, 4>(c, packed);
  }
}

}  // namespace gemv_mma
}  // namespace kfb
