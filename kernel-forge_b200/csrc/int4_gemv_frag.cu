// INT4 GEMV for M <= 32 on a PRIVATE, PREPACKED copy of the weights in MMA-fragment order.
//
// The reference names this as its next step for the INT4 path: reorder the packed weights offline so that every thread
// loads exactly the nibbles of its own MMA fragment and no shared-memory tile is needed (docs/phase4-notes.md:59,
// README.md:104).  The public format (kernelforge/quantize.py:18-23: int32 words of 8 nibbles along K, fp16 scale per
// group) stays what callers hold; kfb_int4_prepack builds the private copy once per weight (same size), and the caller
// keeps it next to the public tensor.
//
// Layout.  Rows are taken in blocks of 16 (the M of mma.m16n8k16), K in blocks of 64.  Block (rb, kb) is 512 contiguous
// bytes, 16 per lane: lane 4 g + t holds the two packed words of row 16 rb + g and the two of row 16 rb + g + 8 that
// cover k in [64 kb + 16 t, 64 kb + 16 t + 16).  Blocks of a row block are contiguous along kb, so a warp that walks K
// issues one perfectly coalesced 512-byte load per step and nothing else: no TMA, no mbarrier, no shared-memory tile,
// no bank conflicts.
//
// The k permutation that makes this work: within a 64-wide block, MMA step s (of 4) multiplies fragment columns
// (2t, 2t + 1, 2t + 8, 2t + 9) of lane t -- which are nibble pair s of that lane's first and second word, i.e. the real
// indices 16 t + 2 s, + 1 and 16 t + 8 + 2 s, + 1 -- with the activations of the same real indices, which the lane
// takes from ITS OWN contiguous 32-byte piece of the activation row.  A dot product does not care in which order k is
// visited, as long as A and B agree.
//
// Arithmetic: nibble pairs become exact fp16 integers ((w >> 4s) & 0x000F000F) | 0x64006400 = 1024 + u, minus 1032 in
// fp16 (exact) = q; mma.sync m16n8k16 with FP32 accumulation, one accumulator per scale group, scaled in FP32 (one
// fp16 scale per row and group), K split over the warps of a CTA with a fixed-order shared-memory reduction, one
// rounding to fp16.  The batch is the N = 8 of the MMA (rows past M are zero), so 1 <= M <= 8 cost the same; 9 <= M <= 32
// run 2 or 4 MMAs per unpacked fragment.
#include "common.cuh"
#include "int4_epilogue.cuh"

namespace kfb {
namespace frag {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxBlocksPerWarp = 24;   // k blocks (of 64) one warp can keep in flight: 24 x 16 B per lane

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// nibble pair s of a packed word -> half2 (q[2s], q[2s + 1]), exact
__device__ __forceinline__ uint32_t pair_q(uint32_t w, int s) {
  uint32_t v = ((w >> (4 * s)) & 0x000F000Fu) | 0x64006400u;   // half2(1024 + u, 1024 + u')
  asm("sub.f16x2 %0, %0, %1;" : "+r"(v) : "r"(0x64086408u));    // - 1032: exact
  return v;
}

// public packed words [N, K/8] -> fragment order (see the header comment).  One thread per 16-byte lane piece.
__global__ void prepack_kernel(const uint32_t* __restrict__ packed, uint4* __restrict__ out, int N, int K) {
  const int KB = K / 64, KW = K / 8;
  const long long total = (long long)(N / 16) * KB * 32;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int lane = (int)(i & 31);
    const long long blk = i >> 5;
    const int kb = (int)(blk % KB);
    const long long rb = blk / KB;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t* r0 = packed + (rb * 16 + g) * KW + kb * 8 + 2 * t;
    const uint32_t* r1 = r0 + (size_t)8 * KW;
    out[i] = make_uint4(r0[0], r0[1], r1[0], r1[1]);
  }
}

// One CTA = kWarps warps = RB row blocks x KS splits of K (RB * KS = kWarps).  G: group size.  NB: the k blocks a warp
// holds in registers (its whole share of K: every weight byte of the call is requested before the first is used).
// EPI: what becomes of each pair of adjacent result rows (int4_epilogue.cuh); kEpiNone stores them (+ bias, + residual).
// MB: blocks of 8 batch rows (the N of the MMA): every unpacked A fragment feeds MB MMAs.
template <int KS, int G, int NB, int EPI, int MB>
__global__ void __launch_bounds__(kThreads)
int4_gemv_frag_kernel(const __half* __restrict__ x, const uint4* __restrict__ wf, const __half* __restrict__ scales,
                      __half* __restrict__ y, int M, int N, int K, const gemv::Fusion fu) {
  constexpr int RB = kWarps / KS;
  constexpr int kBlocksPerGroup = G / 64;
  __shared__ float red[kWarps][16][8 * MB];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rb = blockIdx.x * RB + warp / KS;          // row block of this warp
  const int ks = warp % KS;                            // its share of K
  const int KB = K / 64, SG = K / G;
  const int n_rb = N / 16;
  // K is dealt out in scale groups: groups [g0, g1) of this warp
  const int g0 = (int)((long long)SG * ks / KS), g1 = (int)((long long)SG * (ks + 1) / KS);
  const int kb0 = g0 * kBlocksPerGroup, kb1 = g1 * kBlocksPerGroup;
  const bool live = rb < n_rb;

  // Weights are constants: every block of this warp is requested before the wait for the kernel in front (programmatic
  // dependent launch), so the whole weight stream of the call is in flight while that kernel drains.
  uint4 wbuf[NB];
  const uint4* wp = wf + ((size_t)(live ? rb : 0) * KB) * 32 + lane;
#pragma unroll
  for (int i = 0; i < NB; ++i)
    if (live && kb0 + i < kb1) wbuf[i] = ldg_stream(wp + (size_t)(kb0 + i) * 32);
  // ... and so are the scales: the (at most NB) group scales of rows g and g + 8 of this warp's share of K
  constexpr int kMaxGroups = (NB + kBlocksPerGroup - 1) / kBlocksPerGroup;
  __half sc0[kMaxGroups], sc1[kMaxGroups];
  {
    const __half* srow0 = scales + (size_t)((live ? rb : 0) * 16 + g) * SG;
    const __half* srow1 = srow0 + (size_t)8 * SG;
#pragma unroll
    for (int i = 0; i < kMaxGroups; ++i)
      if (live && g0 + i < g1) { sc0[i] = srow0[g0 + i]; sc1[i] = srow1[g0 + i]; }
  }
  pdl_wait();
  pdl_launch_dependents();

  float acc[MB][4];
#pragma unroll
  for (int j = 0; j < MB; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  if (live) {
    const __half* xrow = x + (size_t)g * K + 16 * t;   // batch row 8 j + g of B fragment j (valid when 8 j + g < M)
    float c[MB][4];
#pragma unroll
    for (int j = 0; j < MB; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      const int kb = kb0 + i;
      if (kb < kb1) {
        uint32_t xs0[MB][4], xs1[MB][4];
#pragma unroll
        for (int j = 0; j < MB; ++j) {
          uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
          if (8 * j + g < M) {
            const __half* xp = xrow + (size_t)(8 * j) * K + (size_t)kb * 64;
            xa = *reinterpret_cast<const uint4*>(xp);        // k = 64 kb + 16 t + [0, 8)
            xb = *reinterpret_cast<const uint4*>(xp + 8);    // k = 64 kb + 16 t + [8, 16)
          }
          xs0[j][0] = xa.x; xs0[j][1] = xa.y; xs0[j][2] = xa.z; xs0[j][3] = xa.w;
          xs1[j][0] = xb.x; xs1[j][1] = xb.y; xs1[j][2] = xb.z; xs1[j][3] = xb.w;
        }
        const uint4 w = wbuf[i];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const uint32_t a0 = pair_q(w.x, s), a1 = pair_q(w.z, s), a2 = pair_q(w.y, s), a3 = pair_q(w.w, s);
#pragma unroll
          for (int j = 0; j < MB; ++j) mma16816(c[j], a0, a1, a2, a3, xs0[j][s], xs1[j][s]);
        }
        if ((kb + 1) % kBlocksPerGroup == 0) {   // end of a scale group
          const int gi = (i + 1) / kBlocksPerGroup - 1;   // group index inside this warp's share (static after unrolling)
          const float s0 = __half2float(sc0[gi]), s1 = __half2float(sc1[gi]);
#pragma unroll
          for (int j = 0; j < MB; ++j) {
            acc[j][0] = fmaf(s0, c[j][0], acc[j][0]); acc[j][1] = fmaf(s0, c[j][1], acc[j][1]);
            acc[j][2] = fmaf(s1, c[j][2], acc[j][2]); acc[j][3] = fmaf(s1, c[j][3], acc[j][3]);
            c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
          }
        }
      }
    }
  }
  // (rows g, g + 8) x (batch 8 j + 2t, + 1) of this warp's share of K
#pragma unroll
  for (int j = 0; j < MB; ++j) {
    red[warp][g][8 * j + 2 * t] = acc[j][0]; red[warp][g][8 * j + 2 * t + 1] = acc[j][1];
    red[warp][g + 8][8 * j + 2 * t] = acc[j][2]; red[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  // fixed-order sum over the K splits; thread -> (row block of the CTA, pair of rows, batch column)
  for (int idx = threadIdx.x; idx < RB * 8 * 8 * MB; idx += kThreads) {
    const int n = idx % (8 * MB), pr = (idx / (8 * MB)) & 7, b = idx / (64 * MB);
    const int row_block = blockIdx.x * RB + b;
    if (row_block < n_rb && n < M) {
      float v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        v0 += red[b * KS + k][2 * pr][n];
        v1 += red[b * KS + k][2 * pr + 1][n];
      }
      gemv::store_pair<EPI>(v0, v1, fu, y, n, row_block * 16 + 2 * pr, N);
    }
  }
}

template <int KS, int G, int NB, int EPI, int MB>
int launch_mb(const void* x, const void* wf, const void* scales, void* y, int M, int N, int K, cudaStream_t stream, const gemv::Fusion& fu) {
  constexpr int RB = kWarps / KS;
  const int grid = ceil_div(N / 16, RB);
  return launch_kernel("int4_gemv_frag_kernel", int4_gemv_frag_kernel<KS, G, NB, EPI, MB>, dim3(grid), dim3(kThreads), 0, stream,
                       pdl_enabled(), static_cast<const __half*>(x), static_cast<const uint4*>(wf),
                       static_cast<const __half*>(scales), static_cast<__half*>(y), M, N, K, fu);
}

template <int KS, int G, int NB, int EPI>
int launch(const void* x, const void* wf, const void* scales, void* y, int M, int N, int K, cudaStream_t stream, const gemv::Fusion& fu) {
  if (M <= 8) return launch_mb<KS, G, NB, EPI, 1>(x, wf, scales, y, M, N, K, stream, fu);
  if constexpr (EPI == gemv::kEpiNone || (KS == 8 && NB <= 12)) {   // (pair epilogues above M = 8: the shapes a decode step has)
    if (M <= 16) return launch_mb<KS, G, NB, EPI, 2>(x, wf, scales, y, M, N, K, stream, fu);
    return launch_mb<KS, G, NB, EPI, 4>(x, wf, scales, y, M, N, K, stream, fu);
  }
  return fail(KFB_ERR_UNSUPPORTED, "this shape is supported for M <= 8 only");
}

template <int G, int EPI>
int pick(const void* x, const void* wf, const void* scales, void* y, int M, int N, int K, cudaStream_t s, const gemv::Fusion& fu) {
  // K is split over as many warps as there are scale groups to hand out (at most the 8 warps of a CTA); a warp's share
  // is ceil(groups / splits) groups, all of it held in registers
  const int sg = K / G;
  const int ks = sg >= 8 ? 8 : sg >= 4 ? 4 : sg >= 2 ? 2 : 1;
  const int need = ceil_div(sg, ks) * (G / 64);
  if (need > kMaxBlocksPerWarp)
    return fail(KFB_ERR_UNSUPPORTED, "K = %d is too long for this kernel (at most %d)", K, 8 * 64 * kMaxBlocksPerWarp);
  if (ks == 8) {
    if (need <= 4) return launch<8, G, 4, EPI>(x, wf, scales, y, M, N, K, s, fu);
    if (need <= 8) return launch<8, G, 8, EPI>(x, wf, scales, y, M, N, K, s, fu);
    if (need <= 12) return launch<8, G, 12, EPI>(x, wf, scales, y, M, N, K, s, fu);
    return launch<8, G, 24, EPI>(x, wf, scales, y, M, N, K, s, fu);
  }
  if (ks == 4) return launch<4, G, 4, EPI>(x, wf, scales, y, M, N, K, s, fu);
  if (ks == 2) return launch<2, G, 4, EPI>(x, wf, scales, y, M, N, K, s, fu);
  return launch<1, G, 4, EPI>(x, wf, scales, y, M, N, K, s, fu);
}

int run(const char* what, const void* x, const void* prepacked, const void* scales, void* y, int M, int N, int K, int group,
        void* stream, const gemv::Fusion& fu) {
  if (int rc = require_sm100()) return rc;
  if (M < 1 || M > 32) return fail(KFB_ERR_INVALID, "%s handles M in [1, 32], got M=%d", what, M);
  if (group != 64 && group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", group);
  if (N < 16 || N % 16 || K < group || K % group || K % 64)
    return fail(KFB_ERR_UNSUPPORTED, "the fragment-order copy needs N %% 16 == 0 and K %% 64 == 0, got N=%d K=%d", N, K);
  if (!x || !prepacked || !scales || !y) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(x) || !aligned16(prepacked)) return fail(KFB_ERR_ALIGNMENT, "x and the prepacked weights must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  if (fu.epi == gemv::kEpiSiluPair)
    return group == 128 ? pick<128, gemv::kEpiSiluPair>(x, prepacked, scales, y, M, N, K, s, fu)
                        : pick<64, gemv::kEpiSiluPair>(x, prepacked, scales, y, M, N, K, s, fu);
  if (fu.epi == gemv::kEpiRopeKv)
    return group == 128 ? pick<128, gemv::kEpiRopeKv>(x, prepacked, scales, y, M, N, K, s, fu)
                        : pick<64, gemv::kEpiRopeKv>(x, prepacked, scales, y, M, N, K, s, fu);
  return group == 128 ? pick<128, gemv::kEpiNone>(x, prepacked, scales, y, M, N, K, s, fu)
                      : pick<64, gemv::kEpiNone>(x, prepacked, scales, y, M, N, K, s, fu);
}

}  // namespace frag
}  // namespace kfb

using namespace kfb;

extern "C" size_t kfb_int4_prepack_bytes(int N, int K) {
  if (N < 16 || K < 64 || N % 16 || K % 64) return 0;
  return (size_t)N * K / 2;
}

extern "C" int kfb_int4_prepack(const void* packed, int N, int K, void* out, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (N < 16 || K < 64 || N % 16 || K % 64)
    return fail(KFB_ERR_UNSUPPORTED, "the fragment-order copy needs N %% 16 == 0 and K %% 64 == 0, got N=%d K=%d", N, K);
  if (!packed || !out) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(packed) || !aligned16(out)) return fail(KFB_ERR_ALIGNMENT, "packed and out must be 16-byte aligned");
  const long long total = (long long)(N / 16) * (K / 64) * 32;
  const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  frag::prepack_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint32_t*>(packed), static_cast<uint4*>(out), N, K);
  KFB_LAUNCH_CHECK("prepack_kernel");
  return KFB_OK;
}

extern "C" int kfb_int4_gemv_prepacked(const void* x, const void* prepacked, const void* scales, void* y, int M, int N, int K,
                                       int group, const void* bias, const void* residual, void* stream) {
  gemv::Fusion fu = {};
  fu.bias = static_cast<const __half*>(bias);
  fu.residual = static_cast<const __half*>(residual);
  return frag::run("int4_gemv_prepacked", x, prepacked, scales, y, M, N, K, group, stream, fu);
}

extern "C" int kfb_int4_gemv_prepacked_silu_pair(const void* x, const void* prepacked, const void* scales, void* act_out, int M,
                                                 int N, int K, int group, void* stream) {
  gemv::Fusion fu = {};
  fu.epi = gemv::kEpiSiluPair;
  return frag::run("int4_gemv_prepacked_silu_pair", x, prepacked, scales, act_out, M, N, K, group, stream, fu);
}

extern "C" int kfb_int4_gemv_prepacked_rope_kv(const void* x, const void* prepacked, const void* scales, int M, int K, int group,
                                               const void* cos_table, const void* sin_table, const void* pos_dev, void* q_out,
                                               void* k_cache, void* v_cache, int H, int Hk, int D, int Lmax, void* stream) {
  if (H < 1 || Hk < 1 || Lmax < 1 || (D != 64 && D != 128))
    return fail(KFB_ERR_INVALID, "int4_gemv_prepacked_rope_kv: bad shape H=%d Hk=%d D=%d Lmax=%d", H, Hk, D, Lmax);
  if (!cos_table || !sin_table || !pos_dev || !q_out || !k_cache || !v_cache) return fail(KFB_ERR_INVALID, "null pointer");
  gemv::Fusion fu = {};
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
  return frag::run("int4_gemv_prepacked_rope_kv", x, prepacked, scales, q_out, M, (H + 2 * Hk) * D, K, group, stream, fu);
}
