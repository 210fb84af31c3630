// The two ends of a decode step that the reference leaves to torch / cuBLAS: the token-embedding gather in front
// of the first RMSNorm, and the fp16 lm_head with the greedy argmax behind it.
//
// The lm_head is the largest single read of a decode step (vocab x hidden fp16: 131 MB for the TinyLlama shape,
// 20 % of the bytes of a step; the reference's notes name it as the next thing to fuse, docs/phase5-notes.md:39, and
// run it as `h @ lm_head.T` on cuBLAS followed by a separate argmax kernel, bench/e2e_model.py:97-141).  Here:
//   * lm_head_gemv_kernel: y[M, V] = x[M, K] W[V, K]^T for 1 <= M <= 32, W streamed once with 128-bit loads straight
//     into mma.sync.m16n8k16 A fragments (16 vocabulary rows per warp; a lane's 16 bytes of a row are 8 consecutive k,
//     and the same 8 k of x are its B fragment -- any consistent assignment of k to fragment slots gives the same dot
//     product, so no shared-memory staging or transposition is needed); FP32 accumulation, one rounding to fp16;
//     the greedy argmax is fused: every warp reduces its 16 rows per batch column and merges into a 64-bit key per
//     batch row with atomicMax (value in the high word, inverted row index in the low word: the maximum is unique, so
//     the result does not depend on the order of the atomics; ties go to the lowest index like torch.argmax);
//   * decode_finalize_kernel: turns the keys into next-token ids (int64, what the embedding reads), clears the keys
//     and advances the device-side position and KV length -- one launch instead of argmax + copy + two adds;
//   * embed_rmsnorm_kernel: gathers the embedding row of each token and applies the first RMSNorm in the same pass.
#include "common.cuh"

namespace kfb {
namespace lmhead {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRowsPerWarp = 16;
constexpr int kUnroll = 8;   // k chunks of 32 in flight per lane: 2 rows x 16 B x 8 = 256 B per lane, 8 KB per warp (4 gave 51 % of the HBM rate: too few bytes in flight at 13 warps per SM)

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cached(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Order-preserving map of a float to an unsigned integer (larger float <=> larger integer).
__device__ __forceinline__ uint32_t ordered_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// NB: blocks of 8 batch columns.  Lane = 4 g + t: vocabulary rows row0 + g and row0 + g + 8, k chunk t of every 32.
template <int NB>
__global__ void __launch_bounds__(kThreads)
lm_head_gemv_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ y,
                    unsigned long long* __restrict__ best, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = (blockIdx.x * kWarps + warp) * kRowsPerWarp;
  if (row0 >= N) {
    pdl_wait();
    pdl_launch_dependents();
    return;
  }
  const int ra = min(row0 + g, N - 1), rb = min(row0 + g + 8, N - 1);   // rows past N: a valid row, never stored
  const uint4* wa = reinterpret_cast<const uint4*>(w + (size_t)ra * K) + t;
  const uint4* wb = reinterpret_cast<const uint4*>(w + (size_t)rb * K) + t;
  const uint4* xr[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) xr[nb] = reinterpret_cast<const uint4*>(x + (size_t)min(8 * nb + g, M - 1) * K) + t;

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nb][e] = 0.f;

  const int chunks = K / 32;   // a chunk = 32 k: four lanes x 16 bytes
  for (int c0 = 0; c0 < chunks; c0 += kUnroll) {
    uint4 va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int c = min(c0 + u, chunks - 1);
      va[u] = ldg_stream(wa + c * 4);
      vb[u] = ldg_stream(wb + c * 4);
    }
    if (c0 == 0) {   // the weights are constants: the first loads are in flight before the wait for the kernel in front
      pdl_wait();
      pdl_launch_dependents();
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (c0 + u < chunks) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const uint4 xv = ldg_cached(xr[nb] + (c0 + u) * 4);
          // fragment slots (2t, 2t+1 | 2t+8, 2t+9) <- this lane's k (0,1 | 2,3), then (4,5 | 6,7)
          mma16816(acc[nb], va[u].x, vb[u].x, va[u].y, vb[u].y, xv.x, xv.y);
          mma16816(acc[nb], va[u].z, vb[u].z, va[u].w, vb[u].w, xv.z, xv.w);
        }
      }
    }
  }

  // acc[nb] = {row g col 2t, row g col 2t+1, row g+8 col 2t, row g+8 col 2t+1}, col = batch row 8 nb + ...
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = 8 * nb + 2 * t + e;
      const __half ha = __float2half_rn(acc[nb][e]), hb = __float2half_rn(acc[nb][2 + e]);
      unsigned long long key = 0ull;
      if (m < M) {
        if (row0 + g < N) {
          y[(size_t)m * N + row0 + g] = ha;
          key = ((unsigned long long)ordered_bits(__half2float(ha)) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)(row0 + g));
        }
        if (row0 + g + 8 < N) {
          y[(size_t)m * N + row0 + g + 8] = hb;
          const unsigned long long kb = ((unsigned long long)ordered_bits(__half2float(hb)) << 32) |
                                        (unsigned long long)(0xFFFFFFFFu - (uint32_t)(row0 + g + 8));
          key = kb > key ? kb : key;
        }
      }
      if (best != nullptr) {
        // maximum over the eight lanes g = 0..7 that hold the same batch column (lane bits 2..4)
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, off);
          key = other > key ? other : key;
        }
        if (g == 0 && m < M) atomicMax(best + m, key);
      }
    }
  }
}

__global__ void decode_finalize_kernel(unsigned long long* __restrict__ best, long long* __restrict__ tok, long long* __restrict__ pos,
                                       int* __restrict__ kv_len, int M) {
  const int m = threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  if (m < M) {
    const unsigned long long key = best[m];
    tok[m] = (long long)(0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull));
    best[m] = 0ull;
    kv_len[m] += 1;
  }
  if (m == 0) pos[0] += 1;
}

// One CTA (256 threads) per token: x_out[row] = embed[tok[row]], y[row] = fp16(fp16(x * rsqrt(mean(x^2) + eps)) * w).
constexpr int kMaxVec = 4;  // hidden <= 256 * 8 * 4
__global__ void __launch_bounds__(kThreads)
embed_rmsnorm_kernel(const long long* __restrict__ tok, const __half* __restrict__ embed, const __half* __restrict__ w,
                     __half* __restrict__ y, __half* __restrict__ x_out, int hidden, int vocab, float eps) {
  __shared__ float warp_part[kWarps];
  pdl_wait();
  pdl_launch_dependents();
  long long id = tok[blockIdx.x];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // an id outside the table reads a valid row instead of faulting
  const size_t src = (size_t)id * hidden, dst = (size_t)blockIdx.x * hidden;
  const int nvec = hidden / 8;
  uint4 vals[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) {
      vals[i] = reinterpret_cast<const uint4*>(embed + src)[v];
      reinterpret_cast<uint4*>(x_out + dst)[v] = vals[i];
      const __half2* h = reinterpret_cast<const __half2*>(&vals[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kWarps; ++i) tot += warp_part[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[v];
      const __half2* wh = reinterpret_cast<const __half2*>(&wv);
      const __half2* h = reinterpret_cast<const __half2*>(&vals[i]);
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        oh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
      }
      reinterpret_cast<uint4*>(y + dst)[v] = o;
    }
  }
}

}  // namespace
}  // namespace lmhead
}  // namespace kfb

using namespace kfb;

extern "C" int kfb_fp16_gemv_argmax(const void* x, const void* w, void* y, void* best, int M, int N, int K, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (M < 1 || M > 32) return fail(KFB_ERR_INVALID, "fp16_gemv_argmax handles M in [1, 32], got M=%d", M);
  if (N < 1 || K < 32 || K % 32) return fail(KFB_ERR_INVALID, "fp16_gemv_argmax needs N >= 1 and K a multiple of 32, got N=%d K=%d", N, K);
  if (!x || !w || !y) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(x) || !aligned16(w) || (best && (reinterpret_cast<uintptr_t>(best) & 7u)))
    return fail(KFB_ERR_ALIGNMENT, "x and w must be 16-byte aligned, the argmax keys 8-byte aligned");
  const int grid = ceil_div(N, lmhead::kWarps * lmhead::kRowsPerWarp);
  auto s = (cudaStream_t)stream;
  auto* b = static_cast<unsigned long long*>(best);
  const auto* xp = static_cast<const __half*>(x);
  const auto* wp = static_cast<const __half*>(w);
  auto* yp = static_cast<__half*>(y);
  const dim3 gd(grid), bd(lmhead::kThreads);
  const bool pdl = pdl_enabled();
  switch (ceil_div(M, 8)) {
    case 1: return launch_kernel("lm_head_gemv_kernel", lmhead::lm_head_gemv_kernel<1>, gd, bd, 0, s, pdl, xp, wp, yp, b, M, N, K);
    case 2: return launch_kernel("lm_head_gemv_kernel", lmhead::lm_head_gemv_kernel<2>, gd, bd, 0, s, pdl, xp, wp, yp, b, M, N, K);
    case 3: return launch_kernel("lm_head_gemv_kernel", lmhead::lm_head_gemv_kernel<3>, gd, bd, 0, s, pdl, xp, wp, yp, b, M, N, K);
    default: return launch_kernel("lm_head_gemv_kernel", lmhead::lm_head_gemv_kernel<4>, gd, bd, 0, s, pdl, xp, wp, yp, b, M, N, K);
  }
}

extern "C" int kfb_decode_finalize(void* best, void* tok, void* pos, void* kv_len, int M, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (M < 1 || M > 1024) return fail(KFB_ERR_INVALID, "decode_finalize handles 1..1024 sequences, got %d", M);
  if (!best || !tok || !pos || !kv_len) return fail(KFB_ERR_INVALID, "null pointer");
  return launch_kernel("decode_finalize_kernel", lmhead::decode_finalize_kernel, dim3(1), dim3(((M + 31) / 32) * 32), 0,
                       (cudaStream_t)stream, pdl_enabled(), static_cast<unsigned long long*>(best), static_cast<long long*>(tok),
                       static_cast<long long*>(pos), static_cast<int*>(kv_len), M);
}

extern "C" int kfb_embed_rmsnorm(const void* tok, const void* embed, const void* weight, void* y, void* x_out, int rows,
                                 int hidden, int vocab, float eps, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (rows < 1 || vocab < 1 || hidden < 8 || hidden % 8 || hidden > lmhead::kThreads * 8 * lmhead::kMaxVec)
    return fail(KFB_ERR_INVALID, "embed_rmsnorm needs rows, vocab >= 1 and hidden a multiple of 8 up to %d, got %d x %d",
                lmhead::kThreads * 8 * lmhead::kMaxVec, rows, hidden);
  if (!tok || !embed || !weight || !y || !x_out) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(embed) || !aligned16(weight) || !aligned16(y) || !aligned16(x_out))
    return fail(KFB_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  return launch_kernel("embed_rmsnorm_kernel", lmhead::embed_rmsnorm_kernel, dim3(rows), dim3(lmhead::kThreads), 0,
                       (cudaStream_t)stream, pdl_enabled(), static_cast<const long long*>(tok), static_cast<const __half*>(embed),
                       static_cast<const __half*>(weight), static_cast<__half*>(y), static_cast<__half*>(x_out), hidden, vocab, eps);
}
