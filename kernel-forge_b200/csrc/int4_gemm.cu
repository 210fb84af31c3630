// INT4 weight-only GEMM for sm_100a:  y[M, N] = x[M, K] @ W_hat[N, K]^T, any M, any N.
//
// Replaces dequant_gemm_tc_kernel + splitk_reduce of the reference
// (csrc/gemm/dequant_gemm_tc_kernel.cuh:55-162: mma.sync, 64x64 tiles, cp.async, N % 64 == 0).
//
// The product is computed transposed, y^T = W_hat x^T, so the 128 weight rows of a tile fill the
// M = 128 dimension of tcgen05.mma and the batch is the MMA N (16..256): small batches are not
// padded up to a 128-row tile.  One CTA per (128 output features, batch tile, K split):
//   warp 4  (1 thread)  TMA: the packed int32 tile (128 rows x 8 words = 64 k) and the fp16 x tile
//                       (batch rows x 64 k, 128-byte swizzle) of each K block, mbarrier ring;
//   warps 0-3 (128 thr) dequantise: thread r unpacks row r (magic-number nibble unpack, exact q,
//                       one fp16 multiply by the group scale = the reference's fp16(q*s),
//                       dequant_gemm_tc_kernel.cuh:100-112) and stores it as a K-major row of the
//                       128-byte-swizzled A tile; fence.proxy.async; then, at the end, the epilogue:
//                       TMEM -> registers -> fp16 y (or FP32 split-K partials), coalesced along N;
//   warp 5  (1 thread)  tcgen05.mma.kind::f16 A[smem] x B[smem] -> FP32 accumulator in TMEM.
// Split-K partial sums are reduced in split order by a second kernel (deterministic).
// Rows past N and batch rows past M are zero-filled by TMA and never stored.
#include "common.cuh"
#include "sm100.cuh"

namespace kfb {
namespace gemm {
namespace {

using namespace sm100;

constexpr int kTileN = 128;   // output features per CTA (MMA M)
constexpr int kBlockK = 64;   // k per pipeline stage (one 128-byte swizzle row of fp16)
constexpr int kDequantWarps = 8;  // two threads per weight row: four packed words each
constexpr int kThreads = (kDequantWarps + 2) * 32;
constexpr int kProducerWarp = kDequantWarps;
constexpr int kMmaWarp = kDequantWarps + 1;

enum WaitCode : uint32_t { kWaitFree = 0x301, kWaitLoaded, kWaitAReady, kWaitAcc };

// Where the fp16 result goes.  Plain call: one buffer [M, N].  Output-feature-sharded call (fused
// all-gather): `count` buffers [M, ld], one per GPU of the group (peer-mapped device pointers, this
// GPU's own buffer included); this rank's N columns are stored at column `col0` of EVERY buffer with
// plain peer stores from the epilogue, so the gather overlaps the computation tile by tile and no
// separate collective kernel runs.  (Stores only: no load ever targets a peer's memory.)
constexpr int kMaxPeers = 8;
struct OutSpec {
  __half* y[kMaxPeers];
  int count;
  int ld;    // row stride of every buffer, in elements
  int col0;  // first column this rank writes
  int bf16;  // the buffers hold bf16 instead of fp16 (the 16-bit stores are the same)
};

template <int MT>
struct Layout {
  // TMA latency (~1400 clocks) + dequantisation + MMA of one K block must be covered by the other stages
  static constexpr int kStages = MT <= 64 ? 4 : (MT == 128 ? 5 : 4);
  static constexpr int kA = kTileN * kBlockK * 2;        // dequantised weights, 16 KB
  static constexpr int kP = kTileN * (kBlockK / 8) * 4;  // packed words, 4 KB
  static constexpr int kX = MT * kBlockK * 2;            // activations
  static constexpr int kStage = kA + kP + kX;            // multiples of 1024
  static constexpr int kBars = kStages * kStage;
  static constexpr int kMisc = kBars + 3 * kStages * 8 + 8;
  static constexpr int kBytes = kMisc + 16;
  static constexpr int kAlloc = kBytes + 1024;
  static constexpr uint32_t kTmemCols = MT < 32 ? 32 : MT;
};

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// 8 packed weights -> 4 half2 of fp16(q * s) in k order
__device__ __forceinline__ uint4 dequant8(uint32_t w, __half2 s2) {
  constexpr uint32_t kMagic = 0x64006400u;
  const __half2 k1032 = u32_as_h2(0x64086408u);
  const __half2 kSixteenth = u32_as_h2(0x2C002C00u);
  const __half2 kMinus72 = u32_as_h2(0xD480D480u);
  const uint32_t h = w >> 8;
  uint4 r;
  r.x = h2_as_u32(__hmul2(__hsub2(u32_as_h2((w & 0x000F000Fu) | kMagic), k1032), s2));
  r.y = h2_as_u32(__hmul2(__hfma2(u32_as_h2((w & 0x00F000F0u) | kMagic), kSixteenth, kMinus72), s2));
  r.z = h2_as_u32(__hmul2(__hsub2(u32_as_h2((h & 0x000F000Fu) | kMagic), k1032), s2));
  r.w = h2_as_u32(__hmul2(__hfma2(u32_as_h2((h & 0x00F000F0u) | kMagic), kSixteenth, kMinus72), s2));
  return r;
}

// The same for bf16 activations: q is exact in fp16, the product q * s is formed in FP32 and rounded once to bf16.
__device__ __forceinline__ uint32_t bf2_mul(uint32_t q2, float s) {
  const float2 f = __half22float2(u32_as_h2(q2));
  const __nv_bfloat162 v = __floats2bfloat162_rn(f.x * s, f.y * s);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint4 dequant8_bf16(uint32_t w, float s) {
  constexpr uint32_t kMagic = 0x64006400u;
  const __half2 k1032 = u32_as_h2(0x64086408u);
  const __half2 kSixteenth = u32_as_h2(0x2C002C00u);
  const __half2 kMinus72 = u32_as_h2(0xD480D480u);
  const uint32_t h = w >> 8;
  uint4 r;
  r.x = bf2_mul(h2_as_u32(__hsub2(u32_as_h2((w & 0x000F000Fu) | kMagic), k1032)), s);
  r.y = bf2_mul(h2_as_u32(__hfma2(u32_as_h2((w & 0x00F000F0u) | kMagic), kSixteenth, kMinus72)), s);
  r.z = bf2_mul(h2_as_u32(__hsub2(u32_as_h2((h & 0x000F000Fu) | kMagic), k1032)), s);
  r.w = bf2_mul(h2_as_u32(__hfma2(u32_as_h2((h & 0x00F000F0u) | kMagic), kSixteenth, kMinus72)), s);
  return r;
}

__device__ __forceinline__ uint16_t round16(float v, bool bf16) {
  if (bf16) {
    const __nv_bfloat16 b = __float2bfloat16_rn(v);
    return *reinterpret_cast<const uint16_t*>(&b);
  }
  const __half h = __float2half_rn(v);
  return *reinterpret_cast<const uint16_t*>(&h);
}

// out: fp16 (bf16) y [M, N] when splits == 1, else FP32 partial [splits][M][N]
template <int MT, bool kBf16>
__global__ void __launch_bounds__(kThreads)
int4_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                 const __half* __restrict__ scales, const OutSpec out, float* __restrict__ partial, int M, int N,
                 int K, int group, int kblocks_per_split, unsigned int* status, unsigned long long* trace) {
  using L = Layout<MT>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* loaded = reinterpret_cast<uint64_t*>(smem + L::kBars);  // TMA landed
  uint64_t* a_ready = loaded + S;                                   // dequantised tile written
  uint64_t* stage_free = a_ready + S;                               // MMAs of the stage retired
  uint64_t* acc_done = stage_free + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile uint32_t* abort_word = tmem_slot + 1;
  const AbortCtx ctx{abort_word, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * MT;
  const int split = blockIdx.z, splits = gridDim.z;
  const int total_kblocks = K / kBlockK;
  const int kb_begin = split * kblocks_per_split;
  const int kb_end = min(total_kblocks, kb_begin + kblocks_per_split);
  const int n_kb = kb_end - kb_begin;  // >= 1 by construction

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&loaded[s], 1);
      mbar_init(&a_ready[s], kDequantWarps);
      mbar_init(&stage_free[s], 1);
    }
    mbar_init(acc_done, 1);
    *abort_word = *reinterpret_cast<volatile unsigned int*>(status);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool dead_on_arrival = *abort_word != 0;
  // optional timeline of CTA (0,0,0) for tuning (builds with -DKFB_TRACE only): 8 clock stamps per K block
#ifdef KFB_TRACE
  const bool tracing = trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#else
  constexpr bool tracing = false;
#endif
  auto stamp = [&](int i, int k) {
    if (tracing && i < 64) trace[i * 8 + k] = clock64();
  };

  if (dead_on_arrival) {
    // fall through to the teardown
  } else if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_w);
      tma_prefetch_desc(&tm_x);
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % S;
        if (!mbar_wait(&stage_free[s], ((uint32_t)(i / S) & 1u) ^ 1u, ctx, kWaitFree)) break;
        stamp(i, 0);
        mbar_arrive_expect_tx(&loaded[s], L::kP + L::kX);
        uint8_t* st = smem + s * L::kStage;
        const int kb = kb_begin + i;
        tma_load_2d(st + L::kA, &tm_w, &loaded[s], kb * (kBlockK / 8), n0);
        tma_load_4d(st + L::kA + L::kP, &tm_x, &loaded[s], kb * kBlockK, m0, 0, 0);  // tm_x is a 4-D map
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(kTileN, MT, kBf16 ? 1 : 0, 0, 0);
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % S;
        const uint32_t ph = (uint32_t)(i / S) & 1u;
        if (!mbar_wait(&a_ready[s], ph, ctx, kWaitAReady)) break;  // implies loaded[s]: the dequant warps waited on it
        stamp(i, 4);
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * L::kStage);
        const uint32_t b_addr = a_addr + L::kA + L::kP;
#pragma unroll
        for (int kk = 0; kk < kBlockK / 16; ++kk)
          mma_ss(tmem_base, smem_desc_sw128(a_addr + kk * 32, 16, 1024), smem_desc_sw128(b_addr + kk * 32, 16, 1024),
                 idesc, (i > 0 || kk > 0) ? 1u : 0u);
        tc_commit(&stage_free[s]);
        stamp(i, 5);
      }
      tc_commit(acc_done);
    }
  } else {
    // ---------------------------------------------------------------- dequantise (two threads per weight row)
    const int r = threadIdx.x & 127;   // weight row inside the tile; a warp covers 32 consecutive rows
    const int half = threadIdx.x >> 7; // which four of the eight packed words of a K block
    const int row = n0 + r;
    const int groups = K / group;
    const __half* srow = scales + (size_t)min(row, N - 1) * groups;
    bool ok = true;
    // The group scale of a K block comes from global memory (L2 latency of several hundred clocks): it is
    // fetched two K blocks ahead so that the load never sits on the critical path of a pipeline stage.
    __half sc_ring[3];
    sc_ring[0] = srow[(kb_begin * kBlockK) / group];
    sc_ring[1] = srow[(min(kb_begin + 1, kb_end - 1) * kBlockK) / group];
    for (int i = 0; i < n_kb; ++i) {
      const int s = i % S;
      const uint32_t ph = (uint32_t)(i / S) & 1u;
      sc_ring[2] = srow[(min(kb_begin + i + 2, kb_end - 1) * kBlockK) / group];
      const __half sc = sc_ring[0];
      sc_ring[0] = sc_ring[1];
      sc_ring[1] = sc_ring[2];
      ok = __all_sync(0xffffffffu, mbar_wait(&loaded[s], ph, ctx, kWaitLoaded));
      if (!ok) break;
      if (threadIdx.x == 0) stamp(i, 1);
      uint8_t* st = smem + s * L::kStage;
      const uint4 w = *reinterpret_cast<const uint4*>(st + L::kA + r * 32 + half * 16);
      const __half2 s2 = __half2half2(sc);
      uint8_t* arow = st + r * 128;
      const int x = r & 7, c = half * 4;
      if constexpr (kBf16) {
        const float sf = __half2float(sc);
        *reinterpret_cast<uint4*>(arow + (((c + 0) ^ x) << 4)) = dequant8_bf16(w.x, sf);
        *reinterpret_cast<uint4*>(arow + (((c + 1) ^ x) << 4)) = dequant8_bf16(w.y, sf);
        *reinterpret_cast<uint4*>(arow + (((c + 2) ^ x) << 4)) = dequant8_bf16(w.z, sf);
        *reinterpret_cast<uint4*>(arow + (((c + 3) ^ x) << 4)) = dequant8_bf16(w.w, sf);
      } else {
        *reinterpret_cast<uint4*>(arow + (((c + 0) ^ x) << 4)) = dequant8(w.x, s2);
        *reinterpret_cast<uint4*>(arow + (((c + 1) ^ x) << 4)) = dequant8(w.y, s2);
        *reinterpret_cast<uint4*>(arow + (((c + 2) ^ x) << 4)) = dequant8(w.z, s2);
        *reinterpret_cast<uint4*>(arow + (((c + 3) ^ x) << 4)) = dequant8(w.w, s2);
      }
      fence_proxy_async_smem();  // generic-proxy stores -> visible to tcgen05.mma
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[s]);
      if (threadIdx.x == 0) stamp(i, 2);
    }
    // ---------------------------------------------------------------- epilogue
    // TMEM lane = weight row n, column = batch row m, but y is [M, N]: going straight to global memory
    // would be 2-byte stores with a stride of N (measured: 60 % of the kernel time).  Each warpgroup
    // (warps 0-3 / 4-7, which own alternate 32-column chunks) transposes its chunk through a shared
    // memory tile [32 m][128 n] and writes rows of 128 outputs with 16-byte stores.
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_done, 0, ctx, kWaitAcc));
    if (threadIdx.x == 0) stamp(63, 6);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t lane_bits = (uint32_t)((warp & 3) * 32) << 16;
      const int wg = warp >> 2;                    // 0 or 1
      uint8_t* tile = smem + wg * L::kStage;       // every stage is free once acc_done has completed
      const bool f32 = splits > 1;
      const int n_valid = min(kTileN, N - n0);     // columns of this tile that exist
      constexpr int kCols = MT >= 32 ? 32 : MT;
      constexpr int kChunks = MT >= 32 ? MT / 32 : 1;
#pragma unroll 1
      for (int ch = wg; ch < kChunks; ch += 2) {
        const int c0 = ch * 32;
        if (m0 + c0 >= M) break;  // uniform per warpgroup: batch rows that do not exist
        uint32_t acc[32];
        if constexpr (MT >= 32) {
          tmem_ld_x32(tmem_base + lane_bits + c0, acc);
        } else {
          tmem_ld_x16(tmem_base + lane_bits + c0, acc);
        }
        tmem_wait_ld();
        if (f32) {
#pragma unroll
          for (int c = 0; c < kCols; ++c) reinterpret_cast<float*>(tile)[c * kTileN + r] = __uint_as_float(acc[c]);
        } else {
#pragma unroll
          for (int c = 0; c < kCols; ++c)
            reinterpret_cast<uint16_t*>(tile)[c * kTileN + r] = round16(__uint_as_float(acc[c]), kBf16);
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");
        const int m_hi = min(kCols, M - (m0 + c0));  // batch rows of this chunk that exist
        if (f32) {
          float* dst = partial + ((size_t)split * M + m0 + c0) * N + n0;
          if ((N & 3) == 0) {
            for (int idx = r; idx < m_hi * 32; idx += 128) {
              const int ml = idx >> 5, seg = idx & 31;
              if (seg * 4 < n_valid)
                *reinterpret_cast<uint4*>(dst + (size_t)ml * N + seg * 4) = reinterpret_cast<const uint4*>(tile)[ml * 32 + seg];
            }
          } else {
            for (int ml = 0; ml < m_hi; ++ml)
              if (r < n_valid) dst[(size_t)ml * N + r] = reinterpret_cast<const float*>(tile)[ml * kTileN + r];
          }
        } else {
          const bool vec = ((out.ld | out.col0) & 7) == 0;  // every row segment starts on a 16-byte boundary
          for (int p = 0; p < out.count; ++p) {
            __half* dst = out.y[p] + (size_t)(m0 + c0) * out.ld + out.col0 + n0;
            if (vec) {
              for (int idx = r; idx < m_hi * 16; idx += 128) {
                const int ml = idx >> 4, seg = idx & 15;
                if (seg * 8 + 8 <= n_valid) {
                  *reinterpret_cast<uint4*>(dst + (size_t)ml * out.ld + seg * 8) = reinterpret_cast<const uint4*>(tile)[ml * 16 + seg];
                } else {
                  for (int e = seg * 8; e < n_valid; ++e) dst[(size_t)ml * out.ld + e] = reinterpret_cast<const __half*>(tile)[ml * kTileN + e];
                }
              }
            } else {
              for (int ml = 0; ml < m_hi; ++ml)
                if (r < n_valid) dst[(size_t)ml * out.ld + r] = reinterpret_cast<const __half*>(tile)[ml * kTileN + r];
            }
          }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory");  // tile is reused by the next chunk
      }
    }
  }

  if (threadIdx.x == 0) stamp(63, 7);
  if (!dead_on_arrival && *abort_word != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

// y[m, col0 + n] = fp16(sum over splits, in split order, of partial[s][m][n]), in every output buffer
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, const OutSpec out,
                                                            int M, int N, int splits) {
  const long long elems = (long long)M * N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * elems + i];
    const long long m = i / N;
    const int n = (int)(i - m * N);
    const uint16_t v = round16(acc, out.bf16 != 0);
    for (int p = 0; p < out.count; ++p) reinterpret_cast<uint16_t*>(out.y[p])[m * out.ld + out.col0 + n] = v;
  }
}

#ifdef KFB_TRACE
unsigned long long* g_trace = nullptr;  // tuning aid, set through kfb_debug_set_gemm_trace
#else
constexpr unsigned long long* g_trace = nullptr;
#endif

struct Plan {
  int mt, m_tiles, n_tiles, splits, kblocks_per_split;
};

Plan make_plan(int M, int N, int K) {
  Plan p;
  p.mt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  p.m_tiles = ceil_div(M, p.mt);
  p.n_tiles = ceil_div(N, kTileN);
  const int kblocks = K / kBlockK;
  const int tiles = p.m_tiles * p.n_tiles;
  // Split K when that is cheaper than letting a grid smaller than the GPU walk all of K.  Cost model (us, fitted to
  // measurements on B200): a CTA spends ~0.45 per K block plus ~2 of fill and drain; a split plan pays the reduce
  // kernel, ~3 plus its traffic (splits FP32 partials read, fp16 written) at ~4 TB/s.  Measured examples: M = 128
  // 8960 x 1536 unsplit 17.3 against 22.7 with 2 splits; M = 1024 256 x 1536 6 splits 15.3 against 19.2 unsplit.
  const int sms = sm_count();
  const int max_splits = kblocks / 4 > 0 ? kblocks / 4 : 1;  // at least 4 K blocks per split
  int splits = 1;
  double best_cost = 1e30;
  for (int sp = 1; sp <= max_splits; ++sp) {
    const int per = ceil_div(kblocks, sp);
    const int real = ceil_div(kblocks, per);
    if (real != sp) continue;
    const int waves = ceil_div(tiles * real, sms);
    double cost = waves * (0.45 * per + 2.0);
    if (real > 1) cost += 3.0 + ((double)real * M * N * 4.0 + (double)M * N * 2.0) / 4.0e6;
    if (cost < best_cost * 0.999) { best_cost = cost; splits = real; }
  }
  p.kblocks_per_split = ceil_div(kblocks, splits);
  p.splits = ceil_div(kblocks, p.kblocks_per_split);  // no empty split
  return p;
}

template <int MT, bool kBf16>
int launch(const Plan& p, const CUtensorMap& tw, const CUtensorMap& tx, const void* scales, const OutSpec& out, float* partial,
           int M, int N, int K, int group, unsigned int* status, cudaStream_t stream) {
  using L = Layout<MT>;
  auto kernel = int4_gemm_kernel<MT, kBf16>;
  static bool configured[64] = {false};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    configured[dev] = true;
  }
  const dim3 grid(p.n_tiles, p.m_tiles, p.splits);
  kernel<<<grid, kThreads, L::kAlloc, stream>>>(tw, tx, (const __half*)scales, out, partial, M, N, K, group,
                                               p.kblocks_per_split, status, g_trace);
  KFB_LAUNCH_CHECK("int4_gemm_kernel");
  if (p.splits > 1) {
    const long long elems = (long long)M * N;
    long long blocks = (elems + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    splitk_reduce_kernel<<<(int)blocks, 256, 0, stream>>>(partial, out, M, N, p.splits);
    KFB_LAUNCH_CHECK("splitk_reduce_kernel");
  }
  return KFB_OK;
}

}  // namespace
}  // namespace gemm
}  // namespace kfb

using namespace kfb;

extern "C" size_t kfb_int4_gemm_ws_bytes(int M, int N, int K, int group) {
  if (M < 1 || N < 1 || K < 64 || (group != 64 && group != 128) || K % group) return 0;
  const gemm::Plan p = gemm::make_plan(M, N, K);
  return p.splits > 1 ? (size_t)p.splits * M * N * sizeof(float) : 0;
}

namespace {

int gemm_common(const void* x, const void* packed, const void* scales, const gemm::OutSpec& out, int M, int N, int K,
                int group, void* ws, size_t ws_bytes, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (M < 1) return fail(KFB_ERR_INVALID, "int4_gemm needs M >= 1, got M=%d", M);
  if (group != 64 && group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", group);
  if (N < 1 || K < group || K % group) return fail(KFB_ERR_INVALID, "K=%d is not a multiple of group_size=%d", K, group);
  if (!x || !packed || !scales) return fail(KFB_ERR_INVALID, "null pointer");
  for (int i = 0; i < out.count; ++i)
    if (!out.y[i] || !aligned16(out.y[i])) return fail(KFB_ERR_ALIGNMENT, "output buffers must be non-null and 16-byte aligned");
  if (!aligned16(x) || !aligned16(packed)) return fail(KFB_ERR_ALIGNMENT, "x and packed must be 16-byte aligned");
  const gemm::Plan p = gemm::make_plan(M, N, K);
  const size_t need = p.splits > 1 ? (size_t)p.splits * M * N * sizeof(float) : 0;
  if (need > 0 && (!ws || ws_bytes < need))
    return fail(KFB_ERR_WORKSPACE, "int4_gemm needs a %zu-byte workspace for %d K splits, got %zu", need, p.splits, ws_bytes);
  if (need > 0 && !aligned16(ws)) return fail(KFB_ERR_ALIGNMENT, "workspace must be 16-byte aligned");
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");

  CUtensorMap tw, tx;
  // packed int32 [N, K/8] seen as 32-bit elements, box 8 words x 128 rows, no swizzle
  if (int rc = make_tmap_2d_plain(&tw, packed, /*elem_bytes=*/4, (uint64_t)K / 8, (uint64_t)N, (uint64_t)K / 2, 8, 128)) return rc;
  // x fp16 [M, K], box 64 k x MT rows, 128-byte swizzle (reuse the 4-D helper with unit outer dims)
  const uint64_t xd[4] = {(uint64_t)K, (uint64_t)M, 1, 1};
  const uint64_t xs[3] = {(uint64_t)K * 2, (uint64_t)M * K * 2, (uint64_t)M * K * 2};
  const uint32_t xb[4] = {64, (uint32_t)p.mt, 1, 1};
  if (int rc = make_tmap_4d_sw128(&tx, x, out.bf16 ? KFB_BF16 : KFB_F16, xd, xs, xb)) return rc;

  cudaStream_t s = (cudaStream_t)stream;
  float* partial = static_cast<float*>(ws);
  if (out.bf16) {
    switch (p.mt) {
      case 16: return gemm::launch<16, true>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
      case 32: return gemm::launch<32, true>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
      case 64: return gemm::launch<64, true>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
      case 128: return gemm::launch<128, true>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
      default: return gemm::launch<256, true>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
    }
  }
  switch (p.mt) {
    case 16: return gemm::launch<16, false>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
    case 32: return gemm::launch<32, false>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
    case 64: return gemm::launch<64, false>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
    case 128: return gemm::launch<128, false>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
    default: return gemm::launch<256, false>(p, tw, tx, scales, out, partial, M, N, K, group, status, s);
  }
}

}  // namespace

extern "C" int kfb_int4_gemm(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K,
                             int group, void* ws, size_t ws_bytes, void* stream) {
  gemm::OutSpec out = {};
  out.y[0] = static_cast<__half*>(y);
  out.count = 1;
  out.ld = N;
  out.col0 = 0;
  if (!y) return fail(KFB_ERR_INVALID, "null pointer");
  return gemm_common(x, packed, scales, out, M, N, K, group, ws, ws_bytes, stream);
}

extern "C" int kfb_int4_gemm_bf16(const void* x, const void* packed, const void* scales, void* y, int M, int N, int K,
                                  int group, void* ws, size_t ws_bytes, void* stream) {
  gemm::OutSpec out = {};
  out.y[0] = static_cast<__half*>(y);
  out.count = 1;
  out.ld = N;
  out.col0 = 0;
  out.bf16 = 1;
  if (!y) return fail(KFB_ERR_INVALID, "null pointer");
  return gemm_common(x, packed, scales, out, M, N, K, group, ws, ws_bytes, stream);
}

extern "C" int kfb_int4_gemm_allgather(const void* x, const void* packed, const void* scales, void* const* y_all,
                                       int n_buffers, int M, int N_local, int K, int group, int ld, int col0, void* ws,
                                       size_t ws_bytes, void* stream) {
  if (n_buffers < 1 || n_buffers > gemm::kMaxPeers)
    return fail(KFB_ERR_INVALID, "n_buffers must be in [1, %d], got %d", gemm::kMaxPeers, n_buffers);
  if (!y_all) return fail(KFB_ERR_INVALID, "null pointer");
  if (col0 < 0 || ld < col0 + N_local)
    return fail(KFB_ERR_INVALID, "columns [%d, %d) do not fit in a row of %d", col0, col0 + N_local, ld);
  gemm::OutSpec out = {};
  for (int i = 0; i < n_buffers; ++i) out.y[i] = static_cast<__half*>(y_all[i]);
  out.count = n_buffers;
  out.ld = ld;
  out.col0 = col0;
  return gemm_common(x, packed, scales, out, M, N_local, K, group, ws, ws_bytes, stream);
}

#ifdef KFB_TRACE
// Tuning aid of -DKFB_TRACE builds (not part of the public header): device buffer of 64 x 8 clock stamps written by
// CTA (0,0,0).
extern "C" void kfb_debug_set_gemm_trace(void* device_buffer) {
  kfb::gemm::g_trace = static_cast<unsigned long long*>(device_buffer);
}
#endif
