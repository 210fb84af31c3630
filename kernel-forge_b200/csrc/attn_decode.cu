// Decode attention (q_len = 1) for sm_100a: split-KV, HBM-bound.
//
// The reference serves decode with its prefill kernel: one CTA per (batch, query head) walks all
// Nk keys serially with 127 of 128 tile rows padding, and K/V are re-read once per query head of a
// group (csrc/attention/attn_v4_kernel.cuh:43-214, grid (1, B*H)).  Here:
//   * grid = (splits, Hk * head-chunks, B): the key range of one (batch, kv head) is split across
//     CTAs so that even B = 1, Hk = 4 fills the 148 SMs;
//   * the G = H / Hk query heads of a KV head are the M rows of the MMA (chunks of 16), so every K/V
//     byte is read from HBM ONCE per group instead of once per query head;
//   * a producer warp streams 64-key K and V tiles with TMA (128-byte swizzle) through a 4-stage
//     mbarrier ring; four consumer warps each take 16 keys of a tile: S = Q K^T and O += P V on
//     mma.sync.m16n8k16 (FP32 accumulate) -- the kernel is bandwidth-bound (8 FLOP per K/V byte at
//     G = 8), tensor cores only keep the ALU cost below the HBM time;
//   * per-warp online softmax (base 2, FP32), warps merged in shared memory in fixed order, one
//     partial (O, m, l) per split written to the caller's workspace and combined in split order by
//     a second small kernel => deterministic.  With one split the result is written directly.
#include "attn.cuh"
#include "sm100.cuh"

namespace kfb {
namespace attn {
namespace {

using namespace sm100;

constexpr int kTileKeys = 64;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
// Depth of the K/V tile ring.  A grid that fills the SMs (large batches) runs 3 CTAs per SM with 4 stages each; a grid
// smaller than the GPU (decode at batch 1-8: B * Hk CTAs) is bound by the bytes ONE SM keeps in flight, so there the ring
// takes (nearly) the whole shared memory and every tile of a short cache is requested at once.
constexpr int kStagesShallow = 4;
template <int D> constexpr int deep_stages() { return D == 64 ? 12 : 6; }
constexpr int kRows = 16;  // query heads per CTA (MMA M)

enum WaitCode : uint32_t { kWaitFull = 0x201, kWaitEmpty };

template <int D, int kStages>
struct Layout {
  static constexpr int kHalf = kTileKeys * 128;       // 64 keys x 64 columns
  static constexpr int kTile = kTileKeys * D * 2;     // one K or V tile
  static constexpr int kStage = 2 * kTile;            // K then V
  static constexpr int kBars = kStages * kStage;
  static constexpr int kMisc = kBars + 2 * kStages * 8;
  static constexpr int kBytes = kMisc + 16;
  static constexpr int kAlloc = kBytes + 1024;
  // the cross-warp merge reuses the tile ring: per warp O[16][D] + m[16] + l[16] floats
  static constexpr int kMergeBytes = kConsumerWarps * kRows * (D + 2) * 4;
  static_assert(kMergeBytes <= kBars, "merge scratch must fit in the tile ring");
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <bool kBf16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
template <bool kBf16>
__device__ __forceinline__ uint16_t pack1(float x) {
  if constexpr (kBf16) {
    __nv_bfloat16 v = __float2bfloat16_rn(x);
    return *reinterpret_cast<uint16_t*>(&v);
  } else {
    __half v = __float2half_rn(x);
    return *reinterpret_cast<uint16_t*>(&v);
  }
}

// byte offset of (key row r, 16-byte chunk c of the 128-byte row) inside a 128B-swizzled 64-key half tile
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// Partial results, per (batch, kv head * chunks + chunk, split): O[16][D], m[16], l[16] floats.
template <int D>
__host__ __device__ constexpr int partial_floats() { return kRows * (D + 2); }

template <int D, bool kBf16, int kStages>
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const uint16_t* __restrict__ q, uint16_t* __restrict__ o, float* __restrict__ partial, int H, int Hk,
                   int Nk, int keys_per_split, float scale_log2, unsigned int* status, const int* __restrict__ kv_len,
                   int force_partial) {
  using L = Layout<D, kStages>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* empty = full + kStages;
  volatile uint32_t* abort_word = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  const AbortCtx ctx{abort_word, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = H / Hk;
  const int chunks = (G + kRows - 1) / kRows;
  const int split = blockIdx.x, splits = gridDim.x;
  const int hk = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int b = blockIdx.z;
  const int h0 = hk * G + chunk * kRows;               // first query head of this CTA
  const int rows = min(kRows, G - chunk * kRows);      // real query heads
  const int key_begin = split * keys_per_split;
  // a static KV cache holds Nk rows of which only kv_len[b] are valid (read on the device, so the
  // same launch can be replayed from a CUDA graph while the cache fills up)
  const int valid = kv_len ? min(Nk, max(kv_len[b], 0)) : Nk;
  const int key_end = min(valid, key_begin + keys_per_split);
  const int n_tiles = key_end > key_begin ? (key_end - key_begin + kTileKeys - 1) / kTileKeys : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    *abort_word = *reinterpret_cast<volatile unsigned int*>(status);  // non-zero: an earlier wait expired
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();               // q, the cache rows and kv_len may be the output of the kernel in front
  pdl_launch_dependents();
  if (*abort_word != 0) return;  // uniform: written before the barrier, nothing has been issued yet

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % kStages;
        if (!mbar_wait(&empty[s], ((uint32_t)(t / kStages) & 1u) ^ 1u, ctx, kWaitEmpty)) break;
        mbar_arrive_expect_tx(&full[s], L::kStage);
        uint8_t* dst = smem + s * L::kStage;
        const int key0 = key_begin + t * kTileKeys;
#pragma unroll
        for (int half = 0; half < D / 64; ++half) {
          tma_load_4d(dst + half * L::kHalf, &tm_k, &full[s], half * 64, key0, hk, b);
          tma_load_4d(dst + L::kTile + half * L::kHalf, &tm_v, &full[s], half * 64, key0, hk, b);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int g = lane >> 2, t4 = lane & 3;
    // Q fragments (A operand, 16 heads x D), rows >= `rows` are zero
    uint32_t qa[D / 16][4];
    {
      const uint16_t* q0 = q + ((size_t)b * H + h0 + g) * D;        // row g      (Nq == 1)
      const uint16_t* q1 = q + ((size_t)b * H + h0 + g + 8) * D;    // row g + 8
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int c = kk * 16 + 2 * t4;
        qa[kk][0] = g < rows ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
        qa[kk][1] = g + 8 < rows ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
        qa[kk][2] = g < rows ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
        qa[kk][3] = g + 8 < rows ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
      }
    }
    const int mat = lane >> 3, mrow = lane & 7;
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % kStages;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (uint32_t)(t / kStages) & 1u, ctx, kWaitFull));
      if (!ok) break;
      const uint32_t k_base = smem_u32(smem + s * L::kStage);
      const uint32_t v_base = k_base + L::kTile;
      const int kw = warp * 16;  // this warp's 16 keys inside the tile

      // S[16 heads x 16 keys]: two n-tiles of 8 keys
      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        // matrices: (keys 0-7, d 0-7) (keys 0-7, d 8-15) (keys 8-15, d 0-7) (keys 8-15, d 8-15)
        const int key = kw + (mat >> 1) * 8 + mrow;
        const int dchunk = kk * 2 + (mat & 1);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(k_base + (dchunk >> 3) * L::kHalf + swz(key, dchunk & 7), r0, r1, r2, r3);
        mma16816<kBf16>(sacc[0], qa[kk], r0, r1);
        mma16816<kBf16>(sacc[1], qa[kk], r2, r3);
      }
      // mask keys past this split's range (TMA zero-fills past Nk; keys of the next split are real data)
      const int key_abs = key_begin + t * kTileKeys + kw + 2 * t4;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (key_abs + nt * 8 + (e & 1) >= key_end) sacc[nt][e] = -INFINITY;

      // online softmax for rows g (e = 0,1) and g + 8 (e = 2,3)
      uint32_t pa[4];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = fmaxf(fmaxf(sacc[0][2 * r], sacc[0][2 * r + 1]), fmaxf(sacc[1][2 * r], sacc[1][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx * scale_log2);
        const float base = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = ex2(m_run[r] - base);
        const float p00 = ex2(fmaf(sacc[0][2 * r], scale_log2, -base));
        const float p01 = ex2(fmaf(sacc[0][2 * r + 1], scale_log2, -base));
        const float p10 = ex2(fmaf(sacc[1][2 * r], scale_log2, -base));
        const float p11 = ex2(fmaf(sacc[1][2 * r + 1], scale_log2, -base));
        l_run[r] = fmaf(l_run[r], alpha, (p00 + p01) + (p10 + p11));  // lane-local part of the row sum
        m_run[r] = m_new;
        pa[r] = pack2<kBf16>(p00, p01);       // a0a1 (row g) / a2a3 (row g+8): keys 2t, 2t+1
        pa[2 + r] = pack2<kBf16>(p10, p11);   // a4a5 / a6a7: keys 2t+8, 2t+9
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          oacc[i][2 * r] *= alpha;
          oacc[i][2 * r + 1] *= alpha;
        }
      }
      // Rows of V past key_end get p = 0, but 0 * NaN = NaN: with a device-side length those rows are
      // whatever the cache buffer holds, so this warp zeroes them in its 16-key slice of the tile first.
      {
        const int first_bad = key_end - (key_begin + t * kTileKeys);  // tile-relative; >= 64 when all rows are valid
        if (first_bad < kw + 16) {
          const int r0 = max(first_bad, kw);
          for (int i = lane; i < (kw + 16 - r0) * 8 * (D / 64); i += 32) {
            const int row = r0 + i / (8 * (D / 64)), rem = i % (8 * (D / 64));
            *reinterpret_cast<uint4*>(smem + s * L::kStage + L::kTile + (rem >> 3) * L::kHalf + row * 128 + (rem & 7) * 16) =
                make_uint4(0u, 0u, 0u, 0u);
          }
          __syncwarp();
        }
      }
      // O[16 x D] += P[16 x 16 keys] V[16 keys x D]
#pragma unroll
      for (int dn = 0; dn < D / 16; ++dn) {
        // matrices: (keys 0-7, d c0) (keys 8-15, d c0) (keys 0-7, d c1) (keys 8-15, d c1), transposed on load
        const int key = kw + (mat & 1) * 8 + mrow;
        const int dchunk = dn * 2 + (mat >> 1);
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(v_base + (dchunk >> 3) * L::kHalf + swz(key, dchunk & 7), r0, r1, r2, r3);
        mma16816<kBf16>(oacc[2 * dn], pa, r0, r1);
        mma16816<kBf16>(oacc[2 * dn + 1], pa, r2, r3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    // finish the row sums across the quad
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
  }

  // ------------------------------------------------------------------ merge the four warps
  __syncthreads();  // every tile has been consumed (or the CTA is aborting): the ring is free
  float* scratch = reinterpret_cast<float*>(smem);
  constexpr int kPerWarp = kRows * (D + 2);
  if (warp < kConsumerWarps) {
    float* mine = scratch + warp * kPerWarp;
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int d = i * 8 + 2 * t4;
      mine[g * D + d] = oacc[i][0];
      mine[g * D + d + 1] = oacc[i][1];
      mine[(g + 8) * D + d] = oacc[i][2];
      mine[(g + 8) * D + d + 1] = oacc[i][3];
    }
    if (t4 == 0) {
      mine[kRows * D + g] = m_run[0];
      mine[kRows * D + g + 8] = m_run[1];
      mine[kRows * D + kRows + g] = l_run[0];
      mine[kRows * D + kRows + g + 8] = l_run[1];
    }
  }
  __syncthreads();
  const bool direct = splits == 1 && !force_partial;   // otherwise (O, m, l) goes to `partial` for a later merge
  float* out_partial = partial + (((size_t)b * gridDim.y + blockIdx.y) * splits + split) * kPerWarp;
  for (int idx = threadIdx.x; idx < rows * D; idx += kThreads) {
    const int r = idx / D, d = idx - r * D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) m_all = fmaxf(m_all, scratch[w * kPerWarp + kRows * D + r]);
    const float base = (m_all == -INFINITY) ? 0.f : m_all;
    float acc = 0.f, l_all = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {  // fixed order
      const float f = ex2(scratch[w * kPerWarp + kRows * D + r] - base);
      acc = fmaf(f, scratch[w * kPerWarp + r * D + d], acc);
      l_all = fmaf(f, scratch[w * kPerWarp + kRows * D + kRows + r], l_all);
    }
    if (direct) {
      o[((size_t)b * H + h0 + r) * D + d] = pack1<kBf16>(l_all > 0.f ? acc / l_all : 0.f);  // no valid key: zeros
    } else {
      out_partial[r * D + d] = acc;
      if (d == 0) {
        out_partial[kRows * D + r] = m_all;
        out_partial[kRows * D + kRows + r] = l_all;
      }
    }
  }
}

// Combines the per-split partials of one (batch, query head).  `sets` > 1: several partial buffers of the same layout,
// `set_stride` floats apart (one per rank of a cache sharded along the sequence).  The block is D x kMergeLanes threads:
// lane j of a column folds partials j, j + kMergeLanes, ... (sets outer, splits inner) into a running (m, acc, l), four
// independent loads in flight, and the kMergeLanes (8, or 1) running triples are merged in lane order through shared memory -- a
// fixed order, so the result does not depend on timing.  (One thread per column walking 100+ splits in two serial
// passes was the whole cost of long-context decode at small batch: 31 us at Nk = 16384, batch 1.)
// A handful of splits (large batches) is folded by one lane per column: the wide block only costs there.
template <int D, bool kBf16, int kMergeLanes>
__global__ void __launch_bounds__(D * kMergeLanes)
attn_decode_merge_kernel(const float* __restrict__ partial, uint16_t* __restrict__ o, int H, int Hk, int splits, int sets,
                         long long set_stride) {
  constexpr int kPer = kRows * (D + 2);
  __shared__ float sm_m[kMergeLanes][D], sm_a[kMergeLanes][D], sm_l[kMergeLanes][D];
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x % D, j = threadIdx.x / D;
  pdl_wait();
  pdl_launch_dependents();
  const int G = H / Hk;
  const int chunks = (G + kRows - 1) / kRows;
  const int hk = h / G, within = h % G;
  const int slot = hk * chunks + within / kRows, r = within % kRows;
  const float* base_ptr = partial + ((size_t)b * (Hk * chunks) + slot) * splits * kPer;
  float m_run = -INFINITY, acc = 0.f, l_run = 0.f;
  const int total = sets * splits;
#pragma unroll 4
  for (int i = j; i < total; i += kMergeLanes) {
    const int t = i / splits, sp = i - t * splits;
    const float* ps = base_ptr + (size_t)t * set_stride + (size_t)sp * kPer;
    const float m_s = ps[kRows * D + r], l_s = ps[kRows * D + kRows + r], o_s = ps[r * D + d];
    const float m_new = fmaxf(m_run, m_s);
    if (m_new > -INFINITY) {
      const float keep = ex2(m_run - m_new), f = ex2(m_s - m_new);   // ex2(-inf) = 0
      acc = fmaf(f, o_s, acc * keep);
      l_run = fmaf(f, l_s, l_run * keep);
      m_run = m_new;
    }
  }
  sm_m[j][d] = m_run; sm_a[j][d] = acc; sm_l[j][d] = l_run;
  __syncthreads();
  if (j == 0) {
    float m_all = -INFINITY;
#pragma unroll
    for (int k = 0; k < kMergeLanes; ++k) m_all = fmaxf(m_all, sm_m[k][d]);
    float a = 0.f, l = 0.f;
    if (m_all > -INFINITY) {
#pragma unroll
      for (int k = 0; k < kMergeLanes; ++k) {
        const float f = ex2(sm_m[k][d] - m_all);
        a = fmaf(f, sm_a[k][d], a);
        l = fmaf(f, sm_l[k][d], l);
      }
    }
    o[((size_t)b * H + h) * D + d] = pack1<kBf16>(l > 0.f ? a / l : 0.f);  // no valid key: zeros
  }
}

struct SplitPlan {
  int chunks, splits, keys_per_split;
};

SplitPlan plan_splits(int B, int H, int Hk, int Nk, int D) {
  // Choose the number of key splits so that the grid fills whole waves of resident CTAs
  // (3 per SM at D = 64, 1 at D = 128: shared memory) while every split keeps at least 2 tiles.
  SplitPlan p;
  const int G = H / Hk;
  p.chunks = ceil_div(G, kRows);
  const long long groups = (long long)B * Hk * p.chunks;
  const int tiles = ceil_div(Nk, kTileKeys);
  const long long slots = (long long)sm_count() * (D == 64 ? 3 : 1);
  int best = 1;
  double best_score = -1.0;
  const int max_splits = tiles >= 4 ? (tiles / 2 < 128 ? tiles / 2 : 128) : 1;
  for (int s = 1; s <= max_splits; ++s) {
    const int per = ceil_div(tiles, s);
    const int real = ceil_div(tiles, per);           // splits actually launched
    if (real != s) continue;
    const double waves = (double)(groups * real) / (double)slots;
    const double full = waves <= 1.0 ? 1.0 : (double)(long long)(waves + 0.999999);
    // time ~ full waves x tiles per split (+1 tile of fixed cost per CTA); lower is better
    const double cost = full * (per + 1.0) + (waves <= 1.0 ? (1.0 - waves) * 0.01 : 0.0);
    const double score = 1.0 / cost;
    if (score > best_score * 1.0001) { best_score = score; best = real; }
  }
  // A split plan needs the merge kernel, a second launch worth about 12 key tiles of a CTA; when the unsplit plan is
  // within that, it wins (end-to-end decode of the 22-layer model at a cache of 784: 0.849 -> 0.843 ms per step at batch
  // 1, 1.125 -> 1.099 at batch 8, 1.630 -> 1.548 at batch 32; with 24 tiles a lone 1024-key call gets slower).
  constexpr double kMergeCostTiles = 12.0;
  if (best > 1) {
    const int per = ceil_div(tiles, best);
    const double waves = (double)(groups * best) / (double)slots;
    const double full = waves <= 1.0 ? 1.0 : (double)(long long)(waves + 0.999999);
    const double unsplit = (double)(long long)((double)groups / (double)slots + 0.999999) * (tiles + 1.0);
    if (full * (per + 1.0) + kMergeCostTiles >= unsplit) best = 1;
  }
  const int tiles_per_split = ceil_div(tiles, best);
  p.keys_per_split = tiles_per_split * kTileKeys;
  p.splits = ceil_div(Nk, p.keys_per_split);
  return p;
}

template <int D, bool kBf16, int kStages>
int launch_stages(const Problem& p, const SplitPlan& plan, const CUtensorMap& tk, const CUtensorMap& tv, float* partial,
                  unsigned int* status, cudaStream_t stream, bool partial_only);

template <int D, bool kBf16>
int launch_merge_lanes(const float* partial, uint16_t* o, int B, int H, int Hk, int splits, int sets, long long set_stride,
                       cudaStream_t stream) {
  const dim3 grid(H, B);
  if ((long long)splits * sets >= 8)
    return launch_kernel("attn_decode_merge_kernel", attn_decode_merge_kernel<D, kBf16, 8>, grid, dim3(D * 8), 0, stream, pdl_enabled(),
                         partial, o, H, Hk, splits, sets, set_stride);
  return launch_kernel("attn_decode_merge_kernel", attn_decode_merge_kernel<D, kBf16, 1>, grid, dim3(D), 0, stream, pdl_enabled(),
                       partial, o, H, Hk, splits, sets, set_stride);
}

template <int D, bool kBf16>
int launch(const Problem& p, const SplitPlan& plan, const CUtensorMap& tk, const CUtensorMap& tv, float* partial,
           unsigned int* status, cudaStream_t stream, bool partial_only = false) {
  const dim3 grid_probe(plan.splits, p.Hk * plan.chunks, p.B);
  const long long ctas = (long long)grid_probe.x * grid_probe.y * grid_probe.z;
  if (ctas <= sm_count() && ceil_div(plan.keys_per_split, kTileKeys) > kStagesShallow)
    return launch_stages<D, kBf16, deep_stages<D>()>(p, plan, tk, tv, partial, status, stream, partial_only);
  return launch_stages<D, kBf16, kStagesShallow>(p, plan, tk, tv, partial, status, stream, partial_only);
}

template <int D, bool kBf16, int kStages>
int launch_stages(const Problem& p, const SplitPlan& plan, const CUtensorMap& tk, const CUtensorMap& tv, float* partial,
                  unsigned int* status, cudaStream_t stream, bool partial_only) {
  using L = Layout<D, kStages>;
  auto kernel = attn_decode_kernel<D, kBf16, kStages>;
  static bool configured[64] = {false};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    configured[dev] = true;
  }
  const dim3 grid(plan.splits, p.Hk * plan.chunks, p.B);
  if (int rc = launch_kernel("attn_decode_kernel", kernel, grid, dim3(kThreads), L::kAlloc, stream, pdl_enabled(), tk, tv,
                             (const uint16_t*)p.q, (uint16_t*)p.o, partial, p.H, p.Hk, p.Nk, plan.keys_per_split,
                             p.scale * 1.4426950408889634f, status, p.kv_len_dev, partial_only ? 1 : 0))
    return rc;
  if (plan.splits > 1 && !partial_only)
    return launch_merge_lanes<D, kBf16>((const float*)partial, (uint16_t*)p.o, p.B, p.H, p.Hk, plan.splits, 1, 0LL, stream);
  return KFB_OK;
}

}  // namespace

size_t decode_ws_bytes(int B, int H, int Hk, int Nk, int D) {
  const SplitPlan plan = plan_splits(B, H, Hk, Nk, D);
  if (plan.splits <= 1) return 0;
  return (size_t)B * Hk * plan.chunks * plan.splits * kRows * (D + 2) * sizeof(float);
}

size_t decode_partial_bytes(int B, int H, int Hk, int Nk, int D, int* splits_out) {
  const SplitPlan plan = plan_splits(B, H, Hk, Nk, D);
  if (splits_out) *splits_out = plan.splits;
  return (size_t)B * Hk * plan.chunks * plan.splits * kRows * (D + 2) * sizeof(float);
}

int launch_merge(const float* partial, void* o, int dtype, int B, int H, int Hk, int D, int splits, int sets, long long set_stride,
                 cudaStream_t stream) {
  if (H > 65535 || B > 65535) return fail(KFB_ERR_INVALID, "B and H must each be <= 65535");
  const bool bf16 = dtype == KFB_BF16;
  if (D == 64)
    return bf16 ? launch_merge_lanes<64, true>(partial, (uint16_t*)o, B, H, Hk, splits, sets, set_stride, stream)
                : launch_merge_lanes<64, false>(partial, (uint16_t*)o, B, H, Hk, splits, sets, set_stride, stream);
  return bf16 ? launch_merge_lanes<128, true>(partial, (uint16_t*)o, B, H, Hk, splits, sets, set_stride, stream)
              : launch_merge_lanes<128, false>(partial, (uint16_t*)o, B, H, Hk, splits, sets, set_stride, stream);
}

int launch_decode(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t stream, bool partial_only) {
  if (p.Hk * ceil_div(p.H / p.Hk, kRows) > 65535 || p.B > 65535 || p.H > 65535)
    return fail(KFB_ERR_INVALID, "B, H and Hk * ceil(H/Hk/16) must each be <= 65535");
  const SplitPlan plan = plan_splits(p.B, p.H, p.Hk, p.Nk, p.D);
  const size_t need = partial_only ? decode_partial_bytes(p.B, p.H, p.Hk, p.Nk, p.D, nullptr) : decode_ws_bytes(p.B, p.H, p.Hk, p.Nk, p.D);
  if (need > 0 && (!ws || ws_bytes < need))
    return fail(KFB_ERR_WORKSPACE, "decode attention needs a %zu-byte workspace, got %zu", need, ws_bytes);
  if (need > 0 && !aligned16(ws)) return fail(KFB_ERR_ALIGNMENT, "workspace must be 16-byte aligned");
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  CUtensorMap tk, tv;
  const uint64_t D = p.D;
  const uint64_t kd[4] = {D, (uint64_t)p.Nk, (uint64_t)p.Hk, (uint64_t)p.B};
  const uint64_t ks[3] = {(uint64_t)p.kv_stride_n * 2, (uint64_t)p.kv_stride_h * 2, (uint64_t)p.kv_stride_b * 2};
  const uint32_t box[4] = {64, kTileKeys, 1, 1};
  if (int rc = make_tmap_4d_sw128(&tk, p.k, p.dtype, kd, ks, box)) return rc;
  if (int rc = make_tmap_4d_sw128(&tv, p.v, p.dtype, kd, ks, box)) return rc;
  const bool bf16 = p.dtype == KFB_BF16;
  float* partial = static_cast<float*>(ws);
  if (p.D == 64)
    return bf16 ? launch<64, true>(p, plan, tk, tv, partial, status, stream, partial_only)
                : launch<64, false>(p, plan, tk, tv, partial, status, stream, partial_only);
  return bf16 ? launch<128, true>(p, plan, tk, tv, partial, status, stream, partial_only)
              : launch<128, false>(p, plan, tk, tv, partial, status, stream, partial_only);
}

}  // namespace attn
}  // namespace kfb

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// The split-KV kernel above hands its per-split partial results (O, m, l) from the first kernel to
// the merge kernel through a workspace that the caller normally allocates.  Some callers cannot do
// that: a serving loop that has already handed all device memory to its KV-cache pool, code running
// inside a CUDA-graph capture (cudaMalloc is illegal there), or a host runtime that simply has no
// allocator of its own.  For them the partials live in the fixed array below, which is part of the
// library image: every GPU that loads the library holds these kMaxScratchBytes until the process
// exits, whether or not the entry point is ever called.
//
// In host code the NAME of a __device__ array is only a host-side stand-in, not a device address,
// so the address is resolved once per device with cudaGetSymbolAddress (that device being current)
// and that pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------------
#include <mutex>

namespace kfb {
namespace attn {
namespace {

constexpr size_t kMaxScratchBytes = 4u << 20;  // 4 MiB: up to 992 (group, split) partials at D = 64, 504 at D = 128
static __device__ __align__(256) unsigned char g_decode_scratch[kMaxScratchBytes];

std::mutex g_scratch_mutex;
void* g_scratch_ptr[64] = {nullptr};

// Device address of g_decode_scratch on the current device (resolved on the first call per device).
int static_scratch(void** out) {
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(KFB_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || !p)
      return fail(KFB_ERR_CUDA, "cudaGetSymbolAddress(decode scratch) failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return KFB_OK;
}

}  // namespace
}  // namespace attn
}  // namespace kfb

extern "C" int kfb_flash_attn_decode_noalloc(const void* q, const void* k, const void* v, void* o, int dtype, int B,
                                             int H, int Hk, int Nk, int D, float scale, const int64_t* kv_strides,
                                             void* stream) {
  using namespace kfb;
  if (int rc = require_sm100()) return rc;
  if (dtype != KFB_F16 && dtype != KFB_BF16) return fail(KFB_ERR_INVALID, "attention takes fp16 or bf16 tensors");
  if (B < 1 || H < 1 || Hk < 1 || Nk < 1) return fail(KFB_ERR_INVALID, "B, H, Hk, Nk must be >= 1");
  if (D != 64 && D != 128) return fail(KFB_ERR_INVALID, "head dim must be one of (64, 128), got %d", D);
  if (H % Hk) return fail(KFB_ERR_INVALID, "query heads (%d) must be a multiple of key/value heads (%d)", H, Hk);
  if (!(scale > 0.0f)) return fail(KFB_ERR_INVALID, "scale must be positive, got %g", (double)scale);
  if (!q || !k || !v || !o) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(KFB_ERR_ALIGNMENT, "q, k, v, o must be 16-byte aligned");
  const size_t need = attn::decode_ws_bytes(B, H, Hk, Nk, D);
  if (need > attn::kMaxScratchBytes)
    return fail(KFB_ERR_WORKSPACE,
                "this problem needs %zu bytes of split-KV scratch but the built-in array holds %zu; "
                "use kfb_flash_attn_fwd with a caller-provided workspace",
                need, attn::kMaxScratchBytes);
  attn::Problem p;
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.dtype = dtype; p.B = B; p.H = H; p.Hk = Hk; p.Nq = 1; p.Nk = Nk; p.D = D;
  p.causal = 0;  // a single query at the last position sees every key
  p.scale = scale;
  if (kv_strides) {
    p.kv_stride_b = kv_strides[0]; p.kv_stride_h = kv_strides[1]; p.kv_stride_n = kv_strides[2];
    if (p.kv_stride_n < D || p.kv_stride_h < 1 || p.kv_stride_b < 1 || (p.kv_stride_b % 8) || (p.kv_stride_h % 8) ||
        (p.kv_stride_n % 8))
      return fail(KFB_ERR_ALIGNMENT, "kv strides must be positive multiples of 8 elements with a row stride >= D");
  } else {
    p.kv_stride_n = D; p.kv_stride_h = (long long)Nk * D; p.kv_stride_b = (long long)Hk * Nk * D;
  }
  void* scratch = nullptr;
  if (int rc = attn::static_scratch(&scratch)) return rc;
  // Every partial the merge kernel reads is written by the split kernel of the same call, so
  // nothing left in the array by an earlier call is ever consumed and nothing needs clearing.
  return attn::launch_decode(p, scratch, attn::kMaxScratchBytes, (cudaStream_t)stream);
}
