// Fused attention forward for sm_100a, general path (any Nq, Nk; GQA; bottom-right causal mask).
//
// Replaces attn_v4_kernel of the reference (csrc/attention/attn_v4_kernel.cuh:43-214), which is an
// mma.sync / ldmatrix / cp.async kernel.  Two kernels built on the Blackwell execution model (TMA into
// 128-byte-swizzled shared-memory tiles, tcgen05.mma issued by one thread, accumulators in TMEM):
//
//   pair::attn_prefill_pair_kernel    one CTA per SM owns TWO adjacent query tiles of 128 rows of one
//                                     (batch, head); steps of 128 keys.  All 512 TMEM columns: two S
//                                     buffers, two O accumulators, two P buffers.  Two softmax
//                                     warpgroups (one per tile) share the exponential unit of the SM
//                                     in alternation while one thread feeds the tensor cores for both.
//   serial::attn_prefill_serial_kernel one CTA per 128 query rows, two CTAs per SM (256 columns each).
//
// Common to both: thread r of a softmax warpgroup owns query row r = TMEM lane r, so row maximum and
// row sum need no shuffles; lazy rescale (the running base of a row only moves when the new maximum
// exceeds it by more than 8 in log2 units -- a factor 256, far inside fp32 range -- and only then is
// O in TMEM rescaled; O and l always share one base, so O / l is unaffected); causal: key steps above
// the diagonal are never loaded or multiplied (loop bound), masking only on the diagonal / ragged
// steps, query tiles are scheduled heaviest-first (query tile is the slowest-varying grid index,
// reversed); GQA: kv head = h / (H / Hk); TMA zero-fills rows past Nq / Nk, those keys are masked.
//
// Numerics (as the reference, attn_v4_kernel.cuh:133-213): scores accumulate in FP32; x = s *
// (scale * log2 e); masked = -inf; p = 2^(x - base); the row sum adds the unrounded p, the PV
// product uses p rounded to fp16/bf16; O / l rounded once.  2^x is ex2.approx.ftz.f32.
#include "attn.cuh"
#include "sm100.cuh"

#include <algorithm>

namespace kfb {
namespace attn {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;   // keys per TMA tile and per step
constexpr int kThreads = 192;  // single-tile kernel
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr uint32_t kTmemCols = 256;
constexpr int kHalfBytes = kBlockN * 128;  // one 64-column half of a tile: 128 rows x 128 bytes
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum WaitCode : uint32_t {
  kWaitQ = 0x101, kWaitKEmpty, kWaitKFull, kWaitVEmpty, kWaitVFull, kWaitSFull, kWaitPReady, kWaitPvDone, kWaitIssuer, kWaitTurn
};

template <int D>
struct Layout {
  static constexpr int kStages = D == 64 ? 2 : 1;
  static constexpr int kTile = kBlockN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kBars = kV + kStages * kTile;
  static constexpr int kNumBars = 4 * kStages + 7;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kBytes = kMisc + 16;
  static constexpr int kAlloc = kBytes + 1024;  // room to align the tiles to 1024 bytes
  static_assert(2 * kAlloc <= 227 * 1024, "two CTAs must fit on one SM");
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
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

// Launch order of the 1-D grid.  (batch, head) pairs are taken in groups of `heads_per_group` whose K/V fit in L2
// together; inside a group the query tile (or tile pair) index is the slower one and runs from the last tile to the
// first, so that under a causal mask every long tile of the group starts before any short one, while the CTAs
// resident at one time still share the K/V of few heads.  (Heaviest-first over ALL heads at once made the resident
// CTAs stream the K/V of every head at the same time: at N = 8192, D = 128 that is 134 MB, more than L2.)
struct TileOrder {
  int q_index, bh;
};
__device__ __forceinline__ TileOrder decode_tile_order(unsigned int block, int n_q, int bh_total, int heads_per_group) {
  const unsigned int per_group = (unsigned int)n_q * (unsigned int)heads_per_group;
  const int group = (int)(block / per_group);
  const int base = group * heads_per_group;
  const int size = min(heads_per_group, bh_total - base);
  const int r = (int)(block - (unsigned int)group * per_group);
  return TileOrder{n_q - 1 - r / size, base + r % size};
}

// ------------------------------------------------------------------------------------------------
// Single-tile kernel: one CTA per 128 query rows, two CTAs resident per SM (256 TMEM columns each).
// One S buffer of 128 keys, QK(j+1) issued behind PV(j), the softmax in two passes over S in TMEM
// (maximum, then exponentials), P aliased on the S columns already consumed.  Used for head dim 128
// and for problems with a single query tile (Nq <= 128: chunked prefill, short prompts), where a
// CTA of the pair kernel below would run half empty.
// ------------------------------------------------------------------------------------------------
namespace serial {

constexpr uint32_t kSerialColS = 0, kSerialColP = 0, kSerialColO = 128;

// Row maximum of the 128 scores of this thread's row.  The four 32-column TMEM loads are issued
// back to back (the data of chunk c+1 is in flight while chunk c is reduced); eight independent
// max chains.  kMask: columns past `limit` (causal diagonal / ragged tile) count as -inf.
template <bool kMask>
__device__ __forceinline__ float row_max(uint32_t s_tmem, int limit) {
  float mx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
  uint32_t v[2][32];
  tmem_ld_x32(s_tmem, v[0]);
  tmem_wait_ld_regs(v[0]);
#pragma unroll
  for (int c = 0; c < kBlockN / 32; ++c) {
    if (c + 1 < kBlockN / 32) tmem_ld_x32(s_tmem + (c + 1) * 32, v[(c + 1) & 1]);  // in flight during chunk c
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float x = __uint_as_float(v[c & 1][i]);
      if (kMask && c * 32 + i > limit) x = -INFINITY;
      mx[i & 7] = fmaxf(mx[i & 7], x);
    }
    if (c + 1 < kBlockN / 32) tmem_wait_ld_regs(v[(c + 1) & 1]);
  }
  return fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
}

// p = 2^(x * scale - base) for the 128 scores of the row, rounded to the I/O type and stored to
// TMEM columns [16c, 16c+16) of `p_tmem` (which may alias the S columns: chunk c of P only covers
// columns that chunk <= c of S has already been read from).  Returns the FP32 row sum.
// ex2.approx.f32 per element; the sum adds the unrounded p (the reference's rule).  (ex2.approx.f16x2 on
// pairs was tried: no faster on B200 -- 409 vs 433 TFLOP/s -- and less accurate, so it is not used.)
// After the first half of the row (64 keys) has been stored, `half_ready` is signalled so the
// issuer can start the first four PV MMAs while the second half is computed.
template <bool kMask, bool kBf16>
__device__ __forceinline__ float exp_and_store(uint32_t s_tmem, uint32_t p_tmem, int limit, float scale_log2, float base,
                                              uint64_t* half_ready) {
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t v[2][32];
  tmem_ld_x32(s_tmem, v[0]);
  tmem_wait_ld_regs(v[0]);
#pragma unroll
  for (int c = 0; c < kBlockN / 32; ++c) {
    if (c + 1 < kBlockN / 32) tmem_ld_x32(s_tmem + (c + 1) * 32, v[(c + 1) & 1]);  // in flight during chunk c
    uint32_t p16[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float x0 = __uint_as_float(v[c & 1][2 * i]), x1 = __uint_as_float(v[c & 1][2 * i + 1]);
      if (kMask && c * 32 + 2 * i > limit) x0 = -INFINITY;
      if (kMask && c * 32 + 2 * i + 1 > limit) x1 = -INFINITY;
      x0 = fmaf(x0, scale_log2, -base);
      x1 = fmaf(x1, scale_log2, -base);
      const float p0 = ex2(x0), p1 = ex2(x1);
      sum[i & 3] += p0 + p1;
      p16[i] = pack2<kBf16>(p0, p1);
    }
    tmem_st_x16(p_tmem + c * 16, p16);
    if (c == 1) {
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(half_ready);
    }
    if (c + 1 < kBlockN / 32) tmem_wait_ld_regs(v[(c + 1) & 1]);
  }
  return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

// Two CTAs are resident per SM (168 registers x 192 threads x 2 = 64512 <= 65536; 83 / 99 KB of
// shared memory each; 256 TMEM columns each): the softmax of one runs under the MMAs of the other.
// Measured at B=2 H=16 N=2048 D=64: 402 TFLOP/s with two resident CTAs, 206 with one.
template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 2)
attn_prefill_serial_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, void* __restrict__ o_ptr, int H, int Hk, int Nq, int Nk,
                    int causal, float scale_log2, int B, int n_q_tiles, int heads_per_group, unsigned int* status) {
  using L = Layout<D>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + S;
  uint64_t* v_full = k_empty + S;
  uint64_t* v_empty = v_full + S;
  uint64_t* s_full = v_empty + S;
  uint64_t* p_ready = s_full + 1;   // [0]: keys 0-63 of P stored, [1]: keys 64-127
  uint64_t* pv_done = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile uint32_t* abort_word = tmem_slot + 1;
  const AbortCtx ctx{abort_word, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileOrder ord = decode_tile_order(blockIdx.x, n_q_tiles, H * B, heads_per_group);
  const int q_tile = ord.q_index;
  const int h = ord.bh % H, b = ord.bh / H;
  const int hk = h / (H / Hk);
  const int q0 = q_tile * kBlockM;
  const int causal_off = Nk - Nq;
  int kv_end = Nk;
  if (causal) kv_end = min(Nk, min(q0 + kBlockM, Nq) + causal_off);
  const int n_tiles = (kv_end + kBlockN - 1) / kBlockN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < S; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(&p_ready[0], 128);
    mbar_init(&p_ready[1], 128);
    mbar_init(pv_done, 1);
    *abort_word = *reinterpret_cast<volatile unsigned int*>(status);  // a wait expired earlier on this device:
    fence_mbar_init();                                                // do no work, return at once
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool dead_on_arrival = *abort_word != 0;

  if (dead_on_arrival) {
    // fall through to the teardown
  } else if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_arrive_expect_tx(q_full, L::kTile);
#pragma unroll
      for (int half = 0; half < D / 64; ++half)
        tma_load_4d(smem + L::kQ + half * kHalfBytes, &tm_q, q_full, half * 64, q0, h, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % S;
        const uint32_t ph = (uint32_t)(j / S) & 1u;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, ctx, kWaitKEmpty)) break;
        mbar_arrive_expect_tx(&k_full[s], L::kTile);
#pragma unroll
        for (int half = 0; half < D / 64; ++half)
          tma_load_4d(smem + L::kK + s * L::kTile + half * kHalfBytes, &tm_k, &k_full[s], half * 64, j * kBlockN, hk, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, ctx, kWaitVEmpty)) break;
        mbar_arrive_expect_tx(&v_full[s], L::kTile);
#pragma unroll
        for (int half = 0; half < D / 64; ++half)
          tma_load_4d(smem + L::kV + s * L::kTile + half * kHalfBytes, &tm_v, &v_full[s], half * 64, j * kBlockN, hk, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ tcgen05.mma issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_f16(kBlockM, kBlockN, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_pv = idesc_f16(kBlockM, D, kBf16 ? 1 : 0, 0, 1);
      const uint32_t q_addr = smem_u32(smem + L::kQ);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % S;
        if (!mbar_wait(&k_full[s], (uint32_t)(j / S) & 1u, ctx, kWaitKFull)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + L::kK + s * L::kTile);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk / 4) * kHalfBytes + (uint32_t)(kk % 4) * 32u;
          mma_ss(tmem_base + kSerialColS, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024),
                 idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[s]);
        tc_commit(s_full);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, ctx, kWaitQ);
      ok = ok && issue_qk(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (!mbar_wait(&p_ready[0], (uint32_t)j & 1u, ctx, kWaitPReady)) break;
        const int s = j % S;
        if (!mbar_wait(&v_full[s], (uint32_t)(j / S) & 1u, ctx, kWaitVFull)) break;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + L::kV + s * L::kTile);
        bool halves_ok = true;
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          if (kk == kBlockN / 32) {  // second half of the keys: wait for the rest of P
            halves_ok = mbar_wait(&p_ready[1], (uint32_t)j & 1u, ctx, kWaitPReady);
            if (!halves_ok) break;
            tc_fence_after_sync();
          }
          // 16 keys per step: 16 rows of 128 bytes; the second 64-column block of V is kHalfBytes away
          mma_ts(tmem_base + kSerialColO, tmem_base + kSerialColP + (uint32_t)kk * 8u,
                 smem_desc_sw128(v_addr + kk * 2048, kHalfBytes, 1024), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        if (!halves_ok) break;
        tc_commit(&v_empty[s]);
        tc_commit(pv_done);
        if (j + 1 < n_tiles) {
          // S(j+1) overwrites the columns P(j) lives in.  tcgen05.mma instructions of one thread execute in
          // issue order, so PV(j) has read P before QK(j+1) writes.
          if (!issue_qk(j + 1)) break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0-3)
    const int row = threadIdx.x;  // query row inside the tile == TMEM lane
    const uint32_t lane_bits = (uint32_t)(warp * 32) << 16;
    const uint32_t s_tmem = tmem_base + kSerialColS + lane_bits;
    const uint32_t o_tmem = tmem_base + kSerialColO + lane_bits;
    float m_base = -INFINITY;  // the base O and l are currently expressed in (log2 units)
    float l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      // every lane polls: measured faster than one polling lane plus a shuffle (416 vs 346 TFLOP/s)
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, (uint32_t)j & 1u, ctx, kWaitSFull));
      if (!ok) break;
      tc_fence_after_sync();
      // S(j) complete implies PV(j-1) complete (the issuer orders them), so O may be touched here.
      const int k0 = j * kBlockN;
      const bool need_mask = (k0 + kBlockN > Nk) || (causal && (k0 + kBlockN - 1 > q0 + causal_off));
      int limit = Nk - 1;
      if (causal) limit = min(limit, q0 + row + causal_off);
      limit -= k0;  // last visible column of this tile for this row

      // ---- pass 1: row maximum
      const float m_tile = (need_mask ? row_max<true>(s_tmem, limit) : row_max<false>(s_tmem, limit)) * scale_log2;
      // lazy rescale: move the base only when the maximum outgrew it by more than the threshold
      const bool grow = m_tile > m_base + kRescaleThreshold || m_base == -INFINITY;
      float alpha = 1.0f;
      if (grow && m_tile != -INFINITY) {
        alpha = ex2(m_base - m_tile);  // 0 when m_base is still -inf
        m_base = m_tile;
      }
      const float base = (m_base == -INFINITY) ? 0.f : m_base;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_x32(o_tmem + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(o_tmem + c * 32, o);
        }
      }
      // ---- pass 2: p = 2^(x - base), row sum, P written over the S columns already consumed
      const uint32_t p_tmem = tmem_base + kSerialColP + lane_bits;
      const float tile_sum = need_mask ? exp_and_store<true, kBf16>(s_tmem, p_tmem, limit, scale_log2, base, &p_ready[0])
                                       : exp_and_store<false, kBf16>(s_tmem, p_tmem, limit, scale_log2, base, &p_ready[0]);
      l_run = fmaf(l_run, alpha, tile_sum);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[1]);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)(n_tiles - 1) & 1u, ctx, kWaitPvDone));
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = 1.0f / l_run;
      const bool store = q0 + row < Nq;
      uint8_t* dst = static_cast<uint8_t*>(o_ptr) + ((((size_t)b * H + h) * Nq + (size_t)(q0 + row)) * D) * 2;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(o_tmem + c * 32, o);
        tmem_wait_ld();
        if (store) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[i] = pack2<kBf16>(__uint_as_float(o[2 * i]) * inv_l, __uint_as_float(o[2 * i + 1]) * inv_l);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(dst + c * 64)[i] =
                make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        }
      }
    }
  }

  // teardown: every role falls through to here, also after an expired wait
  if (!dead_on_arrival && *abort_word != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);  // let copies in flight land
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace serial

// ------------------------------------------------------------------------------------------------
// Pair kernel: one CTA per SM, two query tiles (A = rows [q0, q0+128), B = the next 128) of one
// (batch, head), steps of 128 keys.  384 threads (three warpgroups; warp 11 only takes part in barriers):
//   warps 0-3  softmax of tile A, warps 4-7 softmax of tile B (warp w touches TMEM lanes 32 (w % 4)..);
//   warp 8     TMA producer: both Q tiles once, then K and V tiles of 128 keys through mbarrier rings;
//   warps 9,10 one thread each issues the tcgen05.mma of tile A / tile B from an event loop: whichever
//              of QK(j+1) and PV(j) of its tile has its inputs ready goes next.
// TMEM (all 512 columns), head dim 64:  S_X [128 X, +128)   O_X [256 + 64 X, +64)   P_X [384 + 64 X, +64)
//                          head dim 128: S_X [128 X, +128)   O_X [256 + 128 X, +128), P_X aliased on S_X [.., +64)
// A softmax thread loads the 128 scores of its row into registers in one go and releases the S buffer
// at once (head dim 64), so QK(j+1) of that tile runs while the thread is still working on step j and
// the softmax threads never wait for the tensor cores; P(j) goes to its own columns as soon as PV(j-1)
// has finished reading them.  With head dim 128 the 512 columns leave no room for separate P buffers:
// P(j) overwrites the first 64 columns of S(j) and QK(j+1) is queued behind PV(j) (tcgen05.mma
// instructions of one thread execute in issue order).
// Both tiles read the same K/V tiles, so each is brought into shared memory once for 256 query rows.
//
// What was measured on the way to this form (B=2 H=16 D=64 non-causal, TFLOP/s at N = 2048 / 8192, A/B on one box):
//   one issuer thread for both tiles, softmax warpgroups unordered                          485 / 657
//   one issuer thread per tile (issuing an MMA occupies the thread for about the MMA's duration and a commit for
//     ~130 clocks: one thread feeding both tiles was the bottleneck; polled with mbarrier.test_wait, because a
//     try_wait on a barrier that is not ready may suspend the thread)                        472 / 679
//   + the two warpgroups take turns on the exponential units, baton passed after a block     491 / 695
//   + baton passed half way through a block (this kernel)                                    534 / 765
//   a baton per scheduler (32 threads) instead of per warpgroup                              459 / 621
//   the first TMA loads issued before the set-up barrier                                     459 / 621
//   two threads per query row (640 threads, maxima exchanged through shared memory)          403 / 618
//   25 % of the exponentials as a degree-3 polynomial on the FMA pipe                        527 / 753
// A 128 x 128 score tile costs 1024 clocks of the SM's exponential units; a step timeline of this kernel shows ~1460
// clocks of exponentials per warp and step and ~1200 of everything else (score load, maxima, P store, barriers), the two
// tiles alternating: ~1570 clocks per tile and step, 65 % of the unit's rate.  The polynomial does not help because a
// warp's block of exponentials is bound by its own dependency chain (FMA -> ex2 -> add / convert), not by the unit.
// ------------------------------------------------------------------------------------------------
namespace pair {

#ifdef KFB_TRACE
// Tuning aid of -DKFB_TRACE builds: CTA 0 writes clock stamps [role][step < 32][8] (roles: 0 softmax thread of
// tile A, 1 of tile B, 2 issuer, 3 producer) into a buffer set through kfb_debug_set_attn_trace.
__device__ unsigned long long* g_trace_buf = nullptr;
#define KFB_STAMP(role, j, k)                                                                        \
  do {                                                                                               \
    if (trace_ptr != nullptr && (j) < 32) trace_ptr[((role) * 32 + (j)) * 8 + (k)] = clock64();   \
  } while (0)
#else
#define KFB_STAMP(role, j, k) do { } while (0)
#endif

constexpr int kPairThreads = 384;   // three warpgroups
constexpr int kPairProducerWarp = 8;
constexpr int kPairMmaWarp = 9;
constexpr uint32_t kPairTmemCols = 512;

template <int D>
struct PairLayout {
  static constexpr bool kAliasP = D == 128;
  static constexpr int kStages = D == 64 ? 4 : 2;
  static constexpr int kTile = kBlockN * D * 2;       // bytes of one 128-row tile (Q, K or V)
  static constexpr int kQ = 0;                        // Q_A, Q_B
  static constexpr int kK = 2 * kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kBars = kV + kStages * kTile;
  static constexpr int kNumBars = 1 + 4 * kStages + 10;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kBytes = kMisc + 16;
  static constexpr int kAlloc = kBytes + 1024;
  static_assert(kAlloc <= 227 * 1024, "must fit in shared memory");
  static_assert(2 * kAlloc > 228 * 1024, "one CTA per SM: a CTA allocates all 512 TMEM columns");
  static constexpr uint32_t kColS = 0;                       // + 128 X
  static constexpr uint32_t kColO = 256;                     // + D X
  static constexpr uint32_t kColP = kAliasP ? 0u : 384u;     // + (kAliasP ? 128 : 64) X
  static constexpr uint32_t kStrideP = kAliasP ? 128u : 64u;
};

// Maximum of the 128 scores of this thread's row (in registers); sixteen independent chains of
// three-input maxima.  kMask: columns past `limit` count as -inf.
template <bool kMask>
__device__ __forceinline__ float row_max128(const uint32_t (&v)[4][32], int limit) {
  float mx[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) mx[i] = -INFINITY;
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0 = __uint_as_float(v[c][i]), x1 = __uint_as_float(v[c][i + 1]);
      if (kMask && c * 32 + i > limit) x0 = -INFINITY;
      if (kMask && c * 32 + i + 1 > limit) x1 = -INFINITY;
      mx[i >> 1] = max3(mx[i >> 1], x0, x1);
    }
#pragma unroll
  for (int i = 0; i < 4; ++i) mx[i] = fmaxf(max3(mx[i], mx[i + 4], mx[i + 8]), mx[i + 12]);
  return fmaxf(max3(mx[0], mx[1], mx[2]), mx[3]);
}

// p = 2^(x * scale - base) for the 128 scores of the row, rounded to the I/O type into `p` (two per
// register).  Returns the FP32 row sum of the unrounded p.  Scale-and-subtract and the row sum use the
// two-wide FP32 instructions of sm_100 (one issue slot per two elements); results per element are
// those of the scalar forms.
template <bool kMask, bool kBf16>
__device__ __forceinline__ float exp128(const uint32_t (&v)[4][32], uint32_t (&p)[4][16], int limit, float scale_log2,
                                       float base, uint64_t* pass_baton) {
  float2 sum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
  const float2 sc2 = make_float2(scale_log2, scale_log2), nb2 = make_float2(-base, -base);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 x = make_float2(__uint_as_float(v[c][2 * i]), __uint_as_float(v[c][2 * i + 1]));
      if (kMask && c * 32 + 2 * i > limit) x.x = -INFINITY;
      if (kMask && c * 32 + 2 * i + 1 > limit) x.y = -INFINITY;
      x = __ffma2_rn(x, sc2, nb2);
      const float2 e = make_float2(ex2(x.x), ex2(x.y));
      sum[i & 3] = __fadd2_rn(sum[i & 3], e);
      p[c][i] = pack2<kBf16>(e.x, e.y);
    }
    if (c == 1) mbar_arrive(pass_baton);   // half way: the other warp's first exponentials fill the gaps of the last ones here
  }
  const float2 t = __fadd2_rn(__fadd2_rn(sum[0], sum[1]), __fadd2_rn(sum[2], sum[3]));
  return t.x + t.y;
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kPairThreads, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, void* __restrict__ o_ptr, int B, int H, int Hk, int Nq,
                         int Nk, int causal, float scale_log2, int n_pairs, int heads_per_group, unsigned int* status) {
  using L = PairLayout<D>;
  constexpr int S = L::kStages;
  constexpr bool kAliasP = L::kAliasP;
#ifdef KFB_TRACE
  const unsigned long long t_entry = clock64();
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + S;
  uint64_t* v_full = k_empty + S;
  uint64_t* v_empty = v_full + S;
  uint64_t* s_full = v_empty + S;    // [X]: S_X written by QK
  uint64_t* s_free = s_full + 2;     // [X]: all 128 threads of tile X hold their scores in registers
  uint64_t* p_ready = s_free + 2;    // [X]: P_X stored by all 128 threads
  uint64_t* pv_done = p_ready + 2;   // [X]: the PV product that read P_X has completed (O_X updated)
  uint64_t* turn = pv_done + 2;      // [X]: the other tile's warpgroup is half way through its exponentials: X may start
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile uint32_t* abort_word = tmem_slot + 1;
  const AbortCtx ctx{abort_word, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileOrder ord = decode_tile_order(blockIdx.x, n_pairs, H * B, heads_per_group);
  const int pair_idx = ord.q_index;
  const int h = ord.bh % H, b = ord.bh / H;
  const int hk = h / (H / Hk);
  const int q0 = pair_idx * 2 * kBlockM;
  const int causal_off = Nk - Nq;
  int n_steps[2];
#pragma unroll
  for (int X = 0; X < 2; ++X) {
    const int q0x = q0 + X * kBlockM;
    int kv_end = Nk;
    if (causal) kv_end = min(Nk, min(q0x + kBlockM, Nq) + causal_off);
    n_steps[X] = q0x < Nq ? (kv_end + kBlockN - 1) / kBlockN : 0;   // tile B may not exist
  }
  const int n_max = max(n_steps[0], n_steps[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < S; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 2);   // one arrival per issuer thread
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 2);
    }
    for (int X = 0; X < 2; ++X) {
      mbar_init(&s_full[X], 1);
      mbar_init(&s_free[X], 128);
      mbar_init(&p_ready[X], 128);
      mbar_init(&pv_done[X], 1);
      mbar_init(&turn[X], 128);
    }
    *abort_word = *reinterpret_cast<volatile unsigned int*>(status);  // a wait expired earlier on this device:
    fence_mbar_init();                                                // do no work, return at once
  }
  if (warp == kPairMmaWarp) {   // the first issuer warp also owns the TMEM allocation
    tmem_alloc(tmem_slot, kPairTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool dead_on_arrival = *abort_word != 0;
#ifdef KFB_TRACE
  unsigned long long* const trace_ptr = blockIdx.x == 0 ? g_trace_buf : nullptr;
  if (threadIdx.x == 0 && trace_ptr) { trace_ptr[31 * 8 + 0] = t_entry; trace_ptr[31 * 8 + 1] = clock64(); }
#endif

  // Registers move from the warpgroup of the two single-thread roles to the softmax warpgroups, which keep
  // the 128 scores of a row in registers (2 x 128 x 208 + 128 x 88 = 64512 of 65536).  Each role branch
  // starts with its setmaxnreg, executed by all four warps of its warpgroup.
  if (dead_on_arrival) {
    // fall through to the teardown
  } else if (warp >= kPairProducerWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (warp == kPairProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const int tiles = n_steps[1] > 0 ? 2 : 1;
      mbar_arrive_expect_tx(q_full, (uint32_t)(tiles * L::kTile));
      for (int X = 0; X < tiles; ++X)
#pragma unroll
        for (int half = 0; half < D / 64; ++half)
          tma_load_4d(smem + L::kQ + X * L::kTile + half * kHalfBytes, &tm_q, q_full, half * 64, q0 + X * kBlockM, h, b);
      for (int j = 0; j < n_max; ++j) {
        const int s = j % S;
        const uint32_t ph = (uint32_t)(j / S) & 1u;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, ctx, kWaitKEmpty)) break;
        mbar_arrive_expect_tx(&k_full[s], L::kTile);
#pragma unroll
        for (int half = 0; half < D / 64; ++half)
          tma_load_4d(smem + L::kK + s * L::kTile + half * kHalfBytes, &tm_k, &k_full[s], half * 64, j * kBlockN, hk, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, ctx, kWaitVEmpty)) break;
        mbar_arrive_expect_tx(&v_full[s], L::kTile);
#pragma unroll
        for (int half = 0; half < D / 64; ++half)
          tma_load_4d(smem + L::kV + s * L::kTile + half * kHalfBytes, &tm_v, &v_full[s], half * 64, j * kBlockN, hk, b);
      }
    }
  } else if (warp == kPairMmaWarp || warp == kPairMmaWarp + 1) {
    // ------------------------------------------------------------------ tcgen05.mma issuers (one thread per tile)
    // Issuing an MMA occupies the issuing thread for about as long as the MMA runs, and a commit for ~130 clocks,
    // so one thread feeding both tiles is the bottleneck of the CTA; with one issuer per tile the commits of one
    // overlap the MMAs of the other.  The two threads never touch each other's TMEM columns.  A K / V stage goes
    // back to the producer when BOTH have arrived on its `empty` barrier (count 2): a tile that does not need a
    // key tile (no tile B, or one step less under a causal mask) still arrives for it once it has been loaded.
    if (lane == 0) {
      const int X = warp - kPairMmaWarp;
      constexpr uint32_t idesc_qk = idesc_f16(kBlockM, kBlockN, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_pv = idesc_f16(kBlockM, D, kBf16 ? 1 : 0, 0, 1);
      const uint32_t qa = smem_u32(smem + L::kQ) + (uint32_t)X * L::kTile;
      const uint32_t k_addr0 = smem_u32(smem + L::kK), v_addr0 = smem_u32(smem + L::kV);
      const uint32_t s_col = tmem_base + L::kColS + 128u * X, o_col = tmem_base + L::kColO + (uint32_t)D * X;
      const uint32_t p_col = tmem_base + L::kColP + L::kStrideP * X;
      const int n = n_steps[X];
      int qk_next = 0, pv_next = 0;   // steps handled so far (issued, or passed on for a tile that has no such step)
      bool ok = n == 0 || mbar_wait(q_full, 0, ctx, kWaitQ);
      tc_fence_after_sync();
      uint32_t idle = 0;
      unsigned long long idle_since = 0;
      while (ok && (qk_next < n_max || pv_next < n_max)) {
        bool progress = false;
        // ---- S(j) = Q K(j)^T: needs the S buffer (scores of step j-1 in registers; with aliased P: PV(j-1)
        //      issued, which executes first) and the K tile
        if (qk_next < n_max) {
          const int j = qk_next, s = j % S;
          if (j >= n) {   // not a step of this tile: hand the stage on as soon as it has been filled
            if (mbar_test_wait(&k_full[s], (uint32_t)(j / S) & 1u)) {
              mbar_arrive(&k_empty[s]);
              qk_next = j + 1;
              progress = true;
            }
          } else {
            const bool buffer_free = kAliasP ? (pv_next >= j) : (j == 0 || mbar_test_wait(&s_free[X], (uint32_t)(j - 1) & 1u));
            if (buffer_free && mbar_test_wait(&k_full[s], (uint32_t)(j / S) & 1u)) {
              KFB_STAMP(2 + X, j, 0);
              tc_fence_after_sync();
              const uint32_t ka = k_addr0 + (uint32_t)s * L::kTile;
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (uint32_t)(kk / 4) * kHalfBytes + (uint32_t)(kk % 4) * 32u;
                mma_ss(s_col, smem_desc_sw128(qa + off, 16, 1024), smem_desc_sw128(ka + off, 16, 1024), idesc_qk,
                       kk > 0 ? 1u : 0u);
              }
              KFB_STAMP(2 + X, j, 1);
              tc_commit(&s_full[X]);
              tc_commit(&k_empty[s]);
              KFB_STAMP(2 + X, j, 2);
              qk_next = j + 1;
              progress = true;
            }
          }
        }
        // ---- O += P(j) V(j): needs P (stored by the 128 softmax threads of the tile) and the V tile
        if (pv_next < n_max && pv_next < qk_next) {
          const int j = pv_next, s = j % S;
          if (j >= n) {
            if (mbar_test_wait(&v_full[s], (uint32_t)(j / S) & 1u)) {
              mbar_arrive(&v_empty[s]);
              pv_next = j + 1;
              progress = true;
            }
          } else if (mbar_test_wait(&p_ready[X], (uint32_t)j & 1u) && mbar_test_wait(&v_full[s], (uint32_t)(j / S) & 1u)) {
            KFB_STAMP(2 + X, j, 3);
            tc_fence_after_sync();
            const uint32_t va = v_addr0 + (uint32_t)s * L::kTile;
#pragma unroll
            for (int kk = 0; kk < kBlockN / 16; ++kk) {
              // 16 keys per MMA: 16 rows of 128 bytes; the second 64-column block of V is kHalfBytes away
              mma_ts(o_col, p_col + (uint32_t)kk * 8u, smem_desc_sw128(va + kk * 2048, kHalfBytes, 1024), idesc_pv,
                     (j > 0 || kk > 0) ? 1u : 0u);
            }
            KFB_STAMP(2 + X, j, 4);
            tc_commit(&pv_done[X]);
            tc_commit(&v_empty[s]);
            KFB_STAMP(2 + X, j, 5);
            pv_next = j + 1;
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
          idle_since = 0;
        } else if ((++idle & 63u) == 0) {   // bounded like every other wait of the library
          if (*abort_word != 0) break;
          const unsigned long long now = globaltimer_ns();
          if (idle_since == 0) {
            idle_since = now;
          } else if (now - idle_since > ctx.timeout_ns) {
            *abort_word = kWaitIssuer;
            atomicCAS(status, 0u, (unsigned int)kWaitIssuer);
            break;
          }
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0-7)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int X = warp >> 2;                      // which tile
    const int row = threadIdx.x & 127;            // query row inside the tile == TMEM lane
    const int q0x = q0 + X * kBlockM;
    const int n = n_steps[X];
    const uint32_t lane_bits = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + L::kColS + 128u * X + lane_bits;
    const uint32_t p_tmem = tmem_base + L::kColP + L::kStrideP * X + lane_bits;
    const uint32_t o_tmem = tmem_base + L::kColO + (uint32_t)D * X + lane_bits;
    float m_base = -INFINITY;  // the base O and l are currently expressed in (log2 units)
    float l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_max; ++j) {
      const uint32_t ph = (uint32_t)j & 1u;
      if (j >= n) {
        // no such step for this tile (no tile B, or one step less under a causal mask): only pass the baton on
        if (X == 1 || j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&turn[X], (X == 1 ? ph : ph ^ 1u), ctx, kWaitTurn));
          if (!ok) break;
        }
        mbar_arrive(&turn[X ^ 1]);
        continue;
      }
      // every lane polls: measured faster than one polling lane plus a shuffle
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[X], ph, ctx, kWaitSFull));
      if (!ok) break;
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 0);
      tc_fence_after_sync();
      uint32_t v[4][32];   // the 128 scores of this row, loaded once
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x32(s_tmem + c * 32, v[c]);
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_wait_ld_regs(v[c]);
      if constexpr (!kAliasP) {   // the S buffer can take the next product already
        tc_fence_before_sync();
        mbar_arrive(&s_free[X]);
      }
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 1);
      const int k0 = j * kBlockN;
      const bool need_mask = (k0 + kBlockN > Nk) || (causal && (k0 + kBlockN - 1 > q0x + causal_off));
      int limit = Nk - 1;
      if (causal) limit = min(limit, q0x + row + causal_off);
      limit -= k0;  // last visible column of this step for this row

      const float m_step = (need_mask ? row_max128<true>(v, limit) : row_max128<false>(v, limit)) * scale_log2;
      // lazy rescale: move the base only when the maximum outgrew it by more than the threshold
      const bool grow = m_step > m_base + kRescaleThreshold || m_base == -INFINITY;
      float alpha = 1.0f;
      if (grow && m_step != -INFINITY) {
        alpha = ex2(m_base - m_step);  // 0 when m_base is still -inf
        m_base = m_step;
      }
      const float base = (m_base == -INFINITY) ? 0.f : m_base;
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 2);
      bool rescaled = false;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        // O is rescaled between PV(j-1), which must have finished accumulating, and PV(j), which cannot have
        // started (it waits for this step's P).  Rare after the first steps.
        rescaled = true;
        if constexpr (!kAliasP) {
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[X], (uint32_t)(j - 1) & 1u, ctx, kWaitPvDone));
          if (!ok) break;
          tc_fence_after_sync();
        }
        {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_x32(o_tmem + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(o_tmem + c * 32, o);
          }
        }
      }
      // The two warpgroups take turns on the exponential units: A(0), B(0), A(1), B(1), ...  Left alone they drift into
      // phase: both load scores and take maxima at the same time (units idle), then both want the units.  With the
      // baton one runs its exponentials while the other loads, takes maxima, stores P and synchronises.  The baton is
      // passed half way through, so the tail of one block overlaps the head of the next.  A waits for B(j-1), B for
      // A(j).  (A baton per scheduler -- 32 threads instead of 128 -- measured 15 % slower: 74 against 64 us at
      // B=2 H=16 N=2048; so did issuing the first TMA loads before the set-up barrier.)
      if (X == 1 || j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&turn[X], (X == 1 ? ph : ph ^ 1u), ctx, kWaitTurn));
        if (!ok) break;
      }
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 6);
      uint32_t p16[4][16];
      const float step_sum = need_mask ? exp128<true, kBf16>(v, p16, limit, scale_log2, base, &turn[X ^ 1])
                                       : exp128<false, kBf16>(v, p16, limit, scale_log2, base, &turn[X ^ 1]);
      l_run = fmaf(l_run, alpha, step_sum);
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 3);
      if constexpr (!kAliasP) {
        // PV(j-1) must have finished reading the P columns before they are overwritten.  By now it has: the
        // exponentials above take longer than the product.  (With aliased P it finished before S(j) was
        // written, which this thread has already waited for.)
        if (j > 0 && !rescaled) {
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[X], (uint32_t)(j - 1) & 1u, ctx, kWaitPvDone));
          if (!ok) break;
          tc_fence_after_sync();
        }
      }
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 4);
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_st_x16(p_tmem + c * 16, p16[c]);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[X]);
      if ((threadIdx.x & 127) == 0) KFB_STAMP(X, j, 5);
    }
    // PVs complete in issue order: the last one done means all are
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[X], (uint32_t)(n - 1) & 1u, ctx, kWaitPvDone));
    if (ok && n > 0) {
      if (threadIdx.x == 0) KFB_STAMP(0, 31, 2);
      tc_fence_after_sync();
      const float inv_l = 1.0f / l_run;
      const bool store = q0x + row < Nq;
      uint8_t* dst = static_cast<uint8_t*>(o_ptr) + ((((size_t)b * H + h) * Nq + (size_t)(q0x + row)) * D) * 2;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(o_tmem + c * 32, o);
        tmem_wait_ld();
        if (store) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[i] = pack2<kBf16>(__uint_as_float(o[2 * i]) * inv_l, __uint_as_float(o[2 * i + 1]) * inv_l);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(dst + c * 64)[i] =
                make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        }
      }
    }
  }

  // teardown: every role falls through to here, also after an expired wait
  if (!dead_on_arrival && *abort_word != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);  // let copies in flight land
  }
  if (threadIdx.x == 0) KFB_STAMP(0, 31, 3);
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) KFB_STAMP(0, 31, 4);
  if (warp == kPairMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem_base, kPairTmemCols);
  }
  if (threadIdx.x == kPairMmaWarp * 32) KFB_STAMP(0, 31, 5);
}

}  // namespace pair

// Head dims the pair kernel serves (the others, and single-tile problems, take the single-tile kernel).
constexpr bool pair_kernel_for(int D) {
#ifdef KFB_PAIR_D128
  return D == 64 || D == 128;
#else
  return D == 64;
#endif
}

template <int D, bool kBf16>
int launch(const Problem& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, unsigned int* status,
           cudaStream_t stream) {
  using L = Layout<D>;
  using PL = pair::PairLayout<D>;
  static bool configured[64] = {false};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(serial::attn_prefill_serial_kernel<D, kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      L::kAlloc));
    KFB_CUDA_TRY(cudaFuncSetAttribute(serial::attn_prefill_serial_kernel<D, kBf16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    KFB_CUDA_TRY(cudaFuncSetAttribute(pair::attn_prefill_pair_kernel<D, kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PL::kAlloc));
    configured[dev] = true;
  }
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const int q_tiles = ceil_div(p.Nq, kBlockM);
  const long long bh = (long long)p.B * p.H;
  // heads whose K and V (one KV head each at worst) fit in ~48 MB of L2 together
  const long long kv_bytes_per_head = 4LL * p.Nk * p.D;
  const int heads_per_group = (int)std::min<long long>(bh, std::max<long long>(1, (48LL << 20) / kv_bytes_per_head));
  if (pair_kernel_for(D) && q_tiles >= 2) {
    const int n_pairs = ceil_div(q_tiles, 2);
    if (bh * n_pairs > 0x7fffffffLL) return fail(KFB_ERR_INVALID, "too many query tiles for one launch");
    pair::attn_prefill_pair_kernel<D, kBf16><<<(unsigned)(bh * n_pairs), pair::kPairThreads, PL::kAlloc, stream>>>(
        tq, tk, tv, p.o, p.B, p.H, p.Hk, p.Nq, p.Nk, p.causal, scale_log2, n_pairs, heads_per_group, status);
    KFB_LAUNCH_CHECK("attn_prefill_pair_kernel");
    return KFB_OK;
  }
  if (bh * q_tiles > 0x7fffffffLL) return fail(KFB_ERR_INVALID, "too many query tiles for one launch");
  serial::attn_prefill_serial_kernel<D, kBf16><<<(unsigned)(bh * q_tiles), kThreads, L::kAlloc, stream>>>(
      tq, tk, tv, p.o, p.H, p.Hk, p.Nq, p.Nk, p.causal, scale_log2, p.B, q_tiles, heads_per_group, status);
  KFB_LAUNCH_CHECK("attn_prefill_serial_kernel");
  return KFB_OK;
}

}  // namespace

int launch_prefill(const Problem& p, cudaStream_t stream) {
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  CUtensorMap tq, tk, tv;
  const uint64_t D = p.D;
  const uint64_t qd[4] = {D, (uint64_t)p.Nq, (uint64_t)p.H, (uint64_t)p.B};
  const uint64_t qs[3] = {D * 2, (uint64_t)p.Nq * D * 2, (uint64_t)p.H * p.Nq * D * 2};
  const uint64_t kd[4] = {D, (uint64_t)p.Nk, (uint64_t)p.Hk, (uint64_t)p.B};
  const uint64_t ks[3] = {(uint64_t)p.kv_stride_n * 2, (uint64_t)p.kv_stride_h * 2, (uint64_t)p.kv_stride_b * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  if (int rc = make_tmap_4d_sw128(&tq, p.q, p.dtype, qd, qs, box)) return rc;
  if (int rc = make_tmap_4d_sw128(&tk, p.k, p.dtype, kd, ks, box)) return rc;
  if (int rc = make_tmap_4d_sw128(&tv, p.v, p.dtype, kd, ks, box)) return rc;
  const bool bf16 = p.dtype == KFB_BF16;
  if (p.D == 64) return bf16 ? launch<64, true>(p, tq, tk, tv, status, stream) : launch<64, false>(p, tq, tk, tv, status, stream);
  return bf16 ? launch<128, true>(p, tq, tk, tv, status, stream) : launch<128, false>(p, tq, tk, tv, status, stream);
}

}  // namespace attn
}  // namespace kfb

#ifdef KFB_TRACE
extern "C" void kfb_debug_set_attn_trace(void* device_buffer) {
  cudaMemcpyToSymbol(kfb::attn::pair::g_trace_buf, &device_buffer, sizeof(void*));
}
#endif
