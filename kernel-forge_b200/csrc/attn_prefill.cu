// Fused attention forward for sm_100a, general path (any Nq, Nk; GQA; bottom-right causal mask).
//
// Replaces attn_v4_kernel of the reference (csrc/attention/attn_v4_kernel.cuh:43-214), which is an
// mma.sync / ldmatrix / cp.async kernel.  This one is built on the Blackwell execution model:
//
//   * one CTA per 128 query rows of one (batch, head), two CTAs resident per SM (each takes 256 of
//     the 512 TMEM columns);
//   * 192 threads in three roles:
//       warp 4  (1 thread)  TMA producer: Q once, K and V tiles of 128 keys through mbarrier rings,
//                           128-byte-swizzled shared-memory tiles (a D=64 row is exactly 128 bytes)
//       warp 5  (1 thread)  tcgen05.mma issuer: S = Q K^T into TMEM and O += P V, both in the TS form
//                           (A operand read from TMEM): Q is written to TMEM once by the softmax
//                           threads, P every step; K is the K-major and V the MN-major shared-memory
//                           operand, so V needs no transpose.  An SS-form MMA re-reads its 4 KB A tile
//                           from shared memory every time (6 KB per M128 N64 K16 instruction at 128
//                           bytes per clock = 48 clocks against 16 of tensor time); with Q in TMEM
//                           only the 2 KB of K are read
//       warps 0-3 (128 thr) softmax: thread r owns query row r = TMEM lane r, so row max / row sum
//                           need no shuffles; the 64 scores of a step are loaded from TMEM once and
//                           kept in registers for both the maximum and the exponentials; P is rounded
//                           to the I/O type and written over the S columns it was computed from;
//                           epilogue O / l;
//   * software pipeline over steps of 64 keys with two S buffers in TMEM: the issuer queues QK(t+2)
//     right behind PV(t), so S(t+1) is already complete when the softmax warps finish step t, and
//     PV(t) runs under the softmax of step t+1.  The softmax warps never wait for the tensor cores;
//     they are the critical path (the exponentials: 16 per clock per SM);
//   * lazy rescale: the running base of a row only moves when the new maximum exceeds it by more
//     than 8 (a factor 256, far inside fp16/fp32 range); O in TMEM is rescaled only then (after
//     waiting for the PV of the previous step, the only one that can still be writing O).  O and l
//     always share one base, so the quotient O / l is unaffected;
//   * causal: steps above the diagonal are never multiplied (loop bound), masking only on the
//     diagonal / ragged steps; query tiles are scheduled heaviest-first;
//   * GQA: kv head = h / (H / Hk); TMA zero-fills rows past Nq / Nk, those keys are masked.
//
// TMEM columns of a CTA (256 allocated): S buffer b of step t = 2j + b at [64 b, 64 b + 64), with
// P of the same step (16-bit, 32 columns) aliased on its first 32 columns; O [128, 128 + D);
// Q (16-bit, D / 2 columns, row r in lane r) at [192, 192 + D / 2).
// tcgen05.mma instructions of one thread execute in issue order, so QK(t+2), which overwrites the
// columns of P(t), cannot pass PV(t), which reads them.
//
// Numerics (as the reference, attn_v4_kernel.cuh:133-213): scores accumulate in FP32; x = s *
// (scale * log2 e); masked = -inf; p = 2^(x - base); the row sum adds the unrounded p, the PV
// product uses p rounded to fp16/bf16; O / l rounded once.  2^x is ex2.approx.ftz.f32.
#include "attn.cuh"
#include "sm100.cuh"

#include <cstdlib>

namespace kfb {
namespace attn {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;   // keys per TMA tile
constexpr int kStepN = 64;     // keys per pipeline step (one S buffer)
constexpr int kThreads = 192;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColO = 128;   // S / P buffer b starts at column 64 b
constexpr uint32_t kColQ = 192;   // head dim 64 only: O ends at 192
constexpr int kHalfBytes = kBlockN * 128;  // one 64-column half of a tile: 128 rows x 128 bytes
constexpr int kStepBytes = kStepN * 128;   // 64 rows of 128 bytes inside such a half
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum WaitCode : uint32_t {
  kWaitQ = 0x101, kWaitKEmpty, kWaitKFull, kWaitVEmpty, kWaitVFull, kWaitSFull, kWaitPReady, kWaitPvDone
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

// Maximum of the 64 scores of this thread's row (already in registers); eight independent chains.
// kMask: columns past `limit` (causal diagonal / ragged step) count as -inf.
template <bool kMask>
__device__ __forceinline__ float row_max(const uint32_t (&v)[2][32], int limit) {
  float mx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float x = __uint_as_float(v[c][i]);
      if (kMask && c * 32 + i > limit) x = -INFINITY;
      mx[i & 7] = fmaxf(mx[i & 7], x);
    }
  return fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
}

// p = 2^(x * scale - base) for the 64 scores of the row, rounded to the I/O type and stored to TMEM
// columns [0, 32) of `p_tmem` (the first columns of the S buffer the scores came from).  Returns the
// FP32 row sum, which adds the unrounded p (the reference's rule).  ex2.approx.f32 per element
// (ex2.approx.f16x2 on pairs was tried: no faster on B200 and less accurate).
template <bool kMask, bool kBf16>
__device__ __forceinline__ float exp_and_store(const uint32_t (&v)[2][32], uint32_t p_tmem, int limit, float scale_log2,
                                              float base) {
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t p16[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float x0 = __uint_as_float(v[c][2 * i]), x1 = __uint_as_float(v[c][2 * i + 1]);
      if (kMask && c * 32 + 2 * i > limit) x0 = -INFINITY;
      if (kMask && c * 32 + 2 * i + 1 > limit) x1 = -INFINITY;
      x0 = fmaf(x0, scale_log2, -base);
      x1 = fmaf(x1, scale_log2, -base);
      const float p0 = ex2(x0), p1 = ex2(x1);
      sum[i & 3] += p0 + p1;
      p16[i] = pack2<kBf16>(p0, p1);
    }
    tmem_st_x16(p_tmem + c * 16, p16);
  }
  return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

// Two CTAs are resident per SM (168 registers x 192 threads x 2 = 64512 <= 65536; 83 / 99 KB of
// shared memory each; 256 TMEM columns each), so two softmax warps share every scheduler and its
// exponential unit.
template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 2)
attn_prefill_kernel(const void* __restrict__ q_ptr, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, void* __restrict__ o_ptr, int H, int Hk, int Nq, int Nk,
                    int causal, float scale_log2, unsigned int* status, unsigned long long* trace) {
  static_assert(D == 64, "Q, two S buffers and O share 256 TMEM columns only for head dim 64");
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
  uint64_t* s_full = v_empty + S;    // [b]: S buffer b written by QK
  uint64_t* p_ready = s_full + 2;    // [b]: P of buffer b stored by all 128 softmax threads (S consumed)
  uint64_t* pv_done = p_ready + 2;   // [b]: the PV product that read P of buffer b has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile uint32_t* abort_word = tmem_slot + 1;
  const AbortCtx ctx{abort_word, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // causal: the longest tiles start first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (H / Hk);
  const int q0 = q_tile * kBlockM;
  const int causal_off = Nk - Nq;
  int kv_end = Nk;
  if (causal) kv_end = min(Nk, min(q0 + kBlockM, Nq) + causal_off);
  const int n_steps = (kv_end + kStepN - 1) / kStepN;   // step t = keys [64 t, 64 t + 64) = half (t & 1) of tile t / 2
  const int n_tiles = (n_steps + 1) / 2;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 128);   // every softmax thread has stored its row of Q to TMEM
    for (int s = 0; s < S; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
      mbar_init(&pv_done[i], 1);
    }
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
  // optional timeline of CTA (0,0,0) for tuning: 16 clock stamps per step
  const bool tracing = trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  auto stamp = [&](int j, int k) {
    if (tracing && j < 64) trace[j * 16 + k] = clock64();
  };

  if (dead_on_arrival) {
    // fall through to the teardown
  } else if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
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
      constexpr uint32_t idesc_qk = idesc_f16(kBlockM, kStepN, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_pv = idesc_f16(kBlockM, D, kBf16 ? 1 : 0, 0, 1);
      auto issue_qk = [&](int t) -> bool {   // S buffer (t & 1) = Q K(step t)^T
        const int j = t >> 1, hh = t & 1, s = j % S;
        // the second step of a tile finds it already waited for (same thread, same phase)
        if (!mbar_wait(&k_full[s], (uint32_t)(j / S) & 1u, ctx, kWaitKFull)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + L::kK + s * L::kTile) + (uint32_t)hh * kStepBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk / 4) * kHalfBytes + (uint32_t)(kk % 4) * 32u;
          mma_ts(tmem_base + (uint32_t)hh * kStepN, tmem_base + kColQ + (uint32_t)kk * 8u,
                 smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        if (hh == 1 || t == n_steps - 1) tc_commit(&k_empty[s]);
        tc_commit(&s_full[hh]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, ctx, kWaitQ);
      tc_fence_after_sync();
      ok = ok && issue_qk(0);
      if (n_steps > 1) ok = ok && issue_qk(1);
      for (int t = 0; ok && t < n_steps; ++t) {
        const int j = t >> 1, hh = t & 1, s = j % S;
        if (!mbar_wait(&p_ready[hh], (uint32_t)j & 1u, ctx, kWaitPReady)) break;
        stamp(t, 8);
        if (!mbar_wait(&v_full[s], (uint32_t)(j / S) & 1u, ctx, kWaitVFull)) break;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + L::kV + s * L::kTile);
#pragma unroll
        for (int kk = 0; kk < kStepN / 16; ++kk) {
          // 16 keys per MMA: 16 rows of 128 bytes; the second 64-column block of V is kHalfBytes away
          mma_ts(tmem_base + kColO, tmem_base + (uint32_t)hh * kStepN + (uint32_t)kk * 8u,
                 smem_desc_sw128(v_addr + (hh * 4 + kk) * 2048, kHalfBytes, 1024), idesc_pv, (t > 0 || kk > 0) ? 1u : 0u);
        }
        if (hh == 1 || t == n_steps - 1) tc_commit(&v_empty[s]);
        tc_commit(&pv_done[hh]);
        stamp(t, 9);
        // S(t+2) overwrites the columns P(t) lives in: it is queued behind PV(t) and executes after it
        if (t + 2 < n_steps && !issue_qk(t + 2)) break;
        stamp(t, 10);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0-3)
    const int row = threadIdx.x;  // query row inside the tile == TMEM lane
    const uint32_t lane_bits = (uint32_t)(warp * 32) << 16;
    const uint32_t o_tmem = tmem_base + kColO + lane_bits;
    {
      // this thread's row of Q: global -> registers -> TMEM (rows past Nq: zeros, never stored)
      uint32_t qr[D / 2];
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(q_ptr) +
                                                        ((((size_t)b * H + h) * Nq + (size_t)(q0 + row)) * D) * 2);
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const uint4 u = q0 + row < Nq ? src[i] : make_uint4(0u, 0u, 0u, 0u);
        qr[4 * i + 0] = u.x; qr[4 * i + 1] = u.y; qr[4 * i + 2] = u.z; qr[4 * i + 3] = u.w;
      }
      tmem_st_x32(tmem_base + kColQ + lane_bits, qr);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(q_full);
    }
    float m_base = -INFINITY;  // the base O and l are currently expressed in (log2 units)
    float l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < n_steps; ++t) {
      const int hh = t & 1;
      const uint32_t ph = (uint32_t)(t >> 1) & 1u;
      const uint32_t s_tmem = tmem_base + (uint32_t)hh * kStepN + lane_bits;
      // every lane polls: measured faster than one polling lane plus a shuffle
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[hh], ph, ctx, kWaitSFull));
      if (!ok) break;
      if (threadIdx.x == 0) stamp(t, 0);
      tc_fence_after_sync();
      uint32_t v[2][32];   // the 64 scores of this row, loaded once
      tmem_ld_x32(s_tmem, v[0]);
      tmem_ld_x32(s_tmem + 32, v[1]);
      const int k0 = t * kStepN;
      const bool need_mask = (k0 + kStepN > Nk) || (causal && (k0 + kStepN - 1 > q0 + causal_off));
      int limit = Nk - 1;
      if (causal) limit = min(limit, q0 + row + causal_off);
      limit -= k0;  // last visible column of this step for this row
      tmem_wait_ld_regs(v[0]);
      tmem_wait_ld_regs(v[1]);

      const float m_step = (need_mask ? row_max<true>(v, limit) : row_max<false>(v, limit)) * scale_log2;
      if (threadIdx.x == 0) stamp(t, 1);
      // lazy rescale: move the base only when the maximum outgrew it by more than the threshold
      const bool grow = m_step > m_base + kRescaleThreshold || m_base == -INFINITY;
      float alpha = 1.0f;
      if (grow && m_step != -INFINITY) {
        alpha = ex2(m_base - m_step);  // 0 when m_base is still -inf
        m_base = m_step;
      }
      const float base = (m_base == -INFINITY) ? 0.f : m_base;
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        // PV(t-1) may still be accumulating into O; PV(t) cannot have started (it waits for this step's P)
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[hh ^ 1], (uint32_t)((t - 1) >> 1) & 1u, ctx, kWaitPvDone));
        if (!ok) break;
        tc_fence_after_sync();
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
      if (threadIdx.x == 0) stamp(t, 2);
      // p = 2^(x - base), row sum, P written over the first 32 columns of the S buffer just read
      const float step_sum = need_mask ? exp_and_store<true, kBf16>(v, s_tmem, limit, scale_log2, base)
                                       : exp_and_store<false, kBf16>(v, s_tmem, limit, scale_log2, base);
      l_run = fmaf(l_run, alpha, step_sum);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[hh]);
      if (threadIdx.x == 0) stamp(t, 3);
    }
    // PVs complete in issue order: the last one done means all are
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(n_steps - 1) & 1], (uint32_t)((n_steps - 1) >> 1) & 1u, ctx, kWaitPvDone));
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

// ------------------------------------------------------------------------------------------------
// Head dim 128 keeps the earlier, unpipelined flow: one S buffer of 128 keys, QK(j+1) issued behind
// PV(j), the softmax in two passes over S in TMEM.  With D = 128 both products are tensor-bound (QK
// has K = 128, PV has N = 128) and a tcgen05.mma with N = 64 costs ~48 clocks against ~65 for N = 128,
// so halving the key step costs more tensor time than the pipelining wins back (983 vs 1073 TFLOP/s at
// B=1 H=16 N=8192), and S (2 x 128) + O (128) would not fit the 256 TMEM columns of a CTA either.
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
                    int causal, float scale_log2, int serialize, unsigned int* status, unsigned long long* trace) {
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
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // causal: the longest tiles start first
  const int h = blockIdx.y, b = blockIdx.z;
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
  // optional timeline of CTA (0,0,0) for tuning: 16 clock stamps per key tile
  const bool tracing = trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  auto stamp = [&](int j, int k) {
    if (tracing && j < 64) trace[j * 16 + k] = clock64();
  };

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
        stamp(j, 8);
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
        stamp(j, 9);
        if (j + 1 < n_tiles) {
          // S(j+1) overwrites the columns P(j) lives in.  tcgen05.mma instructions of one thread execute in
          // issue order, so PV(j) has read P before QK(j+1) writes; `serialize` (KFB_ATTN_SERIALIZE=1, a
          // debugging aid) waits for PV(j) explicitly instead.
          if (serialize && !mbar_wait(pv_done, (uint32_t)j & 1u, ctx, kWaitPvDone)) break;
          stamp(j, 10);
          if (!issue_qk(j + 1)) break;
          stamp(j, 11);
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
      if (threadIdx.x == 0) stamp(j, 0);
      tc_fence_after_sync();
      // S(j) complete implies PV(j-1) complete (the issuer orders them), so O may be touched here.
      const int k0 = j * kBlockN;
      const bool need_mask = (k0 + kBlockN > Nk) || (causal && (k0 + kBlockN - 1 > q0 + causal_off));
      int limit = Nk - 1;
      if (causal) limit = min(limit, q0 + row + causal_off);
      limit -= k0;  // last visible column of this tile for this row

      // ---- pass 1: row maximum
      const float m_tile = (need_mask ? row_max<true>(s_tmem, limit) : row_max<false>(s_tmem, limit)) * scale_log2;
      if (threadIdx.x == 0) stamp(j, 1);
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
      if (threadIdx.x == 0) stamp(j, 2);
      // ---- pass 2: p = 2^(x - base), row sum, P written over the S columns already consumed
      const uint32_t p_tmem = tmem_base + kSerialColP + lane_bits;
      const float tile_sum = need_mask ? exp_and_store<true, kBf16>(s_tmem, p_tmem, limit, scale_log2, base, &p_ready[0])
                                       : exp_and_store<false, kBf16>(s_tmem, p_tmem, limit, scale_log2, base, &p_ready[0]);
      l_run = fmaf(l_run, alpha, tile_sum);
      tmem_wait_st();
      if (threadIdx.x == 0) stamp(j, 3);
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

unsigned long long* g_trace = nullptr;  // tuning aid, set through kfb_debug_set_attn_trace

template <int D, bool kBf16>
int launch(const Problem& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, unsigned int* status,
           cudaStream_t stream) {
  using L = Layout<D>;
  static bool configured[64] = {false};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if constexpr (D == 64) {
      KFB_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<D, kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
      KFB_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<D, kBf16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
    }
    {
      KFB_CUDA_TRY(cudaFuncSetAttribute(serial::attn_prefill_serial_kernel<D, kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        L::kAlloc));
      KFB_CUDA_TRY(cudaFuncSetAttribute(serial::attn_prefill_serial_kernel<D, kBf16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
    }
    configured[dev] = true;
  }
  const dim3 grid(ceil_div(p.Nq, kBlockM), p.H, p.B);
  const float scale_log2 = p.scale * 1.4426950408889634f;
  static const bool force_serial = [] { const char* e = getenv("KFB_ATTN_SERIAL"); return e && e[0] == '1'; }();
  bool launched = false;
  if constexpr (D == 64) {
    if (!force_serial) {
      attn_prefill_kernel<D, kBf16><<<grid, kThreads, L::kAlloc, stream>>>(p.q, tk, tv, p.o, p.H, p.Hk, p.Nq, p.Nk, p.causal,
                                                                          scale_log2, status, g_trace);
      launched = true;
    }
  }
  if (!launched)
    serial::attn_prefill_serial_kernel<D, kBf16><<<grid, kThreads, L::kAlloc, stream>>>(tq, tk, tv, p.o, p.H, p.Hk, p.Nq, p.Nk,
                                                                                      p.causal, scale_log2, 0, status, g_trace);
  KFB_LAUNCH_CHECK("attn_prefill_kernel");
  return KFB_OK;
}

}  // namespace

int launch_prefill(const Problem& p, cudaStream_t stream) {
  if (p.H > 65535 || p.B > 65535) return fail(KFB_ERR_INVALID, "B and H must each be <= 65535");
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

// Tuning aid (not part of the public header): device buffer of 64 x 16 clock stamps written by CTA (0,0,0).
extern "C" void kfb_debug_set_attn_trace(void* device_buffer) {
  kfb::attn::g_trace = static_cast<unsigned long long*>(device_buffer);
}
