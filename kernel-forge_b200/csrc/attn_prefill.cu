// Fused attention forward for sm_100a, general path (any Nq, Nk; GQA; bottom-right causal mask).
//
// Replaces attn_v4_kernel of the reference (csrc/attention/attn_v4_kernel.cuh:43-214), which is an
// mma.sync / ldmatrix / cp.async kernel.  This one is built on the Blackwell execution model:
//
//   * one CTA per 128 query rows of one (batch, head); 192 threads in three roles:
//       warp 4  (1 thread)  TMA producer: Q once, K and V tiles of 128 keys through mbarrier rings,
//                           128-byte-swizzled shared-memory tiles (a D=64 row is exactly 128 bytes)
//       warp 5  (1 thread)  tcgen05.mma issuer: S = Q K^T (SS form, both operands K-major) into one of
//                           two TMEM buffers, O += P V (TS form: P is read from TMEM, V is the
//                           MN-major shared-memory operand, so V needs no transpose)
//       warps 0-3 (128 thr) softmax: thread r owns query row r = TMEM lane r, so row max / row sum
//                           need no shuffles; base-2 online softmax with FP32 statistics; P is
//                           rounded to the I/O type and written back to TMEM; O is rescaled in TMEM
//                           only when some row maximum of the warp moved; epilogue O / l -> global
//   * S(j+1) = Q K^T is issued before the softmax of tile j finishes (S is double-buffered), so
//     the tensor pipe works under the softmax;
//   * causal: tiles above the diagonal are never loaded or multiplied (loop bound), masking only
//     on the diagonal / ragged tiles; query tiles are scheduled heaviest-first;
//   * GQA: kv head = h / (H / Hk); TMA zero-fills rows past Nq / Nk, those keys are masked.
//
// TMEM columns (512 allocated, 1 CTA per SM): S0 [0,128) S1 [128,256) P0 [256,320) P1 [320,384)
// O [384, 384 + D).
//
// Numerics (as the reference, attn_v4_kernel.cuh:133-213): scores accumulate in FP32; x = s *
// (scale * log2 e); masked = -inf; base = max(m_old, rowmax) (0 when still -inf); p = 2^(x - base);
// the row sum adds the unrounded p, the PV product uses p rounded to fp16/bf16; O / l rounded once.
// 2^x is ex2.approx.ftz.f32.
#include "attn.cuh"
#include "sm100.cuh"

namespace kfb {
namespace attn {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kThreads = 192;
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColP = 256, kColO = 384;
constexpr int kHalfBytes = kBlockN * 128;  // one 64-column half of a tile: 128 rows x 128 bytes

enum WaitCode : uint32_t {
  kWaitQ = 0x101, kWaitKEmpty, kWaitKFull, kWaitVEmpty, kWaitVFull, kWaitSFull, kWaitPReady, kWaitPvDone
};

template <int D>
struct Layout {
  static constexpr int kStages = D == 64 ? 4 : 2;
  static constexpr int kTile = kBlockN * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kBars = kV + kStages * kTile;
  static constexpr int kNumBars = 4 * kStages + 6;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kBytes = kMisc + 16;
  static constexpr int kAlloc = kBytes + 1024;  // room to align the tiles to 1024 bytes
  static_assert(2 * kAlloc > 227 * 1024, "a second CTA on the SM would block in tcgen05.alloc");
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

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, void* __restrict__ o_ptr, int H, int Hk, int Nq, int Nk,
                    int causal, float scale_log2, unsigned int* status) {
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
  uint64_t* p_ready = s_full + 2;
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
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
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
        const uint32_t d_tmem = tmem_base + kColS + (uint32_t)(j & 1) * 128u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk / 4) * kHalfBytes + (uint32_t)(kk % 4) * 32u;
          mma_ss(d_tmem, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk,
                 kk > 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[s]);
        tc_commit(&s_full[j & 1]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, ctx, kWaitQ);
      ok = ok && issue_qk(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles && !issue_qk(j + 1)) break;
        if (!mbar_wait(&p_ready[j & 1], (uint32_t)(j >> 1) & 1u, ctx, kWaitPReady)) break;
        const int s = j % S;
        if (!mbar_wait(&v_full[s], (uint32_t)(j / S) & 1u, ctx, kWaitVFull)) break;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + L::kV + s * L::kTile);
        const uint32_t p_tmem = tmem_base + kColP + (uint32_t)(j & 1) * 64u;
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          // 16 keys per step: 16 rows of 128 bytes; the second 64-column block of V is kHalfBytes away
          mma_ts(tmem_base + kColO, p_tmem + (uint32_t)kk * 8u, smem_desc_sw128(v_addr + kk * 2048, kHalfBytes, 1024),
                 idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&v_empty[s]);
        tc_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0-3)
    const int row = threadIdx.x;  // query row inside the tile == TMEM lane
    const uint32_t lane_bits = (uint32_t)(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[buf], (uint32_t)(j >> 1) & 1u, ctx, kWaitSFull));
      if (!ok) break;
      tc_fence_after_sync();
      float s[kBlockN];
      const uint32_t s_tmem = tmem_base + kColS + (uint32_t)buf * 128u + lane_bits;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_wait_ld();

      const int k0 = j * kBlockN;
      const bool need_mask = (k0 + kBlockN > Nk) || (causal && (k0 + kBlockN - 1 > q0 + causal_off));
      if (need_mask) {
        int limit = Nk - 1;
        if (causal) limit = min(limit, q0 + row + causal_off);
#pragma unroll
        for (int i = 0; i < kBlockN; ++i)
          if (k0 + i > limit) s[i] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int i = 1; i < kBlockN; ++i) mx = fmaxf(mx, s[i]);
      const float m_new = fmaxf(m_run, mx * scale_log2);
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = ex2(m_run - base);
      float sum = 0.f;
      uint32_t p16[kBlockN / 2];
#pragma unroll
      for (int i = 0; i < kBlockN / 2; ++i) {
        const float p0 = ex2(fmaf(s[2 * i], scale_log2, -base));
        const float p1 = ex2(fmaf(s[2 * i + 1], scale_log2, -base));
        sum += p0 + p1;
        p16[i] = pack2<kBf16>(p0, p1);
      }
      l_run = fmaf(l_run, alpha, sum);
      m_run = m_new;

      if (j > 0) {
        // O holds tiles 0..j-1 once PV(j-1) has completed; P[buf] was last read by PV(j-2)
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)(j - 1) & 1u, ctx, kWaitPvDone));
        if (!ok) break;
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_x32(tmem_base + kColO + lane_bits + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tmem_base + kColO + lane_bits + c * 32, o);
          }
        }
      }
      const uint32_t p_tmem = tmem_base + kColP + (uint32_t)buf * 64u + lane_bits;
      tmem_st_x32(p_tmem, *reinterpret_cast<uint32_t(*)[32]>(&p16[0]));
      tmem_st_x32(p_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&p16[32]));
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[buf]);
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
        tmem_ld_x32(tmem_base + kColO + lane_bits + c * 32, o);
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

template <int D, bool kBf16>
int launch(const Problem& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, unsigned int* status,
           cudaStream_t stream) {
  using L = Layout<D>;
  auto kernel = attn_prefill_kernel<D, kBf16>;
  static bool configured[64] = {false};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
    configured[dev] = true;
  }
  const dim3 grid(ceil_div(p.Nq, kBlockM), p.H, p.B);
  const float scale_log2 = p.scale * 1.4426950408889634f;
  kernel<<<grid, kThreads, L::kAlloc, stream>>>(tq, tk, tv, p.o, p.H, p.Hk, p.Nq, p.Nk, p.causal, scale_log2, status);
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
