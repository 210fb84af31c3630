// One greedy decode step of a Llama-architecture model (INT4 decoder linears, fp16 lm_head) as ONE persistent kernel,
// for batch 1 and 2 on one GPU.  The reference builds a step from ~50 kernels per layer replayed as a CUDA graph
// (bench/e2e_model.py:97-141); the step of separate kernels of this library is 7 per layer.  At this size every one
// of those kernels is latency-bound (a 5 MB weight matrix is 1 us of HBM time but 4 us as a dependent launch), so the
// step below keeps one CTA per SM resident for the whole step and separates the two things a launch boundary ties
// together:
//   * WEIGHTS do not depend on activations.  Every CTA owns a fixed slice of the rows of every matrix; a producer
//     thread walks the static schedule (per layer: qkv, o, gate_up, down; then lm_head) and streams the CTA's slices
//     with bulk asynchronous copies (cp.async.bulk, completion on an mbarrier) into a ring of shared-memory slots, as
//     far ahead as the ring allows (148 CTAs x 176 KB: more than one whole layer).  HBM streams continuously while the
//     consumers wait for activations.
//   * ACTIVATIONS are exchanged through global memory (L2) between stages separated by a grid-wide barrier: an atomic
//     counter, one arrival per CTA, bounded wait.  Five barriers per layer: qkv (+ RoPE, KV-cache write) | attention
//     (split over the keys; the last CTA of a KV head merges the partials) | o_proj (+ residual) | gate_up (RMSNorm
//     prologue, SiLU pair epilogue) | down_proj (+ residual).  RMSNorm is recomputed by every CTA in the prologue of
//     the stage that consumes it (4 KB from L2), so it needs no stage of its own.
// The weight rows are in the private orders of the pair epilogues (int4_gemv.cu: gate_p / up_p interleaved; q and k
// features (j, j + D/2) adjacent): rows are quantised independently, so this is exact, and a CTA's slice of rows is
// contiguous in the public packed format, which is what lets one bulk copy fetch it.
//
// Arithmetic: the same as the separate kernels (exact fp16 x int4 products accumulated in FP32 per 32-weight chunk,
// FP32 group scale, one rounding to fp16, fp16 residual adds, rotate-half RoPE with separately rounded products);
// only summation orders differ.  Attention keeps P in FP32 (the separate decode kernel rounds it to fp16 for its MMA).
//
// Every wait is bounded: ring barriers through sm100::mbar_wait, the grid barrier by %globaltimer.  On expiry the CTA
// records a code (0x901 grid barrier, 0x902 weight ring) in the device status word, poisons the barrier flags so
// that every other CTA leaves its wait at once, waits (bounded) for its own copies in flight, and returns.  The launch
// is cooperative, so all CTAs are co-resident by construction.  Nothing is ever read from or written to another GPU.
#include "common.cuh"
#include "sm100.cuh"

namespace kfb {
namespace persist {

using namespace sm100;

constexpr int kConsumerWarps = 15;
constexpr int kConsumers = kConsumerWarps * 32;      // 480
constexpr int kThreads = kConsumers + 32;            // + the producer warp = 512: 128 registers per thread
constexpr int kSlots = 4;
constexpr int kSlotBytes = 45056;                    // 44 KB: 42 rows of K = 2048, 14 of K = 5632, 11 fp16 rows of 2048
constexpr int kMaxK = 8192;                          // activations of a stage: 2 rows x kMaxK halfs
constexpr int kXsBytes = 2 * kMaxK * 2;
constexpr int kMiscBytes = 4096;
constexpr int kSmemBytes = kSlots * kSlotBytes + kXsBytes + kMiscBytes;
constexpr int kMaxSplits = 32;
constexpr int kMaxOwnRows = 128;                     // rows of the residual stream one CTA may own
constexpr unsigned int kStatusGridBarrier = 0x901, kStatusWeightRing = 0x902, kStatusRopePosition = 0x701;
constexpr unsigned long long kPoison = 1ull << 40;   // added to the barrier counter by a CTA that gives up

struct LayerPtrs {          // one per decoder layer, in device memory (12 pointers)
  const char* qkv_w;  const char* qkv_s;    // packed int32 [ (H + 2 Hk) D, K/8 ], fp16 scales [.., K/G]; rows in RoPE-pair order
  const char* o_w;    const char* o_s;      // [hidden, H D]
  const char* gu_w;   const char* gu_s;     // [2 inter, hidden]; rows gate_p, up_p interleaved
  const char* down_w; const char* down_s;   // [hidden, inter]
  const __half* in_norm; const __half* post_norm;
  __half* k_cache; __half* v_cache;         // [B, Hk, Lmax, D]
};

struct Params {
  const LayerPtrs* layers;
  int L, B, hidden, H, Hk, D, inter, vocab, Lmax, group, splits;
  float eps, scale_log2;
  const __half* embed; const __half* final_norm; const char* lm_head;
  const float* cos_t; const float* sin_t;
  const long long* tok; const long long* pos; const int* kv_len;
  __half* x; __half* q; __half* attn; __half* act; float* part; unsigned int* head_cnt;
  unsigned long long* bar; unsigned long long* flags; __half* logits; unsigned long long* best; unsigned int* status;
  unsigned long long timeout_ns;
};

// ---------------------------------------------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------------------------------------------
// L2-only loads (ld.global.cg) for data other CTAs wrote during this launch: L1 is not coherent across SMs.  Not
// volatile, so the compiler may batch independent loads; every barrier / fence in this file is a compiler memory barrier.
__device__ __forceinline__ uint4 ld_cg(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float ld_cg_f32(const float* p) { return __ldcg(p); }
__device__ __forceinline__ __half ld_cg_h(const __half* p) {
  return __ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.  Both addresses 16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ float dot2_mixed(uint32_t a, unsigned short bl, unsigned short bh, float acc) {
  asm("{\n\t"
      ".reg .b16 al, ah;\n\t"
      "mov.b32 {al, ah}, %1;\n\t"
      "fma.rn.f32.f16 %0, al, %2, %0;\n\t"
      "fma.rn.f32.f16 %0, ah, %3, %0;\n\t"
      "}"
      : "+f"(acc)
      : "r"(a), "h"(bl), "h"(bh));
  return acc;
}

// 32 activations split into 16-bit registers, with the two class sums that remove the offsets of the masked nibble
// forms (1024 + u on nibble pairs 0 and 2 of a word, 1024 + 16 u on pairs 1 and 3).
struct XChunk {
  unsigned short lo[16], hi[16];
  float sxa, sxb;
};
__device__ __forceinline__ void split_x(const uint4 (&xv)[4], XChunk& xc) {
  const uint32_t* xs = reinterpret_cast<const uint32_t*>(xv);
#pragma unroll
  for (int i = 0; i < 16; ++i) asm("mov.b32 {%0, %1}, %2;" : "=h"(xc.lo[i]), "=h"(xc.hi[i]) : "r"(xs[i]));
  float a = 0.f, b = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    a = dot2_mixed(0x3C003C00u, xc.lo[i], xc.hi[i], a);
    b = dot2_mixed(0x3C003C00u, xc.lo[i + 1], xc.hi[i + 1], b);
  }
  xc.sxa = a * -1032.0f;
  xc.sxb = b * -72.0f;
}
// sum over the 32 weights of one 16-byte chunk of q * x (q the signed nibble), exact products, FP32 sums
__device__ __forceinline__ float dot_chunk(const uint4& wv, const XChunk& xc) {
  constexpr uint32_t kMagic = 0x64006400u;
  const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
  float pa = 0.f, pb = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t w = wr[j], h = w >> 8;
    pa = dot2_mixed((w & 0x000F000Fu) | kMagic, xc.lo[4 * j + 0], xc.hi[4 * j + 0], pa);
    pb = dot2_mixed((w & 0x00F000F0u) | kMagic, xc.lo[4 * j + 1], xc.hi[4 * j + 1], pb);
    pa = dot2_mixed((h & 0x000F000Fu) | kMagic, xc.lo[4 * j + 2], xc.hi[4 * j + 2], pa);
    pb = dot2_mixed((h & 0x00F000F0u) | kMagic, xc.lo[4 * j + 3], xc.hi[4 * j + 3], pb);
  }
  return (pa + xc.sxa) + fmaf(pb, 0.0625f, xc.sxb);
}

__device__ __forceinline__ uint32_t ordered_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ---------------------------------------------------------------------------------------------------------------
// the static schedule: which rows of a matrix a CTA owns, and how they are cut into ring slots
// ---------------------------------------------------------------------------------------------------------------
struct Slice {
  int r0, rows, rows_per_chunk;
};
// `unit`: rows are dealt out in units (2 for the pair epilogues; more where the scale rows need it for 16-byte alignment)
__host__ __device__ inline Slice slice_of(int n_rows, int unit, int row_bytes, int cta, int n_ctas) {
  const int units = n_rows / unit;
  const int base = units / n_ctas, rem = units % n_ctas;
  Slice s;
  s.r0 = unit * (cta * base + (cta < rem ? cta : rem));
  s.rows = unit * (base + (cta < rem ? 1 : 0));
  int rpc = (kSlotBytes / row_bytes) / unit * unit;
  s.rows_per_chunk = rpc < unit ? unit : rpc;
  return s;
}
__host__ __device__ inline int int4_unit(int K, int group) {   // smallest even unit whose scale rows are a multiple of 16 bytes
  int u = 2;
  while ((u * (K / group) * 2) % 16) u *= 2;
  return u;
}

#ifdef KFB_TRACE
// Tuning aid of -DKFB_TRACE builds: thread 0 of CTA 0 writes %globaltimer stamps [layer < 8][16] into a buffer set
// through kfb_debug_set_step_trace.
__device__ unsigned long long* g_step_trace = nullptr;
__device__ int g_step_trace_cta = 0;
#define KFB_STEP_STAMP(layer, k)                                                                              \
  do {                                                                                                        \
    if (blockIdx.x == g_step_trace_cta && threadIdx.x == 0 && g_step_trace != nullptr && (layer) < 8) g_step_trace[(layer) * 16 + (k)] = globaltimer_ns(); \
  } while (0)
#else
#define KFB_STEP_STAMP(layer, k) \
  do {                           \
  } while (0)
#endif

struct Shared {
  uint64_t full[kSlots], empty[kSlots];
  volatile uint32_t abort_word;
  volatile uint32_t issued, consumed;     // ring chunks issued by the producer / released by the consumers
  uint32_t flag;
  uint32_t go;        // the CTA-wide decision of the last grid barrier
  __half2 x_own[2][kMaxOwnRows / 2];   // the CTA's own rows of the residual stream
  float red[2][kConsumerWarps];
  float ml[kConsumerWarps][8][2];
  unsigned long long best[kConsumerWarps][2];
};
static_assert(sizeof(Shared) <= kMiscBytes, "misc region too small");

struct Ctx {
  const Params& p;
  char* ring;
  uint4* xs;          // stage activations (or attention scratch)
  Shared* sh;
  AbortCtx abort;
  int cta, n_ctas, warp, lane, tid;
  uint32_t it;        // ring chunk counter (same sequence in producer and consumers)
  unsigned long long barriers;   // grid barriers passed
};

// Grid-wide barrier of the consumer threads.  Returns false when the step was given up (here or in another CTA).
// Arrivals are counted on one word; the last CTA to arrive (it sees the count complete in the value its atomic returns)
// writes the barrier's generation number into one flag per CTA, each on a cache line of its own, and every CTA polls
// only its own flag.  (With all CTAs polling the counter itself, the L2 slice that holds it is saturated by the polls
// and every other line of that slice -- here part of the residual stream -- takes microseconds to read.)
__device__ __forceinline__ void st_release_gpu(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_gpu(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
constexpr int kFlagStride = 16;   // in 8-byte words: one 128-byte line per CTA

// Every consumer thread calls this after every stage, whether its own warp completed the stage or gave it up: the
// decision to go on is taken ONCE per CTA (lane 0 of warp 0, between the two CTA barriers) and read by all, so the
// consumer threads always agree on the sequence of named barriers they execute.
__device__ bool grid_barrier(Ctx& c) {
  consumer_sync();
  if (c.warp == 0) {
    const unsigned long long gen = ++c.barriers;   // every lane of warp 0 keeps the count
#ifdef KFB_TRACE
    if (c.lane == 0 && g_step_trace != nullptr && gen <= 64) g_step_trace[128 + c.cta * 64 + (gen - 1)] = globaltimer_ns();
#endif
    if (c.sh->abort_word == 0) {
      unsigned long long old = 0;
      if (c.lane == 0) {
        __threadfence();
        old = atomicAdd(c.p.bar, 1ull);
      }
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old + 1 == gen * (unsigned long long)c.n_ctas) {   // the last arrival releases every CTA
        __threadfence();   // one fence, then plain (relaxed) flag stores: a release per store would serialise them
        for (int i = c.lane; i < c.n_ctas; i += 32) st_relaxed_gpu(c.p.flags + (size_t)i * kFlagStride, gen);
      }
      if (c.lane == 0) {
        const unsigned long long* mine = c.p.flags + (size_t)c.cta * kFlagStride;
        unsigned long long v = ld_acquire_gpu(mine);
        if (v < gen) {
          const unsigned long long t0 = globaltimer_ns();
          uint32_t spins = 0;
          while ((v = ld_acquire_gpu(mine)) < gen) {
            if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > c.p.timeout_ns) {
              atomicCAS(c.p.status, 0u, kStatusGridBarrier);
              c.sh->abort_word = kStatusGridBarrier;
              break;
            }
          }
        }
        if (v >= kPoison && c.sh->abort_word == 0) c.sh->abort_word = kStatusGridBarrier;
      }
    }
#ifdef KFB_TRACE
    if (c.lane == 0 && g_step_trace != nullptr && gen <= 64) g_step_trace[128 + 160 * 64 + c.cta * 64 + (gen - 1)] = globaltimer_ns();
#endif
    if (c.lane == 0) c.sh->go = c.sh->abort_word == 0 ? 1u : 0u;
  }
  consumer_sync();
  return c.sh->go != 0u;
}

// Warp-uniform: either every lane of the warp sees the slot filled or the whole warp gives the stage up (the shuffles and
// warp barriers of a stage need all 32 lanes).
__device__ __forceinline__ bool wait_full(Ctx& c) {
  const uint32_t slot = c.it % kSlots, parity = (c.it / kSlots) & 1u;
  return mbar_wait_warp(&c.sh->full[slot], parity, c.abort, kStatusWeightRing);
}
__device__ __forceinline__ void release_slot(Ctx& c) {   // every consumer warp, after its last read of the slot
  __syncwarp();
  if (c.lane == 0) mbar_arrive(&c.sh->empty[c.it % kSlots]);
  if (c.tid == 0) c.sh->consumed = c.it + 1;
}

// ---------------------------------------------------------------------------------------------------------------
// producer: walks the schedule and keeps the ring full
// ---------------------------------------------------------------------------------------------------------------
__device__ bool produce(Ctx& c, const char* w, const char* s, int n_rows, int unit, int row_w, int row_s) {
  const Slice sl = slice_of(n_rows, unit, row_w + row_s, c.cta, c.n_ctas);
  for (int c0 = 0; c0 < sl.rows; c0 += sl.rows_per_chunk) {
    const int n = min(sl.rows_per_chunk, sl.rows - c0);
    const uint32_t slot = c.it % kSlots, parity = (c.it / kSlots) & 1u;
    if (!mbar_wait(&c.sh->empty[slot], parity ^ 1u, c.abort, kStatusWeightRing)) return false;
    char* dst = c.ring + (size_t)slot * kSlotBytes;
    const uint32_t wb = (uint32_t)n * row_w, sb = (uint32_t)n * row_s;
    mbar_arrive_expect_tx(&c.sh->full[slot], wb + sb);
    bulk_load(dst, w + (size_t)(sl.r0 + c0) * row_w, wb, &c.sh->full[slot]);
    if (sb) bulk_load(dst + wb, s + (size_t)(sl.r0 + c0) * row_s, sb, &c.sh->full[slot]);
    ++c.it;
    c.sh->issued = c.it;
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------------
// consumers: activations of a stage into shared memory
// ---------------------------------------------------------------------------------------------------------------
// Position of 16-byte vector v (8 halfs) of an activation row.  INT4 stages read a whole 32-activation chunk (4
// vectors) per lane and lanes walk consecutive chunks, so the 4 vectors of a chunk are stored KC apart (conflict-free);
// the fp16 lm_head stage reads consecutive vectors and keeps the natural order.
__device__ __forceinline__ int xs_index(int v, int KC, bool chunked) { return chunked ? (v & 3) * KC + (v >> 2) : v; }

// xs[m] = src row m (as given, or RMS-normalised and scaled by norm_w like kfb_add_rmsnorm).  All consumer threads.
template <int M>
__device__ void stage_x(Ctx& c, const __half* const (&src)[M], int K, const __half* norm_w, bool chunked) {
  const int nvec = K / 8, KC = K / 32;
  constexpr int kMaxVec = (kMaxK / 8 + kConsumers - 1) / kConsumers;   // 3
  uint4 keep[M][kMaxVec], wv[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {   // every load of the stage is issued before the first use: one round trip
    const int v = c.tid + i * kConsumers;
    if (v < nvec) {
#pragma unroll
      for (int m = 0; m < M; ++m) keep[m][i] = ld_cg(reinterpret_cast<const uint4*>(src[m]) + v);
      if (norm_w) wv[i] = reinterpret_cast<const uint4*>(norm_w)[v];
    }
  }
  if (norm_w) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int v = c.tid + i * kConsumers;
        if (v < nvec) {
          const __half2* h = reinterpret_cast<const __half2*>(&keep[m][i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
          }
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      if (c.lane == 0) c.sh->red[m][c.warp] = ss;
    }
    consumer_sync();
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float inv = 0.f;
    if (norm_w) {
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < kConsumerWarps; ++i) tot += c.sh->red[m][i];
      inv = rsqrtf(tot / (float)K + c.p.eps);
    }
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int v = c.tid + i * kConsumers;
      if (v < nvec) {
        uint4 o = keep[m][i];
        if (norm_w) {
          const __half2* wh = reinterpret_cast<const __half2*>(&wv[i]);
          const __half2* h = reinterpret_cast<const __half2*>(&keep[m][i]);
          __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            oh[j] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[j]);
          }
        }
        c.xs[(size_t)m * nvec + xs_index(v, KC, chunked)] = o;
      }
    }
  }
  consumer_sync();
}

// Brings constants a later stage reads right after a barrier (norm weights) into L2 ahead of time.
__device__ __forceinline__ void prefetch_l2(const void* p, int bytes, int tid) {
  for (int off = tid * 128; off < bytes; off += kConsumers * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char*>(p) + off));
}

// ---------------------------------------------------------------------------------------------------------------
// INT4 GEMV stage over the CTA's row slice; rows come in pairs (2p, 2p + 1) handled by one warp
// ---------------------------------------------------------------------------------------------------------------
enum Epi : int { kEpiResidual = 0, kEpiSiluPair = 1, kEpiRopeKv = 2 };

struct EpiArgs {
  const LayerPtrs* lp;    // kEpiRopeKv
  long long pos;
};

// `local_n`: n minus the first row of the CTA's slice.
template <int EPI>
__device__ __forceinline__ void store_pair(const Ctx& c, const EpiArgs& e, float a0, float a1, int m, int n, int N, int local_n) {
  const Params& p = c.p;
  if constexpr (EPI == kEpiResidual) {
    // The rows of the residual stream this CTA owns (o_proj and down_proj deal the hidden rows out identically) live in
    // shared memory for the whole step: the add reads no global memory, and the new value goes out as one 4-byte store.
    // (Reading x back through L2 while the neighbouring CTAs store into the same 32-byte sectors cost microseconds.)
    __half2* own = &c.sh->x_own[m][local_n >> 1];
    const __half2 v = __hadd2(__floats2half2_rn(a0, a1), *own);
    *own = v;
    *reinterpret_cast<__half2*>(p.x + (size_t)m * N + n) = v;
    return;
  }
  const float g = __half2float(__float2half_rn(a0)), u = __half2float(__float2half_rn(a1));
  if constexpr (EPI == kEpiSiluPair) {
    p.act[(size_t)m * (N / 2) + (n >> 1)] = __hmul(__float2half_rn(g / (1.0f + __expf(-g))), __float2half_rn(u));
    return;
  }
  if constexpr (EPI == kEpiRopeKv) {
    const int half = p.D / 2, pr = n >> 1;
    const int q_pairs = p.H * half, k_pairs = p.Hk * half;
    const long long pos = e.pos;
    if (pr < q_pairs + k_pairs) {
      const int head = pr < q_pairs ? pr / half : (pr - q_pairs) / half;
      const int j = pr < q_pairs ? pr % half : (pr - q_pairs) % half;
      const float c0 = p.cos_t[pos * p.D + j], s0 = p.sin_t[pos * p.D + j];
      const float c1 = p.cos_t[pos * p.D + j + half], s1 = p.sin_t[pos * p.D + j + half];
      const __half rlo = __float2half_rn(__fsub_rn(__fmul_rn(g, c0), __fmul_rn(u, s0)));
      const __half rhi = __float2half_rn(__fadd_rn(__fmul_rn(u, c1), __fmul_rn(g, s1)));
      __half* dst = pr < q_pairs ? p.q + ((size_t)m * p.H + head) * p.D
                                 : e.lp->k_cache + (((size_t)m * p.Hk + head) * p.Lmax + pos) * p.D;
      dst[j] = rlo;
      dst[j + half] = rhi;
    } else {
      const int pv = pr - q_pairs - k_pairs, head = pv / half, j = pv % half;
      __half* dst = e.lp->v_cache + (((size_t)m * p.Hk + head) * p.Lmax + pos) * p.D;
      *reinterpret_cast<__half2*>(dst + 2 * j) = __floats2half2_rn(a0, a1);
    }
  }
}

template <int M, int EPI>
__device__ bool int4_stage(Ctx& c, int n_rows, int K, int unit, const EpiArgs& e) {
  const int G = c.p.group;
  const int KC = K / 32, SG = K / G, kcpg = G / 32;
  const int row_w = K / 2, row_s = SG * 2;
  const int nvec = K / 8;
  const Slice sl = slice_of(n_rows, unit, row_w + row_s, c.cta, c.n_ctas);
  for (int c0 = 0; c0 < sl.rows; c0 += sl.rows_per_chunk) {
    const int n = min(sl.rows_per_chunk, sl.rows - c0);
    if (!wait_full(c)) return false;
    const char* slot = c.ring + (size_t)(c.it % kSlots) * kSlotBytes;
    const uint4* wbase = reinterpret_cast<const uint4*>(slot);
    const __half* sbase = reinterpret_cast<const __half*>(slot + (size_t)n * row_w);
    for (int pr = c.warp; pr < n / 2; pr += kConsumerWarps) {
      const uint4* w0 = wbase + (size_t)(2 * pr) * KC;
      const uint4* w1 = w0 + KC;
      const __half* s0 = sbase + (size_t)(2 * pr) * SG;
      const __half* s1 = s0 + SG;
      float acc[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m) acc[m][0] = acc[m][1] = 0.f;
      for (int ch = c.lane; ch < KC; ch += 32) {
        const uint4 wa = w0[ch], wb = w1[ch];
        const float sa = __half2float(s0[ch / kcpg]), sb = __half2float(s1[ch / kcpg]);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          uint4 xv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) xv[j] = c.xs[(size_t)m * nvec + j * KC + ch];
          XChunk xc;
          split_x(xv, xc);
          acc[m][0] = fmaf(sa, dot_chunk(wa, xc), acc[m][0]);
          acc[m][1] = fmaf(sb, dot_chunk(wb, xc), acc[m][1]);
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          acc[m][0] += __shfl_xor_sync(0xffffffffu, acc[m][0], off);
          acc[m][1] += __shfl_xor_sync(0xffffffffu, acc[m][1], off);
        }
      if (c.lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) store_pair<EPI>(c, e, acc[m][0], acc[m][1], m, sl.r0 + c0 + 2 * pr, n_rows, c0 + 2 * pr);
      }
    }
    release_slot(c);

    ++c.it;
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------------
// fp16 lm_head stage with fused argmax
// ---------------------------------------------------------------------------------------------------------------
template <int M>
__device__ bool lm_head_stage(Ctx& c) {
  const Params& p = c.p;
  const int K = p.hidden, nvec = K / 8, row_w = K * 2;
  const Slice sl = slice_of(p.vocab, 1, row_w, c.cta, c.n_ctas);
  unsigned long long best[M];
#pragma unroll
  for (int m = 0; m < M; ++m) best[m] = 0ull;
  for (int c0 = 0; c0 < sl.rows; c0 += sl.rows_per_chunk) {
    const int n = min(sl.rows_per_chunk, sl.rows - c0);
    if (!wait_full(c)) break;   // (the CTA barrier below is still executed by every warp)
    const uint4* wbase = reinterpret_cast<const uint4*>(c.ring + (size_t)(c.it % kSlots) * kSlotBytes);
    for (int r = c.warp; r < n; r += kConsumerWarps) {
      const uint4* wr = wbase + (size_t)r * nvec;
      float acc[M];
#pragma unroll
      for (int m = 0; m < M; ++m) acc[m] = 0.f;
      for (int v = c.lane; v < nvec; v += 32) {
        const uint4 wv = wr[v];
        const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 xv = c.xs[(size_t)m * nvec + v];
          const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int j = 0; j < 4; j += 2) {
            unsigned short l0, h0, l1, h1;
            asm("mov.b32 {%0, %1}, %2;" : "=h"(l0), "=h"(h0) : "r"(xw[j]));
            asm("mov.b32 {%0, %1}, %2;" : "=h"(l1), "=h"(h1) : "r"(xw[j + 1]));
            a0 = dot2_mixed(ww[j], l0, h0, a0);
            a1 = dot2_mixed(ww[j + 1], l1, h1, a1);
          }
          acc[m] += a0 + a1;
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v = acc[m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (c.lane == 0) {
          const int row = sl.r0 + c0 + r;
          const __half hv = __float2half_rn(v);
          p.logits[(size_t)m * p.vocab + row] = hv;
          const unsigned long long key =
              ((unsigned long long)ordered_bits(__half2float(hv)) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)row);
          best[m] = key > best[m] ? key : best[m];
        }
      }
    }
    release_slot(c);
    ++c.it;
  }
  if (c.lane == 0) {
#pragma unroll
    for (int m = 0; m < M; ++m) c.sh->best[c.warp][m] = best[m];
  }
  consumer_sync();
  if (c.tid < M) {
    unsigned long long k = 0ull;
    for (int w = 0; w < kConsumerWarps; ++w) k = c.sh->best[w][c.tid] > k ? c.sh->best[w][c.tid] : k;
    if (k) atomicMax(p.best + c.tid, k);
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------------
// attention of the one new query position over the cache (head dim 64), split over the keys
// ---------------------------------------------------------------------------------------------------------------
// Work item = (batch row, KV head, block of 8 query heads, key split).  Lane = 4 g + part: query head g of the block,
// dims [16 part, 16 part + 16).  A warp walks keys k0 + warp, k0 + warp + 15, ... with an online softmax in registers;
// the warps are merged through shared memory, the splits through global memory by the last CTA to finish a head.
// The cache rows of earlier positions do not depend on this step: they are prefetched into L2 BEFORE the grid barrier
// that publishes q (attn_prefetch), so their HBM round trip overlaps the barrier.
constexpr int kPartFloats = 64 + 2;   // o[64], m, l per (item, query head)

struct AttnItem {
  int b, kvh, qb, hb, s, k0, k1, g_cnt;
};
__device__ __forceinline__ AttnItem attn_item(const Params& p, int item) {
  const int Gq = p.H / p.Hk, QB = (Gq + 7) / 8, S = p.splits;
  AttnItem it;
  it.s = item % S;
  it.hb = item / S;                                   // (b * Hk + kvh) * QB + qb
  it.qb = it.hb % QB;
  const int bk = it.hb / QB;
  it.kvh = bk % p.Hk;
  it.b = bk / p.Hk;
  it.g_cnt = min(8, Gq - it.qb * 8);
  int len = p.kv_len[it.b];
  len = len < 0 ? 0 : (len > p.Lmax ? p.Lmax : len);
  const int per = (len + S - 1) / S;
  it.k0 = it.s * per;
  it.k1 = min(len, it.k0 + per);
  return it;
}

// Before the grid barrier that publishes q: the cache rows this CTA's item will read (all but the row this step writes)
// are asked into L2, so that after the barrier they cost an L2 round trip instead of an HBM one.  One 128-byte row per
// thread and cache.
__device__ __forceinline__ void attn_prefetch(const Ctx& c, const LayerPtrs& lp) {
  const Params& p = c.p;
  const int n_items = p.B * p.Hk * ((p.H / p.Hk + 7) / 8) * p.splits;
  if (c.cta >= n_items) return;
  const AttnItem it = attn_item(p, c.cta);
  const size_t base = ((size_t)it.b * p.Hk + it.kvh) * p.Lmax * 64;
  for (int k = it.k0 + c.tid; k < it.k1; k += kConsumers) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(lp.k_cache + base + (size_t)k * 64));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(lp.v_cache + base + (size_t)k * 64));
  }
}

__device__ void attention_stage(Ctx& c, const LayerPtrs& lp) {
  const Params& p = c.p;
  const int Gq = p.H / p.Hk, QB = (Gq + 7) / 8, S = p.splits;
  const int n_items = p.B * p.Hk * QB * S;
  float* o_sm = reinterpret_cast<float*>(c.xs);   // [warp][g][64]
  const int g = c.lane >> 2, part = c.lane & 3;
  for (int item = c.cta; item < n_items; item += c.n_ctas) {
    const AttnItem it = attn_item(p, item);
    const int b = it.b, kvh = it.kvh, qb = it.qb, hb = it.hb, g_cnt = it.g_cnt, k0 = it.k0, k1 = it.k1;
    const int head = kvh * Gq + qb * 8 + g;            // query head of this lane (valid when g < g_cnt)
    float qf[16], o[16];
    float m_run = -INFINITY, l_run = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = 0.f;
    if (g < g_cnt) {
      const __half* qp = p.q + ((size_t)b * p.H + head) * 64 + part * 16;
      const uint4 q0 = ld_cg(qp), q1 = ld_cg(qp + 8);
      const __half2* h0 = reinterpret_cast<const __half2*>(&q0);
      const __half2* h1 = reinterpret_cast<const __half2*>(&q1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(h0[i]), bq = __half22float2(h1[i]);
        qf[2 * i] = a.x * p.scale_log2; qf[2 * i + 1] = a.y * p.scale_log2;
        qf[8 + 2 * i] = bq.x * p.scale_log2; qf[8 + 2 * i + 1] = bq.y * p.scale_log2;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) qf[i] = 0.f;
    }
    const __half* kc = lp.k_cache + ((size_t)b * p.Hk + kvh) * p.Lmax * 64 + part * 16;
    const __half* vc = lp.v_cache + ((size_t)b * p.Hk + kvh) * p.Lmax * 64 + part * 16;
    auto one_key = [&](const uint4& ka, const uint4& kb, const uint4& va, const uint4& vb) {
      const __half2* kh0 = reinterpret_cast<const __half2*>(&ka);
      const __half2* kh1 = reinterpret_cast<const __half2*>(&kb);
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(kh0[i]), bb = __half22float2(kh1[i]);
        sc = fmaf(qf[2 * i], a.x, sc); sc = fmaf(qf[2 * i + 1], a.y, sc);
        sc = fmaf(qf[8 + 2 * i], bb.x, sc); sc = fmaf(qf[8 + 2 * i + 1], bb.y, sc);
      }
      sc += __shfl_xor_sync(0xffffffffu, sc, 1);
      sc += __shfl_xor_sync(0xffffffffu, sc, 2);
      const float m_new = fmaxf(m_run, sc);
      const float corr = exp2f(m_run - m_new), pw = exp2f(sc - m_new);   // m_run = -inf: corr = 0
      l_run = fmaf(l_run, corr, pw);
      m_run = m_new;
      const __half2* vh0 = reinterpret_cast<const __half2*>(&va);
      const __half2* vh1 = reinterpret_cast<const __half2*>(&vb);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(vh0[i]), bb = __half22float2(vh1[i]);
        o[2 * i] = fmaf(o[2 * i], corr, pw * a.x); o[2 * i + 1] = fmaf(o[2 * i + 1], corr, pw * a.y);
        o[8 + 2 * i] = fmaf(o[8 + 2 * i], corr, pw * bb.x); o[8 + 2 * i + 1] = fmaf(o[8 + 2 * i + 1], corr, pw * bb.y);
      }
    };
    // two keys in flight per warp: the loop is bound by the round trip of a key row, not by arithmetic
    for (int k = k0 + c.warp; k < k1; k += 2 * kConsumerWarps) {
      const int k2 = k + kConsumerWarps;
      const bool two = k2 < k1;
      const size_t r1 = (size_t)k * 64, r2 = (size_t)(two ? k2 : k) * 64;
      const uint4 ka = ld_cg(kc + r1), kb = ld_cg(kc + r1 + 8), va = ld_cg(vc + r1), vb = ld_cg(vc + r1 + 8);
      const uint4 ka2 = ld_cg(kc + r2), kb2 = ld_cg(kc + r2 + 8), va2 = ld_cg(vc + r2), vb2 = ld_cg(vc + r2 + 8);
      one_key(ka, kb, va, vb);
      if (two) one_key(ka2, kb2, va2, vb2);
    }
    // warps -> shared memory
    float* od = o_sm + ((size_t)c.warp * 8 + g) * 64 + part * 16;
#pragma unroll
    for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(od + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
    if (part == 0) { c.sh->ml[c.warp][g][0] = m_run; c.sh->ml[c.warp][g][1] = l_run; }
    consumer_sync();
    // merge the warps: thread -> (query head gg, dims d and d + 32)
    const int gg = c.tid >> 5, d = c.tid & 31;
    if (c.tid < 256) {
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) m_all = fmaxf(m_all, c.sh->ml[w][gg][0]);
      float acc0 = 0.f, acc1 = 0.f, l_all = 0.f;
      if (m_all > -INFINITY) {
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          const float f = exp2f(c.sh->ml[w][gg][0] - m_all);
          acc0 = fmaf(f, o_sm[((size_t)w * 8 + gg) * 64 + d], acc0);
          acc1 = fmaf(f, o_sm[((size_t)w * 8 + gg) * 64 + d + 32], acc1);
          l_all = fmaf(f, c.sh->ml[w][gg][1], l_all);
        }
      }
      if (S == 1) {
        if (gg < g_cnt) {
          __half* dst = p.attn + ((size_t)b * p.H + kvh * Gq + qb * 8 + gg) * 64;
          dst[d] = __float2half_rn(l_all > 0.f ? acc0 / l_all : 0.f);
          dst[d + 32] = __float2half_rn(l_all > 0.f ? acc1 / l_all : 0.f);
        }
      } else {
        float* dst = p.part + ((size_t)item * 8 + gg) * kPartFloats;
        dst[d] = acc0;
        dst[d + 32] = acc1;
        if (d == 0) { dst[64] = m_all; dst[65] = l_all; }
      }
    }
    if (S > 1) {
      __threadfence();
      consumer_sync();
      if (c.tid == 0) {
        const unsigned int old = atomicAdd(p.head_cnt + hb, 1u);
        c.sh->flag = (old == (unsigned int)(S - 1)) ? 1u : 0u;
        if (old == (unsigned int)(S - 1)) p.head_cnt[hb] = 0u;   // every split has arrived: ready for the next layer
      }
      consumer_sync();
      if (c.sh->flag && c.tid < 256) {   // last split of this (batch row, KV head, head block): merge in split order
        __threadfence();
        const float* src = p.part + ((size_t)hb * S * 8 + gg) * kPartFloats;   // split i at + i * 8 * kPartFloats
        float m_all = -INFINITY, acc0 = 0.f, acc1 = 0.f, l_all = 0.f;
        constexpr int kBatch = 8;   // loads of a batch are independent and issued together: one L2 round trip per batch
        for (int i0 = 0; i0 < S; i0 += kBatch) {
          float mv[kBatch], lv[kBatch], ov0[kBatch], ov1[kBatch];
#pragma unroll
          for (int i = 0; i < kBatch; ++i) {
            const float* ps = src + (size_t)(i0 + i < S ? i0 + i : i0) * 8 * kPartFloats;
            mv[i] = ld_cg_f32(ps + 64);
            lv[i] = ld_cg_f32(ps + 65);
            ov0[i] = ld_cg_f32(ps + d);
            ov1[i] = ld_cg_f32(ps + d + 32);
          }
          float m_new = m_all;
#pragma unroll
          for (int i = 0; i < kBatch; ++i)
            if (i0 + i < S) m_new = fmaxf(m_new, mv[i]);
          if (m_new > -INFINITY) {
            const float keep = exp2f(m_all - m_new);   // m_all = -inf: 0
            acc0 *= keep; acc1 *= keep; l_all *= keep;
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
              if (i0 + i < S) {
                const float f = exp2f(mv[i] - m_new);
                acc0 = fmaf(f, ov0[i], acc0);
                acc1 = fmaf(f, ov1[i], acc1);
                l_all = fmaf(f, lv[i], l_all);
              }
            m_all = m_new;
          }
        }
        if (gg < g_cnt) {
          __half* dst = p.attn + ((size_t)b * p.H + kvh * Gq + qb * 8 + gg) * 64;
          dst[d] = __float2half_rn(l_all > 0.f ? acc0 / l_all : 0.f);
          dst[d + 32] = __float2half_rn(l_all > 0.f ? acc1 / l_all : 0.f);
        }
      }
    }
    consumer_sync();   // the scratch is reused by the next item / stage
  }
}

// ---------------------------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(128) char smem[];
  Shared* sh = reinterpret_cast<Shared*>(smem + kSlots * kSlotBytes + kXsBytes);
  Ctx c{p, smem, reinterpret_cast<uint4*>(smem + kSlots * kSlotBytes), sh, AbortCtx{&sh->abort_word, p.status, p.timeout_ns},
        (int)blockIdx.x, (int)gridDim.x, (int)(threadIdx.x >> 5), (int)(threadIdx.x & 31), (int)threadIdx.x, 0u, 0ull};

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlots; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], kConsumerWarps); }
    sh->abort_word = 0; sh->issued = 0; sh->consumed = 0;
    // one decision per CTA (and, the inputs being the same, the same one in every CTA; nothing has been written yet):
    // a device whose status word is set runs nothing, a position outside the cache records its code and runs nothing
    const long long pos0 = p.pos[0];
    const bool in_range = pos0 >= 0 && pos0 < p.Lmax;
    if (!in_range && blockIdx.x == 0) atomicCAS(p.status, 0u, kStatusRopePosition);
    sh->flag = (*reinterpret_cast<volatile unsigned int*>(p.status) == 0u && in_range) ? 1u : 0u;
    fence_mbar_init();
  }
  __syncthreads();
  if (sh->flag == 0u) return;
  __syncthreads();   // flag is reused by the attention stage
  const long long pos = p.pos[0];
  const int hd = p.H * p.D, qkv_rows = (p.H + 2 * p.Hk) * p.D;
  const int G = p.group;
  // o_proj and down_proj deal out the same rows (the hidden features) and must do it identically: one unit for both
  const int unit_in = int4_unit(p.hidden, G), unit_hidden = max(int4_unit(hd, G), int4_unit(p.inter, G));

  if (c.warp == kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    if (c.lane == 0) {
      bool ok = true;
      for (int l = 0; l < p.L && ok; ++l) {
        const LayerPtrs lp = p.layers[l];
        ok = produce(c, lp.qkv_w, lp.qkv_s, qkv_rows, unit_in, p.hidden / 2, p.hidden / G * 2) &&
             produce(c, lp.o_w, lp.o_s, p.hidden, unit_hidden, hd / 2, hd / G * 2) &&
             produce(c, lp.gu_w, lp.gu_s, 2 * p.inter, unit_in, p.hidden / 2, p.hidden / G * 2) &&
             produce(c, lp.down_w, lp.down_s, p.hidden, unit_hidden, p.inter / 2, p.inter / G * 2);
      }
      if (ok) produce(c, p.lm_head, nullptr, p.vocab, 1, p.hidden * 2, 0);
    }
  } else {
    // ---------------------------------------------------------------- consumers
    // A warp whose wait on the weight ring fails skips the rest of that stage; every warp still executes every CTA
    // barrier of the layer, and the grid barrier that follows turns the failure into one CTA-wide decision.
    bool ok = true;
    const __half* xin[M];   // the residual stream entering the layer
#pragma unroll
    for (int m = 0; m < M; ++m) {
      long long id = p.tok[m];
      id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
      xin[m] = p.embed + (size_t)id * p.hidden;
    }
    {   // the CTA's own rows of the residual stream start as its rows of the embedding
      const Slice own = slice_of(p.hidden, unit_hidden, 1, c.cta, c.n_ctas);
      if (c.tid < own.rows / 2) {
#pragma unroll
        for (int m = 0; m < M; ++m) sh->x_own[m][c.tid] = *reinterpret_cast<const __half2*>(xin[m] + own.r0 + 2 * c.tid);
      }
      // (made visible to the other warps by the CTA barriers of the first stage)
    }
    for (int l = 0; l < p.L && ok; ++l) {
      const LayerPtrs* lp = p.layers + l;
      EpiArgs e;
      e.lp = lp; e.pos = pos;
      if (c.cta == l % c.n_ctas) {   // one CTA per layer warms L2 with the norm weights the next stages read after a barrier
        prefetch_l2(lp->post_norm, p.hidden * 2, c.tid);
        prefetch_l2(l + 1 < p.L ? p.layers[l + 1].in_norm : p.final_norm, p.hidden * 2, c.tid);
      }
      // qkv: RMSNorm prologue, RoPE + cache write epilogue
      KFB_STEP_STAMP((l < 4 ? l : 99), 0);
      stage_x<M>(c, xin, p.hidden, lp->in_norm, true);
      KFB_STEP_STAMP((l < 4 ? l : 99), 1);
      int4_stage<M, kEpiRopeKv>(c, qkv_rows, p.hidden, unit_in, e);
      KFB_STEP_STAMP((l < 4 ? l : 99), 2);
      attn_prefetch(c, *lp);
      ok = grid_barrier(c);
      KFB_STEP_STAMP((l < 4 ? l : 99), 3);
      if (!ok) break;
      attention_stage(c, *lp);
      KFB_STEP_STAMP((l < 4 ? l : 99), 4);
      if (!(ok = grid_barrier(c))) break;
      KFB_STEP_STAMP((l < 4 ? l : 99), 5);
      // o_proj + residual -> x
      {
        const __half* a[M];
#pragma unroll
        for (int m = 0; m < M; ++m) a[m] = p.attn + (size_t)m * hd;
        stage_x<M>(c, a, hd, nullptr, true);
      }
      KFB_STEP_STAMP((l < 4 ? l : 99), 6);
      int4_stage<M, kEpiResidual>(c, p.hidden, hd, unit_hidden, e);
      KFB_STEP_STAMP((l < 4 ? l : 99), 7);
      ok = grid_barrier(c);
      KFB_STEP_STAMP((l < 4 ? l : 99), 8);
      if (!ok) break;
#pragma unroll
      for (int m = 0; m < M; ++m) xin[m] = p.x + (size_t)m * p.hidden;
      // gate_up: RMSNorm prologue, SiLU pair epilogue -> act
      stage_x<M>(c, xin, p.hidden, lp->post_norm, true);
      KFB_STEP_STAMP((l < 4 ? l : 99), 9);
      int4_stage<M, kEpiSiluPair>(c, 2 * p.inter, p.hidden, unit_in, e);
      KFB_STEP_STAMP((l < 4 ? l : 99), 10);
      ok = grid_barrier(c);
      KFB_STEP_STAMP((l < 4 ? l : 99), 11);
      if (!ok) break;
      // down_proj + residual -> x
      {
        const __half* a[M];
#pragma unroll
        for (int m = 0; m < M; ++m) a[m] = p.act + (size_t)m * p.inter;
        stage_x<M>(c, a, p.inter, nullptr, true);
      }
      KFB_STEP_STAMP((l < 4 ? l : 99), 12);
      int4_stage<M, kEpiResidual>(c, p.hidden, p.inter, unit_hidden, e);
      KFB_STEP_STAMP((l < 4 ? l : 99), 13);
      ok = grid_barrier(c);
      KFB_STEP_STAMP((l < 4 ? l : 99), 14);
    }
    if (ok) {
      KFB_STEP_STAMP(7, 0);
      stage_x<M>(c, xin, p.hidden, p.final_norm, false);
      lm_head_stage<M>(c);
      KFB_STEP_STAMP(7, 1);
    }
  }
  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (threadIdx.x == 0 && sh->abort_word != 0) {
    // the step was given up: copies the producer has issued but nobody consumed may still be landing in this CTA's
    // shared memory -- wait for them (bounded) before the CTA exits, and make the other CTAs leave their barrier
    atomicAdd(p.bar, kPoison);
    for (int i = 0; i < (int)gridDim.x; ++i) st_release_gpu(p.flags + (size_t)i * kFlagStride, kPoison);
    const unsigned long long t0 = globaltimer_ns();
    for (uint32_t i = sh->consumed; i < sh->issued; ++i) {
      while (!mbar_test_wait(&sh->full[i % kSlots], (i / kSlots) & 1u)) {
        if (globaltimer_ns() - t0 > p.timeout_ns) break;
      }
    }
  }
}

// Self-test of the bounded grid barrier: `launched` CTAs run one barrier that expects `launched + 1` arrivals, so it
// can never complete; every CTA's wait runs out after timeout_ns, records 0x901, and the kernel returns through the same
// give-up path as the decode step (poisoned flags).  outcome[cta] = 1 barrier passed (never), 2 gave up.
__global__ void __launch_bounds__(kThreads, 1)
grid_barrier_selftest_kernel(const __grid_constant__ Params p, unsigned int* __restrict__ outcome) {
  __shared__ Shared sh_store;
  Shared* sh = &sh_store;
  Ctx c{p, nullptr, nullptr, sh, AbortCtx{&sh->abort_word, p.status, p.timeout_ns},
        (int)blockIdx.x, (int)gridDim.x + 1, (int)(threadIdx.x >> 5), (int)(threadIdx.x & 31), (int)threadIdx.x, 0u, 0ull};
  if (threadIdx.x == 0) { sh->abort_word = 0; sh->go = 0; }
  __syncthreads();
  if (c.warp < kConsumerWarps) {
    const bool passed = grid_barrier(c);
    if (c.tid == 0) outcome[blockIdx.x] = passed ? 1u : 2u;
  }
  __syncthreads();
  if (threadIdx.x == 0 && sh->abort_word != 0)
    for (int i = 0; i < (int)gridDim.x; ++i) st_release_gpu(p.flags + (size_t)i * kFlagStride, kPoison);
}

}  // namespace persist
}  // namespace kfb

using namespace kfb;

namespace {

int check_step(const kfb_decode_step_t* s) {
  if (!s) return fail(KFB_ERR_INVALID, "null pointer");
  if (s->batch < 1 || s->batch > 2) return fail(KFB_ERR_UNSUPPORTED, "the persistent decode step handles batch 1 and 2, got %d", s->batch);
  if (s->head_dim != 64) return fail(KFB_ERR_UNSUPPORTED, "the persistent decode step handles head_dim 64, got %d", s->head_dim);
  if (s->group != 64 && s->group != 128) return fail(KFB_ERR_INVALID, "group_size must be one of (64, 128), got %d", s->group);
  if (s->layers < 1 || s->heads < 1 || s->kv_heads < 1 || s->heads % s->kv_heads || s->max_len < 1 || s->vocab < 1)
    return fail(KFB_ERR_INVALID, "bad model shape");
  const int hd = s->heads * s->head_dim;
  const int ks[3] = {s->hidden, hd, s->intermediate};
  for (int k : ks)
    if (k < s->group || k % s->group || k % 32 || k > persist::kMaxK)
      return fail(KFB_ERR_UNSUPPORTED, "every reduction length must be a multiple of the group size and at most %d, got %d", persist::kMaxK, k);
  if (s->hidden % 256) return fail(KFB_ERR_UNSUPPORTED, "hidden must be a multiple of 256, got %d", s->hidden);
  const int unit_in = persist::int4_unit(s->hidden, s->group);
  const int unit_hd = persist::int4_unit(hd, s->group), unit_inter = persist::int4_unit(s->intermediate, s->group);
  const int unit_hidden = unit_hd > unit_inter ? unit_hd : unit_inter;
  if (s->hidden / sm_count() + 2 * unit_hidden > persist::kMaxOwnRows)
    return fail(KFB_ERR_UNSUPPORTED, "hidden = %d gives one CTA more than %d rows of the residual stream", s->hidden, persist::kMaxOwnRows);
  const int rows[4] = {(s->heads + 2 * s->kv_heads) * s->head_dim, s->hidden, 2 * s->intermediate, s->hidden};
  const int kk[4] = {s->hidden, hd, s->hidden, s->intermediate};
  const int units[4] = {unit_in, unit_hidden, unit_in, unit_hidden};
  for (int i = 0; i < 4; ++i) {
    if (rows[i] % units[i]) return fail(KFB_ERR_UNSUPPORTED, "a matrix of %d rows cannot be dealt out in units of %d rows", rows[i], units[i]);
    if ((kk[i] / 2 + kk[i] / s->group * 2) * units[i] > persist::kSlotBytes) return fail(KFB_ERR_UNSUPPORTED, "rows of K = %d do not fit a ring slot", kk[i]);
  }
  const void* ptrs[] = {s->layer_table, s->embed, s->final_norm, s->lm_head, s->cos_table, s->sin_table, s->tok, s->pos, s->kv_len,
                        s->logits, s->best, s->workspace};
  for (const void* q : ptrs)
    if (!q) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(s->embed) || !aligned16(s->final_norm) || !aligned16(s->lm_head) || !aligned16(s->workspace) || !aligned16(s->layer_table))
    return fail(KFB_ERR_ALIGNMENT, "embed, final_norm, lm_head, layer_table and workspace must be 16-byte aligned");
  return KFB_OK;
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

constexpr int kMaxCtas = 256;
struct WsLayout {
  size_t bar, flags, head_cnt, x, q, attn, act, part, total;
};
WsLayout ws_layout(int batch, int hidden, int heads, int kv_heads, int head_dim, int inter, int splits) {
  WsLayout w;
  size_t off = 0;
  w.bar = off; off += 256;
  w.flags = off; off += (size_t)kMaxCtas * persist::kFlagStride * 8;
  const int qb = (heads / kv_heads + 7) / 8;
  w.head_cnt = off; off += align256((size_t)batch * kv_heads * qb * 4);
  w.x = off; off += align256((size_t)batch * hidden * 2);
  w.q = off; off += align256((size_t)batch * heads * head_dim * 2);
  w.attn = off; off += align256((size_t)batch * heads * head_dim * 2);
  w.act = off; off += align256((size_t)batch * inter * 2);
  w.part = off; off += align256((size_t)batch * kv_heads * qb * splits * 8 * persist::kPartFloats * 4);
  w.total = off;
  return w;
}

int pick_splits(int batch, int heads, int kv_heads, int n_ctas) {
  const int qb = (heads / kv_heads + 7) / 8;
  int s = n_ctas / (batch * kv_heads * qb);
  return s < 1 ? 1 : (s > persist::kMaxSplits ? persist::kMaxSplits : s);
}

}  // namespace

#ifdef KFB_TRACE
extern "C" void kfb_debug_set_step_trace(void* device_buffer, int cta) {
  cudaMemcpyToSymbol(kfb::persist::g_step_trace, &device_buffer, sizeof(void*));
  cudaMemcpyToSymbol(kfb::persist::g_step_trace_cta, &cta, sizeof(int));
}
#endif

extern "C" int kfb_selftest_grid_barrier_expiry(unsigned long long timeout_ns, unsigned int* outcome_dev, void* scratch,
                                                size_t scratch_bytes, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (!outcome_dev || !scratch) return fail(KFB_ERR_INVALID, "null pointer");
  if (timeout_ns < 1000ull || timeout_ns > 100000000ull)
    return fail(KFB_ERR_INVALID, "the self-test takes a limit between 1 us and 100 ms, got %llu ns", timeout_ns);
  constexpr int kCtas = 4;
  const size_t need = 256 + (size_t)kCtas * persist::kFlagStride * 8;
  if (scratch_bytes < need || !aligned16(scratch)) return fail(KFB_ERR_WORKSPACE, "the self-test needs %zu bytes of 16-byte aligned scratch", need);
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  cudaStream_t st = (cudaStream_t)stream;
  KFB_CUDA_TRY(cudaMemsetAsync(scratch, 0, need, st));
  persist::Params p = {};
  p.bar = static_cast<unsigned long long*>(scratch);
  p.flags = reinterpret_cast<unsigned long long*>(static_cast<char*>(scratch) + 256);
  p.status = status;
  p.timeout_ns = timeout_ns;
  persist::grid_barrier_selftest_kernel<<<kCtas, persist::kThreads, 0, st>>>(p, outcome_dev);
  KFB_LAUNCH_CHECK("grid_barrier_selftest_kernel");
  return KFB_OK;
}

extern "C" int kfb_decode_step_slice(int n_rows, int K, int group, int unit_rows, int cta, int n_ctas, int* first_row, int* rows,
                                     int* rows_per_chunk) {
  if (n_rows < 1 || K < 32 || n_ctas < 1 || cta < 0 || cta >= n_ctas || !first_row || !rows || !rows_per_chunk)
    return fail(KFB_ERR_INVALID, "bad argument");
  const int row_bytes = group > 0 ? K / 2 + K / group * 2 : K * 2;   // INT4 row + its scales, or an fp16 row
  const int unit = unit_rows > 0 ? unit_rows : (group > 0 ? persist::int4_unit(K, group) : 1);
  if (n_rows % unit) return fail(KFB_ERR_UNSUPPORTED, "a matrix of %d rows cannot be dealt out in units of %d rows", n_rows, unit);
  const persist::Slice sl = persist::slice_of(n_rows, unit, row_bytes, cta, n_ctas);
  *first_row = sl.r0; *rows = sl.rows; *rows_per_chunk = sl.rows_per_chunk;
  return KFB_OK;
}

extern "C" size_t kfb_decode_step_ws_bytes(int batch, int hidden, int heads, int kv_heads, int head_dim, int intermediate) {
  if (batch < 1 || hidden < 1 || heads < 1 || kv_heads < 1 || head_dim < 1 || intermediate < 1 || heads % kv_heads) return 0;
  return ws_layout(batch, hidden, heads, kv_heads, head_dim, intermediate, persist::kMaxSplits).total;
}

extern "C" int kfb_decode_step_persistent(const kfb_decode_step_t* s, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_step(s)) return rc;
  const size_t need = kfb_decode_step_ws_bytes(s->batch, s->hidden, s->heads, s->kv_heads, s->head_dim, s->intermediate);
  if (s->workspace_bytes < need) return fail(KFB_ERR_WORKSPACE, "workspace of %zu bytes, %zu needed", (size_t)s->workspace_bytes, need);
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  cudaStream_t st = (cudaStream_t)stream;

  static bool configured[64] = {false};
  int dev = 0;
  KFB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    KFB_CUDA_TRY(cudaFuncSetAttribute(persist::decode_step_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, persist::kSmemBytes));
    KFB_CUDA_TRY(cudaFuncSetAttribute(persist::decode_step_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, persist::kSmemBytes));
    configured[dev] = true;
  }
  const int n_ctas = sm_count() < kMaxCtas ? sm_count() : kMaxCtas;   // one CTA per SM (shared memory allows no second one)
  const int splits = pick_splits(s->batch, s->heads, s->kv_heads, n_ctas);
  const WsLayout w = ws_layout(s->batch, s->hidden, s->heads, s->kv_heads, s->head_dim, s->intermediate, persist::kMaxSplits);
  char* ws = static_cast<char*>(s->workspace);

  persist::Params p = {};
  p.layers = static_cast<const persist::LayerPtrs*>(s->layer_table);
  p.L = s->layers; p.B = s->batch; p.hidden = s->hidden; p.H = s->heads; p.Hk = s->kv_heads; p.D = s->head_dim;
  p.inter = s->intermediate; p.vocab = s->vocab; p.Lmax = s->max_len; p.group = s->group; p.splits = splits;
  p.eps = s->rms_eps;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)s->head_dim);
  p.embed = static_cast<const __half*>(s->embed);
  p.final_norm = static_cast<const __half*>(s->final_norm);
  p.lm_head = static_cast<const char*>(s->lm_head);
  p.cos_t = static_cast<const float*>(s->cos_table);
  p.sin_t = static_cast<const float*>(s->sin_table);
  p.tok = static_cast<const long long*>(s->tok);
  p.pos = static_cast<const long long*>(s->pos);
  p.kv_len = static_cast<const int*>(s->kv_len);
  p.x = reinterpret_cast<__half*>(ws + w.x);
  p.q = reinterpret_cast<__half*>(ws + w.q);
  p.attn = reinterpret_cast<__half*>(ws + w.attn);
  p.act = reinterpret_cast<__half*>(ws + w.act);
  p.part = reinterpret_cast<float*>(ws + w.part);
  p.head_cnt = reinterpret_cast<unsigned int*>(ws + w.head_cnt);
  p.bar = reinterpret_cast<unsigned long long*>(ws + w.bar);
  p.flags = reinterpret_cast<unsigned long long*>(ws + w.flags);
  p.logits = static_cast<__half*>(s->logits);
  p.best = static_cast<unsigned long long*>(s->best);
  p.status = status;
  p.timeout_ns = sm100::kWaitTimeoutNs;

  // the barrier counter, the per-CTA barrier flags and the per-head arrival counters start every step at zero
  KFB_CUDA_TRY(cudaMemsetAsync(ws + w.bar, 0, w.x - w.bar, st));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ctas);
  cfg.blockDim = dim3(persist::kThreads);
  cfg.dynamicSmemBytes = persist::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = s->batch == 1 ? cudaLaunchKernelEx(&cfg, persist::decode_step_kernel<1>, p)
                                : cudaLaunchKernelEx(&cfg, persist::decode_step_kernel<2>, p);
  if (e != cudaSuccess) return fail(KFB_ERR_CUDA, "launch of decode_step_kernel failed: %s", cudaGetErrorString(e));
  return KFB_OK;
}
