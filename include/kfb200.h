/* kfb200 -- C ABI of the B200 (sm_100a) kernels behind KernelForge's two inference paths.
 *
 * This header is the drop-in boundary.  It replaces the reference's pybind11 module
 * `kernelforge._C` (csrc/bindings.cpp:12-28) and the torch entry points below it
 * (csrc/attention/attn_v4.cu:10-51, csrc/gemm/dequant_gemv.cu:21-36,
 * csrc/gemm/dequant_gemm_tc.cu:7-28) with plain-C entry points: raw device pointers,
 * sizes and a stream, no torch types.
 *
 * Conventions, all functions:
 *   - return KFB_OK (0) or a negative kfb_status; never throw, abort, exit or trap;
 *     kfb_last_error() gives the message of the last failure on the calling thread;
 *   - the caller owns every buffer (inputs, outputs, workspaces); unless a function says
 *     otherwise it allocates nothing, frees nothing and never synchronises, so a call can be
 *     captured in a CUDA graph;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default
 *     stream) of the device that is current on the calling thread;
 *   - data pointers must be 16-byte aligned (the reference demands the same,
 *     csrc/attention/attn_v4.cu:26-31, csrc/gemm/dequant_gemv.cu:17-18);
 *   - thread-safe; the only shared state is a mutex-guarded one-time set-up of kernel
 *     attributes; every host thread keeps its own small cache of encoded TMA tensor maps
 *     (keyed by base address, extents, strides and box), so a loop over the same tensors
 *     encodes each map once.
 */
#ifndef KFB200_H
#define KFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum kfb_status {
  KFB_OK = 0,
  KFB_ERR_INVALID = -1,     /* bad shape / size / flag                                  */
  KFB_ERR_ALIGNMENT = -2,   /* a pointer or stride is not 16-byte aligned               */
  KFB_ERR_UNSUPPORTED = -3, /* legal for the reference but outside what this build runs */
  KFB_ERR_WORKSPACE = -4,   /* workspace pointer NULL or too small                      */
  KFB_ERR_CUDA = -5,        /* a CUDA runtime / driver call failed (see kfb_last_error) */
  KFB_ERR_DEVICE = -6       /* the current device is not compute capability 10.x        */
} kfb_status;

typedef enum kfb_dtype { KFB_F16 = 0, KFB_BF16 = 1, KFB_F32 = 2 } kfb_dtype;

/* Library version (major*10000 + minor*100 + patch). */
int kfb_version(void);
/* Message of the last failed call on this thread ("" if none).  Never NULL. */
const char* kfb_last_error(void);
/* Reads the device status word of the current device into *out (synchronous 4-byte copy).
 * Kernels never trap: every wait on an mbarrier is bounded, and a wait that expires records
 * a non-zero code here and lets the kernel finish.  0 = no wait has ever expired.  (The
 * reference has no counterpart; its errors surface as CUDA errors, csrc/common/check.cuh:11-24.) */
int kfb_device_status(unsigned int* out);
/* Clears the status word of the current device (a 4-byte memset enqueued on `stream`).  The word is sticky: once a
 * wait has expired, every later attention / GEMM / GEMV launch on that device returns at once WITHOUT writing its
 * output, so a host that reads a non-zero status must discard the results enqueued since, find the cause, and call
 * this before it launches again.  Codes: 0x1xx prefill attention, 0x2xx decode attention, 0x3xx-0x5xx the INT4
 * kernels, 0x601 the self-test below, 0x701 kfb_rope_kv_write given a position outside the cache. */
int kfb_device_status_reset(void* stream);
/* Self-test of the bounded-wait path: launches one warp that waits, through the same helper every kernel of the
 * library uses, on an mbarrier that nothing arrives on, with a limit of timeout_ns (1 us .. 100 ms).  The wait runs
 * out, the kernel writes 2 to *outcome_dev (1 would mean the wait completed) and code 0x601 to the status word, and
 * returns normally; nothing faults or traps.  Follow it with kfb_device_status_reset.  No counterpart in the
 * reference (csrc/common/check.cuh:11-24 turns CUDA errors into exceptions; it has no in-kernel waits). */
int kfb_selftest_wait_expiry(unsigned long long timeout_ns, unsigned int* outcome_dev, void* stream);

/* Programmatic dependent launch for every kernel of a decode step (the INT4 GEMVs, decode attention, the fused
 * element-wise kernels, lm_head, finalize).  When on, launches carry the CUDA attribute that lets a kernel become
 * resident while the one in front of it in the stream is still running; each kernel waits for that one
 * (griddepcontrol.wait) before it touches any activation and only then releases its own successor, so results are
 * those of the plain stream order while launch latency -- and, for the GEMVs and the lm_head, the first round trip
 * of the weight stream -- is hidden behind the previous kernel.  Works in CUDA-graph capture.  Process-wide switch,
 * off by default; returns the previous setting.  The reference has no counterpart (its decode step is launch-bound:
 * docs/phase5-notes.md). */
int kfb_set_programmatic_launch(int enable);

/* ---------------------------------------------------------------------------------------
 * INT4 weight format (kernelforge/quantize.py).  packed: int32 [N, K/8], nibble position i
 * (bits 4i..4i+3) of word j holds q[8j + (0,2,4,6,1,3,5,7)[i]] + 8; scales: fp16 [N, K/G].
 * ------------------------------------------------------------------------------------- */

/* quantize_weight (kernelforge/quantize.py:100-105 = quantize_int4 :61-71 + pack_int4 :74-85),
 * bit-exact: scale = fp16(max(absmax/7, 2^-14)), 1 for an all-zero group;
 * q = clamp(rint(w / scale), -8, 7) in IEEE fp32.  w: [N, K] of w_dtype, G in {64,128}. */
int kfb_quantize_pack(const void* w, int w_dtype, int N, int K, int group,
                      void* packed, void* scales, void* stream);

/* unpack_int4 (kernelforge/quantize.py:88-97): packed -> int8 [N, K] in [-8, 7]. */
int kfb_unpack_int4(const void* packed, int N, int K, void* q_out, void* stream);

/* pack_int4 (kernelforge/quantize.py:74-85): int8 [N, K] in [-8, 7] -> packed.  Values are
 * masked to 4 bits; range checking is the caller's job (the Python layer does it). */
int kfb_pack_int4(const void* q, int N, int K, void* packed, void* stream);

/* dequantize (kernelforge/quantize.py:108-114): out [N, K]; KFB_F32 = exact q*scale,
 * KFB_F16 = one fp16 multiply half(q)*scale. */
int kfb_dequantize(const void* packed, const void* scales, int N, int K, int group,
                   void* out, int out_dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * INT4 weight-only linear  y[M, N] = x[M, K] @ W_hat[N, K]^T,  x and y fp16.
 * ------------------------------------------------------------------------------------- */

/* int4_gemv (csrc/gemm/dequant_gemv.cu:21-36, kernel csrc/gemm/dequant_gemv_kernel.cuh:38-109):
 * 1 <= M <= 8, any N >= 1, K % group == 0, group in {64,128}.  FP32 accumulation, one
 * rounding to fp16.  No workspace.  The weights are streamed by the TMA unit into shared
 * memory and multiplied on mma.sync fragments in their masked unsigned form (exact), with
 * a per-group correction from sums of x; a CUDA-core kernel (one FMA per weight, like the
 * reference's) remains for comparison and for very long K.
 * flags: bit 0 = launch with programmatic dependent launch (the weight prefetch of this
 * call may overlap the tail of the previous kernel on the stream; x is read and y written
 * only after the previous kernel has completed).
 *        bit 1 = use the CUDA-core kernel;  bit 2 = use the mma.sync kernel (bits 1 and 2 exclude each other;
 *        with neither, the faster one for the shape is chosen). */
int kfb_int4_gemv(const void* x, const void* packed, const void* scales, void* y,
                  int M, int N, int K, int group, int flags, void* stream);

/* The same weight-streaming kernel for 1 <= M <= 32: every further block of 8 batch rows is one
 * more MMA on the weight fragment that is already unpacked, so the cost per weight byte
 * stays that of the GEMV while the tcgen05 GEMM below still pays for a 128-row tile.
 * No counterpart in the reference (its GEMV stops at M = 8, kernelforge/ops.py:193; from there
 * on it uses the tensor-core GEMM).  Arguments and flags as kfb_int4_gemv; flag bit 1 is
 * honoured for M <= 8 only. */
int kfb_int4_small_batch(const void* x, const void* packed, const void* scales, void* y,
                         int M, int N, int K, int group, int flags, void* stream);

/* int4_gemv for 1 <= M <= 2 with the element-wise neighbours of a decode step fused in (the reference runs each of
 * them as a separate torch kernel: RMSNorm and SiLU * up in the Hugging Face modules it leaves untouched,
 * kernelforge/modules.py:51-68; the bias as `y + bias`, kernelforge/ops.py:300-301):
 *   xform 0: x [M, K] is used as given;
 *   xform 1: x [M, K] is the residual stream; the product uses fp16(fp16(x * rsqrt(mean(x^2) + eps)) * norm_weight[K]);
 *   xform 2: x [M, 2 K] is gate | up; the product uses fp16(fp16(silu(gate)) * up)   (K <= 8192 for xform 1, 2);
 *   then y = fp16(sum), + bias[N] when not NULL, + residual[M, N] when not NULL (fp16 additions, in that order).
 * Larger M: KFB_ERR_UNSUPPORTED (run the separate kernels).  flags: bit 0 as kfb_int4_gemv. */
int kfb_int4_gemv_fused(const void* x, const void* packed, const void* scales, void* y,
                        int M, int N, int K, int group, int xform, const void* norm_weight, float eps,
                        const void* bias, const void* residual, int flags, void* stream);

/* Two more fused forms of the same M <= 2 GEMV, for weight matrices whose ROWS the caller has put into a private order
 * when the model was built (rows are quantised independently, so reordering them is exact; the public packed format
 * of quantize_weight is unchanged).  xform / norm_weight / eps as in kfb_int4_gemv_fused.
 *   kfb_int4_gemv_silu_pair: rows 2p, 2p+1 = gate row p, up row p of a SiLU MLP; writes
 *     act_out[M, N/2] = fp16(fp16(silu(gate . x)) * (up . x)) -- the projection and the SiLU * up kernel in one launch.
 *   kfb_int4_gemv_rope_kv: the fused q / k / v projection of ONE decode position, N = (H + 2 Hk) D rows: for every q
 *     head, then every k head, rows 2j, 2j+1 = features j, j + D/2 (the pair the rotate-half rotary embedding mixes);
 *     then the v heads in natural order.  Rotates q and k with cos_table / sin_table [Lmax, D] at position *pos_dev,
 *     writes q_out [M, H, D] and row pos of k_cache / v_cache [M, Hk, Lmax, D] -- the projection and
 *     kfb_rope_kv_write in one launch; a position outside [0, Lmax) writes nothing and records 0x701.
 * No counterpart in the reference (it leaves these steps to Hugging Face / torch kernels). */
int kfb_int4_gemv_silu_pair(const void* x, const void* packed, const void* scales, void* act_out, int M, int N, int K,
                            int group, int xform, const void* norm_weight, float eps, int flags, void* stream);
int kfb_int4_gemv_rope_kv(const void* x, const void* packed, const void* scales, int M, int K, int group, int xform,
                          const void* norm_weight, float eps, const void* cos_table, const void* sin_table,
                          const void* pos_dev, void* q_out, void* k_cache, void* v_cache, int H, int Hk, int D, int Lmax,
                          int flags, void* stream);

/* One greedy decode step of a Llama-architecture model (INT4 decoder linears of kfb_quantize_pack's format, fp16
 * lm_head, RMSNorm, rotate-half RoPE, SiLU MLP, grouped-query attention over a static KV cache) as ONE persistent
 * cooperative kernel: batch 1 or 2, head_dim 64, one GPU.  It replaces the whole body of the reference's decode step
 * (bench/e2e_model.py:97-141: ~50 kernels per layer there) up to and including the lm_head and the argmax keys;
 * kfb_decode_finalize publishes the token afterwards.  No counterpart in the reference.
 *   layer_table: DEVICE array of `layers` entries of 12 pointers each, in this order: qkv packed, qkv scales, o packed,
 *     o scales, gate_up packed, gate_up scales, down packed, down scales, input RMSNorm weight, post-attention RMSNorm
 *     weight, K cache, V cache ([batch, kv_heads, max_len, head_dim] fp16).  The fused qkv matrix has its rows in the
 *     order of kfb_int4_gemv_rope_kv, the fused gate_up matrix in the order of kfb_int4_gemv_silu_pair (a private row
 *     order of the public packed format, chosen when the model is built).
 *   tok [batch] int64, pos [1] int64 (the cache row this step writes), kv_len [batch] int32 (valid keys including that
 *     row) are read on the device; logits [batch, vocab] fp16 and best [batch] (the argmax keys of kfb_fp16_gemv_argmax,
 *     which must be 0 before the call) are written.
 *   workspace: kfb_decode_step_ws_bytes bytes, 16-byte aligned, contents irrelevant; calls that share it must not overlap.
 * Every in-kernel wait is bounded: an expired wait records 0x901 (grid barrier) or 0x902 (weight ring) in the device
 * status word and the kernel returns; a position outside [0, max_len) records 0x701 and nothing is written. */
/* Self-test of the decode step's bounded grid barrier: 4 CTAs run one barrier that expects 5 arrivals; every wait runs
 * out after timeout_ns (1 us .. 100 ms), outcome_dev[cta] (4 uint32) becomes 2 (1 would mean the barrier completed), the
 * status word gets 0x901 and the kernel returns normally.  scratch: 1 KiB of device memory.  Follow it with
 * kfb_device_status_reset. */
int kfb_selftest_grid_barrier_expiry(unsigned long long timeout_ns, unsigned int* outcome_dev, void* scratch,
                                     size_t scratch_bytes, void* stream);

typedef struct kfb_decode_step_t {
  const void* layer_table;
  int layers, batch, hidden, heads, kv_heads, head_dim, intermediate, vocab, max_len, group;
  float rms_eps;
  const void* embed;       /* fp16 [vocab, hidden] */
  const void* final_norm;  /* fp16 [hidden] */
  const void* lm_head;     /* fp16 [vocab, hidden] */
  const void* cos_table;   /* fp32 [max_len, head_dim] */
  const void* sin_table;
  const void* tok;
  const void* pos;
  const void* kv_len;
  void* logits;
  void* best;
  void* workspace;
  size_t workspace_bytes;
} kfb_decode_step_t;
size_t kfb_decode_step_ws_bytes(int batch, int hidden, int heads, int kv_heads, int head_dim, int intermediate);
/* The static schedule of the persistent step, for inspection (host only, no device needed): the rows of an [n_rows, K]
 * matrix that CTA `cta` of `n_ctas` owns, and how many of them go through one shared-memory ring slot at a time.
 * group > 0: an INT4 matrix with that group size (rows dealt out in the smallest even unit whose scale rows are a multiple
 * of 16 bytes, or in `unit_rows` when > 0); group == 0: an fp16 matrix (the lm_head), unit 1. */
int kfb_decode_step_slice(int n_rows, int K, int group, int unit_rows, int cta, int n_ctas, int* first_row, int* rows,
                          int* rows_per_chunk);
int kfb_decode_step_persistent(const kfb_decode_step_t* step, void* stream);

/* A PRIVATE, PREPACKED copy of a weight in MMA-fragment order, and the M <= 32 GEMV that runs on it -- the reference's
 * stated next step for the INT4 path (docs/phase4-notes.md:59, README.md:104: "reorder the packed weights offline so each
 * thread loads its own MMA fragment nibbles"); nothing of it exists in the reference.  The public format stays what
 * callers exchange; the copy has the same size (N K / 2 bytes) and is built once per weight.
 *   kfb_int4_prepack: packed int32 [N, K/8] -> out (kfb_int4_prepack_bytes(N, K) bytes; 0 = shape not supported:
 *     N % 16 == 0 and K % 64 == 0 are required).  Rows in blocks of 16, K in blocks of 64; block (rb, kb) is 512
 *     contiguous bytes, lane 4 g + t of a warp owning 16 of them: the two words of row 16 rb + g and the two of row
 *     16 rb + g + 8 that cover k in [64 kb + 16 t, 64 kb + 16 t + 16).
 *   kfb_int4_gemv_prepacked: y[M, N] = x[M, K] W^T with the scales in the public layout (fp16 [N, K/group]); 1 <= M <= 32
 *     (flat in M up to 8, then 2 or 4 MMAs per unpacked fragment), K <= 12288.  Same arithmetic contract as kfb_int4_gemv (exact integer weights, FP32 accumulation, FP32 group
 *     scale, one rounding to fp16).
 *     bias [N] / residual [M, N] (fp16, or NULL) are added in the epilogue like kfb_int4_gemv_fused does.
 *   kfb_int4_gemv_prepacked_silu_pair / _rope_kv: the pair epilogues of kfb_int4_gemv_silu_pair / kfb_int4_gemv_rope_kv
 *     (same row orders of the weight, same arguments, same roundings) for M <= 32. */
size_t kfb_int4_prepack_bytes(int N, int K);
int kfb_int4_prepack(const void* packed, int N, int K, void* out, void* stream);
int kfb_int4_gemv_prepacked(const void* x, const void* prepacked, const void* scales, void* y, int M, int N, int K,
                            int group, const void* bias, const void* residual, void* stream);
int kfb_int4_gemv_prepacked_silu_pair(const void* x, const void* prepacked, const void* scales, void* act_out, int M, int N,
                                      int K, int group, void* stream);
int kfb_int4_gemv_prepacked_rope_kv(const void* x, const void* prepacked, const void* scales, int M, int K, int group,
                                    const void* cos_table, const void* sin_table, const void* pos_dev, void* q_out,
                                    void* k_cache, void* v_cache, int H, int Hk, int D, int Lmax, void* stream);

/* int4_gemm (csrc/gemm/dequant_gemm_tc.cu:7-28, kernels csrc/gemm/dequant_gemm_tc_kernel.cuh:55-162):
 * any M >= 1, any N >= 1 (the reference needs N % 64 == 0; N-sharding needs ragged N),
 * K % group == 0.  Weights are dequantised into swizzled shared memory and multiplied on
 * the tcgen05 tensor cores with FP32 accumulation in TMEM.  Split-K partial sums go through
 * `ws` (FP32, fixed-order reduce => deterministic). */
size_t kfb_int4_gemm_ws_bytes(int M, int N, int K, int group);
int kfb_int4_gemm(const void* x, const void* packed, const void* scales, void* y,
                  int M, int N, int K, int group, void* ws, size_t ws_bytes, void* stream);

/* The same GEMM for bf16 activations: x and y bf16, scales stay fp16.  The weights are dequantised to bf16(q * s) (the
 * product formed in FP32, one rounding), FP32 accumulation, one rounding to bf16.  Serves every M >= 1.  The reference
 * takes fp16 activations only (README.md:103 lists bf16 as not done); this entry has no counterpart there. */
int kfb_int4_gemm_bf16(const void* x, const void* packed, const void* scales, void* y,
                       int M, int N, int K, int group, void* ws, size_t ws_bytes, void* stream);

/* int4_gemm for an output-feature-sharded linear, fused with the all-gather that follows it.
 * The reference is single-GPU; this entry point has no counterpart there.
 * This rank holds N_local rows of packed / scales and computes y[:, col0 : col0 + N_local]; the epilogue
 * stores that block into ALL n_buffers output buffers (y_all[i]: fp16 [M, ld], the peer-mapped address of
 * GPU i's full result, this GPU's own buffer included) with plain peer stores over NVLink, tile by tile
 * as the tiles finish, so no separate all-gather kernel runs.  Stores only: nothing is loaded from a
 * peer.  The caller orders the call against the peers (kfb_peer_signal_wait on the stream after the call, before
 * anyone reads y; and no peer may still be reading a buffer that this call overwrites: alternate two buffers).
 * Workspace: kfb_int4_gemm_ws_bytes(M, N_local, K, group). */
int kfb_int4_gemm_allgather(const void* x, const void* packed, const void* scales, void* const* y_all,
                            int n_buffers, int M, int N_local, int K, int group, int ld, int col0,
                            void* ws, size_t ws_bytes, void* stream);

/* Device-side rendezvous of the ranks of one node, enqueued on the stream (no host synchronisation, CUDA-graph
 * capturable): adds 1 to the arrival counter of every rank (peer_counters[i] = peer-mapped address of rank i's counter,
 * this rank's own included) after a system-scope fence -- so everything this stream stored into peer memory before,
 * e.g. by kfb_int4_gemm_allgather, is visible to a rank that sees the arrival -- and then waits until this rank's own
 * counter has received n_ranks more arrivals than the target recorded in *local_target (device uint64, advanced by
 * the kernel).  The wait is bounded: after timeout_ns (1 us .. 10 s) the kernel records 0x801 in the device status
 * word and returns.  Counters are uint64, zero-initialised, in memory every rank can address (symmetric memory);
 * only stores and atomic adds cross the link.  No counterpart in the reference (single GPU). */
int kfb_peer_signal_wait(void* const* peer_counters, int n_ranks, const void* local_counter, void* local_target,
                         unsigned long long timeout_ns, void* stream);

/* All-gather of column blocks over peer memory in one launch: src [M, w_local] fp16 (dense rows) is stored into columns
 * [col0, col0 + w_local) of every rank's [M, ld] fp16 buffer dst_all[i], then the ranks rendezvous as in
 * kfb_peer_signal_wait (every rank launches the same number of CTAs, each signals once).  When the call returns on the
 * stream, every rank's block has arrived in this rank's buffer.  A buffer may be overwritten by the call after the
 * next one at the earliest (alternate two buffers, each with its own counter and target). */
int kfb_peer_allgather(const void* src, void* const* dst_all, void* const* peer_counters, int n_ranks, int M,
                       int w_local, int ld, int col0, const void* local_counter, void* local_target,
                       unsigned long long timeout_ns, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused attention forward  O = softmax(scale * Q K^T + causal mask) V
 * (kernelforge/ops.py:258-274 -> csrc/attention/attn_v4.cu:10-51, kernel attn_v4_kernel.cuh:43-214).
 *   q, o: [B, H, Nq, D] contiguous; k, v: [B, Hk, Nk, D]; dtype KFB_F16 or KFB_BF16;
 *   D in {64, 128}; H % Hk == 0; causal => Nq <= Nk, key j visible to query i iff
 *   j <= i + (Nk - Nq).
 *   kv_strides: NULL for contiguous k/v, else {batch, head, row} strides IN ELEMENTS shared by
 *   k and v (each a multiple of 8; the D axis must be dense), so a KV-cache view
 *   cache[:, :, :Nk] needs no copy.
 *   Prefill (Nq > 1): TMA-staged swizzled tiles, tcgen05 MMA, accumulators in TMEM.
 *   Decode (Nq == 1): split-KV kernel; partial (o, m, l) per split go through `ws`.
 * ------------------------------------------------------------------------------------- */
size_t kfb_flash_attn_ws_bytes(int B, int H, int Hk, int Nq, int Nk, int D);
int kfb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, int dtype,
                       int B, int H, int Hk, int Nq, int Nk, int D, int causal, float scale,
                       const int64_t* kv_strides, void* ws, size_t ws_bytes, void* stream);

/* Decode attention (Nq == 1) against a STATIC KV cache: k, v are [B, Hk, Nk, D] buffers of capacity Nk
 * of which only kv_len_dev[b] rows (a device int32 array of B entries) are valid; the rest is ignored.
 * The length is read by the kernel, so one captured launch can be replayed from a CUDA graph while the
 * cache grows -- what the reference could not do (its kernel takes the length from the tensor shape, so
 * its graph-mode decode falls back to SDPA: bench/e2e_model.py:91-92, README.md:101).
 * Workspace as for kfb_flash_attn_fwd with Nq == 1 (kfb_flash_attn_ws_bytes(B, H, Hk, 1, Nk, D)). */
int kfb_flash_attn_decode_kvlen(const void* q, const void* k, const void* v, void* o, int dtype,
                                int B, int H, int Hk, int Nk, int D, float scale,
                                const int64_t* kv_strides, const int32_t* kv_len_dev,
                                void* ws, size_t ws_bytes, void* stream);

/* Decode attention over a KV cache that is SHARDED ALONG THE SEQUENCE (one shard per GPU for a single long sequence,
 * or any other split the caller makes).  The reference is single-GPU; these entries have no counterpart there.
 *   kfb_flash_attn_decode_partial: runs the split-KV kernel on one shard (k, v: [B, Hk, Nk, D] of this shard, kv_len_dev
 *     as in kfb_flash_attn_decode_kvlen or NULL) and leaves the softmax partials in `partial`: per (batch, kv-head
 *     slot, key split) the unnormalised O (FP32), the running maximum m (log2 units) and the sum l.
 *     kfb_flash_attn_decode_partial_bytes gives the buffer size (and the number of key splits) for the shard shape.
 *   kfb_flash_attn_merge_partials: combines n_sets such buffers (set_stride_bytes apart, e.g. the result of an
 *     all-gather; every set made with the same shard shape Nk_per_set) in set order and writes o [B, H, 1, D].
 *     A shard with no valid key contributes nothing; if no shard has any, the output is zero. */
size_t kfb_flash_attn_decode_partial_bytes(int B, int H, int Hk, int Nk, int D, int* splits_out);
int kfb_flash_attn_decode_partial(const void* q, const void* k, const void* v, int dtype, int B, int H, int Hk,
                                  int Nk, int D, float scale, const int64_t* kv_strides, const int32_t* kv_len_dev,
                                  void* partial, size_t partial_bytes, void* stream);
int kfb_flash_attn_merge_partials(const void* partials, int n_sets, size_t set_stride_bytes, void* o, int dtype,
                                  int B, int H, int Hk, int Nk_per_set, int D, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused element-wise steps of a Llama-architecture decode step (fp16).  The reference leaves these to
 * Hugging Face / torch ops (it replaces only the linears and the attention function,
 * kernelforge/modules.py:51-115); they are here because a batch-1 decode step is launch-bound.
 * ------------------------------------------------------------------------------------- */

/* s = x + residual (skipped when residual is NULL), written to sum_out when not NULL;
 * y = fp16(fp16(s * rsqrt(mean(s^2) + eps)) * weight).  x, residual, y, sum_out: [rows, hidden]. */
int kfb_add_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* sum_out,
                    int rows, int hidden, float eps, void* stream);

/* Rotary embedding + KV-cache write of one decode position.  qkv: [B, (H + 2*Hk) * D] (q heads, then k
 * heads, then v heads, as produced by one fused q/k/v linear); cos_table, sin_table: fp32 [Lmax, D]
 * (rotate-half convention); pos_dev: device int64, the position being written.  q_out: [B, H, D];
 * k_cache, v_cache: [B, Hk, Lmax, D], row `pos` is written.  A position outside [0, Lmax) writes nothing and
 * records code 0x701 in the device status word (the kernel reads the position on the device, e.g. in a graph replay,
 * so the host cannot check it at launch time). */
int kfb_rope_kv_write(const void* qkv, const void* cos_table, const void* sin_table, const void* pos_dev,
                      void* q_out, void* k_cache, void* v_cache, int B, int H, int Hk, int D, int Lmax,
                      void* stream);

/* out[r, c] = fp16(fp16(silu(gate_up[r, c])) * gate_up[r, inter + c]); gate_up: [rows, 2 * inter]. */
int kfb_silu_mul(const void* gate_up, void* out, int rows, int inter, void* stream);

/* The fp16 lm_head of a decode step with the greedy argmax fused: y[M, N] = x[M, K] w[N, K]^T, 1 <= M <= 32,
 * K % 32 == 0, fp16 in, FP32 accumulation, fp16 out; w is streamed once (it is the largest read of a step:
 * docs/phase5-notes.md:39 of the reference, which runs `h @ lm_head.T` on cuBLAS and a separate argmax,
 * bench/e2e_model.py:97-141).  best: NULL, or M 64-bit keys that must be 0 before the call; afterwards key m holds
 * (order-preserving bits of the largest logit of row m) << 32 | (0xFFFFFFFF - its index), lowest index on ties. */
int kfb_fp16_gemv_argmax(const void* x, const void* w, void* y, void* best, int M, int N, int K, void* stream);

/* End of a decode step: tok[m] (int64) = index held in best[m]; best[m] = 0; kv_len[m] (int32) += 1; pos[0] (int64)
 * += 1.  One launch in place of argmax + copy + two adds in the reference's step (bench/e2e_model.py:122-131). */
int kfb_decode_finalize(void* best, void* tok, void* pos, void* kv_len, int M, void* stream);

/* Start of a decode step: x_out[r] = embed[tok[r]] (tok int64, ids clamped to [0, vocab)), y[r] = RMSNorm(x_out[r]) *
 * weight with the rounding of kfb_add_rmsnorm.  embed: fp16 [vocab, hidden]. */
int kfb_embed_rmsnorm(const void* tok, const void* embed, const void* weight, void* y, void* x_out, int rows,
                      int hidden, int vocab, float eps, void* stream);

/* Decode attention (Nq == 1, one query per head at the last cache position) for callers that
 * cannot allocate device memory: a server whose memory pool already owns the whole GPU, code
 * between cudaStreamBeginCapture and EndCapture (cudaMalloc is not allowed there), a host runtime
 * without a device allocator.  This entry point has no counterpart in the reference.
 * It computes exactly what kfb_flash_attn_fwd computes for Nq == 1, but the split-KV partial
 * results go through a 4 MiB array that is part of the library image (each GPU that loads the
 * library holds those 4 MiB until the process exits) instead of a caller workspace; the call
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *   - A problem whose split plan needs more than 4 MiB (kfb_flash_attn_ws_bytes tells) is refused
 *     with KFB_ERR_WORKSPACE: the array holds 992 (batch x kv-head x split) partials at D = 64
 *     and 504 at D = 128.  Small batches fit (B = 1..8 with 4 KV heads: at most 416 partials);
 *     e.g. B = 32, Hk = 4, Nk = 16384 (1280 partials) does not.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Nothing in it has to be cleared between calls
 *     (each call overwrites every value it later reads), but two calls that can overlap on the
 *     GPU -- different streams, or graph branches without a dependency -- race on it: serialise
 *     them.  kv_strides as for kfb_flash_attn_fwd. */
int kfb_flash_attn_decode_noalloc(const void* q, const void* k, const void* v, void* o, int dtype,
                                  int B, int H, int Hk, int Nk, int D, float scale,
                                  const int64_t* kv_strides, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KFB200_H */
