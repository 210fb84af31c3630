// C-ABI entry point of the fused attention forward: argument checks and kernel choice.
// Replaces the torch entry `attn_v4` of the reference (csrc/attention/attn_v4.cu:10-51).
#include "attn.cuh"

using namespace kfb;

namespace {

int check_shape(int dtype, int B, int H, int Hk, int Nq, int Nk, int D, int causal) {
  if (dtype != KFB_F16 && dtype != KFB_BF16) return fail(KFB_ERR_INVALID, "attention takes fp16 or bf16 tensors");
  if (B < 1 || H < 1 || Hk < 1 || Nq < 1 || Nk < 1)
    return fail(KFB_ERR_INVALID, "B, H, Hk, Nq, Nk must be >= 1 (got %d, %d, %d, %d, %d)", B, H, Hk, Nq, Nk);
  if (D != 64 && D != 128) return fail(KFB_ERR_INVALID, "head dim must be one of (64, 128), got %d", D);
  if (H % Hk) return fail(KFB_ERR_INVALID, "query heads (%d) must be a multiple of key/value heads (%d)", H, Hk);
  if (causal && Nq > Nk) return fail(KFB_ERR_INVALID, "causal attention needs Nq <= Nk, got %d > %d", Nq, Nk);
  return KFB_OK;
}

}  // namespace

extern "C" size_t kfb_flash_attn_ws_bytes(int B, int H, int Hk, int Nq, int Nk, int D) {
  if (B < 1 || H < 1 || Hk < 1 || Nq != 1 || Nk < 1 || (D != 64 && D != 128) || H % Hk) return 0;
  return attn::decode_ws_bytes(B, H, Hk, Nk, D);
}

extern "C" int kfb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, int dtype, int B, int H,
                                  int Hk, int Nq, int Nk, int D, int causal, float scale, const int64_t* kv_strides,
                                  void* ws, size_t ws_bytes, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_shape(dtype, B, H, Hk, Nq, Nk, D, causal)) return rc;
  if (!(scale > 0.0f)) return fail(KFB_ERR_INVALID, "scale must be positive, got %g", (double)scale);
  if (!q || !k || !v || !o) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(KFB_ERR_ALIGNMENT, "q, k, v, o must be 16-byte aligned");
  attn::Problem p;
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.dtype = dtype; p.B = B; p.H = H; p.Hk = Hk; p.Nq = Nq; p.Nk = Nk; p.D = D;
  p.causal = causal ? 1 : 0;
  p.scale = scale;
  if (kv_strides) {
    p.kv_stride_b = kv_strides[0]; p.kv_stride_h = kv_strides[1]; p.kv_stride_n = kv_strides[2];
    if (p.kv_stride_n < D || p.kv_stride_h < 1 || p.kv_stride_b < 1 || (p.kv_stride_b % 8) || (p.kv_stride_h % 8) ||
        (p.kv_stride_n % 8))
      return fail(KFB_ERR_ALIGNMENT, "kv strides must be positive multiples of 8 elements with a row stride >= D");
  } else {
    p.kv_stride_n = D; p.kv_stride_h = (long long)Nk * D; p.kv_stride_b = (long long)Hk * Nk * D;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (Nq == 1) return attn::launch_decode(p, ws, ws_bytes, s);
  return attn::launch_prefill(p, s);
}

// Decode attention against a static KV cache whose valid length lives on the device.
extern "C" int kfb_flash_attn_decode_kvlen(const void* q, const void* k, const void* v, void* o, int dtype, int B, int H,
                                           int Hk, int Nk, int D, float scale, const int64_t* kv_strides,
                                           const int32_t* kv_len_dev, void* ws, size_t ws_bytes, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_shape(dtype, B, H, Hk, 1, Nk, D, 0)) return rc;
  if (!(scale > 0.0f)) return fail(KFB_ERR_INVALID, "scale must be positive, got %g", (double)scale);
  if (!q || !k || !v || !o || !kv_len_dev) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(KFB_ERR_ALIGNMENT, "q, k, v, o must be 16-byte aligned");
  attn::Problem p;
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.dtype = dtype; p.B = B; p.H = H; p.Hk = Hk; p.Nq = 1; p.Nk = Nk; p.D = D;
  p.causal = 0;
  p.scale = scale;
  p.kv_len_dev = kv_len_dev;
  if (kv_strides) {
    p.kv_stride_b = kv_strides[0]; p.kv_stride_h = kv_strides[1]; p.kv_stride_n = kv_strides[2];
    if (p.kv_stride_n < D || p.kv_stride_h < 1 || p.kv_stride_b < 1 || (p.kv_stride_b % 8) || (p.kv_stride_h % 8) ||
        (p.kv_stride_n % 8))
      return fail(KFB_ERR_ALIGNMENT, "kv strides must be positive multiples of 8 elements with a row stride >= D");
  } else {
    p.kv_stride_n = D; p.kv_stride_h = (long long)Nk * D; p.kv_stride_b = (long long)Hk * Nk * D;
  }
  return attn::launch_decode(p, ws, ws_bytes, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------
// Decode attention over a KV cache that is sharded along the sequence (across GPUs, or any other split the caller
// makes): each shard produces its softmax partial (unnormalised O, running maximum m, sum l per query head), the
// partials are brought together by the caller (an all-gather) and merged here.  The reference is single-GPU.
// ------------------------------------------------------------------------------------------------
extern "C" size_t kfb_flash_attn_decode_partial_bytes(int B, int H, int Hk, int Nk, int D, int* splits_out) {
  if (B < 1 || H < 1 || Hk < 1 || Nk < 1 || (D != 64 && D != 128) || H % Hk) return 0;
  return attn::decode_partial_bytes(B, H, Hk, Nk, D, splits_out);
}

extern "C" int kfb_flash_attn_decode_partial(const void* q, const void* k, const void* v, int dtype, int B, int H, int Hk,
                                             int Nk, int D, float scale, const int64_t* kv_strides, const int32_t* kv_len_dev,
                                             void* partial, size_t partial_bytes, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_shape(dtype, B, H, Hk, 1, Nk, D, 0)) return rc;
  if (!(scale > 0.0f)) return fail(KFB_ERR_INVALID, "scale must be positive, got %g", (double)scale);
  if (!q || !k || !v || !partial) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(partial))
    return fail(KFB_ERR_ALIGNMENT, "q, k, v and the partial buffer must be 16-byte aligned");
  attn::Problem p;
  p.q = q; p.k = k; p.v = v; p.o = nullptr;
  p.dtype = dtype; p.B = B; p.H = H; p.Hk = Hk; p.Nq = 1; p.Nk = Nk; p.D = D;
  p.causal = 0;
  p.scale = scale;
  p.kv_len_dev = kv_len_dev;
  if (kv_strides) {
    p.kv_stride_b = kv_strides[0]; p.kv_stride_h = kv_strides[1]; p.kv_stride_n = kv_strides[2];
    if (p.kv_stride_n < D || p.kv_stride_h < 1 || p.kv_stride_b < 1 || (p.kv_stride_b % 8) || (p.kv_stride_h % 8) ||
        (p.kv_stride_n % 8))
      return fail(KFB_ERR_ALIGNMENT, "kv strides must be positive multiples of 8 elements with a row stride >= D");
  } else {
    p.kv_stride_n = D; p.kv_stride_h = (long long)Nk * D; p.kv_stride_b = (long long)Hk * Nk * D;
  }
  return attn::launch_decode(p, partial, partial_bytes, (cudaStream_t)stream, /*partial_only=*/true);
}

extern "C" int kfb_flash_attn_merge_partials(const void* partials, int n_sets, size_t set_stride_bytes, void* o, int dtype,
                                             int B, int H, int Hk, int Nk_per_set, int D, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (int rc = check_shape(dtype, B, H, Hk, 1, Nk_per_set, D, 0)) return rc;
  if (n_sets < 1 || n_sets > 64) return fail(KFB_ERR_INVALID, "number of partial sets must be in [1, 64], got %d", n_sets);
  if (!partials || !o) return fail(KFB_ERR_INVALID, "null pointer");
  int splits = 1;
  const size_t bytes = attn::decode_partial_bytes(B, H, Hk, Nk_per_set, D, &splits);
  if (n_sets > 1 && (set_stride_bytes < bytes || set_stride_bytes % 4))
    return fail(KFB_ERR_INVALID, "partial sets must be at least %zu bytes apart, got %zu", bytes, set_stride_bytes);
  return attn::launch_merge(static_cast<const float*>(partials), o, dtype, B, H, Hk, D, splits, n_sets,
                            (long long)(set_stride_bytes / 4), (cudaStream_t)stream);
}
