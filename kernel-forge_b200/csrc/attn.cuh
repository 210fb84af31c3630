// Internal interface between the attention C-ABI entry point (flash_attn.cu) and the two kernels.
#pragma once

#include "common.cuh"

namespace kfb {
namespace attn {

struct Problem {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  int dtype;  // KFB_F16 / KFB_BF16
  int B, H, Hk, Nq, Nk, D;
  int causal;
  float scale;
  long long kv_stride_b, kv_stride_h, kv_stride_n;  // elements
  // decode only: device array of B valid lengths (<= Nk, the capacity of the cache); nullptr = all Nk keys
  const int* kv_len_dev = nullptr;
};

// Prefill / general path: one CTA per 128 query rows, TMA + tcgen05 + TMEM (attn_prefill.cu).
int launch_prefill(const Problem& p, cudaStream_t stream);

// Decode path (Nq == 1): split-KV, one CTA per (batch, kv head, split) (attn_decode.cu).
size_t decode_ws_bytes(int B, int H, int Hk, int Nk, int D);
int launch_decode(const Problem& p, void* ws, size_t ws_bytes, cudaStream_t stream, bool partial_only = false);
// Partial results only (no merge, no output): bytes of the (O, m, l) buffer and the number of key splits per
// (batch, kv-head slot); and the merge of `sets` such buffers, `set_stride` floats apart, into the output.
size_t decode_partial_bytes(int B, int H, int Hk, int Nk, int D, int* splits_out);
int launch_merge(const float* partial, void* o, int dtype, int B, int H, int Hk, int D, int splits, int sets, long long set_stride,
                 cudaStream_t stream);

}  // namespace attn
}  // namespace kfb
