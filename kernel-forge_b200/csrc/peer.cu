// Device-side exchange between the GPUs of one node over peer-mapped memory (NVLink / NVSwitch), for the output-
// feature-sharded INT4 linear and the tensor-parallel decode step.  The reference is single-GPU and has no counterpart.
//
// Everything that crosses the link is a plain STORE or a system-scope atomic ADD into a peer's memory; nothing is ever
// loaded from a peer, and no TMA or multicast operation touches peer memory.
//
//   peer_signal_wait_kernel   a barrier across GPUs inside the stream: every rank adds 1 to an arrival counter in each
//                             peer's memory (after a system-scope fence, so everything the stream wrote to the peers
//                             before -- e.g. the epilogue stores of kfb_int4_gemm_allgather -- is visible first), then
//                             waits until its own counter has received one arrival per rank.  Replaces a host-driven
//                             NCCL all-reduce used as rendezvous.
//   peer_allgather_kernel     all-gather of column blocks: each rank stores its [M, w] block into columns
//                             [col0, col0 + w) of every rank's [M, ld] buffer, signals, and waits in the same launch.
//
// The wait is bounded (timeout_ns, by %globaltimer): when it runs out the kernel records code 0x801 in the device
// status word and returns, so a peer that never arrives cannot hang this GPU.  The expected count lives in device
// memory and is advanced by the kernel itself, so the launches can be captured in a CUDA graph and replayed.
#include "common.cuh"

namespace kfb {
namespace peer {
namespace {

constexpr int kMaxPeers = 8;
constexpr unsigned int kStatusPeerTimeout = 0x801;
constexpr int kGatherCtas = 8;   // the same on every rank: the expected arrival count must not depend on a rank's shard

struct PeerPtrs {
  unsigned long long* counter[kMaxPeers];   // address of the arrival counter in each rank's memory (own included)
  void* data[kMaxPeers];                    // peer_allgather: each rank's result buffer
  int n;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Waits until *counter >= target (bounded).  One thread.
__device__ bool wait_arrivals(const unsigned long long* counter, unsigned long long target, unsigned long long timeout_ns,
                              unsigned int* status) {
  if (ld_acquire_sys(counter) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(counter) < target) {
    __nanosleep(200);
    if (globaltimer_ns() - t0 > timeout_ns) {
      atomicCAS(status, 0u, kStatusPeerTimeout);
      return false;
    }
  }
  return true;
}

__global__ void peer_signal_wait_kernel(const PeerPtrs peers, const unsigned long long* local_counter,
                                        unsigned long long* local_target, unsigned long long timeout_ns, unsigned int* status) {
  pdl_wait();
  pdl_launch_dependents();
  __threadfence_system();   // what this stream stored into the peers before this kernel is visible before the signal
  if ((int)threadIdx.x < peers.n) atomicAdd_system(peers.counter[threadIdx.x], 1ull);
  if (threadIdx.x == 0) {
    const unsigned long long target = *local_target + (unsigned long long)peers.n;
    wait_arrivals(local_counter, target, timeout_ns, status);
    *local_target = target;
    __threadfence_system();
  }
}

// src: [M, w] fp16 (row stride w); every peer's buffer: [M, ld] fp16; this rank writes columns [col0, col0 + w).
__global__ void __launch_bounds__(256)
peer_allgather_kernel(const __half* __restrict__ src, const PeerPtrs peers, int M, int w, int ld, int col0,
                      const unsigned long long* local_counter, unsigned long long* local_target, unsigned long long timeout_ns,
                      unsigned int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const bool vec = ((w | ld | col0) & 7) == 0;
  if (vec) {
    const int wv = w / 8;
    const long long total = (long long)M * wv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const long long m = i / wv;
      const int c = (int)(i - m * wv);
      const uint4 v = reinterpret_cast<const uint4*>(src + m * w)[c];
      for (int p = 0; p < peers.n; ++p)
        reinterpret_cast<uint4*>(static_cast<__half*>(peers.data[p]) + m * ld + col0)[c] = v;
    }
  } else {
    const long long total = (long long)M * w;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const long long m = i / w;
      const int c = (int)(i - m * w);
      const __half v = src[i];
      for (int p = 0; p < peers.n; ++p) static_cast<__half*>(peers.data[p])[m * ld + col0 + c] = v;
    }
  }
  __threadfence_system();
  __syncthreads();   // every thread of this CTA has stored and fenced
  if ((int)threadIdx.x < peers.n) atomicAdd_system(peers.counter[threadIdx.x], 1ull);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const unsigned long long target = *local_target + (unsigned long long)peers.n * gridDim.x;
    wait_arrivals(local_counter, target, timeout_ns, status);
    *local_target = target;
    __threadfence_system();
  }
}

int fill(PeerPtrs* out, void* const* counters, void* const* data, int n) {
  if (n < 1 || n > kMaxPeers) return fail(KFB_ERR_INVALID, "number of ranks must be in [1, %d], got %d", kMaxPeers, n);
  if (!counters) return fail(KFB_ERR_INVALID, "null pointer");
  out->n = n;
  for (int i = 0; i < n; ++i) {
    if (!counters[i] || (reinterpret_cast<uintptr_t>(counters[i]) & 7u)) return fail(KFB_ERR_ALIGNMENT, "arrival counters must be non-null and 8-byte aligned");
    out->counter[i] = static_cast<unsigned long long*>(counters[i]);
    out->data[i] = data ? data[i] : nullptr;
    if (data && (!data[i] || !aligned16(data[i]))) return fail(KFB_ERR_ALIGNMENT, "result buffers must be non-null and 16-byte aligned");
  }
  return KFB_OK;
}

int check_wait_args(const void* local_counter, const void* local_target, unsigned long long timeout_ns) {
  if (!local_counter || !local_target) return fail(KFB_ERR_INVALID, "null pointer");
  if (timeout_ns < 1000ull || timeout_ns > 10000000000ull)
    return fail(KFB_ERR_INVALID, "the wait limit must be between 1 us and 10 s, got %llu ns", timeout_ns);
  return KFB_OK;
}

}  // namespace
}  // namespace peer
}  // namespace kfb

using namespace kfb;

extern "C" int kfb_peer_signal_wait(void* const* peer_counters, int n_ranks, const void* local_counter, void* local_target,
                                    unsigned long long timeout_ns, void* stream) {
  if (int rc = require_sm100()) return rc;
  peer::PeerPtrs pp;
  if (int rc = peer::fill(&pp, peer_counters, nullptr, n_ranks)) return rc;
  if (int rc = peer::check_wait_args(local_counter, local_target, timeout_ns)) return rc;
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  return launch_kernel("peer_signal_wait_kernel", peer::peer_signal_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream,
                       pdl_enabled(), pp, static_cast<const unsigned long long*>(local_counter),
                       static_cast<unsigned long long*>(local_target), timeout_ns, status);
}

extern "C" int kfb_peer_allgather(const void* src, void* const* dst_all, void* const* peer_counters, int n_ranks, int M,
                                  int w_local, int ld, int col0, const void* local_counter, void* local_target,
                                  unsigned long long timeout_ns, void* stream) {
  if (int rc = require_sm100()) return rc;
  if (M < 1 || w_local < 1 || col0 < 0 || ld < col0 + w_local)
    return fail(KFB_ERR_INVALID, "peer_allgather: columns [%d, %d) of %d rows do not fit in a row of %d", col0, col0 + w_local, M, ld);
  if (!src || !dst_all) return fail(KFB_ERR_INVALID, "null pointer");
  if (!aligned16(src)) return fail(KFB_ERR_ALIGNMENT, "src must be 16-byte aligned");
  peer::PeerPtrs pp;
  if (int rc = peer::fill(&pp, peer_counters, dst_all, n_ranks)) return rc;
  if (int rc = peer::check_wait_args(local_counter, local_target, timeout_ns)) return rc;
  unsigned int* status = device_status_word();
  if (!status) return fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  return launch_kernel("peer_allgather_kernel", peer::peer_allgather_kernel, dim3(peer::kGatherCtas), dim3(256), 0,
                       (cudaStream_t)stream, pdl_enabled(), static_cast<const __half*>(src), pp, M, w_local, ld, col0,
                       static_cast<const unsigned long long*>(local_counter), static_cast<unsigned long long*>(local_target),
                       timeout_ns, status);
}
