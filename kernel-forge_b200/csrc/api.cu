// Library-wide entry points: version, per-thread error text, device queries, the per-device status word
// (read / reset / a self-test that lets one bounded wait run out) and the cache of encoded TMA tensor maps.
#include "common.cuh"
#include "sm100.cuh"

#include <atomic>
#include <cstring>
#include <mutex>

namespace kfb {

char* error_buffer() {
  static thread_local char buf[kErrorBufferBytes] = {0};
  return buf;
}

namespace {
std::mutex g_dev_mutex;
int g_sm_count[64];
int g_cc_major[64];
bool g_dev_known[64];

int query_device(int* sms, int* major) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_dev_known[dev]) {
    int s = 0, m = 0;
    if (cudaDeviceGetAttribute(&s, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&m, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
    g_sm_count[dev] = s;
    g_cc_major[dev] = m;
    g_dev_known[dev] = true;
  }
  *sms = g_sm_count[dev];
  *major = g_cc_major[dev];
  return 0;
}
}  // namespace

int sm_count() {
  int s = 0, m = 0;
  return query_device(&s, &m) == 0 ? s : 148;
}

int require_sm100() {
  int s = 0, m = 0;
  if (query_device(&s, &m) != 0) return fail(KFB_ERR_CUDA, "no usable CUDA device is current");
  if (m != 10)
    return fail(KFB_ERR_DEVICE, "kfb200 kernels are built for sm_100a only; current device is sm_%dx", m);
  return KFB_OK;
}

}  // namespace kfb

namespace kfb {

__device__ unsigned int g_status_word = 0;

namespace {
unsigned int* g_status_ptr[64];
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

unsigned int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<unsigned int*>(p);
  }
  return g_status_ptr[dev];
}

namespace {
int resolve_encoder() {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
      return fail(KFB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  return KFB_OK;
}
}  // namespace

namespace {
// Per-thread cache of encoded tensor maps.  An encoded map depends only on the arguments of the encoder (base
// address, element type, extents, strides, box, swizzle), never on the memory contents, so a repeated call with the
// same tensor (a decode loop over one KV cache, a benchmark loop, a layer's weight) reuses the 128-byte map instead
// of calling the driver again.  Thread-local: no lock on the launch path.  Round-robin replacement.
struct TmapKey {
  const void* base;
  uint64_t dims[4];
  uint64_t strides[3];
  uint32_t box[4];
  uint32_t kind;  // element type, rank and swizzle mode
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapCacheEntries = 32;
struct TmapCache {
  TmapEntry e[kTmapCacheEntries];
  int next = 0;
  TmapCache() { std::memset(e, 0, sizeof(e)); }
};
TmapCache& tmap_cache() {
  static thread_local TmapCache c;
  return c;
}
const CUtensorMap* tmap_lookup(const TmapKey& k) {
  TmapCache& c = tmap_cache();
  for (int i = 0; i < kTmapCacheEntries; ++i)
    if (c.e[i].used && std::memcmp(&c.e[i].key, &k, sizeof(TmapKey)) == 0) return &c.e[i].map;
  return nullptr;
}
void tmap_insert(const TmapKey& k, const CUtensorMap& m) {
  TmapCache& c = tmap_cache();
  TmapEntry& slot = c.e[c.next];
  c.next = (c.next + 1) % kTmapCacheEntries;
  slot.key = k;
  slot.map = m;
  slot.used = true;
}
}  // namespace

int make_tmap_2d_plain(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                       uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  if (int rc = resolve_encoder()) return rc;
  if (elem_bytes != 4) return fail(KFB_ERR_INVALID, "make_tmap_2d_plain handles 32-bit elements");
  TmapKey key;
  std::memset(&key, 0, sizeof(key));  // padding bytes take part in the comparison
  key.base = base;
  key.dims[0] = inner; key.dims[1] = outer;
  key.strides[0] = row_bytes;
  key.box[0] = box_inner; key.box[1] = box_outer;
  key.kind = 0x200u | (swizzle128 ? 1u : 0u);
  if (const CUtensorMap* hit = tmap_lookup(key)) {
    *out = *hit;
    return KFB_OK;
  }
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstr[1] = {row_bytes};
  cuuint32_t bdim[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), gdim, gstr, bdim, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(KFB_ERR_CUDA, "cuTensorMapEncodeTiled (2-D) failed with CUresult %d (dims %llu,%llu)", (int)r,
                (unsigned long long)inner, (unsigned long long)outer);
  tmap_insert(key, *out);
  return KFB_OK;
}

int make_tmap_4d_sw128(CUtensorMap* out, const void* base, int dtype, const uint64_t dims[4],
                       const uint64_t strides_bytes[3], const uint32_t box[4]) {
  if (int rc = resolve_encoder()) return rc;
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  for (int i = 0; i < 4; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i < 3; ++i) key.strides[i] = strides_bytes[i];
  key.kind = 0x400u | (dtype == KFB_BF16 ? 1u : 0u);
  if (const CUtensorMap* hit = tmap_lookup(key)) {
    *out = *hit;
    return KFB_OK;
  }
  cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstr[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bdim[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == KFB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(out, dt, 4, const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(KFB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu,%llu,%llu,%llu)", (int)r,
                (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
                (unsigned long long)dims[3]);
  tmap_insert(key, *out);
  return KFB_OK;
}

}  // namespace kfb

extern "C" int kfb_device_status(unsigned int* out) {
  if (!out) return kfb::fail(KFB_ERR_INVALID, "null pointer");
  unsigned int* p = kfb::device_status_word();
  if (!p) return kfb::fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  KFB_CUDA_TRY(cudaMemcpy(out, p, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  return KFB_OK;
}

extern "C" int kfb_device_status_reset(void* stream) {
  unsigned int* p = kfb::device_status_word();
  if (!p) return kfb::fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  KFB_CUDA_TRY(cudaMemsetAsync(p, 0, sizeof(unsigned int), (cudaStream_t)stream));
  return KFB_OK;
}

namespace kfb {
namespace {
// One warp waits on an mbarrier that nothing ever arrives on, through the same bounded-wait helper every kernel of
// the library uses, with the limit given by the caller.  The wait runs out, the code lands in the status word, the
// kernel returns normally.  Nothing faults, traps or spins without a limit.
constexpr uint32_t kSelfTestCode = 0x601;
__global__ void wait_expiry_selftest_kernel(unsigned int* status, unsigned long long timeout_ns, unsigned int* outcome) {
  __shared__ uint64_t bar;
  __shared__ uint32_t cta_word;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    cta_word = 0;
    sm100::fence_mbar_init();
  }
  __syncthreads();
  const sm100::AbortCtx ctx{&cta_word, status, timeout_ns};
  const bool completed = sm100::mbar_wait_warp(&bar, 0, ctx, kSelfTestCode);
  if (threadIdx.x == 0) *outcome = completed ? 1u : 2u;  // 2 = the wait gave up, as it must
}
}  // namespace
}  // namespace kfb

extern "C" int kfb_selftest_wait_expiry(unsigned long long timeout_ns, unsigned int* outcome_dev, void* stream) {
  if (int rc = kfb::require_sm100()) return rc;
  if (!outcome_dev) return kfb::fail(KFB_ERR_INVALID, "null pointer");
  if (timeout_ns < 1000ull || timeout_ns > 100000000ull)
    return kfb::fail(KFB_ERR_INVALID, "the self-test takes a limit between 1 us and 100 ms, got %llu ns", timeout_ns);
  unsigned int* p = kfb::device_status_word();
  if (!p) return kfb::fail(KFB_ERR_CUDA, "cannot resolve the device status word");
  kfb::wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p, timeout_ns, outcome_dev);
  KFB_LAUNCH_CHECK("wait_expiry_selftest_kernel");
  return KFB_OK;
}

namespace kfb {
namespace {
std::atomic<int> g_pdl{0};
}
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
}  // namespace kfb

extern "C" int kfb_set_programmatic_launch(int enable) { return kfb::g_pdl.exchange(enable ? 1 : 0); }

extern "C" int kfb_version(void) { return 200; }

extern "C" const char* kfb_last_error(void) { return kfb::error_buffer(); }
