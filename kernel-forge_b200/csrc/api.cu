// Library-wide entry points: version, per-thread error text, device queries.
#include "common.cuh"

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

int make_tmap_2d_plain(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                       uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  if (int rc = resolve_encoder()) return rc;
  if (elem_bytes != 4) return fail(KFB_ERR_INVALID, "make_tmap_2d_plain handles 32-bit elements");
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
  return KFB_OK;
}

int make_tmap_4d_sw128(CUtensorMap* out, const void* base, int dtype, const uint64_t dims[4],
                       const uint64_t strides_bytes[3], const uint32_t box[4]) {
  if (int rc = resolve_encoder()) return rc;
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

extern "C" int kfb_version(void) { return 100; }

extern "C" const char* kfb_last_error(void) { return kfb::error_buffer(); }
