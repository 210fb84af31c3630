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

extern "C" int kfb_version(void) { return 100; }

extern "C" const char* kfb_last_error(void) { return kfb::error_buffer(); }
