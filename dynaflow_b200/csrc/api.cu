// Library-wide entry points of the C ABI: version, error text, wait deadline,
// status block transfer.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/dynaflow_b200.h"
#include "host_util.h"

namespace df {

static thread_local char g_error[512] = "";
static std::atomic<unsigned long long> g_timeout_ns{2000ull * 1000ull * 1000ull};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

unsigned long long timeout_ns() { return g_timeout_ns.load(std::memory_order_relaxed); }

PFN_encodeTiled get_encode_tiled() {
  static std::once_flag once;
  static PFN_encodeTiled fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<PFN_encodeTiled>(p);
    (void)cudaGetLastError();
  });
  if (fn == nullptr) set_error("the CUDA driver does not provide cuTensorMapEncodeTiled");
  return fn;
}

}  // namespace df

extern "C" {

int df_version(void) { return DF_ABI_VERSION; }

const char* df_last_error(void) { return df::g_error; }

int df_set_timeout_ms(int ms) {
  if (ms <= 0) return df::fail(DF_EINVAL, "timeout must be positive (got %d ms)", ms);
  df::g_timeout_ns.store(static_cast<unsigned long long>(ms) * 1000000ull, std::memory_order_relaxed);
  return DF_OK;
}

int df_sm_count(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return df::fail(DF_ECUDA, "cudaGetDevice failed (no CUDA device?)");
  }
  static int cached[64] = {0};
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return df::fail(DF_ECUDA, "cudaDeviceGetAttribute failed");
  }
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

int df_status_read(const df_status_t* dev_status, df_status_t* host_out, void* stream) {
  if (dev_status == nullptr || host_out == nullptr) return df::fail(DF_EINVAL, "NULL status pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(host_out, dev_status, sizeof(df_status_t), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return df::fail(DF_ECUDA, "status read: %s", cudaGetErrorString(e));
  return DF_OK;
}

int df_status_clear(df_status_t* dev_status, void* stream) {
  if (dev_status == nullptr) return df::fail(DF_EINVAL, "NULL status pointer");
  cudaError_t e = cudaMemsetAsync(dev_status, 0, sizeof(df_status_t), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return df::fail(DF_ECUDA, "status clear: %s", cudaGetErrorString(e));
  return DF_OK;
}

}  // extern "C"
