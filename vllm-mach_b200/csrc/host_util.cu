#include "host_util.h"
#include <cstdarg>
#include <cstring>
#include "ptx.cuh"

namespace mach {

__device__ int g_device_status = 0;

namespace {
thread_local char t_error[512] = "";
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];
int g_smem_optin[kMaxDevices];
int* g_status_ptr[kMaxDevices];
bool g_pdl = true;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return MACH_OK;
  return fail(MACH_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

static int device_attr(int* cache, cudaDeviceAttr attr) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  if (cache[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, attr, dev) == cudaSuccess) cache[dev] = v;
  }
  return cache[dev];
}
int sm_count() {
  const int v = device_attr(g_sm_count, cudaDevAttrMultiProcessorCount);
  return v > 0 ? v : 148;
}
int max_smem_optin() {
  const int v = device_attr(g_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin);
  return v > 0 ? v : 232448;
}

int device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
  return dev < kMaxDeviceSlots ? dev : kMaxDeviceSlots - 1;
}

bool pdl_enabled() { return g_pdl; }
void set_pdl_enabled(bool on) { g_pdl = on; }

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess) g_status_ptr[dev] = (int*)p;
  }
  return g_status_ptr[dev];
}

}  // namespace mach

extern "C" int mach_abi_version(void) { return MACH_ABI_VERSION; }

extern "C" const char* mach_last_error(void) { return mach::t_error; }

extern "C" int mach_device_status(int* status_out, int clear) {
  if (!status_out) return mach::fail(MACH_ERR_INVALID, "device_status: null pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, mach::g_device_status, sizeof(int));
  if (e != cudaSuccess)
    return mach::fail(MACH_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  *status_out = v;
  if (clear && v != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(mach::g_device_status, &zero, sizeof(int));
    if (e != cudaSuccess)
      return mach::fail(MACH_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  }
  return MACH_OK;
}
