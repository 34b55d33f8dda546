#include "host_util.h"
#include <cstdarg>
#include <cstring>
#include <mutex>
#include <vector>
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

namespace {
std::mutex g_occ_mu;
struct OptinEntry { const void* kernel; int dev; };
struct OccEntry { const void* kernel; int dev, threads, smem, cluster; int64_t clusters; };
std::vector<OptinEntry> g_optin;
std::vector<OccEntry> g_occ;
}  // namespace

bool ensure_smem_optin(const void* kernel) {
  const int dev = device_slot();
  std::lock_guard<std::mutex> lock(g_occ_mu);
  for (const OptinEntry& e : g_optin)
    if (e.kernel == kernel && e.dev == dev) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin()) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  g_optin.push_back({kernel, dev});
  return true;
}

int64_t active_clusters(const void* kernel, int threads, int smem_bytes, int cluster_y) {
  const int dev = device_slot();
  {
    std::lock_guard<std::mutex> lock(g_occ_mu);
    for (const OccEntry& e : g_occ)
      if (e.kernel == kernel && e.dev == dev && e.threads == threads && e.smem == smem_bytes &&
          e.cluster == cluster_y)
        return e.clusters;
  }
  // Fallback when the query is refused: whole SMs, one CTA each.
  int64_t clusters = sm_count() / std::max(1, cluster_y);
  if (ensure_smem_optin(kernel)) {
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3((unsigned)sm_count(), (unsigned)cluster_y, 1);
    q.blockDim = dim3((unsigned)threads);
    q.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 1;
    qa[0].val.clusterDim.y = (unsigned)cluster_y;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) == cudaSuccess && n > 0) clusters = n;
    else (void)cudaGetLastError();
  }
  std::lock_guard<std::mutex> lock(g_occ_mu);
  g_occ.push_back({kernel, dev, threads, smem_bytes, cluster_y, clusters});
  return clusters;
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
