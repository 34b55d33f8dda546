// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include "../../include/mach_b200.h"

namespace mach {

// Records `msg` (printf-style) as the calling thread's last error and returns `code`.
int fail(int code, const char* fmt, ...);
// cudaGetLastError() after a launch -> MACH_OK / MACH_ERR_CUDA.
int check_launch(const char* what);
// Index of the current device for per-device host caches (function attributes, occupancy
// queries, symbol addresses are all per device), clamped to [0, kMaxDeviceSlots).
constexpr int kMaxDeviceSlots = 64;
int device_slot();
// Number of SMs of the current device (cached per device).
int sm_count();
// Opt-in shared memory limit per block of the current device.
int max_smem_optin();

// Raises the kernel's dynamic shared memory limit to the device's opt-in maximum (once per
// kernel and device). False if the attribute cannot be set.
bool ensure_smem_optin(const void* kernel);
// How many clusters of `cluster_y` CTAs (block of `threads`, `smem_bytes` of dynamic shared
// memory each) the current device keeps resident at once, as cudaOccupancyMaxActiveClusters
// reports it; cached. A cluster lives inside one GPC, so this can be fewer than SMs / cluster_y.
int64_t active_clusters(const void* kernel, int threads, int smem_bytes, int cluster_y);

// Device address of the status word of the current device (NULL if it cannot be resolved).
int* device_status_ptr();

// Whether kernels of the dense path are launched with programmatic dependent launch.
bool pdl_enabled();
void set_pdl_enabled(bool on);

// cudaLaunchKernelEx with an optional cluster (y-dimension), the programmatic-serialisation
// attribute and the cooperative attribute (the whole grid co-resident, or the launch fails).
template <typename... KArgs, typename... Args>
cudaError_t launch_ex_attrs(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, dim3 cluster, bool pdl, bool cooperative,
                            Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[3];
  int n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cooperative) {
    attr[n].id = cudaLaunchAttributeCooperative;
    attr[n].val.cooperative = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                      cudaStream_t stream, dim3 cluster, bool pdl, Args&&... args) {
  return launch_ex_attrs(kernel, grid, block, smem, stream, cluster, pdl, false,
                         static_cast<Args&&>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace mach
