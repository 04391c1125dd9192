// Kernel launch helper with programmatic dependent launch (PDL).
//
// Every kernel of this library is launched through launch_pdl().  With PDL on, a kernel may be scheduled as
// soon as all CTAs of the previous kernel in the stream have executed griddepcontrol.launch_dependents (or
// exited); it then runs its own set-up (barrier init, TMEM allocation, descriptor prefetch, loads of data
// that no earlier kernel writes) and executes griddepcontrol.wait before its first access to anything an
// earlier kernel may have written.  The wait returns once the earlier kernels have completed and their
// writes are visible, so the data flow is the one of a serialised stream; only set-up and launch latency
// overlap.  Rule for kernels in this library: every thread executes griddep_wait() before its first global
// read or write of non-constant data and before it exits.  The captured form is a programmatic edge of the
// CUDA graph.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <utility>

namespace blitz {

inline int& pdl_flag() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("BLITZ_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}

// Set-up that must run once per device and kernel (function attributes are per device; a process may drive
// several GPUs, and several host threads may make the first call at the same time).  `setup` runs with the
// calling thread's current device; devices beyond kMaxDevicesPerProcess are refused.
constexpr int kMaxDevicesPerProcess = 64;
struct PerDeviceOnce {
  std::atomic<int> done[kMaxDevicesPerProcess];
  std::mutex mu;
  PerDeviceOnce() {
    for (auto& d : done) d.store(0, std::memory_order_relaxed);
  }
  template <typename F>
  cudaError_t run(F&& setup) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevicesPerProcess) return cudaErrorInvalidDevice;
    if (done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    std::lock_guard<std::mutex> g(mu);
    if (done[dev].load(std::memory_order_relaxed)) return cudaSuccess;
    e = setup();
    if (e == cudaSuccess) done[dev].store(1, std::memory_order_release);
    return e;
  }
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_flag() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// Same, with the grid cut into thread-block clusters of `cluster_x` consecutive CTAs (1 = no clusters).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, unsigned cluster_x,
                                      cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (cluster_x > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = cluster_x;
    at[n].val.clusterDim.y = 1;
    at[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_flag()) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = at;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// How many clusters of `cluster_x` CTAs of this kernel can be resident on the device at once (0 on error).
template <typename... KArgs>
inline int max_active_clusters(void (*kern)(KArgs...), dim3 block, size_t smem, unsigned cluster_x) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(cluster_x);
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cluster_x;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(kern), &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

}  // namespace blitz
