// Process-wide state of the library that every kernel file shares (one translation unit, so
// plain definitions are enough): the device-side status words (see wsl_poll_status()), what
// is known about each CUDA device, and the run-time options (see wsl_set_option()).
#pragma once
#include <cuda_runtime.h>

namespace wsl {
__device__ int g_wsl_status[4];

constexpr int kMaxDevices = 64;

// Everything cached about a device is kept per device index: the sm_100 check, the SM count,
// the number of co-resident CTA pairs of the paired GEMM, and (in the launchers) whether a
// kernel's dynamic shared memory limit has been raised there, which is a per-device setting.
struct DeviceInfo {
  int state;          // 0 unknown, 1 sm_100, -1 unusable
  int sms;
  int max_clusters;   // co-resident CTA pairs of the paired GEMM variant (0 = not asked yet)
};

int current_device_index();            // index of the current device, or -1
DeviceInfo* current_device_info();     // nullptr when there is no usable current device
int device_check();      // WSL_OK when the current device is sm_100
int device_sm_count();   // SMs of the current device that launches may fill (all minus the reserved
                         // ones); 0 when device_check() fails

// Run-time options. Initial values come from the environment, read ONCE when the library is
// first used (WSL_PAIR, WSL_ROW_STAGED, WSL_WAIT_LIMIT_MS, WSL_SPLIT_TAIL,
// WSL_DEPENDENT_LAUNCH); afterwards wsl_set_option()
// changes them. Launch paths read this struct, never the environment.
struct Options {
  int pair_tiles;                      // 1: large GEMMs run on CTA pairs (cta_group::2)
  int row_staged;                      // 1: row kernels use their staged (bulk-copy) variants
  int stall_producer;                  // 1: producers never fill their rings (bounded-wait tests)
  unsigned long long wait_limit_ns;    // bound of every device-side wait
  int reserved_sms;                    // SMs the persistent kernels leave free (collective overlap)
  int grid_waves;                      // GEMM grids up to this many times the co-resident CTAs (0 = by launch)
  int profile_bits;                    // only honoured in builds with WSL_PROFILE_SWITCHES
  int merge_simt;                      // 1: W + s B A on the CUDA cores instead of the block GEMM
  int dependent_launch;                // 1: GEMM launches may start while the kernel before them drains
  int split_tail;                      // 1: launches of long tiles may end with a split tail (see SplitPlan)
};
Options& options();

// Launch of a kernel that calls grid_dep_wait() before its first access to global memory:
// with the option on it carries the programmatic-stream-serialization attribute, so its CTAs
// may take SMs and set themselves up while the kernel before it in the stream drains.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
}  // namespace wsl
