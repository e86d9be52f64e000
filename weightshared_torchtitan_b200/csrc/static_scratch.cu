// wsl_lora_linear_bwd_dw_noalloc: the weight-gradient kernel for callers that cannot
// hand the library any scratch memory.
//
// wsl_lora_linear_bwd_dw splits the token contraction of small weight matrices across
// CTAs and needs an fp32 workspace for the partial sums, which its caller normally takes
// from an allocator. Some callers have no allocator to ask at that point: code running
// inside a region where cudaMalloc is forbidden or would deadlock (a stream-ordered
// pipeline whose memory pool is fixed up front, a callback, a process whose device memory
// was handed out entirely at start-up), or a host language binding that only owns the
// tensors it was given. For them the partial sums live in a fixed array that is part of
// the library image itself.
//
// The array is a device global: the name below, used in HOST code, is only a host-side
// handle of that symbol, not a device address. The device address is fetched once per
// device with cudaGetSymbolAddress (with that device current) and that pointer is what
// the kernels receive.
#include "block_gemm.cuh"
#include "status.cuh"
#include "../../include/wsl.h"

namespace wsl {

void build_bwd_dw_desc(GemmDesc& g, const void* dY, long long lddy, const void* U, long long ldu,
                       const void* x, long long ldx, const void* T, long long ldt, float* dW,
                       float* dA, float* dB, long long M, long long N, long long K, long long r);

constexpr unsigned long long kStaticScratchBytes = WSL_NOALLOC_SCRATCH_BYTES;

// Every device that loads this library holds these 64 MiB until the process exits.
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

static float* g_static_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device, resolved on first use.
static int static_scratch_address(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return WSL_ERR_DEVICE;
  }
  if (dev < 0 || dev >= kMaxDevices) return WSL_ERR_TOO_LARGE;
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return WSL_ERR_CUDA;
    }
    g_static_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_scratch_ptr[dev];
  return WSL_OK;
}

}  // namespace wsl

extern "C" int wsl_lora_linear_bwd_dw_noalloc(const void* dY, long long lddy, const void* U,
                                              long long ldu, const void* x, long long ldx,
                                              const void* T, long long ldt, float* dW, float* dA,
                                              float* dB, long long M, long long N, long long K,
                                              long long r, void* stream) {
  using namespace wsl;
  if (M <= 0 || N <= 0 || K <= 0 || r < 0) return WSL_ERR_BAD_ARG;
  if (r == 0 && (dA || dB)) return WSL_ERR_BAD_ARG;
  if (!dW && !dA && !dB) return WSL_ERR_BAD_ARG;
  if ((dW || dB) && !dY) return WSL_ERR_BAD_ARG;
  if ((dW || dA) && !x) return WSL_ERR_BAD_ARG;
  if (dA && !U) return WSL_ERR_BAD_ARG;
  if (dB && !T) return WSL_ERR_BAD_ARG;
  // Size limit: a two-way split of all requested outputs must fit the fixed array.
  long long out_elems = 0;
  if (dW) out_elems += N * K;
  if (dB) out_elems += N * r;
  if (dA) out_elems += r * K;
  if (static_cast<unsigned long long>(out_elems) * 2ull * sizeof(float) > kStaticScratchBytes)
    return WSL_ERR_TOO_LARGE;
  int st = device_check();
  if (st != WSL_OK) return st;
  float* scratch = nullptr;
  st = static_scratch_address(&scratch);
  if (st != WSL_OK) return st;

  GemmDesc g = {};
  build_bwd_dw_desc(g, dY, lddy, U, ldu, x, ldx, T, ldt, dW, dA, dB, M, N, K, r);
  g.workspace = scratch;
  g.workspace_bytes = static_cast<size_t>(kStaticScratchBytes);
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}
