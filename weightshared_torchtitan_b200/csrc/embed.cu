// Factorized-embedding row gather and its scatter-add backward. Both are
// HBM-bound byte movers: 16-byte vector accesses, one thread per vector, rows
// coalesced along the embedding dimension.
#include "block_gemm.cuh"
#include "status.cuh"
#include "../../include/wsl.h"
#include <cuda_bf16.h>

namespace wsl {

// G[m, :] = E[tokens[m], :], rows of `vec_per_row` uint4. Tokens outside [0, V)
// produce a zero row (and never an out-of-range read).
__global__ void __launch_bounds__(256)
embed_gather_kernel(const long long* __restrict__ tokens, const uint4* __restrict__ E,
                    uint4* __restrict__ G, long long M, long long V, int vec_per_row) {
  const long long total = M * vec_per_row;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long m = i / vec_per_row;
    const int c = static_cast<int>(i - m * vec_per_row);
    const long long tok = tokens[m];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tok >= 0 && tok < V) v = E[tok * vec_per_row + c];
    G[i] = v;
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// dE[tokens[m], c] += dG[m, c] with fp32 atomics (order of additions is not fixed).
template <typename T>
__global__ void __launch_bounds__(256)
embed_scatter_add_kernel(const long long* __restrict__ tokens, const T* __restrict__ dG,
                         float* dE, long long M, long long V, int r_e) {
  const long long total = M * r_e;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long m = i / r_e;
    const int c = static_cast<int>(i - m * r_e);
    const long long tok = tokens[m];
    if (tok >= 0 && tok < V) atomicAdd(dE + tok * r_e + c, to_f32<T>(dG[i]));
  }
}

int launch_embed_gather(const long long* tokens, const void* E, void* G, long long M, long long V,
                        long long r_e, int elem_bytes, cudaStream_t stream) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!tokens || !E || !G || M <= 0 || V <= 0 || r_e <= 0) return WSL_ERR_BAD_ARG;
  const long long row_bytes = r_e * elem_bytes;
  if ((row_bytes % 16) != 0 || (reinterpret_cast<uintptr_t>(E) & 15u) ||
      (reinterpret_cast<uintptr_t>(G) & 15u))
    return WSL_ERR_ALIGN;
  const int vec = static_cast<int>(row_bytes / 16);
  const long long total = M * vec;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(device_sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  embed_gather_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      tokens, static_cast<const uint4*>(E), static_cast<uint4*>(G), M, V, vec);
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

int launch_embed_scatter_add(const long long* tokens, const void* dG, float* dE, long long M,
                             long long V, long long r_e, int is_f32, cudaStream_t stream) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!tokens || !dG || !dE || M <= 0 || V <= 0 || r_e <= 0) return WSL_ERR_BAD_ARG;
  if (r_e > 0x7fffffffLL) return WSL_ERR_TOO_LARGE;
  const long long total = M * r_e;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(device_sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (is_f32)
    embed_scatter_add_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        tokens, static_cast<const float*>(dG), dE, M, V, static_cast<int>(r_e));
  else
    embed_scatter_add_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        tokens, static_cast<const __nv_bfloat16*>(dG), dE, M, V, static_cast<int>(r_e));
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

}  // namespace wsl
