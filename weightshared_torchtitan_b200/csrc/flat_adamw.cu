// Optimizer step over the flat fp32 arenas (parameters, gradients, AdamW moments laid out
// alike): global-norm clipping, AdamW and the refresh of the bf16 compute copy in ONE pass
// over memory, after one pass over the gradients for the norm.
//   pass 1  grad_sumsq_kernel : per-block partial sums of g^2 (fixed grid, fixed order)
//   pass 2  adamw_flat_kernel : every block first folds the partials in the same order (the
//           norm is bit-identical in all blocks and from run to run), then per element
//             g' = g * min(1, max_norm / (norm + 1e-6))
//             m  = b1 m + (1 - b1) g' ;  v = b2 v + (1 - b2) g'^2
//             p  = p (1 - lr wd) - (lr / bc1) m / (sqrt(v) / sqrt(bc2) + eps)
//           and writes p again as bf16 into the compute copy.
// HBM-bound: 16 B read + 12 B (+2 B) written per parameter. The arithmetic is that of
// torch.optim.AdamW (decoupled weight decay, bias corrections bc1 = 1 - b1^t, bc2 = 1 - b2^t
// passed by the host) after torch.nn.utils.clip_grad_norm_.
#include "block_gemm.cuh"
#include "status.cuh"
#include "../../include/wsl.h"
#include <cuda_bf16.h>
#include <cstdint>

namespace wsl {

constexpr int SUMSQ_THREADS = 256;

__global__ void __launch_bounds__(SUMSQ_THREADS)
grad_sumsq_kernel(const float4* __restrict__ g, long long n4, float* __restrict__ partials) {
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(SUMSQ_THREADS) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * SUMSQ_THREADS) {
    const float4 v = g[i];
    acc = fmaf(v.x, v.x, acc);
    acc = fmaf(v.y, v.y, acc);
    acc = fmaf(v.z, v.z, acc);
    acc = fmaf(v.w, v.w, acc);
  }
  __shared__ float warp_part[SUMSQ_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < SUMSQ_THREADS / 32; ++w) s += warp_part[w];
    partials[blockIdx.x] = s;
  }
}

struct AdamwArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, max_norm;
};

__global__ void __launch_bounds__(256)
adamw_flat_kernel(float4* __restrict__ p, const float4* __restrict__ g, float4* __restrict__ m,
                  float4* __restrict__ v, uint2* __restrict__ copy, long long n4,
                  const float* __restrict__ partials, int n_partials, const AdamwArgs a) {
  __shared__ float scale_s;
  if (threadIdx.x < 32) {
    // every block folds the partials in the same order: lane l takes l, l + 32, ...
    float s = 0.f;
    for (int i = threadIdx.x; i < n_partials; i += 32) s += partials[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) {
      float sc = 1.f;
      if (a.max_norm > 0.f && n_partials > 0) sc = fminf(1.f, a.max_norm / (sqrtf(s) + 1e-6f));
      scale_s = sc;
    }
  }
  __syncthreads();
  const float sc = scale_s;
  const float decay = 1.f - a.lr * a.weight_decay;
  const float step = a.lr / a.bias_corr1;
  const float inv_sqrt_bc2 = rsqrtf(a.bias_corr2);
  const float omb1 = 1.f - a.beta1, omb2 = 1.f - a.beta2;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += gridDim.x * 256ll) {
    const float4 gv = g[i];
    float4 pv = p[i], mv = m[i], vv = v[i];
    const float gs[4] = {gv.x * sc, gv.y * sc, gv.z * sc, gv.w * sc};
    float* pp = reinterpret_cast<float*>(&pv);
    float* mp = reinterpret_cast<float*>(&mv);
    float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mp[e] = fmaf(a.beta1, mp[e], omb1 * gs[e]);
      vp[e] = fmaf(a.beta2, vp[e], omb2 * gs[e] * gs[e]);
      const float denom = sqrtf(vp[e]) * inv_sqrt_bc2 + a.eps;
      pp[e] = pp[e] * decay - step * (mp[e] / denom);
    }
    p[i] = pv;
    m[i] = mv;
    v[i] = vv;
    if (copy != nullptr) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pv.x, pv.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(pv.z, pv.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      copy[i] = pk;
    }
  }
}

static bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_grad_sumsq(const float* g, long long n, float* partials, cudaStream_t s) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!g || !partials || n <= 0) return WSL_ERR_BAD_ARG;
  if ((n % 4) != 0 || !a16(g)) return WSL_ERR_ALIGN;
  grad_sumsq_kernel<<<WSL_SUMSQ_PARTIALS, SUMSQ_THREADS, 0, s>>>(reinterpret_cast<const float4*>(g), n / 4,
                                                                 partials);
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

int launch_adamw_flat(float* p, const float* g, float* m, float* v, void* copy, long long n,
                      const AdamwArgs& a, const float* partials, int n_partials, cudaStream_t s) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!p || !g || !m || !v || n <= 0 || a.bias_corr1 <= 0.f || a.bias_corr2 <= 0.f) return WSL_ERR_BAD_ARG;
  if (a.max_norm > 0.f && (!partials || n_partials <= 0)) return WSL_ERR_BAD_ARG;
  if ((n % 4) != 0 || !a16(p) || !a16(g) || !a16(m) || !a16(v) ||
      (copy && (reinterpret_cast<uintptr_t>(copy) & 7u) != 0))
    return WSL_ERR_ALIGN;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = 16ll * device_sm_count();
  if (blocks > cap) blocks = cap;
  adamw_flat_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      reinterpret_cast<float4*>(p), reinterpret_cast<const float4*>(g), reinterpret_cast<float4*>(m),
      reinterpret_cast<float4*>(v), static_cast<uint2*>(copy), n / 4, partials,
      a.max_norm > 0.f ? n_partials : 0, a);
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

}  // namespace wsl
