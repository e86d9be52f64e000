// fp32 correctness mode: a plain shared-memory-tiled CUDA-core GEMM with
// arbitrary element strides, so every product on the path (NT, NN, TN) is one
// kernel. fp32 FMA throughout: tensor cores would round the inputs to 10-bit
// mantissas (tf32), which cannot meet the 1e-5 bar of the fp32 configuration.
//   C[i,j] (op)= alpha * sum_k A[i*sai + k*sak] * B[j*sbj + k*sbk]
#include "block_gemm.cuh"
#include "status.cuh"
#include "../../include/wsl.h"

namespace wsl {

constexpr int ST = 64;    // output tile edge
constexpr int SK = 16;    // contraction slice

__global__ void __launch_bounds__(256)
simt_gemm_f32_kernel(const float* __restrict__ A, long long sai, long long sak,
                     const float* __restrict__ B, long long sbj, long long sbk, float* C,
                     long long ldc, int M, int N, int K, float alpha, int accumulate) {
  __shared__ float As[SK][ST + 1];
  __shared__ float Bs[SK][ST + 1];
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;
  const int i0 = blockIdx.y * ST;
  const int j0 = blockIdx.x * ST;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

  for (int k0 = 0; k0 < K; k0 += SK) {
    for (int e = threadIdx.x; e < ST * SK; e += 256) {
      // Walk the contiguous direction fastest for whichever stride is 1.
      int ii, kk;
      if (sak == 1) { kk = e % SK; ii = e / SK; } else { ii = e % ST; kk = e / ST; }
      const int gi = i0 + ii, gk = k0 + kk;
      As[kk][ii] = (gi < M && gk < K) ? A[gi * sai + gk * sak] : 0.f;
      int jj, kb;
      if (sbk == 1) { kb = e % SK; jj = e / SK; } else { jj = e % ST; kb = e / ST; }
      const int gj = j0 + jj, gkb = k0 + kb;
      Bs[kb][jj] = (gj < N && gkb < K) ? B[gj * sbj + gkb * sbk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) av[a] = As[kk][ty * 4 + a];
#pragma unroll
      for (int b = 0; b < 4; ++b) bv[b] = Bs[kk][tx * 4 + b];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int gi = i0 + ty * 4 + a;
    if (gi >= M) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int gj = j0 + tx * 4 + b;
      if (gj >= N) continue;
      float* c = C + gi * ldc + gj;
      const float v = alpha * acc[a][b];
      *c = accumulate ? (*c + v) : v;
    }
  }
}

int launch_simt_gemm_f32(const float* A, long long sai, long long sak, const float* B,
                         long long sbj, long long sbk, float* C, long long ldc, long long M,
                         long long N, long long K, float alpha, int accumulate,
                         cudaStream_t stream) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return WSL_ERR_BAD_ARG;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return WSL_ERR_TOO_LARGE;
  dim3 grid(static_cast<unsigned>((N + ST - 1) / ST), static_cast<unsigned>((M + ST - 1) / ST));
  if (grid.y > 65535u) return WSL_ERR_TOO_LARGE;
  simt_gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, sai, sak, B, sbj, sbk, C, ldc,
                                                 static_cast<int>(M), static_cast<int>(N),
                                                 static_cast<int>(K), alpha, accumulate);
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

}  // namespace wsl
