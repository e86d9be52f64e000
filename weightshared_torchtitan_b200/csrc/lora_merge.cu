// W_eff = W + s * B * A rounded once to bf16: a layer's effective weight, [N, K], from the
// shared W[N, K] and the adapter factors B[N, r], A[r, K]. Used by the backward pass, where
// dX = dY * W_eff replaces a rank-r detour through dY * B. Up to WSL_MAX_PROJ projections of
// one input width go in one launch.
//
// Two implementations. The default runs the rank-r product on the tensor cores (one k-block
// per tile of the block GEMM: operands B, K-major, and A, MN-major) and adds W in the
// epilogue from tiles that TMA brings into the staging buffers, so the pass is bound by the
// 2 * 2 * N * K bytes it has to move. The CUDA-core kernel below (r FMAs per element, issue
// bound from r = 32 up) stays selectable with option MERGE_SIMT, for comparison.
#include "block_gemm.cuh"
#include "status.cuh"
#include "../../include/wsl.h"
#include <cuda_bf16.h>
#include <cstdint>

namespace wsl {

// A thread owns ROWS rows x 8 columns of W; the unpacked A values are shared by its rows, so
// 4 rows cost fewer instructions per element, 2 rows give small matrices twice the threads.

struct MergeProj {
  const __nv_bfloat16* W;
  const __nv_bfloat16* A;
  const __nv_bfloat16* B;
  __nv_bfloat16* out;
  long long N;
  long long begin;   // first work item of this projection (item = ROWS rows x 8 columns)
};
struct MergeParams {
  MergeProj proj[WSL_MAX_PROJ];
  int nproj;
  int K8;            // K / 8
  long long total;   // work items over all projections
  float s;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(u[e] << 16);
    f[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
  }
}

// R = rank (multiple of 8). Work item i of a projection: rows [ROWS * (i / K8), +ROWS), columns
// [8 * (i % K8), +8); consecutive threads take consecutive column groups of the same rows.
template <int R, int ROWS>
__global__ void __launch_bounds__(256)
lora_merge_kernel(const __grid_constant__ MergeParams mp) {
  constexpr int MERGE_ROWS = ROWS;
  for (long long gi = blockIdx.x * 256ll + threadIdx.x; gi < mp.total; gi += gridDim.x * 256ll) {
    int p = 0;
    while (p + 1 < mp.nproj && gi >= mp.proj[p + 1].begin) ++p;
    const MergeProj& P = mp.proj[p];
    const long long i = gi - P.begin;
    const long long n0 = (i / mp.K8) * MERGE_ROWS;
    const int k8 = static_cast<int>(i % mp.K8);
    const int K = mp.K8 * 8;
    // the row of W is needed last but asked for first: its latency hides behind the products
    uint4 wv[MERGE_ROWS];
#pragma unroll
    for (int q = 0; q < MERGE_ROWS; ++q) {
      const long long n = n0 + q < P.N ? n0 + q : P.N - 1;
      wv[q] = *reinterpret_cast<const uint4*>(P.W + n * K + k8 * 8);
    }
    float d[MERGE_ROWS][8];
#pragma unroll
    for (int q = 0; q < MERGE_ROWS; ++q)
#pragma unroll
      for (int e = 0; e < 8; ++e) d[q][e] = 0.f;
#pragma unroll
    for (int j0 = 0; j0 < R; j0 += 8) {
      float b[MERGE_ROWS][8];
#pragma unroll
      for (int q = 0; q < MERGE_ROWS; ++q) {
        const long long n = n0 + q < P.N ? n0 + q : P.N - 1;
        unpack8(*reinterpret_cast<const uint4*>(P.B + n * R + j0), b[q]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a[8];
        unpack8(*reinterpret_cast<const uint4*>(P.A + static_cast<long long>(j0 + j) * K + k8 * 8), a);
#pragma unroll
        for (int q = 0; q < MERGE_ROWS; ++q)
#pragma unroll
          for (int e = 0; e < 8; ++e) d[q][e] = fmaf(b[q][j], a[e], d[q][e]);
      }
    }
#pragma unroll
    for (int q = 0; q < MERGE_ROWS; ++q) {
      if (n0 + q < P.N) {
        float w[8];
        unpack8(wv[q], w);
        uint4 ov;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(fmaf(mp.s, d[q][2 * e], w[2 * e]),
                                                   fmaf(mp.s, d[q][2 * e + 1], w[2 * e + 1]));
          ou[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(P.out + (n0 + q) * K + k8 * 8) = ov;
      }
    }
  }
}

int launch_lora_merge(int nproj, const void* const* W, const void* const* A, const void* const* B,
                      void* const* out, const long long* N, long long K, long long r, float s,
                      cudaStream_t stream) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (nproj < 1 || nproj > WSL_MAX_PROJ || !W || !A || !B || !out || !N || K <= 0 || r <= 0)
    return WSL_ERR_BAD_ARG;
  if ((K % 8) != 0) return WSL_ERR_ALIGN;
  if (K > 0x7fffffffLL) return WSL_ERR_TOO_LARGE;
  if (r != 8 && r != 16 && r != 32 && r != 64 && r != 128) return WSL_ERR_TOO_LARGE;
  if (!options().merge_simt) {
    // out_p[N_p, K] = s * B_p[N_p, r] . A_p[r, K] + W_p on the block GEMM
    GemmDesc g = {};
    g.a_mn = false;
    g.b_mn = true;
    g.nseg = 1;
    g.seg_k[0] = static_cast<int>(r);
    g.nregion = nproj;
    for (int p = 0; p < nproj; ++p) {
      if (!W[p] || !A[p] || !B[p] || !out[p] || N[p] <= 0) return WSL_ERR_BAD_ARG;
      RegionDesc& rd = g.region[p];
      rd.a[0].ptr = B[p];
      rd.a[0].rows = N[p];
      rd.a[0].cols = r;
      rd.a[0].ld = r;
      rd.b[0].ptr = A[p];
      rd.b[0].rows = r;
      rd.b[0].cols = K;
      rd.b[0].ld = K;
      rd.mo = N[p];
      rd.no = K;
      rd.out = out[p];
      rd.ld_out = K;
      rd.mode = kEpiStoreBf16;
      rd.alpha = s;
      rd.addend = W[p];
      rd.ld_addend = K;
    }
    return launch_block_gemm(g, stream);
  }
  MergeParams mp;
  mp.nproj = nproj;
  mp.K8 = static_cast<int>(K / 8);
  mp.s = s;
  long long total = 0;
  for (int p = 0; p < nproj; ++p) {
    if (!W[p] || !A[p] || !B[p] || !out[p] || N[p] <= 0) return WSL_ERR_BAD_ARG;
    if (((reinterpret_cast<uintptr_t>(W[p]) | reinterpret_cast<uintptr_t>(A[p]) |
          reinterpret_cast<uintptr_t>(B[p]) | reinterpret_cast<uintptr_t>(out[p])) & 15u) != 0)
      return WSL_ERR_ALIGN;
    mp.proj[p].W = static_cast<const __nv_bfloat16*>(W[p]);
    mp.proj[p].A = static_cast<const __nv_bfloat16*>(A[p]);
    mp.proj[p].B = static_cast<const __nv_bfloat16*>(B[p]);
    mp.proj[p].out = static_cast<__nv_bfloat16*>(out[p]);
    mp.proj[p].N = N[p];
    mp.proj[p].begin = total;
    total += ((N[p] + 3) / 4) * mp.K8;
  }
  // small matrices: 2 rows per thread so that every SM holds a full set of warps
  const bool two = total < 2048ll * device_sm_count();
  if (two) {
    total = 0;
    for (int p = 0; p < nproj; ++p) {
      mp.proj[p].begin = total;
      total += ((N[p] + 1) / 2) * mp.K8;
    }
  }
  mp.total = total;
  long long blocks = (total + 255) / 256;
  const long long cap = 8ll * device_sm_count();
  if (blocks > cap) blocks = cap;
  const unsigned gb = static_cast<unsigned>(blocks);
#define WSL_MERGE(R)                                                    \
  do {                                                                  \
    if (two) lora_merge_kernel<R, 2><<<gb, 256, 0, stream>>>(mp);       \
    else lora_merge_kernel<R, 4><<<gb, 256, 0, stream>>>(mp);           \
  } while (0)
  switch (r) {
    case 8: WSL_MERGE(8); break;
    case 16: WSL_MERGE(16); break;
    case 32: WSL_MERGE(32); break;
    case 64: WSL_MERGE(64); break;
    default: WSL_MERGE(128); break;
  }
#undef WSL_MERGE
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

}  // namespace wsl
