// The SwiGLU element arithmetic, in ONE place: the stand-alone row kernels and the GEMM
// epilogues that apply the activation (forward) or its derivative (backward) must give the
// same bits, so both call these.
#pragma once
#include <cuda_runtime.h>

namespace wsl {

// The logistic function by the fast exponential and the approximate reciprocal (2 ulp; the
// results are rounded to bf16 or feed fp32 sums of thousands of terms). An IEEE division costs
// about ten instructions, which matters in a GEMM epilogue where four warps do this for a
// whole tile.
__device__ __forceinline__ float logistic(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// silu(x) * b
__device__ __forceinline__ float swiglu_fwd_elem(float x, float b) { return x * logistic(x) * b; }

// d/dx and d/db of silu(x) * b, times the incoming gradient dy
__device__ __forceinline__ void swiglu_bwd_elem(float dy, float x, float b, float& dx, float& db) {
  const float sg = logistic(x);
  dx = dy * b * sg * (1.f + x * (1.f - sg));
  db = dy * x * sg;
}

}  // namespace wsl
