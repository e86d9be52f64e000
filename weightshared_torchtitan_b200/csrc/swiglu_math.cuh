// The SwiGLU element arithmetic, in ONE place: the stand-alone row kernels and the GEMM
// epilogues that apply the activation (forward) or its derivative (backward) must give the
// same bits, so both call these.
#pragma once
#include <cuda_runtime.h>

namespace wsl {

// silu(x) * b
__device__ __forceinline__ float swiglu_fwd_elem(float x, float b) {
  return x / (1.f + __expf(-x)) * b;
}

// d/dx and d/db of silu(x) * b, times the incoming gradient dy
__device__ __forceinline__ void swiglu_bwd_elem(float dy, float x, float b, float& dx, float& db) {
  const float sg = 1.f / (1.f + __expf(-x));
  dx = dy * b * sg * (1.f + x * (1.f - sg));
  db = dy * x * sg;
}

}  // namespace wsl
