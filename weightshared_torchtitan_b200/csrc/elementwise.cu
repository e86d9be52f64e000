// HBM-bound row kernels of the decoder step that sit either side of the projections:
// softmax cross-entropy (forward + gradient in one go, in place), SwiGLU, RMSNorm with an
// optional fused rotary embedding. Each is a plain streaming kernel: 16-byte vector
// accesses, fp32 math, one rounding to the storage type. T is __nv_bfloat16 or float.
#include "swiglu_math.cuh"
#include "block_gemm.cuh"
#include "status.cuh"
#include "../../include/wsl.h"
#include <cuda_bf16.h>

namespace wsl {

template <typename T>
struct Vec;   // 16-byte vector of T
template <>
struct Vec<float> {
  static constexpr int N = 4;
  float v[4];
  __device__ __forceinline__ float get(int i) const { return v[i]; }
  __device__ __forceinline__ void set(int i, float x) { v[i] = x; }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __nv_bfloat16 v[8];
  __device__ __forceinline__ float get(int i) const { return __bfloat162float(v[i]); }
  __device__ __forceinline__ void set(int i, float x) { v[i] = __float2bfloat16_rn(x); }
};
template <typename T>
__device__ __forceinline__ Vec<T> ldv(const T* p) {
  Vec<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void stv(T* p, const Vec<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}
template <typename T>
__device__ __forceinline__ float ld1(const T* p);
template <>
__device__ __forceinline__ float ld1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void st1(T* p, float x);
template <>
__device__ __forceinline__ void st1<float>(float* p, float x) { *p = x; }
template <>
__device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------ softmax cross-entropy
// One CTA per row. Pass 1: running (max, sum of exp) per thread, merged across the block.
// Pass 2: logits[row, j] <- scale * (softmax_j - [j == label]) written IN PLACE in the
// storage type; row_loss[row] = logsumexp - logit[label]. A label outside [0, V) marks an
// ignored row: zero loss, zero gradient.
constexpr int CE_THREADS = 1024;

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(T* logits, long long ld, const long long* __restrict__ labels,
                  float* __restrict__ row_loss, int V, float scale_host,
                  const float* __restrict__ scale_dev) {
  // the gradient scale may have a factor that only exists on the device (1 / number of
  // counted rows, computed from the labels without a host round trip)
  const float scale = scale_dev != nullptr ? scale_host * __ldg(scale_dev) : scale_host;
  __shared__ float red_m[32];
  __shared__ float red_s[32];
  __shared__ float bcast[2];
  T* row = logits + static_cast<long long>(blockIdx.x) * ld;
  const long long label = labels[blockIdx.x];
  const bool ignored = label < 0 || label >= V;
  constexpr int NV = Vec<T>::N;
  const int nvec = V / NV;
  float m = -INFINITY, s = 0.f;
  if (!ignored) {
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      const Vec<T> x = ldv<T>(row + static_cast<long long>(i) * NV);
      float lm = x.get(0);
#pragma unroll
      for (int e = 1; e < NV; ++e) lm = fmaxf(lm, x.get(e));
      if (lm > m) {
        s *= __expf(m - lm);
        m = lm;
      }
#pragma unroll
      for (int e = 0; e < NV; ++e) s += __expf(x.get(e) - m);
    }
    for (int j = nvec * NV + threadIdx.x; j < V; j += CE_THREADS) {
      const float x = ld1<T>(row + j);
      if (x > m) {
        s *= __expf(m - x);
        m = x;
      }
      s += __expf(x - m);
    }
    // merge (m, s) pairs: warp, then block
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float mm = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
      m = mm;
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) {
      red_m[w] = m;
      red_s[w] = s;
    }
    __syncthreads();
    if (w == 0) {
      m = red_m[l];
      s = red_s[l];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float mm = fmaxf(m, m2);
        s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
        m = mm;
      }
      if (l == 0) {
        bcast[0] = m;
        bcast[1] = logf(s) + m;   // logsumexp
        row_loss[blockIdx.x] = bcast[1] - ld1<T>(row + label);
      }
    }
    __syncthreads();
  } else if (threadIdx.x == 0) {
    row_loss[blockIdx.x] = 0.f;
  }
  const float lse = ignored ? 0.f : bcast[1];
  const int lab = static_cast<int>(label);
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    T* p = row + static_cast<long long>(i) * NV;
    Vec<T> x = ldv<T>(p);
#pragma unroll
    for (int e = 0; e < NV; ++e) {
      float g = 0.f;
      if (!ignored) {
        g = __expf(x.get(e) - lse);
        if (i * NV + e == lab) g -= 1.f;
        g *= scale;
      }
      x.set(e, g);
    }
    stv<T>(p, x);
  }
  for (int j = nvec * NV + threadIdx.x; j < V; j += CE_THREADS) {
    float g = 0.f;
    if (!ignored) {
      g = __expf(ld1<T>(row + j) - lse);
      if (j == lab) g -= 1.f;
      g *= scale;
    }
    st1<T>(row + j, g);
  }
}

// ------------------------------------------------------------------------- SwiGLU
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ out,
                  long long nvec) {
  constexpr int NV = Vec<T>::N;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < nvec; i += gridDim.x * 256ll) {
    const Vec<T> a = ldv<T>(g + i * NV), b = ldv<T>(u + i * NV);
    Vec<T> o;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
      o.set(e, swiglu_fwd_elem(a.get(e), b.get(e)));
    }
    stv<T>(out + i * NV, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const T* __restrict__ d, const T* __restrict__ g, const T* __restrict__ u,
                  T* __restrict__ dg, T* __restrict__ du, long long nvec) {
  constexpr int NV = Vec<T>::N;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < nvec; i += gridDim.x * 256ll) {
    const Vec<T> dd = ldv<T>(d + i * NV), a = ldv<T>(g + i * NV), b = ldv<T>(u + i * NV);
    Vec<T> og, ou;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
      float dgv, duv;
      swiglu_bwd_elem(dd.get(e), a.get(e), b.get(e), dgv, duv);
      og.set(e, dgv);
      ou.set(e, duv);
    }
    stv<T>(dg + i * NV, og);
    stv<T>(du + i * NV, ou);
  }
}

// ------------------------------------------------- RMSNorm (+ rotary embedding)
// A row of width D is handled by `lpr` lanes (a power of two <= 32, D = kv * lpr * NV with
// kv <= RN_MAX_VEC), so a warp covers 32/lpr rows at once: hidden-size rows use a whole
// warp, head-size rows (D = 128: 16 lanes in bf16) two per warp. Lane l of a row holds
// elements [(k*lpr + l)*NV, +NV) for k < kv. With rotary (kv == 1, D = head_dim), row r
// belongs to position (r / heads) % seq and
//   y = n * cos + rotate_half(n) * sin,   n = x * rstd * w,   rstd = 1/sqrt(mean(x^2) + eps);
// the rotate_half partner j +- D/2 lives in lane l ^ (lpr/2).
constexpr int RN_MAX_VEC = 8;
constexpr int RN_WARPS = 8;

__device__ __forceinline__ float group_sum(float v, int lpr) {
  for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Each lane group walks `iters` consecutive rows and keeps the scale w (and, with rotary,
// the cos/sin of the current position: iters = heads, so all rows of a group belong to one
// token) in registers, so per row only x is read and y written.
template <typename T, bool ROPE, int KV>
__global__ void __launch_bounds__(RN_WARPS * 32)
rmsnorm_fwd_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w,
                   T* __restrict__ y, long long ldy, float* __restrict__ rstd_out, long long rows,
                   int D, int lpr, float eps, const float* __restrict__ cs,
                   const float* __restrict__ sn, int heads, int seq, int iters) {
  constexpr int NV = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int rpw = 32 / lpr;
  const int l = lane % lpr;
  constexpr int kv = KV;
  const long long group = (blockIdx.x * static_cast<long long>(RN_WARPS) + (threadIdx.x >> 5)) * rpw + lane / lpr;
  const long long row0 = group * iters;
  float wr[KV][NV];
#pragma unroll
  for (int k = 0; k < KV; ++k)
    if (k < kv)
#pragma unroll
      for (int e = 0; e < NV; ++e) wr[k][e] = w[(k * lpr + l) * NV + e];
  float cr[NV], sr[NV];
  if (ROPE) {
    const long long pos = (row0 < rows ? row0 / heads : 0) % seq;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
      cr[e] = cs[pos * D + l * NV + e];
      sr[e] = sn[pos * D + l * NV + e];
      if (l < (lpr >> 1)) sr[e] = -sr[e];   // rotate_half: first half takes -n[j + D/2]
    }
  }
  // software pipeline: the loads of row rr+1 are in flight while row rr is reduced and stored
  Vec<T> nxt[KV];
#pragma unroll
  for (int k = 0; k < KV; ++k) {
    if (row0 < rows) nxt[k] = ldv<T>(x + row0 * ldx + (k * lpr + l) * NV);
    else
#pragma unroll
      for (int e = 0; e < NV; ++e) nxt[k].set(e, 0.f);
  }
  for (int rr = 0; rr < iters; ++rr) {
    const long long row = row0 + rr;
    const bool valid = row < rows;
    Vec<T> xv[KV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < KV; ++k) xv[k] = nxt[k];
    if (rr + 1 < iters) {
      const bool nvalid = row + 1 < rows;
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        if (nvalid) nxt[k] = ldv<T>(x + (row + 1) * ldx + (k * lpr + l) * NV);
        else
#pragma unroll
          for (int e = 0; e < NV; ++e) nxt[k].set(e, 0.f);
      }
    }
#pragma unroll
    for (int k = 0; k < KV; ++k)
#pragma unroll
      for (int e = 0; e < NV; ++e) ss += xv[k].get(e) * xv[k].get(e);
    ss = group_sum(ss, lpr);
    const float rstd = 1.0f / sqrtf(ss / D + eps);
    if (valid && l == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int k = 0; k < KV; ++k)
      if (k < kv) {
        Vec<T> o;
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          float v = xv[k].get(e) * rstd * wr[k][e];
          if (ROPE) {
            const float partner = __shfl_xor_sync(0xffffffffu, v, lpr >> 1);
            v = v * cr[e] + partner * sr[e];
          }
          o.set(e, v);
        }
        if (valid) stv<T>(y + row * ldy + (k * lpr + l) * NV, o);
      }
  }
}

// Backward: dx = rstd * (g - x * rstd^2 * mean(g * x)), g = dn * w, dn = un-rotated dy;
// dw[j] += sum_rows dn[j] * x[j] * rstd (registers -> shared-memory partials -> atomics).
// The row loop is latency-bound, so each lane group loads U rows (dy and x) before it
// computes any of them (U = 4 for one-vector rows, 2 for hidden-size rows); the scale w is
// re-read from L1 per row instead of cached in registers.
template <typename T, bool ROPE, int KV>
__global__ void __launch_bounds__(RN_WARPS * 32, KV <= 2 ? 2 : 1)
rmsnorm_bwd_kernel(const T* __restrict__ dy, long long lddy, const T* __restrict__ x, long long ldx,
                   const float* __restrict__ w, const float* __restrict__ rstd_in,
                   T* __restrict__ dx, long long lddx, float* dw, long long rows, int D, int lpr,
                   const float* __restrict__ cs, const float* __restrict__ sn, int heads, int seq,
                   int iters) {
  constexpr int NV = Vec<T>::N;
  constexpr int U = KV == 1 ? 4 : (KV <= 4 ? 2 : 1);
  extern __shared__ float dw_part[];   // [D]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int rpw = 32 / lpr;
  const int l = lane % lpr;
  for (int j = threadIdx.x; j < D; j += RN_WARPS * 32) dw_part[j] = 0.f;
  __syncthreads();
  float dwacc[KV][NV];
#pragma unroll
  for (int k = 0; k < KV; ++k)
#pragma unroll
    for (int e = 0; e < NV; ++e) dwacc[k][e] = 0.f;
  const long long group = (blockIdx.x * static_cast<long long>(RN_WARPS) + warp) * rpw + lane / lpr;
  const long long row0 = group * iters;
  float cr[NV], sr[NV];
  long long cur_pos = -1;
  for (int rr = 0; rr < iters; rr += U) {
    Vec<T> dv[U][KV], xv[U][KV];
    float rs[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = row0 + rr + u;
      const bool valid = rr + u < iters && row < rows;
      rs[u] = valid ? rstd_in[row] : 0.f;
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        if (valid) {
          dv[u][k] = ldv<T>(dy + row * lddy + (k * lpr + l) * NV);
          xv[u][k] = ldv<T>(x + row * ldx + (k * lpr + l) * NV);
        } else {
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            dv[u][k].set(e, 0.f);
            xv[u][k].set(e, 0.f);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = row0 + rr + u;
      const bool valid = rr + u < iters && row < rows;
      const float rstd = rs[u];
      if (ROPE) {
        const long long pos = (valid ? row / heads : 0) % seq;
        if (pos != cur_pos) {
          cur_pos = pos;
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            cr[e] = cs[pos * D + l * NV + e];
            sr[e] = sn[pos * D + l * NV + e];
          }
        }
      }
      float dn0[NV];   // un-rotated gradient of the (single) vector when ROPE
      if (ROPE) {
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          // dn[j] = dy[j] cos[j] + (j < D/2 ? dy[j+D/2] sin[j+D/2] : -dy[j-D/2] sin[j-D/2])
          const float d = dv[u][0].get(e);
          const float other = __shfl_xor_sync(0xffffffffu, d * sr[e], lpr >> 1);
          dn0[e] = d * cr[e] + (l < (lpr >> 1) ? other : -other);
        }
      }
      float dot = 0.f;
#pragma unroll
      for (int k = 0; k < KV; ++k)
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          const float xe = xv[u][k].get(e);
          const float dne = ROPE ? dn0[e] : dv[u][k].get(e);
          dot += dne * __ldg(w + (k * lpr + l) * NV + e) * xe;
          dwacc[k][e] += dne * xe * rstd;
        }
      dot = group_sum(dot, lpr);
      const float c = dot * rstd * rstd / D;
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        Vec<T> o;
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          const float dne = ROPE ? dn0[e] : dv[u][k].get(e);
          o.set(e, rstd * (dne * __ldg(w + (k * lpr + l) * NV + e) - xv[u][k].get(e) * c));
        }
        if (valid) stv<T>(dx + row * lddx + (k * lpr + l) * NV, o);
      }
    }
  }
  if (dw != nullptr) {
#pragma unroll
    for (int k = 0; k < KV; ++k)
#pragma unroll
      for (int e = 0; e < NV; ++e) atomicAdd(&dw_part[(k * lpr + l) * NV + e], dwacc[k][e]);
    __syncthreads();
    for (int j = threadIdx.x; j < D; j += RN_WARPS * 32) atomicAdd(dw + j, dw_part[j]);
  }
}

}  // namespace wsl
#include "rownorm_staged.cuh"
namespace wsl {

// ------------------------------------------------------------------ host launchers
// Option row_staged = 0 sends every row-kernel call to the direct (register pipelined)
// kernels, for A/B timing of the staged ones.
static bool row_staged_enabled() { return options().row_staged != 0; }

// Wait bound and the bounded-wait test aid of the staged kernels, taken from the library's
// options at launch like the GEMM's.
static RnKnobs rn_knobs() {
  RnKnobs k;
  k.wait_limit_ns = options().wait_limit_ns;
  k.producer_idle = options().stall_producer ? 1 : 0;
  return k;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
static int ce_launch(void* logits, long long ld, const long long* labels, float* row_loss,
                     long long rows, long long V, float scale, const float* scale_dev, cudaStream_t s) {
  ce_fwd_bwd_kernel<T><<<static_cast<unsigned>(rows), CE_THREADS, 0, s>>>(
      static_cast<T*>(logits), ld, labels, row_loss, static_cast<int>(V), scale, scale_dev);
  return cudaGetLastError() == cudaSuccess ? WSL_OK : WSL_ERR_CUDA;
}

int launch_ce(void* logits, long long ld, const long long* labels, float* row_loss, long long rows,
              long long V, float scale, const float* scale_dev, int is_f32, cudaStream_t s) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!logits || !labels || !row_loss || rows <= 0 || V <= 0 || ld < V) return WSL_ERR_BAD_ARG;
  if (rows > 0x7fffffffLL || V > 0x7fffffffLL) return WSL_ERR_TOO_LARGE;
  const int nv = is_f32 ? 4 : 8;
  if (!aligned16(logits) || (ld % nv) != 0) return WSL_ERR_ALIGN;
  st = is_f32 ? ce_launch<float>(logits, ld, labels, row_loss, rows, V, scale, scale_dev, s)
              : ce_launch<__nv_bfloat16>(logits, ld, labels, row_loss, rows, V, scale, scale_dev, s);
  if (st == WSL_OK) ++g_launch_count;
  return st;
}

int launch_swiglu(const void* g, const void* u, void* out, const void* d, void* dg, void* du,
                  long long n, int is_f32, cudaStream_t s) {
  int st = device_check();
  if (st != WSL_OK) return st;
  if (!g || !u || n <= 0) return WSL_ERR_BAD_ARG;
  const int nv = is_f32 ? 4 : 8;
  if ((n % nv) != 0 || !aligned16(g) || !aligned16(u)) return WSL_ERR_ALIGN;
  const long long nvec = n / nv;
  long long blocks = (nvec + 255) / 256;
  const long long cap = 32ll * device_sm_count();
  if (blocks > cap) blocks = cap;
  const unsigned gb = static_cast<unsigned>(blocks);
  if (d == nullptr) {
    if (!out || !aligned16(out)) return WSL_ERR_BAD_ARG;
    if (is_f32)
      swiglu_fwd_kernel<float><<<gb, 256, 0, s>>>(static_cast<const float*>(g), static_cast<const float*>(u),
                                                  static_cast<float*>(out), nvec);
    else
      swiglu_fwd_kernel<__nv_bfloat16><<<gb, 256, 0, s>>>(
          static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u),
          static_cast<__nv_bfloat16*>(out), nvec);
  } else {
    if (!dg || !du || !aligned16(d) || !aligned16(dg) || !aligned16(du)) return WSL_ERR_BAD_ARG;
    if (is_f32)
      swiglu_bwd_kernel<float><<<gb, 256, 0, s>>>(static_cast<const float*>(d), static_cast<const float*>(g),
                                                  static_cast<const float*>(u), static_cast<float*>(dg),
                                                  static_cast<float*>(du), nvec);
    else
      swiglu_bwd_kernel<__nv_bfloat16><<<gb, 256, 0, s>>>(
          static_cast<const __nv_bfloat16*>(d), static_cast<const __nv_bfloat16*>(g),
          static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(dg),
          static_cast<__nv_bfloat16*>(du), nvec);
  }
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

// lanes per row for a width-D row, or 0 when the kernels do not cover D.
static int rms_lanes(long long D, int nv) {
  if (D <= 0 || (D % nv) != 0) return 0;
  long long lanes = D / nv;
  if (lanes >= 32) {
    // kv = 10 and 16 (hidden sizes 2560 and 4096 in bf16) exist as staged kernels only
    const long long kv = D / (32 * nv);
    return (D % (32 * nv)) == 0 && (kv == 1 || kv == 2 || kv == 4 || kv == 8 || (nv == 8 && (kv == 10 || kv == 16)))
               ? 32 : 0;
  }
  return (lanes & (lanes - 1)) == 0 ? static_cast<int>(lanes) : 0;
}

static int rms_check(const void* x, long long ldx, long long rows, long long D, int is_f32,
                     const float* cs, const float* sn, long long heads, long long seq) {
  if (!x || rows <= 0 || D <= 0 || ldx < D) return WSL_ERR_BAD_ARG;
  const int nv = is_f32 ? 4 : 8;
  const int lpr = rms_lanes(D, nv);
  if (lpr == 0) return WSL_ERR_TOO_LARGE;
  if ((ldx % nv) != 0 || !aligned16(x)) return WSL_ERR_ALIGN;
  if ((cs == nullptr) != (sn == nullptr)) return WSL_ERR_BAD_ARG;
  if (cs != nullptr && (heads <= 0 || seq <= 0 || lpr < 2 || D != static_cast<long long>(lpr) * nv))
    return WSL_ERR_BAD_ARG;
  return WSL_OK;
}

// res / h_out: optional residual addend and sum output (dense [rows, D]); then the rows that
// are normalised are h = x + res. Only the staged kernel does that: rows must be dense.
int launch_rmsnorm_fwd(const void* x, long long ldx, const void* res, void* h_out, const float* w,
                       void* y, long long ldy, float* rstd, long long rows, long long D, float eps,
                       const float* cs, const float* sn, long long heads, long long seq, int is_f32,
                       cudaStream_t s) {
  int st = device_check();
  if (st != WSL_OK) return st;
  st = rms_check(x, ldx, rows, D, is_f32, cs, sn, heads, seq);
  if (st != WSL_OK) return st;
  if (!w || !y || !aligned16(y) || ldy < D) return WSL_ERR_BAD_ARG;
  const int lpr = rms_lanes(D, is_f32 ? 4 : 8);
  // rows per lane group: all heads of one token with rotary (one cos/sin fetch), else enough
  // to amortise the register copy of w while still filling the GPU
  long long iters = cs ? heads : 4;
  if (!cs && rows < 4ll * RN_WARPS * (32 / lpr) * device_sm_count()) iters = 1;
  const long long rows_per_block = static_cast<long long>(RN_WARPS) * (32 / lpr) * iters;
  const unsigned gb = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
  const int d = static_cast<int>(D), h = static_cast<int>(heads), sq = static_cast<int>(seq);
  const int kvn = static_cast<int>(D / (static_cast<long long>(lpr) * (is_f32 ? 4 : 8)));
  const bool fused = res != nullptr;
  if (fused && (cs || !h_out || ldx != D || !aligned16(res) || !aligned16(h_out))) return WSL_ERR_BAD_ARG;
  if ((fused || kvn > 8 || row_staged_enabled()) && ldx == D &&
      (!cs || (heads % 4 == 0 && aligned16(cs) && aligned16(sn)))) {
    // rotary rows: two half-row vectors per lane (the staged kernels' layout), else as above
    const int s_kv = cs ? 2 : kvn;
    const int s_lpr = cs ? static_cast<int>(D / (2 * (is_f32 ? 4 : 8))) : lpr;
    const int cw = rn_fwd_compute_warps(s_kv);
    const long long tile_rows = static_cast<long long>(cw) * (32 / s_lpr) * rn_rows_per_group(s_kv);
    const long long n_tiles = (rows + tile_rows - 1) / tile_rows;
    const unsigned sgb = static_cast<unsigned>(n_tiles < device_sm_count() ? n_tiles : device_sm_count());
    const size_t ssmem = rn_fwd_staged_smem(d, fused);
#define WSL_RNFS(T, R, KVN, RES)                                                                   \
  do {                                                                                             \
    static bool attr_set_dev[kMaxDevices] = {};   /* the limit is a per-device setting */        \
    const int dev_i = current_device_index();                                                      \
    if (dev_i < 0) return WSL_ERR_DEVICE;                                                          \
    if (!attr_set_dev[dev_i]) {                                                                    \
      if (cudaFuncSetAttribute(rmsnorm_fwd_staged_kernel<T, R, KVN, RES>,                          \
                               cudaFuncAttributeMaxDynamicSharedMemorySize,                        \
                               static_cast<int>(rn_fwd_staged_smem(4096, RES))) != cudaSuccess)    \
        return WSL_ERR_CUDA;                                                                       \
      attr_set_dev[dev_i] = true;                                                                  \
    }                                                                                              \
    launch_dependent(rmsnorm_fwd_staged_kernel<T, R, KVN, RES>, dim3(sgb), dim3((cw + 1) * 32), ssmem, s,  \
        static_cast<const T*>(x), static_cast<const T*>(res), static_cast<T*>(h_out), w,           \
        static_cast<T*>(y), ldy, rstd, rows, d, s_lpr, eps, cs, sn, h, sq, n_tiles, rn_knobs());   \
  } while (0)
#define WSL_RNFS_RES(T, KVN)                                      \
  do {                                                            \
    if (fused) WSL_RNFS(T, false, KVN, true);                     \
    else WSL_RNFS(T, false, KVN, false);                          \
  } while (0)
#define WSL_RNFS_KV(T)                                            \
  do {                                                            \
    if (cs) WSL_RNFS(T, true, 2, false);                          \
    else if (s_kv == 1) WSL_RNFS_RES(T, 1);                       \
    else if (s_kv == 2) WSL_RNFS_RES(T, 2);                       \
    else if (s_kv == 4) WSL_RNFS_RES(T, 4);                       \
    else if (s_kv == 8) WSL_RNFS_RES(T, 8);                       \
    else return WSL_ERR_TOO_LARGE;                                \
  } while (0)
    if (is_f32) WSL_RNFS_KV(float);
    else if (s_kv == 10) WSL_RNFS_RES(__nv_bfloat16, 10);
    else if (s_kv == 16) WSL_RNFS_RES(__nv_bfloat16, 16);
    else WSL_RNFS_KV(__nv_bfloat16);
#undef WSL_RNFS_KV
#undef WSL_RNFS_RES
#undef WSL_RNFS
    if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
    ++g_launch_count;
    return WSL_OK;
  }
  if (fused) return WSL_ERR_BAD_ARG;   // the direct kernel has no residual input
  if (kvn > 8) return WSL_ERR_TOO_LARGE;   // rows this wide exist as staged kernels (dense rows) only
#define WSL_RN(T, R, KVN)                                                                          \
  rmsnorm_fwd_kernel<T, R, KVN><<<gb, RN_WARPS * 32, 0, s>>>(                                      \
      static_cast<const T*>(x), ldx, w, static_cast<T*>(y), ldy, rstd, rows, d, lpr, eps, cs, sn, \
      h, sq, static_cast<int>(iters))
#define WSL_RN_KV(T)                                              \
  do {                                                            \
    if (cs) WSL_RN(T, true, 1);                                   \
    else if (kvn == 1) WSL_RN(T, false, 1);                       \
    else if (kvn == 2) WSL_RN(T, false, 2);                       \
    else if (kvn == 4) WSL_RN(T, false, 4);                       \
    else if (kvn == 8) WSL_RN(T, false, 8);                       \
    else return WSL_ERR_TOO_LARGE;                                \
  } while (0)
  if (is_f32) WSL_RN_KV(float); else WSL_RN_KV(__nv_bfloat16);
#undef WSL_RN_KV
#undef WSL_RN
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

// dres: optional gradient of the residual stream (dense [rows, D]) that is added to dx. Only
// the staged kernel does that: rows must be dense.
int launch_rmsnorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const void* dres,
                       const float* w, const float* rstd, void* dx, long long lddx, float* dw,
                       long long rows, long long D, const float* cs, const float* sn, long long heads,
                       long long seq, int is_f32, cudaStream_t s) {
  int st = device_check();
  if (st != WSL_OK) return st;
  st = rms_check(x, ldx, rows, D, is_f32, cs, sn, heads, seq);
  if (st != WSL_OK) return st;
  if (!dy || !w || !rstd || !dx || !aligned16(dy) || !aligned16(dx) || lddy < D || lddx < D)
    return WSL_ERR_BAD_ARG;
  // enough rows per warp that the dw atomics stay a small fraction of the work
  const int lpr = rms_lanes(D, is_f32 ? 4 : 8);
  const long long rows_per_pass = static_cast<long long>(RN_WARPS) * (32 / lpr);
  // wide rows run one CTA per SM (register-heavy): few, long-lived CTAs keep the number of
  // contended dw atomics small; narrow rows fit several CTAs per SM
  const long long kv_host = D / (static_cast<long long>(lpr) * (is_f32 ? 4 : 8));
  const long long target_blocks = (kv_host >= 4 ? 2ll : 8ll) * device_sm_count();
  long long rpw = (rows + target_blocks * rows_per_pass - 1) / (target_blocks * rows_per_pass);
  if (rpw < 1) rpw = 1;
  const unsigned gb = static_cast<unsigned>((rows + rows_per_pass * rpw - 1) / (rows_per_pass * rpw));
  const int d = static_cast<int>(D), h = static_cast<int>(heads), sq = static_cast<int>(seq);
  const size_t smem = static_cast<size_t>(D) * sizeof(float);
  const int kvn = static_cast<int>(D / (static_cast<long long>(lpr) * (is_f32 ? 4 : 8)));
  // contiguous rows take the staged kernel (bulk copies need 16-byte aligned, dense tiles)
  const bool fused = dres != nullptr;
  if (fused && (cs || lddy != D || ldx != D || !aligned16(dres))) return WSL_ERR_BAD_ARG;
  if ((fused || kvn > 8 || row_staged_enabled()) && lddy == D && ldx == D &&
      (!cs || (heads % 4 == 0 && aligned16(cs) && aligned16(sn)))) {
    // rotary rows: two half-row vectors per lane (the staged kernels' layout), else as above
    const int s_kv = cs ? 2 : kvn;
    const int s_lpr = cs ? static_cast<int>(D / (2 * (is_f32 ? 4 : 8))) : lpr;
    const int rpg = rn_rows_per_group(s_kv);
    const int cw = rn_compute_warps(s_kv, s_kv * (is_f32 ? 4 : 8), cs != nullptr);
    const long long tile_rows = static_cast<long long>(cw) * (32 / s_lpr) * rpg;
    const long long n_tiles = (rows + tile_rows - 1) / tile_rows;
    const unsigned sgb = static_cast<unsigned>(n_tiles < device_sm_count() ? n_tiles : device_sm_count());
    const size_t ssmem = rn_staged_smem(d, fused);
#define WSL_RNS(T, R, KVN, DRES)                                                                   \
  do {                                                                                             \
    static bool attr_set_dev[kMaxDevices] = {};   /* the limit is a per-device setting */        \
    const int dev_i = current_device_index();                                                      \
    if (dev_i < 0) return WSL_ERR_DEVICE;                                                          \
    if (!attr_set_dev[dev_i]) {                                                                    \
      if (cudaFuncSetAttribute(rmsnorm_bwd_staged_kernel<T, R, KVN, DRES>,                         \
                               cudaFuncAttributeMaxDynamicSharedMemorySize,                        \
                               static_cast<int>(rn_staged_smem(4096, DRES))) != cudaSuccess)       \
        return WSL_ERR_CUDA;                                                                       \
      attr_set_dev[dev_i] = true;                                                                  \
    }                                                                                              \
    launch_dependent(rmsnorm_bwd_staged_kernel<T, R, KVN, DRES>, dim3(sgb), dim3((cw + 1) * 32), ssmem, s, \
        static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(dres), w, rstd, \
        static_cast<T*>(dx), lddx, dw, rows, d, s_lpr, cs, sn, h, sq, n_tiles, rn_knobs());        \
  } while (0)
#define WSL_RNS_RES(T, KVN)                                       \
  do {                                                            \
    if (fused) WSL_RNS(T, false, KVN, true);                      \
    else WSL_RNS(T, false, KVN, false);                           \
  } while (0)
#define WSL_RNS_KV(T)                                             \
  do {                                                            \
    if (cs) WSL_RNS(T, true, 2, false);                           \
    else if (s_kv == 1) WSL_RNS_RES(T, 1);                        \
    else if (s_kv == 2) WSL_RNS_RES(T, 2);                        \
    else if (s_kv == 4) WSL_RNS_RES(T, 4);                        \
    else if (s_kv == 8) WSL_RNS_RES(T, 8);                        \
    else return WSL_ERR_TOO_LARGE;                                \
  } while (0)
    if (is_f32) WSL_RNS_KV(float);
    else if (s_kv == 10) WSL_RNS_RES(__nv_bfloat16, 10);
    else if (s_kv == 16) WSL_RNS_RES(__nv_bfloat16, 16);
    else WSL_RNS_KV(__nv_bfloat16);
#undef WSL_RNS_KV
#undef WSL_RNS_RES
#undef WSL_RNS
    if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
    ++g_launch_count;
    return WSL_OK;
  }
  if (fused) return WSL_ERR_BAD_ARG;   // the direct kernel has no residual-gradient input
  if (kvn > 8) return WSL_ERR_TOO_LARGE;   // rows this wide exist as staged kernels (dense rows) only
#define WSL_RNB(T, R, KVN)                                                                         \
  rmsnorm_bwd_kernel<T, R, KVN><<<gb, RN_WARPS * 32, smem, s>>>(                                   \
      static_cast<const T*>(dy), lddy, static_cast<const T*>(x), ldx, w, rstd, static_cast<T*>(dx), \
      lddx, dw, rows, d, lpr, cs, sn, h, sq, static_cast<int>(rpw))
#define WSL_RNB_KV(T)                                             \
  do {                                                            \
    if (cs) WSL_RNB(T, true, 1);                                  \
    else if (kvn == 1) WSL_RNB(T, false, 1);                      \
    else if (kvn == 2) WSL_RNB(T, false, 2);                      \
    else if (kvn == 4) WSL_RNB(T, false, 4);                      \
    else if (kvn == 8) WSL_RNB(T, false, 8);                      \
    else return WSL_ERR_TOO_LARGE;                                \
  } while (0)
  if (is_f32) WSL_RNB_KV(float); else WSL_RNB_KV(__nv_bfloat16);
#undef WSL_RNB_KV
#undef WSL_RNB
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

}  // namespace wsl
