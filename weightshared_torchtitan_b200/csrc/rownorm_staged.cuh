// Staged RMSNorm (+ rotary) kernels for dense rows. Same arithmetic as the direct kernels of
// elementwise.cu, but the inputs reach the SM as 32 KB bulk copies (cp.async.bulk) into a
// ring of shared-memory stages that a producer warp keeps full, so the bytes in flight per SM
// do not depend on how many rows the compute warps hold in registers.
//
// One persistent CTA per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... A tile is
// CW * (32 / lpr) lane groups (CW compute warps, lpr lanes per row) x RPG consecutive rows per
// group, RPG = 8 / KV: 32 KB per operand with 8 compute warps. rstd (backward) and, with
// rotary, the cos/sin of the group's token (heads must be a multiple of RPG so that a group's
// rows share one position) of tile i + 1 are fetched into registers while tile i is computed.
// With rotary a lane holds KV = 2 vectors of a head row, one in each half of the row, so the
// rotate_half partner of every element sits in the same lane and no shuffle is needed.
// The rows of the ragged last tile that do not exist are zero-filled in shared memory by their
// lane group, so that the arithmetic needs no per-row predicate; only the stores have one.
// Every mbarrier wait is bounded; a wait that runs out records WSL_ERR_TIMEOUT (role 4) and
// all warps leave.
//
// The row loops are issue-bound with this few warps, so the per-element instruction count is
// what is tuned: packed bf16 conversions, reciprocal square root by MUFU + one Newton step
// (<= 1 ulp), the scale w read as float4 from shared memory, and products shared between the
// row reduction, the scale gradient and the output.
#pragma once

namespace wsl {

// stages of the ring: as many as fit next to the scale copies, by operand tiles per stage
__host__ __device__ constexpr int rn_stages(int nops) { return nops == 1 ? 6 : (nops == 2 ? 3 : 2); }
constexpr int RN_TILE_BYTES = 32768;
constexpr unsigned long long RN_WAIT_LIMIT_NS = 2000000000ull;   // default bound of every wait

// Launch-time knobs shared by the staged kernels: the bound of the mbarrier waits and the
// diagnostic switch "the producer never fills the ring" (exercises the bounded waits).
struct RnKnobs {
  unsigned long long wait_limit_ns;
  int producer_idle;
};

// compute warps of the backward: rows of 32+ elements per lane, and rotary rows (two sets of
// cos/sin registers), need more than the 168 registers a 9-warp CTA leaves each thread, so
// they run 7 compute warps (8 warps in all: 255 registers)
// Rows wider than 8 vectors per lane (KV = 10, 16: hidden sizes 2560 and 4096 in bf16) take one
// row per warp and tile, and as many compute warps as fit a 32 KB tile (512 KV bytes per row).
__host__ __device__ constexpr int rn_rows_per_group(int kv) { return kv <= 8 ? 8 / kv : 1; }
__host__ __device__ constexpr int rn_fwd_compute_warps(int kv) { return kv <= 8 ? 8 : 64 / kv; }
__host__ __device__ constexpr int rn_compute_warps(int kv, int elems_per_lane, bool rope) {
  return kv > 8 ? 64 / kv : ((elems_per_lane >= 32 || rope) ? 7 : 8);
}

// shared memory: stages | barriers (full[S], empty[S]) | abort, drain words | w[D] | dw[D]
__host__ __device__ constexpr size_t rn_head_bytes(int stages, int nops) {
  return static_cast<size_t>(stages) * nops * RN_TILE_BYTES + 2 * stages * sizeof(uint64_t) + 16;
}
// backward: dy, x (+ the gradient of the residual stream); forward: x (+ the residual addend)
__host__ __device__ constexpr size_t rn_staged_smem(int D, bool dres) {
  return rn_head_bytes(rn_stages(dres ? 3 : 2), dres ? 3 : 2) + 2 * static_cast<size_t>(D) * sizeof(float);
}
__host__ __device__ constexpr size_t rn_fwd_staged_smem(int D, bool res) {
  return rn_head_bytes(rn_stages(res ? 2 : 1), res ? 2 : 1) + static_cast<size_t>(D) * sizeof(float);
}

template <typename T>
__device__ __forceinline__ void unpack(const Vec<T>& v, float (&f)[Vec<T>::N]);
template <>
__device__ __forceinline__ void unpack<float>(const Vec<float>& v, float (&f)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = v.v[i];
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const Vec<__nv_bfloat16>& v, float (&f)[8]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <typename T>
__device__ __forceinline__ Vec<T> pack(const float (&f)[Vec<T>::N]);
template <>
__device__ __forceinline__ Vec<float> pack<float>(const float (&f)[4]) {
  Vec<float> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = f[i];
  return r;
}
template <>
__device__ __forceinline__ Vec<__nv_bfloat16> pack<__nv_bfloat16>(const float (&f)[8]) {
  Vec<__nv_bfloat16> r;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return r;
}

// Independent accumulation chains of a row reduction: one per element position of a vector
// for the widest rows, a single one otherwise (see the forward kernel).
__host__ __device__ constexpr int rn_sum_chains(int kv, int nv) { return kv >= 16 ? nv : 1; }

// Sum of N (1, 4 or 8) partial sums, pairwise.
template <int N>
__device__ __forceinline__ float tree_sum(const float (&v)[N]) {
  static_assert(N == 1 || N == 4 || N == 8, "one chain, or a vector of 4 floats or 8 bf16");
  if constexpr (N == 1) {
    return v[0];
  } else if constexpr (N == 4) {
    return (v[0] + v[1]) + (v[2] + v[3]);
  } else {
    return ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
  }
}

// 1 / sqrt(a), a > 0: hardware approximation refined by one Newton step.
__device__ __forceinline__ float rsqrt_refined(float a) {
  const float y = rsqrtf(a);
  const float h = 0.5f * a * y;
  return fmaf(y, fmaf(-h, y, 0.5f), y);   // y + y * (0.5 - 0.5 a y^2)
}

// The shared copy of the scale is laid out so that the lanes of a row read consecutive float4:
// quarter q (4 floats) of vector (k, l) sits at float4 index (k * NV/4 + q) * lpr + l.
template <int NV>
__device__ __forceinline__ int scale_slot(int j, int lpr) {
  const int vec = j / NV, e = j % NV;
  return (((vec / lpr) * (NV / 4) + e / 4) * lpr + vec % lpr) * 4 + (e & 3);
}
template <int NV>
__device__ __forceinline__ void load_scale(const float* w_s, int k, int lpr, int l, float (&wk)[NV]) {
#pragma unroll
  for (int q = 0; q < NV / 4; ++q) {
    const float4 t = *reinterpret_cast<const float4*>(w_s + ((k * (NV / 4) + q) * lpr + l) * 4);
    wk[4 * q] = t.x;
    wk[4 * q + 1] = t.y;
    wk[4 * q + 2] = t.z;
    wk[4 * q + 3] = t.w;
  }
}

// Producer warp: keeps a ring of STAGES stages full. Stage s holds NOPS operand tiles of
// RN_TILE_BYTES each (tile i of this CTA = rows [t * tile_rows, ...) with
// t = blockIdx.x + i * gridDim.x, dense rows of row_bytes); full barriers are bar0 + 8 s,
// empty barriers bar0 + 8 (STAGES + s). Leaves early when a wait runs out or another role
// set the abort flag, and then waits (bounded) for the copies it had already asked for.
template <int NOPS, int STAGES>
__device__ __forceinline__ void rn_producer_loop(const unsigned char* src0, const unsigned char* src1,
                                                 const unsigned char* src2, size_t row_bytes, int tile_rows, long long rows,
                                                 int my_tiles, uint32_t stage0, uint32_t bar0,
                                                 volatile int* abortp, volatile int* drainp, int lane,
                                                 const RnKnobs& knobs) {
  int issued = 0;
  int s = 0;
  uint32_t ph = 0;
  if (knobs.producer_idle) return;   // diagnostic: the consumers' waits must run out by themselves
  for (int i = 0; i < my_tiles; ++i) {
    if (i >= STAGES &&
        !__all_sync(0xffffffffu, mbar_wait(bar0 + 8u * (STAGES + s), ph ^ 1u, abortp, knobs.wait_limit_ns))) {
      if (lane == 0) record_timeout(4, i);
      break;
    }
    if (elect_one()) {
      const long long r0 = (blockIdx.x + static_cast<long long>(i) * gridDim.x) * tile_rows;
      const long long nrows = min(static_cast<long long>(tile_rows), rows - r0);
      const uint32_t bytes = static_cast<uint32_t>(nrows * row_bytes);
      const uint32_t dst = stage0 + static_cast<uint32_t>(s) * NOPS * RN_TILE_BYTES;
      mbar_arrive_expect_tx(bar0 + 8u * s, NOPS * bytes);
      bulk_load_1d(dst, src0 + r0 * row_bytes, bytes, bar0 + 8u * s);
      if (NOPS > 1) bulk_load_1d(dst + RN_TILE_BYTES, src1 + r0 * row_bytes, bytes, bar0 + 8u * s);
      if (NOPS > 2) bulk_load_1d(dst + 2 * RN_TILE_BYTES, src2 + r0 * row_bytes, bytes, bar0 + 8u * s);
    }
    __syncwarp();
    ++issued;
    if (++s == STAGES) {
      s = 0;
      ph ^= 1u;
    }
  }
  if (*abortp != 0) {
    for (int i = max(issued - STAGES, 0); i < issued; ++i)
      mbar_wait(bar0 + 8u * (i % STAGES), static_cast<uint32_t>(i / STAGES) & 1u, drainp,
                knobs.wait_limit_ns);
  }
}

// Zero the rows [first_missing, RPG) of this lane group's slice of a tile (ragged last tile).
template <typename T, int KV>
__device__ __forceinline__ void zero_missing_rows(unsigned char* tile, int g, int rpg, int first_missing,
                                                  size_t row_bytes, int lpr, int l) {
  constexpr int NV = Vec<T>::N;
  for (int r = first_missing; r < rpg; ++r)
#pragma unroll
    for (int k = 0; k < KV; ++k)
      *reinterpret_cast<uint4*>(tile + static_cast<size_t>(g * rpg + r) * row_bytes +
                                static_cast<size_t>(k * lpr + l) * NV * sizeof(T)) = make_uint4(0, 0, 0, 0);
}

// --------------------------------------------------------------------------- forward
// y = n * cos + rotate_half(n) * sin with n = x * rstd * w is evaluated as
// rstd * (x[j] * (w[j] cos[j]) + x[p] * (w[p] sin'[j])), p = j +- D/2 the rotate_half partner
// of j and sin' = -sin in the first half: the two coefficient vectors are built once per tile.
// RES: the row that is normalised is h = x + res (the residual add that precedes the norm),
// rounded to the storage type exactly as a separate add kernel would, and also written out.
template <typename T, bool ROPE, int KV, bool RES>
__global__ void __launch_bounds__((rn_fwd_compute_warps(KV) + 1) * 32, 1)
rmsnorm_fwd_staged_kernel(const T* __restrict__ x, const T* __restrict__ res, T* __restrict__ h_out,
                          const float* __restrict__ w, T* __restrict__ y,
                          long long ldy, float* __restrict__ rstd_out, long long rows, int D, int lpr,
                          float eps, const float* __restrict__ cs, const float* __restrict__ sn,
                          int heads, int seq, long long n_tiles, const RnKnobs knobs) {
  static_assert(!(ROPE && RES), "the residual add precedes hidden-size norms only");
  constexpr int NV = Vec<T>::N;
  constexpr int RPG = rn_rows_per_group(KV);
  constexpr int CW = rn_fwd_compute_warps(KV);
  constexpr int THREADS = (CW + 1) * 32;
  constexpr int NOPS = RES ? 2 : 1;
  // very wide rows do not fit in registers: they are read from shared memory twice
  constexpr bool PACKED = KV * NV > 64;
  constexpr int KF = PACKED ? 1 : KV;
  constexpr int S = rn_stages(NOPS);
  extern __shared__ __align__(128) unsigned char rn_smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(rn_smem + S * NOPS * RN_TILE_BYTES);
  volatile int* abortp = reinterpret_cast<volatile int*>(bars + 2 * S);
  volatile int* drainp = abortp + 1;   // stays 0: the flag of the tear-down waits
  float* w_s = reinterpret_cast<float*>(rn_smem + rn_head_bytes(S, NOPS));
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int rpw = 32 / lpr;
  const int l = lane % lpr;
  const int tile_rows = CW * rpw * RPG;
  const uint32_t stage0 = smem_u32(rn_smem);
  const uint32_t bar0 = smem_u32(bars);
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar0 + 8u * s, 1);
      mbar_init(bar0 + 8u * (S + s), CW);
    }
    *abortp = 0;
    *drainp = 0;
    fence_barrier_init();
  }
  grid_dep_wait();     // global memory is touched from here on (see ptx_sm100.cuh)
  grid_dep_launch();
  for (int j = threadIdx.x; j < D; j += THREADS) w_s[scale_slot<NV>(j, lpr)] = w[j];
  __syncthreads();
  const int my_tiles = static_cast<int>((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const size_t row_bytes = static_cast<size_t>(D) * sizeof(T);
  if (warp == CW) {
    rn_producer_loop<NOPS, S>(reinterpret_cast<const unsigned char*>(x),
                              reinterpret_cast<const unsigned char*>(res), nullptr, row_bytes, tile_rows,
                              rows, my_tiles, stage0, bar0, abortp, drainp, lane, knobs);
    return;
  }
  const float inv_D = 1.0f / static_cast<float>(D);
  const int g = warp * rpw + lane / lpr;   // lane group within the CTA
  static_assert(!ROPE || KV == 2, "rotary rows are held as two half-row vectors per lane");
  constexpr int KR = ROPE ? KV : 1;
  float cr_n[KR][NV], sr_n[KR][NV];
  auto prefetch = [&](int i) {
    const long long row0 = (blockIdx.x + static_cast<long long>(i) * gridDim.x) * tile_rows +
                           static_cast<long long>(g) * RPG;
    const long long pos = (row0 < rows ? row0 / heads : 0) % seq;
#pragma unroll
    for (int k = 0; k < KR; ++k) {
      const float4* c = reinterpret_cast<const float4*>(cs + pos * D + (k * lpr + l) * NV);
      const float4* sp = reinterpret_cast<const float4*>(sn + pos * D + (k * lpr + l) * NV);
#pragma unroll
      for (int q = 0; q < NV / 4; ++q) {
        const float4 a = c[q], b = sp[q];
        cr_n[k][4 * q] = a.x; cr_n[k][4 * q + 1] = a.y; cr_n[k][4 * q + 2] = a.z; cr_n[k][4 * q + 3] = a.w;
        sr_n[k][4 * q] = b.x; sr_n[k][4 * q + 1] = b.y; sr_n[k][4 * q + 2] = b.z; sr_n[k][4 * q + 3] = b.w;
      }
    }
  };
  if (ROPE && my_tiles > 0) prefetch(0);
  int s = 0;
  uint32_t ph = 0;
  for (int i = 0; i < my_tiles; ++i) {
    float wc[KR][NV], ws[KR][NV];
    if (ROPE) {
      float wk[KR][NV];
#pragma unroll
      for (int k = 0; k < KR; ++k) load_scale<NV>(w_s, k, lpr, l, wk[k]);
#pragma unroll
      for (int k = 0; k < KR; ++k)
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          wc[k][e] = wk[k][e] * cr_n[k][e];
          ws[k][e] = wk[KR - 1 - k][e] * (k == 0 ? -sr_n[k][e] : sr_n[k][e]);
        }
      if (i + 1 < my_tiles) prefetch(i + 1);
    }
    if (!__all_sync(0xffffffffu, mbar_wait(bar0 + 8u * s, ph, abortp, knobs.wait_limit_ns))) {
      if (lane == 0) record_timeout(4, i);
      break;
    }
    unsigned char* sx = rn_smem + static_cast<size_t>(s) * NOPS * RN_TILE_BYTES;
    const long long row0 = (blockIdx.x + static_cast<long long>(i) * gridDim.x) * tile_rows +
                           static_cast<long long>(g) * RPG;
    const int have = static_cast<int>(min(static_cast<long long>(RPG), max(rows - row0, 0ll)));
    if (have < RPG) {
      zero_missing_rows<T, KV>(sx, g, RPG, have, row_bytes, lpr, l);
      if (RES) zero_missing_rows<T, KV>(sx + RN_TILE_BYTES, g, RPG, have, row_bytes, lpr, l);
    }
    const unsigned char* srow = sx + static_cast<size_t>(g * RPG) * row_bytes + static_cast<size_t>(l) * NV * sizeof(T);
    T* yrow = y + row0 * ldy + l * NV;
    T* hrow = RES ? h_out + row0 * D + l * NV : nullptr;
#pragma unroll
    for (int r = 0; r < RPG; ++r) {
      float f_[KF][NV];
      // vector k of the row (x, or x + res rounded to the storage type) as floats
      auto load_vec = [&](int k, float (&f)[NV], bool store_h) {
        const Vec<T> v = ldv<T>(reinterpret_cast<const T*>(srow + r * row_bytes) + k * lpr * NV);
        unpack<T>(v, f);
        if (RES) {
          float a[NV];
          unpack<T>(ldv<T>(reinterpret_cast<const T*>(srow + RN_TILE_BYTES + r * row_bytes) + k * lpr * NV), a);
#pragma unroll
          for (int e = 0; e < NV; ++e) f[e] += a[e];
          const Vec<T> hv = pack<T>(f);
          if (store_h && r < have) stv<T>(hrow + static_cast<long long>(r) * D + k * lpr * NV, hv);
          unpack<T>(hv, f);   // normalise the value that was stored
        }
      };
      // The widest rows (one warp per scheduler, which hides no latency) keep one partial sum
      // per element position: NV independent chains of KV fused multiply-adds instead of one
      // chain of KV * NV. Measured at 4096 columns 55.4 -> 53.3 us; narrower rows, which run
      // two warps per scheduler, lose 1-2 % to the extra registers and keep the single chain.
      constexpr int NACC = rn_sum_chains(KV, NV);
      float ssv[NACC];
#pragma unroll
      for (int e = 0; e < NACC; ++e) ssv[e] = 0.f;
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        float (&f)[NV] = f_[PACKED ? 0 : k];
        load_vec(k, f, true);
#pragma unroll
        for (int e = 0; e < NV; ++e) ssv[e % NACC] = fmaf(f[e], f[e], ssv[e % NACC]);
      }
      if (PACKED) asm volatile("" ::: "memory");   // keep the second read a read, not 128 live registers
      float ss = tree_sum<NACC>(ssv);
      ss = group_sum(ss, lpr);
      const float rstd = rsqrt_refined(fmaf(ss, inv_D, eps));
      if (r < have && l == 0 && rstd_out) rstd_out[row0 + r] = rstd;
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        float o[NV];
        if (ROPE) {
#pragma unroll
          for (int e = 0; e < NV; ++e)
            o[e] = fmaf(f_[PACKED ? 0 : KV - 1 - k][e], ws[ROPE ? k : 0][e],
                        f_[PACKED ? 0 : k][e] * wc[ROPE ? k : 0][e]) * rstd;
        } else {
          float (&f)[NV] = f_[PACKED ? 0 : k];
          if (PACKED) load_vec(k, f, false);
          float wk[NV];
          load_scale<NV>(w_s, k, lpr, l, wk);
#pragma unroll
          for (int e = 0; e < NV; ++e) o[e] = f[e] * rstd * wk[e];
        }
        if (r < have) stv<T>(yrow + r * ldy + k * lpr * NV, pack<T>(o));
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar0 + 8u * (S + s));
    if (++s == S) {
      s = 0;
      ph ^= 1u;
    }
  }
}

// -------------------------------------------------------------------------- backward
// DRES: dx also receives dres, the gradient that reaches the same tensor through the residual
// stream (the add that autograd would otherwise run as a kernel of its own).
// dx = rstd * w * dn - x * rstd^3 * mean(dn * w * x), dn = un-rotated dy;
// dw[j] += sum_rows dn[j] * x[j] * rstd (registers -> shared-memory partials -> atomics).
template <typename T, bool ROPE, int KV, bool DRES>
__global__ void __launch_bounds__((rn_compute_warps(KV, KV * Vec<T>::N, ROPE) + 1) * 32, 1)
rmsnorm_bwd_staged_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ dres,
                          const float* __restrict__ w, const float* __restrict__ rstd_in,
                          T* __restrict__ dx, long long lddx, float* dw, long long rows, int D, int lpr,
                          const float* __restrict__ cs, const float* __restrict__ sn, int heads,
                          int seq, long long n_tiles, const RnKnobs knobs) {
  constexpr int NV = Vec<T>::N;
  constexpr int RPG = rn_rows_per_group(KV);
  constexpr int CW = rn_compute_warps(KV, KV * NV, ROPE);
  constexpr int THREADS = (CW + 1) * 32;
  constexpr int NOPS = DRES ? 3 : 2;
  constexpr int S = rn_stages(NOPS);
  static_assert(!(ROPE && DRES), "the residual stream meets hidden-size norms only");
  extern __shared__ __align__(128) unsigned char rn_smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(rn_smem + S * NOPS * RN_TILE_BYTES);
  volatile int* abortp = reinterpret_cast<volatile int*>(bars + 2 * S);
  volatile int* drainp = abortp + 1;
  float* w_s = reinterpret_cast<float*>(rn_smem + rn_head_bytes(S, NOPS));
  float* dw_part = w_s + D;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int rpw = 32 / lpr;
  const int l = lane % lpr;
  const int tile_rows = CW * rpw * RPG;
  const uint32_t stage0 = smem_u32(rn_smem);
  const uint32_t bar0 = smem_u32(bars);
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar0 + 8u * s, 1);
      mbar_init(bar0 + 8u * (S + s), CW);
    }
    *abortp = 0;
    *drainp = 0;
    fence_barrier_init();
  }
  grid_dep_wait();     // global memory is touched from here on (see ptx_sm100.cuh)
  grid_dep_launch();
  for (int j = threadIdx.x; j < D; j += THREADS) {
    dw_part[j] = 0.f;
    w_s[scale_slot<NV>(j, lpr)] = w[j];
  }
  __syncthreads();
  const int my_tiles = static_cast<int>((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const size_t row_bytes = static_cast<size_t>(D) * sizeof(T);

  if (warp == CW) {
    rn_producer_loop<NOPS, S>(reinterpret_cast<const unsigned char*>(dy),
                              reinterpret_cast<const unsigned char*>(x),
                              reinterpret_cast<const unsigned char*>(dres), row_bytes, tile_rows, rows,
                              my_tiles, stage0, bar0, abortp, drainp, lane, knobs);
  } else {
    const float inv_D = 1.0f / static_cast<float>(D);
    const int g = warp * rpw + lane / lpr;
    float dwacc[KV][NV];
#pragma unroll
    for (int k = 0; k < KV; ++k)
#pragma unroll
      for (int e = 0; e < NV; ++e) dwacc[k][e] = 0.f;
    static_assert(!ROPE || KV == 2, "rotary rows are held as two half-row vectors per lane");
    constexpr int KR = ROPE ? KV : 1;
    float w_own[KR][NV];
    if (ROPE) {
#pragma unroll
      for (int k = 0; k < KR; ++k) load_scale<NV>(w_s, k, lpr, l, w_own[k]);
    }
    float rs_n[RPG], cr_n[KR][NV], sr_n[KR][NV];
    auto prefetch = [&](int i) {
      const long long row0 = (blockIdx.x + static_cast<long long>(i) * gridDim.x) * tile_rows +
                             static_cast<long long>(g) * RPG;
#pragma unroll
      for (int r = 0; r < RPG; ++r) rs_n[r] = row0 + r < rows ? rstd_in[row0 + r] : 0.f;
      if (ROPE) {
        const long long pos = (row0 < rows ? row0 / heads : 0) % seq;
#pragma unroll
        for (int k = 0; k < KR; ++k) {
          const float4* c = reinterpret_cast<const float4*>(cs + pos * D + (k * lpr + l) * NV);
          const float4* sp = reinterpret_cast<const float4*>(sn + pos * D + (k * lpr + l) * NV);
#pragma unroll
          for (int q = 0; q < NV / 4; ++q) {
            const float4 a = c[q], b = sp[q];
            cr_n[k][4 * q] = a.x; cr_n[k][4 * q + 1] = a.y; cr_n[k][4 * q + 2] = a.z; cr_n[k][4 * q + 3] = a.w;
            sr_n[k][4 * q] = b.x; sr_n[k][4 * q + 1] = b.y; sr_n[k][4 * q + 2] = b.z; sr_n[k][4 * q + 3] = b.w;
          }
        }
      }
    };
    if (my_tiles > 0) prefetch(0);
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < my_tiles; ++i) {
      float rs[RPG], cr[KR][NV], sr[KR][NV];
#pragma unroll
      for (int r = 0; r < RPG; ++r) rs[r] = rs_n[r];
      if (ROPE) {
#pragma unroll
        for (int k = 0; k < KR; ++k)
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            cr[k][e] = cr_n[k][e];
            sr[k][e] = sr_n[k][e];
          }
      }
      if (i + 1 < my_tiles) prefetch(i + 1);
      if (!__all_sync(0xffffffffu, mbar_wait(bar0 + 8u * s, ph, abortp, knobs.wait_limit_ns))) {
        if (lane == 0) record_timeout(4, i);
        break;
      }
      unsigned char* sdy = rn_smem + static_cast<size_t>(s) * NOPS * RN_TILE_BYTES;
      unsigned char* sx = sdy + RN_TILE_BYTES;
      unsigned char* sdr = sdy + 2 * RN_TILE_BYTES;   // DRES only
      const long long row0 = (blockIdx.x + static_cast<long long>(i) * gridDim.x) * tile_rows +
                             static_cast<long long>(g) * RPG;
      const int have = static_cast<int>(min(static_cast<long long>(RPG), max(rows - row0, 0ll)));
      if (have < RPG) {
        zero_missing_rows<T, KV>(sdy, g, RPG, have, row_bytes, lpr, l);
        zero_missing_rows<T, KV>(sx, g, RPG, have, row_bytes, lpr, l);
        if (DRES) zero_missing_rows<T, KV>(sdr, g, RPG, have, row_bytes, lpr, l);
      }
      const size_t goff = static_cast<size_t>(g * RPG) * row_bytes + static_cast<size_t>(l) * NV * sizeof(T);
      T* dxrow = dx + row0 * lddx + l * NV;
#pragma unroll
      for (int r = 0; r < RPG; ++r) {
        const float rstd = rs[r];
        // very wide rows do not fit in registers next to the dw accumulators: they read the
        // row from shared memory a second time for the outputs
        constexpr bool PACKED = KV * NV > 32;
        constexpr int KF = PACKED ? 1 : KV;
        float dn_[KF][NV], xf_[KF][NV];
        constexpr int NACC = rn_sum_chains(KV, NV);   // independent chains, as in the forward
        float dotv[NACC];
#pragma unroll
        for (int e = 0; e < NACC; ++e) dotv[e] = 0.f;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
          float (&dn)[NV] = dn_[PACKED ? 0 : k];
          float (&xf)[NV] = xf_[PACKED ? 0 : k];
          const size_t off = goff + r * row_bytes + static_cast<size_t>(k) * lpr * NV * sizeof(T);
          const Vec<T> dv = ldv<T>(reinterpret_cast<const T*>(sdy + off));
          const Vec<T> xv = ldv<T>(reinterpret_cast<const T*>(sx + off));
          unpack<T>(dv, dn);
          unpack<T>(xv, xf);
          if (!ROPE) {
            float wk[NV];
            load_scale<NV>(w_s, k, lpr, l, wk);
#pragma unroll
            for (int e = 0; e < NV; ++e) {
              const float p = dn[e] * xf[e];
              dotv[e % NACC] = fmaf(p, wk[e], dotv[e % NACC]);
              dwacc[k][e] = fmaf(p, rstd, dwacc[k][e]);
            }
          }
        }
        if (ROPE) {
          // dn[j] = dy[j] cos[j] + (j < D/2 ? dy[j + D/2] sin[j + D/2] : -dy[j - D/2] sin[j - D/2])
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            const float d0 = dn_[0][e], d1 = dn_[KF - 1][e];
            dn_[0][e] = fmaf(d0, cr[0][e], d1 * sr[KR - 1][e]);
            dn_[KF - 1][e] = fmaf(d1, cr[KR - 1][e], -(d0 * sr[0][e]));
          }
#pragma unroll
          for (int k = 0; k < KF; ++k)
#pragma unroll
            for (int e = 0; e < NV; ++e) {
              const float p = dn_[k][e] * xf_[k][e];
              dotv[e % NACC] = fmaf(p, w_own[ROPE ? k : 0][e], dotv[e % NACC]);
              dwacc[k][e] = fmaf(p, rstd, dwacc[k][e]);
            }
        }
        float dot = tree_sum<NACC>(dotv);
        dot = group_sum(dot, lpr);
        if (PACKED) asm volatile("" ::: "memory");   // keep the second read a read, not 128 live registers
        const float c3 = dot * inv_D * rstd * rstd * rstd;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
          float (&dn)[NV] = dn_[PACKED ? 0 : k];
          float (&xf)[NV] = xf_[PACKED ? 0 : k];
          if (PACKED) {
            const size_t off = goff + r * row_bytes + static_cast<size_t>(k) * lpr * NV * sizeof(T);
            unpack<T>(ldv<T>(reinterpret_cast<const T*>(sdy + off)), dn);
            unpack<T>(ldv<T>(reinterpret_cast<const T*>(sx + off)), xf);
          }
          float wk[NV];
          if (!ROPE) load_scale<NV>(w_s, k, lpr, l, wk);
          float o[NV];
#pragma unroll
          for (int e = 0; e < NV; ++e)
            o[e] = fmaf(dn[e] * (ROPE ? w_own[ROPE ? k : 0][e] : wk[e]), rstd, -(xf[e] * c3));
          if (DRES) {
            float a[NV];
            const size_t off = goff + r * row_bytes + static_cast<size_t>(k) * lpr * NV * sizeof(T);
            unpack<T>(ldv<T>(reinterpret_cast<const T*>(sdr + off)), a);
#pragma unroll
            for (int e = 0; e < NV; ++e) o[e] += a[e];
          }
          if (r < have) stv<T>(dxrow + r * lddx + k * lpr * NV, pack<T>(o));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar0 + 8u * (S + s));
      if (++s == S) {
        s = 0;
        ph ^= 1u;
      }
    }
    if (dw != nullptr) {
#pragma unroll
      for (int k = 0; k < KV; ++k)
#pragma unroll
        for (int e = 0; e < NV; ++e) atomicAdd(&dw_part[(k * lpr + l) * NV + e], dwacc[k][e]);
    }
  }
  __syncthreads();
  if (dw != nullptr)
    for (int j = threadIdx.x; j < D; j += THREADS) atomicAdd(dw + j, dw_part[j]);
}

}  // namespace wsl
