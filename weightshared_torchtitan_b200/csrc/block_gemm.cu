// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   out_region[mo, no] (op)= alpha * sum over segments  A_seg * B_seg^T
//
// One launch covers up to kMaxRegion output regions that share the contraction,
// and the contraction is a concatenation of up to kMaxSeg segments, each with
// its own pair of TMA tensor maps. That one shape serves every GEMM on the
// shared-W + LoRA path:
//   forward   y  = [x | T] . [W | B]^T                    2 segments, K-major / K-major
//   dX        dX = [dY_q | U_q | dY_k | ...] . [...]      2 per projection, K-major / MN-major
//   dW,dA,dB  [dY | U]^T . [x | T]                        3 regions, MN-major / MN-major
//   pre-pass  T  = s x A^T,  U = s dY B                    1 segment, narrow N tile
//
// CTA layout (192 threads, one CTA per SM, grid = min(#SM, #tiles)):
//   warp 0    TMA producer: fills a 4-stage ring of [128 x 64] A and [bn x 64] B
//             bf16 tiles, 128-byte swizzled, completion on `full` mbarriers
//   warp 1    allocates 512 TMEM columns, one lane issues tcgen05.mma
//             (M=128, N=bn<=256, K=16 per instruction) into one of two fp32
//             accumulators; tcgen05.commit frees ring stages and publishes tiles
//   warps 2-5 epilogue: tcgen05.ld of their 32-lane quarter, scale, convert,
//             store/accumulate to global, then hand the accumulator back
// Every mbarrier wait is bounded; a wait that runs out records WSL_ERR_TIMEOUT in
// g_wsl_status and all roles fall through to the common tear-down.
#include "block_gemm.cuh"
#include "ptx_sm100.cuh"
#include "status.cuh"
#include "swiglu_math.cuh"

#include <cuda_bf16.h>
#include <cudaTypedefs.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <mutex>

#include "../../include/wsl.h"

namespace wsl {

constexpr int BM = 128;
constexpr int BN_MAX = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;       // 16 KiB
constexpr int B_STAGE_BYTES = BN_MAX * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SLAB_BYTES = 64 * BK * 2;          // one MN-major slab: 64 k-rows of 128 B
constexpr int EPI_STAGE_BYTES = 128 * 128;       // epilogue staging: 128 rows x 128 B, two of them
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // 2 s

struct Region {
  signed char a_map[kMaxSeg];
  signed char b_map[kMaxSeg];
  int m_tiles;
  int n_tiles;
  int tile_begin;
  int bn;
  int rows;
  int cols;
  void* out;
  long long ld;
  int mode;
  float alpha;
  long long ws_off;   // split-K: float offset of this region's partials in the workspace
  int transposed;     // fp32 output element (row, col) of the tile lives at out[col * ld + row]
  int out_map;        // tensor map of the output for the TMA-store epilogue, or -1
  int group;          // rasterisation: M-tiles per group (their A rows stay L2-resident)
  int splits;         // split-K factor of this region (1 = none)
  int unit_begin;     // first work unit of this region (units = tile_count * splits)
  // The tiles of the region's rasterisation this entry covers: all of them, except where a
  // launch ends with a split TAIL -- then the parent entry stops short (tile_count < tiles)
  // and a copy of it at the end of the launch covers the rest (tile_off > 0, splits > 1),
  // its partials packed tile by tile into the workspace (see SplitPlan).
  int tile_off;
  int tile_count;
  int tail;           // 1 for such a tail entry
  // k-blocks this region really has: the launch's kb_total, except where regions of different
  // contraction lengths share a launch (one segment, GemmDesc::ragged_k) -- then a region's
  // splits divide ITS blocks and nothing is spent on the zeros beyond its end
  int kb_own;
  void* copy;         // bf16 copy of alpha * acc (RegionDesc::copy), or nullptr
  long long ld_copy;
  // kEpiSwiGLU regions (pair launches): the second CTA of a pair loads its half of the B tile
  // from these maps at contraction coordinate kk - b2_shift; tensor maps out_map, out_map + 1
  // and out_map + 2 are g, u and silu(g) * u.
  signed char b2_map[kMaxSeg];
  int b2_shift[kMaxSeg];
  int swiglu;
  int addend_map;     // tensor map of RegionDesc::addend, or -1
};

struct GemmParams {
  alignas(64) CUtensorMap maps[kMaxMaps];
  Region reg[kMaxRegion];
  int seg_k[kMaxSeg];
  int nseg;
  int nregion;
  int total_tiles;
  int total_units;    // work units over all regions (tiles x the region's split factor)
  int kb_total;       // k-blocks summed over the segments
  int stages;         // one-CTA variant: depth of the operand ring (4, or 8 in the narrow form)
  int stage_bytes;    // one-CTA variant: bytes per stage (48 KiB, or 24 KiB in the narrow form)
  float* workspace;   // [splits][rows x cols] fp32 partials per region when splits > 1
  // Profiling switches, a bit mask that only builds with WSL_PROFILE_SWITCHES look at (normal
  // builds compile the tests out): 1 skip epilogue stores, 2 skip TMA loads, 4 skip MMAs (time
  // the other parts alone), 32 direct-store epilogue instead of the staged TMA store.
  int dbg;
  int stall_producer;                 // test aid: the producer never fills the ring (bounded waits)
  // Epilogues that read matrices of the output's shape through TMA (all regions alike):
  // 0 none, 1 out = alpha acc + addend (64-column chunks), 2 SwiGLU backward from g = addend and
  // u = addend2 into two outputs (32-column chunks, 64-byte swizzle).
  int aux_mode;
  // Staging slots of 16 KiB the epilogue owns behind the operand ring: 2 normally; the
  // weight-merge launch (one k-block per tile, so a short ring) runs with 8, which lets the
  // addend tiles be fetched six chunks ahead instead of one.
  int epi_slots;
  unsigned long long wait_limit_ns;   // bound of every mbarrier wait
  // Row gather (factorized embedding): when set, the rows of region 0 / segment 0's A operand
  // (gather_a, K-major) or the k-rows of its B operand (gather_b, MN-major) are the rows
  // tokens[i] of the mapped matrix, fetched by TMA tile::gather4.
  const long long* gather_tokens;
  long long gather_count;
  int gather_a;
  int gather_b;
};

struct TileInfo {
  int r;
  int m0;
  int n0;
  int split;
};

// Segment-local k-block range [lo, hi) that split `split` of `splits` owns, given that the
// segment starts at flattened k-block index `base` and has `nkb` blocks.
__device__ __forceinline__ void split_range(int kb_total, int splits, int split, int base, int nkb,
                                            int& lo, int& hi) {
  const int g_lo = static_cast<int>((static_cast<long long>(kb_total) * split) / splits);
  const int g_hi = static_cast<int>((static_cast<long long>(kb_total) * (split + 1)) / splits);
  lo = max(g_lo - base, 0);
  hi = min(g_hi - base, nkb);
}

__device__ __forceinline__ void record_timeout(int role, int tile) {
  if (atomicCAS(&g_wsl_status[0], 0, WSL_ERR_TIMEOUT) == 0) {
    g_wsl_status[1] = role;
    g_wsl_status[2] = static_cast<int>(blockIdx.x);
    g_wsl_status[3] = tile;
  }
}

template <int NV>
__device__ __forceinline__ void epilogue_store(const Region& R, int row, int col0,
                                               const uint32_t (&v)[NV]) {
  if (row >= R.rows) return;
  const float alpha = R.alpha;
  if (R.transposed) {
    // one fp32 per lane and column: lanes hold consecutive rows, i.e. consecutive addresses
    float* o = static_cast<float*>(R.out) + row;
    const bool acc = (R.mode == kEpiAccumF32);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (col0 + j < R.cols) {
        float* dst = o + static_cast<long long>(col0 + j) * R.ld;
        const float f = alpha * __uint_as_float(v[j]);
        *dst = acc ? (*dst + f) : f;
      }
    }
    return;
  }
  if (R.mode == kEpiStoreBf16) {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(R.out) + static_cast<long long>(row) * R.ld + col0;
#pragma unroll
    for (int j = 0; j < NV; j += 8) {
      if (col0 + j < R.cols) {
        uint4 pk;
        uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = alpha * __uint_as_float(v[j + 2 * e]);
          const float hi = alpha * __uint_as_float(v[j + 2 * e + 1]);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
          w[e] = *reinterpret_cast<uint32_t*>(&h2);
        }
        *reinterpret_cast<uint4*>(o + j) = pk;
      }
    }
  } else {
    float* o = static_cast<float*>(R.out) + static_cast<long long>(row) * R.ld + col0;
    const bool acc = (R.mode == kEpiAccumF32);
#pragma unroll
    for (int j = 0; j < NV; j += 4) {
      if (col0 + j < R.cols) {
        float4 f;
        f.x = alpha * __uint_as_float(v[j]);
        f.y = alpha * __uint_as_float(v[j + 1]);
        f.z = alpha * __uint_as_float(v[j + 2]);
        f.w = alpha * __uint_as_float(v[j + 3]);
        float4* dst = reinterpret_cast<float4*>(o + j);
        if (acc) {
          const float4 old = *dst;
          f.x += old.x;
          f.y += old.y;
          f.z += old.z;
          f.w += old.w;
        }
        *dst = f;
      }
    }
  }
}

// Named barrier 1 joins the 128 epilogue threads (warps 2-5).
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// AND-vote over the 128 epilogue threads, so that they leave the tile loop together.
__device__ __forceinline__ bool epi_vote_and(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(ok))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h2);
}

// Per-variant constants. PAIR = two CTAs (a cluster of 2, tcgen05 cta_group::2) share one
// 256 x bn tile: each CTA owns 128 rows of A and of the accumulator and loads HALF of the
// B tile, so a stage is 32 KiB (6-deep ring) instead of 48 KiB (4-deep).
// The one-CTA variant also has a NARROW form for launches whose tiles are at most 64 columns
// wide (rank-r pre-passes, adapter gradients): the B tile is then 8 KiB, a stage 24 KiB, and
// the same shared memory holds an 8-deep ring, which doubles the bytes in flight of these
// HBM-latency-bound launches. Stage count and size of the one-CTA variant are therefore
// run-time values (GemmParams::stages, stage_bytes); kMaxStages sizes the barrier array.
template <bool PAIR>
struct Cfg {
  static constexpr int kStages = PAIR ? 6 : 4;
  static constexpr int kMaxStages = PAIR ? 6 : 8;
  static constexpr int kBStageBytes = PAIR ? B_STAGE_BYTES / 2 : B_STAGE_BYTES;
  static constexpr int kStageBytes = A_STAGE_BYTES + kBStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * EPI_STAGE_BYTES + 1024;
  static constexpr int kTileM = PAIR ? 2 * BM : BM;
};
constexpr int NARROW_BN = 64;
constexpr int NARROW_STAGES = 8;
constexpr int NARROW_STAGE_BYTES = A_STAGE_BYTES + NARROW_BN * 128;   // 24 KiB
static_assert(NARROW_STAGES * NARROW_STAGE_BYTES == Cfg<false>::kStages * Cfg<false>::kStageBytes,
              "both forms of the one-CTA ring fill the same shared memory");

// Work unit u -> (region, tile, split). Units are ordered region by region (the large
// region first), and inside a region split-major, so with round-robin assignment every
// worker gets its share of the expensive units before the cheap narrow ones fill the gaps.
template <bool PAIR>
__device__ __forceinline__ TileInfo decode_tile_t(const GemmParams& p, int u) {
  int r = 0;
  while (r + 1 < p.nregion && u >= p.reg[r + 1].unit_begin) ++r;
  const Region& R = p.reg[r];
  const int ul = u - R.unit_begin;
  const int tiles_r = R.tile_count;
  const int split = ul / tiles_r;
  const int lt = ul - split * tiles_r + R.tile_off;
  const int G = R.group;
  const int per_group = G * R.n_tiles;
  const int g = lt / per_group;
  const int first_m = g * G;
  const int gsz = min(R.m_tiles - first_m, G);
  const int rem = lt - g * per_group;
  const int mt = first_m + rem % gsz;
  const int nt = rem / gsz;
  return {r, mt * Cfg<PAIR>::kTileM, nt * R.bn, split};
}

// Role loops are executed by ALL 32 lanes of their warp with warp-uniform control flow;
// only the TMA / MMA / commit instructions themselves are issued by one elected lane.
// (A loop run by a single lane of a diverged warp keeps its state in per-thread registers
// and pays a vector-to-uniform register move in front of every tcgen05.mma operand; the
// issuing thread then cannot keep the tensor pipe fed.)
template <bool A_MN, bool B_MN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
block_gemm_kernel(const __grid_constant__ GemmParams p) {
  using C = Cfg<PAIR>;
  constexpr int SMAX = C::kMaxStages;
  const int S = PAIR ? C::kStages : p.stages;
  const uint32_t stage_bytes = PAIR ? static_cast<uint32_t>(C::kStageBytes) : static_cast<uint32_t>(p.stage_bytes);
  extern __shared__ __align__(1024) uint8_t smem_dyn[];
  constexpr int kMaxEpiSlots = 8;
  __shared__ __align__(8) uint64_t bars[2 * SMAX + 4 + kMaxEpiSlots];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  // Clusters of 2 are consecutive blocks of the 1-D grid: rank 0 is the leader.
  const int rank = PAIR ? static_cast<int>(blockIdx.x & 1u) : 0;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int nworkers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (SMAX + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * SMAX + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * SMAX + 2 + b); };
  auto aux_bar = [&](uint32_t b) { return bar0 + 8u * (2 * SMAX + 4 + b); };   // addend tiles landed
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), PAIR ? 8 : 4);   // one arrival per epilogue warp (of both CTAs)
    }
    for (int b = 0; b < kMaxEpiSlots; ++b) mbar_init(aux_bar(b), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && elect_one())   // the operand maps live in the kernel parameters: nothing to wait for
    for (int i = 0; i < p.nregion * p.nseg * 2 && i < kMaxMaps; ++i) tma_prefetch_desc(&p.maps[i]);
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(&tmem_base_smem), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&tmem_base_smem), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_smem);
  const int units = p.total_units;
  // Barriers and tensor memory are set up; from here on the kernel reads and writes global
  // memory, which has to wait for the kernel before it in the stream. The one after it may
  // be staged already: its CTAs take the SMs as this grid's CTAs leave them and do their own
  // set-up while the last tiles here are still running.
  grid_dep_wait();
  grid_dep_launch();
#ifdef WSL_PROFILE_SWITCHES
  const int dbg = p.dbg;
#else
  constexpr int dbg = 0;
#endif

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int u = worker; ok && u < units; u += nworkers) {
      const int t = u;
      const TileInfo ti = decode_tile_t<PAIR>(p, u);
      const int split = ti.split;
      const Region& R = p.reg[ti.r];
      const int b_rows = PAIR ? (R.bn >> 1) : R.bn;          // B rows this CTA loads
      const int b_slabs = (b_rows + 63) >> 6;
      const uint32_t tx_cta = A_STAGE_BYTES + (B_MN ? b_slabs * SLAB_BYTES : b_rows * BK * 2);
      const int m0 = ti.m0 + BM * rank;
      // gate|up tiles: both CTAs load the SAME 128 weight rows, the leader from the gate
      // matrices, its peer from the up matrices
      const bool dual_b = PAIR && R.swiglu != 0;
      const int n0 = dual_b ? (ti.n0 >> 1) : ti.n0 + b_rows * rank;
      // Gathered A operand: the four row ids of this lane depend on the tile only, so they are
      // read once per tile, not once per k-block (a dependent global load in front of every
      // stage would set the pace of the whole ring).
      int ga4[4] = {-1, -1, -1, -1};
      if (!A_MN && p.gather_tokens != nullptr && p.gather_a && ti.r == 0) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const long long row = static_cast<long long>(m0) + 4 * lane + e;
          if (row < p.gather_count) ga4[e] = static_cast<int>(__ldg(p.gather_tokens + row));
        }
      }
      int kb_base = 0;
      for (int sg = 0; ok && sg < p.nseg; ++sg) {
        const bool gather = p.gather_tokens != nullptr && ti.r == 0 && sg == 0;
        const CUtensorMap* ma = &p.maps[R.a_map[sg]];
        const CUtensorMap* mb = &p.maps[(dual_b && rank == 1) ? R.b2_map[sg] : R.b_map[sg]];
        const int b_kshift = (dual_b && rank == 1) ? R.b2_shift[sg] : 0;
        const int klen = p.seg_k[sg];
        const int nkb = (klen + BK - 1) / BK;
        int lo, hi;
        split_range(R.kb_own, R.splits, split, kb_base, min(nkb, R.kb_own - kb_base), lo, hi);
        kb_base += nkb;
        for (int kk = lo * BK; kk < hi * BK; kk += BK) {
          // Gathered B operand: the k-rows of this block are 64 token ids; lane l fetches rows
          // 4 (l mod 16) .. +3 of every slab, so it needs four ids per k-block. They are read
          // BEFORE the wait for a free stage, which hides their latency behind the ring.
          int gb4[4] = {-1, -1, -1, -1};
          if (B_MN && gather && p.gather_b) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const long long row = static_cast<long long>(kk) + 4 * (lane & 15) + e;
              if (row < p.gather_count) gb4[e] = static_cast<int>(__ldg(p.gather_tokens + row));
            }
          }
          ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1u, abortp, p.wait_limit_ns));
          if (!ok) {
            if (lane == 0) record_timeout(1, t);
            break;
          }
          if (elect_one() && !p.stall_producer) {
            const uint32_t sa = smem_base + s * stage_bytes;
            const uint32_t sb = sa + A_STAGE_BYTES;
            if (dbg & 2) {
              if (rank == 0) mbar_arrive(full_bar(s));
            } else if (PAIR) {
              // both CTAs' bytes are counted on the leader's barrier
              if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2u * tx_cta);
              const uint32_t fb = map_to_cta(full_bar(s), 0);
              if (A_MN) {
                tma_load_2d_pair(sa, ma, fb, m0, kk);
                tma_load_2d_pair(sa + SLAB_BYTES, ma, fb, m0 + 64, kk);
              } else if (!(gather && p.gather_a)) {
                tma_load_2d_pair(sa, ma, fb, kk, m0);
              }
              if (B_MN) {
                if (!(gather && p.gather_b))
                  for (int j = 0; j < b_slabs; ++j)
                    tma_load_2d_pair(sb + j * SLAB_BYTES, mb, fb, n0 + 64 * j, kk);
              } else {
                // (a coordinate left of the matrix, or beyond its last column, reads as zeros)
                tma_load_2d_pair(sb, mb, fb, kk - b_kshift, n0);
              }
            } else {
              const uint32_t fb = full_bar(s);
              mbar_arrive_expect_tx(fb, tx_cta);
              if (A_MN) {
                tma_load_2d(sa, ma, fb, m0, kk);
                tma_load_2d(sa + SLAB_BYTES, ma, fb, m0 + 64, kk);
              } else if (!(gather && p.gather_a)) {
                tma_load_2d(sa, ma, fb, kk, m0);
              }
              if (B_MN) {
                if (!(gather && p.gather_b))
                  for (int j = 0; j < b_slabs; ++j)
                    tma_load_2d(sb + j * SLAB_BYTES, mb, fb, n0 + 64 * j, kk);
              } else {
                tma_load_2d(sb, mb, fb, kk, n0);
              }
            }
          }
          if (gather && !(dbg & 2) && !p.stall_producer) {
            // Gathered operand: every lane fetches 4 rows (512 B) per tile::gather4 into its own
            // CTA's stage (in a pair the bytes count on the leader's barrier, like the tiled
            // loads); a row id outside the matrix reads as zeros.
            const uint32_t fb = PAIR ? map_to_cta(full_bar(s), 0) : full_bar(s);
            const uint32_t sa = smem_base + s * stage_bytes;
            const uint32_t sb = sa + A_STAGE_BYTES;
            if (!A_MN && p.gather_a) {
              if (PAIR) tma_gather4_2d_pair(sa + lane * 512, ma, fb, kk, ga4[0], ga4[1], ga4[2], ga4[3]);
              else tma_gather4_2d(sa + lane * 512, ma, fb, kk, ga4[0], ga4[1], ga4[2], ga4[3]);
            }
            if (B_MN && p.gather_b) {
              for (int q4 = lane; q4 < 16 * b_slabs; q4 += 32) {
                const int j = q4 >> 4;            // slab
                const int g4 = q4 & 15;           // group of 4 k-rows inside the slab (= lane & 15)
                const uint32_t dst = sb + j * SLAB_BYTES + g4 * 512;
                if (PAIR) tma_gather4_2d_pair(dst, mb, fb, n0 + 64 * j, gb4[0], gb4[1], gb4[2], gb4[3]);
                else tma_gather4_2d(dst, mb, fb, n0 + 64 * j, gb4[0], gb4[1], gb4[2], gb4[3]);
              }
            }
          }
          __syncwarp();
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------- MMA issuer (leader CTA only in a pair)
    if (!PAIR || rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      // Descriptor constants: K-major tiles step 32 B per MMA inside the swizzled row,
      // MN-major tiles step 16 k-rows (2 KiB); slabs of 64 MN elements are SLAB_BYTES
      // apart (leading offset), 8-row groups 1 KiB (stride offset).
      const uint64_t a_hi = A_MN ? smem_desc_sw128(0, SLAB_BYTES, 1024) : smem_desc_sw128(0, 16, 1024);
      const uint64_t b_hi = B_MN ? smem_desc_sw128(0, SLAB_BYTES, 1024) : smem_desc_sw128(0, 16, 1024);
      constexpr uint32_t a_step = (A_MN ? 2048u : 32u) >> 4;
      constexpr uint32_t b_step = (B_MN ? 2048u : 32u) >> 4;
      for (int u = worker; ok && u < units; u += nworkers, ++it) {
        const int t = u;
        const TileInfo ti = decode_tile_t<PAIR>(p, u);
        const int split = ti.split;
        const Region& R = p.reg[ti.r];
        const uint32_t idesc = umma_idesc_bf16(C::kTileM, R.bn, A_MN ? 1 : 0, B_MN ? 1 : 0);
        const int buf = it & 1;
        const uint32_t tph = (static_cast<uint32_t>(it) >> 1) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(buf), tph ^ 1u, abortp, p.wait_limit_ns));
        if (!ok) {
          if (lane == 0) record_timeout(2, t);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN_MAX);
        uint32_t accumulate = 0;
        int kb_base = 0;
        for (int sg = 0; ok && sg < p.nseg; ++sg) {
          const int klen = p.seg_k[sg];
          const int nkb = (klen + BK - 1) / BK;
          int lo, hi;
          split_range(R.kb_own, R.splits, split, kb_base, min(nkb, R.kb_own - kb_base), lo, hi);
          kb_base += nkb;
          for (int kk = lo * BK; kk < hi * BK; kk += BK) {
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, abortp, p.wait_limit_ns));
            if (!ok) {
              if (lane == 0) record_timeout(2, t);
              break;
            }
            tc_fence_after_sync();
            const int kvalid = min(BK, klen - kk);
            const int nk = (dbg & 4) ? 0 : ((kvalid + 15) >> 4);
            const uint32_t sa = smem_base + s * stage_bytes;
            const uint32_t sb = sa + A_STAGE_BYTES;
            const uint32_t a_lo = (sa & 0x3FFFFu) >> 4;
            const uint32_t b_lo = (sb & 0x3FFFFu) >> 4;
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                if (k < nk) {
                  const uint64_t adesc = a_hi | static_cast<uint64_t>(a_lo + k * a_step);
                  const uint64_t bdesc = b_hi | static_cast<uint64_t>(b_lo + k * b_step);
                  if (PAIR) umma_bf16_pair(d_tmem, adesc, bdesc, idesc, accumulate);
                  else umma_bf16(d_tmem, adesc, bdesc, idesc, accumulate);
                  accumulate = 1;
                }
              }
              if (PAIR) umma_commit_pair(empty_bar(s), 3);
              else umma_commit(empty_bar(s));
            }
            __syncwarp();
            accumulate = nk > 0 ? 1u : accumulate;
            if (++s == S) {
              s = 0;
              ph ^= 1u;
            }
          }
        }
        if (ok && elect_one()) {
          if (PAIR) umma_commit_pair(tfull_bar(buf), 3);
          else umma_commit(tfull_bar(buf));
        }
        __syncwarp();
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    const int trow = q * 32 + lane;                       // row inside this CTA's 128-row tile
    const bool issuer = (warp == 2 && lane == 0);         // issues the TMA stores
    const uint32_t epi_base = smem_base + S * stage_bytes;
    uint32_t chunk_ctr = 0;
    int it = 0;
    // Addend tiles (out = alpha acc + addend) are fetched into the staging buffers by TMA one
    // 64-column chunk AHEAD of the chunk being computed; this walks the same chunk sequence.
    int pf_u = worker, pf_c = 0;
    uint32_t pf_ctr = 0;
    const uint32_t n_slots = static_cast<uint32_t>(p.epi_slots);
    // With more than two slots the fetch runs n_slots - 2 chunks ahead and a slot is reused
    // two stores after it was handed to TMA, so the issuer never waits for the store it has
    // just issued; with two slots it runs one chunk ahead and has to.
    const int pf_dist = n_slots > 2 ? static_cast<int>(n_slots) - 2 : 1;
    auto prefetch_addend = [&]() {
      if (pf_u >= units) return;
      const TileInfo pt = decode_tile_t<PAIR>(p, pf_u);
      const Region& PR = p.reg[pt.r];
      const uint32_t slot = pf_ctr % n_slots;
      const uint32_t dst = epi_base + slot * EPI_STAGE_BYTES;
      mbar_arrive_expect_tx(aux_bar(slot), EPI_STAGE_BYTES);
      if (p.aux_mode == 1) {
        tma_load_2d(dst, &p.maps[PR.addend_map], aux_bar(slot), pt.n0 + pf_c, pt.m0 + BM * rank);
        pf_c += 64;
      } else {   // two half-width tiles (g, u) share the slot
        tma_load_2d(dst, &p.maps[PR.addend_map], aux_bar(slot), pt.n0 + pf_c, pt.m0 + BM * rank);
        tma_load_2d(dst + EPI_STAGE_BYTES / 2, &p.maps[PR.addend_map + 1], aux_bar(slot), pt.n0 + pf_c,
                    pt.m0 + BM * rank);
        pf_c += 32;
      }
      ++pf_ctr;
      if (pf_c >= PR.bn) {
        pf_c = 0;
        pf_u += nworkers;
      }
    };
    if (p.aux_mode != 0 && issuer && !p.stall_producer)
      for (int i = 0; i < pf_dist; ++i) prefetch_addend();
    for (int u = worker; u < units; u += nworkers, ++it) {
      const int t = u;
      const TileInfo ti = decode_tile_t<PAIR>(p, u);
      const int split = ti.split;
      Region R = p.reg[ti.r];
      if (R.splits > 1) {
        // partial sums go to this split's slice of the workspace; splitk_reduce_kernel folds
        // them into the real output in a fixed order afterwards
        if (R.tail) {
          // packed: one dense [tile rows x BN_MAX] block per (split, tile) of the tail; the
          // base is moved back by the tile's origin so that (row, col) indexing still works
          const long long blk = static_cast<long long>(split) * R.tile_count + (u - R.unit_begin - split * R.tile_count);
          R.out = p.workspace + R.ws_off + blk * (C::kTileM * BN_MAX) -
                  (static_cast<long long>(ti.m0) * BN_MAX + ti.n0);
          R.ld = BN_MAX;
        } else {
          R.out = p.workspace + R.ws_off + static_cast<long long>(split) * R.rows * R.cols;
          R.ld = R.transposed ? R.rows : R.cols;
        }
        R.mode = kEpiStoreF32;
        R.alpha = 1.f;
        R.out_map = -1;
        R.copy = nullptr;   // the reduce kernel writes the copy from the folded sum
      }
      if (dbg & 1) R.rows = 0;   // debug: read TMEM, store nothing
      Region RC = R;             // the bf16 copy of the tile, written with direct stores
      RC.out = R.copy;
      RC.ld = R.ld_copy;
      RC.mode = kEpiStoreBf16;
      RC.transposed = 0;
      const int buf = it & 1;
      const uint32_t tph = (static_cast<uint32_t>(it) >> 1) & 1u;
      const bool ok = epi_vote_and(mbar_wait(tfull_bar(buf), tph, abortp, p.wait_limit_ns));
      if (!ok) {
        if (issuer) record_timeout(3, t);
        break;
      }
      tc_fence_after_sync();
      const int row0 = ti.m0 + BM * rank;
      const int row = row0 + trow;
      const uint32_t taddr =
          tmem_base + static_cast<uint32_t>(buf * BN_MAX) + (static_cast<uint32_t>(q * 32) << 16);
      if (p.aux_mode == 2) {
        // ---- SwiGLU backward: dh = bf16(alpha * acc) never leaves the SM; with the g and u
        // tiles that TMA has brought into the staging slot, every thread turns its row of 32
        // columns into d gate and d up in place, and the two half-slots are stored.
        const float alpha = R.alpha;
        const uint32_t swz = static_cast<uint32_t>((trow >> 1) & 3);   // 64-byte swizzle: 16-B piece ^ row bits 1-2
        bool okc = true;
        for (int c = 0; c < R.bn; c += 32, ++chunk_ctr) {
          const uint32_t slot = chunk_ctr & 1u;
          const uint32_t sbuf = epi_base + slot * EPI_STAGE_BYTES;
          const uint32_t grow = sbuf + static_cast<uint32_t>(trow) * 64u;
          const uint32_t urow = grow + EPI_STAGE_BYTES / 2;
          if (issuer && !p.stall_producer) {
            tma_wait_group_read<0>();
            prefetch_addend();
          }
          okc = epi_vote_and(mbar_wait(aux_bar(slot), (chunk_ctr >> 1) & 1u, abortp, p.wait_limit_ns));
          if (!okc) break;
          uint32_t v[32];
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t off = (static_cast<uint32_t>(j) ^ swz) << 4;
            uint32_t gw[4], uw[4];
            ld_shared_v4(grow + off, gw);
            ld_shared_v4(urow + off, uw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float dg[2], du[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const float dy = __bfloat162float(__float2bfloat16_rn(alpha * __uint_as_float(v[8 * j + 2 * e + h])));
                const float gx = __uint_as_float(h ? (gw[e] & 0xffff0000u) : (gw[e] << 16));
                const float ux = __uint_as_float(h ? (uw[e] & 0xffff0000u) : (uw[e] << 16));
                swiglu_bwd_elem(dy, gx, ux, dg[h], du[h]);
              }
              gw[e] = pack_bf16(dg[0], dg[1]);
              uw[e] = pack_bf16(du[0], du[1]);
            }
            st_shared_v4(grow + off, gw[0], gw[1], gw[2], gw[3]);
            st_shared_v4(urow + off, uw[0], uw[1], uw[2], uw[3]);
          }
          fence_proxy_async_smem();
          epi_bar_sync();
          if (issuer && R.rows > 0) {
            tma_store_2d(&p.maps[R.out_map], sbuf, ti.n0 + c, row0);
            tma_store_2d(&p.maps[R.out_map + 1], sbuf + EPI_STAGE_BYTES / 2, ti.n0 + c, row0);
            tma_commit_group();
          }
        }
        if (!okc) {
          if (issuer) record_timeout(3, t);
          break;
        }
      } else if (p.aux_mode == 1) {
        // ---- out = alpha * acc + addend (bf16): the addend chunk is already on its way into
        // the staging buffer; every thread adds its row in place, then the buffer is stored.
        const float alpha = R.alpha;
        const uint32_t swz = static_cast<uint32_t>(trow & 7);
        bool okc = true;
        for (int c = 0; c < R.bn; c += 64, ++chunk_ctr) {
          const uint32_t slot = chunk_ctr % n_slots;
          const uint32_t sbuf = epi_base + slot * EPI_STAGE_BYTES;
          const uint32_t srow = sbuf + static_cast<uint32_t>(trow) * 128u;
          if (issuer && !p.stall_producer) {
            // the slot the next fetch goes to was last stored from one (two slots) or two
            // (more slots) chunks ago: that store must have read it
            if (n_slots > 2) tma_wait_group_read<1>();
            else tma_wait_group_read<0>();
            prefetch_addend();
          }
          okc = epi_vote_and(mbar_wait(aux_bar(slot), (chunk_ctr / n_slots) & 1u, abortp, p.wait_limit_ns));
          if (!okc) break;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c + 32 * h, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t addr = srow + ((static_cast<uint32_t>(4 * h + j) ^ swz) << 4);
              uint32_t w[4];
              ld_shared_v4(addr, w);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = fmaf(alpha, __uint_as_float(v[8 * j + 2 * e]), __uint_as_float(w[e] << 16));
                const float hi =
                    fmaf(alpha, __uint_as_float(v[8 * j + 2 * e + 1]), __uint_as_float(w[e] & 0xffff0000u));
                w[e] = pack_bf16(lo, hi);
              }
              st_shared_v4(addr, w[0], w[1], w[2], w[3]);
            }
          }
          fence_proxy_async_smem();
          epi_bar_sync();
          if (issuer && R.rows > 0) {
            tma_store_2d(&p.maps[R.out_map], sbuf, ti.n0 + c, row0);
            tma_commit_group();
          }
        }
        if (!okc) {
          if (issuer) record_timeout(3, t);
          break;
        }
      } else if (PAIR && R.swiglu != 0) {
        // ---- gate|up tile: accumulator columns [0,128) are g, [128,256) are u for the same
        // 128 output columns. Three staged 64-column stores per half: g, u (what the backward
        // needs) and silu(g) * u computed from the bf16-rounded g and u, exactly what a
        // separate pass over the stored matrices would produce.
        const int ocol0 = ti.n0 >> 1;
        const uint32_t swz = static_cast<uint32_t>(trow & 7);
        for (int c = 0; c < 128; c += 64) {
#pragma unroll 1
          for (int part = 0; part < 3; ++part, ++chunk_ctr) {
            const uint32_t sbuf = epi_base + (chunk_ctr & 1u) * EPI_STAGE_BYTES;
            const uint32_t srow = sbuf + static_cast<uint32_t>(trow) * 128u;
            if (issuer) tma_wait_group_read<1>();
            epi_bar_sync();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32];
              if (part < 2) {
                tmem_ld_32x32(taddr + (part == 1 ? 128 : 0) + c + 32 * h, v);
                tmem_ld_wait();
              } else {
                uint32_t w[32];
                tmem_ld_32x32(taddr + c + 32 * h, v);
                tmem_ld_32x32(taddr + 128 + c + 32 * h, w);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j])));
                  const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(w[j])));
                  v[j] = __float_as_uint(swiglu_fwd_elem(g, u));
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                st_shared_v4(srow + ((static_cast<uint32_t>(4 * h + j) ^ swz) << 4),
                             pack_bf16(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                             pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                             pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                             pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
            }
            fence_proxy_async_smem();
            epi_bar_sync();
            if (issuer && R.rows > 0) {
              tma_store_2d(&p.maps[R.out_map + part], sbuf, ocol0 + c, row0);
              tma_commit_group();
            }
          }
        }
      } else if (R.out_map >= 0) {
        // ---- staged epilogue: TMEM -> registers -> swizzled shared memory -> TMA store (or
        // TMA reduce-add for the in-place fp32 accumulation). 128-byte rows: 64 bf16 or 32 fp32
        // columns per chunk; two staging buffers so a store drains while the next chunk fills.
        const CUtensorMap* om = &p.maps[R.out_map];
        const bool f32 = R.mode != kEpiStoreBf16;
        const float alpha = R.alpha;
        const int step = f32 ? 32 : 64;
        const uint32_t swz = static_cast<uint32_t>(trow & 7);
        for (int c = 0; c < R.bn; c += step, ++chunk_ctr) {
          const uint32_t sbuf = epi_base + (chunk_ctr & 1u) * EPI_STAGE_BYTES;
          const uint32_t srow = sbuf + static_cast<uint32_t>(trow) * 128u;
          if (issuer) tma_wait_group_read<1>();   // the store that last used this buffer has read it
          epi_bar_sync();
          if (f32) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c, v);
            tmem_ld_wait();
            if (RC.out != nullptr) epilogue_store<32>(RC, row, ti.n0 + c, v);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_shared_v4(srow + ((static_cast<uint32_t>(j) ^ swz) << 4),
                           __float_as_uint(alpha * __uint_as_float(v[4 * j])),
                           __float_as_uint(alpha * __uint_as_float(v[4 * j + 1])),
                           __float_as_uint(alpha * __uint_as_float(v[4 * j + 2])),
                           __float_as_uint(alpha * __uint_as_float(v[4 * j + 3])));
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32];
              tmem_ld_32x32(taddr + c + 32 * h, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j)
                st_shared_v4(srow + ((static_cast<uint32_t>(4 * h + j) ^ swz) << 4),
                             pack_bf16(alpha * __uint_as_float(v[8 * j]), alpha * __uint_as_float(v[8 * j + 1])),
                             pack_bf16(alpha * __uint_as_float(v[8 * j + 2]), alpha * __uint_as_float(v[8 * j + 3])),
                             pack_bf16(alpha * __uint_as_float(v[8 * j + 4]), alpha * __uint_as_float(v[8 * j + 5])),
                             pack_bf16(alpha * __uint_as_float(v[8 * j + 6]), alpha * __uint_as_float(v[8 * j + 7])));
            }
          }
          fence_proxy_async_smem();
          epi_bar_sync();
          if (issuer && R.rows > 0) {
            if (R.mode == kEpiAccumF32) tma_reduce_add_2d(om, sbuf, ti.n0 + c, row0);
            else tma_store_2d(om, sbuf, ti.n0 + c, row0);
            tma_commit_group();
          }
        }
      } else {
        for (int c = 0; c < R.bn; c += 32) {
          if (R.bn - c >= 32) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c, v);
            tmem_ld_wait();
            epilogue_store<32>(R, row, ti.n0 + c, v);
            if (RC.out != nullptr) epilogue_store<32>(RC, row, ti.n0 + c, v);
          } else {
            uint32_t v[16];
            tmem_ld_32x16(taddr + c, v);
            tmem_ld_wait();
            epilogue_store<16>(R, row, ti.n0 + c, v);
            if (RC.out != nullptr) epilogue_store<16>(RC, row, ti.n0 + c, v);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));
        else mbar_arrive(tempty_bar(buf));
      }
    }
    if (issuer) tma_wait_group<0>();   // all stores of this CTA have completed
  }

  // ---------------------------------------------------------------- tear-down
  if (*abortp != 0) {
    // Give TMA copies that are still in flight time to land before the CTA's
    // shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's shared memory and barriers stay valid until both are done
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Fold split-K partials into the outputs in a fixed order (deterministic), all regions of
// the launch in one kernel:  out[i,j] (op)= alpha * (ws[0][i,j] + ... + ws[S-1][i,j]).
struct ReduceRegion {
  const float4* ws;
  void* out;
  long long ld;
  long long begin;    // first float4 index of this region in the flattened index space
  int rows;
  int cols4;
  int mode;
  float alpha;
  int splits;
  __nv_bfloat16* copy;   // RegionDesc::copy, or nullptr
  long long ld_copy;
};
struct ReduceParams {
  ReduceRegion reg[kMaxRegion];
  long long total;    // float4 elements over all regions
  int nregion;
};

__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const __grid_constant__ ReduceParams rp) {
  grid_dep_wait();
  grid_dep_launch();
  for (long long gi = blockIdx.x * 256ll + threadIdx.x; gi < rp.total; gi += gridDim.x * 256ll) {
    int r = 0;
    while (r + 1 < rp.nregion && gi >= rp.reg[r + 1].begin) ++r;
    const ReduceRegion& R = rp.reg[r];
    const long long i = gi - R.begin;
    const long long per = static_cast<long long>(R.rows) * R.cols4;
    float4 a = R.ws[i];
    for (int s = 1; s < R.splits; ++s) {
      const float4 b = R.ws[s * per + i];
      a.x += b.x;
      a.y += b.y;
      a.z += b.z;
      a.w += b.w;
    }
    a.x *= R.alpha;
    a.y *= R.alpha;
    a.z *= R.alpha;
    a.w *= R.alpha;
    const long long row = i / R.cols4;
    const int c = static_cast<int>(i - row * R.cols4) * 4;
    if (R.copy != nullptr) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(a.z, a.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(R.copy + row * R.ld_copy + c) = pk;
    }
    if (R.mode == kEpiStoreBf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(a.z, a.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(R.out) + row * R.ld + c) = pk;
    } else {
      float4* dst = reinterpret_cast<float4*>(static_cast<float*>(R.out) + row * R.ld + c);
      if (R.mode == kEpiAccumF32) {
        const float4 o = *dst;
        a.x += o.x;
        a.y += o.y;
        a.z += o.z;
        a.w += o.w;
      }
      *dst = a;
    }
  }
}

// Fold of a split tail (see SplitPlan): for tile j of the tail entry `tr`,
//   out[tile j] (op)= alpha * (block(0, j) + ... + block(S-1, j)),
// the blocks being the dense [tile rows x BN_MAX] partials the main kernel left in the
// workspace. `parts` blocks of 256 threads share a tile by rows.
template <bool PAIR>
__global__ void __launch_bounds__(256)
tail_reduce_kernel(const __grid_constant__ GemmParams p, int tr, int parts) {
  constexpr int TM = Cfg<PAIR>::kTileM;
  grid_dep_wait();
  grid_dep_launch();
  const Region& R = p.reg[tr];
  const int j = static_cast<int>(blockIdx.x) / parts;
  const int part = static_cast<int>(blockIdx.x) % parts;
  const TileInfo ti = decode_tile_t<PAIR>(p, R.unit_begin + j);   // split 0 of tile j
  const int rows_per = TM / parts;
  const int c4n = R.bn / 4;
  const long long blk = static_cast<long long>(TM) * BN_MAX;
  const float* ws = p.workspace + R.ws_off;
  for (int idx = threadIdx.x; idx < rows_per * c4n; idx += 256) {
    const int lr = part * rows_per + idx / c4n;
    const int lc = (idx % c4n) * 4;
    const long long row = ti.m0 + lr;
    const int col = ti.n0 + lc;
    if (row >= R.rows || col >= R.cols) continue;
    const float* src = ws + j * blk + static_cast<long long>(lr) * BN_MAX + lc;
    float4 a = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < R.splits; ++s) {
      const float4 b = *reinterpret_cast<const float4*>(src + static_cast<long long>(s) * R.tile_count * blk);
      a.x += b.x;
      a.y += b.y;
      a.z += b.z;
      a.w += b.w;
    }
    a.x *= R.alpha;
    a.y *= R.alpha;
    a.z *= R.alpha;
    a.w *= R.alpha;
    if (R.copy != nullptr || R.mode == kEpiStoreBf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(a.z, a.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      if (R.copy != nullptr)
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(R.copy) + row * R.ld_copy + col) = pk;
      if (R.mode == kEpiStoreBf16)
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(R.out) + row * R.ld + col) = pk;
    }
    if (R.mode != kEpiStoreBf16) {
      float4* dst = reinterpret_cast<float4*>(static_cast<float*>(R.out) + row * R.ld + col);
      if (R.mode == kEpiAccumF32) {
        const float4 o = *dst;
        a.x += o.x;
        a.y += o.y;
        a.z += o.z;
        a.w += o.w;
      }
      *dst = a;
    }
  }
}

// ============================================================== host side
unsigned long long g_launch_count = 0;

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

static DeviceInfo g_devices[kMaxDevices] = {};

int current_device_index() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return (dev >= 0 && dev < kMaxDevices) ? dev : -1;
}

DeviceInfo* current_device_info() {
  const int dev = current_device_index();
  if (dev < 0) return nullptr;
  DeviceInfo& d = g_devices[dev];
  if (d.state == 0) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      d.state = -1;
    } else if (major != 10) {
      d.state = -1;
    } else {
      d.sms = sms;
      d.state = 1;
    }
  }
  return d.state > 0 ? &d : nullptr;
}

int device_check() { return current_device_info() != nullptr ? WSL_OK : WSL_ERR_DEVICE; }

Options& options() {
  static Options o = [] {
    Options v;
    const char* e = getenv("WSL_PAIR");
    v.pair_tiles = (e && e[0] == '0') ? 0 : 1;
    e = getenv("WSL_ROW_STAGED");
    v.row_staged = (e && e[0] == '0') ? 0 : 1;
    v.stall_producer = 0;
    v.wait_limit_ns = WAIT_LIMIT_NS;
    if ((e = getenv("WSL_WAIT_LIMIT_MS")) != nullptr) {
      const long ms = atol(e);
      if (ms > 0 && ms <= 10000) v.wait_limit_ns = static_cast<unsigned long long>(ms) * 1000000ull;
    }
    v.reserved_sms = 0;
    v.grid_waves = 0;
    v.merge_simt = 0;
    e = getenv("WSL_DEPENDENT_LAUNCH");
    v.dependent_launch = (e && e[0] == '0') ? 0 : 1;
    e = getenv("WSL_SPLIT_TAIL");
    v.split_tail = (e && e[0] == '0') ? 0 : 1;
    v.profile_bits = 0;
    if ((e = getenv("WSL_DBG")) != nullptr) v.profile_bits = atoi(e);
    return v;
  }();
  return o;
}

// SMs the persistent kernels of the current launch may occupy: all of them, minus the ones
// the caller reserved for a collective that runs beside them (wsl_set_option).
static int usable_sms(const DeviceInfo& d) {
  const int rsv = options().reserved_sms;
  int n = d.sms - (rsv > 0 ? rsv : 0);
  return n < 2 ? 2 : n;
}
// What every launcher sizes its grid with: the SMs of the current device minus the reserved ones.
int device_sm_count() {
  const DeviceInfo* d = current_device_info();
  return d ? usable_sms(*d) : 0;
}

static int ensure_encode() {
  if (g_encode) return WSL_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault,
                                       &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || fn == nullptr) {
    cudaGetLastError();
    return WSL_ERR_DRIVER;
  }
  g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  return WSL_OK;
}

// Tensor map over a row-major output matrix (bf16 or fp32) for the staged epilogue: box of
// 128 bytes x 128 rows, 128-byte swizzle.
// Encoded tensor maps are a pure function of (address, shape, pitch, box, type), and a training
// step presents the same few hundred combinations again and again (weights never move, the
// caching allocator hands activations the same addresses), so the 128-byte results are kept in
// a small direct-mapped table instead of being re-encoded by the driver on every launch.
struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_cols, box_rows, kind;   // kind: 0 bf16 operand, 1 bf16 output, 2 fp32 output
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_cols == o.box_cols &&
           box_rows == o.box_rows && kind == o.kind;
  }
};
struct MapSlot {
  MapKey key;
  int dev;
  bool used;
  alignas(64) CUtensorMap map;
};
constexpr int kMapSlots = 4096;
static MapSlot* g_map_cache = nullptr;
static std::mutex g_map_mutex;

static inline size_t map_hash(const MapKey& k, int dev) {
  unsigned long long h = reinterpret_cast<unsigned long long>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<unsigned long long>(k.rows) * 0xC2B2AE3D27D4EB4Full + (h >> 29);
  h ^= static_cast<unsigned long long>(k.cols) * 0x165667B19E3779F9ull + (h << 7);
  h ^= static_cast<unsigned long long>(k.ld) * 0x27D4EB2F165667C5ull + (h >> 31);
  h ^= static_cast<unsigned long long>((k.box_cols << 12) ^ (k.box_rows << 2) ^ k.kind ^ (dev << 24)) *
       0x85EBCA77C2B2AE63ull;
  return static_cast<size_t>((h ^ (h >> 32)) & (kMapSlots - 1));
}

// Looks the key up; on a miss runs `encode` into the slot. Returns a WSL_* status.
template <typename Encode>
static int cached_map(CUtensorMap* out, const MapKey& key, Encode encode) {
  const int dev = current_device_index();
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache == nullptr) g_map_cache = new MapSlot[kMapSlots]();
  MapSlot& s = g_map_cache[map_hash(key, dev)];
  if (!(s.used && s.dev == dev && s.key == key)) {
    CUresult res = encode(&s.map);
    if (res == CUDA_ERROR_INVALID_CONTEXT) {
      // A thread that has made no runtime call yet (an autograd worker whose first action is
      // one of these launches) has no context bound for the driver API: bind the device's
      // primary context the way the runtime does, then encode again.
      cudaFree(nullptr);
      res = encode(&s.map);
    }
    if (res != CUDA_SUCCESS) {
      s.used = false;
      // the one failure of this library that depends on a driver rule the caller cannot see:
      // say which tensor was refused
      fprintf(stderr,
              "wsl: cuTensorMapEncodeTiled refused a tensor (CUresult %d): ptr %p, %lld x %lld, pitch %lld "
              "elements, box %d x %d, kind %d\n",
              static_cast<int>(res), key.ptr, key.rows, key.cols, key.ld, key.box_cols, key.box_rows, key.kind);
      return WSL_ERR_DRIVER;
    }
    s.key = key;
    s.dev = dev;
    s.used = true;
  }
  memcpy(out, &s.map, sizeof(CUtensorMap));
  return WSL_OK;
}

// Tensor map over a row-major bf16 matrix with a box of 32 columns (64 bytes) x 128 rows and
// 64-byte swizzle: the half-width epilogue tiles of the SwiGLU backward.
static int make_map_half(CUtensorMap* m, void* ptr, long long rows, long long cols, long long ld) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2u};
  cuuint32_t box[2] = {32u, 128u};
  cuuint32_t estr[2] = {1, 1};
  const MapKey key = {ptr, rows, cols, ld, 32, 128, 3};
  return cached_map(m, key, [&](CUtensorMap* dst) {
    return g_encode(dst, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

static int make_map_out(CUtensorMap* m, void* ptr, long long rows, long long cols, long long ld,
                        bool f32) {
  const int es = f32 ? 4 : 2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), 128u};
  cuuint32_t estr[2] = {1, 1};
  const MapKey key = {ptr, rows, cols, ld, 128 / es, 128, f32 ? 2 : 1};
  return cached_map(m, key, [&](CUtensorMap* dst) {
    return g_encode(dst, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr,
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

// Tensor map over a row-major bf16 matrix [rows, cols] (pitch ld elements) with a
// box of box_cols (<= 64) x box_rows, 128-byte swizzle, zero fill outside.
static int make_map_bf16(CUtensorMap* m, const Mat& t, int box_cols, int box_rows) {
  if (t.ptr == nullptr || t.rows <= 0 || t.cols <= 0) return WSL_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0 || (t.ld % 8) != 0 || t.ld < t.cols)
    return WSL_ERR_ALIGN;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(t.cols), static_cast<cuuint64_t>(t.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(t.ld) * 2u};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  const MapKey key = {t.ptr, t.rows, t.cols, t.ld, box_cols, box_rows, 0};
  return cached_map(m, key, [&](CUtensorMap* dst) {
    return g_encode(dst, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(t.ptr), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

// Relative cost of one k-block of a tile with MMA N = bn: wide tiles are bound by the
// MMAs, narrow ones by their operand loads.
double tile_weight(long long no) {
  const long long n_tiles = (no + BN_MAX - 1) / BN_MAX;
  const double bn = static_cast<double>((no + n_tiles - 1) / n_tiles);
  return bn / BN_MAX < 0.4 ? 0.4 : bn / BN_MAX;
}

// Split-K plan of a launch. `tiles[i]`, `weight[i]`, `elems[i]`: tile count (in the kernel's
// own tiling), per-k-block cost weight and output elements of region i, in launch order.
// The first region gets S, narrow regions (weight < 1: bound by operand loads, cheap per
// unit) are split at least into one unit per worker so they spread over the whole GPU. The
// work units are dealt round-robin to `workers` exactly as the kernel does; the S with the
// smallest simulated makespan wins, charging the workspace round trip (partials written and
// read once at ~6.5 MB/us) and the reduce launch. One k-block of a full tile ~ 0.27 us.
// Returns the workspace bytes the plan needs (0 = no split anywhere).
// `kb_own` (may be null): the k-blocks region i really has when regions of different
// contraction lengths share a launch (kb_total = the longest). Such a region is split in
// proportion to its length, so that units stay about equally long, and a region that stays
// whole writes its output itself while the others go through the workspace.
size_t plan_splits(int nregion, const long long* tiles, const double* weight, const long long* elems,
                   int kb_total, size_t ws_limit_bytes, int workers, int* splits_out, const int* kb_own = nullptr) {
  for (int i = 0; i < nregion; ++i) splits_out[i] = 1;
  long long total = 0;
  for (int i = 0; i < nregion; ++i) total += tiles[i];
  if (total >= 6ll * workers || nregion > kMaxRegion) return 0;
  const int s_cap = kb_total / 8 < 16 ? (kb_total / 8 < 1 ? 1 : kb_total / 8) : 16;
  double best = 1e30;
  int best_s[kMaxRegion];
  size_t best_bytes = 0;
  for (int i = 0; i < nregion; ++i) best_s[i] = 1;
  double load[256];
  const int W = workers < 256 ? workers : 256;
  for (int S = 1; S <= s_cap; ++S) {
    int sr[kMaxRegion];
    size_t bytes = 0;
    bool any = false;
    for (int i = 0; i < nregion; ++i) {
      sr[i] = S;
      if (S > 1 && i > 0 && weight[i] < 1.0) {
        long long fine = (W + tiles[i] - 1) / tiles[i];
        if (fine > s_cap) fine = s_cap;
        if (fine > sr[i]) sr[i] = static_cast<int>(fine);
      }
      if (kb_own != nullptr) {
        // in proportion to the region's own length, never more splits than it has 8-block runs
        long long own = (static_cast<long long>(sr[i]) * kb_own[i] + kb_total / 2) / kb_total;
        const long long cap_i = kb_own[i] / 8 < 1 ? 1 : kb_own[i] / 8;
        if (own > cap_i) own = cap_i;
        sr[i] = own < 1 ? 1 : static_cast<int>(own);
      }
      if (sr[i] > 1) {
        bytes += static_cast<size_t>(sr[i]) * elems[i] * 4;
        any = true;
      }
    }
    if (any && kb_own == nullptr) {
      // regions of one length: either every region goes through the workspace or none
      bytes = 0;
      for (int i = 0; i < nregion; ++i) {
        if (sr[i] < 2) sr[i] = 2 <= s_cap ? 2 : 1;
        bytes += static_cast<size_t>(sr[i]) * elems[i] * 4;
      }
    }
    if (any && bytes > ws_limit_bytes) break;
    for (int w = 0; w < W; ++w) load[w] = 0.0;
    long long u = 0;
    for (int i = 0; i < nregion; ++i) {
      const int kbi = kb_own != nullptr ? kb_own[i] : kb_total;
      const double kb = static_cast<double>((kbi + sr[i] - 1) / sr[i]);
      for (long long j = 0; j < tiles[i] * sr[i]; ++j, ++u) load[u % W] += kb * weight[i] + 6.0;
    }
    double mk = 0.0;
    for (int w = 0; w < W; ++w) mk = load[w] > mk ? load[w] : mk;
    double t = mk * 0.27;
    if (any) t += 2.0 * static_cast<double>(bytes) / 6.5e6 + 4.0;
    if (t < best) {
      best = t;
      best_bytes = any ? bytes : 0;
      for (int i = 0; i < nregion; ++i) best_s[i] = sr[i];
    }
  }
  for (int i = 0; i < nregion; ++i) splits_out[i] = best_s[i];
  return best_bytes;
}

// How many times the co-resident CTA count a grid may have. One wave = the persistent form:
// every CTA (pair) walks its share of the statically dealt work units. With long tiles (many
// k-blocks) and several units per worker, TWO waves of half-as-long-lived CTAs let the
// hardware hand work to whichever SM frees up first, which evens out unequal tile times and
// SMs that another kernel (a collective) is holding; measured on B200 at the 8B-shape step
// 809.8 -> 802.2 ms alone and 801.1 -> 794.1 ms beside an overlapped all-reduce, while at the
// 0.6B shape (16-48 k-blocks per tile) the extra CTA set-up costs 0.5 %.
static int auto_grid_waves(int kb_total, long long units, long long cap) {
  const int opt = options().grid_waves;
  if (opt >= 1) return opt;
  return (kb_total >= 56 && units >= 4 * cap) ? 2 : 1;
}


// Makespan, in k-block units, of a launch whose work units come in `nseg` runs of `count[i]`
// units costing `cost[i]` each, dealt the way the kernel deals them: unit u belongs to CTA
// (pair) u % n_cta, n_cta = min(units, workers x grid waves); when the grid holds more CTAs
// than fit at once they start in index order, each as soon as an earlier one has finished.
static double simulate_makespan(int nseg, const long long* count, const double* cost, int kb_total,
                                int workers) {
  long long units = 0;
  for (int i = 0; i < nseg; ++i) units += count[i];
  if (units <= 0 || workers <= 0) return 0.0;
  const long long cap = static_cast<long long>(workers) * auto_grid_waves(kb_total, units, workers);
  const int n_cta = static_cast<int>(units < cap ? units : cap);
  constexpr int kMaxCta = 1024;
  if (n_cta > kMaxCta) return 1e30;
  double load[kMaxCta];
  for (int c = 0; c < n_cta; ++c) load[c] = 0.0;
  long long u = 0;
  for (int i = 0; i < nseg; ++i) {
    // whole passes over the CTAs cost every CTA the same; only the ragged ends go one by one
    long long left = count[i];
    while (left > 0 && (u % n_cta) != 0) { load[u % n_cta] += cost[i]; ++u; --left; }
    const long long passes = left / n_cta;
    if (passes > 0) {
      for (int c = 0; c < n_cta; ++c) load[c] += cost[i] * static_cast<double>(passes);
      u += passes * n_cta;
      left -= passes * n_cta;
    }
    while (left > 0) { load[u % n_cta] += cost[i]; ++u; --left; }
  }
  double mk = 0.0;
  if (n_cta <= workers) {
    for (int c = 0; c < n_cta; ++c) mk = load[c] > mk ? load[c] : mk;
    return mk;
  }
  // min-heap of the times at which the `workers` places become free
  double slot[kMaxCta];
  for (int w = 0; w < workers; ++w) slot[w] = 0.0;
  for (int c = 0; c < n_cta; ++c) {
    const double t = slot[0] + load[c];
    mk = t > mk ? t : mk;
    int i = 0;
    for (;;) {   // replace the root by t and sift it down
      const int l = 2 * i + 1, r = l + 1;
      int m = i;
      double mv = t;
      if (l < workers && slot[l] < mv) { m = l; mv = slot[l]; }
      if (r < workers && slot[r] < mv) { m = r; mv = slot[r]; }
      if (m == i) break;
      slot[i] = slot[m];
      i = m;
    }
    slot[i] = t;
  }
  return mk;
}

// What launch_block_gemm does with the contraction of a launch that was given a workspace.
// Either nothing, or every region is split (`splits`, the plan of plan_splits: launches with
// few tiles), or a TAIL: the last `tail_tiles` tiles (in rasterisation order) of region
// `tail_parent` leave their place in the launch order and run at its very end, each split
// `tail_splits` ways. A launch of many long tiles (a weight gradient contracts over every
// token) otherwise ends with a partial wave in which most CTAs idle for a whole tile time:
// 384 tile pairs on 74 CTA pairs take 6 waves for 5.2 waves of work. With the tail's tiles
// cut into short units the last wave is short too. Only the tail goes through the
// workspace (one dense [tile rows x 256] fp32 block per split and tile); everything else keeps
// its in-place epilogue, and the fixed-order fold keeps results bit-reproducible.
constexpr double kTailParentWeight = 0.75;   // only (nearly) full-width tiles are worth a tail
struct SplitPlan {
  int splits[kMaxRegion];   // per region of the launch (uniform plan), all 1 with a tail
  int tail_parent;          // -1: no tail
  int tail_tiles;
  int tail_splits;
  size_t bytes;             // workspace the plan needs
};

struct PlanKey {
  long long mo[kMaxRegion], no[kMaxRegion];
  int kb_own[kMaxRegion];
  size_t ws_limit;
  int nregion, kb_total, workers, pair, allow_tail, waves_opt, tail_opt;
};
struct PlanSlot {
  bool used;
  PlanKey key;
  SplitPlan plan;
};
constexpr int kPlanSlots = 256;
static PlanSlot g_plans[kPlanSlots] = {};
static std::mutex g_plan_mutex;

static SplitPlan plan_launch_uncached(int nregion, const long long* mo, const long long* no, int kb_total,
                                      size_t ws_limit, int workers, bool pair, bool allow_tail,
                                      const int* kb_own) {
  SplitPlan out;
  for (int i = 0; i < kMaxRegion; ++i) out.splits[i] = 1;
  out.tail_parent = -1;
  out.tail_tiles = 0;
  out.tail_splits = 1;
  out.bytes = 0;
  if (nregion < 1 || nregion > kMaxRegion || workers <= 0) return out;
  long long tiles[kMaxRegion], elems[kMaxRegion];
  double weight[kMaxRegion];
  const long long th = pair ? 2 * BM : BM;
  for (int i = 0; i < nregion; ++i) {
    tiles[i] = ((mo[i] + th - 1) / th) * ((no[i] + BN_MAX - 1) / BN_MAX);
    weight[i] = tile_weight(no[i]);
    elems[i] = mo[i] * no[i];
  }
  out.bytes = plan_splits(nregion, tiles, weight, elems, kb_total, ws_limit, workers, out.splits, kb_own);
  if (kb_own != nullptr) return out;   // regions of different lengths: all narrow, no tail
  if (!allow_tail || !options().split_tail || nregion + 1 > kMaxRegion || kb_total < 64) return out;
  // time of the plan so far, by the same clock as the candidates below
  long long cnt[kMaxRegion + 1];
  double cst[kMaxRegion + 1];
  for (int i = 0; i < nregion; ++i) {
    cnt[i] = tiles[i] * out.splits[i];
    cst[i] = static_cast<double>((kb_total + out.splits[i] - 1) / out.splits[i]) * weight[i] + 6.0;
  }
  double best = simulate_makespan(nregion, cnt, cst, kb_total, workers) * 0.27;
  if (out.bytes > 0) best += 2.0 * static_cast<double>(out.bytes) / 6.5e6 + 4.0;
  // The tail comes off the region with the most tiles. Launches that also carry narrow
  // regions (the rank-r products dB, dA beside dW) are left alone: their cheap units already
  // fill most of the last wave, and a tail measured between +9 % and -4 % on them.
  int parent = -1;
  for (int i = 0; i < nregion; ++i) {
    if (weight[i] < kTailParentWeight) return out;
    if (tiles[i] >= 2 && (parent < 0 || tiles[i] >= tiles[parent])) parent = i;
  }
  if (parent < 0) return out;
  long long t_max = workers + workers / 4;   // a wave of tiles and a little more
  if (t_max > tiles[parent] - 1) t_max = tiles[parent] - 1;
  static const int kTailSplits[] = {2, 3, 4, 5, 6, 8};
  const int s_cap = kb_total / 8 < 8 ? kb_total / 8 : 8;
  const size_t block_bytes = static_cast<size_t>(th) * BN_MAX * 4;
  double best_tail = 1e30;
  long long best_t = 0;
  int best_s = 1;
  for (long long t = 1; t <= t_max; ++t) {
    for (int si = 0; si < 6 && kTailSplits[si] <= s_cap; ++si) {
      const int S = kTailSplits[si];
      const size_t bytes = static_cast<size_t>(S) * t * block_bytes;
      if (bytes > ws_limit) break;
      for (int i = 0; i < nregion; ++i) {
        cnt[i] = i == parent ? tiles[i] - t : tiles[i];
        cst[i] = static_cast<double>(kb_total) * weight[i] + 6.0;
      }
      cnt[nregion] = t * S;
      cst[nregion] = static_cast<double>((kb_total + S - 1) / S) * weight[parent] + 6.0;
      const double tm = simulate_makespan(nregion + 1, cnt, cst, kb_total, workers) * 0.27 +
                        2.0 * static_cast<double>(bytes) / 6.5e6 + 4.0;
      if (tm < best_tail) {
        best_tail = tm;
        best_t = t;
        best_s = S;
      }
    }
  }
  // (measured gains are about half of what this model predicts: idle SMs in a partial wave
  // are not a pure loss on a power-capped part, the busy ones clock higher meanwhile)
  if (best_tail < 0.95 * best) {
    for (int i = 0; i < kMaxRegion; ++i) out.splits[i] = 1;
    out.tail_parent = parent;
    out.tail_tiles = static_cast<int>(best_t);
    out.tail_splits = best_s;
    out.bytes = static_cast<size_t>(best_s) * best_t * block_bytes;
  }
  return out;
}

// Plans repeat launch after launch (the same few shapes every layer, every step): a small
// table keyed by everything the plan depends on saves the search.
SplitPlan plan_launch(int nregion, const long long* mo, const long long* no, int kb_total, size_t ws_limit,
                      int workers, bool pair, bool allow_tail, const int* kb_own = nullptr) {
  PlanKey key;
  std::memset(&key, 0, sizeof(key));
  for (int i = 0; i < nregion && i < kMaxRegion; ++i) {
    key.mo[i] = mo[i];
    key.no[i] = no[i];
    key.kb_own[i] = kb_own != nullptr ? kb_own[i] : -1;
  }
  key.ws_limit = ws_limit;
  key.nregion = nregion;
  key.kb_total = kb_total;
  key.workers = workers;
  key.pair = pair ? 1 : 0;
  key.allow_tail = allow_tail ? 1 : 0;
  key.waves_opt = options().grid_waves;
  key.tail_opt = options().split_tail;
  unsigned long long h = 1469598103934665603ull;
  const unsigned char* kb = reinterpret_cast<const unsigned char*>(&key);
  for (size_t i = 0; i < sizeof(key); ++i) h = (h ^ kb[i]) * 1099511628211ull;
  // open addressing over a few neighbouring slots; a full neighbourhood overwrites its first
  constexpr int kProbe = 8;
  const unsigned home = static_cast<unsigned>(h % kPlanSlots);
  {
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (int i = 0; i < kProbe; ++i) {
      const PlanSlot& sl = g_plans[(home + i) % kPlanSlots];
      if (sl.used && std::memcmp(&sl.key, &key, sizeof(key)) == 0) return sl.plan;
    }
  }
  const SplitPlan plan = plan_launch_uncached(nregion, mo, no, kb_total, ws_limit, workers, pair, allow_tail, kb_own);
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  int put = 0;
  for (int i = 0; i < kProbe; ++i)
    if (!g_plans[(home + i) % kPlanSlots].used) { put = i; break; }
  PlanSlot& slot = g_plans[(home + put) % kPlanSlots];
  slot.used = true;
  slot.key = key;
  slot.plan = plan;
  return plan;
}

// The launch uses CTA pairs (256-row tiles) when its first region is large enough.
bool use_pair_tiles(long long mo0, long long no0);

long long region_tiles(bool pair, long long mo, long long no) {
  const long long tm = pair ? 2 * BM : BM;
  return ((mo + tm - 1) / tm) * ((no + BN_MAX - 1) / BN_MAX);
}
int split_workers(bool pair, int num_sms) { return pair ? num_sms / 2 : num_sms; }
int kblocks(long long k) { return static_cast<int>((k + BK - 1) / BK); }

template <bool A_MN, bool B_MN, bool PAIR>
static int launch_variant(const GemmParams& p, long long units, cudaStream_t stream) {
  static bool attr_set[kMaxDevices] = {};   // per instantiation and device
  auto kern = block_gemm_kernel<A_MN, B_MN, PAIR>;
  constexpr int smem = Cfg<PAIR>::kSmemBytes;
  const int dev = current_device_index();
  DeviceInfo* di = current_device_info();
  if (dev < 0 || di == nullptr) return WSL_ERR_DEVICE;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      cudaGetLastError();
      return WSL_ERR_CUDA;
    }
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().dependent_launch ? 2 : 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  long long workers;
  const int sms = usable_sms(*di);
  if (PAIR) {
    if (di->max_clusters == 0) {
      cfg.gridDim = dim3(2 * (di->sms / 2));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = di->sms / 2;
      }
      di->max_clusters = n < di->sms / 2 ? n : di->sms / 2;
    }
    const long long fit = di->max_clusters < sms / 2 ? di->max_clusters : sms / 2;
    const long long cap = fit * auto_grid_waves(p.kb_total, units, fit);
    workers = units < cap ? units : cap;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * workers));
  } else {
    const long long cap1 = static_cast<long long>(sms) * auto_grid_waves(p.kb_total, units, sms);
    workers = units < cap1 ? units : cap1;
    cfg.gridDim = dim3(static_cast<unsigned>(workers));
  }
  if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
    cudaGetLastError();
    return WSL_ERR_CUDA;
  }
  ++g_launch_count;
  return WSL_OK;
}

static bool pair_mode_enabled() { return options().pair_tiles != 0; }

bool use_pair_tiles(long long mo0, long long no0) {
  static const long long min_n = getenv("WSL_PAIR_MIN_N") ? atoll(getenv("WSL_PAIR_MIN_N")) : 128;   // EXPERIMENT
  return pair_mode_enabled() && mo0 >= 512 && no0 >= min_n;
}

int launch_block_gemm(const GemmDesc& g, cudaStream_t stream) {
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return WSL_ERR_DEVICE;
  const int g_num_sms = usable_sms(*di);   // what the split planner and the grids may count on
  int st = ensure_encode();
  if (st != WSL_OK) return st;
  if (g.nseg < 1 || g.nseg > kMaxSeg || g.nregion < 1 || g.nregion > kMaxRegion)
    return WSL_ERR_BAD_ARG;
  if (g.nseg * g.nregion * 2 + g.nregion > kMaxMaps) return WSL_ERR_BAD_ARG;

  GemmParams p;
  p.nseg = g.nseg;
  p.nregion = g.nregion;
  for (int s = 0; s < kMaxSeg; ++s) p.seg_k[s] = s < g.nseg ? g.seg_k[s] : 0;
  for (int s = 0; s < g.nseg; ++s)
    if (g.seg_k[s] <= 0) return WSL_ERR_BAD_ARG;

  // CTA pairs (256-row tiles) for the large GEMMs; single CTAs for narrow/short ones.
  if (g.gather_tokens != nullptr) {
    if ((g.gather_a && g.a_mn) || (g.gather_b && !g.b_mn) || (g.gather_a && g.gather_b) ||
        g.gather_count <= 0)
      return WSL_ERR_BAD_ARG;
  }
  // The weight-merge launch (out = alpha acc + addend, one or two k-blocks per tile) is a
  // streaming pass bound by how far ahead its addend tiles are fetched: it runs on single
  // CTAs with a 2-stage operand ring and 8 staging slots instead of 4 stages and 2 slots.
  int kb_all = 0;
  for (int sgi = 0; sgi < g.nseg; ++sgi) kb_all += (g.seg_k[sgi] + BK - 1) / BK;
  const bool deep_epilogue = g.region[0].addend != nullptr && g.region[0].mode == kEpiStoreBf16 && kb_all <= 4;
  const bool pair = !deep_epilogue && use_pair_tiles(g.region[0].mo, g.region[0].no);
  const int bm_tile = pair ? 2 * BM : BM;
  const int bn_round = pair ? 32 : 16;
  // Split plan of a launch that brought a workspace.
  SplitPlan plan;
  for (int r = 0; r < kMaxRegion; ++r) plan.splits[r] = 1;
  plan.tail_parent = -1;
  plan.tail_tiles = 0;
  plan.tail_splits = 1;
  plan.bytes = 0;
  // regions of different contraction lengths in one launch: each one's own k-blocks
  const bool ragged = g.ragged_k && g.nseg == 1;
  int kb_own[kMaxRegion];
  for (int r = 0; r < g.nregion; ++r) {
    const long long ak = g.a_mn ? g.region[r].a[0].rows : g.region[r].a[0].cols;
    long long kb = (ak + BK - 1) / BK;
    kb = kb < 1 ? 1 : (kb > kb_all ? kb_all : kb);
    kb_own[r] = ragged ? static_cast<int>(kb) : kb_all;
  }
  if (g.workspace != nullptr) {
    long long pmo[kMaxRegion], pno[kMaxRegion];
    bool plain = g.gather_tokens == nullptr;   // a tail needs ordinary regions
    for (int r = 0; r < g.nregion; ++r) {
      const RegionDesc& rd = g.region[r];
      pmo[r] = rd.mo;
      pno[r] = rd.no;
      plain = plain && rd.addend == nullptr && !rd.transposed && rd.mode >= kEpiStoreBf16 && rd.mode <= kEpiAccumF32;
    }
    plan = plan_launch(g.nregion, pmo, pno, kb_all, g.workspace_bytes, split_workers(pair, g_num_sms), pair, plain,
                       ragged ? kb_own : nullptr);
  }
  int nmaps = 0;
  long long tiles = 0;
  for (int r = 0; r < g.nregion; ++r) {
    const RegionDesc& rd = g.region[r];
    Region& R = p.reg[r];
    if (rd.mo <= 0 || rd.no <= 0 || rd.out == nullptr) return WSL_ERR_BAD_ARG;
    const int vec = (rd.mode == kEpiStoreBf16 || rd.mode == kEpiSwiGLU || rd.mode == kEpiSwiGLUBwd) ? 8 : 4;
    if (rd.transposed) {
      if (rd.mode == kEpiStoreBf16) return WSL_ERR_BAD_ARG;
      if ((rd.mo % 4) != 0 || (rd.ld_out % 4) != 0 || rd.ld_out < rd.mo ||
          (reinterpret_cast<uintptr_t>(rd.out) & 15u) != 0)
        return WSL_ERR_ALIGN;
    } else if ((rd.no % vec) != 0 || (rd.ld_out % vec) != 0 || rd.ld_out < rd.no ||
               (reinterpret_cast<uintptr_t>(rd.out) & 15u) != 0) {
      return WSL_ERR_ALIGN;
    }
    const bool swiglu = rd.mode == kEpiSwiGLU;
    if ((rd.addend != nullptr) != (g.region[0].addend != nullptr) || rd.mode != g.region[0].mode && rd.addend != nullptr)
      return WSL_ERR_BAD_ARG;
    if ((rd.mode == kEpiSwiGLUBwd) != (rd.addend2 != nullptr)) return WSL_ERR_BAD_ARG;
    if (rd.addend != nullptr) {
      if ((rd.mode != kEpiStoreBf16 && rd.mode != kEpiSwiGLUBwd) || rd.transposed || rd.copy != nullptr ||
          g.workspace != nullptr)
        return WSL_ERR_BAD_ARG;
      if ((reinterpret_cast<uintptr_t>(rd.addend) & 15u) != 0 || (rd.ld_addend % 8) != 0 || rd.ld_addend < rd.no)
        return WSL_ERR_ALIGN;
      if (rd.mode == kEpiSwiGLUBwd &&
          (rd.out2 == nullptr || ((reinterpret_cast<uintptr_t>(rd.addend2) | reinterpret_cast<uintptr_t>(rd.out2)) & 15u) != 0))
        return WSL_ERR_ALIGN;
    }
    if (swiglu) {
      if (!pair || g.a_mn || g.b_mn || rd.transposed || rd.copy != nullptr || (rd.no % 128) != 0 ||
          rd.out2 == nullptr || rd.out3 == nullptr || g.workspace != nullptr)
        return WSL_ERR_BAD_ARG;
      if (((reinterpret_cast<uintptr_t>(rd.out2) | reinterpret_cast<uintptr_t>(rd.out3)) & 15u) != 0)
        return WSL_ERR_ALIGN;
    }
    long long n_tiles = (rd.no + BN_MAX - 1) / BN_MAX;
    long long bn = (rd.no + n_tiles - 1) / n_tiles;
    bn = (bn + bn_round - 1) / bn_round * bn_round;
    if (rd.addend != nullptr) bn = (bn + 63) / 64 * 64;   // whole staging chunks (64 or 32 columns)
    if (swiglu) {   // one tile = 128 output columns of g next to the same 128 of u
      n_tiles = rd.no / 128;
      bn = BN_MAX;
    }
    const long long m_tiles = (rd.mo + bm_tile - 1) / bm_tile;
    if (m_tiles * n_tiles + tiles > 0x7fffffffLL) return WSL_ERR_TOO_LARGE;
    R.m_tiles = static_cast<int>(m_tiles);
    R.n_tiles = static_cast<int>(n_tiles);
    R.tile_begin = static_cast<int>(tiles);
    R.bn = static_cast<int>(bn);
    R.rows = static_cast<int>(rd.mo);
    R.cols = static_cast<int>(rd.no);
    R.out = rd.out;
    R.ld = rd.ld_out;
    R.mode = rd.mode;
    R.alpha = rd.alpha;
    R.ws_off = 0;
    R.transposed = rd.transposed ? 1 : 0;
    R.out_map = -1;
    R.swiglu = swiglu ? 1 : 0;
    R.addend_map = -1;
    for (int s = 0; s < kMaxSeg; ++s) {
      R.b2_map[s] = 0;
      R.b2_shift[s] = 0;
    }
    if (rd.copy != nullptr) {
      if (rd.transposed || rd.mode == kEpiStoreBf16) return WSL_ERR_BAD_ARG;
      if ((rd.no % 8) != 0 || (rd.ld_copy % 8) != 0 || rd.ld_copy < rd.no ||
          (reinterpret_cast<uintptr_t>(rd.copy) & 15u) != 0)
        return WSL_ERR_ALIGN;
    }
    R.copy = rd.copy;
    R.ld_copy = rd.ld_copy;
    {
      // A rows of one group (all contraction segments) should sit in about a third of the
      // 126 MB L2 while the B tiles stream past them; at least one wave of workers wide.
      long long ktot = 0;
      for (int sgi = 0; sgi < g.nseg; ++sgi) ktot += g.seg_k[sgi];
      long long grp = (40ll << 20) / (2 * ktot * bm_tile);
      if (grp < 4) grp = 4;
      if (grp > (pair ? 16 : 32)) grp = pair ? 16 : 32;   // keep a wave a 2-D patch of tiles
      if (grp > m_tiles) grp = m_tiles;
      R.group = static_cast<int>(grp);
    }
    tiles += m_tiles * n_tiles;
    for (int s = 0; s < kMaxSeg; ++s) {
      R.a_map[s] = 0;
      R.b_map[s] = 0;
    }
    for (int s = 0; s < g.nseg; ++s) {
      const Mat& a = rd.a[s];
      const Mat& b = rd.b[s];
      // Shape checks: K-major operand is [mo|no, k]; MN-major operand is [k, mo|no].
      // (a gathered operand is the source matrix [V, cols]; its row count is free)
      const bool ga0 = g.gather_tokens != nullptr && g.gather_a && r == 0 && s == 0;
      const bool gb0 = g.gather_tokens != nullptr && g.gather_b && r == 0 && s == 0;
      const long long ak = g.a_mn ? a.rows : a.cols, bk = g.b_mn ? b.rows : b.cols;
      const bool a_k_ok = g.a_mn ? (ga0 ? true : ak == g.seg_k[s]) : ak == g.seg_k[s];
      const bool b_k_ok = g.b_mn ? (gb0 ? true : bk == g.seg_k[s]) : bk == g.seg_k[s];
      const bool ragged_ok = g.ragged_k && ak == bk && ak > 0 && ak <= g.seg_k[s];
      // gate|up tiles: each of the two B matrices may cover only part of the segment
      const bool dual_ok = swiglu && a_k_ok && bk > 0 && bk <= g.seg_k[s] && rd.b2[s].rows == rd.no &&
                           rd.b2[s].cols > 0 && rd.b2_k_shift[s] >= 0 && (rd.b2_k_shift[s] % 8) == 0 &&
                           rd.b2_k_shift[s] + rd.b2[s].cols <= g.seg_k[s];
      if (swiglu ? !dual_ok : !((a_k_ok && b_k_ok) || ragged_ok)) return WSL_ERR_BAD_ARG;
      if (g.a_mn ? a.cols != rd.mo : (!ga0 && a.rows != rd.mo)) return WSL_ERR_BAD_ARG;
      if (g.b_mn ? b.cols != rd.no : b.rows != rd.no) return WSL_ERR_BAD_ARG;
      const bool ga = g.gather_tokens != nullptr && g.gather_a && r == 0 && s == 0;
      const bool gb = g.gather_tokens != nullptr && g.gather_b && r == 0 && s == 0;
      if (ga) st = make_map_bf16(&p.maps[nmaps], a, BK, 1);          // gather4: box of one row
      else st = g.a_mn ? make_map_bf16(&p.maps[nmaps], a, 64, BK) : make_map_bf16(&p.maps[nmaps], a, BK, BM);
      if (st != WSL_OK) return st;
      R.a_map[s] = static_cast<signed char>(nmaps++);
      if (gb) st = make_map_bf16(&p.maps[nmaps], b, 64, 1);
      else st = g.b_mn ? make_map_bf16(&p.maps[nmaps], b, 64, BK)
                       : make_map_bf16(&p.maps[nmaps], b, BK, static_cast<int>(pair ? bn / 2 : bn));
      if (st != WSL_OK) return st;
      R.b_map[s] = static_cast<signed char>(nmaps++);
      if (swiglu) {
        if (nmaps + 4 > kMaxMaps) return WSL_ERR_BAD_ARG;
        st = make_map_bf16(&p.maps[nmaps], rd.b2[s], BK, static_cast<int>(bn / 2));
        if (st != WSL_OK) return st;
        R.b2_map[s] = static_cast<signed char>(nmaps++);
        R.b2_shift[s] = rd.b2_k_shift[s];
      }
    }
  }
  p.total_tiles = static_cast<int>(tiles);
  int kb_total = 0;
  for (int sgi = 0; sgi < g.nseg; ++sgi) kb_total += (g.seg_k[sgi] + BK - 1) / BK;
  p.kb_total = kb_total;
  {
    int max_bn = 0;
    for (int r = 0; r < g.nregion; ++r) max_bn = p.reg[r].bn > max_bn ? p.reg[r].bn : max_bn;
    const bool narrow = !pair && max_bn <= NARROW_BN;
    p.stages = narrow ? NARROW_STAGES : Cfg<false>::kStages;
    p.stage_bytes = narrow ? NARROW_STAGE_BYTES : Cfg<false>::kStageBytes;
    p.epi_slots = 2;
    if (deep_epilogue) {
      p.stages = 2;
      p.stage_bytes = Cfg<false>::kStageBytes;
      p.epi_slots = (Cfg<false>::kStages - 2) * Cfg<false>::kStageBytes / EPI_STAGE_BYTES + 2;   // 8
    }
  }
  p.workspace = plan.bytes > 0 ? g.workspace : nullptr;
  bool any_split = false;
  int tail_region = -1;
  {
    // regions that are split keep their partials in the workspace one after the other;
    // the others write their outputs themselves
    long long off = 0, ub = 0;
    for (int r = 0; r < g.nregion; ++r) {
      Region& R = p.reg[r];
      R.splits = plan.splits[r];
      R.unit_begin = static_cast<int>(ub);
      R.ws_off = off;
      R.tile_off = 0;
      R.tile_count = R.m_tiles * R.n_tiles;
      R.tail = 0;
      R.kb_own = kb_own[r];
      if (R.splits > R.kb_own) return WSL_ERR_BAD_ARG;   // every split owns at least one block
      if (r == plan.tail_parent) R.tile_count -= plan.tail_tiles;
      any_split = any_split || R.splits > 1;
      if (R.splits > 1) off += static_cast<long long>(R.splits) * g.region[r].mo * g.region[r].no;
      ub += static_cast<long long>(R.tile_count) * R.splits;
    }
    if (plan.tail_parent >= 0) {
      // the tail: a second entry for the parent region, last in the launch order
      if (g.nregion + 1 > kMaxRegion || any_split || plan.tail_tiles < 1 ||
          plan.tail_tiles >= p.reg[plan.tail_parent].m_tiles * p.reg[plan.tail_parent].n_tiles)
        return WSL_ERR_BAD_ARG;
      tail_region = g.nregion;
      Region& T = p.reg[tail_region];
      T = p.reg[plan.tail_parent];
      T.tile_off = p.reg[plan.tail_parent].tile_count;
      T.tile_count = plan.tail_tiles;
      T.tail = 1;
      T.splits = plan.tail_splits;
      T.unit_begin = static_cast<int>(ub);
      T.ws_off = 0;
      off = static_cast<long long>(T.splits) * T.tile_count * bm_tile * BN_MAX;
      ub += static_cast<long long>(T.tile_count) * T.splits;
      p.nregion = g.nregion + 1;
    }
    if (ub > 0x7fffffffLL) return WSL_ERR_TOO_LARGE;
    if (off > 0 && static_cast<size_t>(off) * 4 > g.workspace_bytes) return WSL_ERR_BAD_ARG;
    p.total_units = static_cast<int>(ub);
  }
  p.gather_tokens = g.gather_tokens;
  p.gather_count = g.gather_count;
  p.gather_a = g.gather_a ? 1 : 0;
  p.gather_b = g.gather_b ? 1 : 0;
  const Options& opt = options();
  p.dbg = opt.profile_bits & (1 | 2 | 4 | 32);
  p.stall_producer = opt.stall_producer;
  p.wait_limit_ns = opt.wait_limit_ns;
#ifndef WSL_PROFILE_SWITCHES
  p.dbg = 0;
#endif
  if (!(p.dbg & 32)) {
    // staged TMA-store epilogue where the tile width is a whole number of 128-byte chunks
    // (split regions write fp32 partials to the workspace with plain stores instead)
    for (int r = 0; r < g.nregion; ++r) {
      const RegionDesc& rd = g.region[r];
      if (p.reg[r].splits > 1) continue;
      if (rd.mode == kEpiSwiGLU || rd.mode == kEpiSwiGLUBwd) continue;   // their maps are made below
      const bool f32 = rd.mode != kEpiStoreBf16;
      if (rd.transposed || (p.reg[r].bn % (f32 ? 32 : 64)) != 0) continue;
      st = make_map_out(&p.maps[nmaps], rd.out, rd.mo, rd.no, rd.ld_out, f32);
      if (st != WSL_OK) return st;
      p.reg[r].out_map = nmaps++;
    }
  }
  p.aux_mode = g.region[0].addend == nullptr ? 0 : (g.region[0].mode == kEpiSwiGLUBwd ? 2 : 1);
  for (int r = 0; r < g.nregion && p.aux_mode == 1; ++r) {
    const RegionDesc& rd = g.region[r];
    if (p.reg[r].out_map < 0 || nmaps + 1 > kMaxMaps) return WSL_ERR_BAD_ARG;
    st = make_map_out(&p.maps[nmaps], const_cast<void*>(rd.addend), rd.mo, rd.no, rd.ld_addend, false);
    if (st != WSL_OK) return st;
    p.reg[r].addend_map = nmaps++;
  }
  for (int r = 0; r < g.nregion && p.aux_mode == 2; ++r) {
    // g, u in and d gate, d up out: four maps over [mo, no] bf16 matrices with boxes of 32
    // columns x 128 rows, 64-byte swizzle (two of them share a 16 KiB staging slot)
    const RegionDesc& rd = g.region[r];
    if (any_split || nmaps + 4 > kMaxMaps) return WSL_ERR_BAD_ARG;
    p.reg[r].addend_map = nmaps;
    st = make_map_half(&p.maps[nmaps++], const_cast<void*>(rd.addend), rd.mo, rd.no, rd.ld_addend);
    if (st == WSL_OK) st = make_map_half(&p.maps[nmaps++], const_cast<void*>(rd.addend2), rd.mo, rd.no, rd.ld_addend);
    p.reg[r].out_map = nmaps;
    if (st == WSL_OK) st = make_map_half(&p.maps[nmaps++], rd.out, rd.mo, rd.no, rd.ld_out);
    if (st == WSL_OK) st = make_map_half(&p.maps[nmaps++], rd.out2, rd.mo, rd.no, rd.ld_out);
    if (st != WSL_OK) return st;
  }
  for (int r = 0; r < g.nregion; ++r) {
    const RegionDesc& rd = g.region[r];
    if (rd.mode != kEpiSwiGLU) continue;
    if (nmaps + 3 > kMaxMaps) return WSL_ERR_BAD_ARG;
    void* outs[3] = {rd.out, rd.out2, rd.out3};
    p.reg[r].out_map = nmaps;
    for (int i = 0; i < 3; ++i) {
      st = make_map_out(&p.maps[nmaps++], outs[i], rd.mo, rd.no, rd.ld_out, false);
      if (st != WSL_OK) return st;
    }
  }
  const long long units = p.total_units;
#define WSL_LAUNCH(AM, BM_) (pair ? launch_variant<AM, BM_, true>(p, units, stream) \
                                  : launch_variant<AM, BM_, false>(p, units, stream))
  if (g.a_mn && g.b_mn) st = WSL_LAUNCH(true, true);
  else if (!g.a_mn && g.b_mn) st = WSL_LAUNCH(false, true);
  else if (!g.a_mn && !g.b_mn) st = WSL_LAUNCH(false, false);
  else st = WSL_LAUNCH(true, false);
#undef WSL_LAUNCH
  if (st != WSL_OK) return st;
  if (tail_region >= 0) {
    constexpr int kParts = 16;   // blocks per tail tile: a few hundred blocks for 10-90 tiles
    const unsigned blocks = static_cast<unsigned>(p.reg[tail_region].tile_count) * kParts;
    if (pair) launch_dependent(tail_reduce_kernel<true>, dim3(blocks), dim3(256), 0, stream, p, tail_region, kParts);
    else launch_dependent(tail_reduce_kernel<false>, dim3(blocks), dim3(256), 0, stream, p, tail_region, kParts);
    if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
    ++g_launch_count;
    return WSL_OK;
  }
  if (!any_split) return st;
  ReduceParams rp;
  rp.nregion = 0;
  long long total = 0;
  for (int r = 0; r < g.nregion; ++r) {
    if (p.reg[r].splits < 2) continue;
    const RegionDesc& rd = g.region[r];
    // output orientation: a transposed region's result matrix is [no, mo]
    const long long orows = rd.transposed ? rd.no : rd.mo;
    const long long ocols = rd.transposed ? rd.mo : rd.no;
    ReduceRegion& R = rp.reg[rp.nregion++];
    R.ws = reinterpret_cast<const float4*>(p.workspace + p.reg[r].ws_off);
    R.out = rd.out;
    R.ld = rd.ld_out;
    R.begin = total;
    R.rows = static_cast<int>(orows);
    R.cols4 = static_cast<int>(ocols / 4);
    R.mode = rd.mode;
    R.alpha = rd.alpha;
    R.splits = p.reg[r].splits;
    R.copy = static_cast<__nv_bfloat16*>(rd.copy);
    R.ld_copy = rd.ld_copy;
    total += orows * (ocols / 4);
  }
  rp.total = total;
  long long blocks = (total + 255) / 256;
  if (blocks > 8ll * g_num_sms) blocks = 8ll * g_num_sms;
  launch_dependent(splitk_reduce_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, rp);
  if (cudaGetLastError() != cudaSuccess) return WSL_ERR_CUDA;
  ++g_launch_count;
  return WSL_OK;
}

}  // namespace wsl
