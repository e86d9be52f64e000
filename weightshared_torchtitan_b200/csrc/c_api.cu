// The extern "C" surface declared in include/wsl.h. This file is the single
// translation unit of libwsl.so: it pulls in the kernel sources so that the
// device-side status words are one definition without relocatable device code.
#include "block_gemm.cu"
#include "simt_gemm.cu"
#include "embed.cu"
#include "static_scratch.cu"
#include "elementwise.cu"
#include "lora_merge.cu"
#include "flat_adamw.cu"

namespace wsl {
int launch_simt_gemm_f32(const float* A, long long sai, long long sak, const float* B,
                         long long sbj, long long sbk, float* C, long long ldc, long long M,
                         long long N, long long K, float alpha, int accumulate,
                         cudaStream_t stream);

static inline Mat mat(const void* p, long long rows, long long cols, long long ld) {
  Mat m;
  m.ptr = p;
  m.rows = rows;
  m.cols = cols;
  m.ld = ld;
  return m;
}
// The regions of a weight-gradient launch (token contraction, MN-major operands), for P
// projections that read the same x:
//   dW_p[N_p,K] += dY_p^T x ;  dB_p[N_p,r_p] += dY_p^T T_p ;  dA_p[r_p,K] += U_p^T x, run as its
//   transpose x^T U_p -> [K, r_p] so that the narrow dimension r is the MMA N (cheap) instead
//   of a mostly-empty 128-row M tile.
// All wide (dW) regions come first, then the narrow ones, so the round-robin deal hands out
// the expensive units before the cheap ones.
struct BwdDwProj {
  const void* dY; long long lddy;
  const void* U; long long ldu;
  const void* T; long long ldt;
  float* dW; float* dA; float* dB;
  long long N; long long r;
  void* dWl;   // optional bf16 copy [N, K] of this call's dY^T x (see RegionDesc::copy)
};

int build_bwd_dw_group(GemmDesc& g, int nproj, const BwdDwProj* pj, const void* x, long long ldx,
                       long long M, long long K) {
  g.a_mn = true;
  g.b_mn = true;
  g.nseg = 1;
  g.seg_k[0] = static_cast<int>(M);
  int nr = 0;
  auto add = [&](const void* a, long long a_cols, long long lda, const void* b, long long b_cols,
                 long long ldb, float* out, long long ld_out, bool transposed, void* copy = nullptr) {
    RegionDesc& rd = g.region[nr++];
    rd.copy = copy;
    rd.ld_copy = copy ? ld_out : 0;
    rd.a[0].ptr = a;
    rd.a[0].rows = M;
    rd.a[0].cols = a_cols;
    rd.a[0].ld = lda;
    rd.b[0].ptr = b;
    rd.b[0].rows = M;
    rd.b[0].cols = b_cols;
    rd.b[0].ld = ldb;
    rd.mo = a_cols;
    rd.no = b_cols;
    rd.out = out;
    rd.ld_out = ld_out;
    rd.mode = kEpiAccumF32;
    rd.alpha = 1.f;
    rd.transposed = transposed;
  };
  int want = 0;
  for (int p = 0; p < nproj; ++p) want += (pj[p].dW ? 1 : 0) + (pj[p].dB ? 1 : 0) + (pj[p].dA ? 1 : 0);
  if (want == 0 || want > kMaxRegion) return WSL_ERR_BAD_ARG;
  for (int p = 0; p < nproj; ++p)
    if (pj[p].dW) add(pj[p].dY, pj[p].N, pj[p].lddy, x, K, ldx, pj[p].dW, K, false, pj[p].dWl);
  for (int p = 0; p < nproj; ++p)
    if (pj[p].dB) add(pj[p].dY, pj[p].N, pj[p].lddy, pj[p].T, pj[p].r, pj[p].ldt, pj[p].dB, pj[p].r, false);
  for (int p = 0; p < nproj; ++p)
    if (pj[p].dA) add(x, K, ldx, pj[p].U, pj[p].r, pj[p].ldu, pj[p].dA, K, true);
  g.nregion = nr;
  return WSL_OK;
}

void build_bwd_dw_desc(GemmDesc& g, const void* dY, long long lddy, const void* U, long long ldu,
                       const void* x, long long ldx, const void* T, long long ldt, float* dW,
                       float* dA, float* dB, long long M, long long N, long long K, long long r) {
  BwdDwProj pj = {dY, lddy, U, ldu, T, ldt, dW, dA, dB, N, r, nullptr};
  build_bwd_dw_group(g, 1, &pj, x, ldx, M, K);
}

static inline bool bad_dtype(int dtype) { return dtype != WSL_BF16 && dtype != WSL_F32; }
static inline const float* f32(const void* p) { return static_cast<const float*>(p); }
}  // namespace wsl

using namespace wsl;

extern "C" {

int wsl_version(void) { return (0 << 16) | 4; }

const char* wsl_status_string(int status) {
  switch (status) {
    case WSL_OK: return "ok";
    case WSL_ERR_BAD_ARG: return "bad argument (null pointer, non-positive or inconsistent size)";
    case WSL_ERR_ALIGN: return "pointer or pitch violates the 16-byte alignment rule";
    case WSL_ERR_DEVICE: return "no CUDA device or current device is not sm_100";
    case WSL_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
    case WSL_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case WSL_ERR_DRIVER: return "cuTensorMapEncodeTiled unavailable or rejected the tensor";
    case WSL_ERR_TOO_LARGE: return "size beyond a fixed limit of the library";
    default: return "unknown status";
  }
}

unsigned long long wsl_launch_count(void) { return g_launch_count; }

int wsl_poll_status(int words[4]) {
  int st = device_check();
  if (st != WSL_OK) return st;
  int w[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(w, g_wsl_status, sizeof(w)) != cudaSuccess) {
    cudaGetLastError();
    return WSL_ERR_CUDA;
  }
  if (words)
    for (int i = 0; i < 4; ++i) words[i] = w[i];
  return w[0];
}

int wsl_set_option(int option, long long value) {
  Options& o = options();
  switch (option) {
    case WSL_OPT_WAIT_LIMIT_MS:
      if (value <= 0 || value > 10000) return WSL_ERR_BAD_ARG;
      o.wait_limit_ns = static_cast<unsigned long long>(value) * 1000000ull;
      return WSL_OK;
    case WSL_OPT_STALL_PRODUCER: o.stall_producer = value != 0; return WSL_OK;
    case WSL_OPT_PAIR_TILES: o.pair_tiles = value != 0; return WSL_OK;
    case WSL_OPT_ROW_STAGED: o.row_staged = value != 0; return WSL_OK;
    case WSL_OPT_RESERVED_SMS:
      if (value < 0 || value > 64) return WSL_ERR_BAD_ARG;
      o.reserved_sms = static_cast<int>(value);
      return WSL_OK;
    case WSL_OPT_PROFILE_BITS: o.profile_bits = static_cast<int>(value); return WSL_OK;
    case WSL_OPT_MERGE_SIMT: o.merge_simt = value != 0; return WSL_OK;
    case WSL_OPT_GRID_WAVES:
      if (value < 0 || value > 8) return WSL_ERR_BAD_ARG;
      o.grid_waves = static_cast<int>(value);
      return WSL_OK;
    case WSL_OPT_SPLIT_TAIL: o.split_tail = value != 0; return WSL_OK;
    case WSL_OPT_DEPENDENT_LAUNCH: o.dependent_launch = value != 0; return WSL_OK;
    default: return WSL_ERR_BAD_ARG;
  }
}

long long wsl_get_option(int option) {
  const Options& o = options();
  switch (option) {
    case WSL_OPT_WAIT_LIMIT_MS: return static_cast<long long>(o.wait_limit_ns / 1000000ull);
    case WSL_OPT_STALL_PRODUCER: return o.stall_producer;
    case WSL_OPT_PAIR_TILES: return o.pair_tiles;
    case WSL_OPT_ROW_STAGED: return o.row_staged;
    case WSL_OPT_RESERVED_SMS: return o.reserved_sms;
    case WSL_OPT_PROFILE_BITS: return o.profile_bits;
    case WSL_OPT_MERGE_SIMT: return o.merge_simt;
    case WSL_OPT_GRID_WAVES: return o.grid_waves;
    case WSL_OPT_SPLIT_TAIL: return o.split_tail;
    case WSL_OPT_DEPENDENT_LAUNCH: return o.dependent_launch;
    default: return WSL_ERR_BAD_ARG;
  }
}

int wsl_reset_status(void) {
  int st = device_check();
  if (st != WSL_OK) return st;
  const int w[4] = {0, 0, 0, 0};
  if (cudaMemcpyToSymbol(g_wsl_status, w, sizeof(w)) != cudaSuccess) {
    cudaGetLastError();
    return WSL_ERR_CUDA;
  }
  return WSL_OK;
}

int wsl_linear_fwd(const void* x, long long ldx, const void* W, void* y, long long ldy,
                   long long M, long long N, long long K, int out_f32, int dtype, void* stream) {
  if (bad_dtype(dtype) || !x || !W || !y || M <= 0 || N <= 0 || K <= 0) return WSL_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == WSL_F32)
    return launch_simt_gemm_f32(f32(x), ldx, 1, f32(W), K, 1, static_cast<float*>(y), ldy, M, N, K,
                                1.f, 0, s);
  GemmDesc g = {};
  g.a_mn = false;
  g.b_mn = false;
  g.nseg = 1;
  g.seg_k[0] = static_cast<int>(K);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(x, M, K, ldx);
  r0.b[0] = mat(W, N, K, K);
  r0.mo = M;
  r0.no = N;
  r0.out = y;
  r0.ld_out = ldy;
  r0.mode = out_f32 ? kEpiStoreF32 : kEpiStoreBf16;
  r0.alpha = 1.f;
  return launch_block_gemm(g, s);
}

int wsl_lora_prepass(const void* x, long long ldx, const void* A_cat, void* T, long long ldt,
                     long long M, long long K, long long r_tot, float sc, int dtype,
                     void* stream) {
  if (bad_dtype(dtype) || !x || !A_cat || !T || M <= 0 || K <= 0 || r_tot <= 0)
    return WSL_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == WSL_F32)
    return launch_simt_gemm_f32(f32(x), ldx, 1, f32(A_cat), K, 1, static_cast<float*>(T), ldt, M,
                                r_tot, K, sc, 0, s);
  GemmDesc g = {};
  g.nseg = 1;
  g.seg_k[0] = static_cast<int>(K);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(x, M, K, ldx);
  r0.b[0] = mat(A_cat, r_tot, K, K);
  r0.mo = M;
  r0.no = r_tot;
  r0.out = T;
  r0.ld_out = ldt;
  r0.mode = kEpiStoreBf16;
  r0.alpha = sc;
  return launch_block_gemm(g, s);
}

int wsl_lora_linear_fwd(const void* x, long long ldx, const void* W, const void* T,
                        long long ldt, const void* B, void* y, long long ldy, long long M,
                        long long N, long long K, long long r, int dtype, void* stream) {
  if (bad_dtype(dtype) || !x || !W || !y || M <= 0 || N <= 0 || K <= 0 || r < 0)
    return WSL_ERR_BAD_ARG;
  if (r > 0 && (!T || !B)) return WSL_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == WSL_F32) {
    int st = launch_simt_gemm_f32(f32(x), ldx, 1, f32(W), K, 1, static_cast<float*>(y), ldy, M, N,
                                  K, 1.f, 0, s);
    if (st != WSL_OK || r == 0) return st;
    return launch_simt_gemm_f32(f32(T), ldt, 1, f32(B), r, 1, static_cast<float*>(y), ldy, M, N, r,
                                1.f, 1, s);
  }
  GemmDesc g = {};
  g.nseg = r > 0 ? 2 : 1;
  g.seg_k[0] = static_cast<int>(K);
  g.seg_k[1] = static_cast<int>(r);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(x, M, K, ldx);
  r0.b[0] = mat(W, N, K, K);
  if (r > 0) {
    r0.a[1] = mat(T, M, r, ldt);
    r0.b[1] = mat(B, N, r, r);
  }
  r0.mo = M;
  r0.no = N;
  r0.out = y;
  r0.ld_out = ldy;
  r0.mode = kEpiStoreBf16;
  r0.alpha = 1.f;
  return launch_block_gemm(g, s);
}

int wsl_lora_linear_fwd_group(int nproj, const void* x, long long ldx, const void* const* W,
                              const void* const* T, const long long* ldt, const void* const* B,
                              void* const* y, const long long* ldy, const long long* N,
                              const long long* r, long long M, long long K, void* stream) {
  if (nproj < 1 || nproj > WSL_MAX_PROJ || !x || !W || !y || !ldy || !N || !r || M <= 0 || K <= 0)
    return WSL_ERR_BAD_ARG;
  // one contraction layout for all regions: [x | T_p], so the ranks must agree
  const long long r0v = r[0];
  for (int p = 0; p < nproj; ++p) {
    if (!W[p] || !y[p] || N[p] <= 0 || r[p] != r0v || r[p] < 0) return WSL_ERR_BAD_ARG;
    if (r0v > 0 && (!T || !ldt || !B || !T[p] || !B[p])) return WSL_ERR_BAD_ARG;
  }
  GemmDesc g = {};
  g.nseg = r0v > 0 ? 2 : 1;
  g.seg_k[0] = static_cast<int>(K);
  g.seg_k[1] = static_cast<int>(r0v);
  g.nregion = nproj;
  for (int p = 0; p < nproj; ++p) {
    RegionDesc& rd = g.region[p];
    rd.a[0] = mat(x, M, K, ldx);
    rd.b[0] = mat(W[p], N[p], K, K);
    if (r0v > 0) {
      rd.a[1] = mat(T[p], M, r0v, ldt[p]);
      rd.b[1] = mat(B[p], N[p], r0v, r0v);
    }
    rd.mo = M;
    rd.no = N[p];
    rd.out = y[p];
    rd.ld_out = ldy[p];
    rd.mode = kEpiStoreBf16;
    rd.alpha = 1.f;
  }
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}

int wsl_lora_swiglu_supported(long long M, long long N, long long K, long long r) {
  return (M > 0 && N > 0 && K > 0 && r >= 0 && (N % 128) == 0 && (r % 8) == 0 && use_pair_tiles(M, 2 * N)) ? 1 : 0;
}

int wsl_lora_swiglu_fwd(const void* x, long long ldx, const void* W_gate, const void* W_up,
                        const void* T_cat, long long ldt, const void* B_gate, const void* B_up,
                        void* g_out, void* u_out, void* h_out, long long ld_out, long long M,
                        long long N, long long K, long long r, void* stream) {
  if (!x || !W_gate || !W_up || !g_out || !u_out || !h_out || M <= 0 || N <= 0 || K <= 0 || r < 0)
    return WSL_ERR_BAD_ARG;
  if (r > 0 && (!T_cat || !B_gate || !B_up)) return WSL_ERR_BAD_ARG;
  if (!wsl_lora_swiglu_supported(M, N, K, r)) return WSL_ERR_BAD_ARG;
  GemmDesc g = {};
  g.nseg = r > 0 ? 2 : 1;
  g.seg_k[0] = static_cast<int>(K);
  g.seg_k[1] = static_cast<int>(2 * r);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(x, M, K, ldx);
  r0.b[0] = mat(W_gate, N, K, K);
  r0.b2[0] = mat(W_up, N, K, K);
  r0.b2_k_shift[0] = 0;
  if (r > 0) {
    // [T_gate | T_up] . [B_gate 0 ; 0 B_up]^T: the gate rows see columns [0, r) of T_cat, the
    // up rows columns [r, 2r)
    r0.a[1] = mat(T_cat, M, 2 * r, ldt);
    r0.b[1] = mat(B_gate, N, r, r);
    r0.b2[1] = mat(B_up, N, r, r);
    r0.b2_k_shift[1] = static_cast<int>(r);
  }
  r0.mo = M;
  r0.no = N;
  r0.out = g_out;
  r0.out2 = u_out;
  r0.out3 = h_out;
  r0.ld_out = ld_out;
  r0.mode = kEpiSwiGLU;
  r0.alpha = 1.f;
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}

int wsl_lora_bwd_prepass(const void* dY, long long lddy, const void* B, void* U, long long ldu,
                         long long M, long long N, long long r, float sc, int dtype,
                         void* stream) {
  if (bad_dtype(dtype) || !dY || !B || !U || M <= 0 || N <= 0 || r <= 0) return WSL_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == WSL_F32)   // U[m,j] = s * sum_n dY[m,n] * B[n,j]
    return launch_simt_gemm_f32(f32(dY), lddy, 1, f32(B), 1, r, static_cast<float*>(U), ldu, M, r,
                                N, sc, 0, s);
  GemmDesc g = {};
  g.a_mn = false;
  g.b_mn = true;
  g.nseg = 1;
  g.seg_k[0] = static_cast<int>(N);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(dY, M, N, lddy);
  r0.b[0] = mat(B, N, r, r);
  r0.mo = M;
  r0.no = r;
  r0.out = U;
  r0.ld_out = ldu;
  r0.mode = kEpiStoreBf16;
  r0.alpha = sc;
  return launch_block_gemm(g, s);
}

int wsl_lora_linear_bwd_dx(int nproj, const void* const* dY, const long long* lddy,
                           const void* const* U, const long long* ldu, const void* const* W,
                           const void* const* A, const long long* N, const long long* r, void* dX,
                           long long lddx, long long M, long long K, int dtype, void* stream) {
  if (bad_dtype(dtype) || nproj < 1 || nproj > WSL_MAX_PROJ || !dY || !lddy || !W || !N || !r ||
      !dX || M <= 0 || K <= 0)
    return WSL_ERR_BAD_ARG;
  for (int p = 0; p < nproj; ++p) {
    if (!dY[p] || !W[p] || N[p] <= 0 || r[p] < 0) return WSL_ERR_BAD_ARG;
    if (r[p] > 0 && (!U || !ldu || !A || !U[p] || !A[p])) return WSL_ERR_BAD_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == WSL_F32) {
    int acc = 0;
    for (int p = 0; p < nproj; ++p) {
      // dX[m,k] += sum_n dY[m,n] * W[n,k]
      int st = launch_simt_gemm_f32(f32(dY[p]), lddy[p], 1, f32(W[p]), 1, K,
                                    static_cast<float*>(dX), lddx, M, K, N[p], 1.f, acc, s);
      if (st != WSL_OK) return st;
      acc = 1;
      if (r[p] > 0) {
        st = launch_simt_gemm_f32(f32(U[p]), ldu[p], 1, f32(A[p]), 1, K, static_cast<float*>(dX),
                                  lddx, M, K, r[p], 1.f, 1, s);
        if (st != WSL_OK) return st;
      }
    }
    return WSL_OK;
  }
  GemmDesc g = {};
  g.a_mn = false;
  g.b_mn = true;
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  int ns = 0;
  for (int p = 0; p < nproj; ++p) {
    g.seg_k[ns] = static_cast<int>(N[p]);
    r0.a[ns] = mat(dY[p], M, N[p], lddy[p]);
    r0.b[ns] = mat(W[p], N[p], K, K);
    ++ns;
    if (r[p] > 0) {
      g.seg_k[ns] = static_cast<int>(r[p]);
      r0.a[ns] = mat(U[p], M, r[p], ldu[p]);
      r0.b[ns] = mat(A[p], r[p], K, K);
      ++ns;
    }
  }
  g.nseg = ns;
  r0.mo = M;
  r0.no = K;
  r0.out = dX;
  r0.ld_out = lddx;
  r0.mode = kEpiStoreBf16;
  r0.alpha = 1.f;
  return launch_block_gemm(g, s);
}

int wsl_swiglu_bwd_in_dx_supported(long long M, long long N, long long K, long long r) {
  return (M > 0 && N > 0 && K > 0 && r >= 0 && (K % 64) == 0 && (N % 8) == 0 && (r % 8) == 0 &&
          use_pair_tiles(M, K)) ? 1 : 0;
}

int wsl_lora_linear_bwd_dx_swiglu(const void* dY, long long lddy, const void* U, long long ldu,
                                  const void* W, const void* A, const void* g, const void* u,
                                  void* dgate, void* dup, long long ld_gu, long long M, long long N,
                                  long long K, long long r, void* stream) {
  if (!dY || !W || !g || !u || !dgate || !dup || M <= 0 || N <= 0 || K <= 0 || r < 0) return WSL_ERR_BAD_ARG;
  if (r > 0 && (!U || !A)) return WSL_ERR_BAD_ARG;
  if (!wsl_swiglu_bwd_in_dx_supported(M, N, K, r)) return WSL_ERR_BAD_ARG;
  GemmDesc gd = {};
  gd.a_mn = false;
  gd.b_mn = true;
  gd.nregion = 1;
  RegionDesc& r0 = gd.region[0];
  int ns = 0;
  gd.seg_k[ns] = static_cast<int>(N);
  r0.a[ns] = mat(dY, M, N, lddy);
  r0.b[ns] = mat(W, N, K, K);
  ++ns;
  if (r > 0) {
    gd.seg_k[ns] = static_cast<int>(r);
    r0.a[ns] = mat(U, M, r, ldu);
    r0.b[ns] = mat(A, r, K, K);
    ++ns;
  }
  gd.nseg = ns;
  r0.mo = M;
  r0.no = K;
  r0.out = dgate;
  r0.out2 = dup;
  r0.ld_out = ld_gu;
  r0.mode = kEpiSwiGLUBwd;
  r0.alpha = 1.f;
  r0.addend = g;
  r0.addend2 = u;
  r0.ld_addend = ld_gu;
  return launch_block_gemm(gd, static_cast<cudaStream_t>(stream));
}

int wsl_lora_linear_bwd_dw(const void* dY, long long lddy, const void* U, long long ldu,
                           const void* x, long long ldx, const void* T, long long ldt, float* dW,
                           float* dA, float* dB, long long M, long long N, long long K,
                           long long r, void* workspace, unsigned long long workspace_bytes,
                           int dtype, void* stream) {
  if (bad_dtype(dtype) || M <= 0 || N <= 0 || K <= 0 || r < 0) return WSL_ERR_BAD_ARG;
  if (r == 0 && (dA || dB)) return WSL_ERR_BAD_ARG;
  if (!dW && !dA && !dB) return WSL_ERR_BAD_ARG;
  if ((dW || dB) && !dY) return WSL_ERR_BAD_ARG;
  if ((dW || dA) && !x) return WSL_ERR_BAD_ARG;
  if (dA && !U) return WSL_ERR_BAD_ARG;
  if (dB && !T) return WSL_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == WSL_F32) {
    int st = WSL_OK;
    if (dW)   // dW[n,k] += sum_m dY[m,n] * x[m,k]
      st = launch_simt_gemm_f32(f32(dY), 1, lddy, f32(x), 1, ldx, dW, K, N, K, M, 1.f, 1, s);
    if (st == WSL_OK && dB)
      st = launch_simt_gemm_f32(f32(dY), 1, lddy, f32(T), 1, ldt, dB, r, N, r, M, 1.f, 1, s);
    if (st == WSL_OK && dA)
      st = launch_simt_gemm_f32(f32(U), 1, ldu, f32(x), 1, ldx, dA, K, r, K, M, 1.f, 1, s);
    return st;
  }
  GemmDesc g = {};
  build_bwd_dw_desc(g, dY, lddy, U, ldu, x, ldx, T, ldt, dW, dA, dB, M, N, K, r);
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return WSL_ERR_ALIGN;
  g.workspace = static_cast<float*>(workspace);
  g.workspace_bytes = static_cast<size_t>(workspace_bytes);
  return launch_block_gemm(g, s);
}

int wsl_lora_linear_bwd_dw_group(int nproj, const void* const* dY, const long long* lddy,
                                 const void* const* U, const long long* ldu, const void* x,
                                 long long ldx, const void* const* T, const long long* ldt,
                                 float* const* dW, float* const* dA, float* const* dB,
                                 const long long* N, const long long* r, long long M, long long K,
                                 void* workspace, unsigned long long workspace_bytes, void* stream) {
  if (nproj < 1 || nproj > WSL_MAX_PROJ || !dY || !lddy || !x || !N || !r || !dW || !dA || !dB ||
      M <= 0 || K <= 0)
    return WSL_ERR_BAD_ARG;
  BwdDwProj pj[WSL_MAX_PROJ];
  for (int p = 0; p < nproj; ++p) {
    if (N[p] <= 0 || r[p] < 0 || !dY[p]) return WSL_ERR_BAD_ARG;
    if (r[p] == 0 && (dA[p] || dB[p])) return WSL_ERR_BAD_ARG;
    if (dA[p] && (!U || !ldu || !U[p])) return WSL_ERR_BAD_ARG;
    if (dB[p] && (!T || !ldt || !T[p])) return WSL_ERR_BAD_ARG;
    pj[p] = {dY[p], lddy[p], U ? U[p] : nullptr, ldu ? ldu[p] : 0, T ? T[p] : nullptr, ldt ? ldt[p] : 0,
             dW[p], dA[p], dB[p], N[p], r[p], nullptr};
  }
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return WSL_ERR_ALIGN;
  GemmDesc g = {};
  int st = build_bwd_dw_group(g, nproj, pj, x, ldx, M, K);
  if (st != WSL_OK) return st;
  g.workspace = static_cast<float*>(workspace);
  g.workspace_bytes = static_cast<size_t>(workspace_bytes);
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}

int wsl_bwd_dw_layer_group(int nproj, const void* const* dY, const long long* lddy, const void* x,
                           long long ldx, float* const* dW, void* const* dWl, const long long* N,
                           long long M, long long K, void* workspace,
                           unsigned long long workspace_bytes, void* stream) {
  if (nproj < 1 || nproj > WSL_MAX_PROJ || !dY || !lddy || !x || !N || !dW || !dWl || M <= 0 || K <= 0)
    return WSL_ERR_BAD_ARG;
  BwdDwProj pj[WSL_MAX_PROJ];
  for (int p = 0; p < nproj; ++p) {
    if (N[p] <= 0 || !dY[p] || !dW[p] || !dWl[p]) return WSL_ERR_BAD_ARG;
    pj[p] = {dY[p], lddy[p], nullptr, 0, nullptr, 0, dW[p], nullptr, nullptr, N[p], 0, dWl[p]};
  }
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return WSL_ERR_ALIGN;
  GemmDesc g = {};
  int st = build_bwd_dw_group(g, nproj, pj, x, ldx, M, K);
  if (st != WSL_OK) return st;
  g.workspace = static_cast<float*>(workspace);
  g.workspace_bytes = static_cast<size_t>(workspace_bytes);
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}

int wsl_lora_adapter_grads_from_dw(int nproj, const void* const* dWl, const void* const* A,
                                   const void* const* B, float* const* dA, float* const* dB,
                                   const long long* N, const long long* K, const long long* r, float s,
                                   void* workspace, unsigned long long workspace_bytes,
                                   void* stream) {
  if (nproj < 1 || nproj > WSL_MAX_ADAPTER_PROJ || !dWl || !A || !B || !dA || !dB || !N || !K || !r)
    return WSL_ERR_BAD_ARG;
  long long n_max = 0, k_max = 0;
  for (int p = 0; p < nproj; ++p) {
    if (!dWl[p] || !A[p] || !B[p] || !dA[p] || !dB[p] || N[p] <= 0 || K[p] <= 0 || r[p] <= 0)
      return WSL_ERR_BAD_ARG;
    n_max = N[p] > n_max ? N[p] : n_max;
    k_max = K[p] > k_max ? K[p] : k_max;
  }
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return WSL_ERR_ALIGN;
  // dB_p[N, r] += s * dWl_p[N, K] * A_p[r, K]^T: both operands K-major, one region per projection.
  // Projections of different sizes share the launch: the contraction runs to the longest and
  // the shorter operands read as zeros beyond their end.
  GemmDesc gb = {};
  gb.a_mn = false;
  gb.b_mn = false;
  gb.nseg = 1;
  gb.seg_k[0] = static_cast<int>(k_max);
  gb.ragged_k = true;
  gb.nregion = nproj;
  gb.workspace = static_cast<float*>(workspace);
  gb.workspace_bytes = static_cast<size_t>(workspace_bytes);
  for (int p = 0; p < nproj; ++p) {
    RegionDesc& rd = gb.region[p];
    rd.a[0] = mat(dWl[p], N[p], K[p], K[p]);
    rd.b[0] = mat(A[p], r[p], K[p], K[p]);
    rd.mo = N[p];
    rd.no = r[p];
    rd.out = dB[p];
    rd.ld_out = r[p];
    rd.mode = kEpiAccumF32;
    rd.alpha = s;
  }
  int st = launch_block_gemm(gb, static_cast<cudaStream_t>(stream));
  if (st != WSL_OK) return st;
  // dA_p[r, K] += s * B_p[N, r]^T * dWl_p[N, K], run as its transpose (dWl_p^T B_p, [K, r]) with
  // the contraction over N: both operands MN-major, results written transposed.
  GemmDesc ga = {};
  ga.a_mn = true;
  ga.b_mn = true;
  ga.nseg = 1;
  ga.seg_k[0] = static_cast<int>(n_max);
  ga.ragged_k = true;
  ga.nregion = nproj;
  ga.workspace = static_cast<float*>(workspace);
  ga.workspace_bytes = static_cast<size_t>(workspace_bytes);
  for (int p = 0; p < nproj; ++p) {
    RegionDesc& rd = ga.region[p];
    rd.a[0] = mat(dWl[p], N[p], K[p], K[p]);
    rd.b[0] = mat(B[p], N[p], r[p], r[p]);
    rd.mo = K[p];
    rd.no = r[p];
    rd.out = dA[p];
    rd.ld_out = K[p];
    rd.mode = kEpiAccumF32;
    rd.alpha = s;
    rd.transposed = true;
  }
  return launch_block_gemm(ga, static_cast<cudaStream_t>(stream));
}

unsigned long long wsl_adapter_grads_workspace_bytes(int nproj, const long long* N, const long long* K,
                                                     const long long* r) {
  if (nproj < 1 || nproj > WSL_MAX_ADAPTER_PROJ || !N || !K || !r) return 0;
  long long eb = 0, ea = 0;
  for (int p = 0; p < nproj; ++p) {
    eb += N[p] * r[p];
    ea += r[p] * K[p];
  }
  return splitk_workspace_bytes(eb > ea ? eb : ea);
}

int wsl_lora_merge_weight(int nproj, const void* const* W, const void* const* A, const void* const* B,
                          void* const* Weff, const long long* N, long long K, long long r, float s,
                          void* stream) {
  return launch_lora_merge(nproj, W, A, B, Weff, N, K, r, s, static_cast<cudaStream_t>(stream));
}

unsigned long long wsl_bwd_dw_group_workspace_bytes(int nproj, const long long* N, const long long* r,
                                                    long long M, long long K) {
  if (nproj < 1 || nproj > WSL_MAX_PROJ || !N || !r || M <= 0 || K <= 0) return 0;
  // same region order and tiling rule as the launch itself
  long long mo[kMaxRegion], no[kMaxRegion];
  int nr = 0;
  const bool pair = use_pair_tiles(N[0], K);
  for (int p = 0; p < nproj; ++p) { mo[nr] = N[p]; no[nr++] = K; }
  for (int p = 0; p < nproj; ++p)
    if (r[p] > 0) { mo[nr] = N[p]; no[nr++] = r[p]; }
  for (int p = 0; p < nproj; ++p)
    if (r[p] > 0) { mo[nr] = K; no[nr++] = r[p]; }
  const int sms = device_check() == WSL_OK ? device_sm_count() : 148;
  return plan_launch(nr, mo, no, kblocks(M), ~static_cast<size_t>(0), split_workers(pair, sms), pair, true).bytes;
}

unsigned long long wsl_bwd_dw_workspace_bytes(long long M, long long N, long long K, long long r,
                                              int want_dW, int want_dA, int want_dB) {
  if (M <= 0 || N <= 0 || K <= 0 || r < 0) return 0;
  long long mo[3], no[3];
  int nr = 0;
  const bool pair = want_dW ? use_pair_tiles(N, K)
                            : (want_dB && r > 0 ? use_pair_tiles(N, r) : use_pair_tiles(K, r));
  if (want_dW) { mo[nr] = N; no[nr++] = K; }
  if (want_dB && r > 0) { mo[nr] = N; no[nr++] = r; }
  if (want_dA && r > 0) { mo[nr] = K; no[nr++] = r; }
  if (nr == 0) return 0;
  const int sms = device_check() == WSL_OK ? device_sm_count() : 148;
  return plan_launch(nr, mo, no, kblocks(M), ~static_cast<size_t>(0), split_workers(pair, sms), pair, true).bytes;
}

int wsl_embed_gather(const long long* tokens, const void* E_small, void* G, long long M,
                     long long V, long long r_e, int dtype, void* stream) {
  if (bad_dtype(dtype)) return WSL_ERR_BAD_ARG;
  return launch_embed_gather(tokens, E_small, G, M, V, r_e, dtype == WSL_F32 ? 4 : 2,
                             static_cast<cudaStream_t>(stream));
}

int wsl_embed_fwd(const long long* tokens, const void* E_small, const void* P, void* h,
                  long long ldh, long long M, long long V, long long r_e, long long d,
                  void* stream) {
  if (!tokens || !E_small || !P || !h || M <= 0 || V <= 0 || r_e <= 0 || d <= 0)
    return WSL_ERR_BAD_ARG;
  GemmDesc g = {};
  g.nseg = 1;
  g.seg_k[0] = static_cast<int>(r_e);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(E_small, V, r_e, r_e);     // source matrix; rows are picked by token id
  r0.b[0] = mat(P, d, r_e, r_e);
  r0.mo = M;
  r0.no = d;
  r0.out = h;
  r0.ld_out = ldh;
  r0.mode = kEpiStoreBf16;
  r0.alpha = 1.f;
  g.gather_tokens = tokens;
  g.gather_count = M;
  g.gather_a = true;
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}

int wsl_embed_bwd_dproj(const long long* tokens, const void* dH, long long lddh,
                        const void* E_small, float* dP, long long M, long long V, long long r_e,
                        long long d, void* workspace, unsigned long long workspace_bytes,
                        void* stream) {
  if (!tokens || !dH || !E_small || !dP || M <= 0 || V <= 0 || r_e <= 0 || d <= 0)
    return WSL_ERR_BAD_ARG;
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return WSL_ERR_ALIGN;
  GemmDesc g = {};
  g.a_mn = true;
  g.b_mn = true;
  g.nseg = 1;
  g.seg_k[0] = static_cast<int>(M);
  g.nregion = 1;
  RegionDesc& r0 = g.region[0];
  r0.a[0] = mat(dH, M, d, lddh);
  r0.b[0] = mat(E_small, V, r_e, r_e);     // source matrix; contraction rows picked by token id
  r0.mo = d;
  r0.no = r_e;
  r0.out = dP;
  r0.ld_out = r_e;
  r0.mode = kEpiAccumF32;
  r0.alpha = 1.f;
  g.gather_tokens = tokens;
  g.gather_count = M;
  g.gather_b = true;
  g.workspace = static_cast<float*>(workspace);
  g.workspace_bytes = static_cast<size_t>(workspace_bytes);
  return launch_block_gemm(g, static_cast<cudaStream_t>(stream));
}

int wsl_embed_scatter_add(const long long* tokens, const void* dG, float* dE, long long M,
                          long long V, long long r_e, int dtype, void* stream) {
  if (bad_dtype(dtype)) return WSL_ERR_BAD_ARG;
  return launch_embed_scatter_add(tokens, dG, dE, M, V, r_e, dtype == WSL_F32 ? 1 : 0,
                                  static_cast<cudaStream_t>(stream));
}

int wsl_ce_fwd_bwd(void* logits, long long ld, const long long* labels, float* row_loss,
                   long long rows, long long V, float scale, const float* scale_dev, int dtype,
                   void* stream) {
  if (bad_dtype(dtype)) return WSL_ERR_BAD_ARG;
  return launch_ce(logits, ld, labels, row_loss, rows, V, scale, scale_dev, dtype == WSL_F32,
                   static_cast<cudaStream_t>(stream));
}

int wsl_swiglu_fwd(const void* gate, const void* up, void* out, long long n, int dtype, void* stream) {
  if (bad_dtype(dtype)) return WSL_ERR_BAD_ARG;
  return launch_swiglu(gate, up, out, nullptr, nullptr, nullptr, n, dtype == WSL_F32,
                       static_cast<cudaStream_t>(stream));
}

int wsl_swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup,
                   long long n, int dtype, void* stream) {
  if (bad_dtype(dtype) || !dout) return WSL_ERR_BAD_ARG;
  return launch_swiglu(gate, up, nullptr, dout, dgate, dup, n, dtype == WSL_F32,
                       static_cast<cudaStream_t>(stream));
}

int wsl_rmsnorm_fwd(const void* x, long long ldx, const float* w, void* y, long long ldy, float* rstd,
                    long long rows, long long D, float eps, const float* rope_cos,
                    const float* rope_sin, long long heads, long long seq, int dtype, void* stream) {
  if (bad_dtype(dtype)) return WSL_ERR_BAD_ARG;
  return launch_rmsnorm_fwd(x, ldx, nullptr, nullptr, w, y, ldy, rstd, rows, D, eps, rope_cos, rope_sin,
                            heads, seq, dtype == WSL_F32, static_cast<cudaStream_t>(stream));
}

int wsl_grad_sumsq_partials(const float* g, long long n, float* partials, void* stream) {
  return launch_grad_sumsq(g, n, partials, static_cast<cudaStream_t>(stream));
}

int wsl_adamw_flat_step(float* p, const float* g, float* m, float* v, void* p_copy, long long n,
                        float lr, float beta1, float beta2, float eps, float weight_decay,
                        float bias_corr1, float bias_corr2, const float* sumsq_partials,
                        int n_partials, float max_norm, void* stream) {
  const AdamwArgs a = {lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, max_norm};
  return launch_adamw_flat(p, g, m, v, p_copy, n, a, sumsq_partials, n_partials,
                           static_cast<cudaStream_t>(stream));
}

int wsl_add_rmsnorm_fwd(const void* x, const void* res, const float* w, void* h, void* y, float* rstd,
                        long long rows, long long D, float eps, int dtype, void* stream) {
  if (bad_dtype(dtype) || !res || !h) return WSL_ERR_BAD_ARG;
  return launch_rmsnorm_fwd(x, D, res, h, w, y, D, rstd, rows, D, eps, nullptr, nullptr, 0, 0,
                            dtype == WSL_F32, static_cast<cudaStream_t>(stream));
}

int wsl_add_rmsnorm_bwd(const void* dy, const void* h, const void* dres, const float* w,
                        const float* rstd, void* dx, float* dw, long long rows, long long D,
                        int dtype, void* stream) {
  if (bad_dtype(dtype) || !dres) return WSL_ERR_BAD_ARG;
  return launch_rmsnorm_bwd(dy, D, h, D, dres, w, rstd, dx, D, dw, rows, D, nullptr, nullptr, 0, 0,
                            dtype == WSL_F32, static_cast<cudaStream_t>(stream));
}

int wsl_rmsnorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* w,
                    const float* rstd, void* dx, long long lddx, float* dw, long long rows,
                    long long D, const float* rope_cos, const float* rope_sin, long long heads,
                    long long seq, int dtype, void* stream) {
  if (bad_dtype(dtype)) return WSL_ERR_BAD_ARG;
  return launch_rmsnorm_bwd(dy, lddy, x, ldx, nullptr, w, rstd, dx, lddx, dw, rows, D, rope_cos, rope_sin,
                            heads, seq, dtype == WSL_F32, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
