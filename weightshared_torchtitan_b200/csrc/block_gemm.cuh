// Host-side description of one launch of the tcgen05 block GEMM
// (see block_gemm.cu). Internal to the library: the C-ABI in include/wsl.h is
// the public surface.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace wsl {

constexpr int kMaxMaps = 32;    // tensor maps carried in the kernel parameters
constexpr int kMaxSeg = 6;      // contraction segments (K-concatenation)
constexpr int kMaxRegion = 10;  // output regions sharing one launch (3 projections x dW, dB, dA, + a split tail)

enum EpilogueMode : int {
  kEpiStoreBf16 = 0,   // out(bf16)  = alpha * acc
  kEpiStoreF32 = 1,    // out(fp32)  = alpha * acc
  kEpiAccumF32 = 2,    // out(fp32) += alpha * acc   (tiles own their outputs: plain RMW)
  // Gate and up projection of a SwiGLU MLP in one accumulator tile (see RegionDesc::b2):
  // out(bf16) = g, out2 = u, out3 = silu(g) * u with g, u rounded to bf16 first.
  kEpiSwiGLU = 3,
  // Backward of that activation in the epilogue of the GEMM that produces dh (the input
  // gradient of the down projection): with g = addend and u = addend2 (bf16 [mo, no]),
  //   out(bf16) = d gate = dh u silu'(g),  out2(bf16) = d up = dh silu(g),  dh = bf16(alpha * acc).
  kEpiSwiGLUBwd = 4,
};

// A row-major bf16 matrix in device memory: `rows` x `cols`, row pitch `ld` elements.
struct Mat {
  const void* ptr;
  long long rows;
  long long cols;
  long long ld;
};

// One output region: out[mo, no] (op)= alpha * sum_seg A_seg * B_seg^T.
// With K-major operands A_seg is stored [mo, k_seg] and B_seg [no, k_seg];
// with MN-major operands A_seg is stored [k_seg, mo] and B_seg [k_seg, no].
struct RegionDesc {
  Mat a[kMaxSeg];
  Mat b[kMaxSeg];
  long long mo;
  long long no;
  void* out;
  long long ld_out;
  int mode;
  float alpha;
  // fp32 modes only: write the tile transposed, i.e. the result matrix is [no, mo] with
  // pitch ld_out and tile element (i, j) goes to out[j * ld_out + i]. Lets a product whose
  // natural output is short and wide (dA = U^T x, [r, K]) run as its tall-and-narrow
  // transpose (x^T U, [K, r]) with a narrow, cheap MMA N.
  bool transposed;
  // Optional second output of an fp32, non-transposed region: copy[mo, no] (bf16, pitch
  // ld_copy) = alpha * product of THIS launch, whatever `mode` does to `out`. Gives a caller
  // that accumulates in place (dW += dY^T x) the addend itself, rounded to bf16, as the
  // operand of a follow-up GEMM. nullptr = none.
  void* copy;
  long long ld_copy;
  // kEpiSwiGLU only (K-major operands, CTA-pair launch): the 256-column accumulator tile holds
  // 128 columns of  g = sum_seg A_seg b[seg]^T  and the SAME 128 output columns of
  // u = sum_seg A_seg b2[seg]^T  side by side, so the epilogue has both halves of every
  // silu(g) * u in front of it. `no` counts the output columns of ONE of them (a multiple of
  // 128); out / out2 / out3 are the three [mo, no] bf16 results (pitch ld_out each).
  // b2_k_shift[seg]: contraction offset of b2 inside the segment, in elements; b[seg] covers
  // segment columns [0, b.cols) and b2[seg] covers [shift, shift + b2.cols), the rest of each
  // reads as zeros. That expresses the block-diagonal adapter factor  [T_g | T_u] . [B_g 0; 0 B_u]^T
  // without materialising the zero blocks.
  Mat b2[kMaxSeg];
  int b2_k_shift[kMaxSeg];
  void* out2;
  void* out3;
  // kEpiStoreBf16 only: out = alpha * acc + addend, with addend a bf16 matrix of the output's
  // shape (pitch ld_addend). The epilogue brings the addend tile into its staging buffers by
  // TMA one chunk ahead, adds in place and stores, so the addend is read once, in full lines.
  // Either every region of a launch has an addend or none (W_eff = W + s B A is the user).
  const void* addend;
  long long ld_addend;
  const void* addend2;   // kEpiSwiGLUBwd: the second input matrix (u), pitch ld_addend
};

struct GemmDesc {
  bool a_mn;   // A operands are MN-major (contraction index is the slow one in memory)
  bool b_mn;
  int nseg;
  int seg_k[kMaxSeg];   // contraction length of each segment (same for all regions)
  int nregion;
  RegionDesc region[kMaxRegion];
  // Optional scratch for split-K (fp32, 16-byte aligned). When the tile grid is too small
  // to fill the GPU the contraction is split, partials land here and a second kernel folds
  // them into the outputs in a fixed order. nullptr disables splitting.
  float* workspace;
  size_t workspace_bytes;
  // Row gather for region 0 / segment 0 (factorized embedding). With gather_a the A operand
  // (K-major) is described by its SOURCE matrix [V, k] and tile row i reads source row
  // tokens[i]; with gather_b the B operand (MN-major) is the source [V, no] and contraction
  // row k reads source row tokens[k]. gather_count = number of token ids.
  const long long* gather_tokens;
  long long gather_count;
  bool gather_a;
  bool gather_b;
  // Operands may have fewer rows/columns along the contraction than seg_k says; what is
  // missing counts as zeros (the TMA out-of-bounds fill). Lets regions with different
  // contraction lengths share one launch (seg_k = the longest).
  bool ragged_k;
};

// Workspace that lets launch_block_gemm split any contraction of these output sizes up to
// its maximum factor (16): 16 * 4 * sum(mo * no) bytes.
inline size_t splitk_workspace_bytes(long long out_elems) { return static_cast<size_t>(out_elems) * 64u; }

// Enqueues the GEMM on `stream`. Returns a WSL_* status code (include/wsl.h).
int launch_block_gemm(const GemmDesc& g, cudaStream_t stream);

// Number of kernel launches this library has enqueued since load (all kernels).
extern unsigned long long g_launch_count;

}  // namespace wsl
