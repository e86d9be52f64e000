/*
 * wsl.h -- C ABI of the B200 (sm_100a) shared-W + LoRA linear hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*), enqueues its kernels on that stream and
 * returns an int status (WSL_OK or a negative WSL_ERR_*). Nothing here
 * allocates, frees or synchronises, and nothing throws; the caller owns all
 * memory. There is no CPU fallback: on a machine without an sm_100 device
 * every compute entry point returns WSL_ERR_DEVICE.
 *
 * The reference (muchanem/weightshared_torchtitan) has no FFI of its own; its
 * interface for this path is Python (nn.Module + autograd). Each declaration
 * below names the reference lines whose arithmetic it replaces. File paths are
 * relative to the reference project root.
 *
 * Conventions
 *   - matrices are row-major, last dimension contiguous; `ld*` arguments are row
 *     pitches in ELEMENTS (pass the number of columns for a packed matrix);
 *   - dtype WSL_BF16: activations/weights are bf16, accumulation is fp32 on the
 *     tcgen05 tensor cores, gradients of parameters (dW, dA, dB, dE, dP) are fp32;
 *   - dtype WSL_F32 : everything is fp32 and runs on the CUDA cores (the
 *     correctness mode of the reference's CPU-runnable configuration);
 *   - bf16 matrices must be 16-byte aligned with pitches that are multiples of
 *     8 elements (TMA requirement); violations return WSL_ERR_ALIGN;
 *   - s is the LoRA scale alpha/rank (the reference fixes alpha = 2*rank, so s = 2).
 */
#ifndef WSL_H_
#define WSL_H_

#ifdef __cplusplus
extern "C" {
#endif

#define WSL_OK 0
#define WSL_ERR_BAD_ARG (-1)   /* null pointer, non-positive or unsupported size */
#define WSL_ERR_ALIGN (-2)     /* pointer or pitch breaks the 16-byte rule */
#define WSL_ERR_DEVICE (-3)    /* no CUDA device, or the current device is not sm_100 */
#define WSL_ERR_CUDA (-4)      /* a CUDA runtime call or kernel launch failed */
#define WSL_ERR_TIMEOUT (-5)   /* a bounded device-side wait ran out (see wsl_poll_status) */
#define WSL_ERR_DRIVER (-6)    /* cuTensorMapEncodeTiled unavailable or refused the tensor */
#define WSL_ERR_TOO_LARGE (-7) /* size beyond a documented fixed limit */

#define WSL_BF16 0
#define WSL_F32 1

#define WSL_NOALLOC_SCRATCH_BYTES (64ull << 20) /* fixed scratch of wsl_lora_linear_bwd_dw_noalloc */

#define WSL_MAX_PROJ 3 /* projections that can share one input in wsl_lora_linear_bwd_dx */
#define WSL_MAX_ADAPTER_PROJ 9   /* projections per wsl_lora_adapter_grads_from_dw call */

/* Library version, (major << 16) | minor. */
int wsl_version(void);

/* Static, NUL-terminated description of a status code. */
const char* wsl_status_string(int status);

/* Number of kernel launches the library has enqueued since it was loaded. */
unsigned long long wsl_launch_count(void);

/*
 * Device-side status words of the CURRENT device: words[0] = 0 or the first
 * recorded WSL_ERR_TIMEOUT, words[1] = role that gave up (1 producer, 2 MMA
 * issuer, 3 epilogue of the GEMM; 4 a warp of the staged row kernels), words[2] = block index,
 * words[3] = tile index.
 * Copies from the device, so it waits for work already enqueued on the legacy
 * default stream's peers to the extent cudaMemcpyFromSymbol does; call it
 * after synchronising the stream of interest. Returns words[0].
 * Replaces: the reference reports errors by Python exceptions/asserts
 * (torchtitan/models/llama3/model/model.py:126).
 */
int wsl_poll_status(int words[4]);
int wsl_reset_status(void);

/*
 * Run-time options of the library (process-wide). Initial values come from the environment,
 * read once when the library is first used: WSL_PAIR (PAIR_TILES), WSL_ROW_STAGED
 * (ROW_STAGED), WSL_WAIT_LIMIT_MS (WAIT_LIMIT_MS), WSL_SPLIT_TAIL (SPLIT_TAIL), WSL_DEPENDENT_LAUNCH (DEPENDENT_LAUNCH). wsl_set_option returns WSL_OK or
 * WSL_ERR_BAD_ARG; wsl_get_option returns the value.
 *   WAIT_LIMIT_MS   bound of every device-side wait, 1..10000 ms (default 2000)
 *   STALL_PRODUCER  test aid: the copy-issuing warps never fill their rings, so the waits
 *                   of the other warps run into the bound and WSL_ERR_TIMEOUT is recorded
 *   PAIR_TILES      0 keeps the large GEMMs on single CTAs instead of CTA pairs
 *   ROW_STAGED      0 sends the RMSNorm calls to their direct (non-staged) kernels
 *   RESERVED_SMS    0..64 SMs the persistent kernels leave unoccupied, for a collective that
 *                   runs beside them on another stream (the gradient all-reduce overlapped
 *                   with the backward pass; the reference overlaps by DDP buckets,
 *                   torchtitan/models/llama3/infra/parallelize.py:428-444)
 *   GRID_WAVES      GEMM grids of up to this many times the CTAs that fit at once: 1 = persistent (one
 *                   CTA or pair per SM walks its share of the tiles), 2..8 = that many waves of
 *                   shorter-lived CTAs which the hardware deals to SMs as they free up (evens out
 *                   unequal tile times and SMs held by another kernel), 0 (default) = two waves for
 *                   launches with long tiles and at least four tiles per CTA, else one
 *   SPLIT_TAIL      0 keeps weight-gradient launches from cutting the tiles of their last, partial wave
 *                   of work into split-K units (see wsl_lora_linear_bwd_dw); default 1
 *   DEPENDENT_LAUNCH 0 launches every kernel with plain stream ordering; 1 (default) launches the GEMM, RMSNorm
 *                   and fold kernels with programmatic stream serialization: their CTAs take SMs and set
 *                   themselves up while the kernel before them in the stream drains, and wait for it
 *                   (griddepcontrol.wait) before they touch global memory
 *   MERGE_SIMT      1 runs wsl_lora_merge_weight on the CUDA cores instead of the tensor cores
 *   PROFILE_BITS    only honoured by builds compiled with -DWSL_PROFILE_SWITCHES
 * No counterpart in the reference (its knobs are Python config fields).
 */
#define WSL_OPT_WAIT_LIMIT_MS 1
#define WSL_OPT_STALL_PRODUCER 2
#define WSL_OPT_PAIR_TILES 3
#define WSL_OPT_ROW_STAGED 4
#define WSL_OPT_RESERVED_SMS 5
#define WSL_OPT_PROFILE_BITS 6
#define WSL_OPT_MERGE_SIMT 7
#define WSL_OPT_GRID_WAVES 8
#define WSL_OPT_SPLIT_TAIL 9
#define WSL_OPT_DEPENDENT_LAUNCH 10
int wsl_set_option(int option, long long value);
long long wsl_get_option(int option);

/*
 * y[M,N] = x[M,K] * W[N,K]^T           (plain projection, no adapter)
 * Replaces F.linear of the base projections: torchtitan/models/llama3/model/
 * model.py:392-394 and torchtitan/experiments/qwen3/model/model.py:184,218,251.
 * out_f32 != 0 writes fp32 instead of bf16 (bf16 mode only).
 */
int wsl_linear_fwd(const void* x, long long ldx, const void* W, void* y, long long ldy,
                   long long M, long long N, long long K, int out_f32, int dtype, void* stream);

/*
 * T[M,r_tot] = s * x[M,K] * A_cat[r_tot,K]^T
 * The rank-r pre-pass of the adapter. A_cat may stack the A matrices of all
 * projections that read the same x (q|k|v, gate|up), so x is read once.
 * The scale s is folded in here; wsl_lora_linear_fwd and wsl_lora_linear_bwd_dw
 * expect this scaled T.
 * Replaces self.w_a(x) and the "* (alpha/rank)" of LoRAModule.forward:
 * torchtitan/models/llama3/model/model.py:189-192.
 */
int wsl_lora_prepass(const void* x, long long ldx, const void* A_cat, void* T, long long ldt,
                     long long M, long long K, long long r_tot, float s, int dtype, void* stream);

/*
 * y[M,N] = x[M,K] * W[N,K]^T + T[M,r] * B[N,r]^T
 * One GEMM whose contraction runs over the concatenation [x | T] . [W | B]^T,
 * accumulated in fp32, rounded once. T is the scaled pre-pass output (column
 * slice of T_cat with pitch ldt).
 * Replaces base(x) + LoRAModule.forward(x) joined by broadcast_add with equal
 * widths: torchtitan/models/llama3/model/model.py:111-145,189-192,392-398.
 */
int wsl_lora_linear_fwd(const void* x, long long ldx, const void* W, const void* T,
                        long long ldt, const void* B, void* y, long long ldy, long long M,
                        long long N, long long K, long long r, int dtype, void* stream);

/*
 * wsl_lora_linear_fwd for nproj <= WSL_MAX_PROJ projections that read the same x and have the
 * same rank (q|k|v, gate|up) in ONE launch (bf16): y_p = x W_p^T + T_p B_p^T.
 * Replaces the same lines as wsl_lora_linear_fwd at the call sites that share an input:
 * torchtitan/experiments/qwen3/model/model.py:184,251.
 */
int wsl_lora_linear_fwd_group(int nproj, const void* x, long long ldx, const void* const* W,
                              const void* const* T, const long long* ldt, const void* const* B,
                              void* const* y, const long long* ldy, const long long* N,
                              const long long* r, long long M, long long K, void* stream);

/*
 * The gate and up projections of a SwiGLU MLP and the activation in ONE launch (bf16):
 *   g[M,N] = x W_gate^T + T_cat[:, 0:r] B_gate^T
 *   u[M,N] = x W_up^T   + T_cat[:, r:2r] B_up^T
 *   h[M,N] = silu(g) * u        (from g and u as stored, i.e. rounded to bf16)
 * Every accumulator tile holds 128 columns of g next to the same 128 columns of u (the two
 * CTAs of a pair load the gate and the up weights), so the epilogue writes h without g and u
 * being read back; g and u are still stored because the backward needs them. T_cat is the
 * scaled pre-pass output of wsl_lora_prepass with A_cat = [A_gate; A_up].
 * wsl_lora_swiglu_supported() tells whether a shape can take this path (N % 128 == 0, r % 8
 * == 0, large enough for CTA-pair tiles); otherwise use wsl_lora_linear_fwd_group and
 * wsl_swiglu_fwd, which give bit-identical results.
 * Replaces F.silu(self.w1(x)) * self.w3(x) with LoRA on both projections:
 * torchtitan/experiments/qwen3/model/model.py:251, torchtitan/models/llama3/model/model.py:189-192.
 */
int wsl_lora_swiglu_supported(long long M, long long N, long long K, long long r);
int wsl_lora_swiglu_fwd(const void* x, long long ldx, const void* W_gate, const void* W_up,
                        const void* T_cat, long long ldt, const void* B_gate, const void* B_up,
                        void* g, void* u, void* h, long long ld_out, long long M, long long N,
                        long long K, long long r, void* stream);

/*
 * U[M,r] = s * dY[M,N] * B[N,r]
 * Backward pre-pass (the autograd MmBackward of w_b together with the
 * MulBackward of the scale): torchtitan/models/llama3/model/model.py:191.
 */
int wsl_lora_bwd_prepass(const void* dY, long long lddy, const void* B, void* U, long long ldu,
                         long long M, long long N, long long r, float s, int dtype, void* stream);

/*
 * dX[M,K] = sum_{p < nproj} ( dY_p[M,N_p] * W_p[N_p,K] + U_p[M,r_p] * A_p[r_p,K] )
 * Input gradient of up to WSL_MAX_PROJ projections that read the same x (q,k,v or
 * gate,up), summed inside one fp32 accumulator and rounded once.
 * Replaces the two MmBackward nodes per projection and the AddBackward at the
 * shared input: autograd of torchtitan/models/llama3/model/model.py:191,392-398.
 */
int wsl_lora_linear_bwd_dx(int nproj, const void* const* dY, const long long* lddy,
                           const void* const* U, const long long* ldu, const void* const* W,
                           const void* const* A, const long long* N, const long long* r, void* dX,
                           long long lddx, long long M, long long K, int dtype, void* stream);

/*
 * Input gradient of the DOWN projection of a SwiGLU MLP with the activation's backward in its
 * epilogue (bf16): dh[M,K] = dY[M,N] W[N,K] + U[M,r] A[r,K] stays on the SM; with the stored
 * g and u of wsl_lora_swiglu_fwd (pitch ld_gu) the launch writes
 *   dgate[M,K] = dh u silu'(g),   dup[M,K] = dh silu(g)      (dh rounded to bf16 first)
 * i.e. what wsl_lora_linear_bwd_dx followed by wsl_swiglu_bwd gives, bit for bit, without dh
 * being written and read back. K is the MLP's inner width here. r = 0 (U, A NULL) takes a W
 * that already contains the adapter (wsl_lora_merge_weight). The g and u tiles reach the
 * epilogue by TMA one 32-column chunk ahead of the arithmetic.
 * wsl_swiglu_bwd_in_dx_supported() tells whether a shape can take this path (K % 64 == 0 and
 * large enough for CTA-pair tiles).
 * Replaces the autograd backward of w2(F.silu(w1(x)) * w3(x)) between w2's MmBackward and the
 * SiluBackward / MulBackward pair: torchtitan/experiments/qwen3/model/model.py:251.
 */
int wsl_swiglu_bwd_in_dx_supported(long long M, long long N, long long K, long long r);
int wsl_lora_linear_bwd_dx_swiglu(const void* dY, long long lddy, const void* U, long long ldu,
                                  const void* W, const void* A, const void* g, const void* u,
                                  void* dgate, void* dup, long long ld_gu, long long M, long long N,
                                  long long K, long long r, void* stream);

/*
 * dW[N,K] += dY^T x ;  dA[r,K] += U^T x ;  dB[N,r] += dY^T T      (all fp32, in place)
 * U and T carry the scale s already. dW is the gradient buffer of the SHARED
 * base weight: every layer that reuses W adds into the same fp32 buffer. Any of
 * dW, dA, dB may be NULL to skip that product.
 * workspace: optional fp32 scratch of workspace_bytes (16-byte aligned; NULL/0 allowed).
 * When the [N,K] tile grid is too small to fill the GPU (short weight matrices, long
 * token count) the token contraction is split across CTAs, partial sums go to the
 * workspace and a second kernel adds them into dW/dA/dB in a fixed order, so results stay
 * bit-reproducible. When the grid is large but its last wave of tiles is only partly
 * full (every tile contracts over all M tokens, so an idle wave is long), just the tiles
 * of that wave are split that way. wsl_bwd_dw_workspace_bytes() gives the size that allows
 * the best split; a smaller or absent workspace only costs speed. The workspace contents are
 * garbage afterwards; calls that overlap on the GPU need separate workspaces.
 * Replaces the MmBackward weight gradients and AccumulateGrad of
 * torchtitan/models/llama3/model/model.py:191,392-394 (one dW per use, cast and
 * added into W.grad by autograd in the reference).
 */
int wsl_lora_linear_bwd_dw(const void* dY, long long lddy, const void* U, long long ldu,
                           const void* x, long long ldx, const void* T, long long ldt, float* dW,
                           float* dA, float* dB, long long M, long long N, long long K,
                           long long r, void* workspace, unsigned long long workspace_bytes,
                           int dtype, void* stream);

/*
 * wsl_lora_linear_bwd_dw for nproj <= WSL_MAX_PROJ projections that read the same x (q|k|v,
 * gate|up) in ONE launch: dW_p += dY_p^T x, dA_p += U_p^T x, dB_p += dY_p^T T_p. All
 * projections must want all three products when r_p > 0 (dA_p/dB_p NULL only with r_p = 0);
 * dW_p is required. More tiles per launch fill the GPU better than one launch per
 * projection. Workspace as above; wsl_bwd_dw_group_workspace_bytes gives its size.
 * Replaces the same autograd nodes as wsl_lora_linear_bwd_dw, for the q/k/v and gate/up
 * call sites that share an input (torchtitan/experiments/qwen3/model/model.py:184,251).
 */
int wsl_lora_linear_bwd_dw_group(int nproj, const void* const* dY, const long long* lddy,
                                 const void* const* U, const long long* ldu, const void* x,
                                 long long ldx, const void* const* T, const long long* ldt,
                                 float* const* dW, float* const* dA, float* const* dB,
                                 const long long* N, const long long* r, long long M, long long K,
                                 void* workspace, unsigned long long workspace_bytes, void* stream);
unsigned long long wsl_bwd_dw_group_workspace_bytes(int nproj, const long long* N, const long long* r,
                                                    long long M, long long K);

/*
 * Backward through the layer's own weight gradient (bf16 mode), for callers that need dW
 * anyway (the shared base weight is trained). With G_l = dY^T x of THIS layer,
 *     dB = s * G_l * A^T      and      dA = s * B^T * G_l
 * are the same rank-r products as dY^T T and U^T x, but read the [N,K] matrix G_l instead of
 * streaming the M-row activations again, and dX = dY * (W + s B A) needs no pre-pass over dY.
 * Three entry points:
 *
 * wsl_lora_merge_weight:  Weff_p[N_p,K] = bf16( W_p[N_p,K] + s * B_p[N_p,r] * A_p[r,K] ) for
 *   nproj projections with the same K and rank (r = 8, 16, 32, 64 or 128) in one launch: one
 *   streaming pass over W, r FMAs per element; dense row-major matrices. Give Weff_p to
 *   wsl_lora_linear_bwd_dx as W_p with U_p = A_p = NULL.
 * wsl_bwd_dw_layer_group: dW_p[N_p,K] += dY_p^T x (fp32, in place, shared across layers) and
 *   dWl_p[N_p,K] = bf16(dY_p^T x) (this launch's addend alone, dense) for nproj projections
 *   that read the same x, one launch. Workspace: wsl_bwd_dw_group_workspace_bytes with r = 0.
 * wsl_lora_adapter_grads_from_dw: dA_p[r_p,K_p] += s * B_p^T dWl_p, dB_p[N_p,r_p] += s * dWl_p
 *   A_p^T (fp32, in place; A_p, B_p, dWl_p dense bf16) for up to WSL_MAX_ADAPTER_PROJ
 *   projections of any sizes (all seven of a decoder layer) in two launches. The optional
 *   workspace (wsl_adapter_grads_workspace_bytes) lets the short contractions be split over
 *   the GPU, folded in a fixed order.
 *
 * The bf16 rounding of G_l and of Weff is of the same order as the bf16 rounding of U and T
 * in the direct formulation. Replaces the same autograd nodes as wsl_lora_linear_bwd_dx/_dw:
 * torchtitan/models/llama3/model/model.py:191,392-398.
 */
int wsl_lora_merge_weight(int nproj, const void* const* W, const void* const* A, const void* const* B,
                          void* const* Weff, const long long* N, long long K, long long r, float s,
                          void* stream);
int wsl_bwd_dw_layer_group(int nproj, const void* const* dY, const long long* lddy, const void* x,
                           long long ldx, float* const* dW, void* const* dWl, const long long* N,
                           long long M, long long K, void* workspace,
                           unsigned long long workspace_bytes, void* stream);
int wsl_lora_adapter_grads_from_dw(int nproj, const void* const* dWl, const void* const* A,
                                   const void* const* B, float* const* dA, float* const* dB,
                                   const long long* N, const long long* K, const long long* r, float s,
                                   void* workspace, unsigned long long workspace_bytes,
                                   void* stream);
unsigned long long wsl_adapter_grads_workspace_bytes(int nproj, const long long* N, const long long* K,
                                                     const long long* r);

/* Workspace size (bytes, possibly 0) wsl_lora_linear_bwd_dw wants for these sizes; the
 * want_* flags say which of dW, dA, dB will be non-NULL. No reference counterpart. */
unsigned long long wsl_bwd_dw_workspace_bytes(long long M, long long N, long long K, long long r,
                                              int want_dW, int want_dA, int want_dB);

/*
 * wsl_lora_linear_bwd_dw for callers that cannot allocate (bf16 mode only).
 * No counterpart in the reference: it exists for hosts that may not call cudaMalloc (or
 * any allocator) around this call -- a pipeline whose memory was all handed out at
 * start-up, a callback, a foreign-language binding that only owns the tensors it was
 * given -- and therefore cannot supply the split-K workspace of the entry point above.
 * The partial sums live in a WSL_NOALLOC_SCRATCH_BYTES (64 MiB) array that is part of the
 * library image; every GPU that loads the library holds it until the process exits. The
 * call itself allocates and frees nothing.
 *   - Limit: 2 * 4 bytes * (elements of the requested dW, dA, dB) must not exceed the
 *     array, i.e. about 8.3 M output elements; larger requests return WSL_ERR_TOO_LARGE
 *     (weight matrices that big fill the GPU without a split: use the entry point above
 *     with a NULL workspace).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any
 *     stream capture begins.
 *   - All calls share the one array and it keeps the previous call's partial sums. Every
 *     element a call reads back it has written first, so nothing needs clearing between
 *     calls, but two calls that overlap on the GPU (different streams, or graphs replayed
 *     concurrently) race on it; serialise them.
 * Same arithmetic and result as wsl_lora_linear_bwd_dw.
 */
int wsl_lora_linear_bwd_dw_noalloc(const void* dY, long long lddy, const void* U, long long ldu,
                                   const void* x, long long ldx, const void* T, long long ldt,
                                   float* dW, float* dA, float* dB, long long M, long long N,
                                   long long K, long long r, void* stream);

/*
 * G[M,r_e] = E_small[tokens[m], :]          (bit-exact row gather)
 * tokens are int64 in [0, V). Replaces aten::embedding behind
 * nn.Embedding: torchtitan/experiments/qwen3/model/model.py:350,441.
 */
int wsl_embed_gather(const long long* tokens, const void* E_small, void* G, long long M,
                     long long V, long long r_e, int dtype, void* stream);

/*
 * h[M,d] = E_small[tokens, :] * P[d,r_e]^T        (bf16)
 * The factorized embedding in one kernel: the TMA producer of the tcgen05 GEMM fetches the
 * rows E_small[tokens[m]] with tile::gather4 straight into the swizzled operand tile, so the
 * gathered matrix is never written to memory. A token id outside [0, V) contributes a zero
 * row. Every 256-column tile of h gathers the rows again and a gather4 instruction moves 4 x 128
 * bytes, so for wide outputs (d above ~1024) wsl_embed_gather followed by wsl_linear_fwd is
 * faster (measured 107 against 288 us at 16384 tokens, r_e = 1024, d = 4096); the results are
 * the same bits.
 * Replaces nn.Embedding (torchtitan/experiments/qwen3/model/model.py:350,441); the
 * factorization itself (E_small, P) is not in the reference.
 */
int wsl_embed_fwd(const long long* tokens, const void* E_small, const void* P, void* h,
                  long long ldh, long long M, long long V, long long r_e, long long d,
                  void* stream);

/*
 * dP[d,r_e] += dH[M,d]^T * E_small[tokens, :]     (fp32 in place; operands bf16)
 * The projection gradient of the factorized embedding, again gathering E_small's rows in
 * the TMA producer. workspace: optional split-K scratch as in wsl_lora_linear_bwd_dw
 * (4 * 16 * d * r_e bytes always suffices).
 */
int wsl_embed_bwd_dproj(const long long* tokens, const void* dH, long long lddh,
                        const void* E_small, float* dP, long long M, long long V, long long r_e,
                        long long d, void* workspace, unsigned long long workspace_bytes,
                        void* stream);

/*
 * dE[tokens[m], :] += dG[m, :]              (fp32 scatter-add, atomics)
 * dG is bf16 (WSL_BF16) or fp32 (WSL_F32); dE is fp32 [V, r_e].
 * Replaces embedding_dense_backward behind nn.Embedding (same lines).
 */
int wsl_embed_scatter_add(const long long* tokens, const void* dG, float* dE, long long M,
                          long long V, long long r_e, int dtype, void* stream);

/* ---- rows either side of the projections (HBM-bound streaming kernels) ---- */

/*
 * Mean-token cross-entropy, forward and gradient in one pass over the logits, IN PLACE:
 *   row_loss[i] = logsumexp(logits[i,:]) - logits[i, labels[i]]
 *   logits[i,j] <- scale * (softmax(logits[i,:])[j] - [j == labels[i]])
 * logits is [rows, V] (pitch ld) in the storage type; a label outside [0, V) marks an
 * ignored row (zero loss, zero gradient), as ignore_index = -100 does in the reference. The
 * caller sums row_loss; the gradient scale is scale * (*scale_dev), where scale_dev is an
 * optional device scalar (NULL = 1): pass 1 / (number of counted rows) in one of the two --
 * the device scalar lets a caller derive the count from the labels without a host round trip.
 * Replaces F.cross_entropy(pred.flatten(0,1).float(), labels.flatten(0,1)) with
 * reduction='mean' and its backward: torchtitan/components/loss.py:18-22.
 */
int wsl_ce_fwd_bwd(void* logits, long long ld, const long long* labels, float* row_loss,
                   long long rows, long long V, float scale, const float* scale_dev, int dtype,
                   void* stream);

/*
 * out = silu(gate) * up over n contiguous elements (n % 8 == 0 for bf16, % 4 for fp32), and
 * its backward (dgate, dup from dout, gate, up).
 * Replaces F.silu(self.w1(x)) * self.w3(x): torchtitan/experiments/qwen3/model/model.py:251.
 */
int wsl_swiglu_fwd(const void* gate, const void* up, void* out, long long n, int dtype, void* stream);
int wsl_swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup,
                   long long n, int dtype, void* stream);

/*
 * y[r,:] = x[r,:] * rstd[r] * w, rstd = 1/sqrt(mean(x[r,:]^2) + eps); rstd [rows] fp32 is
 * written for the backward (may be NULL). With rope_cos / rope_sin ([seq, D] fp32, both or
 * neither) the normalised row is rotated: y = n*cos + rotate_half(n)*sin at position
 * (r / heads) % seq -- the q/k head norm followed by the rotary embedding in one pass.
 * Supported widths: D/vec a power of two <= 32, or D = {1, 2, 4, 8} * 32 * vec (vec = 8 for
 * bf16, 4 for fp32: up to 2048 / 1024), or, in bf16 with dense rows (pitch = D), D = 2560
 * and 4096 ({10, 16} * 32 * vec, the hidden sizes of the 4B and 8B shapes); other widths return
 * WSL_ERR_TOO_LARGE. Rotary needs D <= 32*vec. w and dw are fp32 [D]; dw is accumulated
 * (+=, atomics) and may be NULL.
 * Replaces nn.RMSNorm and apply_rotary_emb:
 * torchtitan/experiments/qwen3/model/model.py:40-90,136-143,195-203,288-289,312-313.
 */
int wsl_rmsnorm_fwd(const void* x, long long ldx, const float* w, void* y, long long ldy, float* rstd,
                    long long rows, long long D, float eps, const float* rope_cos,
                    const float* rope_sin, long long heads, long long seq, int dtype, void* stream);
int wsl_rmsnorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* w,
                    const float* rstd, void* dx, long long lddx, float* dw, long long rows,
                    long long D, const float* rope_cos, const float* rope_sin, long long heads,
                    long long seq, int dtype, void* stream);

/*
 * The residual add that precedes a hidden-size RMSNorm, and its mirror image in the backward,
 * folded into the norm kernels (dense rows, no rotary):
 *   forward : h = x + res (rounded to the storage type and written out), y = RMSNorm(h) * w
 *   backward: dx = dRMSNorm(dy; h, w, rstd) + dres, dw += ...   (dres = the gradient that
 *             reaches h through the residual stream; dx is the gradient of both x and res)
 * One pass over memory less each way than an add kernel followed by the norm kernel.
 * Replaces `h = h + self.attention(...)`, `out = h + self.feed_forward(self.ffn_norm(h))` and
 * the norm that reads the sum: torchtitan/experiments/qwen3/model/model.py:310-313.
 * Widths as wsl_rmsnorm_fwd; rows dense with pitch D.
 */
int wsl_add_rmsnorm_fwd(const void* x, const void* res, const float* w, void* h, void* y, float* rstd,
                        long long rows, long long D, float eps, int dtype, void* stream);
int wsl_add_rmsnorm_bwd(const void* dy, const void* h, const void* dres, const float* w,
                        const float* rstd, void* dx, float* dw, long long rows, long long D,
                        int dtype, void* stream);

/*
 * The optimizer step over flat fp32 arenas (parameters p, gradients g, AdamW moments m and v,
 * n elements each, the same layout): global-norm clipping, AdamW with decoupled weight decay
 * and the refresh of the bf16 compute copy of the parameters, in one pass over the gradients
 * (wsl_grad_sumsq_partials: WSL_SUMSQ_PARTIALS partial sums of g^2, fixed order) and one pass
 * over everything (wsl_adamw_flat_step: folds the partials into the norm, then per element
 *   g' = g * min(1, max_norm / (norm + 1e-6));  m = b1 m + (1-b1) g';  v = b2 v + (1-b2) g'^2;
 *   p = p (1 - lr wd) - (lr / bias_corr1) m / (sqrt(v) / sqrt(bias_corr2) + eps),
 * bias_corr = 1 - beta^t from the host; p_copy, if not NULL, receives p as bf16).
 * max_norm <= 0 skips the clip (partials may then be NULL). n a multiple of 4, 16-byte
 * aligned buffers. g itself is left as it is (not scaled in place).
 * Replaces torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW.step + the per-use weight casts
 * of autocast: torchtitan/distributed/utils.py:316-394, torchtitan/components/optimizer.py:243-326,
 * torchtitan/train.py:479-497.
 */
#define WSL_SUMSQ_PARTIALS 1184
int wsl_grad_sumsq_partials(const float* g, long long n, float* partials, void* stream);
int wsl_adamw_flat_step(float* p, const float* g, float* m, float* v, void* p_copy, long long n,
                        float lr, float beta1, float beta2, float eps, float weight_decay,
                        float bias_corr1, float bias_corr2, const float* sumsq_partials,
                        int n_partials, float max_norm, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WSL_H_ */
