/* C ABI of libb200scan: recurrent-scan kernels for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only.  Every tensor argument is a DEVICE pointer to a dense,
 * contiguous buffer in the layout stated per function; complex64 is interleaved (re, im)
 * float pairs.  `stream` is a cudaStream_t passed as void*.  All work is enqueued on that
 * stream; no entry point except the two *_status readers synchronises, and none allocates or
 * frees device memory (so calls are legal during CUDA-graph capture).  The library keeps no
 * mutable state between calls apart from per-device caches filled on first use (SM count,
 * kernel attributes, the address of the static scratch array): make the first call of each
 * entry point on a device from one thread; after that, concurrent calls from several host
 * threads are fine as long as each uses its own workspace.  b200_diag_fwd_static is the one
 * exception: all its calls share one array (see there).
 *
 * Return value: B200_OK, or a B200_ERR_* code for an argument the host side can reject.  A
 * kernel that gives up on a bounded wait records B200_ERR_TIMEOUT in its workspace header and
 * finishes with a zero carry; b200_workspace_status() reads that word back (it synchronises
 * the stream), so a caller that wants the check makes it between steps.
 *
 * Paths in the "replaces" notes are relative to the tsfast project root (v0.5.0).
 */
#ifndef B200SCAN_H_
#define B200SCAN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_ERR_ARG 1         /* null pointer, non-positive size, unknown dtype */
#define B200_ERR_WORKSPACE 2   /* workspace missing, misaligned or too small */
#define B200_ERR_LAUNCH 3      /* the CUDA runtime refused a memset or a launch */
#define B200_ERR_UNSUPPORTED 4 /* size outside what the kernel handles */
#define B200_ERR_TIMEOUT 5     /* device side: a look-back wait ran out of polls */

#define B200_F32 0 /* float32 */
#define B200_C64 1 /* complex64, interleaved */

/* Library version (major*100 + minor). */
int b200_version(void);

/* Read the error word of a workspace after the work enqueued on `stream` has finished.
 * Synchronises `stream`.  Returns B200_OK or the B200_ERR_* code a kernel recorded. */
int b200_workspace_status(const void* workspace, void* stream);

/* ---- S1: diagonal scan with time-invariant coefficients -------------------------------
 * x_t = lam * x_{t-1} + v_t.   lam [M,N], v/out [M,L,N], x0 [M,N] or NULL (zero start).
 * Replaces diag_fwd / diag_bwd of tsfast/models/_core/scan_backends/diagonal_c.py:413-442
 * (CPU) and _diag_fwd_kernel / _diag_bwd_kernel of scan_backends/diagonal_triton.py:82-228,
 * i.e. the bodies of the ops tsfast::scan_diagonal(_bwd) in tsfast/models/_core/scan.py:100-134.
 * Backward: g [M,L,N] upstream gradient, out = forward result; writes glam [M,N] (per lane,
 * summed over time), gv [M,L,N] and, when x0 != NULL, gx0 [M,N] (gx0 may be NULL otherwise). */
size_t b200_diag_workspace_bytes(int dtype, int backward, int64_t M, int64_t L, int64_t N);
int b200_diag_fwd(int dtype, int64_t M, int64_t L, int64_t N, const void* lam, const void* v,
                  const void* x0, void* out, void* workspace, size_t workspace_bytes, void* stream);
int b200_diag_bwd(int dtype, int64_t M, int64_t L, int64_t N, const void* g, const void* lam,
                  const void* out, const void* x0, void* glam, void* gv, void* gx0,
                  void* workspace, size_t workspace_bytes, void* stream);

/* S1 forward for callers that may not allocate device memory at all.  (No counterpart in the
 * reference; added for this library's users.)  Think of a controller or observer running an
 * identified LRU/S5 model inside a fixed-rate loop, or a process that was handed a fixed device
 * arena by its host application: a cudaMalloc there either is forbidden or costs an unbounded
 * stall, and even torch's caching allocator may fall through to one.  Same arguments and result
 * as b200_diag_fwd, minus the workspace: the cross-tile state of the look-back kernel lives in a
 * 4 MiB array inside the library image (held by every GPU that loads the library until exit).
 * Limits and rules:
 *  - problems whose look-back state exceeds 4 MiB are refused with B200_ERR_UNSUPPORTED
 *    (b200_diag_workspace_bytes(dtype, 0, M, L, N) > 4194304; a tile is about 100 steps of 64 to
 *    128 lanes and roughly 2700 tiles fit, e.g. 16 x 1000 x 64 complex uses 176 of them);
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress)
 *    with that device current; make that first call before any stream capture;
 *  - every call reuses the one array (it zeroes the words that must start at zero itself), so two
 *    calls that can overlap on the GPU - different streams, or different host threads - race;
 *    keep calls of this entry point on one stream or order them with events;
 *  - it calls no cudaMalloc/cudaFree and no allocating library routine. */
int b200_diag_fwd_static(int dtype, int64_t M, int64_t L, int64_t N, const void* lam, const void* v,
                         const void* x0, void* out, void* stream);
/* Device-side status of the b200_diag_fwd_static calls enqueued on `stream` so far (the error
 * word at the head of the shared array): B200_OK or B200_ERR_TIMEOUT.  Synchronises `stream`,
 * allocates nothing.  (No counterpart in the reference.) */
int b200_diag_static_status(void* stream);

/* Test and tuning probe for S1/S2: the same launch path as b200_diag_* / b200_sel_* with the
 * choices the regular entry points make themselves handed in.  mode 0 = kernel chosen by shape,
 * 1 = look-back tiles, 2 = streaming chains; vcap caps the streaming kernel's vector width
 * (0 = none); spin_limit is the number of polls a look-back wait makes before it gives up
 * (0 = the default, about a second); mute_tile >= 0 names one look-back tile that publishes
 * nothing, so that its successors' waits run out, the launch records B200_ERR_TIMEOUT and still
 * returns (-1 = none).  varying selects S2, backward the adjoint; lam/val/xsrc/x0/out/glam/gx0
 * as in the regular entry points (val = v forward, g backward; xsrc = forward output, backward
 * only).  The workspace is the one b200_diag/sel_workspace_bytes sizes.  (No counterpart in the
 * reference.) */
int b200_diag_probe(int mode, int vcap, int spin_limit, int64_t mute_tile, int dtype, int varying, int backward,
                    int64_t M, int64_t L, int64_t N, const void* lam, const void* val, const void* xsrc,
                    const void* x0, void* out, void* glam, void* gx0, void* workspace, size_t workspace_bytes,
                    void* stream);

/* ---- S2: diagonal scan with time-varying coefficients ---------------------------------
 * x_t = lam_t * x_{t-1} + v_t.   lam, v, out [B,L,N]; x0 [B,N] or NULL.
 * Replaces sel_fwd / sel_bwd of tsfast/models/_core/scan_backends/selective_c.py:52-120 (CPU)
 * and _sel_fwd / _sel_bwd of scan_backends/selective_triton.py:48-109, i.e. the bodies of
 * tsfast::scan_selective(_bwd) in tsfast/models/_core/scan.py:157-195; complex64 follows the
 * doubling-scan semantics there.  Backward writes glam [B,L,N], gv [B,L,N], gx0 [B,N]. */
size_t b200_sel_workspace_bytes(int dtype, int backward, int64_t B, int64_t L, int64_t N);
int b200_sel_fwd(int dtype, int64_t B, int64_t L, int64_t N, const void* lam, const void* v,
                 const void* x0, void* out, void* workspace, size_t workspace_bytes, void* stream);
int b200_sel_bwd(int dtype, int64_t B, int64_t L, int64_t N, const void* g, const void* lam,
                 const void* out, const void* x0, void* glam, void* gv, void* gx0,
                 void* workspace, size_t workspace_bytes, void* stream);

/* ---- S4: all-pole IIR scan (dynoNet denominator) -----------------------------------------
 * y_t = w_t - sum_{i=1..na} a_i y_{t-i}, float32, 1 <= na <= 16.  a, y0 [lanes,na]; w, y
 * [lanes,L] with time contiguous per lane; y0[j] = y_{-1-j} (newest first) or NULL for a zero
 * start.  Replaces the generated allpole_fwd / allpole_bwd kernels and the host-side head
 * corrections of tsfast/models/architectures/dynonet/allpole_triton.py:59-123,174-213, i.e. the
 * bodies of tsfast::dynonet_allpole(_bwd).  Backward: g upstream gradient, y forward output;
 * writes grad_a [lanes,na] (finished, with sign and initial-state terms), gw [lanes,L] and, when
 * y0 != NULL, grad_y0 [lanes,na].  No workspace is needed. */
int b200_allpole_fwd(int64_t lanes, int64_t L, int64_t na, const void* a, const void* w, const void* y0,
                     void* y, void* stream);
int b200_allpole_bwd(int64_t lanes, int64_t L, int64_t na, const void* g, const void* a, const void* y,
                     const void* y0, void* ga, void* gw, void* gy0, void* stream);

/* ---- dynoNet G-block forward: FIR numerator + all-pole denominator + sum over inputs, fused --
 * For every batch row b and output channel i:  y[b,i,t] = sum_j allpole(a[i,j], w_ij)[t] with
 * w_ij[t] = sum_{k<nb} taps[i,j,k] * ub[b,j, t + nb-1 - k], where row ub[b,j,:] holds the carried
 * input tail (nb-1 samples) followed by u[b,:,j] (pitch floats per row, zero filled past
 * L+nb-1).  Replaces the body of LinearDynamicalOperator.forward for the "scan" backend,
 * tsfast/models/architectures/dynonet/core.py:199-250 (cat + flipped grouped conv1d :214-220,
 * the all-pole dispatch :228-231, the new state :240-246 and the pair sum :250), without the
 * [B, I*O, L] numerator output ever reaching memory.  float32, 1 <= na <= 4, nb in {4, 8, 16}
 * (pad taps and tail with zeros up to the next size); pairs are indexed j*O + i as in the
 * reference.  taps [O,I,nb], a [O,I,na], x0 [B,I*O,na] or NULL (newest first), y [B,O,L] (the
 * reference returns this tensor transposed to [B,L,O] as a view), y_pairs [B,I*O,L] or NULL (the
 * per-pair outputs the adjoint needs), x_last [B,I*O,na].  With y == NULL (y_pairs required) the
 * kernel runs one warp per filter instead of one per (batch row, output channel) and writes only the
 * per-pair outputs, for blocks with too few outputs to fill the GPU; the caller sums them over the
 * inputs.  No workspace. */
int b200_gblock_fwd(int64_t B, int64_t L, int64_t I, int64_t O, int64_t na, int64_t nb, int64_t pitch,
                    const void* ub, const void* taps, const void* a, const void* x0, void* y, void* y_pairs,
                    void* x_last, void* stream);

/* Builds the input rows the two G-block entry points read, ub [B*I, pitch], from u [B,L,I] (channel
 * last, dense) and the carried tail [B,nb-1,I] or NULL: row (b,j) = nb_padded-nb zeros, the tail,
 * u[b,:,j], zeros up to the pitch.  Replaces the torch.cat + transpose that feed conv1d in
 * dynonet/core.py:212-220. */
int b200_gblock_pack_rows(int64_t B, int64_t L, int64_t I, int64_t nb_padded, int64_t nb, int64_t pitch,
                          const void* u, const void* tail, void* ub, void* stream);

/* Adjoint of b200_gblock_fwd for an upstream gradient gy [B,O,L] on y (same layouts, nb padded the
 * same way): the all-pole adjoint of every pair (reading gy and the [O,I,na] coefficients in
 * place through a row map, so the [B,I*O,L] broadcast of gy is never built) followed by the
 * numerator adjoint.  Replaces what autograd runs for dynonet/core.py:214-250: the backward of
 * sum/view, tsfast::dynonet_allpole_bwd (allpole_triton.py:174-213) and the grouped conv1d
 * gradients.  Writes gub [B*I,pitch] (gradient w.r.t. the rows of ub: carried tail, then input),
 * gtaps [B,O,I,nb] and ga [B,I*O,na] (per batch row; the caller sums over B), gx0 [B,I*O,na] when
 * x0 != NULL.  With gub_per_filter != 0 the numerator adjoint runs one warp per filter (for blocks
 * with too few inputs to fill the GPU) and gub is [B*I*O,pitch], one row per pair j*O+i, which the
 * caller sums over i.  The workspace holds the numerator-output gradient [B,I*O,L]. */
size_t b200_gblock_bwd_workspace_bytes(int64_t B, int64_t L, int64_t I, int64_t O);
int b200_gblock_bwd(int64_t B, int64_t L, int64_t I, int64_t O, int64_t na, int64_t nb, int64_t pitch,
                    const void* gy, const void* ub, const void* taps, const void* a, const void* y_pairs,
                    const void* x0, void* gub, int64_t gub_per_filter, void* gtaps, void* ga, void* gx0,
                    void* workspace, size_t workspace_bytes, void* stream);

/* ---- S3: fused Mamba selective-scan section ---------------------------------------------
 * delta = softplus(draw) (threshold 20); h_t = exp(delta_t A) h_{t-1} + delta_t u_t B_t;
 * out_t = (h_t . C_t + Dp u_t) * z_t * sigmoid(z_t); hlast = h_L.  All float32.
 * draw, u, z, out [B,L,D]; A [D,N]; Bt, Ct [B,L,N]; Dp [D]; h0, hlast [B,D,N] (h0 may be NULL);
 * 1 <= N <= 128.  Replaces mamba_fwd / mamba_bwd of tsfast/models/architectures/mamba/
 * backend_c.py:106-245 (CPU C ABI) and _mamba_fwd / _mamba_bwd of mamba/mamba_triton.py:85-286,
 * i.e. the bodies of tsfast::mamba_scan, mamba_scan_train and mamba_scan_bwd.
 * chk: state checkpoints [B, ceil(L / b200_mamba_chk_interval()), D, N] written by the forward
 * for the backward (slot k = state after step (k+1)*interval - 1); pass NULL for inference.
 * Backward: gout [B,L,D] upstream gradient, ghlast [B,D,N] or NULL (zero); writes gdraw, gu, gz
 * [B,L,D], gA [D,N], gBt, gCt [B,L,N], gDp [D] and, when h0 != NULL, gh0 [B,D,N].  Sums over
 * channels and batch go through partial buffers in the workspace, added in a fixed order. */
int b200_mamba_chk_interval(void);
int b200_mamba_fwd(int64_t B, int64_t L, int64_t D, int64_t N, const void* draw, const void* A, const void* Bt,
                   const void* Ct, const void* u, const void* z, const void* Dp, const void* h0, void* out,
                   void* hlast, void* chk, void* stream);
size_t b200_mamba_bwd_workspace_bytes(int64_t B, int64_t L, int64_t D, int64_t N);
int b200_mamba_bwd(int64_t B, int64_t L, int64_t D, int64_t N, const void* draw, const void* A, const void* Bt,
                   const void* Ct, const void* u, const void* z, const void* Dp, const void* h0, const void* chk,
                   const void* gout, const void* ghlast, void* gdraw, void* gA, void* gBt, void* gCt, void* gu,
                   void* gz, void* gDp, void* gh0, void* workspace, size_t workspace_bytes, void* stream);

/* ---- Mamba causal depthwise convolution + SiLU (the step that feeds S3) --------------------
 * out[b,t,d] = silu(bias[d] + sum_{k<K} w[d,k] X(b, t-(K-1)+k, d)), X = cat(tail, x) along time.
 * float32, 2 <= K <= 8.  x [B,L,D] with unit channel stride and the given element strides along
 * batch and time (a chunk view of a wider projection is read in place); tail [B,D,K-1]; w [D,K];
 * bias [D] or NULL; out [B,L,D] dense.  Replaces _conv_fwd / _conv_bwd and the eager tail-gradient
 * code of tsfast/models/architectures/mamba/conv_triton.py:81-191,198-281 (ops
 * tsfast::mamba_conv_silu(_bwd)); semantics of _causal_depthwise_silu, mamba/core.py:38-58.
 * Backward: gy [B,L,D] dense; writes gx [B,L,D] dense, gtail [B,D,K-1], gw [D,K] and, when
 * bias != NULL, gb [D]; weight/bias gradients go through per-(batch, segment) partials in the
 * workspace, added in a fixed order. */
int b200_conv_silu_fwd(int64_t B, int64_t L, int64_t D, int64_t K, const void* x, int64_t x_stride_b,
                       int64_t x_stride_l, const void* tail, const void* w, const void* bias, void* out,
                       void* stream);
size_t b200_conv_silu_bwd_workspace_bytes(int64_t B, int64_t L, int64_t D, int64_t K);
int b200_conv_silu_bwd(int64_t B, int64_t L, int64_t D, int64_t K, const void* gy, const void* x,
                       int64_t x_stride_b, int64_t x_stride_l, const void* tail, const void* w,
                       const void* bias, void* gx, void* gtail, void* gw, void* gb, void* workspace,
                       size_t workspace_bytes, void* stream);

/* ---- Boundary projections of the LRU / S5 layers on the tensor cores ------------------------
 * C[M,N] = A1[M,K1] * B1[N,K1]^T  (+ A2[M,K2] * B2[N,K2]^T when K2 > 0)  (+ bias[N] on every row when
 * bias != NULL), float32 in and out.
 * Replaces the two real GEMMs behind complex_in_proj / real_out_proj of
 * tsfast/models/_core/scan.py:272-313 (called from architectures/lru.py:99,107 and s5.py:185,195) and
 * the feed-through product added to the readout (lru.py:107): with the interleaved weight layouts
 * those functions build, in-projection is (A1 = u, B1 = [2n, d]) and readout + feed-through is
 * (A1 = view_as_real(x) [M, 2n], B1 = [out, 2n]; A2 = u, B2 = D).  With a bias it is also the
 * x_proj / dt_proj pair that produces draw, B_t, C_t for the Mamba section
 * (architectures/mamba/core.py:150-152).  The same entry point computes the input gradients
 * (A1 = upstream gradient, B1 = the transposed weight).
 * Arithmetic: tcgen05.mma.kind::tf32 with every operand split into a TF32 head and a TF32 tail
 * (three MMAs per product, float32 accumulation in tensor memory): float32-faithful, a few 1e-6
 * relative.  A1/A2 row-major with row pitches lda1/lda2 (floats, multiples of 4, 16-byte aligned
 * base), B1/B2 row-major [N, K] with pitches ldb1/ldb2, C row-major with pitch ldc (multiple of 4,
 * 16-byte aligned).  M, N, K1, K2 are free (partial tiles read zeros).  The workspace holds the split
 * weights and the status header (b200_workspace_status). */
size_t b200_proj_gemm_workspace_bytes(int64_t N, int64_t K1, int64_t K2);
int b200_proj_gemm(int64_t M, int64_t N, int64_t K1, const void* A1, int64_t lda1, const void* B1, int64_t ldb1,
                   int64_t K2, const void* A2, int64_t lda2, const void* B2, int64_t ldb2, const void* bias, void* C,
                   int64_t ldc, void* workspace, size_t workspace_bytes, void* stream);

/* Weight gradient of such a product: dW[N,K] = G[M,N]^T * A[M,K], the reduction running over the M
 * tokens.  Replaces what autograd runs for the weight of each of the GEMMs above (a float32 SIMT GEMM
 * with a 256 000-long reduction in the full-model configuration).  Same arithmetic; both operands are
 * read token-major in place (no transposed copy).  G and A row-major with pitches ldg / lda (multiples
 * of 4, 16-byte aligned bases), dW row-major with pitch lddw.  The token axis is cut into slices that
 * are accumulated in tensor memory and added in a fixed order, so results are reproducible; the
 * workspace holds the slices' partial tiles. */
size_t b200_proj_wgrad_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200_proj_wgrad(int64_t M, int64_t N, int64_t K, const void* G, int64_t ldg, const void* A, int64_t lda, void* dW,
                    int64_t lddw, void* workspace, size_t workspace_bytes, void* stream);

/* ---- Pointwise glue of the LRU / S5 blocks (float32) -------------------------------------------
 * LayerNorm over the last axis of x [M,D] (D <= 512): y = (x - mean) * rstd * gamma + beta with the
 * biased variance and eps inside the square root, mean / rstd [M] saved for the adjoint; gamma and
 * beta [D] may be NULL (1 and 0).  Replaces nn.LayerNorm in the pre-norm blocks,
 * tsfast/models/architectures/lru.py:141,146 and s5.py:226,234 (PyTorch's kernel spends 0.38 ms on
 * the [256000,128] rows of the full-model configuration, this one the time of one pass over HBM).
 * Backward: g upstream gradient; writes dx [M,D] and, when not NULL, dgamma / dbeta [D]; the
 * per-CTA partial rows in the workspace are added in a fixed order. */
int b200_layernorm_fwd(int64_t M, int64_t D, const void* x, const void* gamma, const void* beta, float eps, void* y,
                       void* mean, void* rstd, void* stream);
size_t b200_layernorm_bwd_workspace_bytes(int64_t M, int64_t D);
int b200_layernorm_bwd(int64_t M, int64_t D, const void* g, const void* x, const void* gamma, const void* mean,
                       const void* rstd, void* dx, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
                       void* stream);

/* Gated residual out = u + a * sigmoid(b), all [M,D] with row pitches ldu/lda/ldb/ldo in floats (a and
 * b may be the two halves of one [M,2D] tensor).  Replaces F.glu followed by the residual addition of
 * the LRU block (lru.py:148-149) and the "half GLU" h * sigmoid(out2(h)) + u of the S5 block
 * (s5.py:240-255) in one pass.  Backward: ga = g * sigmoid(b), gb = g * a * sigmoid(b) (1 - sigmoid(b));
 * the gradient of u is g itself. */
int b200_gated_residual_fwd(int64_t M, int64_t D, const void* u, int64_t ldu, const void* a, int64_t lda, const void* b,
                            int64_t ldb, void* out, int64_t ldo, void* stream);
int b200_gated_residual_bwd(int64_t M, int64_t D, const void* g, int64_t ldg, const void* a, int64_t lda, const void* b,
                            int64_t ldb, void* ga, int64_t ldga, void* gb, int64_t ldgb, void* stream);

/* Column sums out[c] = sum_m x[m,c] of a float32 matrix [M,D] (row pitch ldx floats, D <= 1024 when
 * rows are 16-byte aligned, else D <= 256), added in a fixed order: the bias gradient of the linear
 * layers around the scans (the `glu` / encoder / decoder nn.Linear of lru.py:142,197,201 and `out1` /
 * `out2` / encoder / decoder of s5.py:229-230,302,318, whose autograd emits a column reduction of the
 * output gradient).  M = 0 writes zeros. */
size_t b200_colsum_workspace_bytes(int64_t M, int64_t D);
int b200_colsum(int64_t M, int64_t D, const void* x, int64_t ldx, void* out, void* workspace, size_t workspace_bytes,
                void* stream);

/* Parameter prologues of the LRU and S5 layers: from the stored parameters to what the projection GEMM
 * and the scan consume, one launch forward and one for the adjoint (PyTorch runs a dozen tiny kernels
 * forward and twice that backward, per layer and step).
 *   LRU (LRU.eigenvalues and the gamma scaling in LRU.forward, lru.py:79-83,97-99):
 *     lam[j] = exp(-exp(nu_log[j])) * exp(i exp(theta_log[j]))                      complex64 [n]
 *     W[2j] = exp(gamma_log[j]) B_re[j],  W[2j+1] = exp(gamma_log[j]) B_im[j]       float32 [2n, d]
 *   S5 (S5.discretize, s5.py:154-170; mode 0 "zoh", 1 "bilinear"; clip_eigs clamps Lambda_re to <= -1e-4;
 *   step = step_rescale * exp(log_step)):
 *     lam_bar[j] complex64 [p],  W[2j] + i W[2j+1] = B_bar[j] = c_j (B_re[j] + i B_im[j])   float32 [2p, d]
 * W is the input-projection weight with interleaved (re, im) rows: u W^T has the memory layout of the
 * complex [.., n] tensor complex_in_proj returns (_core/scan.py:272-292).  The adjoint takes the
 * gradients of lam / lam_bar (complex64, PyTorch's convention) and of W (either may be null = zero)
 * and writes the gradient of every parameter. */
int b200_lru_prologue_fwd(int64_t n, int64_t d, const void* nu_log, const void* theta_log, const void* gamma_log,
                          const void* B_re, const void* B_im, void* lam, void* W, void* stream);
int b200_lru_prologue_bwd(int64_t n, int64_t d, const void* nu_log, const void* theta_log, const void* gamma_log,
                          const void* B_re, const void* B_im, const void* glam, const void* gW, void* g_nu, void* g_theta,
                          void* g_gamma, void* gB_re, void* gB_im, void* stream);
int b200_s5_discretize_fwd(int64_t p, int64_t d, int mode, int clip_eigs, float step_rescale, const void* Lambda_re,
                           const void* Lambda_im, const void* log_step, const void* B_re, const void* B_im, void* lam_bar,
                           void* W, void* stream);
int b200_s5_discretize_bwd(int64_t p, int64_t d, int mode, int clip_eigs, float step_rescale, const void* Lambda_re,
                           const void* Lambda_im, const void* log_step, const void* B_re, const void* B_im,
                           const void* glam_bar, const void* gW, void* gLambda_re, void* gLambda_im, void* g_log_step,
                           void* gB_re, void* gB_im, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200SCAN_H_ */
