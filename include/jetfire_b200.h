/*
 * jetfire_b200 — C ABI of the B200 (sm_100a) implementation of the Jetfire INT8 data-flow hot path.
 *
 * One entry point per kernel of the reference's operator layer.  The reference has no C ABI: its boundary
 * is a set of Python callables (Jetfire/Nonlinear/*.py, Jetfire/Linear/*.py) and a pybind module
 * (JetfireGEMMKernel/BlockQuantize/cpp_extension/bindings.cpp:6-35).  Each declaration below cites the
 * reference callable it stands behind.
 *
 * Conventions
 *   - all pointers are DEVICE pointers unless stated otherwise; payloads are int8 [M,N] row-major, scales are
 *     IEEE fp16 [M/32, N/32] row-major holding (block absmax)/127; the quantisation block is 32x32;
 *   - M and N (and K) must be positive multiples of 32; payload pointers must be 16-byte aligned;
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default stream),
 *     allocates nothing, never synchronises, and returns 0 on success or a negative jf_status;
 *   - stochastic rounding uses a counter-based Philox4x32-10 keyed by (seed, offset): one call with counter (e/8, offset)
 *     serves the 8 elements e = row*N+col .. +7; element e takes the 16-bit half (e & 1) of word (e >> 1) & 3 and
 *     noise = h * 2^-16 - 0.5.  Passing a non-NULL `noise` (fp32 [M,N], values in [-0.5,0.5)) overrides the generator
 *     (used to reproduce the reference bit for bit in tests).
 */
#ifndef JETFIRE_B200_H
#define JETFIRE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    JF_OK = 0,
    JF_ERR_NULL = -1,        /* a required pointer is NULL */
    JF_ERR_SHAPE = -2,       /* a dimension is not a positive multiple of 32 (or exceeds a documented limit) */
    JF_ERR_ALIGN = -3,       /* a pointer or leading dimension breaks the 16-byte alignment rule */
    JF_ERR_DTYPE = -4,       /* unknown dtype code */
    JF_ERR_LAUNCH = -5,      /* the CUDA runtime reported a launch error (see jf_last_cuda_error) */
    JF_ERR_UNSUPPORTED = -6, /* the device is not sm_100 or a needed driver entry point is missing */
    JF_ERR_ARG = -7          /* any other invalid argument */
} jf_status;

typedef enum { JF_F32 = 0, JF_F16 = 1, JF_BF16 = 2 } jf_dtype;

/* Text for a status code, and the last CUDA error code seen by this library on the calling thread. */
const char* jf_status_string(int status);
int jf_last_cuda_error(void);
/* ABI version of this header (bumped on any signature change). */
int jf_abi_version(void);

/* ------------------------------------------------------------------------------------------------------------
 * Nonlinear operators (reference: Triton kernels in Jetfire/Nonlinear)
 * ---------------------------------------------------------------------------------------------------------- */

/* int8_quantize(x, QB, stochastic)            Jetfire/Nonlinear/quantize.py:128-164 (kernel :33-117)
 * int8_quantize_transpose(x, QB, stochastic)  Jetfire/Nonlinear/quantize_transpose.py:131-171 (kernel :33-129)
 * x: [M,N] of x_dtype.  q: int8 [M,N], s: fp16 [M/32,N/32].  qt (optional, may be NULL): int8 [N,M] = q^T. */
int jf_int8_quantize(const void* x, int x_dtype, int64_t M, int64_t N, int8_t* q, void* s, int8_t* qt,
                     int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* stream);

/* The same round-to-nearest quantisation for up to 8 tensors of one dtype in one launch: x[j] is [M[j], N[j]], q[j] / s[j] its payload
 * and scales.  For the weight matrices a caller quantises at the start of every forward pass (INT8_GPT2/qmodel.py:92, 139, 199-200:
 * four int8_quantize calls per transformer block); results are identical to `count` calls of jf_int8_quantize.  `x`, `M`, `N`, `q`, `s`
 * are host arrays of length `count` (1..8); they are copied into the kernel parameters. */
int jf_int8_quantize_multi(int count, const void* const* x, int x_dtype, const int64_t* M, const int64_t* N, int8_t* const* q,
                           void* const* s, void* stream);

/* int8_dequantize(x, s_x, QB)                 Jetfire/Nonlinear/dequantize.py:86-116 (kernel :28-84)
 * y: fp32 [M,N] = fp32(fp16(q) * s)  (the product is rounded to fp16 first, as the reference does). */
int jf_int8_dequantize(const int8_t* q, const void* s, int64_t M, int64_t N, float* y, void* stream);

/* int8_transpose(x)                           Jetfire/Nonlinear/transpose.py:69-97 (kernel :29-67)
 * y: int8 [N,M]. */
int jf_int8_transpose(const int8_t* x, int64_t M, int64_t N, int8_t* y, void* stream);

/* int8_gelu_forward(x, s_x, QB)               Jetfire/Nonlinear/gelu_fwd.py:128-162 (kernel :34-126)
 * Both GELU entry points use a per-device table in device memory (32 MB each, static storage of the library)
 * that the first call on a device fills with one extra kernel on that call's stream; later calls on other streams wait for the
 * fill through an event.  That first call must not be made on a stream that is being captured (JF_ERR_UNSUPPORTED). */
int jf_int8_gelu_forward(const int8_t* qx, const void* sx, int64_t M, int64_t N, int8_t* qy, void* sy, void* stream);

/* int8_gelu_backward(x, s_x, g, s_g, QB, stochastic)   Jetfire/Nonlinear/gelu_bwd.py:173-215 (kernel :28-171) */
int jf_int8_gelu_backward(const int8_t* qx, const void* sx, const int8_t* qg, const void* sg, int64_t M, int64_t N,
                          int8_t* qd, void* sd, int stochastic, const float* noise, uint64_t seed, uint64_t offset,
                          void* stream);

/* int8_layernorm_forward(x, sx, weight, mean, rstd, QB, eps)   Jetfire/Nonlinear/layernorm.py:430-465 (kernel :74-190)
 * gamma fp32 [N]; mean, rstd fp32 [M] are INPUTS (the reference takes the statistics from the caller, has no bias
 * and ignores eps). */
int jf_int8_layernorm_forward(const int8_t* qx, const void* sx, const float* gamma, const float* mean, const float* rstd,
                              int64_t M, int64_t N, int8_t* qy, void* sy, void* stream);

/* int8_layernorm_backward(x, sx, g, sg, w, QB, m, v, stochastic, eps)   Jetfire/Nonlinear/layernorm.py:467-526
 * (kernels :197-402 and :404-428).  qd/sd: quantised dx; dgamma: fp32 [N].
 * slab: width of the column slab over which the two row reductions of dx are taken; the reference uses 128
 * (its tile width) although it divides by N; pass 128 for reference behaviour.  The reference needs N to be a multiple
 * of the slab; here the last slab may be shorter (N only has to be a multiple of 32, e.g. 1600).
 * scratch: fp32 [(M/32) * N] workspace for the per-32-row partial sums of dgamma (contents on return unspecified). */
int jf_int8_layernorm_backward(const int8_t* qx, const void* sx, const int8_t* qg, const void* sg, const float* gamma,
                               const float* mean, const float* rstd, int64_t M, int64_t N, int slab, int8_t* qd, void* sd,
                               float* dgamma, float* scratch, int stochastic, const float* noise, uint64_t seed,
                               uint64_t offset, void* stream);

/* int8_add_Ifp_Ig16_Ofp_Og(x1, x2, s_x2, QB, stochastic)   Jetfire/Nonlinear/add.py:164-211 (kernel :29-162)
 * x1: [M,N] of x1_dtype (fp32 or bf16/fp16 residual).  y1: fp32 [M,N] = x1 + q2*s2.  qy/sy: block-quantised y1;
 * the reference converts the quotient to int8 by truncation toward zero, and so does this. */
int jf_int8_add(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1,
                int8_t* qy, void* sy, int stochastic, const float* noise, uint64_t seed, uint64_t offset, void* stream);

/* int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1, x2, s_x2, QB)   Jetfire/Nonlinear/add_mean_var.py:179-231 (kernel :28-177)
 * As jf_int8_add without stochastic rounding, plus mean[M] and rstd[M] = 1/sqrt(E[y^2]-mean^2) of the fp32 sum.
 * scratch: fp32 [2 * M * ceil(N/128)] workspace for the per-tile row partial sums. */
int jf_int8_add_meanvar(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N, float* y1,
                        int8_t* qy, void* sy, float* mean, float* rstd, float* scratch, void* stream);

/* Allocation-free variant of jf_int8_add_meanvar.  It has no counterpart in the reference.
 * For hosts that cannot hand the library a workspace (a plug-in interface that passes only inputs and outputs, a runtime
 * with one fixed device arena and no allocator calls after start-up, a loop that must avoid cudaMalloc because it
 * synchronises the device): the row-partial workspace is a fixed 4 MiB array inside the library image, resident on every
 * GPU that loads the library until the process exits.  Same arguments and results as jf_int8_add_meanvar minus `scratch`.
 * Limit: 2 * M * ceil(N/128) <= 1048576 floats; larger shapes return JF_ERR_SHAPE (use jf_int8_add_meanvar instead).
 * The first call on each device resolves the array's device address (cudaGetSymbolAddress); make that first call
 * outside any stream capture.  The call itself never calls cudaMalloc/cudaFree or any allocating routine.
 * All calls on a device share the one array, which keeps the previous call's contents: nothing in it needs to start at
 * zero (every partial is rewritten before it is read), but two calls whose kernels overlap on the GPU (different streams
 * without ordering) race on it.  The array used is the one of the calling thread's CURRENT device (cudaGetDevice), which
 * must be the device of `stream` and of every operand. */
int jf_int8_add_meanvar_noalloc(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N,
                                float* y1, int8_t* qy, void* sy, float* mean, float* rstd, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Per-block INT8 GEMMs (reference: JetfireGEMMKernel/BlockQuantize/cpp_extension, called from Jetfire/Linear)
 *
 * All three compute, for each 32-wide K block p in ascending order,
 *     I_p = A_blk x B_blk^T (int32),   acc = fma(sa[i,p]*sb[j,p], (float)I_p, acc)   (fp32)
 * and differ in operand layout and epilogue.  Scale tensors are addressed with explicit element strides so both the
 * natural [rows/32, cols/32] layout and the transposed copies the reference passes are accepted without a copy.
 *
 * op16 / op16_bytes (all three): optional scratch for exact fp16 copies of both operands, 2 * (M*K + N*K) bytes, 16-byte
 * aligned.  When it is given (and large enough) the GEMM first writes the two copies ([M,K] and [N,K], transposing where the
 * operand is stored [K, rows]) and then runs on them with tcgen05.mma kind::f16, whose fp32 accumulator already holds
 * float(I_p): the consumers skip the int32 -> fp32 conversion that bounds the int8-operand kernel.  Results are bit-identical
 * either way (every partial sum is an integer below 2^24).  It pays for large GEMMs only (8192^3: 1.75 -> 1.49 ms including the
 * conversion passes); jf_igemm_op16_bytes says when.  NULL / 0 selects the int8-operand kernel.
 * ---------------------------------------------------------------------------------------------------------- */

/* Output selector of the re-quantising GEMMs. */
typedef enum {
    JF_OUT_INT8 = 0,     /* int8 payload + fp16 scales                                                          */
    JF_OUT_DEQUANT_F16 = 1 /* fp16 [M,N] = fp16(q) * scale: the torch dequantisation of linear_fwd.py:30 / linear_bwd.py:27 */
} jf_gemm_out;

/* Forward  Y[M,N] = X[M,K] * W[N,K]^T.
 * igemm_output_int_quantize_bias_rowcol(X, Wt, bias, biasmax, SXt, SWt, M, N, K)
 *   JetfireGEMMKernel/BlockQuantize/cpp_extension/igemm/igemm_BlockSquare32OutputIntQuantizeBiasRowCol.cu:386-434
 *   (kernel :20-383), called from Jetfire/Linear/linear_fwd.py:23 with bias = 0.
 * sx(i,p) = sx[i*sx_stride_m + p*sx_stride_k], sw(j,p) = sw[j*sw_stride_n + p*sw_stride_k] (fp16).
 * out_mode JF_OUT_INT8: y8 int8 [M,N] and sy fp16 [M/32,N/32];  JF_OUT_DEQUANT_F16: y16 fp16 [M,N] (y8/sy may be NULL). */
int jf_igemm_forward(const int8_t* x, const int8_t* w, const void* sx, int64_t sx_stride_m, int64_t sx_stride_k,
                     const void* sw, int64_t sw_stride_n, int64_t sw_stride_k, int64_t M, int64_t N, int64_t K,
                     int out_mode, int8_t* y8, void* sy, void* y16, void* op16, int64_t op16_bytes, void* stream);

/* Input gradient  dX[M,N] = dY[M,K] * W[K,N]   (K = out features, N = in features; W is read in place, no transpose).
 * igemm_output_int_quantize_stochastic(X, W, SXt, SW, M, N, K)
 *   .../igemm/igemm_BlockSquare32OutputIntQuantizeStochastic.cu:372-419 (kernel :18-369), from Jetfire/Linear/linear_bwd.py:17.
 * sg(i,p) = sg[i*sg_stride_m + p*sg_stride_k];  sw(p,j) = sw[p*sw_stride_k + j*sw_stride_n].
 * stochastic != 0: q = clamp(rint(127*acc/amax + noise), -127, 127) with the Philox noise described above. */
int jf_igemm_dgrad(const int8_t* g, const int8_t* w, const void* sg, int64_t sg_stride_m, int64_t sg_stride_k,
                   const void* sw, int64_t sw_stride_k, int64_t sw_stride_n, int64_t M, int64_t N, int64_t K,
                   int out_mode, int8_t* dx8, void* sdx, void* dx16, int stochastic, const float* noise, uint64_t seed,
                   uint64_t offset, void* op16, int64_t op16_bytes, void* stream);

/* Weight gradient  dW[M,N] = dY^T * X   (K = tokens, M = out features, N = in features).
 * igemm_output_fp_no_quantize(X, W, SXt, SW, M, N, K)
 *   .../igemm/igemm_BlockSquare32OutputFp.cu:340-382 (kernel :16-337), from Jetfire/Linear/linear_bwd.py:19.
 * g_transposed = 0: g is dY itself, int8 [K, M] row-major, read in place (no materialised transpose);
 * g_transposed = 1: g is the materialised dY^T, int8 [M, K] row-major, as the reference passes it.
 * x is int8 [K, N] row-major in both cases.
 * sg(p,i) = sg[p*sg_stride_k + i*sg_stride_m];  sx(p,j) = sx[p*sx_stride_k + j*sx_stride_n].
 * out_dtype: JF_F16 (reference) or JF_F32.  split_k >= 1: the K blocks are cut into contiguous ranges of
 * ceil(nblocks/split_k) blocks, each accumulated from zero and summed in ascending order (deterministic);
 * split_k = 1 reproduces the reference's single sequential accumulation; split_k = 0 lets the library choose.
 * scratch: fp32 [splits * M * N] workspace, required when the effective split (jf_igemm_wgrad_plan) is > 1. */
int jf_igemm_wgrad(const int8_t* g, int g_transposed, const int8_t* x, const void* sg, int64_t sg_stride_k,
                   int64_t sg_stride_m, const void* sx, int64_t sx_stride_k, int64_t sx_stride_n, int64_t M, int64_t N,
                   int64_t K, int out_dtype, void* dw, int split_k, float* scratch, void* op16, int64_t op16_bytes, void* stream);

/* Effective split-K the library would use for (M,N,K,split_k) on the current device (>= 1), so that the caller can
 * size `scratch`.  Host-only; launches nothing. */
int jf_igemm_wgrad_plan(int64_t M, int64_t N, int64_t K, int split_k);

/* Size of the fp16 operand scratch (bytes) for a GEMM of these dimensions if the fp16-operand path is expected to pay for its
 * conversion passes, else 0.  Host-only; launches nothing.  No counterpart in the reference. */
int64_t jf_igemm_op16_bytes(int64_t M, int64_t N, int64_t K);

/* Plain int8 x int8 -> int32 product C[M,N] = A[M,K] * B[N,K]^T (test/diagnostic entry point).
 * igemm_basic_int8_gemm   .../igemm/igemm_BasicInt8Gemm.cu:14-110. */
int jf_igemm_int32(const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c, void* stream);

/* Reads and clears the device-side flag raised when a bounded wait inside a GEMM kernel expired (0 = none).
 * Synchronises the device, so callers poll it at their own synchronisation points (end of an optimiser step, end of a timed
 * region): a non-zero value means that GEMM results since the last poll are invalid.  No counterpart in the reference. */
int jf_igemm_error_flag(void);

/* ------------------------------------------------------------------------------------------------------------
 * Language-model head loss (the caller's un-quantised tail):  F.cross_entropy(logits.view(-1, V), targets.view(-1),
 * ignore_index=-1) of INT8_GPT2/qmodel.py:433-439, for bf16 logits, without materialising fp32 logits.
 * forward : lse[r] = log sum_c exp(logits[r, c]);  loss_rows[r] = lse[r] - logits[r, targets[r]]  (0 when targets[r] is outside
 *           [0, V): an ignored position).  The caller averages loss_rows over the positions that count.
 * backward: IN PLACE  logits[r, c] <- (exp(logits[r, c] - lse[r]) - [c == targets[r]]) * (*grad_out) * inv_count  as bf16
 *           (zero rows for ignored positions); `grad_out` is a device pointer to the upstream scalar gradient.
 * logits: bf16 [rows, V] row-major, 16-byte aligned, V a multiple of 8 (every row 16-byte aligned); targets int64 [rows].
 * ------------------------------------------------------------------------------------------------------------ */
int jf_lm_loss_forward(const void* logits_bf16, const int64_t* targets, int64_t rows, int64_t V, float* lse, float* loss_rows,
                       void* stream);
int jf_lm_loss_backward(void* logits_bf16, const int64_t* targets, const float* lse, const float* grad_out, float inv_count,
                        int64_t rows, int64_t V, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Optimiser step of the caller (the un-quantised tail):  scaler.unscale_(optimizer); clip_grad_norm_(params, max_norm);
 * scaler.step(optimizer); scaler.update()  of INT8_GPT2/train.py:320-329 (AdamW, torch's GradScaler), as one entry point that reads
 * every gradient twice and the optimiser state once and never writes the unscaled or clipped gradients.
 * Parameters, first and second moments are three flat fp32 device buffers of `total_chunks * jf_adamw_chunk_elements()` floats in
 * which tensor t occupies the elements starting at start_chunk[t] * jf_adamw_chunk_elements(); segments are back to back
 * (start_chunk[t+1] = start_chunk[t] + ceil(numel[t] / chunk)), numel[t] is a multiple of 4.  grads[t] is the device address of
 * tensor t's fp32 gradient (contiguous, 16-byte aligned).  `grads`, `numel`, `start_chunk`, `weight_decay` are HOST arrays of
 * n_tensors entries (copied into kernel parameters).  max_norm <= 0 disables clipping.  `partial` is a device workspace of
 * total_chunks floats.
 * `state` is 8 device floats owned by the caller, read and updated by the call:
 *   [0] loss scale (the gradients are scale x the true gradients; the caller multiplies its loss by this value; initialise to 1
 *       for training without loss scaling), [1] steps since the scale last changed, [2] optimiser steps taken (initialise 0; the
 *       bias corrections use it), [3] norm of the true gradients, [4] factor the raw gradients were multiplied by
 *       (min(1, max_norm / (norm + 1e-6)) / scale), [5] 1 if this call found a non-finite gradient and therefore changed nothing
 *       but the scale (scale *= backoff_factor), [6], [7] scratch.
 * After growth_interval consecutive good steps the scale is multiplied by growth_factor (growth_interval = 0: never).
 * Arithmetic is fp32 with the expressions of torch.optim.AdamW (scalar factors formed in double and rounded once, as torch does);
 * results agree with torch to rounding (the norm is summed in a different, fixed, order). */
int64_t jf_adamw_chunk_elements(void);
int jf_adamw_clip_step(int64_t n_tensors, const void* const* grads, const int64_t* numel, const int64_t* start_chunk,
                       const float* weight_decay, float* params_flat, float* m_flat, float* v_flat, int64_t total_chunks,
                       double lr, double beta1, double beta2, double eps, double max_norm, float* state, int64_t growth_interval,
                       double growth_factor, double backoff_factor, float* partial, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* JETFIRE_B200_H */
