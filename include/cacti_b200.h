/* cacti_b200.h -- C ABI of libcacti_b200.so: hand-written sm_100a kernels that replace
 * the Futhark-generated forward/backward thunks (and the cuBLAS GEMM thunks) of cacti.
 *
 * The ABI follows the conventions of cacti's own FFI crate so that a new symbol
 * table can sit beside the existing ones (cacti_gpu_cu_ffi/src/bindings.rs:378-504):
 *   - every function returns int: 0 = success, anything else is an error code
 *     (cacti_gpu_cu_ffi/src/lib.rs:96-105 maps non-zero to Err(code));
 *   - device pointers are 64-bit integers (CUdeviceptr, cacti_gpu_cu_ffi/src/types.rs:22-25);
 *   - streams are raw CUstream handles (types.rs:78), NULL = the legacy default stream
 *     the reference runs on (src/pctx/nvgpu.rs:263);
 *   - element types use cudaDataType_t codes (types.rs:97-102).
 * No function allocates, frees or synchronises (except where a comment says so);
 * outputs and workspaces are caller-allocated, as for the reference's GEMM thunks
 * (src/thunk/op.rs:4574-4578).  One control thread per device context, as in the
 * reference (src/ctx.rs:21-29).  No function aborts the process or traps the device:
 * a bad argument is a return code, a bad index inside device data is a code written
 * to a caller-supplied status word.
 *
 * Modes: the reference runs a thunk as Apply (fresh output), Accumulate (out += f(args),
 * an elementwise add in the output's dtype, src/thunk/mod.rs:1691-1733) or Initialize
 * (src/thunk/mod.rs:347-351).  Here every gradient output takes `beta`: 0 = Apply,
 * 1 = Accumulate, with the new value rounded to the output dtype before the add.
 *
 * Layout: packed row-major, reductions over the innermost dimension
 * (src/cell/mod.rs:1913-1926).  Arguments may be views at an arbitrary element
 * offset (src/cell/mod.rs:2111-2122): a kernel checks 16-byte alignment at run time
 * and falls back to an element-wise path, so any element-aligned pointer is legal.
 */
#ifndef CACTI_B200_H_
#define CACTI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t cacti_b200_dptr;     /* CUdeviceptr */
typedef void*    cacti_b200_stream;   /* CUstream    */

/* return codes */
enum {
  CACTI_B200_OK                = 0,
  CACTI_B200_ERR_INVALID_VALUE = 1,  /* null pointer, negative size, size overflow      */
  CACTI_B200_ERR_DTYPE         = 2,  /* dtype code not supported by this entry point    */
  CACTI_B200_ERR_WORKSPACE     = 3,  /* workspace missing or smaller than *_workspace_bytes */
  CACTI_B200_ERR_LAUNCH        = 4,  /* the CUDA runtime refused a launch; see cacti_b200_last_cuda_error */
  CACTI_B200_ERR_SHAPE         = 5,  /* shape outside what the entry point supports     */
  CACTI_B200_ERR_INDEX_RANGE   = 6,  /* written to a status word: token/target index out of range */
  CACTI_B200_ERR_NO_DEVICE     = 7,  /* current device is not an sm_100 part            */
  CACTI_B200_ERR_SCRATCH_LIMIT = 8   /* shape needs more scratch than a *_noalloc entry point has built in */
};

/* element types: cudaDataType_t codes (cacti_gpu_cu_ffi/src/types.rs:97-102) */
enum {
  CACTI_B200_R_32F  = 0,
  CACTI_B200_R_16F  = 2,
  CACTI_B200_R_16BF = 14,
  CACTI_B200_R_32I  = 10,   /* index type: int32 targets/tokens */
  CACTI_B200_R_16U  = 22    /* index type: uint16 tokens (src/librarium/llama.rs:383-384) */
};

/* mask_mode of the row softmax */
enum {
  CACTI_B200_MASK_NONE   = 0,
  CACTI_B200_MASK_CAUSAL = 1,  /* column c of row r is masked when c > q_pos(r) */
  /* Same values as CACTI_B200_MASK_CAUSAL, but the zero fill of the masked outputs stops at column
   * B(q_pos) = (q_pos rounded down to a multiple of 256) + 256 when q_off is a multiple of 256, else q_pos + 320;
   * columns at or beyond B are left untouched.  For outputs whose only consumers are block matmuls with a
   * CACTI_B200_TRI_A_* hint (diag = q_off), which read nothing at or beyond B.  No counterpart in the reference. */
  CACTI_B200_MASK_CAUSAL_TRIM = 2
};

int         cacti_b200_version(void);               /* 10000*major + 100*minor + patch */
const char* cacti_b200_error_string(int code);
int         cacti_b200_last_cuda_error(void);       /* cudaError_t of the last failed launch on this thread */
/* Device-side sticky error word (no counterpart in the reference): every wait inside a kernel is bounded; a
 * wait that runs out records a code here instead of hanging.  0 = none; 1 a staged row copy, 2 a matmul pipeline,
 * 3 an attention pipeline, 4 a partial sum of the k-split matmul schedule, 5 the self-test below.  The call
 * synchronises the whole device (cudaDeviceSynchronize), then reads and clears the word; call it from the device's
 * one control thread with nothing else being launched. */
int         cacti_b200_device_error(unsigned* out);
/* Diagnostic, no counterpart in the reference: launches one small CTA whose threads wait, with a limit of `polls`
 * polls (1..4096), on a barrier that nothing arms, and then leave the way every kernel of this library leaves when a
 * wait runs out: together, with their tensor memory released.  result: u32[3] in device memory, written as
 * {1 = the kernel reached its end, 1 = row group 0 left as one, 1 = row group 1 left as one}.  Afterwards
 * cacti_b200_device_error reports code 5.  Nothing faults and nothing waits without a limit. */
int         cacti_b200_selftest_bounded_wait(cacti_b200_dptr result, int polls, cacti_b200_stream stream);
/* Launch-shape knobs ("softmax_threads", "rmsnorm_gpref", ...) for measurement sweeps.  No counterpart
 * in the reference; results do not depend on them. */
int         cacti_b200_tune(const char* name, int value);

/* ---- K1 RMSNorm -----------------------------------------------------------------
 * Replaces the 8-thunk chain of src/librarium/llama.rs:442-451
 * (Cast src/thunk/op.rs:621, Square :2522, InnerMean :3150, AddScalar :1395, Sqrt :2609,
 * BroadcastDiv :2358, BroadcastMul :2058, lossy Cast) and its adjoint chain.
 *   y  = T(f32(gamma) * f32(x) / sqrt(mean(f32(x)^2) + eps))                [rows, cols]
 *   dx = T(gamma*dy/s - x * sum_j(gamma_j dy_j x_j) / (cols * s^3))
 *   dgamma_j = sum_rows dy_ij * x_ij / s_i, written in `dgamma_dtype`
 *              (dtype, or CACTI_B200_R_32F for a partial that a collective reduces).
 * Statistics are recomputed in the backward; the fused form reads x and dy once.
 * The workspace holds per-CTA column partials (deterministic two-stage reduction,
 * no floating-point atomics). */
size_t cacti_b200_rmsnorm_workspace_bytes(int64_t rows, int64_t cols);
int cacti_b200_rmsnorm_fwd(cacti_b200_dptr y, cacti_b200_dptr x, cacti_b200_dptr gamma, float eps,
                           int64_t rows, int64_t cols, int dtype, cacti_b200_stream stream);
/* Residual add fused into the norm that follows it: sum = T(a + b) (AddFutThunkSpec, src/thunk/op.rs:1480-1535; the
 * `stream + o_stream` adds of src/librarium/llama.rs:514,533), y = rmsnorm(sum) as cacti_b200_rmsnorm_fwd.  Both
 * outputs are bit-identical to cacti_b200_add followed by cacti_b200_rmsnorm_fwd; the sum is read back from
 * registers instead of HBM.  `sum` may alias `a` or `b`. */
int cacti_b200_add_rmsnorm_fwd(cacti_b200_dptr y, cacti_b200_dptr sum, cacti_b200_dptr a, cacti_b200_dptr b,
                               cacti_b200_dptr gamma, float eps, int64_t rows, int64_t cols, int dtype,
                               cacti_b200_stream stream);
int cacti_b200_rmsnorm_bwd(cacti_b200_dptr dx, cacti_b200_dptr dgamma, cacti_b200_dptr dy,
                           cacti_b200_dptr x, cacti_b200_dptr gamma, float eps,
                           int64_t rows, int64_t cols, int dtype, int dgamma_dtype,
                           int beta_dx, int beta_dgamma,
                           cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_stream stream);
int cacti_b200_rmsnorm_fwd_bwd(cacti_b200_dptr y, cacti_b200_dptr dx, cacti_b200_dptr dgamma,
                               cacti_b200_dptr x, cacti_b200_dptr gamma, cacti_b200_dptr dy, float eps,
                               int64_t rows, int64_t cols, int dtype, int dgamma_dtype,
                               int beta_dx, int beta_dgamma,
                               cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_stream stream);

/* Same computation as cacti_b200_rmsnorm_fwd_bwd for callers that have no workspace to give.  It has no
 * counterpart in the reference.  It is meant for hosts such as cacti's pctx, which takes almost all device
 * memory into its own arena at start-up and hands thunks only cells from that arena: when the arena is
 * exhausted, or at a point where the host must not enter the CUDA allocator, such a caller cannot produce the
 * workspace the entry point above asks for.  Here the dgamma partials go to an array that is part of the
 * library image (about 4.6 MiB on every device that loads the library, for the life of the process); the
 * function itself calls no cudaMalloc / cudaFree and no allocating library routine.
 * Limits: cols <= 4096 and rows <= 1212416, whichever kernel the shape is routed to; larger shapes return
 * CACTI_B200_ERR_SCRATCH_LIMIT.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call outside any stream capture.
 * All calls share the one array: two calls whose kernels may overlap on the GPU (different streams) race on
 * it.  Nothing in it has to be cleared between calls; every launch overwrites the part it later reads. */
int cacti_b200_rmsnorm_fwd_bwd_noalloc(cacti_b200_dptr y, cacti_b200_dptr dx, cacti_b200_dptr dgamma,
                                       cacti_b200_dptr x, cacti_b200_dptr gamma, cacti_b200_dptr dy, float eps,
                                       int64_t rows, int64_t cols, int dtype, int dgamma_dtype,
                                       int beta_dx, int beta_dgamma, cacti_b200_stream stream);

/* ---- K2 masked row softmax --------------------------------------------------------
 * Replaces cast + BlockTriElemAffine (src/thunk/op.rs:4189-4278) + InnerSoftmax (:3257-3383)
 * + lossy cast (src/librarium/llama.rs:502-505), and the adjoint InnerSoftmaxPostAdj
 * (:3386-3457) with its recomputed softmax (:3376-3382) and the mask adjoint (:4265-4276).
 *   P  = T(softmax_row(mask(f32(S))));  dS = T(mask'(u - (sum u) y)), u = y*f32(dP)
 * q_pos(r) = (r / q_div) % q_mod + q_off.  The reference layout [B,Sq,H,Sk] has
 * q_div = H, q_mod = Sq; a [B,H,Sq,Sk] layout has q_div = 1, q_mod = Sq.
 * Masked inputs are not read; masked outputs are written as exact zeros. */
int cacti_b200_softmax_fwd(cacti_b200_dptr p, cacti_b200_dptr s, int64_t rows, int64_t cols,
                           int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off,
                           int dtype, cacti_b200_stream stream);
int cacti_b200_softmax_bwd(cacti_b200_dptr ds, cacti_b200_dptr s, cacti_b200_dptr dp,
                           int64_t rows, int64_t cols,
                           int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off,
                           int dtype, int beta_ds, cacti_b200_stream stream);
int cacti_b200_softmax_fwd_bwd(cacti_b200_dptr p, cacti_b200_dptr ds, cacti_b200_dptr s, cacti_b200_dptr dp,
                               int64_t rows, int64_t cols,
                               int mask_mode, int64_t q_div, int64_t q_mod, int64_t q_off,
                               int dtype, int beta_ds, cacti_b200_stream stream);

/* ---- K3 RoPE -----------------------------------------------------------------------
 * Replaces symplectic_embed (src/librarium/llama.rs:463-465): BroadcastMul + InnerSymplecticMap
 * (:975-1049) + BroadcastMul + Add (src/thunk/op.rs:1480-1535), and their adjoints.
 *   y = x*cos + rot(x)*sin, rot(x) = [-x[hd/2:], x[:hd/2]];  dx = dy*cos + R(dy*sin)
 * x: [tokens, heads, head_dim]; cos, sin: [pos_mod, head_dim]; position of a token row t
 * is (t + pos_off) % pos_mod.  f16 follows the reference's f16 arithmetic (one rounding
 * per primitive); f32 and bf16 compute in f32 and round once.
 * rope_tables fills cos/sin as init_constants does (src/librarium/llama.rs:389-411). */
int cacti_b200_rope_tables(cacti_b200_dptr cos, cacti_b200_dptr sin, int64_t seq, int64_t head_dim,
                           float theta, int dtype, cacti_b200_stream stream);
int cacti_b200_rope_fwd(cacti_b200_dptr y, cacti_b200_dptr x, cacti_b200_dptr cos, cacti_b200_dptr sin,
                        int64_t tokens, int64_t heads, int64_t head_dim, int64_t pos_mod, int64_t pos_off,
                        int dtype, cacti_b200_stream stream);
int cacti_b200_rope_bwd(cacti_b200_dptr dx, cacti_b200_dptr dy, cacti_b200_dptr cos, cacti_b200_dptr sin,
                        int64_t tokens, int64_t heads, int64_t head_dim, int64_t pos_mod, int64_t pos_off,
                        int dtype, int beta_dx, cacti_b200_stream stream);
int cacti_b200_rope_fwd_bwd(cacti_b200_dptr y, cacti_b200_dptr dx, cacti_b200_dptr x, cacti_b200_dptr dy,
                            cacti_b200_dptr cos, cacti_b200_dptr sin,
                            int64_t tokens, int64_t heads, int64_t head_dim, int64_t pos_mod, int64_t pos_off,
                            int dtype, int beta_dx, cacti_b200_stream stream);

/* Forward RoPE with a head-pitched output: y is [n_tokens, heads, head_pitch], each head's head_dim rotated values
 * followed by zeros, bit-identical to cacti_b200_rope_fwd followed by cacti_b200_block_pad to head_pitch columns (the
 * layout the fused attention reads q and k in; saves that pass).  16-bit types, head_dim % 4 == 0, head_pitch % 4 == 0. */
int cacti_b200_rope_fwd_pitched(cacti_b200_dptr y, cacti_b200_dptr x, cacti_b200_dptr cos, cacti_b200_dptr sin,
                                int64_t n_tokens, int64_t heads, int64_t head_dim, int64_t head_pitch, int64_t pos_mod,
                                int64_t pos_offset, int dtype, cacti_b200_stream stream);

/* ---- K4 SwiGLU -----------------------------------------------------------------------
 * Replaces StandardSilu (src/thunk/op.rs:2867-2910) + Mul (:2001-2056) of
 * src/librarium/llama.rs:526-527 and their adjoints (Logistic :2821-2865 recomputed).
 *   h = silu(g)*u;  du = silu(g)*dh;  dg = (dh*u) * (y*(1-t)+t), y = silu(g), t = sigmoid(g)
 * n = number of elements.  f16 keeps the reference's per-primitive f16 rounding. */
int cacti_b200_swiglu_fwd(cacti_b200_dptr h, cacti_b200_dptr gate, cacti_b200_dptr up,
                          int64_t n, int dtype, cacti_b200_stream stream);
int cacti_b200_swiglu_bwd(cacti_b200_dptr dgate, cacti_b200_dptr dup,
                          cacti_b200_dptr gate, cacti_b200_dptr up, cacti_b200_dptr dh,
                          int64_t n, int dtype, int beta_dgate, int beta_dup, cacti_b200_stream stream);
int cacti_b200_swiglu_fwd_bwd(cacti_b200_dptr h, cacti_b200_dptr dgate, cacti_b200_dptr dup,
                              cacti_b200_dptr gate, cacti_b200_dptr up, cacti_b200_dptr dh,
                              int64_t n, int dtype, int beta_dgate, int beta_dup, cacti_b200_stream stream);

/* ---- K5 softmax cross-entropy ----------------------------------------------------------
 * Replaces cast + InnerSoftmaxCategoricalNLL (src/thunk/op.rs:3460-3569) and its adjoint
 * (recomputed InnerSoftmax, InnerOneHot :883-997, Sub :1782, BroadcastMul), call site
 * src/librarium/llama.rs:542-545.
 *   loss_i = -log softmax(f32(x_i))[k_i];  dlogits = T(w_i * (softmax(x_i) - onehot(k_i)))
 * w_i = w_rows[i] when w_rows != 0, else w_scalar.  loss_sum (optional, f32[1]) receives
 * sum_i w_i*loss_i, reduced in a fixed order; loss_rows (optional, f32[rows]) the per-row
 * losses.  When loss_sum is requested and loss_rows is 0, `workspace` must hold
 * cacti_b200_softmax_nll_workspace_bytes(rows) bytes.  target_dtype: R_32I or R_16U.
 * A target outside [0, vocab) (the reference asserts, src/thunk/op.rs:3538) writes
 * CACTI_B200_ERR_INDEX_RANGE to *status (u32, optional), the row's loss becomes NaN and its
 * gradient omits the one-hot term; nothing traps. */
size_t cacti_b200_softmax_nll_workspace_bytes(int64_t rows);
int cacti_b200_softmax_nll_fwd_bwd(cacti_b200_dptr loss_sum, cacti_b200_dptr loss_rows, cacti_b200_dptr dlogits,
                                   cacti_b200_dptr logits, cacti_b200_dptr targets, int target_dtype,
                                   cacti_b200_dptr w_rows, float w_scalar,
                                   int64_t rows, int64_t vocab, int dtype, int beta_dlogits,
                                   cacti_b200_dptr status, cacti_b200_dptr workspace, size_t workspace_bytes,
                                   cacti_b200_stream stream);
/* forward only: dlogits = 0 skips the gradient */

/* ---- K6 embedding gather / scatter-add ----------------------------------------------------
 * gather replaces OuterSelect (src/thunk/op.rs:1229-1314): out[i,:] = table[tok[i],:], a bit-exact copy.
 * scatter_add is its adjoint (a Futhark vjp in the reference): dtable[v,:] (+)= sum_{i: tok[i]=v} dy[i,:],
 * summed in f32 in token order and rounded once; beta = 0 also zero-fills untouched rows.
 * Out-of-range tokens are reported through *status and skipped. */
int cacti_b200_gather_rows(cacti_b200_dptr out, cacti_b200_dptr table, cacti_b200_dptr tokens, int token_dtype,
                           int64_t n_tokens, int64_t vocab, int64_t cols, int dtype,
                           cacti_b200_dptr status, cacti_b200_stream stream);
size_t cacti_b200_scatter_add_rows_workspace_bytes(int64_t n_tokens, int64_t vocab);
int cacti_b200_scatter_add_rows(cacti_b200_dptr dtable, cacti_b200_dptr dy, cacti_b200_dptr tokens, int token_dtype,
                                int64_t n_tokens, int64_t vocab, int64_t cols, int dtype, int beta,
                                cacti_b200_dptr workspace, size_t workspace_bytes,
                                cacti_b200_dptr status, cacti_b200_stream stream);

/* ---- K7 add / accumulate ------------------------------------------------------------------
 * accumulate replaces the NVRTC kernels accumulate_1d_{f32,f16,u16}_idx32
 * (src/pctx/nvgpu.rs:2598-2668): dst[i] += src[i].  add replaces AddFutThunkSpec
 * (src/thunk/op.rs:1480-1535, the residual adds of src/librarium/llama.rs:514,533). */
int cacti_b200_accumulate(cacti_b200_dptr dst, cacti_b200_dptr src, int64_t n, int dtype, cacti_b200_stream stream);
int cacti_b200_add(cacti_b200_dptr out, cacti_b200_dptr a, cacti_b200_dptr b, int64_t n, int dtype,
                   cacti_b200_stream stream);

/* ---- K8 AdamW32 parameter update --------------------------------------------------------------
 * Replaces the three in-place optimizer thunks AdamW32::step stages per parameter (src/librarium/adamw.rs:46-61):
 * init_online_average_scale, init_online_average_square_scale and init_online_adamw_update32
 * (src/op.rs:950-1023; Futhark bodies src/thunk/op.rs:3929-3934, :3991-3998, :4051-4055), plus the lossy cast that
 * refreshes the 16-bit parameter from its f32 master.
 *   m <- m + a1*(s*g - m);  v <- v + a2*((s*g)^2 - v);  w <- w - lr*(u*m/(sqrt(v) + e) + wd*w)
 * u = unbias2/unbias1, e = eps*unbias2, unbias1 = 1-(1-a1)^iter_nr, unbias2 = sqrt(1-(1-a2)^iter_nr) (src/op.rs:985-1012).
 * master, grad1_avg, grad2_avg: f32[n], updated in place; grad: grad_dtype[n]; param_out: param_dtype[n] or 0.
 * a1, a2 are the reference's averaging rates (its defaults 0.1 and 0.001 correspond to beta1 0.9, beta2 0.999).
 * iter_nr <= 0 is CACTI_B200_ERR_INVALID_VALUE (the reference panics).  Results are bit-identical to running the
 * three f32 programs in sequence. */
int cacti_b200_adamw32_step(cacti_b200_dptr master, cacti_b200_dptr grad1_avg, cacti_b200_dptr grad2_avg,
                            cacti_b200_dptr param_out, cacti_b200_dptr grad, int64_t n, int grad_dtype, int param_dtype,
                            float grad_unscale, float lr, float wd, float a1, float a2, float eps, int iter_nr,
                            cacti_b200_stream stream);

/* ---- G1 / G2 matmul and block matmul ------------------------------------------------------------
 * gemm replaces MatrixMulF16F32GpuThunkImpl -> cublas_gemm (src/thunk/op.rs:4413-4716,
 * cacti_gpu_cu_ffi/src/lib.rs:727-791); gemm_strided_batched replaces BlockMatrixMulF16F32GpuThunkImpl ->
 * cublas_gemm_batched (src/thunk/op.rs:5025-5471, lib.rs:793-885).
 *   C[m,n] = T(alpha * op(A) op(B) + beta * C), 16-bit operands (R_16F or R_16BF), fp32 accumulation.
 * Row-major storage: A is [m,k] with lda (trans_a = 0) or [k,m] (trans_a = 1); B is [k,n] with ldb
 * (trans_b = 0) or [n,k] (trans_b = 1); C is [m,n] with ldc.  alpha and beta are host pointers
 * (lib.rs:748).  The reference's `x.matmul(false, W, true)` (src/librarium/llama.rs:478) is trans_b = 1.
 * Block form: block (i, j), i < batch_outer, j < batch_inner, starts at base + i*stride_outer +
 * j*stride_inner (elements); a stride of 0 broadcasts that operand (src/thunk/op.rs:5181-5182).  For
 * the reference's 4-d layout [nrow, blk_rows, ncol, blk_cols] (src/thunk/op.rs:4936-5022): ld =
 * ncol*blk_cols, stride_outer = blk_rows*ncol*blk_cols, stride_inner = blk_cols.
 * Operands whose base or strides are not multiples of 16 bytes are repacked into `workspace`
 * (cacti_b200_gemm_workspace_bytes; 256-byte aligned); aligned operands need none.  C may have any
 * element-aligned address and strides. */
size_t cacti_b200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch_outer, int64_t batch_inner);
int cacti_b200_gemm(cacti_b200_dptr c, cacti_b200_dptr a, cacti_b200_dptr b, int64_t m, int64_t n, int64_t k,
                    int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                    const float* alpha, const float* beta, int dtype,
                    cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_stream stream);
int cacti_b200_gemm_strided_batched(cacti_b200_dptr c, cacti_b200_dptr a, cacti_b200_dptr b,
                                    int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                                    int trans_a, int trans_b, const float* alpha, const float* beta,
                                    int64_t batch_outer, int64_t batch_inner,
                                    int64_t stride_a_outer, int64_t stride_a_inner,
                                    int64_t stride_b_outer, int64_t stride_b_inner,
                                    int64_t stride_c_outer, int64_t stride_c_inner, int dtype,
                                    cacti_b200_dptr workspace, size_t workspace_bytes, cacti_b200_stream stream);

/* Block matmul with a triangular-structure hint, for the block matmuls around a causally masked softmax
 * (src/librarium/llama.rs:501-507 and their adjoints, src/spine.rs:447-690).  The reference multiplies the full blocks:
 * half of the scores it computes are overwritten by block_causal_attention_mask, and half of the products with the
 * probabilities are products with exact zeros.  Same arguments and result as cacti_b200_gemm_strided_batched, except:
 *   CACTI_B200_TRI_C_LOWER  only C[r, c] with c <= r + diag is wanted (scores, and the adjoint of the probabilities):
 *                           output tiles wholly beyond the diagonal are neither computed nor written; elements of C
 *                           with c > r + diag are unspecified after the call (the causal softmax never reads them).
 *   CACTI_B200_TRI_A_LOWER  the caller guarantees op(A)[r, kk] == 0 for kk > r + diag (P V, dS K);
 *   CACTI_B200_TRI_A_UPPER  the caller guarantees op(A)[r, kk] == 0 for kk < r - diag (P^T dO, dS^T Q):
 *                           k-blocks that hold only such zeros are skipped.  Of the stored matrix (P or dS, row =
 *                           query q, column = key) nothing is read at or beyond column B(q + diag) as defined for
 *                           CACTI_B200_MASK_CAUSAL_TRIM, so that region need not hold zeros, or anything.
 * Where C is specified it is bit-identical to the unhinted call (the skipped products are exact zeros).
 * r, c, kk are indices inside one block; diag = 0 for equal query and key lengths.
 * operand_flags: CACTI_B200_OPERAND_A_PADDED / _B_PADDED say that every stored row of that operand is followed by
 * zeros up to the next multiple of 64 elements (lda / ldb at least that; what cacti_b200_block_pad to 128 produces for
 * head_dim 100): the matmul then reads the padding instead of repacking the operand or clipping its loads.
 * This entry point has no counterpart in the reference, whose cuBLAS call cannot express the structure. */
#define CACTI_B200_TRI_NONE 0
#define CACTI_B200_TRI_C_LOWER 1
#define CACTI_B200_TRI_A_LOWER 2
#define CACTI_B200_TRI_A_UPPER 3
#define CACTI_B200_OPERAND_A_PADDED 1
#define CACTI_B200_OPERAND_B_PADDED 2
int cacti_b200_gemm_strided_batched_tri(cacti_b200_dptr c, cacti_b200_dptr a, cacti_b200_dptr b,
                                        int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                                        int trans_a, int trans_b, const float* alpha, const float* beta,
                                        int64_t batch_outer, int64_t batch_inner,
                                        int64_t stride_a_outer, int64_t stride_a_inner,
                                        int64_t stride_b_outer, int64_t stride_b_inner,
                                        int64_t stride_c_outer, int64_t stride_c_inner, int tri_mode, int64_t diag,
                                        int operand_flags, int dtype, cacti_b200_dptr workspace, size_t workspace_bytes,
                                        cacti_b200_stream stream);

/* ---- A1 block padding and fused causal attention ------------------------------------------------------------
 * block_pad replaces BlockPadFutThunkSpec (src/thunk/op.rs:4065-4186), which the reference stages before a block
 * matmul whose blocks are not 16-byte multiples (src/op.rs:1454-1482): dst[nrow, rows, ncol, cols_pad] =
 * src[nrow, rows, ncol, cols] with zeros in the added columns.  16-bit types. */
int cacti_b200_block_pad(cacti_b200_dptr dst, cacti_b200_dptr src, int64_t nrow, int64_t rows, int64_t ncol,
                         int64_t cols, int64_t cols_pad, int dtype, cacti_b200_stream stream);

/* Fused causal attention forward: the thunk sequence block_matmul_scale, cast, block_causal_attention_mask,
 * inner_softmax, lossy_cast, block_matmul of src/librarium/llama.rs:501-507 as one kernel; the [B, S, H, S] scores and
 * probabilities never reach HBM.  No single counterpart in the reference.
 *   q, k, v : [batch, seq, heads, 128] of dtype (R_16F / R_16BF), head_dim columns of data then zeros
 *             (cacti_b200_block_pad with cols_pad = 128); 16-byte aligned
 *   ctx     : [batch, seq, heads, head_dim], 8-byte aligned
 *   stats   : [batch, heads, seq, 4] f32, 16-byte aligned: word 0 the row maximum m of the rounded scaled scores,
 *             word 1 the sum of exp(s - m) over the unmasked keys (what a backward pass needs to rebuild the
 *             probabilities); words 2 and 3 are scratch of cacti_b200_attention_bwd_prep
 * Scores are rounded to dtype as block_matmul_scale stores them and the softmax runs in f32 on the rounded values
 * with the row maximum subtracted, as the reference does.  exp(s - m) is rounded to dtype before the product with V
 * and the division by the row sum is applied to the f32 result, where the reference rounds the quotient first: ctx
 * agrees with the unfused chain to rounding noise (relative 2^-11 per probability), not bit for bit.
 * Requires seq % 128 == 0, head_dim <= 128, head_dim % 4 == 0 (else CACTI_B200_ERR_SHAPE); query i sees keys <= i. */
int cacti_b200_attention_fwd(cacti_b200_dptr ctx, cacti_b200_dptr stats, cacti_b200_dptr q, cacti_b200_dptr k,
                             cacti_b200_dptr v, int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, float alpha,
                             int dtype, cacti_b200_stream stream);

/* Backward companion of cacti_b200_attention_fwd: rebuilds, tile by tile on the tensor cores, the probabilities and the
 * score adjoints that the reference obtains from its stored scores (block matmul dP = dO V^T, then
 * InnerSoftmaxPostAdj with the recomputed softmax, src/thunk/op.rs:3376-3457):
 *   y = exp(s - m) / l,  P = T(y),  dS = T(y * T(dP) - c * y),  s = T(alpha q.k),  c = dO . O
 * (c equals sum_j y_j dP_j in exact arithmetic; taking it from the stored context row removes the pass over the whole
 * row; it is computed first, by a small streaming kernel, into word 2 of each row's stats: two launches).
 * p, ds: [batch, seq, heads, seq]; entries above the diagonal are written (as zeros) up to the bound B of
 * CACTI_B200_MASK_CAUSAL_TRIM and left untouched beyond it: feed them to cacti_b200_gemm_strided_batched_tri with
 * CACTI_B200_TRI_A_UPPER (dV = P^T dO, dK = alpha dS^T Q) and CACTI_B200_TRI_A_LOWER (dQ = alpha dS K).
 * q, k, v, dctx: [batch, seq, heads, 128] zero-padded (cacti_b200_block_pad); ctx: [batch, seq, heads, head_dim] and
 * stats as produced by cacti_b200_attention_fwd.  Same shape limits.  No single counterpart in the reference. */
int cacti_b200_attention_bwd_prep(cacti_b200_dptr p, cacti_b200_dptr ds, cacti_b200_dptr q, cacti_b200_dptr k,
                                  cacti_b200_dptr v, cacti_b200_dptr dctx, cacti_b200_dptr ctx, cacti_b200_dptr stats,
                                  int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, float alpha, int dtype,
                                  cacti_b200_stream stream);

/* Whole adjoint of the fused attention in one call: dq, dk, dv [batch, seq, heads, head_dim] from q, k, v, dctx (padded
 * to 128 columns as above), ctx and stats of cacti_b200_attention_fwd.  Same arithmetic and rounding points as
 * cacti_b200_attention_bwd_prep followed by the three hinted block matmuls (dV = P^T dO, dQ = alpha dS K,
 * dK = alpha dS^T Q), but P and dS stay in shared memory: one kernel per 128 query rows accumulates dQ over the key
 * tiles before it, one kernel per 128 keys accumulates dK and dV over the query rows after it, each output element by
 * one CTA in a fixed order (no floating-point atomics; S and dP are formed once per kernel).  Three launches (c = dO . O
 * first, into word 2 of stats).  Results agree with the chain above to the summation order inside the tensor cores.
 * It needs no [batch, seq, heads, seq] buffers (4.3 GB for P and dS at 8 sequences of 2048), but evaluates the
 * exponentials twice, which is what bounds these kernels: measured 2.10 ms against 1.42 ms for the chain at
 * [8, 2048, 32, 100].  A caller short of memory takes this one, a caller short of time the chain.
 * dq, dk, dv, ctx 8-byte aligned; same shape limits as cacti_b200_attention_fwd.  No counterpart in the reference. */
int cacti_b200_attention_bwd(cacti_b200_dptr dq, cacti_b200_dptr dk, cacti_b200_dptr dv, cacti_b200_dptr q, cacti_b200_dptr k,
                             cacti_b200_dptr v, cacti_b200_dptr dctx, cacti_b200_dptr ctx, cacti_b200_dptr stats,
                             int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, float alpha, int dtype,
                             cacti_b200_stream stream);

#ifdef __cplusplus
}
#endif
#endif  /* CACTI_B200_H_ */
