/*
 * ftb200 -- C ABI of the B200 (sm_100a) causal linear-attention kernels.
 *
 * This is the drop-in boundary for the native functions of the reference package
 * fast_transformers.causal_product:
 *
 *   causal_dot_product(queries, keys, values, product)                     -> void
 *       fast_transformers/causal_product/causal_product_cuda.cu:1273-1285  (CUDA)
 *       fast_transformers/causal_product/causal_product_cpu.cpp:82-124     (CPU)
 *   causal_dot_backward(queries, keys, values, grad_out, gq, gk, gv)       -> void
 *       fast_transformers/causal_product/causal_product_cuda.cu:1438-1467  (CUDA)
 *       fast_transformers/causal_product/causal_product_cpu.cpp:133-209    (CPU)
 *
 * which the autograd Function reaches through its per-device tables
 * (fast_transformers/causal_product/__init__.py:23-30, 44-49, 64-72).
 *
 * Conventions shared by every entry point
 *   - All data pointers are DEVICE pointers on the current CUDA device of the calling
 *     thread.  The caller allocates every output; the library fills it in place and keeps
 *     no reference (the reference's ownership rule, __init__.py:41,59-61).  Outputs do not
 *     need to be zeroed.
 *   - Tensors are 4-D (N, H, L, dim) with the last dimension contiguous (the reference
 *     asserts stride(3)==1, causal_product_cuda.cu:774-777).  `*_strides` points at three
 *     64-bit ELEMENT strides {batch, head, position}; they may describe permuted views such
 *     as (N, L, H, dim) storage.
 *   - `dtype` is the element type of Q, K, V, grad_out and of the outputs: FTB_F32 or
 *     FTB_BF16.  States are always fp32, stored as (N, H, D, M) contiguous.
 *   - `mode` selects the arithmetic: FTB_MODE_FP32_SIMT (fp32 FMA on CUDA cores, any D, M
 *     up to 512) or FTB_MODE_MMA (tcgen05 tensor cores: TF32 operands for fp32 I/O, bf16
 *     operands for bf16 I/O, fp32 accumulation and fp32 running state).  FTB_MODE_MMA takes
 *     D = M = 64 (fp32, bf16) and D = M = 128 (bf16); and, for fp32, any D and M that are multiples
 *     of 64 (256 random features of a 64-wide query, say, or 128-wide heads): the sums over 64-wide
 *     feature blocks are then taken inside the tensor cores, up to four blocks per launch (no
 *     initial / final states or prepared workspaces for such shapes: FTB_ERR_UNSUPPORTED).
 *     FTB_MODE_MMA_X3 (ftb_causal_dot_product, ftb_causal_dot_backward and the workspace query
 *     only; fp32, D = M = 64; no states or prepared workspaces) also runs on the tensor cores
 *     but keeps fp32 accuracy: every operand is split into a TF32-exact high part and a low part
 *     and every product becomes three (hi hi + lo hi + hi lo, fp32 accumulation).  Its results
 *     belong to the tier of FTB_MODE_FP32_SIMT (1e-5 against fp64) at several times its speed.
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, not synchronised.
 *     FTB_MODE_MMA grids are launched with programmatic stream serialisation: their blocks
 *     may be placed on SMs while the kernel in front of them in the stream drains, but the
 *     first grid of a call touches no global memory before that kernel has completed, so
 *     the ordering a caller observes is that of ordinary launches (also under stream
 *     capture).  FTB200_NO_PDL=1 in the environment selects ordinary launches.
 *   - `workspace` is caller-provided scratch of at least ftb_causal_workspace_bytes(...)
 *     bytes, 256-byte aligned; it may be NULL when that function returns 0.
 *   - Return value: FTB_OK or one of the error codes below.  Nothing is enqueued when an
 *     error is returned.  The library is re-entrant: forward (caller thread) and backward
 *     (autograd thread) may run concurrently.  What it keeps between calls is small and listed
 *     here: per-device caches of looked-up values (SM count, the addresses of the device status
 *     word and of the static scratch array), the launch counter and -- while ftb_timing_enable
 *     is on -- the list of recorded events, the device status word itself, and the static
 *     scratch array of ftb_causal_dot_product_static (shared by all calls on a device).
 */
#ifndef FTB200_H
#define FTB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FTB_OK 0
#define FTB_ERR_UNSUPPORTED 1 /* no kernel for this shape / dtype / mode            */
#define FTB_ERR_ALIGNMENT 2   /* pointer or stride alignment required by the mode    */
#define FTB_ERR_WORKSPACE 3   /* workspace missing or too small                      */
#define FTB_ERR_CUDA 4        /* a CUDA runtime call failed (see ftb_last_cuda_error)*/
#define FTB_ERR_TIMEOUT 5     /* a bounded device-side wait expired                  */
#define FTB_ERR_INVALID 6     /* NULL pointer, negative size, unknown enum           */
#define FTB_ERR_STATIC_LIMIT 7 /* scratch need exceeds FTB_STATIC_SCRATCH_BYTES      */

#define FTB_F32 0
#define FTB_BF16 1

#define FTB_MODE_FP32_SIMT 0
#define FTB_MODE_MMA 1
#define FTB_MODE_MMA_X3 2

/* Library / ABI version (major*1000 + minor). */
int ftb_version(void);

/* Static description of a status code. */
const char *ftb_status_string(int status);

/* cudaError_t of the most recent failed runtime call made by this thread (0 if none). */
int ftb_last_cuda_error(void);

/*
 * Launch accounting (no counterpart in the reference; used by the benchmark).
 * ftb_launch_count: kernels launched by this library in this process so far.
 * ftb_timing_enable(1): from now on every launch (made by any host thread) is bracketed by
 *   CUDA events on its stream.  ftb_timing_read synchronises those events, adds the elapsed
 *   milliseconds and launch counts per kernel kind into the two arrays (length nkinds),
 *   and forgets the recorded launches.  ftb_timing_enable(0) stops recording.
 */
#define FTB_KERNEL_STATE_SUM 0    /* per-segment totals  sum x (x) y                 */
#define FTB_KERNEL_STATE_PREFIX 1 /* exclusive prefix/suffix of the segment totals   */
#define FTB_KERNEL_SIMT_SCAN 2    /* fp32 CUDA-core segment scan                     */
#define FTB_KERNEL_MMA_FWD 3      /* tcgen05 forward                                 */
#define FTB_KERNEL_MMA_BWD 4      /* tcgen05 backward                                */
#define FTB_KERNEL_MMA_STATE 5    /* tcgen05 per-segment totals                      */
#define FTB_KERNEL_MMA_BWD_QR 6   /* tcgen05 grad_Q scan + reverse totals, one grid  */
#define FTB_KERNEL_MMA_BWD_MULTI 7 /* tcgen05 two or three gradient scans, one grid  */
#define FTB_KERNEL_RECURRENT_STEP 8 /* one recurrent step                              */
#define FTB_KERNEL_NORMALISER 9   /* denominator Q . cumsum(K) and its gradients      */
#define FTB_KERNEL_FEATURE_MAP 10 /* elu(x)+1 (x key-length mask) and its gradient    */
#define FTB_KERNEL_RANK_EXCHANGE 11 /* push / receive of per-rank states over peer memory */
#define FTB_KERNEL_APPLY_STATE 12  /* out = a . S for one fixed state per (batch, head) */
#define FTB_KERNEL_KINDS 13
uint64_t ftb_launch_count(void);
/*
 * Device-side status word of the current device: 0, or the FTB_ERR_* code recorded by a kernel
 * whose bounded wait expired (FTB_ERR_TIMEOUT).  Synchronises the whole device first (every stream,
 * non-blocking ones included).  reset != 0 clears it.
 * The reference has no counterpart (its kernels contain no waits).
 */
int ftb_device_status(int reset);
void ftb_timing_enable(int enable);
int ftb_timing_read(float *ms_by_kind, int *launches_by_kind, int nkinds);

/*
 * Scratch bytes needed by ftb_causal_dot_product (backward == 0) or
 * ftb_causal_dot_backward (backward != 0) for this problem.  `want_state` is non-zero when
 * the call will pass a non-NULL final_state / state outputs.
 */
size_t ftb_causal_workspace_bytes(int64_t N, int64_t H, int64_t L, int64_t D, int64_t M,
                                  int dtype, int mode, int backward, int want_state);

/*
 * Forward:  out[n,h,i,:] = q_i . (S_init + sum_{j<=i} k_j (x) v_j)
 * Replaces causal_dot_product(queries, keys, values, product)
 * (causal_product_cuda.cu:1273-1285 / causal_product_cpu.cpp:82-124).
 *
 * initial_state : optional (N,H,D,M) fp32 state added before position 0 (NULL = zeros);
 *                 used when a sequence is split across devices or continued.
 * final_state   : optional (N,H,D,M) fp32 output, S_init + sum over all L positions.
 * workspace_has_states : non-zero when ftb_causal_state_sum(k, v, ...) has just been run with this
 *                 same workspace, shape, dtype and mode (and final_state is NULL): the
 *                 per-segment states it left there are used instead of sweeping K and V again.
 *                 Honoured in FTB_MODE_MMA; ignored (recomputed) otherwise.
 */
int ftb_causal_dot_product(const void *q, const void *k, const void *v, void *out,
                           int64_t N, int64_t H, int64_t L, int64_t D, int64_t M,
                           const int64_t *q_strides, const int64_t *k_strides,
                           const int64_t *v_strides, const int64_t *out_strides,
                           int dtype, int mode, const float *initial_state,
                           float *final_state, int workspace_has_states, void *workspace,
                           size_t workspace_bytes, void *stream);

/*
 * The forward product with the layer's normaliser applied on the way out:
 *
 *   out[n,h,i,:] = ( q_i . sum_{j<=i} k_j (x) v_j ) / (den[n,h,i] + eps)
 *
 * -- lines 95-104 of fast_transformers/attention/causal_linear_attention.py (Z = 1 / (Q . cumsum(K)
 * + eps), V' = causal_linear(Q, K, V) * Z) without the product ever reaching memory unscaled.
 * `den` holds one fp32 value per (batch, head, position) with element strides `den_strides`
 * {batch, head, position} (what ftb_causal_normaliser wrote).  FTB_MODE_MMA with the shapes the
 * 64- and 128-wide kernels take (no wide feature dimension); no states.  Everything else as
 * ftb_causal_dot_product, the workspace included.
 */
int ftb_causal_dot_product_normalised(const void *q, const void *k, const void *v, const float *den,
                                      void *out, int64_t N, int64_t H, int64_t L, int64_t D, int64_t M,
                                      const int64_t *q_strides, const int64_t *k_strides,
                                      const int64_t *v_strides, const int64_t *den_strides,
                                      const int64_t *out_strides, int dtype, int mode, float eps,
                                      void *workspace, size_t workspace_bytes, void *stream);

/*
 * Backward: gq_i = S_i g_i ; gk_i = R_i v_i ; gv_i = R_i^T k_i with
 *           S_i = S_init + sum_{j<=i} k_j (x) v_j   and   R_i = R_init + sum_{j>=i} q_j (x) g_j.
 * Replaces causal_dot_backward(queries, keys, values, grad_out, grad_queries, grad_keys,
 * grad_values) (causal_product_cuda.cu:1438-1467 / causal_product_cpu.cpp:133-209).
 *
 * initial_state      : optional (N,H,D,M) fp32, the same S_init the forward used.
 * grad_q, grad_k, grad_v : a NULL pointer skips that gradient (and the state sweep only it
 *                      needs); at least one must be given.
 * initial_grad_state : optional (N,H,D,M) fp32, R contributed by positions AFTER this
 *                      range (sequence split across devices); NULL = zeros.
 * forward_workspace  : optional; the workspace buffer the forward call on the same
 *                      q, k, v, shape, dtype, mode and initial_state used, if its contents are
 *                      still intact.  It holds the per-segment forward states, which the
 *                      backward then does not recompute (one pass over K and V saved).
 *                      NULL = recompute.  The reference keeps nothing but Q, K, V either.
 * workspace_has_grad_states : non-zero when ftb_causal_state_sum(q, grad_out, ..., reverse = 1)
 *                      has just been run on the SECOND half of `workspace` (offset
 *                      ftb_causal_workspace_bytes(..., backward = 1, 0) / 2); honoured in
 *                      FTB_MODE_MMA, ignored otherwise.
 */
int ftb_causal_dot_backward(const void *q, const void *k, const void *v, const void *grad_out,
                            void *grad_q, void *grad_k, void *grad_v, int64_t N, int64_t H,
                            int64_t L, int64_t D, int64_t M, const int64_t *q_strides,
                            const int64_t *k_strides, const int64_t *v_strides,
                            const int64_t *go_strides, const int64_t *gq_strides,
                            const int64_t *gk_strides, const int64_t *gv_strides, int dtype,
                            int mode, const float *initial_state,
                            const float *initial_grad_state, const void *forward_workspace,
                            int workspace_has_grad_states, void *workspace,
                            size_t workspace_bytes, void *stream);

/*
 * Whole-range state  state[n,h,:,:] = sum_l x[n,h,l,:] (x) y[n,h,l,:]   ((N,H,D,M) fp32).
 * With (x, y) = (K, V) it is what a sequence shard contributes to the forward state of
 * the shards after it; with (x, y) = (Q, grad_out) what it contributes to the backward
 * state of the shards before it.  The reference has no such entry point (it is single
 * device); the sum is the one accumulated by causal_product_cpu.cpp:107-113,186-192.
 * The per-segment states it leaves in `workspace` can be handed to the forward / backward entry
 * points (workspace_has_states / workspace_has_grad_states); pass reverse = 1 when they will seed
 * the backward's descending scans (x = Q, y = grad_out).
 *
 * state == NULL: only partial sums are produced -- ftb_causal_state_parts(...) blocks of (D,M) floats
 * per (batch, head) pair, contiguous at the start of `workspace`, pair after pair -- for a caller
 * that adds them up itself (ftb_exchange_push_parts does, on the way to the peers); the workspace
 * can be handed on exactly as after a call with a state.  ftb_causal_state_parts returns 0 where
 * the workspace would not hold raw partial sums (FTB_MODE_FP32_SIMT or very many segments); the
 * call with state == NULL then returns FTB_ERR_UNSUPPORTED.
 */
int ftb_causal_state_parts(int64_t N, int64_t H, int64_t L, int64_t D, int64_t M, int dtype, int mode);
int ftb_causal_state_sum(const void *x, const void *y, float *state, int64_t N, int64_t H,
                         int64_t L, int64_t D, int64_t M, const int64_t *x_strides,
                         const int64_t *y_strides, int dtype, int mode, int reverse,
                         void *workspace, size_t workspace_bytes, void *stream);

/*
 * The denominator of the attention layer, den[n,h,l] = Q_l . sum_{j<=l} K_j, and its gradients
 * gQ_l = g_l * sum_{j<=l} K_j, gK_j = sum_{l>=j} g_l * Q_l.  Replaces the torch calls of
 * fast_transformers/attention/causal_linear_attention.py:95
 * (`torch.einsum("nlhi,nlhi->nlh", Q, K.cumsum(1))`) and their autograd.
 *
 * q, k, grad_q, grad_k : (N,H,L,D) views, fp32 or bf16, last dimension contiguous, element strides
 *        of {batch, head, position}; den, grad_den : (N,H,L) views with strides of the same three.
 * D <= 256 (FTB_ERR_UNSUPPORTED beyond).  fp32 accumulation; every tensor is streamed once.
 * workspace: ftb_causal_normaliser_workspace_bytes(N,H,L,D,backward) bytes (per-segment sums).
 * In the backward a NULL grad_q or grad_k skips that gradient.
 */
size_t ftb_causal_normaliser_workspace_bytes(int64_t N, int64_t H, int64_t L, int64_t D, int backward);
int ftb_causal_normaliser(const void *q, const void *k, void *den, int64_t N, int64_t H, int64_t L,
                          int64_t D, const int64_t *q_strides, const int64_t *k_strides,
                          const int64_t *den_strides, int dtype, void *workspace,
                          size_t workspace_bytes, void *stream);
int ftb_causal_normaliser_backward(const void *q, const void *k, const void *grad_den, void *grad_q,
                                   void *grad_k, int64_t N, int64_t H, int64_t L, int64_t D,
                                   const int64_t *q_strides, const int64_t *k_strides,
                                   const int64_t *grad_den_strides, const int64_t *grad_q_strides,
                                   const int64_t *grad_k_strides, int dtype, void *workspace,
                                   size_t workspace_bytes, void *stream);

/*
 * The same, ADDED to what grad_q / grad_k hold (the layer's backward: the product's gradients are
 * there already, the denominator's join them without a pass of their own).
 */
int ftb_causal_normaliser_backward_add(const void *q, const void *k, const void *grad_den,
                                       void *grad_q, void *grad_k, int64_t N, int64_t H, int64_t L,
                                       int64_t D, const int64_t *q_strides, const int64_t *k_strides,
                                       const int64_t *grad_den_strides, const int64_t *grad_q_strides,
                                       const int64_t *grad_k_strides, int dtype, void *workspace,
                                       size_t workspace_bytes, void *stream);

/*
 * The same, with the layer's default feature map phi(x) = elu(x) + 1 (and the key-length weights
 * w, one fp32 value per (batch, position), or NULL) taken along: with xq, xk the raw inputs of the
 * map (same shapes as grad_q, grad_k; element strides {batch, head, position}),
 *     grad_q <- (grad_q + n_q) * phi'(xq)        grad_k <- (grad_k + n_k) * w * phi'(xk)
 * i.e. what fast_transformers/feature_maps/base.py:71-73 and attention/causal_linear_attention.py:83
 * contribute to the backward, without a pass of their own.  D = 16, 32, 64 or 128 with 16-byte
 * aligned rows (other shapes: FTB_ERR_UNSUPPORTED, nothing is changed).
 */
int ftb_causal_normaliser_backward_elu(const void *q, const void *k, const void *grad_den,
                                       void *grad_q, void *grad_k, const void *xq, const void *xk,
                                       const float *key_weights, int64_t N, int64_t H, int64_t L,
                                       int64_t D, const int64_t *q_strides, const int64_t *k_strides,
                                       const int64_t *grad_den_strides, const int64_t *grad_q_strides,
                                       const int64_t *grad_k_strides, const int64_t *xq_strides,
                                       const int64_t *xk_strides, int dtype, void *workspace,
                                       size_t workspace_bytes, void *stream);

/*
 * The layer's division, backward: with y = out * Z, Z = 1 / (den + eps) per row
 * (fast_transformers/attention/causal_linear_attention.py:95-104),
 *     grad_out = grad_y * Z        grad_den = -Z * sum_m grad_y * y
 * in one pass.  grad_y, y, grad_out: `rows` contiguous rows of M fp32 values (M = 16, 32, 64 or 128;
 * 16-byte aligned); den, grad_den: one fp32 value per row.
 */
int ftb_normalised_output_grads(const float *grad_y, const float *y, const float *den, float *grad_out,
                                float *grad_den, int64_t rows, int64_t M, float eps, void *stream);

/*
 * The default feature map phi(x) = elu(x) + 1 (fast_transformers/feature_maps/base.py:71-73) with
 * the layer's key-length mask (fast_transformers/attention/causal_linear_attention.py:83) folded
 * in, and its gradient grad_x = grad_y * w * (x > 0 ? 1 : exp(x)).  x, y (grad_y, grad_x):
 * contiguous tensors of `total` elements, fp32 or bf16.  row_mask: NULL, or fp32 weights, one per
 * `elements_per_mask_entry` consecutive elements (for (N,L,H,E) keys and an (N,L) mask: H*E).
 */
int ftb_elu_feature_map(const void *x, void *y, const float *row_mask, int64_t total,
                        int64_t elements_per_mask_entry, int dtype, void *stream);
int ftb_elu_feature_map_backward(const void *x, const void *grad_y, void *grad_x,
                                 const float *row_mask, int64_t total,
                                 int64_t elements_per_mask_entry, int dtype, void *stream);

/*
 * Favor's positive random features (fast_transformers/feature_maps/fourier_features.py:218-243,
 * `stabilize` off), one pass on the tensor cores:
 *     xs = x * softmax_temp^(1/2);  u = xs omega;  off = |xs|^2 / 2 + log(n) / 2
 *     out = [exp(u - off), exp(-u - off)]                      n = 2 * half features per row
 * x: `rows` rows of E = 64 fp32 values, x_row_stride elements apart (16-byte aligned rows);
 * omega_t: the TRANSPOSE of the reference's `omega` buffer, (half, E) fp32 contiguous, half = 64 or
 * 128; out: rows x n fp32, out_row_stride elements apart.  The product runs with TF32 operands
 * (the features match fp64 to about 1e-3 relative): it belongs to the FTB_MODE_MMA tier; other
 * shapes return FTB_ERR_UNSUPPORTED and the caller keeps the reference's torch formulation.
 */
int ftb_favor_feature_map(const float *x, const float *omega_t, float *out, int64_t rows, int64_t E,
                          int64_t half, int64_t x_row_stride, int64_t out_row_stride, float softmax_temp,
                          void *stream);

/*
 * The gradient of ftb_favor_feature_map's input, one pass: with phi = [p, m] the map's output and
 * g = grad_phi,
 *     grad_u = g_p p - g_m m;   grad_off = -sum(g phi)
 *     grad_x = softmax_temp^(1/2) (grad_u omega^T) + softmax_temp grad_off x
 * (what autograd derives from fourier_features.py:218-243).  grad_phi, phi: rows x n fp32 (row
 * strides in elements, rows 16-byte aligned); x: rows x 64; omega: the reference's buffer as it
 * is, (E, half) fp32 contiguous; grad_x: rows x 64.  Same shapes and tier as the forward.
 */
int ftb_favor_feature_map_backward(const float *grad_phi, const float *phi, const float *x,
                                   const float *omega, float *grad_x, int64_t rows, int64_t E,
                                   int64_t half, int64_t grad_phi_row_stride, int64_t phi_row_stride,
                                   int64_t x_row_stride, int64_t grad_x_row_stride, float softmax_temp,
                                   void *stream);

/*
 * One step of the same attention as a recurrent model with a fixed-size state.  Replaces the
 * arithmetic of RecurrentLinearAttention.forward
 * (fast_transformers/recurrent/attention/self_attention/linear_attention.py:55-90), which the
 * reference writes as torch calls:  Q = phi(q), K = phi(k);  z += K;  S += K (x) v;
 * y = (Q . S) / (Q . z + eps).
 *
 * q, k : (N,H,D), v, out : (N,H,M), fp32 or bf16, last dimension contiguous, element strides of
 *        {batch, head} given per tensor.
 * S    : (N,H,D,M) fp32 contiguous, z : (N,H,D) fp32 contiguous -- the state, UPDATED IN PLACE
 *        (zeros for a new sequence; ftb_causal_dot_product's final_state plus the sum of the
 *        key features continue a prefix that was processed in batch form).
 * feature_map : FTB_FEATURE_NONE (q, k are features already) or FTB_FEATURE_ELU1
 *        (phi(x) = elu(x) + 1, the reference's default, applied inside the kernel).
 * D <= 512 (FTB_ERR_UNSUPPORTED beyond).  Inference only: no gradient entry point.
 */
#define FTB_FEATURE_NONE 0
#define FTB_FEATURE_ELU1 1
int ftb_recurrent_linear_step(const void *q, const void *k, const void *v, float *S, float *z,
                              void *out, int64_t N, int64_t H, int64_t D, int64_t M,
                              const int64_t *q_strides, const int64_t *k_strides,
                              const int64_t *v_strides, const int64_t *out_strides, int dtype,
                              int feature_map, float eps, void *stream);

/*
 * One fixed state applied to every position:  out[n,h,l,:] = a[n,h,l,:] . S[n,h]  with S the
 * (N,H,Da,Dc) fp32 state (or, state_is_transposed != 0, stored as (N,H,Dc,Da) and applied as its
 * transpose).  With ftb_causal_state_sum this is the whole of NON-causal linear attention and of its
 * gradients -- the reference writes them as torch.einsum calls
 * (fast_transformers/attention/linear_attention.py:72-78: KV = einsum("nshd,nshm->nhmd", K, V),
 * V' = einsum("nlhd,nhmd,nlh->nlhm", Q, KV, Z)):
 *     S = state_sum(K, V);   out = apply(Q, S);
 *     grad_Q = apply(G, S, transposed);   R = state_sum(Q, G);
 *     grad_K = apply(V, R, transposed);   grad_V = apply(K, R).
 * a, out: (N,H,L,Da) / (N,H,L,Dc) views, fp32 or bf16, last dimension contiguous, element strides of
 * {batch, head, position}.  FTB_MODE_MMA takes the shapes the causal product takes in that mode
 * (FTB_ERR_UNSUPPORTED otherwise, FTB_ERR_ALIGNMENT for rows that do not start on 16 bytes);
 * FTB_MODE_FP32_SIMT takes any Da, Dc.  No scratch memory.
 */
int ftb_linear_apply_state(const void *a, const float *state, void *out, int64_t N, int64_t H, int64_t L,
                           int64_t Da, int64_t Dc, const int64_t *a_strides, const int64_t *out_strides,
                           int dtype, int mode, int state_is_transposed, void *stream);

/*
 * One step of linear CROSS attention over a fixed memory: y = (Q . S) / (Q . z + eps) with
 * Q = phi(q); the state [S (N,H,D,M), z (N,H,D)] -- built once from the memory's keys and values with
 * ftb_causal_state_sum and a sum of the key features -- is only read.  Replaces the arithmetic of
 * RecurrentCrossLinearAttention.forward
 * (fast_transformers/recurrent/attention/cross_attention/linear_attention.py:49-71).
 * Arguments as for ftb_recurrent_linear_step, without k and v.
 */
int ftb_recurrent_cross_linear_step(const void *q, const float *S, const float *z, void *out, int64_t N,
                                    int64_t H, int64_t D, int64_t M, const int64_t *q_strides,
                                    const int64_t *out_strides, int dtype, int feature_map, float eps,
                                    void *stream);

/*
 * Exchange of per-rank states between the GPUs of ONE node without a library collective, for a
 * sequence split across devices (no counterpart in the reference, which is single device; the
 * quantity exchanged is the state of ftb_causal_state_sum).  Every rank creates one buffer and
 * maps the buffers of its peers:
 *
 *   ftb_exchange_create   allocates and zeroes the buffer for states of `elems` floats (a multiple
 *                         of 4) among `world` ranks (<= 16) on the current device and writes its
 *                         FTB_EXCHANGE_HANDLE_BYTES-byte inter-process handle; synchronous.
 *   ftb_exchange_open     maps a peer's buffer from its handle (another process of the same node);
 *                         ftb_exchange_close unmaps it; ftb_exchange_destroy frees the own buffer,
 *                         after every peer has closed it.
 *   ftb_exchange_push     stores `state` into the slot of this rank in the buffers of the ranks
 *                         after it (before it when reverse != 0) and then releases a per-slot
 *                         counter; `buffers` holds `world` pointers in rank order, this rank's own
 *                         buffer at [rank].
 *   ftb_exchange_push_parts  the same for a state given as partial sums: `units` units (the (batch,
 *                         head) pairs) of `unit_elems` floats each, every unit as `parts_per_unit`
 *                         consecutive blocks of unit_elems floats whose sum is the unit's state
 *                         (the layout ftb_causal_state_sum leaves with state == NULL); the blocks
 *                         are added up in a fixed order while they are pushed.
 *   ftb_exchange_receive  waits until the ranks before this one (after it when reverse != 0) have
 *                         delivered, and writes the sum of their states to `out` (zeros when there
 *                         are none).  The wait is bounded (a second unless changed with
 *                         ftb_exchange_wait_limit_ms); on expiry `out` is filled with NaN and
 *                         FTB_ERR_TIMEOUT is recorded in the device status word (read it with
 *                         ftb_device_status before trusting a step).
 *   ftb_exchange_wait_limit_ms  sets how long the kernels launched from now on wait for a peer
 *                         (milliseconds, > 0; process-wide) and returns the previous limit; 0 or a
 *                         negative value only reads it.
 *
 * All ranks must issue the same sequence of push / receive pairs, each rank its push before its
 * receive on one stream.  The exchange number lives in the buffers and is advanced by the kernels,
 * so a captured pair can be replayed.  Every rank must be running on a GPU of its own: a receive
 * waits for kernels of OTHER GPUs only.
 */
#define FTB_EXCHANGE_HANDLE_BYTES 64
size_t ftb_exchange_bytes(int world, int64_t elems);
int ftb_exchange_create(int world, int64_t elems, void **buffer, unsigned char *handle);
int ftb_exchange_open(const unsigned char *handle, void **peer_buffer);
int ftb_exchange_close(void *peer_buffer);
int ftb_exchange_destroy(void *buffer);
int ftb_exchange_wait_limit_ms(int ms);
int ftb_exchange_push(const float *state, int64_t elems, void *const *buffers, int rank, int world,
                      int reverse, void *stream);
int ftb_exchange_push_parts(const float *parts, int64_t unit_elems, int parts_per_unit, int64_t units,
                            void *const *buffers, int rank, int world, int reverse, void *stream);
int ftb_exchange_receive(void *buffer, float *out, int64_t elems, int rank, int world, int reverse,
                         void *stream);

/*
 * Forward product that allocates nothing (it has no counterpart in the reference, whose kernels
 * use no scratch memory at all).
 *
 * Meant for callers that cannot call cudaMalloc when the product runs: code living inside
 * somebody else's memory pool, a serving or real-time loop whose allocator is frozen after
 * start-up, plugin hosts that forbid allocation from plugins.  It computes exactly what
 * ftb_causal_dot_product computes (no initial/final state), but its per-segment state scratch is
 * a static device array inside the library instead of a caller workspace:
 *
 *   - limit: the scratch need, ftb_causal_workspace_bytes(N,H,L,D,M,dtype,mode,0,0), must not
 *     exceed FTB_STATIC_SCRATCH_BYTES (16 MiB); larger problems return FTB_ERR_STATIC_LIMIT and
 *     enqueue nothing.  Every GPU that loads the library holds those 16 MiB until exit.
 *   - the first call on a device resolves the array's device address synchronously (once per
 *     device, whichever host thread makes it); make that call before starting any stream capture.
 *   - all calls on a device share the one array: calls whose kernels can overlap on the GPU
 *     (different streams, no ordering between them) race on it and must be serialised by the
 *     caller.  Stale contents from an earlier call are harmless -- each call writes what it reads.
 *   - it calls no cudaMalloc / cudaFree or other allocating routine; inputs and the output are
 *     still the caller's buffers.
 */
#define FTB_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
int ftb_causal_dot_product_static(const void *q, const void *k, const void *v, void *out,
                                  int64_t N, int64_t H, int64_t L, int64_t D, int64_t M,
                                  const int64_t *q_strides, const int64_t *k_strides,
                                  const int64_t *v_strides, const int64_t *out_strides,
                                  int dtype, int mode, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FTB200_H */
