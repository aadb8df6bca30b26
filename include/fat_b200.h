/*
 * fat_b200.h — C ABI of the B200 (sm_100a) Algebraic-Transformer hot path.
 *
 * One shared library (libfat_b200.so) exports these entry points.  They take raw device
 * pointers, sizes, element strides, a dtype tag, scalars and a CUDA stream (passed as
 * void* so that no CUDA header is needed to bind them).  They never allocate device
 * memory, never synchronise, never throw: each returns FAT_OK or one of the error codes
 * below, and a human-readable detail is available from fat_last_error().  All launches
 * are asynchronous on the given stream.  The caller owns every buffer, including scratch
 * ("workspace") whose size is reported by the matching *_workspace_bytes function.
 *
 * Each entry point replaces one launcher of the reference implementation
 * (SkyeGunasekaran/fastAlgebraicTransformer); the citation names the reference file and
 * lines whose behaviour it reproduces.
 */
#ifndef FAT_B200_H
#define FAT_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FAT_API __attribute__((visibility("default")))
#else
#define FAT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types of tensor arguments */
enum fat_dtype { FAT_F32 = 0, FAT_BF16 = 1, FAT_F16 = 2, FAT_F64 = 3 };

/* return codes */
enum fat_status {
  FAT_OK = 0,
  FAT_ERR_DTYPE = 1,        /* dtype tag not supported by this entry point              */
  FAT_ERR_SHAPE = 2,        /* negative / zero / inconsistent sizes                     */
  FAT_ERR_UNSUPPORTED = 3,  /* valid request outside what the kernels implement         */
  FAT_ERR_ALIGNMENT = 4,    /* a forced fast path needs aligned pointers / strides      */
  FAT_ERR_WORKSPACE = 5,    /* workspace pointer null or too small                      */
  FAT_ERR_LAUNCH = 6,       /* the CUDA runtime rejected a launch (see fat_last_error)  */
  FAT_ERR_NULL = 7          /* a required pointer is null                               */
};

/* attention kernel family selector */
enum fat_attn_path {
  FAT_PATH_AUTO = 0,        /* tensor-core kernels when eligible, else the SIMT kernels */
  FAT_PATH_SIMT = 1,        /* fp32-accumulating CUDA-core kernels (any dtype, D<=128)  */
  FAT_PATH_TENSOR = 2,      /* tcgen05/TMEM kernels (bf16/f16, D in {64,128}); error if not eligible */
  FAT_PATH_TENSOR_DETERMINISTIC = 3   /* same, but the backward never uses the fused kernel, whose d_q is
                               accumulated across key tiles with float32 reduce-adds in an unordered sequence:
                               bit-reproducible gradients at the price of recomputing the scores twice */
};

/* Device-side status word.  The caller allocates one int32 per device, zeroes it, passes it to the
 * attention entry points and reads it back when it wants to know (reading needs a synchronise, so it
 * is left to the caller).  0 = nothing to report.  Otherwise:
 *   bits 24..27 = FAT_DEV_WAIT_TIMEOUT with a detail in bits 0..23: a bounded wait inside a kernel ran
 *                 out and the kernel gave up (its outputs are undefined, the context stays usable);
 *   bit 28      = fat_attn_decode found a sequence whose key/value cache has no room for the new row
 *                 (or a negative length): nothing was appended and that sequence's output is zero;
 *   bit 29      = the tensor-core backward found |q| or |k| >= 65536 in a bfloat16 tensor.  It forms
 *                 d_q and d_k from float16 copies of q and k (see fat_attn_bwd), which were clamped to
 *                 65504: those two gradients are wrong for this call; use FAT_PATH_SIMT for such data;
 *   bit 30      = the fused backward found its shared memory misaligned and did nothing. */
enum fat_device_status { FAT_DEV_OK = 0, FAT_DEV_WAIT_TIMEOUT = 1, FAT_DEV_CACHE_FULL = 0x10000000, FAT_DEV_F16_RANGE = 0x20000000,
                         FAT_DEV_SMEM_ALIGN = 0x40000000 };

FAT_API int fat_version(void);
FAT_API const char* fat_error_string(int code);
FAT_API const char* fat_last_error(void);   /* thread-local detail of the last non-zero return */
/* Number of kernels this library has launched in this process so far (every entry point counts each of its
 * launches; launches recorded into a CUDA graph count once, at capture).  A diagnostic with no counterpart
 * in the reference: benchmarks use it to state how many of this library's kernels ran in a timed region. */
FAT_API unsigned long long fat_launch_count(void);

/* ------------------------------------------------------------------------------------
 * Rational SwiGLU.  out = gate * sigma(gate) * value, sigma(x) = (x/(|x|+1)+1)/2.
 * Tensors are [n_rows, n_cols] with unit column stride and the given row strides (in
 * elements), so the two halves of a packed [rows, 2*ffn] projection can be passed in place.
 * Replaces RationalSwiGLU.forward / swiglu_fwd_kernel   (fused_ops.py:196-229, 490-516)
 * and      RationalSwiGLU.backward / swiglu_bwd_kernel  (fused_ops.py:236-288, 518-539).
 * dtypes: F32, BF16, F16, F64.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_swiglu_fwd(const void* gate, const void* value, void* out,
                   int64_t n_rows, int64_t n_cols,
                   int64_t gate_row_stride, int64_t value_row_stride, int64_t out_row_stride,
                   int dtype, void* stream);

FAT_API int fat_swiglu_bwd(const void* d_out, const void* gate, const void* value,
                   void* d_gate, void* d_value,
                   int64_t n_rows, int64_t n_cols,
                   int64_t d_out_row_stride, int64_t gate_row_stride, int64_t value_row_stride,
                   int64_t d_gate_row_stride, int64_t d_value_row_stride,
                   int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Shifted cross-entropy of the language-model head, forward and gradient in one pass.
 * Replaces the loss of AlgebraicTransformerLM.forward (algebraic_model.py:229-235):
 *   F.cross_entropy(logits[..., :-1, :].contiguous().view(-1, V), labels[..., 1:].contiguous().view(-1), ignore_index)
 * logits [B, T, V] (unit stride along V), labels [B, T] int64.  Row (b, t) is scored against labels[b, t+1]; the
 * last position of every sequence and targets equal to ignore_index (or outside [0, V)) contribute nothing.
 *   row_loss [B*T] float32: the row's -log softmax(logits)[target], 0 for rows that do not count;
 *   d_logits [B*T, V] (dtype of logits, dense): (softmax - onehot) / n_valid[0], 0 for rows that do not count; may be
 *            null (loss only) and may be the logits buffer itself when that is dense (the gradient replaces the logits);
 *   n_valid: device pointer to the number of rows that count, as float32 (the caller counts the labels).
 * loss = sum(row_loss) / n_valid.  fat_scale_unless_one multiplies d_logits by the scalar gradient that reaches the
 * loss and returns without touching memory when that scalar is exactly 1.  dtypes: F32, BF16, F16.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_shifted_ce_fwd(const void* logits, const int64_t* labels, const float* n_valid, float* row_loss,
                 void* d_logits, int B, int T, int V, int64_t logits_batch_stride, int64_t logits_token_stride,
                 int64_t labels_batch_stride, int64_t labels_token_stride, int64_t ignore_index, int dtype, void* stream);

FAT_API int fat_scale_unless_one(void* x, int64_t n, const float* scale, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Mean-error normalisation.  mean_r = mean_c |x_rc| (float32, [n_rows], saved for the
 * backward), y = x / (mean + eps) * weight.
 * Replaces MeanErrorNorm.forward / mean_error_norm_fwd_kernel (fused_ops.py:295-342, 542-569).
 * The backward produces d_x AND d_weight (the reference computes d_weight with two extra
 * PyTorch passes, fused_ops.py:593-597; here it comes from per-block partial sums held in
 * the workspace and a second small reduction kernel).  sign(0) = 0.
 * Replaces MeanErrorNorm.backward / mean_error_norm_bwd_kernel (fused_ops.py:349-423, 572-599).
 * d_weight has the dtype of x.  dtypes: F32, BF16, F16, F64.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_norm_fwd(const void* x, const void* weight, void* y, float* mean,
                 int64_t n_rows, int64_t n_cols, int64_t x_row_stride, int64_t y_row_stride,
                 double eps, int dtype, void* stream);

FAT_API size_t fat_norm_bwd_workspace_bytes(int64_t n_rows, int64_t n_cols, int dtype);

FAT_API int fat_norm_bwd(const void* d_out, const void* x, const void* weight, const float* mean,
                 void* d_x, void* d_weight, void* workspace, size_t workspace_bytes,
                 int64_t n_rows, int64_t n_cols,
                 int64_t d_out_row_stride, int64_t x_row_stride, int64_t d_x_row_stride,
                 double eps, int dtype, void* stream);

/* Residual addition fused with the normalisation that follows it in a pre-norm block:
 *   h = x + residual (rounded to the tensor dtype, written to h_out), y = norm(h) * weight, mean = mean|h|.
 * Replaces the pair `x = x + sublayer(...)` / `self.norm(x)` of AlgebraicBlock.forward and of the model's final
 * norm (algebraic_model.py:149-152, 224): one pass over four tensors instead of an addition pass over three and a
 * normalisation pass over two.  Results are bit-identical to fat_norm_fwd applied to the rounded sum.
 * Backward: d_sum = d_h + [gradient of the normalisation w.r.t. h] (d_h may be NULL: no gradient reached h
 * along the residual path); d_sum is the gradient of both x and residual.  Workspace as for fat_norm_bwd.
 * Rows the register kernels do not take (unaligned, odd widths) run as two passes. */
FAT_API int fat_add_norm_fwd(const void* x, const void* residual, const void* weight, void* h_out, void* y, float* mean,
                 int64_t n_rows, int64_t n_cols, int64_t x_row_stride, int64_t residual_row_stride,
                 int64_t h_row_stride, int64_t y_row_stride, double eps, int dtype, void* stream);

FAT_API int fat_add_norm_bwd(const void* d_y, const void* d_h, const void* h, const void* weight, const float* mean,
                 void* d_sum, void* d_weight, void* workspace, size_t workspace_bytes,
                 int64_t n_rows, int64_t n_cols, int64_t d_y_row_stride, int64_t d_h_row_stride,
                 int64_t h_row_stride, int64_t d_sum_row_stride, double eps, int dtype, void* stream);

/* Mean-error-norm backward for callers that cannot provide scratch memory.
 * (No counterpart in the reference: its backward lets PyTorch allocate whatever it needs.)
 *
 * Some hosts of this library may not allocate device memory when they call in: a plugin
 * invoked from inside another framework's memory plan, a runtime whose arena is already carved
 * up, a callback running where cudaMalloc is forbidden.  fat_norm_bwd needs a workspace for
 * the per-block partial sums of d_weight; this variant keeps that workspace in a fixed 16 MiB
 * array that is part of the library image, so the caller passes inputs and outputs only.  It
 * calls no allocator of any kind.
 *
 *  - Limit: fat_norm_bwd_workspace_bytes(n_rows, n_cols, dtype) must not exceed
 *    fat_norm_bwd_static_capacity() (16 MiB; the workspace is one row of partial sums per
 *    block of the kernel's grid, two blocks per SM: on a 148-SM B200 up to 14168 columns for
 *    F32/BF16/F16, 7084 for F64); larger requests return FAT_ERR_WORKSPACE and launch nothing.
 *  - Every GPU on which the library is loaded holds the 16 MiB until the process exits.
 *  - The first call on each device looks up the array's device address (one host-side
 *    query, with that device current).  Make that first call before starting a stream capture.
 *    The address is remembered per device ordinal and belongs to the device's primary context
 *    (the one the CUDA runtime uses): a process that destroys and re-creates that context
 *    (cudaDeviceReset) or calls in under a context of its own must not use this entry point.
 *  - All calls on one device share the array.  It is fully rewritten by each call before it
 *    is read, so nothing has to be cleared, but two calls that overlap on the GPU (different
 *    streams) race on it: serialise them.
 * Results are identical to fat_norm_bwd. */
FAT_API size_t fat_norm_bwd_static_capacity(void);

FAT_API int fat_norm_bwd_static(const void* d_out, const void* x, const void* weight, const float* mean,
                 void* d_x, void* d_weight,
                 int64_t n_rows, int64_t n_cols,
                 int64_t d_out_row_stride, int64_t x_row_stride, int64_t d_x_row_stride,
                 double eps, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Rational softmax over the last dimension.  p = sigma(x)^4 / (sum_c sigma(x)^4 + eps).
 * Replaces RationalSoftmax.forward / rational_softmax_fwd_kernel (fused_ops.py:52-106, 435-462).
 * The backward recomputes p from x (the row is held in registers), so it reads only d_out
 * and x:  d_x = 2 sigma^3 r^2 / (Z+eps) * (d_out - sum_c d_out p),  r = 1/(|x|+1).
 * Replaces RationalSoftmax.backward / rational_softmax_bwd_kernel (fused_ops.py:113-189, 464-487).
 * dtypes: F32, BF16, F16, F64.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_softmax_fwd(const void* x, void* p, int64_t n_rows, int64_t n_cols,
                    int64_t x_row_stride, int64_t p_row_stride,
                    double eps, int dtype, void* stream);

FAT_API int fat_softmax_bwd(const void* d_out, const void* x, void* d_x,
                    int64_t n_rows, int64_t n_cols,
                    int64_t d_out_row_stride, int64_t x_row_stride, int64_t d_x_row_stride,
                    double eps, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Rational attention with ALiBi.  For head h, query i, key j (j <= i when causal):
 *     s_ij = scale * q_i.k_j - slope_h * |i-j|,   f_ij = sigma(s_ij)^4,
 *     L_i  = sum_j f_ij  (float32 [B,H,T], contiguous, WITHOUT eps),
 *     O_i  = sum_j f_ij v_j / (L_i + eps).
 * q, k, v, out are [B,H,T,D] with unit stride along D; *_strides point to three element
 * strides {batch, head, token}, so views of a packed [B,T,3,H,D] projection are consumed
 * in place.  slopes is float32 [H].  status may be null.
 * out_lo (optional, may be null; same dtype and strides as out) receives the rounding residual
 * of the output, out_lo = round(O - out): with 16-bit tensors out + out_lo carries O to ~16
 * significant bits, which the backward needs for Delta_i = d_out_i . O_i to stay inside the
 * 16-bit tolerance.  The reference has no such tensor (it keeps only the rounded output).
 * Replaces rational_attention_forward / rational_attention_fwd_kernel (forward.py:49-159, 267-319).
 * dtypes: F32, BF16, F16.  D <= 128.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_attn_fwd(const void* q, const void* k, const void* v, const float* slopes,
                 void* out, void* out_lo, float* L,
                 int B, int H, int T, int D,
                 const int64_t* q_strides, const int64_t* k_strides,
                 const int64_t* v_strides, const int64_t* out_strides,
                 double scale, double eps, int causal, int dtype, int path,
                 int* status, void* stream);

/* Backward: given d_out, the saved out and L, produces d_q, d_k, d_v (same dtype as q):
 *     Delta_i = d_out_i . out_i,   dP_ij = d_out_i . v_j,   r = 1/(|s|+1),
 *     dS_ij = 2 sigma^3 r^2 (dP_ij - Delta_i) / (L_i + eps),
 *     d_q = scale dS k,  d_k = scale dS^T q,  d_v = P^T d_out.
 * out_lo is the optional residual written by the forward (null: Delta uses the rounded out).
 * The workspace holds Delta (and, for the tensor-core path, 1/(L+eps), max|d_out| per (batch, head)
 * and a float32 d_q accumulator).
 * Tensor-core path: dS enters the d_q and d_k contractions as float16 (bfloat16's 8 significand bits
 * would leave a few elements in 10^4 outside rel 2e-2 / abs 1e-2), scaled by a power of two chosen
 * from max|d_out| of the (batch, head), so gradients of any magnitude keep their precision.  For
 * bfloat16 tensors q and k take part in those contractions as float16 copies made in shared memory:
 * exact for magnitudes in [2^-14, 65504], absolute error <= 2^-25 below, clamped (and reported in the
 * status word, bit 29) from 65536 on.
 * Replaces rational_attention_backward / rational_attention_bwd_dq_kernel /
 * rational_attention_bwd_dkv_kernel (backward.py:62-158, 165-266, 273-341).
 * ---------------------------------------------------------------------------------- */
FAT_API size_t fat_attn_bwd_workspace_bytes(int B, int H, int T, int D, int dtype, int path);

FAT_API int fat_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* out_lo, const float* L,
                 const void* d_out, const float* slopes,
                 void* d_q, void* d_k, void* d_v,
                 void* workspace, size_t workspace_bytes,
                 int B, int H, int T, int D,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const int64_t* out_strides, const int64_t* d_out_strides,
                 const int64_t* d_q_strides, const int64_t* d_k_strides, const int64_t* d_v_strides,
                 double scale, double eps, int causal, int dtype, int path,
                 int* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Padding mask over the keys.  The reference's model takes attention_mask [B, T] (0 = padding) and, on its PyTorch path
 * only, fills the scores of padded keys with -1e4 before the rational softmax (algebraic_model.py:128-131:
 * scores.masked_fill_(mask[:, None, None, :] == 0, -1e4)); its Triton path never sees the mask (algebraic_model.py:93-104).
 * Here the attention kernels of both families honour it: a masked key gets weight zero for every query (the reference's
 * -1e4 leaves sigma^4 = 6e-18), its d_k and d_v rows come out as zero, and a query that sees no key at all gets a zero
 * output row.  The kernels read the mask as bits: fat_key_mask_words(T) = 4 * ceil(T / 128) 32-bit words per batch element,
 * bit (j & 31) of word (j >> 5) set = key j takes part, bits from T on clear.  fat_pack_key_mask builds them from a
 * byte mask [B, T] (non-zero = the key takes part; element strides given).  fat_attn_fwd_masked / fat_attn_bwd_masked are
 * fat_attn_fwd / fat_attn_bwd with the packed mask as one more argument (null = no mask: the same call as the plain entry
 * point); the backward must be given the mask its forward was given.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_key_mask_words(int T);
FAT_API int fat_pack_key_mask(const uint8_t* mask, uint32_t* bits, int B, int T, int64_t mask_batch_stride,
                 int64_t mask_token_stride, void* stream);
FAT_API int fat_attn_fwd_masked(const void* q, const void* k, const void* v, const float* slopes, const uint32_t* key_mask_bits,
                 void* out, void* out_lo, float* L, int B, int H, int T, int D,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides, const int64_t* out_strides,
                 double scale, double eps, int causal, int dtype, int path, int* status, void* stream);
FAT_API int fat_attn_bwd_masked(const void* q, const void* k, const void* v, const void* out, const void* out_lo, const float* L,
                 const void* d_out, const float* slopes, const uint32_t* key_mask_bits, void* d_q, void* d_k, void* d_v,
                 void* workspace, size_t workspace_bytes, int B, int H, int T, int D,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const int64_t* out_strides, const int64_t* d_out_strides,
                 const int64_t* d_q_strides, const int64_t* d_k_strides, const int64_t* d_v_strides,
                 double scale, double eps, int causal, int dtype, int path, int* status, void* stream);

/* ------------------------------------------------------------------------------------
 * Decode step: rational attention of ONE new token per sequence over a key/value cache.
 *     out[b,h,:] = sum_j f_j v_j / (sum_j f_j + eps),  f_j = sigma(q . k_j scale - slope_h (n_b - j))^4,  j = 0..n_b
 * where n_b = n_cached[b] rows are already in the cache and the new token's key/value rows (k_new, v_new) are first
 * appended at row n_b by the same launch (n_cached itself is not changed: the caller advances it once per model step,
 * after all layers).  It equals row n_b of the causal forward over the n_b + 1 tokens, which is what the reference's
 * generate() recomputes from scratch for every new token (algebraic_model.py:239-265: the whole prefix runs through
 * forward() again; there is no cache in the reference).
 *   q, k_new, v_new, out: [B, H, D] with element strides {batch, head} and unit stride along D;
 *   k_cache, v_cache:     [B, H, capacity, D] with element strides {batch, head, token};
 *   n_cached:             int32 [B] on the device (a CUDA graph of the step can be replayed as it grows).
 * A sequence with n_cached[b] < 0 or >= capacity gets zeros, nothing is appended and bit 28 of the status word is set.
 * Bit-reproducible from run to run (the partial sums of a key range meet in one fixed order).  Pointers 16-byte aligned,
 * strides multiples of 16 bytes.  dtypes: F32, BF16, F16.  D in {32, 64, 128}.
 * ---------------------------------------------------------------------------------- */
FAT_API int fat_attn_decode(const void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                 const int32_t* n_cached, const float* slopes, void* out,
                 int B, int H, int capacity, int D,
                 const int64_t* q_strides, const int64_t* k_new_strides, const int64_t* v_new_strides,
                 const int64_t* out_strides, const int64_t* k_cache_strides, const int64_t* v_cache_strides,
                 double scale, double eps, int dtype, int* status, void* stream);

/* Which kernel family FAT_PATH_AUTO would pick for these arguments (FAT_PATH_SIMT or
 * FAT_PATH_TENSOR), for the forward (backward = 0) or the backward (backward = 1) launch.
 * Host-only, no launch. */
FAT_API int fat_attn_select_path(int T, int D, int dtype, int aligned16, int causal, int backward);

#ifdef __cplusplus
}
#endif
#endif /* FAT_B200_H */
