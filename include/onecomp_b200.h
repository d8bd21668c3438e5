/*
 * C ABI of libonecomp_b200.so: hand-written sm_100a kernels for the GPTQ / QEP
 * layer-quantization path of OneComp (v1.4.0).
 *
 * OneComp exposes no FFI for this path; its boundary is the Python quantizer
 * protocol (GPTQ.quantize_layer, Quantizer.calculate_hessian / adjust_weight,
 * compute_hessian_and_crossterm, pack_int_weights ...).  Each entry point
 * below replaces the torch call sites named in its comment (paths are relative
 * to the OneComp source tree) and is what a binding for that call site would
 * bind.  Conventions:
 *
 *   - plain pointers and sizes only; every pointer is DEVICE memory unless it
 *     says otherwise; matrices are row-major with an explicit leading dimension
 *     in elements;
 *   - nothing here allocates: scratch is passed in, its size comes from the
 *     matching *_workspace_bytes function;
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*);
 *   - the return value is 0 on success or a negative OC_ERR_* code, with a
 *     message available from oc_last_error() (per host thread);
 *   - `status` words are device ints written by the kernels (0 = fine); the
 *     caller reads them after synchronising.
 */
#ifndef ONECOMP_B200_H
#define ONECOMP_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define OC_OK 0
#define OC_ERR_INVALID_ARG (-1)
#define OC_ERR_CUDA (-2)
#define OC_ERR_UNSUPPORTED (-3)
#define OC_ERR_WORKSPACE (-4)
#define OC_ERR_TOO_LARGE (-5)

/* 16-bit element type of weights (`w_dtype`) and activations (`x_dtype`).  The reference works on
 * whatever dtype the model was loaded in (fp16 by default, bf16 for the models that need it,
 * onecomp/model_config.py:32-63) by casting to fp32; so do these kernels.  Outputs that the
 * reference leaves in the module's dtype (corrected weight, dequantized weight) use the same type. */
#define OC_DTYPE_F16 0
#define OC_DTYPE_BF16 1

int oc_version(void);
const char* oc_last_error(void);
/* kernels launched by this library in the calling process so far; reset returns the old count */
long long oc_launch_count(void);
long long oc_launch_count_reset(void);

/* ---- second moments -------------------------------------------------------
 * H <- a_old*H + a_new * Xq^T Xq   and, when C != NULL,
 * C <- a_old*C + a_new * (Xf - Xq)^T Xq,   X* = [n_tok, d] fp16 (ld elements), H, C = [d, d] fp32.
 *
 * Replaces the fp32 cast + scale + SGEMM of Quantizer.calculate_hessian
 * (onecomp/quantizer/_quantizer.py:811-830), calculate_delta_hatX (:869-893),
 * compute_hessian_and_crossterm (onecomp/qep/_quantize_with_qep_arch.py:182-196)
 * and _compute_per_module_hessians (:252-262).  The running mean of the
 * reference is a_old = n/(n+t), a_new = 2/(n+t).
 *
 * xq and xf are read with the same row stride ld.
 *
 * Tensor-core path (tcgen05 + TMA): taken when d, ld are multiples of 8, ldh of 4,
 * pointers 16-byte aligned, n_tok > 0, status != NULL and (for C) delta_scratch
 * (2 * n_tok * d 16-bit elements) is given: it receives Xf - Xq as two 16-bit terms
 * (the rounded difference and its rounding error), so that the product uses the fp32
 * difference the reference forms (:885) to about 2^-22 (fp16) / 2^-16 (bf16) relative, not
 * its 16-bit rounding.  The path writes only the tiles of H that touch the upper
 * triangle: call oc_mirror_upper(H) once after the last accumulation.  C is
 * written in full.  Any other shape runs an fp32 FMA kernel that writes H in full.
 * chunk_tokens (0 = 512): tokens per tensor-core accumulation chain.
 * sm_count: CTAs to launch at most (0 = 148).
 * engine: 0 = automatic, 1 = the FMA kernel, 2 = tensor cores with one CTA per 128 x 256 tile,
 * 3 = tensor cores with one CTA pair (cta_group::2) per 256 x 256 tile.
 * status: 0, or 101..104 / 201..204 when a bounded pipeline wait expired (result invalid).
 */
int oc_moment_accum(const void* xq, const void* xf, void* delta_scratch, long long n_tok, int d,
                    long long ld, float* H, float* C, long long ldh, float a_old, float a_new,
                    int chunk_tokens, int sm_count, int engine, int x_dtype, int* status, void* stream);

/* Same computation as oc_moment_accum for callers that cannot allocate device memory (no
 * counterpart in the reference, which allocates freely through torch).  A host that runs
 * inside another runtime's stream capture, inside a memory pool it does not own, or under a
 * rule that its device footprint must not grow after start-up cannot provide delta_scratch;
 * here that scratch is a fixed 64 MiB device array inside the library image, held on every
 * GPU that loads the library until the process exits.  Inputs and outputs are still the
 * caller's.  Limits and rules:
 *   - with C != NULL, n_tok * ld must not exceed oc_moment_static_capacity() (16 Mi
 *     activation elements; the array holds two 16-bit terms for each); larger calls return
 *     OC_ERR_TOO_LARGE: feed the tokens in several calls;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture;
 *   - the call itself performs no cudaMalloc / cudaFree and calls no allocating routine;
 *   - all calls share the one array and it keeps the previous call's contents; nothing in it
 *     has to start at zero (each call overwrites the part it reads), but two calls that
 *     overlap on the GPU (different streams, no ordering) race on it: order them.
 * Everything else (tensor-core path conditions, oc_mirror_upper afterwards, status codes)
 * is as for oc_moment_accum. */
long long oc_moment_static_capacity(void);
int oc_moment_accum_static(const void* xq, const void* xf, long long n_tok, int d, long long ld,
                           float* H, float* C, long long ldh, float a_old, float a_new,
                           int chunk_tokens, int sm_count, int x_dtype, int* status, void* stream);

/* lower triangle <- upper triangle */
int oc_mirror_upper(float* M, long long ld, int n, void* stream);

/* ---- inverse-Hessian factor -------------------------------------------------
 * U upper triangular, U^T U = (P Hfix P^T + shift I)^-1 where Hfix is H with 1 on
 * dead diagonals (H[j][j] == 0), shift = rel_shift * percdamp * mean(diag Hfix), and
 * P sorts columns by descending diagonal when actorder != 0 (stable; identity
 * otherwise).  Replaces run_gptq's dead-column fix, argsort and gathers
 * (onecomp/quantizer/gptq/_gptq.py:693-702) and _compute_inverse_hessian
 * (:594-643: damping, cholesky, cholesky_inverse, cholesky upper) with one blocked
 * Cholesky factorisation and one triangular inverse.  H is not modified.
 *
 * Outputs: U [n,n] (ldu), perm/invperm int32 [n], dead uint8 [n] (original column
 * order), damp_out float[2] = {percdamp*mean, mean}, status int = 0 or (index+1) of
 * the first non-positive pivot (then U is meaningless: add damping and call again,
 * as the reference's retry loop does; reuse_perm = 1 keeps perm/invperm).
 */
long long oc_hinv_workspace_bytes(int n);
int oc_hinv_factor(const float* H, long long ldh, int n, float percdamp, float rel_shift,
                   int actorder, int reuse_perm, float* U, long long ldu, int* perm, int* invperm,
                   unsigned char* dead, float* damp_out, int* status, void* workspace,
                   long long workspace_bytes, void* stream);

/* The same factorisation for `batch` matrices of equal size (the experts of a mixture), first
 * attempt only (shift = percdamp * mean): H and U [batch, n, n] contiguous, perm / invperm / dead
 * [batch, n], damp_out [batch, 2], status [batch]; the workspace is batch times
 * oc_hinv_workspace_bytes(n).  The panel chain is walked once and every launch covers all
 * matrices.  Problems whose status is non-zero are repeated singly with more damping. */
int oc_hinv_factor_batched(int batch, const float* H, int n, float percdamp, int actorder, float* U,
                           int* perm, int* invperm, unsigned char* dead, float* damp_out, int* status,
                           void* workspace, long long workspace_bytes, void* stream);

/* ---- GPTQ column loop ---------------------------------------------------------
 * Quantizes W [out, d] fp16 (ldw) given U from oc_hinv_factor.  Replaces run_gptq's
 * float conversion, per-channel fit, dead-column zeroing, act-order gather, the
 * per-column loop with group fitting (find_params), the lazy-batch trailing update
 * and the inverse permutation (onecomp/quantizer/gptq/_gptq.py:678-768, 800-840,
 * 886-926), plus the packing of GPTQ.quantize_layer (:445-464; layout
 * onecomp/quantizer/gptq/gptq_layer.py:36-83) and the dequantised weight used for
 * propagation (:153-168).
 *
 * perm / invperm / dead may be NULL (no act-order / no dead columns).
 * blocksize 1..128.  groupsize -1 (per channel) or >= 1; G = 1 or ceil(d/groupsize).
 * mse != 0 adds the reference's shrink search to every parameter fit (:928-950): int(0.8*q_grid)
 * candidate ranges p = 1 - i/q_grid, error sum |deq - x|^q_norm, first minimum wins.
 * Outputs, each optional (NULL skips it); ld_out is the row count of the whole
 * layer when `out` is a row slab of it (pass pointers already offset to the slab;
 * slabs must start on multiples of 32 rows), else `out`:
 *   qweight  int32 [d*bits/32, ld_out]   packed codes, original column order
 *   qzeros   int32 [G, ld_out*bits/32]   packed (zero - 1) & mask
 *   scales16 fp16  [G, ld_out]
 *   scales32 fp32  [G, ld_out]           scales before the fp16 cast
 *   zeros    int32 [G, ld_out]           raw zero points
 *   codes    int32 [out, d]              unpacked codes, original column order
 *   w_hat    fp16  [out, d] (ldwh)       fp16( float(fp16 scale) * (code - zero) )
 */
long long oc_gptq_workspace_bytes(int out, int d, int groupsize);
int oc_gptq_quantize(const void* W, long long ldw, int out, int d, const float* U, long long ldu,
                     const int* perm, const int* invperm, const unsigned char* dead, int wbits,
                     int groupsize, int sym, int blocksize, int mse, int q_grid, float q_norm,
                     int sm_count, int* qweight, int* qzeros,
                     void* scales16, float* scales32, int* zeros, long long ld_out, int* codes,
                     void* w_hat, long long ldwh, int w_dtype, void* workspace,
                     long long workspace_bytes, void* stream);

/* ---- round-to-nearest fallback -----------------------------------------------------
 * Group-wise RTN of W [out, d] fp16 for MoE experts that saw no calibration token
 * (_rtn_fallback_result, onecomp/qep/_quantize_with_qep_arch.py:290-320; rule of
 * pseudo_quantize_tensor, onecomp/quantizer/rtn/quantizer.py:64-181: symmetric range
 * mirrored on both sides, scale clamped to >= 1e-5).  groupsize -1 = whole row; d must be a
 * multiple of the group size.  Outputs: scales, zeros fp32 [out, G]; codes int32 [out, d];
 * deq fp16 [out, d] = fp16((code - zero) * scale). */
int oc_rtn_quantize(const void* W, long long ldw, int out, int d, int wbits, int groupsize, int sym,
                    float* scales, float* zeros, int* codes, void* deq, int w_dtype, void* stream);

/* ---- QEP weight correction ------------------------------------------------------
 * W <- fp16( Wz + perccorr * (Wz C) (P^T U^T U P) ), Wz = W with dead columns zeroed,
 * in place on W [out, d] fp16.  Replaces Quantizer.adjust_weight's SGEMM, potrf and
 * potrs (onecomp/quantizer/_quantizer.py:398-432) given the factor of the same damped
 * Hessian.  out <= 65535 per call.
 */
long long oc_qep_workspace_bytes(int out, int d);
int oc_qep_adjust(void* W, long long ldw, int out, int d, const float* C, long long ldc,
                  const float* U, long long ldu, const int* perm, const unsigned char* dead,
                  float perccorr, int w_dtype, void* workspace, long long workspace_bytes, void* stream);

/* The same column loop for `batch` problems of equal shape, e.g. the experts of a mixture, each
 * with its own factor: every array holds the problems one after another (W [batch, out, ldw],
 * U [batch, d, ldu], perm / invperm / dead [batch, d], qweight [batch, d*bits/32, out], qzeros
 * [batch, G, out*bits/32], scales / zeros [batch, G, out], codes [batch, out, d], w_hat
 * [batch, out, d]); the workspace is batch times oc_gptq_workspace_bytes.  One chain of launches
 * serves all problems (the reference quantizes them one after another,
 * onecomp/qep/_quantize_with_qep_arch.py:546-613). */
int oc_gptq_quantize_batched(int batch, const void* W, long long ldw, int out, int d, const float* U,
                             long long ldu, const int* perm, const int* invperm, const unsigned char* dead,
                             int wbits, int groupsize, int sym, int blocksize, int mse, int q_grid,
                             float q_norm, int sm_count, int* qweight, int* qzeros, void* scales16,
                             float* scales32, int* zeros, int* codes, void* w_hat, int w_dtype,
                             void* workspace, long long workspace_bytes, void* stream);

/* ---- block passes of the QEP driver ----------------------------------------------------
 * y = weight * fp16( float(x) * rsqrt(mean(float(x)^2) + eps) ) for x, y [rows, d] fp16 and
 * weight [d] fp16: the RMSNorm of Llama / Mistral / Qwen blocks in one kernel.  The reference's
 * driver runs the model's own module here (seven elementwise torch kernels through fp32
 * temporaries, inside the block forwards of onecomp/qep/_quantize_with_qep_arch.py:179-180 and
 * onecomp/utils/blockwise.py:527-533). */
int oc_rmsnorm_f16(const void* x, long long ldx, const void* weight, float eps, long long rows, int d,
                   void* y, long long ldy, void* stream);

/* Rotary position embedding of one tensor, y = x*cos + rotate_half(x)*sin with
 * rotate_half(x) = cat(-x[D/2:], x[:D/2]) (the `apply_rotary_pos_emb` of the Llama / Qwen model
 * code that the same block forwards run as six elementwise torch kernels).  x, y: fp16
 * [B, H, S, D], element strides (xsb, xsh, xss, 1) and (ysb, ysh, yss, 1); cos, sin: fp16
 * [B or 1, S, D], strides (cb, cs, 1) with cb = 0 for a broadcast batch.  D % 16 == 0.  Every
 * product and the sum are rounded to fp16 separately, like the unfused operators. */
int oc_rope_f16(const void* x, void* y, const void* cos, const void* sin, long long B, int H, int S, int D,
                long long xsb, long long xsh, long long xss, long long ysb, long long ysh, long long yss,
                long long cb, long long cs, int sm_count, void* stream);

/* y = fp16(fp16(silu(gate)) * up) over n contiguous fp16 elements (y may alias gate): the
 * `act_fn(gate_proj(x)) * up_proj(x)` of the gated MLP in the same block forwards. */
int oc_swiglu_f16(const void* gate, const void* up, void* y, long long n, int sm_count, void* stream);

/* ---- packed-layout utilities (onecomp/quantizer/gptq/gptq_layer.py:36-170) --------
 * pack_int_weights / unpack_int_weights: codes int32 [out, d] <-> qweight int32
 * [d*bits/32, out].  pack_zeros / unpack_zeros: zeros int32 [G, out] <-> qzeros int32
 * [G, out*bits/32]; `add` is added before masking (-1 stores the v1 offset, +1
 * restores it).  bits in {2, 3, 4, 8}.
 */
int oc_pack_qweight(const int* codes, int out, int d, int bits, int* qweight, void* stream);
int oc_unpack_qweight(const int* qweight, int out, int d, int bits, int* codes, void* stream);
int oc_pack_qzeros(const int* zeros, int G, int out, int bits, int add, int* qzeros, void* stream);
int oc_unpack_qzeros(const int* qzeros, int G, int out, int bits, int add, int* zeros, void* stream);

/* GPTQResult.compute_dequantized_weight (onecomp/quantizer/gptq/_gptq.py:84-168) on a
 * packed result: w16[r][c] = fp16( float(scales16[g_idx[c]][r]) * (q - ((stored zero + 1) & mask)) ).
 * g_idx int32 [d] (NULL = one group). */
int oc_dequantize_packed(const int* qweight, const int* qzeros, const void* scales16,
                         const int* g_idx, int out, int d, int bits, void* w16, long long ldw,
                         void* stream);

/* fp32 GEMM engine: C = beta*C + alpha*opA(A)*opB(B); transX = 1 means the operand is
 * stored transposed ([K,M] / [N,K]); flags: see OC_GEMM_* in csrc/common.cuh (0 = dense). */
int oc_gemm_f32(const float* A, long long lda, const float* B, long long ldb, float* C,
                long long ldc, int M, int N, int K, float alpha, float beta, int transA,
                int transB, int flags, void* stream);
/* Engine behind every fp32 product of this library (oc_gemm_f32, the Cholesky and inverse
 * updates, the GPTQ trailing update, the QEP products): mode 0 (default) runs 16-byte aligned
 * operands on the tensor cores as 3xTF32 (fp32-grade accuracy), mode 1 always uses the fp32 FMA
 * kernel.  Returns the previous mode.  oc_gemm_tc_status() is 0 unless a bounded pipeline wait
 * of the tensor-core engine expired on the current device (201..205). */
int oc_set_gemm_engine(int mode);
int oc_gemm_tc_status(void);
/* Output tile of the tensor-core engine for plain products (flags == 0): 0 (default) picks
 * 128x128 or 128x256 tiles per product by the number of waves of tiles over the SMs, 1 forces
 * 128x128, 2 forces 128x256.  Both cut k into the same accumulation chains, so the result bits do
 * not depend on the choice.  Returns the previous setting. */
int oc_set_gemm_tile_shape(int mode);
/* The shape oc_set_gemm_tile_shape(0) gives a product of M x N (x batch) with `flags` on a device
 * with `sms` SMs: 1 = 128x128, 2 = 128x256 (fewer waves of tiles, a wide tile counted as 1.6 narrow
 * ones; lower-tiles-only products count the tiles that reach the diagonal).  Host arithmetic only. */
int oc_gemm_tile_choice(int M, int N, int batch, int flags, int sms);

#ifdef __cplusplus
}
#endif
#endif
