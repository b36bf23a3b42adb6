/* cinnamon_b200 — C ABI of the B200 (sm_100a) FP8 training kernels.
 *
 * A drop-in for the GPU half of cinnamon's src/kernels.py (shyampathak22/cinnamon):
 * each entry point replaces one Triton launch of that file.  Every pointer is a
 * DEVICE pointer unless stated otherwise; sizes are in elements; `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  Nothing here
 * synchronises the host with the device.
 *
 * Every function returns 0 on success or one of the CINN_ERR_* codes; the text of
 * the last failure on the calling thread is available from cinn_last_error().
 * The reference signals bad arguments with Python `assert` (src/kernels.py:194-195,
 * 237-238, 296, 683); the Python layer above this ABI turns non-zero codes into
 * AssertionError / RuntimeError accordingly.
 */
#ifndef CINNAMON_B200_H
#define CINNAMON_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CINN_OK 0
#define CINN_ERR_INVALID 1
#define CINN_ERR_CUDA 2
#define CINN_ERR_UNSUPPORTED 3
#define CINN_ERR_DEVICE 4

/* element type tags */
#define CINN_BF16 0
#define CINN_F32 1
#define CINN_F16 2
#define CINN_F32_BF16 3 /* GEMM output only: the bf16-rounded result stored as fp32 (what autograd makes of a bf16
                           gradient for an fp32 parameter, without the separate cast kernel) */

/* fp32 division flavour used for amax/448 and x/scale */
#define CINN_DIV_FULL 0 /* PTX div.full.f32: what Triton emits for the reference kernels on a GPU */
#define CINN_DIV_RN 1   /* IEEE round-to-nearest: what a CPU restatement of the reference computes */

/* layout of the B operand of cinn_fp8_gemm */
#define CINN_B_NK 0 /* B stored (N, K), reduction axis contiguous  (a weight as nn.Linear keeps it) */
#define CINN_B_KN 1 /* B stored (K, N), output axis contiguous     (what fp8_matmul_dsv3 documents) */

int cinn_version(void);
const char* cinn_last_error(void);

/* Row-wise 1 x block_size quantisation to e4m3 with one fp32 scale per tile.
 * Replaces quantize_fp8_rowwise_kernel + quantize_fp8_rowwise (src/kernels.py:19-71, 178-216).
 * x: (M, N) of x_dtype, element (m, n) at x[m*ld_m + n*ld_n] (any non-negative strides, as the
 * reference passes x.stride(), :209).  q: (M, N) bytes, contiguous.  scales: (M, ceil(N/block_size)). */
int cinn_quant_rowwise(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n,
                       void* q, float* scales, int block_size, int round_scale, int div_mode, void* stream);

/* Both 1 x 128 quantisations of one (M, N) matrix with contiguous rows of pitch ld, in one pass over it:
 *   q_row (M, N), s_row (M, ceil(N/128)): tiles along N, as cinn_quant_rowwise(x);
 *   q_col (N, M), s_col (N, ceil(M/128)): tiles along M of the transpose, as cinn_quant_rowwise(x^T).
 * Replaces the two quantize_fp8_rowwise calls of FP8MatmulFunction.backward on grad_flat and on
 * grad_flat.t() (src/kernels.py:771 and :781-783); the results are bit-identical to those two calls. */
int cinn_quant_rowwise_dual(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row,
                            void* q_col, float* s_col, int round_scale, int div_mode, void* stream);

/* Diagnostic (no reference counterpart).  With CINN_DIV_FULL the quantisers form x / scale as
 * x * rcp.approx(scale), the reciprocal taken once per scale.  This call checks on the current GPU that the
 * product has the bits of div.full.f32(x, scale) - the instruction Triton emits for the reference kernels
 * (src/kernels.py:60, :121) - for every positive bf16 and fp16 amax (both scale kinds), every 16-bit x and
 * 65536 fp32 patterns per scale, and writes the number of differing pairs to *mismatches (host memory).
 * Synchronises the stream. */
int cinn_selfcheck_division(unsigned long long* mismatches, void* stream);

/* Row-wise 1 x 128 quantisation of x (M, N; contiguous rows of pitch ld; N a multiple of 16) together with the
 * 128 x 128 block re-quantisation of that result, in one pass over x:
 *   q_row (M, N), s_row (M, ceil(N/128)):                  as cinn_quant_rowwise(x);
 *   q_block (M, N), s_block (ceil(M/128), ceil(N/128)):    as cinn_requant_row_to_block(q_row, s_row).
 * Replaces the quantize_fp8_rowwise of FP8MatmulFunction.forward (src/kernels.py:746) plus the
 * dequantize_fp8_rowwise -> quantize_fp8_blockwise pair its backward runs on the saved activations (:784-787);
 * bit-identical to those calls.  round_scale applies to the row-wise scales only, as in the reference. */
int cinn_quant_rowwise_with_block(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row,
                                  void* q_block, float* s_block, int round_scale, int div_mode, void* stream);

/* The same with the block-scaled bytes written transposed: q_block_t is (N, M) with M contiguous (M a multiple of
 * 16), s_block unchanged.  That is the layout in which the weight-gradient GEMM of FP8MatmulFunction.backward
 * (src/kernels.py:788: grad_weight = dy^T @ x_block) reads x_block with the token axis - its reduction axis -
 * contiguous, i.e. K-major, like the forward reads a weight. */
int cinn_quant_rowwise_with_block_t(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row,
                                    void* q_block_t, float* s_block, int round_scale, int div_mode, void* stream);

/* Block-wise block_m x block_n quantisation.
 * Replaces quantize_fp8_blockwise_kernel + quantize_fp8_blockwise (src/kernels.py:74-132, 219-259).
 * scales: (ceil(M/block_m), ceil(N/block_n)). */
int cinn_quant_blockwise(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n,
                         void* q, float* scales, int block_m, int block_n, int round_scale, int div_mode,
                         void* stream);

/* 128 x 128 block-wise quantisation of x (M, N; contiguous rows of pitch ld; M, N, ld multiples of 4) that also
 * writes the byte-transposed copy q_t (N, M) in the same pass; one set of scales serves both (a block and its
 * transpose share their scale).  Replaces quantize_fp8_blockwise on the weight (src/kernels.py:747) plus the
 * `w_fp8.t().contiguous()` copy (:748): the forward reads q, the input gradient (:774) reads q_t, both with their
 * reduction axis innermost. */
int cinn_quant_blockwise_t(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q, void* q_t, float* scales,
                           int round_scale, int div_mode, void* stream);

/* Row-scaled e4m3 (1x128 tiles) -> block-scaled e4m3 (128x128) in one pass.
 * Replaces dequantize_fp8_rowwise followed by quantize_fp8_blockwise in the weight-gradient path
 * (src/kernels.py:784-787) without the fp32 temporary.  xq: (M, K) bytes, xs: (M, ceil(K/128)).
 * out: (M, K) bytes, or (K, M) when transpose_out != 0.  scales: (ceil(M/128), ceil(K/128)). */
int cinn_requant_row_to_block(const void* xq, const float* xs, int64_t M, int64_t K, void* out, float* scales,
                              int transpose_out, int div_mode, void* stream);

/* out[r, c] = e4m3(q[r, c]) * scales[(r / block_m) * ceil(N/block_n) + c / block_n].
 * Replaces dequantize_fp8_kernel + dequantize_fp8 (bf16 out, src/kernels.py:135-173, 284-314) and
 * dequantize_fp8_rowwise (fp32 out with block_m = 1, src/kernels.py:262-281). */
int cinn_dequant(const void* q, const float* scales, void* out, int out_dtype, int64_t M, int64_t N,
                 int block_m, int block_n, void* stream);

/* h = silu(h12[:, :I]) * h12[:, I:] in fp32, rounded to the dtype of h12, then quantised row-wise (1x128) to e4m3.
 * Replaces the torch ops between the two grouped GEMMs of GroupedExperts.forward (src/layers.py:72-74:
 * `h12.float().chunk(2)`, `F.silu(h1) * h2`, `.to(dtype)`) fused with the quantisation of the second GEMM's input.
 * h12: (T, 2*I), contiguous.  q: (T, I) bytes.  scales: (T, ceil(I/128)).  I must be a multiple of 8. */
int cinn_swiglu_quant_rowwise(const void* h12, int dtype, int64_t T, int64_t I, void* q, float* scales, int div_mode,
                              void* stream);

/* The same for a buffer of which only the first n_rows_dev[0] rows (a count in DEVICE memory, at most T) hold data:
 * the rows an expert-parallel rank received in this step, known on the device only.  Rows past the count are
 * neither read nor written. */
int cinn_swiglu_quant_rowwise_n(const void* h12, int dtype, int64_t T, int64_t I, const int64_t* n_rows_dev, void* q,
                                float* scales, int div_mode, void* stream);

/* out (C, R) = in (R, C; row pitch ld_in) transposed, bytes.  Replaces the `.t().contiguous()` copies of
 * e4m3 operands (src/kernels.py:748). */
int cinn_transpose_bytes(const void* in, int64_t ld_in, void* out, int64_t R, int64_t C, void* stream);

/* Block-scaled FP8 GEMM:  C[M, N] = sum_kb (A[:, kb] * sA[:, kb]) @ (B[kb, :] * sB[kb, nb]).
 * Replaces fp8_gemm_kernel + fp8_matmul_dsv3 (src/kernels.py:588-664, 667-702).
 * A: (M, K) e4m3, K contiguous.  sA: (M, ceil(K/128)) fp32, row pitch ld_sa.
 * B: e4m3 in the layout named by b_layout.  sB: element (kb, nb) at sB[kb*sb_stride_k + nb*sb_stride_n].
 * C: (M, N) contiguous, out_dtype CINN_BF16 (what the reference returns), CINN_F16, CINN_F32 or CINN_F32_BF16.
 * K must be a multiple of 16; N a multiple of 8 for bf16 output, 4 for fp32 output. */
int cinn_fp8_gemm(const void* A, const float* sA, int64_t ld_sa, const void* B, const float* sB,
                  int64_t sb_stride_k, int64_t sb_stride_n, void* C, int64_t M, int64_t N, int64_t K,
                  int b_layout, int out_dtype, void* stream);

/* Grouped (per-expert) block-scaled FP8 GEMM over ragged row ranges:
 * for each expert e:  C[starts[e]:ends[e], :] = A[starts[e]:ends[e], :] @ W[e]^T.
 * Replaces grouped_gemm_kernel + moe_grouped_gemm (src/kernels.py:440-523, 526-581); the reference runs it in
 * fp16, here the operands are e4m3 with 1x128 / 128x128 scales like the dense GEMM.
 * A: (T, d_in) e4m3.  sA: (T, ceil(d_in/128)).  W: (E, d_out, d_in) e4m3.  sW: (E, ceil(d_out/128), ceil(d_in/128)).
 * starts/ends: int64 device arrays of length E, read on the device (no host synchronisation, no padding).
 * C: (T, d_out).  Rows that belong to no expert are left untouched. */
int cinn_fp8_grouped_gemm(const void* A, const float* sA, const void* W, const float* sW,
                          const int64_t* starts, const int64_t* ends, int64_t E, int64_t T, int64_t d_in,
                          int64_t d_out, void* C, int out_dtype, void* stream);

/* The grouped GEMM in the reference's own precision: A (total_rows, d_in) and W (n_experts, d_out, d_in) both bf16 or
 * both fp16 (in_dtype), fp32 accumulation on the tensor cores (tcgen05 kind::f16), C (total_rows, d_out) of out_dtype.
 * Replaces grouped_gemm_kernel + moe_grouped_gemm (src/kernels.py:440-581) without the change of numerics that the
 * e4m3 entry point above makes: same ragged device-side row ranges, no padding, rows outside every range untouched.
 * d_in a multiple of 8, at most 384 experts, 16-byte aligned buffers. */
int cinn_grouped_gemm_16bit(const void* A, const void* W, int in_dtype, const int64_t* expert_starts, const int64_t* expert_ends,
                            int64_t n_experts, int64_t total_rows, int64_t d_in, int64_t d_out, void* C, int out_dtype,
                            void* stream);

/* Input gradient of the grouped GEMM:  dX[starts[e]:ends[e], :] = dY[starts[e]:ends[e], :] @ W[e].
 * No counterpart in the reference: its moe_grouped_gemm is not differentiable (src/kernels.py:526-581 is a plain
 * function), so routed experts receive no gradient there; the arithmetic mirrors the dense dgrad
 * (src/kernels.py:771-774).  dY: (T, d_out) e4m3 with scales (T, ceil(d_out/128)); W, sW as in
 * cinn_fp8_grouped_gemm (the weight bytes are read as stored, never transposed); dX: (T, d_in). */
int cinn_fp8_grouped_gemm_dgrad(const void* dY, const float* sdY, const void* W, const float* sW, const int64_t* starts,
                                const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* dX,
                                int out_dtype, void* stream);

/* Weight gradient of the grouped GEMM: dW[e] = dY[starts[e]:ends[e]]^T @ X[starts[e]:ends[e]] for every expert,
 * with the operands quantised expert by expert as FP8MatmulFunction.backward does for one Linear
 * (src/kernels.py:780-788: dY^T in 1 x 128 tiles along the tokens, the saved row-quantised x re-quantised in
 * 128 x 128 blocks; token counts padded with zero rows to a multiple of 16).  The reference's grouped GEMM has no
 * backward (src/kernels.py:526-581).
 * dY: (T, d_out) of dy_dtype; x_q (T, d_in) e4m3 with x_scales (T, ceil(d_in/128)) as the forward saved them;
 * starts_host / ends_host: the E row ranges in HOST memory (the caller has read them back; every expert is a
 * GEMM problem of its own); dW: (E, d_out, d_in) of out_dtype (CINN_F32, CINN_F32_BF16 or CINN_BF16), experts
 * without rows are zeroed; scratch: device memory of at least
 * cinn_fp8_grouped_wgrad_scratch_bytes(largest expert's rows, d_in, d_out) bytes, reused expert after expert.
 * d_in and d_out multiples of 16. */
int64_t cinn_fp8_grouped_wgrad_scratch_bytes(int64_t max_rows, int64_t d_in, int64_t d_out);
int cinn_fp8_grouped_wgrad(const void* dY, int dy_dtype, const void* x_q, const float* x_scales, const int64_t* starts_host,
                           const int64_t* ends_host, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* scratch,
                           int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, void* stream);

/* The same weight gradients for all experts in four launches, with the row ranges read on the DEVICE
 * (expert_starts / expert_ends are device arrays here; no host read-back): the experts' segments are padded to whole
 * 128-row tiles on the device, dY^T and x are quantised per segment in one launch each, and one GEMM reduces every
 * expert over its own K blocks (tcgen05, two-SM tiles).  Same arithmetic as cinn_fp8_grouped_wgrad; an expert
 * without rows gets zeros.  d_in and d_out multiples of 256; scratch: cinn_fp8_grouped_wgrad_fused_scratch_bytes
 * bytes, 256-byte aligned.
 * dy_q_row (total_rows, d_out) e4m3 + dy_row_scales (total_rows, d_out / 128), both or neither (NULL): when given
 * (bf16 / fp16 dY), the pass that quantises dY^T also leaves the row-wise quantisation of dY there for the rows inside
 * expert ranges - the operand of cinn_fp8_grouped_gemm_dgrad - so that dY is read once for both gradients. */
int64_t cinn_fp8_grouped_wgrad_fused_scratch_bytes(int64_t total_rows, int64_t n_experts, int64_t d_in, int64_t d_out);
int cinn_fp8_grouped_wgrad_fused(const void* dY, int dy_dtype, const void* x_q, const float* x_scales, const int64_t* expert_starts,
                                 const int64_t* expert_ends, int64_t n_experts, int64_t total_rows, int64_t d_in, int64_t d_out,
                                 void* scratch, int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, void* dy_q_row,
                                 float* dy_row_scales, void* stream);

/* y[t, :] = sum_j gates[t, j] * rows[pos[t, j], :]  for t < n_tokens, j < top_k; fp32 result, no atomics.
 * Replaces the gate multiply, torch.zeros and scatter_add_ at the end of MoE.forward (src/layers.py:157-160).
 * rows: (n_rows, d) bf16 / fp16 / fp32.  pos: (n_tokens, top_k) int64 row indices (negative = skip), ascending per
 * token to reproduce the summation order of the reference.  gates: (n_tokens, top_k) fp32.  y: (n_tokens, d) fp32.
 * d must be a multiple of 8, top_k at most 32. */
int cinn_moe_combine(const void* rows, int dtype, const int64_t* pos, const float* gates, void* y, int64_t n_tokens,
                     int64_t n_rows, int top_k, int64_t d, void* stream);

/* The same with the shared experts' output folded in: y[t, :] = addend[t, :] + sum_j ...  (the
 * `shared_out + routed_out` of MoE.forward, src/layers.py:179).  addend: (n_tokens, d) bf16 / fp16 / fp32, or
 * NULL for the plain combine. */
int cinn_moe_combine_add(const void* rows, int dtype, const int64_t* pos, const float* gates, const void* addend,
                         int addend_dtype, void* y, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, void* stream);

/* Zero the rows of buf (n_rows x row_bytes) that no range [starts[r], ends[r]) covers (device-side int64 ranges,
 * clamped to the buffer).  The backward of the grouped GEMM uses it so that rows of no expert get a zero input
 * gradient without a fill of the whole buffer.  No reference counterpart (the reference's grouped GEMM,
 * src/kernels.py:526-581, has no backward). */
int cinn_zero_rows_outside(void* buf, int64_t n_rows, int64_t row_bytes, const int64_t* starts, const int64_t* ends,
                           int64_t n_ranges, void* stream);

/* Backward of cinn_moe_combine (the reference's gate multiply + scatter_add_, src/layers.py:157-160, is
 * differentiated by autograd there): d_rows[pos[t, j]] = gates[t, j] * dy[t] (type of rows; rows that no pair names
 * are left untouched) and d_gates[t, j] = < rows[pos[t, j]], dy[t] > (fp32; 0 for a skipped pair).  dy (T, d) fp32. */
int cinn_moe_combine_backward(const void* rows, int rows_dtype, const int64_t* pos, const float* gates, const float* dy,
                              void* d_rows, float* d_gates, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, void* stream);

/* Sparse attention over per-query index lists, forward.
 * Replaces sparse_attention_fwd_kernel + SparseAttentionFunction.forward (src/kernels.py:913-1052, 1194-1245).
 * q, k: (B, H, L, d_qk), v: (B, H, L, d_v) of `dtype`, contiguous; idx: (B, L, K) int64, shared by the heads.
 * Key idx[b, t, j] takes part in query t when 0 <= idx <= t.  out: (B, H, L, d_v) fp32; lse: (B, H, L) fp32;
 * attn_weights: (B, H, L, K) fp32 probabilities (0 for keys that do not take part; a query without any valid
 * key gets all-zero weights, zero output and lse 0). */
int cinn_sparse_attn_fwd(const void* q, const void* k, const void* v, int dtype, const int64_t* idx, float* out, float* lse,
                         float* attn_weights, int64_t B, int64_t H, int64_t L, int64_t K, int64_t d_qk, int64_t d_v,
                         float scale, void* stream);

/* Backward of the above.  Replaces sparse_attention_bwd_kernel + SparseAttentionFunction.backward
 * (src/kernels.py:1055-1186, 1247-1289).  grad_out: (B, H, L, d_v) of `grad_dtype` (the inputs' type or fp32);
 * out, lse: as saved by the forward.  grad_q is written; grad_k and grad_v (fp32, same shapes as k and v) are
 * ACCUMULATED into with fp32 atomics, so the caller zeroes them first, as the reference does (:1257-1259). */
int cinn_sparse_attn_bwd(const void* grad_out, int grad_dtype, const float* out, const float* lse, const void* q,
                         const void* k, const void* v, int dtype, const int64_t* idx, float* grad_q, float* grad_k,
                         float* grad_v, int64_t B, int64_t H, int64_t L, int64_t K, int64_t d_qk, int64_t d_v, float scale,
                         void* stream);


/* Lightning indexer logits: out[b, t, s] = sum_h relu(q[b, t, h, :] . k[b, s, :]) * w[b, t, h], fp16.
 * Replaces lightning_indexer_kernel + lightning_indexer_fused (src/kernels.py:321-433): dot-product operands
 * rounded to fp16, fp32 accumulation, ReLU and head weights in fp32.  q: (B, Lq, H, d), k: (B, Lk, d),
 * w: (B, Lq, H) of `dtype`, with element strides q_strides[4], k_strides[3], w_strides[3] (HOST arrays, as the
 * reference passes .stride(), :419-421); out: (B, Lq, Lk) fp16, contiguous. */
int cinn_lightning_indexer(const void* q, const void* k, const void* w, int dtype, void* out, int64_t B, int64_t Lq,
                           int64_t Lk, int64_t H, int64_t d, const int64_t* q_strides, const int64_t* k_strides,
                           const int64_t* w_strides, void* stream);

/* SwiGLU between the two expert GEMMs, unquantised (the training path; cinn_swiglu_quant_rowwise is the
 * inference path): h (T, I) = silu(h12[:, :I]) * h12[:, I:], fp32 arithmetic, rounded to `dtype`
 * (src/layers.py:71-74), and its backward grad_h12 (T, 2I) from grad_h (T, I).  I a multiple of 8. */
int cinn_swiglu(const void* h12, void* h, int dtype, int64_t T, int64_t I, void* stream);
int cinn_swiglu_backward(const void* h12, const void* grad_h, void* grad_h12, int dtype, int64_t T, int64_t I, void* stream);

/* Dispatch gather of quantised tokens: out_q[r, :] = q[idx[r], :], out_scales[r, :] = scales[idx[r], :] for
 * r < n_out, in one pass (the `flat_x[token_indices]` of MoE.forward, src/layers.py:140, on tokens that were
 * quantised once before the gather).  q: (n_src, d) e4m3 bytes, d a multiple of 16; scales: (n_src, n_scales)
 * fp32; idx: (n_out) int64, entries outside [0, n_src) leave their output row untouched. */
int cinn_gather_rows(const void* q, const float* scales, const int64_t* idx, void* out_q, float* out_scales, int64_t n_out,
                     int64_t n_src, int64_t d, int64_t n_scales, void* stream);

/* Row scatter: out[idx[r], :] = in[r, :] for r < n_rows; rows of row_bytes bytes (a multiple of 16), out has
 * n_dst rows, entries of idx outside [0, n_dst) are skipped.  Brings the expert outputs of an expert-parallel
 * rank from the expert-grouped order back to the order in which the rows arrived, before they travel home
 * (the reference keeps every expert on every rank, src/layers.py:89-179, and has no such step). */
int cinn_scatter_rows(const void* in, const int64_t* idx, void* out, int64_t n_rows, int64_t n_dst, int64_t row_bytes,
                      void* stream);

/* Expert-parallel dispatch by peer stores (no reference counterpart: the reference keeps every expert on every
 * rank, src/layers.py:89-179).  Pair r of this rank, r < n_pairs (sorted by expert: sorted_experts[r], source token
 * token_indices[r]), is copied - e4m3 row of q (n_tokens, d) and its n_scales fp32 scales - into the receive
 * buffers of the rank that owns its expert, at row base_send[e] + (r - my_start[e]).  peer_q / peer_scales:
 * DEVICE arrays of n_ranks base addresses (as int64) of the ranks' receive buffers, which must be mapped into
 * this process (symmetric memory / CUDA IPC); capacity_rows: rows each of them holds.  base_send, my_start:
 * (experts_per_rank * n_ranks) int64 device arrays (cinnamon_b200/p2p.py builds them from the all-gathered
 * counts).  Table entries that point outside the buffers skip the row and set the device status word.
 * The caller orders the exchange: a barrier over the ranks before (the buffers are free) and after (all rows
 * have landed). */
int cinn_p2p_dispatch(const void* q, const float* scales, const int64_t* token_indices, const int64_t* sorted_experts,
                      const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_scales,
                      int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t n_scales, int experts_per_rank, int n_ranks,
                      int64_t capacity_rows, void* stream);

/* The way home by peer stores: row r < n_rows of this rank's expert-grouped outputs (row_bytes each, a multiple of
 * 16) belongs to segment i = (local expert, source rank) with seg_start[i] <= r < seg_start[i + 1] and is copied
 * to rank i % n_ranks at row home_base[i] + (r - seg_start[i]) of its buffer peer_home[rank] (capacity_rows
 * rows): the position of the pair in that rank's sorted order, which is what cinn_moe_combine reads.
 * seg_start: (n_segments + 1), home_base: (n_segments) int64 device arrays. */
int cinn_p2p_return(const void* rows, const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home,
                    int64_t n_rows, int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity_rows, void* stream);

/* cinn_fp8_grouped_gemm whose finished output rows go to arbitrary addresses: row r of the result is stored at
 * the BYTE address row_dst[r] (device array, T entries; 0 = drop the row) instead of C + r * d_out.  The addresses
 * may lie in another GPU's memory that is mapped into this process: with the table of cinn_p2p_row_table the
 * down-projection of an expert-parallel rank writes every expert output straight to the rank its token lives on,
 * under the GEMM rather than after it.  out_dtype CINN_BF16 or CINN_F16, d_out a multiple of 8, every address
 * 16-byte aligned.  No reference counterpart. */
int cinn_fp8_grouped_gemm_scatter(const void* A, const float* sA, const void* W, const float* sW, const int64_t* starts,
                                  const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out,
                                  const int64_t* row_dst, int out_dtype, void* stream);

/* The destinations of cinn_p2p_return as a table: row_dst[r] = peer_home[rank] + row * row_bytes for r < n_rows;
 * 0 for rows at or past seg_start[n_segments] (n_rows may be the buffer's capacity when the true row count is
 * known on the device only), 0 and a status code where the tables point outside the buffers. */
int cinn_p2p_row_table(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
                       int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity_rows, int64_t* row_dst, void* stream);

/* Stream-ordered barrier over the ranks of one node for the peer-store exchange (no reference counterpart).
 * peer_flags: DEVICE array of n_ranks base addresses of the ranks' flag arrays (n_ranks uint32 each, zeroed once,
 * in symmetric memory); epoch: 1, 2, 3, ... the same sequence on every rank.  Work enqueued before the barrier on
 * every rank's stream is complete (and its peer stores visible) before work enqueued after it starts.  The wait is
 * bounded (about 2 s): a rank that never arrives leaves a code in the device status word instead of a hung GPU.
 * Every rank must run on a GPU of its own. */
int cinn_p2p_barrier(const int64_t* peer_flags, int rank, int n_ranks, unsigned epoch, void* stream);

/* Limit, in SM clock cycles, of the bounded wait in cinn_p2p_barrier (default 4e9, about two seconds; cycles <= 0
 * restores the default).  Returns the previous limit.  Applies to barriers launched afterwards.  When a wait runs
 * out the barrier kernel returns, cinn_device_status reports (5 << 8) | 3, and whatever the layer computed after
 * that barrier is invalid (rows may not have arrived): the caller discards the step.  No reference counterpart
 * (the reference has no device-side waits). */
long long cinn_set_wait_limit_cycles(long long cycles);

/* The exchange plan of an expert-parallel layer call in one launch (no reference counterpart: the reference keeps
 * every expert on every rank, src/layers.py:89-179).  my_counts (n_experts int64, device): pairs this rank routed
 * to every global expert.  peer_counts: DEVICE array of n_ranks base addresses of the ranks' (n_ranks, n_experts)
 * int64 count matrices in symmetric memory; peer_flags as in cinn_p2p_barrier, flag slots
 * [flag_slot, flag_slot + n_ranks) are used with `epoch` (1, 2, 3, ... the same on every rank).  The kernel writes
 * this rank's counts into row `rank` of every matrix, flags it, waits (bounded, code (5 << 8) | 5 on expiry) for
 * the rows of all ranks, and derives the address tables of the exchange:
 *   base_send, my_start (n_experts); starts, ends (n_experts / n_ranks); seg_start (n_experts / n_ranks * n_ranks + 1);
 *   home_base (n_experts / n_ranks * n_ranks); total_rows (1)   - all int64, device.
 * Every rank must run on a GPU of its own.  Passing this kernel also means every rank has finished what it had
 * enqueued before it, so the receive buffers of the previous layer call are free. */
int cinn_p2p_plan(const int64_t* my_counts, const int64_t* peer_counts, const int64_t* peer_flags, int rank, int n_ranks,
                  int n_experts, int flag_slot, unsigned epoch, int64_t* base_send, int64_t* my_start, int64_t* starts,
                  int64_t* ends, int64_t* seg_start, int64_t* home_base, int64_t* total_rows, void* stream);

/* cinn_p2p_dispatch for the pairs of the local experts [expert_lo, expert_hi) of every rank (0 and experts_per_rank:
 * all pairs), whose last CTA flags "these rows have landed" to every rank (slot flag_slot + rank, value epoch).
 * Destinations are served in the order rank + 1, rank + 2, ..., rank, so that the ranks write to different peers at
 * any moment.  Several calls with disjoint expert ranges and different flag slots let the owner start on the experts
 * of one range while the rows of the next are still on their way.  done_counter: one zeroed uint32 in device memory,
 * left zero.  Pairs with cinn_p2p_row_table_wait.  my_start must hold n_experts entries (cinn_p2p_plan's).
 * n_sms: 0 = CTAs on every SM; > 0 = one large CTA on each of that many SMs, so that a persistent GEMM enqueued on
 * another stream (capped with cinn_set_gemm_sm_limit to the remaining SMs) runs beside the stores. */
int cinn_p2p_dispatch_signal(const void* q, const float* s, const int64_t* token_indices, const int64_t* sorted_experts,
                             const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_s,
                             int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t n_scales, int experts_per_rank, int n_ranks,
                             int64_t capacity_rows, const int64_t* peer_flags, int rank, int flag_slot, unsigned epoch,
                             unsigned* done_counter, int expert_lo, int expert_hi, int n_sms, void* stream);

/* cinn_p2p_row_table that first waits (bounded, code (5 << 8) | 6 on expiry) for the flags of cinn_p2p_dispatch_signal
 * from all ranks: work enqueued after it sees every row dispatched under that flag slot.  With n_rows = 0 it only
 * waits. */
int cinn_p2p_row_table_wait(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
                            int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity_rows, int64_t* row_dst,
                            const int64_t* peer_flags, int rank, int flag_slot, unsigned epoch, void* stream);

/* Routing of MoE.forward (src/layers.py:122-148) on the device: scores = sigmoid(logits), the top_k experts of
 * scores + bias per token (ties: the lower expert id), gates = score / (sum of the k scores + 1e-9), and the
 * (token, expert) pairs sorted by expert in the order of a stable sort.
 *   logits (n_tokens, n_experts) fp32: the router's output; bias (n_experts) fp32.
 *   workspace: cinn_moe_route_workspace_ints(n_tokens, n_experts) ints of device memory, contents irrelevant.
 *   top_experts / top_gates (n_tokens, top_k): the selection in descending order of score + bias.
 *   token_indices / sorted_scores / sorted_experts (n_tokens * top_k): source token, gate and expert of every row
 *   of the sorted order (`sort_order // top_k`, `expanded_scores[sort_order]`, `sorted_idx`, :135-142).
 *   counts (n_experts) int64: rows per expert (`torch.bincount`, :145).
 *   pair_pos / pair_gate (n_tokens, top_k): per token its rows in ascending order with their gates: the input of
 *   cinn_moe_combine.
 * n_experts <= 1024, top_k <= min(32, n_experts), n_tokens * top_k < 2^31.  No host synchronisation. */
int64_t cinn_moe_route_workspace_ints(int64_t n_tokens, int n_experts);
int cinn_moe_route(const float* logits, const float* bias, int64_t n_tokens, int n_experts, int top_k, int* workspace,
                   int* top_experts, float* top_gates, int64_t* token_indices, float* sorted_scores,
                   int64_t* sorted_experts, int64_t* counts, int64_t* pair_pos, float* pair_gate, void* stream);

/* cinn_moe_route for callers that have no device memory to give as a workspace and may not allocate any: a
 * serving process that handed all of HBM to its own arena at start-up, a job running at the memory limit, a
 * latency-bound loop that cannot afford the device-wide synchronisation an allocation can imply.  This entry
 * point has no counterpart in the reference; it is an addition of this library.
 * The scratch is a fixed 2 MiB array inside the library (every GPU that loads the library holds it until the
 * process exits); inputs and outputs are still the caller's.  It allocates and frees nothing.
 *   - Limit: cinn_moe_route_workspace_ints(n_tokens, n_experts) <= cinn_moe_route_static_max_ints() (524288),
 *     e.g. 262016 tokens at 256 experts; larger problems are refused with CINN_ERR_INVALID and a message.
 *   - The first call on each device looks up the array's device address (with that device current); make that
 *     first call before any stream capture begins.
 *   - All calls on one device share the array: calls that overlap on the GPU race, so keep them on one stream
 *     (or otherwise ordered).  Nothing needs clearing between calls; the kernels overwrite what they read.
 * Arguments and results are exactly those of cinn_moe_route, without `workspace`. */
int64_t cinn_moe_route_static_max_ints(void);
int cinn_moe_route_static(const float* logits, const float* bias, int64_t n_tokens, int n_experts, int top_k,
                          int* top_experts, float* top_gates, int64_t* token_indices, float* sorted_scores,
                          int64_t* sorted_experts, int64_t* counts, int64_t* pair_pos, float* pair_gate, void* stream);

/* Caps the number of SMs the persistent GEMM kernels (cinn_fp8_gemm, cinn_fp8_grouped_gemm*) occupy from now
 * on, process-wide; 0 = all of them (the default).  Returns the previous cap.  For callers that run other
 * kernels beside a GEMM on another stream, e.g. the send/receive kernels of an all-to-all, which otherwise wait
 * until a GEMM has let go of an SM.  No reference counterpart (the reference's kernels are not persistent). */
int cinn_set_gemm_sm_limit(int n_sms);

/* Reads (and with reset != 0 clears) the device-side status word of the current device into the HOST int
 * *out.  0 means no kernel of this library has given up on a bounded wait since the last reset; any other
 * value is (role << 8) | reason.  This call synchronises with the device.  No counterpart in the reference,
 * whose kernels have no waits. */
int cinn_device_status(int* out, int reset);

#ifdef __cplusplus
}
#endif
#endif
