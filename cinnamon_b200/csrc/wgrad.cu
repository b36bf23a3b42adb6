// Weight gradient of the grouped (per-expert) GEMM: dW[e] = dY[rows of e]^T @ X[rows of e], with the operands
// quantised as FP8MatmulFunction.backward quantises them (src/kernels.py:780-788), expert by expert:
// dY^T in 1 x 128 tiles along the expert's tokens, x (already row-quantised by the forward) de-quantised and
// re-quantised in 128 x 128 blocks, both zero-padded to a multiple of 16 tokens.  The reference's grouped GEMM has
// no backward at all (src/kernels.py:526-581).
//
// The experts' row ranges are ragged, so each expert is its own GEMM problem; what this file removes is the host
// cost of walking them from Python: one call enqueues three launches per non-empty expert (transposing quantiser,
// re-quantiser, dense GEMM straight into the expert's slice of dW) from a plain loop, reusing one caller-provided
// scratch buffer (the launches of one stream run in order, so the next expert may overwrite it).
#include "common.cuh"

namespace cinn {

int quantize_transposed_padded(const void* x, int dtype, int64_t M, int64_t N_in, int64_t N, int64_t L, void* q,
                               float* scales, int div_mode, cudaStream_t st);
int requant_row_to_block_padded(const void* xq, const float* xs, int64_t M_in, int64_t M, int64_t K, void* out, float* scales,
                                int div_mode, cudaStream_t st);
int fp8_gemm(const void* A, const float* sA, int64_t ld_sa, const void* B, const float* sB, int64_t sbk, int64_t sbn,
             void* C, int64_t M, int64_t N, int64_t K, int b_layout, int out_dtype, cudaStream_t st);

static inline int64_t up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// bytes of scratch one expert with n_pad (a multiple of 16) rows needs
static int64_t wgrad_scratch_for(int64_t n_pad, int64_t d_in, int64_t d_out) {
    const int64_t nt = (n_pad + 127) / 128, nkb = (d_in + 127) / 128;
    return up(d_out * n_pad, 256) + up(d_out * nt * 4, 256) + up(n_pad * d_in, 256) + up(nt * nkb * 4, 256);
}

int64_t grouped_wgrad_scratch_bytes(int64_t max_rows, int64_t d_in, int64_t d_out) {
    return wgrad_scratch_for(up(max_rows < 0 ? 0 : max_rows, 16), d_in, d_out);
}

int fp8_grouped_wgrad(const void* dY, int dy_dtype, const void* x_q, const float* x_s, const int64_t* starts_host,
                      const int64_t* ends_host, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* scratch,
                      int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(E >= 0 && T >= 0 && d_in > 0 && d_out > 0, "grouped_wgrad: bad shape");
    if (E == 0) return CINN_OK;
    CINN_CHECK_ARG(starts_host && ends_host && dW, "grouped_wgrad: null pointer");
    CINN_CHECK_ARG(d_in % 16 == 0 && d_out % 16 == 0, "grouped_wgrad: d_in (%lld) and d_out (%lld) must be multiples of 16",
                   (long long)d_in, (long long)d_out);
    CINN_CHECK_ARG(out_dtype == CINN_F32 || out_dtype == CINN_F32_BF16 || out_dtype == CINN_BF16,
                   "grouped_wgrad: the gradient is fp32 (optionally holding bf16-rounded values) or bf16");
    CINN_CHECK_ARG(dy_dtype == CINN_BF16 || dy_dtype == CINN_F16 || dy_dtype == CINN_F32, "grouped_wgrad: unknown dtype tag %d", dy_dtype);
    const int64_t dy_size = dy_dtype == CINN_F32 ? 4 : 2, w_size = out_dtype == CINN_BF16 ? 2 : 4;
    const int64_t nkb = (d_in + 127) / 128;
    for (int64_t e = 0; e < E; ++e) {
        int64_t s = starts_host[e], t = ends_host[e];
        if (s < 0) s = 0;
        if (t > T) t = T;
        uint8_t* dw_e = static_cast<uint8_t*>(dW) + e * d_out * d_in * w_size;
        const int64_t n = t - s;
        if (n <= 0) {                                            // an expert without tokens gets no gradient
            CINN_CHECK_CUDA(cudaMemsetAsync(dw_e, 0, (size_t)(d_out * d_in * w_size), st));
            continue;
        }
        CINN_CHECK_ARG(dY && x_q && x_s && scratch, "grouped_wgrad: null pointer");
        const int64_t n_pad = up(n, 16), nt = (n_pad + 127) / 128;
        CINN_CHECK_ARG(wgrad_scratch_for(n_pad, d_in, d_out) <= scratch_bytes,
                       "grouped_wgrad: expert %lld has %lld rows and needs %lld bytes of scratch, %lld were given",
                       (long long)e, (long long)n, (long long)wgrad_scratch_for(n_pad, d_in, d_out), (long long)scratch_bytes);
        uint8_t* base = static_cast<uint8_t*>(scratch);
        uint8_t* gt_q = base;
        float* gt_s = reinterpret_cast<float*>(gt_q + up(d_out * n_pad, 256));
        uint8_t* xb_q = reinterpret_cast<uint8_t*>(gt_s) + up(d_out * nt * 4, 256);
        float* xb_s = reinterpret_cast<float*>(xb_q + up(n_pad * d_in, 256));
        // dY[s:t]^T: logical (d_out, n) with element (m, j) at dY[(s + j) * d_out + m]
        int rc = quantize_transposed_padded(static_cast<const uint8_t*>(dY) + s * d_out * dy_size, dy_dtype, d_out, n, n_pad, d_out,
                                            gt_q, gt_s, div_mode, st);
        if (rc) return rc;
        rc = requant_row_to_block_padded(static_cast<const uint8_t*>(x_q) + s * d_in, x_s + s * nkb, n, n_pad, d_in, xb_q, xb_s,
                                         div_mode, st);
        if (rc) return rc;
        rc = fp8_gemm(gt_q, gt_s, nt, xb_q, xb_s, nkb, 1, dw_e, d_out, d_in, n_pad, 1 /* B stored (K, N) */, out_dtype, st);
        if (rc) return rc;
    }
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// The same gradients in four launches for all experts and without the host knowing the row ranges: the experts'
// segments are padded to whole 128-row tiles on the device (segment_tiles), dY^T and x are quantised per segment in
// one launch each, and one grouped-K GEMM reduces every expert over its own K blocks.  Same tiles, same bytes and
// the same sums as the per-expert loop above (zero padding changes neither an amax nor a product).
// Needs d_out and d_in multiples of 256; starts / ends are DEVICE arrays here.
// ---------------------------------------------------------------------------
int segment_tiles(const int64_t* starts, const int64_t* ends, int E, int64_t T, int* kb_start, int* tile_src, int* tile_cnt,
                  int max_tiles, cudaStream_t st);
int quantize_transposed_segmented(const void* x, int dtype, int64_t M, int64_t L, void* q, float* scales, int max_tiles,
                                  const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode, cudaStream_t st);
int quantize_dual_segmented(const void* x, int dtype, int64_t T, int64_t N, void* q_row, float* s_row, void* q_col, float* s_col,
                            int max_tiles, const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode,
                            cudaStream_t st);
int requant_row_to_block_segmented(const void* xq, const float* xs, int64_t K, void* out, float* scales, int max_tiles,
                                   const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode, cudaStream_t st);
int fp8_gemm_grouped_k(const void* A, const float* sA, const void* B, const float* sB, const int* kb_start, int64_t E,
                       int64_t M, int64_t N, int64_t max_tiles, void* C, int out_dtype, cudaStream_t st);

static inline int64_t fused_max_tiles(int64_t T, int64_t E) { return (T + 127) / 128 + E; }

int64_t grouped_wgrad_fused_scratch_bytes(int64_t T, int64_t E, int64_t d_in, int64_t d_out) {
    const int64_t mt = fused_max_tiles(T < 0 ? 0 : T, E < 0 ? 0 : E), nkb = (d_in + 127) / 128;
    return up((E + 1 + 2 * mt) * 4, 256) + up(d_out * mt * 128, 256) + up(d_out * mt * 4, 256) + up(d_in * mt * 128, 256) +
           up(mt * nkb * 4, 256);
}

int fp8_grouped_wgrad_fused(const void* dY, int dy_dtype, const void* x_q, const float* x_s, const int64_t* starts_dev,
                            const int64_t* ends_dev, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* scratch,
                            int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, void* dy_q_row, float* dy_s_row,
                            cudaStream_t st) {
    CINN_CHECK_ARG(E >= 1 && E <= 1024 && T >= 0 && d_in > 0 && d_out > 0, "grouped_wgrad_fused: bad shape");
    CINN_CHECK_ARG((dy_q_row == nullptr) == (dy_s_row == nullptr), "grouped_wgrad_fused: pass both row-wise outputs or neither");
    CINN_CHECK_ARG(dy_q_row == nullptr || dy_dtype == CINN_BF16 || dy_dtype == CINN_F16,
                   "grouped_wgrad_fused: the row-wise quantisation of dY comes with 2-byte gradients only");
    CINN_CHECK_ARG(d_in % 256 == 0 && d_out % 256 == 0, "grouped_wgrad_fused: d_in (%lld) and d_out (%lld) must be multiples of 256",
                   (long long)d_in, (long long)d_out);
    CINN_CHECK_ARG(dY && x_q && x_s && starts_dev && ends_dev && scratch && dW, "grouped_wgrad_fused: null pointer");
    CINN_CHECK_ARG(scratch_bytes >= grouped_wgrad_fused_scratch_bytes(T, E, d_in, d_out) && (reinterpret_cast<uintptr_t>(scratch) & 255) == 0,
                   "grouped_wgrad_fused: the scratch buffer must hold %lld bytes and be 256-byte aligned",
                   (long long)grouped_wgrad_fused_scratch_bytes(T, E, d_in, d_out));
    const int64_t mt = fused_max_tiles(T, E), nkb = (d_in + 127) / 128;
    uint8_t* base = static_cast<uint8_t*>(scratch);
    int* kb_start = reinterpret_cast<int*>(base);
    int* tile_src = kb_start + (E + 1);
    int* tile_cnt = tile_src + mt;
    uint8_t* a_q = base + up((E + 1 + 2 * mt) * 4, 256);
    float* a_s = reinterpret_cast<float*>(a_q + up(d_out * mt * 128, 256));
    uint8_t* b_q = reinterpret_cast<uint8_t*>(a_s) + up(d_out * mt * 4, 256);
    float* b_s = reinterpret_cast<float*>(b_q + up(d_in * mt * 128, 256));
    int rc = segment_tiles(starts_dev, ends_dev, (int)E, T, kb_start, tile_src, tile_cnt, (int)mt, st);
    if (rc) return rc;
    if (dy_q_row != nullptr)
        // both quantisations of dY in one pass: the caller's grouped input gradient reads the row-wise one
        rc = quantize_dual_segmented(dY, dy_dtype, T, d_out, dy_q_row, dy_s_row, a_q, a_s, (int)mt, tile_src, tile_cnt, kb_start + E,
                                     div_mode, st);
    else
        rc = quantize_transposed_segmented(dY, dy_dtype, d_out, d_out, a_q, a_s, (int)mt, tile_src, tile_cnt, kb_start + E, div_mode, st);
    if (rc) return rc;
    rc = requant_row_to_block_segmented(x_q, x_s, d_in, b_q, b_s, (int)mt, tile_src, tile_cnt, kb_start + E, div_mode, st);
    if (rc) return rc;
    return fp8_gemm_grouped_k(a_q, a_s, b_q, b_s, kb_start, E, d_out, d_in, mt, dW, out_dtype, st);
}

}  // namespace cinn
