// extern "C" surface of the library: argument marshalling only.
#include "common.cuh"
#include "../../include/cinnamon_b200.h"
#include <mutex>

namespace cinn {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int quantize(bool blockwise, const void* x, int dtype, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, void* q,
             float* scales, int bm, int bn, int round_scale, int div_mode, cudaStream_t st);
int quantize_dual(const void* x, int dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row, void* q_col,
                  float* s_col, int round_scale, int div_mode, cudaStream_t st);
int selfcheck_division(unsigned long long* mismatches, cudaStream_t st);
int requant_row_to_block(const void* xq, const float* xs, int64_t M, int64_t K, void* out, float* scales,
                         int transpose_out, int div_mode, cudaStream_t st);
int dequantize(const void* q, const float* scales, void* out, int out_dtype, int64_t M, int64_t N, int bm, int bn,
               cudaStream_t st);
int transpose_bytes(const void* in, int64_t ld_in, void* out, int64_t R, int64_t C, cudaStream_t st);
int swiglu_quant_rowwise(const void* h12, int dtype, int64_t T_rows, int64_t I, void* q, float* scales, int div_mode,
                         cudaStream_t st, const int64_t* n_rows_dev);
int fp8_gemm(const void* A, const float* sA, int64_t ld_sa, const void* B, const float* sB, int64_t sbk, int64_t sbn,
             void* C, int64_t M, int64_t N, int64_t K, int b_layout, int out_dtype, cudaStream_t st);
int fp8_grouped_gemm(const void* A, const float* sA, const void* W, const float* sW, const int64_t* starts,
                     const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* C, int out_dtype,
                     cudaStream_t st, const long long* row_dst);
int p2p_row_table(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows, int64_t row_bytes,
                  int n_segments, int n_ranks, int64_t capacity, long long* row_dst, cudaStream_t st);   // rows past seg_start[n_segments] get 0

int read_device_status(int* out, int reset);
int fp8_grouped_gemm_dgrad(const void* dY, const float* sdY, const void* W, const float* sW, const int64_t* starts,
                           const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* dX, int out_dtype,
                           cudaStream_t st);
int gather_rows(const void* q, const float* s, const int64_t* idx, void* out_q, float* out_s, int64_t n_out, int64_t n_src,
                int64_t d, int64_t ns, cudaStream_t st);
int sparse_attn_fwd(const void* q, const void* k, const void* v, int dtype, const int64_t* idx, float* out, float* lse,
                    float* attn_w, int64_t B, int64_t H, int64_t L, int64_t K, int64_t Dqk, int64_t Dv, float scale,
                    cudaStream_t st);
int sparse_attn_bwd(const void* d_out, int grad_dtype, const float* out, const float* lse, const void* q, const void* k,
                    const void* v, int dtype, const int64_t* idx, float* dq, float* dk, float* dv, int64_t B, int64_t H,
                    int64_t L, int64_t K, int64_t Dqk, int64_t Dv, float scale, cudaStream_t st);
int lightning_indexer(const void* q, const void* k, const void* w, int dtype, void* out, int64_t B, int64_t Lq, int64_t Lk,
                      int64_t H, int64_t d, const int64_t* q_strides, const int64_t* k_strides, const int64_t* w_strides,
                      cudaStream_t st);
int scatter_rows(const void* in, const int64_t* idx, void* out, int64_t n_rows, int64_t n_dst, int64_t row_bytes,
                 cudaStream_t st);
int set_gemm_sm_limit(int n);
int p2p_dispatch(const void* q, const float* s, const int64_t* token_indices, const int64_t* sorted_experts,
                 const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_s,
                 int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t ns, int e_local, int n_ranks, int64_t capacity,
                 cudaStream_t st);
int p2p_return(const void* rows, const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
               int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity, cudaStream_t st);
int p2p_barrier(const int64_t* peer_flags, int me, int n_ranks, unsigned epoch, cudaStream_t st);
long long set_p2p_wait_limit(long long cycles);
int64_t grouped_wgrad_fused_scratch_bytes(int64_t T, int64_t E, int64_t d_in, int64_t d_out);
int fp8_grouped_wgrad_fused(const void* dY, int dy_dtype, const void* x_q, const float* x_s, const int64_t* starts_dev,
                            const int64_t* ends_dev, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* scratch,
                            int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, void* dy_q_row, float* dy_s_row,
                            cudaStream_t st);
int grouped_gemm_16bit(const void* A, const void* W, int in_dtype, const int64_t* starts, const int64_t* ends, int64_t E,
                       int64_t T, int64_t d_in, int64_t d_out, void* C, int out_dtype, cudaStream_t st);
int zero_rows_outside(void* buf, int64_t T, int64_t row_bytes, const int64_t* starts, const int64_t* ends, int64_t E,
                      cudaStream_t st);
int moe_combine_backward(const void* rows, int dtype, const int64_t* pos, const float* gates, const float* dy, void* d_rows,
                         float* d_gates, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, cudaStream_t st);
int p2p_plan(const int64_t* my_counts, const int64_t* peer_counts, const int64_t* peer_flags, int me, int G, int E,
             int flag_slot, unsigned epoch, int64_t* base_send, int64_t* my_start, int64_t* starts, int64_t* ends,
             int64_t* seg_start, int64_t* home_base, int64_t* total_rows, cudaStream_t st);
int p2p_dispatch_signal(const void* q, const float* s, const int64_t* token_indices, const int64_t* sorted_experts,
                        const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_s,
                        int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t ns, int e_local, int n_ranks, int64_t capacity,
                        const int64_t* peer_flags, int me, int flag_slot, unsigned epoch, unsigned* done, int e_lo, int e_hi,
                        int n_sms, cudaStream_t st);
int p2p_row_table_wait(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
                       int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity, long long* row_dst,
                       const int64_t* peer_flags, int me, int flag_slot, unsigned epoch, cudaStream_t st);
int64_t grouped_wgrad_scratch_bytes(int64_t max_rows, int64_t d_in, int64_t d_out);
int fp8_grouped_wgrad(const void* dY, int dy_dtype, const void* x_q, const float* x_s, const int64_t* starts_host,
                      const int64_t* ends_host, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* scratch,
                      int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, cudaStream_t st);
int quantize_row_block(const void* x, int dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row, void* q_blk,
                       float* s_blk, int round_scale, int div_mode, cudaStream_t st, int transpose_block);
int quantize_block_t(const void* x, int dtype, int64_t M, int64_t N, int64_t ld, void* q, void* q_t, float* scales,
                     int round_scale, int div_mode, cudaStream_t st);
int swiglu(const void* h12, const void* dh, void* out, int dtype, int64_t T_rows, int64_t I, int backward, cudaStream_t st);
int64_t moe_route_workspace_ints(int64_t T, int E);
int moe_route(const float* logits, const float* bias, int64_t T, int E, int top_k, int* workspace, int* top_experts,
              float* top_gates, int64_t* token_indices, float* sorted_scores, int64_t* sorted_experts, int64_t* counts,
              int64_t* pair_pos, float* pair_gate, cudaStream_t st);
int64_t moe_route_static_max_ints();
int moe_route_static(const float* logits, const float* bias, int64_t T, int E, int top_k, int* top_experts, float* top_gates,
                     int64_t* token_indices, float* sorted_scores, int64_t* sorted_experts, int64_t* counts,
                     int64_t* pair_pos, float* pair_gate, cudaStream_t st);
int moe_combine(const void* rows, int dtype, const int64_t* pos, const float* gates, const void* addend, int addend_dtype,
                void* y, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, cudaStream_t st);

}  // namespace cinn

extern "C" {

int cinn_version(void) { return 100; }

const char* cinn_last_error(void) { return cinn::g_err; }

int cinn_quant_rowwise(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, void* q,
                       float* scales, int block_size, int round_scale, int div_mode, void* stream) {
    return cinn::quantize(false, x, x_dtype, M, N, ld_m, ld_n, q, scales, 1, block_size, round_scale, div_mode,
                          (cudaStream_t)stream);
}

int cinn_quant_blockwise(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, void* q,
                         float* scales, int block_m, int block_n, int round_scale, int div_mode, void* stream) {
    return cinn::quantize(true, x, x_dtype, M, N, ld_m, ld_n, q, scales, block_m, block_n, round_scale, div_mode,
                          (cudaStream_t)stream);
}

int cinn_quant_blockwise_t(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q, void* q_t, float* scales,
                           int round_scale, int div_mode, void* stream) {
    return cinn::quantize_block_t(x, x_dtype, M, N, ld, q, q_t, scales, round_scale, div_mode, (cudaStream_t)stream);
}

int cinn_quant_rowwise_dual(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row,
                            void* q_col, float* s_col, int round_scale, int div_mode, void* stream) {
    return cinn::quantize_dual(x, x_dtype, M, N, ld, q_row, s_row, q_col, s_col, round_scale, div_mode, (cudaStream_t)stream);
}

int cinn_selfcheck_division(unsigned long long* mismatches, void* stream) {
    return cinn::selfcheck_division(mismatches, (cudaStream_t)stream);
}

int cinn_quant_rowwise_with_block(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row,
                                  void* q_block, float* s_block, int round_scale, int div_mode, void* stream) {
    return cinn::quantize_row_block(x, x_dtype, M, N, ld, q_row, s_row, q_block, s_block, round_scale, div_mode,
                                    (cudaStream_t)stream, 0);
}

int cinn_quant_rowwise_with_block_t(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row,
                                    void* q_block_t, float* s_block, int round_scale, int div_mode, void* stream) {
    return cinn::quantize_row_block(x, x_dtype, M, N, ld, q_row, s_row, q_block_t, s_block, round_scale, div_mode,
                                    (cudaStream_t)stream, 1);
}

int cinn_requant_row_to_block(const void* xq, const float* xs, int64_t M, int64_t K, void* out, float* scales,
                              int transpose_out, int div_mode, void* stream) {
    return cinn::requant_row_to_block(xq, xs, M, K, out, scales, transpose_out, div_mode, (cudaStream_t)stream);
}

int cinn_dequant(const void* q, const float* scales, void* out, int out_dtype, int64_t M, int64_t N, int block_m,
                 int block_n, void* stream) {
    return cinn::dequantize(q, scales, out, out_dtype, M, N, block_m, block_n, (cudaStream_t)stream);
}

int cinn_swiglu_quant_rowwise(const void* h12, int dtype, int64_t T, int64_t I, void* q, float* scales, int div_mode,
                              void* stream) {
    return cinn::swiglu_quant_rowwise(h12, dtype, T, I, q, scales, div_mode, (cudaStream_t)stream, nullptr);
}

int cinn_swiglu_quant_rowwise_n(const void* h12, int dtype, int64_t T, int64_t I, const int64_t* n_rows_dev, void* q,
                                float* scales, int div_mode, void* stream) {
    return cinn::swiglu_quant_rowwise(h12, dtype, T, I, q, scales, div_mode, (cudaStream_t)stream, n_rows_dev);
}

int cinn_transpose_bytes(const void* in, int64_t ld_in, void* out, int64_t R, int64_t C, void* stream) {
    return cinn::transpose_bytes(in, ld_in, out, R, C, (cudaStream_t)stream);
}

int cinn_fp8_gemm(const void* A, const float* sA, int64_t ld_sa, const void* B, const float* sB, int64_t sb_stride_k,
                  int64_t sb_stride_n, void* C, int64_t M, int64_t N, int64_t K, int b_layout, int out_dtype,
                  void* stream) {
    return cinn::fp8_gemm(A, sA, ld_sa, B, sB, sb_stride_k, sb_stride_n, C, M, N, K, b_layout, out_dtype,
                          (cudaStream_t)stream);
}

int cinn_fp8_grouped_gemm(const void* A, const float* sA, const void* W, const float* sW, const int64_t* starts,
                          const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* C,
                          int out_dtype, void* stream) {
    return cinn::fp8_grouped_gemm(A, sA, W, sW, starts, ends, E, T, d_in, d_out, C, out_dtype, (cudaStream_t)stream, nullptr);
}

int cinn_fp8_grouped_gemm_dgrad(const void* dY, const float* sdY, const void* W, const float* sW, const int64_t* starts,
                                const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* dX,
                                int out_dtype, void* stream) {
    return cinn::fp8_grouped_gemm_dgrad(dY, sdY, W, sW, starts, ends, E, T, d_in, d_out, dX, out_dtype, (cudaStream_t)stream);
}

int cinn_moe_combine(const void* rows, int dtype, const int64_t* pos, const float* gates, void* y, int64_t n_tokens,
                     int64_t n_rows, int top_k, int64_t d, void* stream) {
    return cinn::moe_combine(rows, dtype, pos, gates, nullptr, 0, y, n_tokens, n_rows, top_k, d, (cudaStream_t)stream);
}

int cinn_moe_combine_add(const void* rows, int dtype, const int64_t* pos, const float* gates, const void* addend,
                         int addend_dtype, void* y, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, void* stream) {
    return cinn::moe_combine(rows, dtype, pos, gates, addend, addend_dtype, y, n_tokens, n_rows, top_k, d,
                             (cudaStream_t)stream);
}

int cinn_gather_rows(const void* q, const float* scales, const int64_t* idx, void* out_q, float* out_scales, int64_t n_out,
                     int64_t n_src, int64_t d, int64_t n_scales, void* stream) {
    return cinn::gather_rows(q, scales, idx, out_q, out_scales, n_out, n_src, d, n_scales, (cudaStream_t)stream);
}

int cinn_sparse_attn_fwd(const void* q, const void* k, const void* v, int dtype, const int64_t* idx, float* out, float* lse,
                         float* attn_weights, int64_t B, int64_t H, int64_t L, int64_t K, int64_t d_qk, int64_t d_v,
                         float scale, void* stream) {
    return cinn::sparse_attn_fwd(q, k, v, dtype, idx, out, lse, attn_weights, B, H, L, K, d_qk, d_v, scale, (cudaStream_t)stream);
}

int cinn_sparse_attn_bwd(const void* grad_out, int grad_dtype, const float* out, const float* lse, const void* q,
                         const void* k, const void* v, int dtype, const int64_t* idx, float* grad_q, float* grad_k,
                         float* grad_v, int64_t B, int64_t H, int64_t L, int64_t K, int64_t d_qk, int64_t d_v, float scale,
                         void* stream) {
    return cinn::sparse_attn_bwd(grad_out, grad_dtype, out, lse, q, k, v, dtype, idx, grad_q, grad_k, grad_v, B, H, L, K, d_qk,
                                 d_v, scale, (cudaStream_t)stream);
}

int cinn_lightning_indexer(const void* q, const void* k, const void* w, int dtype, void* out, int64_t B, int64_t Lq,
                           int64_t Lk, int64_t H, int64_t d, const int64_t* q_strides, const int64_t* k_strides,
                           const int64_t* w_strides, void* stream) {
    return cinn::lightning_indexer(q, k, w, dtype, out, B, Lq, Lk, H, d, q_strides, k_strides, w_strides, (cudaStream_t)stream);
}

int cinn_scatter_rows(const void* in, const int64_t* idx, void* out, int64_t n_rows, int64_t n_dst, int64_t row_bytes,
                      void* stream) {
    return cinn::scatter_rows(in, idx, out, n_rows, n_dst, row_bytes, (cudaStream_t)stream);
}

int cinn_set_gemm_sm_limit(int n_sms) { return cinn::set_gemm_sm_limit(n_sms); }

int cinn_p2p_dispatch(const void* q, const float* scales, const int64_t* token_indices, const int64_t* sorted_experts,
                      const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_scales,
                      int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t n_scales, int experts_per_rank, int n_ranks,
                      int64_t capacity_rows, void* stream) {
    return cinn::p2p_dispatch(q, scales, token_indices, sorted_experts, base_send, my_start, peer_q, peer_scales, n_pairs,
                              n_tokens, d, n_scales, experts_per_rank, n_ranks, capacity_rows, (cudaStream_t)stream);
}

int cinn_p2p_return(const void* rows, const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home,
                    int64_t n_rows, int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity_rows, void* stream) {
    return cinn::p2p_return(rows, seg_start, home_base, peer_home, n_rows, row_bytes, n_segments, n_ranks, capacity_rows,
                            (cudaStream_t)stream);
}

int cinn_fp8_grouped_gemm_scatter(const void* A, const float* sA, const void* W, const float* sW, const int64_t* starts,
                                  const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out,
                                  const int64_t* row_dst, int out_dtype, void* stream) {
    return cinn::fp8_grouped_gemm(A, sA, W, sW, starts, ends, E, T, d_in, d_out, nullptr, out_dtype, (cudaStream_t)stream,
                                  reinterpret_cast<const long long*>(row_dst));
}

int cinn_p2p_row_table(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
                       int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity_rows, int64_t* row_dst, void* stream) {
    return cinn::p2p_row_table(seg_start, home_base, peer_home, n_rows, row_bytes, n_segments, n_ranks, capacity_rows,
                               reinterpret_cast<long long*>(row_dst), (cudaStream_t)stream);
}

int64_t cinn_fp8_grouped_wgrad_scratch_bytes(int64_t max_rows, int64_t d_in, int64_t d_out) {
    return cinn::grouped_wgrad_scratch_bytes(max_rows, d_in, d_out);
}

int cinn_fp8_grouped_wgrad(const void* dY, int dy_dtype, const void* x_q, const float* x_scales, const int64_t* starts_host,
                           const int64_t* ends_host, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* scratch,
                           int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, void* stream) {
    return cinn::fp8_grouped_wgrad(dY, dy_dtype, x_q, x_scales, starts_host, ends_host, E, T, d_in, d_out, scratch,
                                   scratch_bytes, dW, out_dtype, div_mode, (cudaStream_t)stream);
}

int cinn_swiglu(const void* h12, void* h, int dtype, int64_t T, int64_t I, void* stream) {
    return cinn::swiglu(h12, nullptr, h, dtype, T, I, 0, (cudaStream_t)stream);
}

int cinn_swiglu_backward(const void* h12, const void* grad_h, void* grad_h12, int dtype, int64_t T, int64_t I, void* stream) {
    return cinn::swiglu(h12, grad_h, grad_h12, dtype, T, I, 1, (cudaStream_t)stream);
}

int cinn_p2p_barrier(const int64_t* peer_flags, int rank, int n_ranks, unsigned epoch, void* stream) {
    return cinn::p2p_barrier(peer_flags, rank, n_ranks, epoch, (cudaStream_t)stream);
}

long long cinn_set_wait_limit_cycles(long long cycles) { return cinn::set_p2p_wait_limit(cycles); }

int64_t cinn_fp8_grouped_wgrad_fused_scratch_bytes(int64_t total_rows, int64_t n_experts, int64_t d_in, int64_t d_out) {
    return cinn::grouped_wgrad_fused_scratch_bytes(total_rows, n_experts, d_in, d_out);
}

int cinn_fp8_grouped_wgrad_fused(const void* dY, int dy_dtype, const void* x_q, const float* x_scales, const int64_t* expert_starts,
                                 const int64_t* expert_ends, int64_t n_experts, int64_t total_rows, int64_t d_in, int64_t d_out,
                                 void* scratch, int64_t scratch_bytes, void* dW, int out_dtype, int div_mode, void* dy_q_row,
                                 float* dy_row_scales, void* stream) {
    return cinn::fp8_grouped_wgrad_fused(dY, dy_dtype, x_q, x_scales, expert_starts, expert_ends, n_experts, total_rows, d_in, d_out,
                                         scratch, scratch_bytes, dW, out_dtype, div_mode, dy_q_row, dy_row_scales,
                                         (cudaStream_t)stream);
}

int cinn_grouped_gemm_16bit(const void* A, const void* W, int in_dtype, const int64_t* expert_starts, const int64_t* expert_ends,
                            int64_t n_experts, int64_t total_rows, int64_t d_in, int64_t d_out, void* C, int out_dtype,
                            void* stream) {
    return cinn::grouped_gemm_16bit(A, W, in_dtype, expert_starts, expert_ends, n_experts, total_rows, d_in, d_out, C, out_dtype,
                                    (cudaStream_t)stream);
}

int cinn_zero_rows_outside(void* buf, int64_t n_rows, int64_t row_bytes, const int64_t* starts, const int64_t* ends,
                           int64_t n_ranges, void* stream) {
    return cinn::zero_rows_outside(buf, n_rows, row_bytes, starts, ends, n_ranges, (cudaStream_t)stream);
}

int cinn_moe_combine_backward(const void* rows, int rows_dtype, const int64_t* pos, const float* gates, const float* dy,
                              void* d_rows, float* d_gates, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, void* stream) {
    return cinn::moe_combine_backward(rows, rows_dtype, pos, gates, dy, d_rows, d_gates, n_tokens, n_rows, top_k, d,
                                      (cudaStream_t)stream);
}

int cinn_p2p_plan(const int64_t* my_counts, const int64_t* peer_counts, const int64_t* peer_flags, int rank, int n_ranks,
                  int n_experts, int flag_slot, unsigned epoch, int64_t* base_send, int64_t* my_start, int64_t* starts,
                  int64_t* ends, int64_t* seg_start, int64_t* home_base, int64_t* total_rows, void* stream) {
    return cinn::p2p_plan(my_counts, peer_counts, peer_flags, rank, n_ranks, n_experts, flag_slot, epoch, base_send, my_start,
                          starts, ends, seg_start, home_base, total_rows, (cudaStream_t)stream);
}

int cinn_p2p_dispatch_signal(const void* q, const float* s, const int64_t* token_indices, const int64_t* sorted_experts,
                             const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_s,
                             int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t n_scales, int experts_per_rank, int n_ranks,
                             int64_t capacity_rows, const int64_t* peer_flags, int rank, int flag_slot, unsigned epoch,
                             unsigned* done_counter, int expert_lo, int expert_hi, int n_sms, void* stream) {
    return cinn::p2p_dispatch_signal(q, s, token_indices, sorted_experts, base_send, my_start, peer_q, peer_s, n_pairs, n_tokens,
                                     d, n_scales, experts_per_rank, n_ranks, capacity_rows, peer_flags, rank, flag_slot, epoch,
                                     done_counter, expert_lo, expert_hi, n_sms, (cudaStream_t)stream);
}

int cinn_p2p_row_table_wait(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
                            int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity_rows, int64_t* row_dst,
                            const int64_t* peer_flags, int rank, int flag_slot, unsigned epoch, void* stream) {
    return cinn::p2p_row_table_wait(seg_start, home_base, peer_home, n_rows, row_bytes, n_segments, n_ranks, capacity_rows,
                                    (long long*)row_dst, peer_flags, rank, flag_slot, epoch, (cudaStream_t)stream);
}

int64_t cinn_moe_route_workspace_ints(int64_t n_tokens, int n_experts) {
    return cinn::moe_route_workspace_ints(n_tokens, n_experts);
}

int cinn_moe_route(const float* logits, const float* bias, int64_t n_tokens, int n_experts, int top_k, int* workspace,
                   int* top_experts, float* top_gates, int64_t* token_indices, float* sorted_scores,
                   int64_t* sorted_experts, int64_t* counts, int64_t* pair_pos, float* pair_gate, void* stream) {
    return cinn::moe_route(logits, bias, n_tokens, n_experts, top_k, workspace, top_experts, top_gates, token_indices,
                           sorted_scores, sorted_experts, counts, pair_pos, pair_gate, (cudaStream_t)stream);
}

int64_t cinn_moe_route_static_max_ints(void) { return cinn::moe_route_static_max_ints(); }

int cinn_moe_route_static(const float* logits, const float* bias, int64_t n_tokens, int n_experts, int top_k,
                          int* top_experts, float* top_gates, int64_t* token_indices, float* sorted_scores,
                          int64_t* sorted_experts, int64_t* counts, int64_t* pair_pos, float* pair_gate, void* stream) {
    return cinn::moe_route_static(logits, bias, n_tokens, n_experts, top_k, top_experts, top_gates, token_indices,
                                  sorted_scores, sorted_experts, counts, pair_pos, pair_gate, (cudaStream_t)stream);
}

int cinn_device_status(int* out, int reset) {
    if (!out) { cinn::set_error("cinn_device_status: null pointer"); return CINN_ERR_INVALID; }
    return cinn::read_device_status(out, reset);
}

}  // extern "C"
