// MoE routing on the device: top-k selection and the stable sort of (token, expert) pairs by expert.
//
// Replaces the chain of torch calls at the head of cinnamon's MoE.forward (src/layers.py:122-148):
// sigmoid, + expert_bias, topk, gather, normalise, sort by expert, token_indices, bincount.  Three launches:
//
//   route_topk_kernel     one warp per token: sigmoid scores, the k largest of score + bias (ties: the lower
//                         expert id), gates = score / (sum of the k scores + 1e-9); every CTA of 128 tokens also
//                         leaves a histogram of the experts it selected in the workspace
//   route_scan_kernel     one CTA: per expert, the running sum of those histograms over the CTAs (the
//                         histograms become offsets) -> counts; exclusive scan over experts -> first row
//   route_scatter_kernel  the same CTAs again: every pair gets the next free row of its expert, pairs taken in
//                         (token, slot) order, so the order is that of a stable sort and the same on every
//                         run; writes token_indices / sorted_scores / sorted_experts, and per token its k rows
//                         in ascending order with their gates (what the combine pass reads)
//
// The workspace (ceil(T / 128) * E ints) is the only memory beyond inputs and outputs.
#include "common.cuh"
#include <mutex>

namespace cinn {

constexpr int ROUTE_TOKENS_PER_CTA = 128;
constexpr int ROUTE_MAX_EXPERTS = 1024;
constexpr int ROUTE_MAX_TOPK = 32;

template <int VPL>      // expert values per lane, E <= 32 * VPL
__global__ void __launch_bounds__(256)
route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int top_k,
                  int* __restrict__ top_experts, float* __restrict__ top_gates, int* __restrict__ hist) {
    __shared__ int s_hist[ROUTE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < E; e += 256) s_hist[e] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t_begin = blockIdx.x * ROUTE_TOKENS_PER_CTA;
    const int t_end = min(t_begin + ROUTE_TOKENS_PER_CTA, T);
    float b[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) b[i] = (lane + 32 * i < E) ? bias[lane + 32 * i] : 0.0f;
    for (int t = t_begin + warp; t < t_end; t += 8) {
        float s[VPL], sel[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int e = lane + 32 * i;
            if (e < E) {
                const float x = logits[(int64_t)t * E + e];
                s[i] = __fdiv_rn(1.0f, 1.0f + expf(-x));                  // torch.sigmoid in fp32
                sel[i] = s[i] + b[i];
                if (sel[i] != sel[i]) sel[i] = -INFINITY;                  // a NaN is never selected
            } else {
                s[i] = 0.0f;
                sel[i] = -INFINITY;
            }
        }
        float my_score = 0.0f;
        int my_expert = 0;
        for (int r = 0; r < top_k; ++r) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < VPL; ++i)
                if (sel[i] > best) { best = sel[i]; best_e = lane + 32 * i; }
            if (best == -INFINITY) best_e = 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
            }
            // fewer than k selectable experts (E < k, or NaNs): fall back to the lowest unused ids
            if (best_e == 0x7fffffff) best_e = r < E ? r : 0;
            float sc = 0.0f;
#pragma unroll
            for (int i = 0; i < VPL; ++i)
                if (lane + 32 * i == best_e) { sc = s[i]; sel[i] = -INFINITY; }
            sc = __shfl_sync(0xffffffffu, sc, best_e & 31);
            if (lane == r) { my_score = sc; my_expert = best_e; }
        }
        float sum = lane < top_k ? my_score : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane < top_k) {
            top_experts[(int64_t)t * top_k + lane] = my_expert;
            top_gates[(int64_t)t * top_k + lane] = __fdiv_rn(my_score, sum + 1e-9f);
            atomicAdd(&s_hist[my_expert], 1);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += 256) hist[(int64_t)blockIdx.x * E + e] = s_hist[e];
}

__global__ void __launch_bounds__(1024)
route_scan_kernel(int* __restrict__ hist, int n_ctas, int E, int64_t* __restrict__ counts, int* __restrict__ first_row) {
    __shared__ int s_scan[ROUTE_MAX_EXPERTS];
    const int e = threadIdx.x;
    int total = 0;
    if (e < E) {
        for (int b = 0; b < n_ctas; ++b) {
            const int v = hist[(int64_t)b * E + e];
            hist[(int64_t)b * E + e] = total;
            total += v;
        }
        counts[e] = total;
    }
    s_scan[e] = e < E ? total : 0;
    __syncthreads();
    // inclusive scan over experts (Hillis-Steele; E <= 1024 = blockDim)
    for (int o = 1; o < 1024; o <<= 1) {
        const int v = e >= o ? s_scan[e - o] : 0;
        __syncthreads();
        s_scan[e] += v;
        __syncthreads();
    }
    if (e < E) first_row[e] = s_scan[e] - total;
}

__global__ void __launch_bounds__(256)
route_scatter_kernel(const int* __restrict__ top_experts, const float* __restrict__ top_gates, const int* __restrict__ hist,
                     const int* __restrict__ first_row, int T, int E, int top_k, int64_t* __restrict__ token_indices,
                     float* __restrict__ sorted_scores, int64_t* __restrict__ sorted_experts,
                     int64_t* __restrict__ pair_pos, float* __restrict__ pair_gate) {
    __shared__ int s_next[ROUTE_MAX_EXPERTS];                                  // next free row of every expert
    __shared__ int s_pos[ROUTE_TOKENS_PER_CTA * ROUTE_MAX_TOPK];
    for (int e = threadIdx.x; e < E; e += 256) s_next[e] = first_row[e] + hist[(int64_t)blockIdx.x * E + e];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t_begin = blockIdx.x * ROUTE_TOKENS_PER_CTA;
    const int n_tok = min(ROUTE_TOKENS_PER_CTA, T - t_begin);
    const int n_pairs = n_tok * top_k;
    const int64_t pair0 = (int64_t)t_begin * top_k;
    for (int base = 0; base < n_pairs; base += 256) {
        const int p = base + threadIdx.x;
        const bool live = p < n_pairs;
        const int e = live ? top_experts[pair0 + p] : -1 - lane;              // dead lanes match nobody
        for (int w = 0; w < 8; ++w) {                                          // warps take their turn: (token, slot) order
            if (warp == w) {
                const unsigned peers = __match_any_sync(0xffffffffu, e);
                const int leader = __ffs(peers) - 1;
                int row = 0;
                if (live && lane == leader) {
                    row = s_next[e];
                    s_next[e] = row + __popc(peers);
                }
                row = __shfl_sync(0xffffffffu, row, leader) + __popc(peers & ((1u << lane) - 1u));
                if (live) {
                    s_pos[p] = row;
                    token_indices[row] = t_begin + p / top_k;
                    sorted_scores[row] = top_gates[pair0 + p];
                    sorted_experts[row] = e;
                }
            }
            __syncthreads();
        }
    }
    // per token: its rows in ascending order, gates alongside (insertion sort, k <= 32)
    for (int tl = threadIdx.x; tl < n_tok; tl += 256) {
        int pos[ROUTE_MAX_TOPK];
        float gate[ROUTE_MAX_TOPK];
        for (int j = 0; j < top_k; ++j) {
            const int v = s_pos[tl * top_k + j];
            const float g = top_gates[pair0 + tl * top_k + j];
            int i = j;
            while (i > 0 && pos[i - 1] > v) { pos[i] = pos[i - 1]; gate[i] = gate[i - 1]; --i; }
            pos[i] = v;
            gate[i] = g;
        }
        for (int j = 0; j < top_k; ++j) {
            pair_pos[(int64_t)(t_begin + tl) * top_k + j] = pos[j];
            pair_gate[(int64_t)(t_begin + tl) * top_k + j] = gate[j];
        }
    }
}

int64_t moe_route_workspace_ints(int64_t T, int E) {
    return ((T + ROUTE_TOKENS_PER_CTA - 1) / ROUTE_TOKENS_PER_CTA) * (int64_t)E + E;
}

int moe_route(const float* logits, const float* bias, int64_t T, int E, int top_k, int* workspace, int* top_experts,
              float* top_gates, int64_t* token_indices, float* sorted_scores, int64_t* sorted_experts, int64_t* counts,
              int64_t* pair_pos, float* pair_gate, cudaStream_t st) {
    CINN_CHECK_ARG(T >= 0 && E >= 1 && E <= ROUTE_MAX_EXPERTS, "moe_route: 1 <= E <= %d experts (got %d)", ROUTE_MAX_EXPERTS, E);
    CINN_CHECK_ARG(top_k >= 1 && top_k <= ROUTE_MAX_TOPK && top_k <= E, "moe_route: 1 <= top_k <= min(E, %d) (got %d)",
                   ROUTE_MAX_TOPK, top_k);
    CINN_CHECK_ARG(T * (int64_t)top_k < (1LL << 31), "moe_route: too many (token, expert) pairs");
    CINN_CHECK_ARG(counts != nullptr, "moe_route: null pointer");
    if (T == 0) {
        CINN_CHECK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int64_t) * E, st));
        return CINN_OK;
    }
    CINN_CHECK_ARG(logits && bias && workspace && top_experts && top_gates && token_indices && sorted_scores &&
                   sorted_experts && pair_pos && pair_gate, "moe_route: null pointer");
    const int n_ctas = (int)((T + ROUTE_TOKENS_PER_CTA - 1) / ROUTE_TOKENS_PER_CTA);
    int* hist = workspace;
    int* first_row = workspace + (int64_t)n_ctas * E;
#define CINN_TOPK(V) route_topk_kernel<V><<<n_ctas, 256, 0, st>>>(logits, bias, (int)T, E, top_k, top_experts, top_gates, hist)
    if (E <= 32) CINN_TOPK(1);
    else if (E <= 64) CINN_TOPK(2);
    else if (E <= 128) CINN_TOPK(4);
    else if (E <= 256) CINN_TOPK(8);
    else if (E <= 512) CINN_TOPK(16);
    else CINN_TOPK(32);
#undef CINN_TOPK
    CINN_CHECK_LAUNCH();
    route_scan_kernel<<<1, 1024, 0, st>>>(hist, n_ctas, E, counts, first_row);
    CINN_CHECK_LAUNCH();
    route_scatter_kernel<<<n_ctas, 256, 0, st>>>(top_experts, top_gates, hist, first_row, (int)T, E, top_k, token_indices,
                                                 sorted_scores, sorted_experts, pair_pos, pair_gate);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// The same routing for callers that cannot hand over a workspace.  The scratch lives in a fixed array inside
// the library image: every GPU that loads the library holds these 2 MiB until the process exits.  All calls on
// a device share it, so two calls that overlap on that GPU (different streams, different threads) race; the
// routing kernels overwrite every word they later read, so nothing has to be cleared between calls.
// ---------------------------------------------------------------------------
constexpr int64_t ROUTE_STATIC_MAX_INTS = 1 << 19;                     // 2 MiB
static __device__ __align__(256) int g_route_scratch[ROUTE_STATIC_MAX_INTS];

constexpr int ROUTE_MAX_DEVICES = 64;
static std::mutex g_route_scratch_mutex;
static int* g_route_scratch_ptr[ROUTE_MAX_DEVICES] = {};               // device address of the array, per device

// In host code `g_route_scratch` is only a handle for the symbol, not an address a kernel can use; the device
// address is asked for once per device, with that device current.
static int route_scratch_address(int** out) {
    int dev = -1;
    CINN_CHECK_CUDA(cudaGetDevice(&dev));
    CINN_CHECK_ARG(dev >= 0 && dev < ROUTE_MAX_DEVICES, "moe_route_static: device ordinal %d is beyond %d", dev,
                   ROUTE_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_route_scratch_mutex);
    if (g_route_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        CINN_CHECK_CUDA(cudaGetSymbolAddress(&p, g_route_scratch));
        g_route_scratch_ptr[dev] = static_cast<int*>(p);
    }
    *out = g_route_scratch_ptr[dev];
    return CINN_OK;
}

int64_t moe_route_static_max_ints() { return ROUTE_STATIC_MAX_INTS; }

int moe_route_static(const float* logits, const float* bias, int64_t T, int E, int top_k, int* top_experts, float* top_gates,
                     int64_t* token_indices, float* sorted_scores, int64_t* sorted_experts, int64_t* counts,
                     int64_t* pair_pos, float* pair_gate, cudaStream_t st) {
    CINN_CHECK_ARG(T >= 0 && E >= 1 && E <= ROUTE_MAX_EXPERTS, "moe_route_static: 1 <= E <= %d experts (got %d)",
                   ROUTE_MAX_EXPERTS, E);
    const int64_t need = moe_route_workspace_ints(T, E);
    CINN_CHECK_ARG(need <= ROUTE_STATIC_MAX_INTS,
                   "moe_route_static: %lld tokens x %d experts need %lld ints of scratch, the built-in array holds %lld; "
                   "use cinn_moe_route with a workspace of your own",
                   (long long)T, E, (long long)need, (long long)ROUTE_STATIC_MAX_INTS);
    int* scratch = nullptr;
    int rc = route_scratch_address(&scratch);
    if (rc) return rc;
    return moe_route(logits, bias, T, E, top_k, scratch, top_experts, top_gates, token_indices, sorted_scores,
                     sorted_experts, counts, pair_pos, pair_gate, st);
}

}  // namespace cinn
