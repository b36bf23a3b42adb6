// MoE combine: y[t, :] = sum_j gate[t, j] * rows[pos[t, j], :]   (fp32 result)
//
// Replaces the three torch passes at the end of cinnamon's MoE.forward (src/layers.py:157-160:
// `sorted_out * sorted_scores[:, None]`, `torch.zeros`, `scatter_add_`) by one gather-style pass
// without atomics: every token reads the rows of its own (token, expert) pairs.  With the
// positions of a token given in ascending order the fp32 sum has the order of the reference's
// scatter-add over the sorted pairs.
#include "common.cuh"
#include <atomic>

namespace cinn {

template <typename T>
__device__ __forceinline__ void load8f(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8f<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <>
__device__ __forceinline__ void load8f<__half>(const __half* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <>
__device__ __forceinline__ void load8f<float>(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

constexpr int kMaxTopK = 32;

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ rows, const int64_t* __restrict__ pos, const float* __restrict__ gates,
                   const void* __restrict__ addend, int addend_dtype, float* __restrict__ y, int64_t n_rows, int top_k,
                   int d) {
    __shared__ int64_t s_pos[kMaxTopK];
    __shared__ float s_gate[kMaxTopK];
    const int64_t t = blockIdx.x;
    if (threadIdx.x < top_k) {
        const int64_t p = pos[t * top_k + threadIdx.x];
        s_pos[threadIdx.x] = (p >= 0 && p < n_rows) ? p : -1;
        s_gate[threadIdx.x] = gates[t * top_k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x * 8; c < d; c += 256 * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top_k; ++j) {
            const int64_t p = s_pos[j];
            if (p < 0) continue;
            float v[8];
            load8f<T>(rows + p * d + c, v);
            const float g = s_gate[j];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(v[i], g));   // product then sum, as the reference
        }
        if (addend != nullptr) {                   // shared-expert output + routed sum (src/layers.py:179)
            float a[8];
            if (addend_dtype == CINN_BF16) load8f<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(addend) + t * d + c, a);
            else if (addend_dtype == CINN_F16) load8f<__half>(reinterpret_cast<const __half*>(addend) + t * d + c, a);
            else load8f<float>(reinterpret_cast<const float*>(addend) + t * d + c, a);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(a[i], acc[i]);
        }
        float4* out = reinterpret_cast<float4*>(y + t * d + c);
        out[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        out[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

int moe_combine(const void* rows, int dtype, const int64_t* pos, const float* gates, const void* addend, int addend_dtype,
                void* y, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, cudaStream_t st) {
    CINN_CHECK_ARG(n_tokens >= 0 && n_rows >= 0 && d >= 0, "moe_combine: negative shape");
    if (n_tokens == 0 || d == 0) return CINN_OK;
    CINN_CHECK_ARG(pos && gates && y && (rows || n_rows == 0), "moe_combine: null pointer");
    CINN_CHECK_ARG(top_k >= 1 && top_k <= kMaxTopK, "moe_combine: top_k must be in [1, %d]", kMaxTopK);
    CINN_CHECK_ARG(d % 8 == 0 && d < (1LL << 31), "moe_combine: the row width (%lld) must be a multiple of 8", (long long)d);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(rows) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0,
                   "moe_combine: rows and y must be 16-byte aligned");
    CINN_CHECK_ARG(n_tokens < (1LL << 31), "moe_combine: too many tokens");
    CINN_CHECK_ARG(addend == nullptr || addend_dtype == CINN_BF16 || addend_dtype == CINN_F16 || addend_dtype == CINN_F32,
                   "moe_combine: unknown addend dtype tag %d", addend_dtype);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(addend) & 15) == 0, "moe_combine: the addend must be 16-byte aligned");
    const unsigned grid = (unsigned)n_tokens;
    switch (dtype) {
        case CINN_BF16: moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)rows, pos, gates, addend, addend_dtype, (float*)y, n_rows, top_k, (int)d); break;
        case CINN_F16: moe_combine_kernel<__half><<<grid, 256, 0, st>>>((const __half*)rows, pos, gates, addend, addend_dtype, (float*)y, n_rows, top_k, (int)d); break;
        case CINN_F32: moe_combine_kernel<float><<<grid, 256, 0, st>>>((const float*)rows, pos, gates, addend, addend_dtype, (float*)y, n_rows, top_k, (int)d); break;
        default: set_error("moe_combine: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// SwiGLU between the two grouped GEMMs, for training (src/layers.py:71-74: h1, h2 = h12.float().chunk(2);
// h = (silu(h1) * h2).to(dtype)) and its backward:
//   dh1 = dh * h2 * sig(h1) * (1 + h1 * (1 - sig(h1))),   dh2 = dh * silu(h1),   fp32 arithmetic, results rounded
// to the activation type.  One pass each, 16-byte vectors, a thread owns eight consecutive columns of one row.
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__device__ __forceinline__ void store8f(T* p, const float (&v)[8]) {
    if constexpr (sizeof(T) == 4) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        T t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = from_float<T>(v[i]);
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(t);
    }
}

// Backward of the combine pass, y[t] = sum_j gate[t, j] * rows[pos[t, j]] (+ addend[t]):
//   d_rows[pos[t, j]] = gate[t, j] * dy[t]         (every row belongs to exactly one pair: no accumulation)
//   d_gate[t, j]      = < rows[pos[t, j]], dy[t] >
// One warp per (token, slot) pair, 16-byte vectors.  Rows that no pair names are left as the caller initialised them.
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_backward_kernel(const T* __restrict__ rows, const int64_t* __restrict__ pos, const float* __restrict__ gates,
                            const float* __restrict__ dy, T* __restrict__ d_rows, float* __restrict__ d_gates,
                            int64_t n_pairs, int64_t n_rows, int top_k, int d) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 8;
    for (int64_t pr = warp; pr < n_pairs; pr += n_warps) {
        const int64_t p = pos[pr];
        if (p < 0 || p >= n_rows) {
            if (lane == 0) d_gates[pr] = 0.0f;
            continue;
        }
        const int64_t t = pr / top_k;
        const float g = gates[pr];
        float dot = 0.0f;
        for (int c = lane * 8; c < d; c += 32 * 8) {
            float r[8], gy[8], o[8];
            load8f<T>(rows + p * d + c, r);
            load8f<float>(dy + t * d + c, gy);
#pragma unroll
            for (int i = 0; i < 8; ++i) { o[i] = g * gy[i]; dot = fmaf(r[i], gy[i], dot); }
            store8f<T>(d_rows + p * d + c, o);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) d_gates[pr] = dot;
    }
}

template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ h12, const T* __restrict__ dh, T* __restrict__ out, int64_t T_rows, int I) {
    const int per_row = I >> 3;
    const int64_t total = T_rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t row = i / per_row;
        const int col = (int)(i - row * per_row) << 3;
        float a[8], b[8];
        load8f<T>(h12 + row * 2 * (int64_t)I + col, a);
        load8f<T>(h12 + row * 2 * (int64_t)I + I + col, b);
        if constexpr (!BACKWARD) {
            float h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = (a[j] / (1.0f + expf(-a[j]))) * b[j];
            store8f<T>(out + row * (int64_t)I + col, h);
        } else {
            float g[8], d1[8], d2[8];
            load8f<T>(dh + row * (int64_t)I + col, g);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float sig = 1.0f / (1.0f + expf(-a[j]));
                d1[j] = g[j] * b[j] * sig * (1.0f + a[j] * (1.0f - sig));
                d2[j] = g[j] * a[j] * sig;
            }
            store8f<T>(out + row * 2 * (int64_t)I + col, d1);
            store8f<T>(out + row * 2 * (int64_t)I + I + col, d2);
        }
    }
}

template <typename T>
static int swiglu_typed(const T* h12, const T* dh, T* out, int64_t T_rows, int64_t I, bool backward, cudaStream_t st) {
    int64_t blocks = (T_rows * (I / 8) + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (backward) swiglu_kernel<T, true><<<(unsigned)blocks, 256, 0, st>>>(h12, dh, out, T_rows, (int)I);
    else swiglu_kernel<T, false><<<(unsigned)blocks, 256, 0, st>>>(h12, dh, out, T_rows, (int)I);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// forward: out (T, I) = silu(h12[:, :I]) * h12[:, I:];  backward: out (T, 2I) = d h12 given dh (T, I)
int swiglu(const void* h12, const void* dh, void* out, int dtype, int64_t T_rows, int64_t I, int backward, cudaStream_t st) {
    CINN_CHECK_ARG(T_rows >= 0 && I >= 0, "swiglu: negative shape");
    if (T_rows == 0 || I == 0) return CINN_OK;
    CINN_CHECK_ARG(h12 && out && (!backward || dh), "swiglu: null pointer");
    CINN_CHECK_ARG(I % 8 == 0 && I < (1LL << 30), "swiglu: the hidden width (%lld) must be a multiple of 8", (long long)I);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(h12) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(dh) & 15) == 0, "swiglu: buffers must be 16-byte aligned");
    switch (dtype) {
        case CINN_BF16: return swiglu_typed((const __nv_bfloat16*)h12, (const __nv_bfloat16*)dh, (__nv_bfloat16*)out, T_rows, I, backward != 0, st);
        case CINN_F16: return swiglu_typed((const __half*)h12, (const __half*)dh, (__half*)out, T_rows, I, backward != 0, st);
        case CINN_F32: return swiglu_typed((const float*)h12, (const float*)dh, (float*)out, T_rows, I, backward != 0, st);
        default: set_error("swiglu: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

// ---------------------------------------------------------------------------
// Dispatch gather: out_q[r, :] = q[idx[r], :] (e4m3 bytes) and out_s[r, :] = s[idx[r], :] (their 1x128 scales)
// in one pass: the `flat_x[token_indices]` of MoE.forward (src/layers.py:140) applied to tokens that were
// quantised once, before the gather.  One warp per output row, 16-byte vectors.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t* __restrict__ q, const float* __restrict__ s, const int64_t* __restrict__ idx,
                   uint8_t* __restrict__ out_q, float* __restrict__ out_s, int64_t n_out, int64_t n_src, int d, int ns) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 8;
    const int vecs = d >> 4;
    for (int64_t r = warp; r < n_out; r += n_warps) {
        const int64_t src = idx[r];
        if (src < 0 || src >= n_src) continue;                                    // rows outside the source stay untouched
        const uint4* in = reinterpret_cast<const uint4*>(q + src * d);
        uint4* out = reinterpret_cast<uint4*>(out_q + r * d);
        for (int v = lane; v < vecs; v += 32) __stcs(out + v, __ldg(in + v));
        for (int c = lane; c < ns; c += 32) out_s[r * ns + c] = s[src * ns + c];
    }
}

int gather_rows(const void* q, const float* s, const int64_t* idx, void* out_q, float* out_s, int64_t n_out, int64_t n_src,
                int64_t d, int64_t ns, cudaStream_t st) {
    CINN_CHECK_ARG(n_out >= 0 && n_src >= 0 && d >= 0 && ns >= 0, "gather_rows: negative shape");
    if (n_out == 0 || d == 0) return CINN_OK;
    CINN_CHECK_ARG(q && s && idx && out_q && out_s, "gather_rows: null pointer");
    CINN_CHECK_ARG(d % 16 == 0 && d < (1LL << 31) && ns < (1LL << 31), "gather_rows: the row width (%lld) must be a multiple of 16",
                   (long long)d);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(out_q) & 15) == 0,
                   "gather_rows: byte buffers must be 16-byte aligned");
    int64_t blocks = (n_out + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)q, s, idx, (uint8_t*)out_q, out_s, n_out, n_src, (int)d,
                                                        (int)ns);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// Row scatter: out[idx[r], :] = in[r, :] for rows of `row_bytes` bytes (a multiple of 16).  The way back from the
// expert-grouped order to the arrival order before the rows travel home (the inverse of the regrouping gather).
// One warp per row, 16-byte vectors.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const uint4* __restrict__ in, const int64_t* __restrict__ idx, uint4* __restrict__ out, int64_t n_rows,
                    int64_t n_dst, int vecs) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 8;
    for (int64_t r = warp; r < n_rows; r += n_warps) {
        const int64_t dst = idx[r];
        if (dst < 0 || dst >= n_dst) continue;
        const uint4* src = in + r * vecs;
        uint4* o = out + dst * vecs;
        for (int v = lane; v < vecs; v += 32) __stcs(o + v, __ldcs(src + v));
    }
}

int scatter_rows(const void* in, const int64_t* idx, void* out, int64_t n_rows, int64_t n_dst, int64_t row_bytes,
                 cudaStream_t st) {
    CINN_CHECK_ARG(n_rows >= 0 && n_dst >= 0 && row_bytes >= 0, "scatter_rows: negative shape");
    if (n_rows == 0 || row_bytes == 0) return CINN_OK;
    CINN_CHECK_ARG(in && idx && out, "scatter_rows: null pointer");
    CINN_CHECK_ARG(row_bytes % 16 == 0 && row_bytes / 16 < (1LL << 31), "scatter_rows: the row size (%lld bytes) must be a multiple of 16",
                   (long long)row_bytes);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
                   "scatter_rows: buffers must be 16-byte aligned");
    int64_t blocks = (n_rows + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    scatter_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>((const uint4*)in, idx, (uint4*)out, n_rows, n_dst, (int)(row_bytes / 16));
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// Expert-parallel exchange by peer stores.  Every rank holds receive buffers that the other ranks of the node
// can address (symmetric memory); `peer_*` are device arrays with one base address per rank (this rank's own
// buffer included).  The destination row of every source row is a closed formula of the routing counts of all
// ranks (tables built on the host side, see cinnamon_b200/p2p.py), so no rank needs to be told where to write.
// Rows whose table entries point outside the buffers are skipped and counted in a device status word.
// ---------------------------------------------------------------------------
__device__ int g_moe_status = 0;      // 0 = fine, otherwise (5 << 8) | reason

// Dispatch: pair r of this rank (sorted by expert) -> the rank owning its expert, in that rank's expert-grouped
// order.  Fuses `flat_x[token_indices]` (src/layers.py:140), the two dispatch all-to-alls and the regrouping.
// SIGNAL: the CTA that finishes last tells every rank "all my rows have landed" (release store of `epoch` into
// slot flag_slot + me of each rank's flag array), which replaces a separate barrier launch after the dispatch; the
// consumer waits for the flags of all ranks (p2p_row_table with wait, or p2p_wait_flags).  `done` is a zeroed
// device counter that the last CTA resets.
// Launched with 256 threads per CTA on every SM, or ("narrow") with 1024 threads and so much dynamic shared memory
// that one CTA fills an SM, one CTA per SM on a chosen number of SMs: the stores are bound by NVLink, not by the SMs,
// and a persistent GEMM launched beside it then finds the other SMs free.
template <bool SIGNAL>
__global__ void __launch_bounds__(1024)
p2p_dispatch_kernel(const uint8_t* __restrict__ q, const float* __restrict__ s, const int64_t* __restrict__ token_indices,
                    const int64_t* __restrict__ sorted_experts, const int64_t* __restrict__ base_send,
                    const int64_t* __restrict__ my_start, const int64_t* __restrict__ peer_q,
                    const int64_t* __restrict__ peer_s, int64_t n_pairs, int64_t n_tokens, int d, int ns, int e_local,
                    int n_ranks, int64_t capacity, const int64_t* __restrict__ peer_flags = nullptr, int me = 0,
                    int flag_slot = 0, unsigned epoch = 0, unsigned* __restrict__ done = nullptr, int e_lo = 0, int e_hi = 0) {
    const int lane = threadIdx.x & 31;
    const int wpc = blockDim.x >> 5;                         // warps per CTA
    const int64_t warp = (int64_t)blockIdx.x * wpc + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * wpc;
    const int vecs = d >> 4;
    // The signalling variant sends the pairs of the local experts [e_lo, e_hi) of every rank: one run of the sorted
    // pairs per destination rank, taken in the order me + 1, me + 2, ..., me, so that at any moment the ranks write
    // to different destinations instead of all to rank 0 first.  seg_begin: running length of the runs, seg_src:
    // where each run starts among the sorted pairs.
    __shared__ long long seg_begin[65], seg_src[64];
    int64_t total = n_pairs;
    if constexpr (SIGNAL) {
        if (threadIdx.x == 0) {
            long long run = 0;
            const int E = e_local * n_ranks;
            for (int k = 0; k < n_ranks; ++k) {
                const int r = (me + 1 + k) % n_ranks;
                const int ea = r * e_local + e_lo, eb = r * e_local + e_hi;
                const long long a = my_start[ea], b = eb < E ? my_start[eb] : (long long)n_pairs;
                seg_begin[k] = run;
                seg_src[k] = a;
                run += b > a ? b - a : 0;
            }
            seg_begin[n_ranks] = run;
        }
        __syncthreads();
        total = seg_begin[n_ranks];
    }
    for (int64_t v = warp; v < total; v += n_warps) {
        int64_t r = v;
        if constexpr (SIGNAL) {
            int k = 0;
            while (k + 1 < n_ranks && seg_begin[k + 1] <= v) ++k;
            r = seg_src[k] + (v - seg_begin[k]);
        }
        const int64_t e = sorted_experts[r];
        const int64_t tok = token_indices[r];
        bool ok = e >= 0 && e < (int64_t)e_local * n_ranks && tok >= 0 && tok < n_tokens;
        int64_t dst = 0;
        int rank = 0;
        if (ok) {
            rank = (int)(e / e_local);
            dst = base_send[e] + (r - my_start[e]);
            ok = dst >= 0 && dst < capacity;
        }
        if (!ok) {
            if (lane == 0) atomicCAS(&g_moe_status, 0, (5 << 8) | 1);
            continue;
        }
        const uint4* in = reinterpret_cast<const uint4*>(q + tok * d);
        uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(peer_q[rank]) + dst * d);
        for (int v4 = lane; v4 < vecs; v4 += 32) out[v4] = __ldg(in + v4);
        float* so = reinterpret_cast<float*>(peer_s[rank]) + dst * ns;
        for (int c = lane; c < ns; c += 32) so[c] = s[tok * ns + c];
    }
    if constexpr (SIGNAL) {
        __shared__ bool last;
        __threadfence_system();                          // this thread's peer stores are visible system-wide
        __syncthreads();
        if (threadIdx.x == 0) last = atomicAdd(done, 1u) == gridDim.x - 1;
        __syncthreads();
        if (last) {
            __threadfence_system();
            if (threadIdx.x == 0) *done = 0;
            if ((int)threadIdx.x < n_ranks) {
                unsigned* remote = reinterpret_cast<unsigned*>(peer_flags[threadIdx.x]) + flag_slot + me;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
            }
        }
    }
}

// Return: row r of this rank's expert-grouped outputs -> the rank its token lives on, at the position of its
// pair in that rank's sorted order.  Fuses the inverse permutation and the combine all-to-all.
__global__ void __launch_bounds__(256)
p2p_return_kernel(const uint4* __restrict__ rows, const int64_t* __restrict__ seg_start, const int64_t* __restrict__ home_base,
                  const int64_t* __restrict__ peer_home, int64_t n_rows, int n_segments, int n_ranks, int vecs,
                  int64_t capacity) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 8;
    for (int64_t r = warp; r < n_rows; r += n_warps) {
        // segment of row r: the first one whose end (the next start) lies beyond r; empty segments are stepped over
        int lo = 0, hi = n_segments;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (seg_start[mid + 1] > r) hi = mid; else lo = mid + 1;
        }
        bool ok = lo < n_segments && seg_start[lo] <= r;
        int64_t dst = 0;
        if (ok) {
            dst = home_base[lo] + (r - seg_start[lo]);
            ok = dst >= 0 && dst < capacity;
        }
        if (!ok) {
            if (lane == 0) atomicCAS(&g_moe_status, 0, (5 << 8) | 2);
            continue;
        }
        const uint4* in = rows + r * vecs;
        uint4* out = reinterpret_cast<uint4*>(peer_home[lo % n_ranks]) + dst * vecs;
        for (int v = lane; v < vecs; v += 32) out[v] = __ldcs(in + v);
    }
}

// Barrier over the ranks of one node on flags in symmetric memory: thread g tells rank g that this rank has
// arrived (release store, system scope, of the epoch into slot `me` of rank g's flag array) and waits until rank g
// has said the same (acquire loads of slot g of this rank's own array).  Kernels enqueued earlier on the stream
// have completed, so their peer stores are ordered before the flag.  The wait is bounded (about two seconds):
// when it runs out the kernel records a code in the status word and returns.  Each rank must own its GPU: ranks
// that share one could wait for a kernel that cannot run beside them.
// The limit is a launch argument (cinn_set_wait_limit_cycles), so a test can make the wait run out in a millisecond.
static std::atomic<long long> g_p2p_wait_limit{4000000000LL};
long long set_p2p_wait_limit(long long cycles) { return g_p2p_wait_limit.exchange(cycles > 0 ? cycles : 4000000000LL); }

__global__ void __launch_bounds__(64)
p2p_barrier_kernel(const int64_t* __restrict__ peer_flags, int me, int n_ranks, unsigned epoch, long long wait_limit) {
    const int g = threadIdx.x;
    if (g >= n_ranks) return;
    __threadfence_system();
    unsigned* remote = reinterpret_cast<unsigned*>(peer_flags[g]) + me;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const unsigned* mine = reinterpret_cast<const unsigned*>(peer_flags[me]) + g;
    const long long t0 = clock64();
    for (unsigned spin = 1;; ++spin) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int)(seen - epoch) >= 0) break;
        if ((spin & 63u) == 0 && clock64() - t0 > wait_limit) {
            atomicCAS(&g_moe_status, 0, (5 << 8) | 3);
            break;
        }
    }
}

// Bounded wait of thread g (< n_ranks) for slot flag_slot + g of this rank's own flag array to reach `epoch`.
// Returns false (and records `code`) when the limit runs out.
__device__ __forceinline__ bool p2p_wait_flag(const int64_t* peer_flags, int me, int g, int flag_slot, unsigned epoch,
                                              long long wait_limit, int code) {
    const unsigned* mine = reinterpret_cast<const unsigned*>(peer_flags[me]) + flag_slot + g;
    const long long t0 = clock64();
    for (unsigned spin = 1;; ++spin) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int)(seen - epoch) >= 0) return true;
        if ((spin & 63u) == 0 && clock64() - t0 > wait_limit) {
            atomicCAS(&g_moe_status, 0, code);
            return false;
        }
    }
}

// The exchange plan in one launch (one CTA): this rank's routing counts (E) are written into slot `me` of every
// rank's (G, E) count matrix in symmetric memory and flagged; once the counts of all ranks have arrived (bounded
// wait) the address tables of the exchange are derived from the matrix - the arithmetic of p2p.exchange_tables:
//   base_send[e]  destination row of my first pair of expert e, on the rank that owns e
//   my_start[e]   first position of expert e among my sorted pairs
//   starts/ends   row range of each of my local experts in my expert-grouped receive buffer
//   seg_start     first row of segment (local expert, source rank), expert-major; last entry = total rows
//   home_base     row on the source rank where that segment's outputs go
// Replaces an all-gather of the counts plus about twenty small tensor operations per layer call.
constexpr int PLAN_MAX_E = 1024, PLAN_MAX_G = 16;

__global__ void __launch_bounds__(256)
p2p_plan_kernel(const int64_t* __restrict__ my_counts, const int64_t* __restrict__ peer_counts,
                const int64_t* __restrict__ peer_flags, int me, int G, int E, int flag_slot, unsigned epoch,
                long long wait_limit, int64_t* __restrict__ base_send, int64_t* __restrict__ my_start,
                int64_t* __restrict__ starts, int64_t* __restrict__ ends, int64_t* __restrict__ seg_start,
                int64_t* __restrict__ home_base, int64_t* __restrict__ total_rows) {
    __shared__ long long per_expert[PLAN_MAX_E];      // column sums
    __shared__ long long starts_all[PLAN_MAX_E];      // first row of expert e on the rank that owns it
    __shared__ long long row_total[PLAN_MAX_G];
    __shared__ int ok_all;
    const int tid = threadIdx.x;
    const int e_local = E / G;
    if (tid == 0) ok_all = 1;
    // 1. my counts into every rank's matrix (my own included)
    for (int i = tid; i < G * E; i += 256) {
        const int g = i / E, e = i - g * E;
        reinterpret_cast<long long*>(peer_counts[g])[(int64_t)me * E + e] = my_counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < G) {
        unsigned* remote = reinterpret_cast<unsigned*>(peer_flags[tid]) + flag_slot + me;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
        if (!p2p_wait_flag(peer_flags, me, tid, flag_slot, epoch, wait_limit, (5 << 8) | 5)) ok_all = 0;
    }
    __syncthreads();
    // 2. tables from the (G, E) matrix (read past L1: peers wrote it)
    const long long* C = reinterpret_cast<const long long*>(peer_counts[me]);
    for (int e = tid; e < E; e += 256) {
        long long sum = 0;
        for (int g = 0; g < G; ++g) sum += ok_all ? __ldcg(C + (int64_t)g * E + e) : 0;
        per_expert[e] = sum;
    }
    __syncthreads();
    if (tid < G) {                                   // thread r: running start of the experts owned by rank r
        long long run = 0;
        for (int el = 0; el < e_local; ++el) {
            starts_all[tid * e_local + el] = run;
            run += per_expert[tid * e_local + el];
        }
        row_total[tid] = run;
    }
    __syncthreads();
    const int lo = me * e_local;
    for (int e = tid; e < E; e += 256) {
        long long below = 0;                          // rows of lower-ranked sources for expert e
        for (int g = 0; g < me; ++g) below += ok_all ? __ldcg(C + (int64_t)g * E + e) : 0;
        base_send[e] = starts_all[e] + below;
    }
    if (tid == 0) {                                  // my sorted pairs: exclusive running sum of my own counts
        long long run = 0;
        for (int e = 0; e < E; ++e) { my_start[e] = run; run += my_counts[e]; }
        *total_rows = row_total[me];
        seg_start[(int64_t)e_local * G] = row_total[me];
    }
    for (int el = tid; el < e_local; el += 256) {
        starts[el] = starts_all[lo + el];
        ends[el] = starts_all[lo + el] + per_expert[lo + el];
        long long below = 0;
        for (int g = 0; g < G; ++g) {
            seg_start[(int64_t)el * G + g] = starts_all[lo + el] + below;
            below += ok_all ? __ldcg(C + (int64_t)g * E + lo + el) : 0;
        }
    }
    if (tid < G) {                                   // thread g: where rank g's pairs of my local experts sit in its sorted order
        long long run = 0;
        for (int e = 0; e < lo + e_local; ++e) {
            if (e >= lo) home_base[(int64_t)(e - lo) * G + tid] = run;
            run += ok_all ? __ldcg(C + (int64_t)tid * E + e) : 0;
        }
    }
}

int p2p_plan(const int64_t* my_counts, const int64_t* peer_counts, const int64_t* peer_flags, int me, int G, int E,
             int flag_slot, unsigned epoch, int64_t* base_send, int64_t* my_start, int64_t* starts, int64_t* ends,
             int64_t* seg_start, int64_t* home_base, int64_t* total_rows, cudaStream_t st) {
    CINN_CHECK_ARG(G >= 1 && G <= PLAN_MAX_G && E >= G && E <= PLAN_MAX_E && E % G == 0 && me >= 0 && me < G && flag_slot >= 0,
                   "p2p_plan: 1 <= ranks <= %d, experts <= %d and divisible by the ranks (got %d, %d)", PLAN_MAX_G, PLAN_MAX_E, G, E);
    CINN_CHECK_ARG(my_counts && peer_counts && peer_flags && base_send && my_start && starts && ends && seg_start && home_base &&
                   total_rows, "p2p_plan: null pointer");
    p2p_plan_kernel<<<1, 256, 0, st>>>(my_counts, peer_counts, peer_flags, me, G, E, flag_slot, epoch,
                                       g_p2p_wait_limit.load(std::memory_order_relaxed), base_send, my_start, starts, ends,
                                       seg_start, home_base, total_rows);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// p2p_row_table that first waits (bounded) until every rank has flagged "all my rows have landed"
// (p2p_dispatch_signal): the table is built - and the GEMMs that follow it on the stream start - only then.
__global__ void __launch_bounds__(256)
p2p_row_table_wait_kernel(const int64_t* __restrict__ seg_start, const int64_t* __restrict__ home_base,
                          const int64_t* __restrict__ peer_home, int64_t n_rows, int n_segments, int n_ranks, int64_t row_bytes,
                          int64_t capacity, long long* __restrict__ row_dst, const int64_t* __restrict__ peer_flags, int me,
                          int flag_slot, unsigned epoch, long long wait_limit) {
    if ((int)threadIdx.x < n_ranks) p2p_wait_flag(peer_flags, me, threadIdx.x, flag_slot, epoch, wait_limit, (5 << 8) | 6);
    __syncthreads();
    for (int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * 256) {
        int lo = 0, hi = n_segments;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (seg_start[mid + 1] > r) hi = mid; else lo = mid + 1;
        }
        long long addr = 0;
        if (r < seg_start[n_segments]) {
            if (lo < n_segments && seg_start[lo] <= r) {
                const int64_t dst = home_base[lo] + (r - seg_start[lo]);
                if (dst >= 0 && dst < capacity) addr = peer_home[lo % n_ranks] + dst * row_bytes;
            }
            if (addr == 0) atomicCAS(&g_moe_status, 0, (5 << 8) | 4);
        }
        row_dst[r] = addr;
    }
}

int p2p_row_table_wait(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
                       int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity, long long* row_dst,
                       const int64_t* peer_flags, int me, int flag_slot, unsigned epoch, cudaStream_t st) {
    CINN_CHECK_ARG(n_rows >= 0 && row_bytes >= 0 && n_segments >= 1 && n_ranks >= 1 && n_ranks <= 64 && capacity >= 0 &&
                   me >= 0 && me < n_ranks && flag_slot >= 0, "p2p_row_table_wait: bad shape");
    CINN_CHECK_ARG(seg_start && home_base && peer_home && peer_flags && (row_dst || n_rows == 0), "p2p_row_table_wait: null pointer");
    CINN_CHECK_ARG(row_bytes % 16 == 0, "p2p_row_table_wait: the row size (%lld bytes) must be a multiple of 16", (long long)row_bytes);
    int64_t blocks = (n_rows + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    if (blocks < 1) blocks = 1;                                 // the wait happens even when there is no row
    p2p_row_table_wait_kernel<<<(unsigned)blocks, 256, 0, st>>>(seg_start, home_base, peer_home, n_rows, n_segments, n_ranks,
                                                               row_bytes, capacity, row_dst, peer_flags, me, flag_slot, epoch,
                                                               g_p2p_wait_limit.load(std::memory_order_relaxed));
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int p2p_barrier(const int64_t* peer_flags, int me, int n_ranks, unsigned epoch, cudaStream_t st) {
    CINN_CHECK_ARG(peer_flags != nullptr && n_ranks >= 1 && n_ranks <= 64 && me >= 0 && me < n_ranks,
                   "p2p_barrier: 1 <= ranks <= 64 and 0 <= rank < ranks (got %d, %d)", n_ranks, me);
    p2p_barrier_kernel<<<1, 64, 0, st>>>(peer_flags, me, n_ranks, epoch, g_p2p_wait_limit.load(std::memory_order_relaxed));
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// The same addresses as p2p_return_kernel computes, written out as a table (one byte address per row of the
// expert-grouped order, 0 = no destination): the grouped GEMM takes it and stores every finished output row
// straight to its home, so the way home runs under the GEMM instead of after it.
__global__ void __launch_bounds__(256)
p2p_row_table_kernel(const int64_t* __restrict__ seg_start, const int64_t* __restrict__ home_base,
                     const int64_t* __restrict__ peer_home, int64_t n_rows, int n_segments, int n_ranks, int64_t row_bytes,
                     int64_t capacity, long long* __restrict__ row_dst) {
    for (int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * 256) {
        int lo = 0, hi = n_segments;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (seg_start[mid + 1] > r) hi = mid; else lo = mid + 1;
        }
        long long addr = 0;
        if (r < seg_start[n_segments]) {                      // rows past the last segment hold no data: no destination
            if (lo < n_segments && seg_start[lo] <= r) {
                const int64_t dst = home_base[lo] + (r - seg_start[lo]);
                if (dst >= 0 && dst < capacity) addr = peer_home[lo % n_ranks] + dst * row_bytes;
            }
            if (addr == 0) atomicCAS(&g_moe_status, 0, (5 << 8) | 4);
        }
        row_dst[r] = addr;
    }
}

int p2p_row_table(const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows, int64_t row_bytes,
                  int n_segments, int n_ranks, int64_t capacity, long long* row_dst, cudaStream_t st) {
    CINN_CHECK_ARG(n_rows >= 0 && row_bytes >= 0 && n_segments >= 1 && n_ranks >= 1 && capacity >= 0, "p2p_row_table: bad shape");
    if (n_rows == 0) return CINN_OK;
    CINN_CHECK_ARG(seg_start && home_base && peer_home && row_dst, "p2p_row_table: null pointer");
    CINN_CHECK_ARG(row_bytes % 16 == 0, "p2p_row_table: the row size (%lld bytes) must be a multiple of 16", (long long)row_bytes);
    int64_t blocks = (n_rows + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    p2p_row_table_kernel<<<(unsigned)blocks, 256, 0, st>>>(seg_start, home_base, peer_home, n_rows, n_segments, n_ranks, row_bytes,
                                                          capacity, row_dst);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int p2p_dispatch(const void* q, const float* s, const int64_t* token_indices, const int64_t* sorted_experts,
                 const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_s,
                 int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t ns, int e_local, int n_ranks, int64_t capacity,
                 cudaStream_t st) {
    CINN_CHECK_ARG(n_pairs >= 0 && n_tokens >= 0 && d >= 0 && ns >= 0 && e_local >= 1 && n_ranks >= 1 && capacity >= 0,
                   "p2p_dispatch: bad shape");
    if (n_pairs == 0 || d == 0) return CINN_OK;
    CINN_CHECK_ARG(q && s && token_indices && sorted_experts && base_send && my_start && peer_q && peer_s,
                   "p2p_dispatch: null pointer");
    CINN_CHECK_ARG(d % 16 == 0 && d < (1LL << 31) && ns < (1LL << 31), "p2p_dispatch: the row width (%lld) must be a multiple of 16",
                   (long long)d);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(q) & 15) == 0, "p2p_dispatch: q must be 16-byte aligned");
    int64_t blocks = (n_pairs + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    p2p_dispatch_kernel<false><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)q, s, token_indices, sorted_experts, base_send,
                                                                my_start, peer_q, peer_s, n_pairs, n_tokens, (int)d, (int)ns,
                                                                e_local, n_ranks, capacity);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int p2p_dispatch_signal(const void* q, const float* s, const int64_t* token_indices, const int64_t* sorted_experts,
                        const int64_t* base_send, const int64_t* my_start, const int64_t* peer_q, const int64_t* peer_s,
                        int64_t n_pairs, int64_t n_tokens, int64_t d, int64_t ns, int e_local, int n_ranks, int64_t capacity,
                        const int64_t* peer_flags, int me, int flag_slot, unsigned epoch, unsigned* done, int e_lo, int e_hi,
                        int n_sms, cudaStream_t st) {
    CINN_CHECK_ARG(n_pairs >= 0 && n_tokens >= 0 && d > 0 && ns >= 0 && e_local >= 1 && n_ranks >= 1 && n_ranks <= 64 &&
                   capacity >= 0 && me >= 0 && me < n_ranks && flag_slot >= 0, "p2p_dispatch_signal: bad shape");
    CINN_CHECK_ARG(0 <= e_lo && e_lo < e_hi && e_hi <= e_local,
                   "p2p_dispatch_signal: the local expert range [%d, %d) must lie inside [0, %d)", e_lo, e_hi, e_local);
    CINN_CHECK_ARG(q && s && token_indices && sorted_experts && base_send && my_start && peer_q && peer_s && peer_flags && done,
                   "p2p_dispatch_signal: null pointer");
    CINN_CHECK_ARG(d % 16 == 0 && d < (1LL << 31) && ns < (1LL << 31),
                   "p2p_dispatch_signal: the row width (%lld) must be a multiple of 16", (long long)d);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(q) & 15) == 0, "p2p_dispatch_signal: q must be 16-byte aligned");
    CINN_CHECK_ARG(n_sms >= 0, "p2p_dispatch_signal: negative SM count");
    if (n_sms > 0) {
        // narrow: one CTA of 1024 threads per SM on n_sms SMs; 120 KiB of (unused) dynamic shared memory keeps a
        // second CTA of this kernel off the same SM
        constexpr int kHold = 120 * 1024;
        static thread_local bool configured[64] = {};
        int dev = 0;
        CINN_CHECK_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            CINN_CHECK_CUDA(cudaFuncSetAttribute(p2p_dispatch_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kHold));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
        const int grid = n_sms < sm_count() ? n_sms : sm_count();
        p2p_dispatch_kernel<true><<<(unsigned)grid, 1024, kHold, st>>>((const uint8_t*)q, s, token_indices, sorted_experts,
                                                                      base_send, my_start, peer_q, peer_s, n_pairs, n_tokens,
                                                                      (int)d, (int)ns, e_local, n_ranks, capacity, peer_flags, me,
                                                                      flag_slot, epoch, done, e_lo, e_hi);
        CINN_CHECK_LAUNCH();
        return CINN_OK;
    }
    int64_t blocks = (n_pairs + 7) / 8;                     // with no rows one CTA still signals
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    p2p_dispatch_kernel<true><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)q, s, token_indices, sorted_experts, base_send,
                                                               my_start, peer_q, peer_s, n_pairs, n_tokens, (int)d, (int)ns,
                                                               e_local, n_ranks, capacity, peer_flags, me, flag_slot, epoch, done,
                                                               e_lo, e_hi);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int p2p_return(const void* rows, const int64_t* seg_start, const int64_t* home_base, const int64_t* peer_home, int64_t n_rows,
               int64_t row_bytes, int n_segments, int n_ranks, int64_t capacity, cudaStream_t st) {
    CINN_CHECK_ARG(n_rows >= 0 && row_bytes >= 0 && n_segments >= 1 && n_ranks >= 1 && capacity >= 0, "p2p_return: bad shape");
    if (n_rows == 0 || row_bytes == 0) return CINN_OK;
    CINN_CHECK_ARG(rows && seg_start && home_base && peer_home, "p2p_return: null pointer");
    CINN_CHECK_ARG(row_bytes % 16 == 0 && row_bytes / 16 < (1LL << 31), "p2p_return: the row size (%lld bytes) must be a multiple of 16",
                   (long long)row_bytes);
    CINN_CHECK_ARG((reinterpret_cast<uintptr_t>(rows) & 15) == 0, "p2p_return: rows must be 16-byte aligned");
    int64_t blocks = (n_rows + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    p2p_return_kernel<<<(unsigned)blocks, 256, 0, st>>>((const uint4*)rows, seg_start, home_base, peer_home, n_rows, n_segments,
                                                       n_ranks, (int)(row_bytes / 16), capacity);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// Zero the rows of a (T, row_bytes) buffer that no expert's range [starts[e], ends[e]) covers: the input gradient of
// the grouped GEMM writes every covered row, so only the others need clearing (instead of a fill of the whole
// buffer before the GEMM).  One CTA per 128 rows marks the covered ones in shared memory, then clears the rest.
__global__ void __launch_bounds__(256)
zero_rows_outside_kernel(uint8_t* __restrict__ buf, int64_t T, int64_t row_bytes, const int64_t* __restrict__ starts,
                         const int64_t* __restrict__ ends, int E) {
    __shared__ int covered[128];
    const int64_t r0 = (int64_t)blockIdx.x * 128;
    if (threadIdx.x < 128) covered[threadIdx.x] = 0;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += 256) {
        int64_t s = starts[e], t = ends[e];
        if (s < r0) s = r0;
        if (t > r0 + 128) t = r0 + 128;
        for (int64_t r = s; r < t; ++r) covered[r - r0] = 1;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int rl = warp; rl < 128; rl += 8) {
        const int64_t r = r0 + rl;
        if (r >= T || covered[rl]) continue;
        uint8_t* row = buf + r * row_bytes;
        if ((row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
            for (int64_t v = lane; v < (row_bytes >> 4); v += 32) reinterpret_cast<uint4*>(row)[v] = make_uint4(0, 0, 0, 0);
        } else {
            for (int64_t b = lane; b < row_bytes; b += 32) row[b] = 0;
        }
    }
}

int zero_rows_outside(void* buf, int64_t T, int64_t row_bytes, const int64_t* starts, const int64_t* ends, int64_t E,
                      cudaStream_t st) {
    CINN_CHECK_ARG(T >= 0 && row_bytes >= 0 && E >= 0 && E < (1LL << 31), "zero_rows_outside: negative shape");
    if (T == 0 || row_bytes == 0) return CINN_OK;
    CINN_CHECK_ARG(buf && (E == 0 || (starts && ends)), "zero_rows_outside: null pointer");
    const int64_t blocks = (T + 127) / 128;
    CINN_CHECK_ARG(blocks < (1LL << 31), "zero_rows_outside: too many rows");
    zero_rows_outside_kernel<<<(unsigned)blocks, 256, 0, st>>>((uint8_t*)buf, T, row_bytes, starts, ends, (int)E);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int moe_combine_backward(const void* rows, int dtype, const int64_t* pos, const float* gates, const float* dy, void* d_rows,
                         float* d_gates, int64_t n_tokens, int64_t n_rows, int top_k, int64_t d, cudaStream_t st) {
    CINN_CHECK_ARG(n_tokens >= 0 && n_rows >= 0 && d >= 0, "moe_combine_backward: negative shape");
    if (n_tokens == 0 || d == 0) return CINN_OK;
    CINN_CHECK_ARG(rows && pos && gates && dy && d_rows && d_gates, "moe_combine_backward: null pointer");
    CINN_CHECK_ARG(top_k >= 1 && top_k <= kMaxTopK, "moe_combine_backward: top_k must be in [1, %d]", kMaxTopK);
    CINN_CHECK_ARG(d % 8 == 0 && d < (1LL << 31), "moe_combine_backward: the row width (%lld) must be a multiple of 8", (long long)d);
    CINN_CHECK_ARG(((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(d_rows)) & 15) == 0,
                   "moe_combine_backward: rows, dy and d_rows must be 16-byte aligned");
    const int64_t n_pairs = n_tokens * top_k;
    int64_t blocks = (n_pairs + 7) / 8;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    switch (dtype) {
        case CINN_BF16: moe_combine_backward_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)rows, pos, gates, dy, (__nv_bfloat16*)d_rows, d_gates, n_pairs, n_rows, top_k, (int)d); break;
        case CINN_F16: moe_combine_backward_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half*)rows, pos, gates, dy, (__half*)d_rows, d_gates, n_pairs, n_rows, top_k, (int)d); break;
        case CINN_F32: moe_combine_backward_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)rows, pos, gates, dy, (float*)d_rows, d_gates, n_pairs, n_rows, top_k, (int)d); break;
        default: set_error("moe_combine_backward: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int read_moe_status(int* out, int reset) {
    int v = 0;
    CINN_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_moe_status, sizeof(int)));
    if (reset && v != 0) {
        int z = 0;
        CINN_CHECK_CUDA(cudaMemcpyToSymbol(g_moe_status, &z, sizeof(int)));
    }
    *out = v;
    return CINN_OK;
}

}  // namespace cinn
