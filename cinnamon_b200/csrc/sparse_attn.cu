// Sparse attention over per-query index lists: O(L * K) gathers instead of an L x L score matrix.
//
// Semantics of cinnamon's sparse_attention_fwd_kernel / sparse_attention_bwd_kernel
// (src/kernels.py:913-1186): for query t of batch b and head h, the keys are k[b, h, idx[b, t, j]] for
// j < K; a key takes part when idx <= t (causal); p = softmax(scale * q.k) over the valid keys (all zero when
// none is valid, lse = 0 then); out = sum_j p_j v[b, h, idx_j]; the probabilities are returned as well.
// Backward: delta = dO.O, dp_j = p_j (dO.v_j - delta), dq = scale * sum_j dp_j k_j,
// dk[idx_j] += scale * dp_j q, dv[idx_j] += p_j dO (fp32 atomics, as in the reference).
//
// One warp per (b, h, t).  The index list, the scores and the fp32 query live in the warp's slice of shared
// memory.  Scores: one lane per key, the key row read with 16-byte loads (rows of one (b, h) are a few hundred
// KiB and stay in L1/L2).  Output and gradients: one lane per pair of feature columns, so every gathered value
// row is read (and every gradient row is updated) with coalesced accesses.
#include "common.cuh"
#include <cmath>

namespace cinn {

namespace {

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

// Part of the dot product of an fp32 vector in shared memory with a row of T in global memory: eight lanes share a
// row, lane l8 of them takes the 16-byte chunks l8, l8 + 8, ... (so the eight lanes read 128 contiguous bytes per
// step), up to four chunks are fetched before any is used.  The caller adds the eight partial sums.
template <typename T>
__device__ __forceinline__ float dot_row_part(const float* __restrict__ qs, const T* __restrict__ row, int D, int l8, bool vec) {
    float acc = 0.0f;
    if (vec) {
        constexpr int PER = 16 / (int)sizeof(T);                // elements per 16-byte load
        const int chunks = D / PER;
        for (int c0 = l8; c0 < chunks; c0 += 32) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + 8 * u;
                raw[u] = c < chunks ? __ldg(reinterpret_cast<const uint4*>(row) + c) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + 8 * u;
                if (c < chunks) {
                    const float* qv = qs + c * PER;
                    if constexpr (sizeof(T) == 4) {
                        const float4 f = *reinterpret_cast<const float4*>(&raw[u]);
                        const float4 q0 = *reinterpret_cast<const float4*>(qv);
                        acc = fmaf(f.x, q0.x, acc); acc = fmaf(f.y, q0.y, acc); acc = fmaf(f.z, q0.z, acc); acc = fmaf(f.w, q0.w, acc);
                    } else {
                        const T* e = reinterpret_cast<const T*>(&raw[u]);
                        const float4 q0 = *reinterpret_cast<const float4*>(qv);
                        const float4 q1 = *reinterpret_cast<const float4*>(qv + 4);
                        float a0 = to_float<T>(e[0]) * q0.x, a1 = to_float<T>(e[1]) * q0.y;
                        a0 = fmaf(to_float<T>(e[2]), q0.z, a0); a1 = fmaf(to_float<T>(e[3]), q0.w, a1);
                        a0 = fmaf(to_float<T>(e[4]), q1.x, a0); a1 = fmaf(to_float<T>(e[5]), q1.y, a1);
                        a0 = fmaf(to_float<T>(e[6]), q1.z, a0); a1 = fmaf(to_float<T>(e[7]), q1.w, a1);
                        acc += a0 + a1;
                    }
                }
            }
        }
    } else {
        for (int d = l8; d < D; d += 8) acc = fmaf(to_float<T>(row[d]), qs[d], acc);
    }
    return acc;
}

// sum over the eight lanes that share a row
__device__ __forceinline__ float group8_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// shared memory of one warp, in floats: K ints (index, -1 = not valid) + K floats (score / probability) + the
// fp32 query; the backward adds K floats (dp) and the fp32 dO row
__host__ __device__ inline size_t pad4(int n) { return (size_t)((n + 3) & ~3); }
__host__ __device__ inline size_t warp_smem_floats(int K, int Dqk, int Dv, bool backward) {
    return backward ? 3 * pad4(K) + pad4(Dqk) + pad4(Dv) : 2 * pad4(K) + pad4(Dqk);
}

}  // namespace

template <typename T>
__global__ void __launch_bounds__(256)
sparse_attn_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       const int64_t* __restrict__ idx, float* __restrict__ out, float* __restrict__ lse,
                       float* __restrict__ attn_w, int B, int H, int L, int K, int Dqk, int Dv, float scale,
                       int warps_per_cta, bool vec_qk) {
    extern __shared__ __align__(16) float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp >= warps_per_cta) return;
    float* base = sm + (size_t)warp * warp_smem_floats(K, Dqk, Dv, false);
    int* s_idx = reinterpret_cast<int*>(base);
    float* s_p = base + pad4(K);
    float* s_q = base + 2 * pad4(K);
    const int64_t n_queries = (int64_t)B * H * L;
    for (int64_t w = (int64_t)blockIdx.x * warps_per_cta + warp; w < n_queries; w += (int64_t)gridDim.x * warps_per_cta) {
        const int t = (int)(w % L);
        const int64_t bh = w / L;
        const int b = (int)(bh / H);
        const T* kb = k + bh * (int64_t)L * Dqk;
        const T* vb = v + bh * (int64_t)L * Dv;
        const T* qrow = q + w * Dqk;
        for (int d = lane; d < Dqk; d += 32) s_q[d] = to_float<T>(qrow[d]);
        const int64_t* irow = idx + ((int64_t)b * L + t) * K;
        for (int j = lane; j < K; j += 32) {
            const int64_t i = irow[j];
            s_idx[j] = (i >= 0 && i <= t) ? (int)i : -1;                 // causal: a key after the query is ignored
        }
        __syncwarp();
        float mx = -INFINITY;
        const int grp = lane >> 3, l8 = lane & 7;                     // four keys per step, eight lanes per key
        for (int j0 = 0; j0 < K; j0 += 4) {
            const int j = j0 + grp;
            const int i = j < K ? s_idx[j] : -1;
            float part = 0.0f;
            if (i >= 0) part = dot_row_part<T>(s_q, kb + (int64_t)i * Dqk, Dqk, l8, vec_qk);
            const float red = group8_sum(part);                       // every lane takes part in the shuffles
            const float sc = i >= 0 ? red * scale : -INFINITY;
            if (l8 == 0 && j < K) s_p[j] = sc;
            mx = fmaxf(mx, sc);
        }
        __syncwarp();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
        for (int j = lane; j < K; j += 32)
            if (s_idx[j] >= 0) sum += expf(s_p[j] - mx);
        sum = warp_sum(sum);
        const bool any = sum > 0.0f;
        const float l = any ? mx + logf(sum) : 0.0f;
        float* aw = attn_w + w * K;
        for (int j = lane; j < K; j += 32) {
            const float p = s_idx[j] >= 0 ? expf(s_p[j] - l) : 0.0f;
            s_p[j] = p;
            aw[j] = p;
        }
        if (lane == 0) lse[w] = l;
        __syncwarp();
        // out[d] = sum_j p_j v[idx_j][d]: lanes own feature columns, the row of every key is read coalesced
        float* orow = out + w * Dv;
        for (int d0 = lane * 2; d0 < Dv; d0 += 64) {
            float a0 = 0.0f, a1 = 0.0f;
            const bool two = d0 + 1 < Dv;
#pragma unroll 8
            for (int j = 0; j < K; ++j) {
                const int i = max(s_idx[j], 0);                         // a key that takes no part has p = 0
                const float p = s_p[j];
                const T* vr = vb + (int64_t)i * Dv + d0;
                a0 = fmaf(p, to_float<T>(vr[0]), a0);
                if (two) a1 = fmaf(p, to_float<T>(vr[1]), a1);
            }
            orow[d0] = a0;
            if (two) orow[d0 + 1] = a1;
        }
        __syncwarp();
    }
}

template <typename T, typename TG>
__global__ void __launch_bounds__(256)
sparse_attn_bwd_kernel(const TG* __restrict__ d_out, const float* __restrict__ out, const float* __restrict__ lse,
                       const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       const int64_t* __restrict__ idx, float* __restrict__ dq, float* __restrict__ dk,
                       float* __restrict__ dv, int B, int H, int L, int K, int Dqk, int Dv, float scale,
                       int warps_per_cta, bool vec_qk, bool vec_v, int atom_qk, int atom_v) {
    // atom_qk / atom_v: widest vector (4, 2 or 1 floats) the gradient buffers' widths AND addresses allow
    extern __shared__ __align__(16) float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp >= warps_per_cta) return;
    float* base = sm + (size_t)warp * warp_smem_floats(K, Dqk, Dv, true);
    int* s_idx = reinterpret_cast<int*>(base);
    float* s_pp = base + pad4(K);                           // probability
    float* s_p = base + 2 * pad4(K);                        // dp
    float* s_q = base + 3 * pad4(K);
    float* s_do = s_q + pad4(Dqk);
    const int64_t n_queries = (int64_t)B * H * L;
    for (int64_t w = (int64_t)blockIdx.x * warps_per_cta + warp; w < n_queries; w += (int64_t)gridDim.x * warps_per_cta) {
        const int t = (int)(w % L);
        const int64_t bh = w / L;
        const int b = (int)(bh / H);
        const T* kb = k + bh * (int64_t)L * Dqk;
        const T* vb = v + bh * (int64_t)L * Dv;
        float* dkb = dk + bh * (int64_t)L * Dqk;
        float* dvb = dv + bh * (int64_t)L * Dv;
        const T* qrow = q + w * Dqk;
        for (int d = lane; d < Dqk; d += 32) s_q[d] = to_float<T>(qrow[d]);
        float delta = 0.0f;
        for (int d = lane; d < Dv; d += 32) {
            const float g = to_float<TG>(d_out[w * Dv + d]);
            s_do[d] = g;
            delta = fmaf(g, out[w * Dv + d], delta);
        }
        delta = warp_sum(delta);
        const int64_t* irow = idx + ((int64_t)b * L + t) * K;
        for (int j = lane; j < K; j += 32) {
            const int64_t i = irow[j];
            s_idx[j] = (i >= 0 && i <= t) ? (int)i : -1;
        }
        __syncwarp();
        const float l = lse[w];
        const int grp = lane >> 3, l8 = lane & 7;                     // four keys per step, eight lanes per key
        for (int j0 = 0; j0 < K; j0 += 4) {
            const int j = j0 + grp;
            const int i = j < K ? s_idx[j] : -1;
            float qk = 0.0f, dov = 0.0f;
            if (i >= 0) {
                qk = dot_row_part<T>(s_q, kb + (int64_t)i * Dqk, Dqk, l8, vec_qk);
                dov = dot_row_part<T>(s_do, vb + (int64_t)i * Dv, Dv, l8, vec_v);
            }
            qk = group8_sum(qk);
            dov = group8_sum(dov);
            if (l8 == 0 && j < K) {
                const float p = i >= 0 ? expf(qk * scale - l) : 0.0f;
                s_pp[j] = p;
                s_p[j] = p * (dov - delta);
            }
        }
        __syncwarp();
        // dq[d] = scale * sum_j dp_j k_j[d];  dk[idx_j][d] += scale * dp_j q[d]
        const bool pair_qk = atom_qk >= 2, pair_v = atom_v >= 2;         // 8-byte aligned float2 atomics
        const bool quad_qk = atom_qk >= 4, quad_v = atom_v >= 4;         // one 16-byte atomic per lane and key
        if (quad_qk) {
            for (int d0 = lane * 4; d0 < Dqk; d0 += 128) {
                float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const float4 qv = *reinterpret_cast<const float4*>(s_q + d0);
                for (int j = 0; j < K; ++j) {
                    const int i = s_idx[j];
                    if (i < 0) continue;
                    const float dp = s_p[j] * scale;
                    const T* kr = kb + (int64_t)i * Dqk + d0;
#pragma unroll
                    for (int c = 0; c < 4; ++c) a[c] = fmaf(dp, to_float<T>(kr[c]), a[c]);
                    atomicAdd(reinterpret_cast<float4*>(dkb + (int64_t)i * Dqk + d0), make_float4(dp * qv.x, dp * qv.y, dp * qv.z, dp * qv.w));
                }
                *reinterpret_cast<float4*>(dq + w * Dqk + d0) = make_float4(a[0], a[1], a[2], a[3]);
            }
        } else
        for (int d0 = lane * 2; d0 < Dqk; d0 += 64) {
            float a0 = 0.0f, a1 = 0.0f;
            const bool two = d0 + 1 < Dqk;
            const float q0 = s_q[d0], q1 = two ? s_q[d0 + 1] : 0.0f;
            for (int j = 0; j < K; ++j) {
                const int i = s_idx[j];
                if (i < 0) continue;
                const float dp = s_p[j] * scale;
                const T* kr = kb + (int64_t)i * Dqk + d0;
                float* dst = dkb + (int64_t)i * Dqk + d0;
                a0 = fmaf(dp, to_float<T>(kr[0]), a0);
                if (two) a1 = fmaf(dp, to_float<T>(kr[1]), a1);
                if (pair_qk) {
                    atomicAdd(reinterpret_cast<float2*>(dst), make_float2(dp * q0, dp * q1));
                } else {
                    atomicAdd(dst, dp * q0);
                    if (two) atomicAdd(dst + 1, dp * q1);
                }
            }
            dq[w * Dqk + d0] = a0;
            if (two) dq[w * Dqk + d0 + 1] = a1;
        }
        // dv[idx_j][d] += p_j dO[d]
        if (quad_v) {
            for (int d0 = lane * 4; d0 < Dv; d0 += 128) {
                const float4 gv = *reinterpret_cast<const float4*>(s_do + d0);
                for (int j = 0; j < K; ++j) {
                    const int i = s_idx[j];
                    if (i < 0) continue;
                    const float p = s_pp[j];
                    atomicAdd(reinterpret_cast<float4*>(dvb + (int64_t)i * Dv + d0), make_float4(p * gv.x, p * gv.y, p * gv.z, p * gv.w));
                }
            }
        } else
        for (int d0 = lane * 2; d0 < Dv; d0 += 64) {
            const bool two = d0 + 1 < Dv;
            const float g0 = s_do[d0], g1 = two ? s_do[d0 + 1] : 0.0f;
            for (int j = 0; j < K; ++j) {
                const int i = s_idx[j];
                if (i < 0) continue;
                const float p = s_pp[j];
                float* dst = dvb + (int64_t)i * Dv + d0;
                if (pair_v) {
                    atomicAdd(reinterpret_cast<float2*>(dst), make_float2(p * g0, p * g1));
                } else {
                    atomicAdd(dst, p * g0);
                    if (two) atomicAdd(dst + 1, p * g1);
                }
            }
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
constexpr size_t SPARSE_SMEM_LIMIT = 96 * 1024;

static int sparse_launch_shape(int K, int Dqk, int Dv, bool backward, int64_t n_queries, int* warps, unsigned* grid, size_t* smem) {
    const size_t per_warp = warp_smem_floats(K, Dqk, Dv, backward) * sizeof(float);
    CINN_CHECK_ARG(per_warp <= SPARSE_SMEM_LIMIT, "sparse_attention: %d indices per query with %d + %d features need %zu bytes "
                   "of shared memory per warp (limit %zu)", K, Dqk, Dv, per_warp, SPARSE_SMEM_LIMIT);
    int w = (int)(SPARSE_SMEM_LIMIT / per_warp);
    if (w > 8) w = 8;
    int64_t g = (n_queries + w - 1) / w;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (g > cap) g = cap;
    *warps = w; *grid = (unsigned)g; *smem = per_warp * w;
    return CINN_OK;
}

template <typename K>
static int allow_smem(K kern) {
    CINN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SPARSE_SMEM_LIMIT));
    return CINN_OK;
}

static int check_sparse_args(int64_t B, int64_t H, int64_t L, int64_t K, int64_t Dqk, int64_t Dv) {
    CINN_CHECK_ARG(B >= 0 && H >= 0 && L >= 0 && K >= 0 && Dqk >= 1 && Dv >= 1, "sparse_attention: bad shape");
    CINN_CHECK_ARG(L < (1LL << 31) && K < (1LL << 24) && Dqk < (1LL << 16) && Dv < (1LL << 16) && B * H < (1LL << 31),
                   "sparse_attention: dimension too large");
    return CINN_OK;
}

template <typename T>
static int sparse_fwd_typed(const T* q, const T* k, const T* v, const int64_t* idx, float* out, float* lse, float* attn_w,
                            int B, int H, int L, int K, int Dqk, int Dv, float scale, cudaStream_t st) {
    int warps; unsigned grid; size_t smem;
    int rc = sparse_launch_shape(K, Dqk, Dv, false, (int64_t)B * H * L, &warps, &grid, &smem);
    if (rc) return rc;
    rc = allow_smem(sparse_attn_fwd_kernel<T>);
    if (rc) return rc;
    const bool vec_qk = (Dqk * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0;
    sparse_attn_fwd_kernel<T><<<grid, 256, smem, st>>>(q, k, v, idx, out, lse, attn_w, B, H, L, K, Dqk, Dv, scale, warps, vec_qk);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int sparse_attn_fwd(const void* q, const void* k, const void* v, int dtype, const int64_t* idx, float* out, float* lse,
                    float* attn_w, int64_t B, int64_t H, int64_t L, int64_t K, int64_t Dqk, int64_t Dv, float scale,
                    cudaStream_t st) {
    int rc = check_sparse_args(B, H, L, K, Dqk, Dv);
    if (rc) return rc;
    if (B * H * L == 0) return CINN_OK;
    CINN_CHECK_ARG(q && k && v && out && lse && (K == 0 || (idx && attn_w)), "sparse_attention: null pointer");
    switch (dtype) {
        case CINN_BF16: return sparse_fwd_typed((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, idx, out, lse, attn_w, (int)B, (int)H, (int)L, (int)K, (int)Dqk, (int)Dv, scale, st);
        case CINN_F16: return sparse_fwd_typed((const __half*)q, (const __half*)k, (const __half*)v, idx, out, lse, attn_w, (int)B, (int)H, (int)L, (int)K, (int)Dqk, (int)Dv, scale, st);
        case CINN_F32: return sparse_fwd_typed((const float*)q, (const float*)k, (const float*)v, idx, out, lse, attn_w, (int)B, (int)H, (int)L, (int)K, (int)Dqk, (int)Dv, scale, st);
        default: set_error("sparse_attention: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

template <typename T, typename TG>
static int sparse_bwd_typed(const TG* d_out, const float* out, const float* lse, const T* q, const T* k, const T* v,
                            const int64_t* idx, float* dq, float* dk, float* dv, int B, int H, int L, int K, int Dqk, int Dv,
                            float scale, cudaStream_t st) {
    int warps; unsigned grid; size_t smem;
    int rc = sparse_launch_shape(K, Dqk, Dv, true, (int64_t)B * H * L, &warps, &grid, &smem);
    if (rc) return rc;
    rc = allow_smem(sparse_attn_bwd_kernel<T, TG>);
    if (rc) return rc;
    const bool vec_qk = (Dqk * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0;
    const bool vec_v = (Dv * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(v) & 15) == 0;
    // 16- and 8-byte atomics and stores need rows that start on such boundaries: width and base address both
    auto widest = [](int D, const void* a, const void* b) {
        const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
        if ((D & 3) == 0 && (bits & 15) == 0) return 4;
        if ((D & 1) == 0 && (bits & 7) == 0) return 2;
        return 1;
    };
    sparse_attn_bwd_kernel<T, TG><<<grid, 256, smem, st>>>(d_out, out, lse, q, k, v, idx, dq, dk, dv, B, H, L, K, Dqk, Dv, scale,
                                                         warps, vec_qk, vec_v, widest(Dqk, dk, dq), widest(Dv, dv, dv));
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// dq is written; dk and dv are ACCUMULATED into (the caller zeroes them, as the reference does, :1257-1259)
int sparse_attn_bwd(const void* d_out, int grad_dtype, const float* out, const float* lse, const void* q, const void* k,
                    const void* v, int dtype, const int64_t* idx, float* dq, float* dk, float* dv, int64_t B, int64_t H,
                    int64_t L, int64_t K, int64_t Dqk, int64_t Dv, float scale, cudaStream_t st) {
    int rc = check_sparse_args(B, H, L, K, Dqk, Dv);
    if (rc) return rc;
    if (B * H * L == 0) return CINN_OK;
    CINN_CHECK_ARG(d_out && out && lse && q && k && v && dq && dk && dv && (K == 0 || idx), "sparse_attention: null pointer");
    CINN_CHECK_ARG(grad_dtype == dtype || grad_dtype == CINN_F32, "sparse_attention: the output gradient must have the inputs' "
                   "type or be fp32 (tags %d, %d)", grad_dtype, dtype);
#define CINN_SB(T, TG) sparse_bwd_typed((const TG*)d_out, out, lse, (const T*)q, (const T*)k, (const T*)v, idx, dq, dk, dv, (int)B, \
                                        (int)H, (int)L, (int)K, (int)Dqk, (int)Dv, scale, st)
    switch (dtype) {
        case CINN_BF16: return grad_dtype == CINN_F32 ? CINN_SB(__nv_bfloat16, float) : CINN_SB(__nv_bfloat16, __nv_bfloat16);
        case CINN_F16: return grad_dtype == CINN_F32 ? CINN_SB(__half, float) : CINN_SB(__half, __half);
        case CINN_F32: return CINN_SB(float, float);
        default: set_error("sparse_attention: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
#undef CINN_SB
}

}  // namespace cinn
