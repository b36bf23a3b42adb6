// Lightning indexer logits: I[b, t, s] = sum_h relu(q[b, t, h, :] . k[b, s, :]) * w[b, t, h], fp16 result.
//
// Semantics of cinnamon's lightning_indexer_kernel / lightning_indexer_fused (src/kernels.py:321-433): the
// operands of the dot product are rounded to fp16 (:374), products are accumulated in fp32, ReLU and the head
// weights are applied in fp32 (:377), the logits are stored as fp16 (:381).
//
// One CTA: 16 queries x 64 keys.  The key tile is kept transposed in shared memory as fp16 ([d][key], so the 16
// lanes that share a query read 16 consecutive keys), the queries of all heads as fp16 ([query][head][d],
// broadcast reads).  A thread owns one query and four keys: per head a d-long dot product for each of the four,
// then relu * w into the running sum.  The work is tiny next to the GEMMs (d is 64-128, a handful of heads); the
// kernel is bound by writing the (B, Lq, Lk) logits once.
#include "common.cuh"

namespace cinn {

namespace {
template <typename T> __device__ __forceinline__ __half to_half_rn(T v);
template <> __device__ __forceinline__ __half to_half_rn<float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __half to_half_rn<__half>(__half v) { return v; }
template <> __device__ __forceinline__ __half to_half_rn<__nv_bfloat16>(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }
template <typename T> __device__ __forceinline__ float w_to_float(T v);
template <> __device__ __forceinline__ float w_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float w_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float w_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
}  // namespace

constexpr int IDX_TQ = 16, IDX_TK = 64;

template <typename T>
__global__ void __launch_bounds__(256)
indexer_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ w, __half* __restrict__ out,
               int Lq, int Lk, int H, int d, int64_t sqb, int64_t sqq, int64_t sqh, int64_t sqd, int64_t skb, int64_t skk,
               int64_t skd, int64_t swb, int64_t swq, int64_t swh) {
    extern __shared__ __align__(16) unsigned char idx_smem[];
    __half* sK = reinterpret_cast<__half*>(idx_smem);                 // [d][IDX_TK + 2]
    __half* sQ = sK + (size_t)d * (IDX_TK + 2);                       // [IDX_TQ][H][d]
    const int b = blockIdx.z, q0 = blockIdx.y * IDX_TQ, k0 = blockIdx.x * IDX_TK;
    const int tid = threadIdx.x;
    for (int e = tid; e < IDX_TK * d; e += 256) {
        const int kk = e / d, dd = e - kk * d;
        const int s = k0 + kk;
        sK[dd * (IDX_TK + 2) + kk] = s < Lk ? to_half_rn<T>(k[b * skb + s * skk + dd * skd]) : __float2half_rn(0.0f);
    }
    for (int e = tid; e < IDX_TQ * H * d; e += 256) {
        const int dd = e % d, h = (e / d) % H, qq = e / (d * H);
        const int t = q0 + qq;
        sQ[e] = t < Lq ? to_half_rn<T>(q[b * sqb + t * sqq + h * sqh + dd * sqd]) : __float2half_rn(0.0f);
    }
    __syncthreads();
    const int tq = tid >> 4, tk = tid & 15;
    const int t = q0 + tq;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int h = 0; h < H; ++h) {
        float dot[4] = {0.f, 0.f, 0.f, 0.f};
        const __half* qh = sQ + ((size_t)tq * H + h) * d;
        for (int dd = 0; dd < d; ++dd) {
            const float qv = __half2float(qh[dd]);
            const __half* kr = sK + dd * (IDX_TK + 2) + tk;
#pragma unroll
            for (int i = 0; i < 4; ++i) dot[i] = fmaf(qv, __half2float(kr[16 * i]), dot[i]);
        }
        const float wh = t < Lq ? w_to_float<T>(w[b * swb + t * swq + h * swh]) : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(fmaxf(dot[i], 0.0f), wh, acc[i]);
    }
    if (t < Lq) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = k0 + tk + 16 * i;
            if (s < Lk) out[((int64_t)b * Lq + t) * Lk + s] = __float2half_rn(acc[i]);
        }
    }
}

template <typename T>
static int indexer_typed(const T* q, const T* k, const T* w, __half* out, int B, int Lq, int Lk, int H, int d, const int64_t* sq,
                         const int64_t* sk, const int64_t* sw, cudaStream_t st) {
    const size_t smem = ((size_t)d * (IDX_TK + 2) + (size_t)IDX_TQ * H * d) * sizeof(__half);
    CINN_CHECK_ARG(smem <= 160 * 1024, "lightning_indexer: %d heads of width %d need %zu bytes of shared memory (limit 163840)",
                   H, d, smem);
    CINN_CHECK_CUDA(cudaFuncSetAttribute(indexer_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    dim3 grid((unsigned)((Lk + IDX_TK - 1) / IDX_TK), (unsigned)((Lq + IDX_TQ - 1) / IDX_TQ), (unsigned)B);
    CINN_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "lightning_indexer: too many queries or batches");
    indexer_kernel<T><<<grid, 256, smem, st>>>(q, k, w, out, Lq, Lk, H, d, sq[0], sq[1], sq[2], sq[3], sk[0], sk[1], sk[2], sw[0],
                                               sw[1], sw[2]);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int lightning_indexer(const void* q, const void* k, const void* w, int dtype, void* out, int64_t B, int64_t Lq, int64_t Lk,
                      int64_t H, int64_t d, const int64_t* q_strides, const int64_t* k_strides, const int64_t* w_strides,
                      cudaStream_t st) {
    CINN_CHECK_ARG(B >= 0 && Lq >= 0 && Lk >= 0 && H >= 1 && d >= 1, "lightning_indexer: bad shape");
    if (B == 0 || Lq == 0 || Lk == 0) return CINN_OK;
    CINN_CHECK_ARG(q && k && w && out && q_strides && k_strides && w_strides, "lightning_indexer: null pointer");
    CINN_CHECK_ARG(Lq < (1LL << 31) && Lk < (1LL << 31) && H < 4096 && d < 65536, "lightning_indexer: dimension too large");
    switch (dtype) {
        case CINN_BF16: return indexer_typed((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)w, (__half*)out, (int)B, (int)Lq, (int)Lk, (int)H, (int)d, q_strides, k_strides, w_strides, st);
        case CINN_F16: return indexer_typed((const __half*)q, (const __half*)k, (const __half*)w, (__half*)out, (int)B, (int)Lq, (int)Lk, (int)H, (int)d, q_strides, k_strides, w_strides, st);
        case CINN_F32: return indexer_typed((const float*)q, (const float*)k, (const float*)w, (__half*)out, (int)B, (int)Lq, (int)Lk, (int)H, (int)d, q_strides, k_strides, w_strides, st);
        default: set_error("lightning_indexer: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

}  // namespace cinn
