// FP8 (e4m3) quantisers and de-quantisers: HBM-bound amax / scale / cast passes.
//
// Arithmetic follows cinnamon's Triton kernels (src/kernels.py:41-71 row-wise,
// :97-132 block-wise, :149-173 block de-quantise, :262-281 row-wise
// de-quantise): amax over the tile with masked elements counted as 0, floor
// 1e-4, scale = amax/448 (or the next power of two), q = clamp(x/scale) -> e4m3.
// The division flavour is a template parameter: div.full.f32 is what Triton
// emits for those kernels on a GPU, IEEE division is what a CPU computes.
//
// Layout: every kernel moves 16-byte vectors per lane where alignment allows,
// reduces amax with warp shuffles, and writes packed e4m3 (4-16 bytes per lane).
#include "common.cuh"
#include "tma.cuh"
#include <type_traits>
#include <mutex>

namespace cinn {

// ---------------------------------------------------------------------------
// typed 8-element / 4-element vector loads, widened to fp32
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 r = *reinterpret_cast<const uint4*>(p);
        uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
        uint2 r = *reinterpret_cast<const uint2*>(p);
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
    }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
        uint4 r = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
        uint2 r = *reinterpret_cast<const uint2*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&r);
        float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
};
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
        float4 a = *reinterpret_cast<const float4*>(p);
        float4 b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
        float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
};

// ---------------------------------------------------------------------------
// Row-wise 1x128, contiguous rows, vector path.
// A half-warp owns one tile (16 lanes x 8 elements).  Each thread keeps UNROLL tiles per
// round and fetches the raw vectors of the next round before it converts the current one,
// so loads stay in flight during the arithmetic.  Tile coordinates advance incrementally
// (no division in the loop).
// ---------------------------------------------------------------------------
template <typename T> struct Raw8 { uint4 a; };
template <> struct Raw8<float> { float4 a, b; };

template <typename T>
__device__ __forceinline__ Raw8<T> load_raw8(const T* p) {
    Raw8<T> r;
    if constexpr (sizeof(T) == 4) {
        r.a = __ldcs(reinterpret_cast<const float4*>(p));
        r.b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    } else {
        r.a = __ldcs(reinterpret_cast<const uint4*>(p));
    }
    return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> zero_raw8() {
    Raw8<T> r;
    if constexpr (sizeof(T) == 4) { r.a = make_float4(0.f, 0.f, 0.f, 0.f); r.b = r.a; }
    else r.a = make_uint4(0u, 0u, 0u, 0u);
    return r;
}
template <typename T>
__device__ __forceinline__ void unpack_raw8(const Raw8<T>& r, float (&v)[8]) {
    if constexpr (sizeof(T) == 4) {
        v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    } else {
        const __half2* h = reinterpret_cast<const __half2*>(&r.a);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
}

template <typename T, int DIV, bool ROUND, int UNROLL>
__global__ void __launch_bounds__(256)
quant_row_vec_kernel(const T* __restrict__ x, int64_t ld, uint8_t* __restrict__ q, float* __restrict__ scales,
                     int N, int nb, int64_t total_tiles, int step_rows, int step_cols) {
    // the n-th tile of this half-warp is hw + n * n_hw; (step_rows, step_cols) = divmod(n_hw, nb)
    const int sub = threadIdx.x & 15;
    const int64_t hw = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);
    const int64_t n_hw = (int64_t)gridDim.x * 16;
    int64_t t = hw;                                  // this half-warp's next tile to FETCH
    int row = (int)(hw / nb);
    int cb = (int)(hw - (int64_t)row * nb);
    int64_t tw = hw & ~(int64_t)1;                   // warp-uniform loop variable

    Raw8<T> nxt[UNROLL];
    int64_t nxt_off[UNROLL];                         // output offset row * N + col, or -1
    int64_t nxt_tile[UNROLL];
    auto fetch = [&]() {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int col = cb * 128 + sub * 8;
            const bool live = t < total_tiles;
            const bool inb = live && col < N;
            nxt[u] = inb ? load_raw8<T>(x + (int64_t)row * ld + col) : zero_raw8<T>();
            nxt_off[u] = inb ? (int64_t)row * N + col : -1;
            nxt_tile[u] = live ? t : -1;
            t += n_hw;
            row += step_rows;
            cb += step_cols;
            if (cb >= nb) { cb -= nb; row += 1; }
        }
    };
    fetch();
    for (; tw < total_tiles; tw += n_hw * UNROLL) {
        Raw8<T> cur[UNROLL];
        int64_t off[UNROLL], tile[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) { cur[u] = nxt[u]; off[u] = nxt_off[u]; tile[u] = nxt_tile[u]; }
        if (tw + n_hw * UNROLL < total_tiles) fetch();
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float v[8];
            unpack_raw8<T>(cur[u], v);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float s = scale_from_amax<DIV, ROUND>(amax);
            const float d = divisor_of<DIV>(s);
            float y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = scaled_clamped<DIV>(v[i], d);
            if (off[u] >= 0) {
                uint2 o2;
                o2.x = cvt_e4m3x4(y[0], y[1], y[2], y[3]);
                o2.y = cvt_e4m3x4(y[4], y[5], y[6], y[7]);
                __stcs(reinterpret_cast<uint2*>(q + off[u]), o2);
            }
            if (sub == 0 && tile[u] >= 0) scales[tile[u]] = s;
        }
    }
}

// ---------------------------------------------------------------------------
// Row-wise, arbitrary strides / ragged sizes / any tile length: one warp per tile.
// ---------------------------------------------------------------------------
template <typename T, int DIV, bool ROUND>
__global__ void __launch_bounds__(256)
quant_row_generic_kernel(const T* __restrict__ x, int64_t ld_m, int64_t ld_n, uint8_t* __restrict__ q,
                         float* __restrict__ scales, int N, int nb, int block, int64_t total_tiles) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 8;
    for (int64_t t = warp; t < total_tiles; t += n_warps) {
        const int64_t row = t / nb;
        const int c0 = (int)(t - row * nb) * block;
        const int c1 = min(c0 + block, N);
        float amax = 0.0f;
        for (int c = c0 + lane; c < c1; c += 32) amax = fmaxf(amax, fabsf(Elem<T>::to_f(x[row * ld_m + c * ld_n])));
        amax = warp_max(amax);
        const float s = scale_from_amax<DIV, ROUND>(amax);
        const float d = divisor_of<DIV>(s);
        for (int c = c0 + lane; c < c1; c += 32) {
            const float y = scaled_clamped<DIV>(Elem<T>::to_f(x[row * ld_m + c * ld_n]), d);
            q[row * (int64_t)N + c] = (uint8_t)(cvt_e4m3x2(y, 0.0f) & 0xff);
        }
        if (lane == 0) scales[t] = s;
    }
}

// ---------------------------------------------------------------------------
// Row-wise 1x128 over a TRANSPOSED view: logical x is (M, N) with element
// (m, n) at x[m + n * L], i.e. the tile axis n is the strided one.  This is
// what the weight-gradient path needs (tiles along tokens of dy^T,
// src/kernels.py:781-783) without first materialising the transpose.
// One CTA: 64 logical rows (contiguous in memory) x one 128-wide tile.
// ---------------------------------------------------------------------------
// SEG: the tile axis is cut into per-expert segments, each padded to whole tiles: tile cb reads tile_cnt[cb] source
// positions starting at tile_src[cb] (the rest of the tile counts as zeros) and only the first *n_tiles tiles exist
// (`nb` is then the capacity of the output along the tile axis, in tiles).  One launch quantises dY^T of every expert
// for the grouped weight gradient, with tiles that never straddle two experts.
template <typename T, int DIV, bool ROUND, bool SEG = false>
__global__ void __launch_bounds__(256, 3)
quant_row_transposed_kernel(const T* __restrict__ x, int64_t L, uint8_t* __restrict__ q,
                            float* __restrict__ scales, int M, int N, int nb, int tiles_per_cta, int N_in,
                            const int* __restrict__ tile_src = nullptr, const int* __restrict__ tile_cnt = nullptr,
                            const int* __restrict__ n_tiles = nullptr) {
    // N_in <= N: only the first N_in positions along the tile axis are read, the rest count as zeros (a ragged
    // expert range padded to a multiple of 16 without a padded copy of the input)
    constexpr int TM = 64;            // logical rows per CTA
    __shared__ __align__(16) float s_amax[2][8][TM];
    // staged output: 64 logical rows x 128 bytes; the 16-byte chunk index of a row is XOR-ed
    // with (row / 8) so that the 4-byte stores of a warp fall into 32 different banks
    __shared__ __align__(16) uint32_t s_out[2][TM * 32];

    // blockIdx.x runs along m: CTAs that are scheduled together read neighbouring 128-byte pieces of the
    // same memory rows, which keeps DRAM pages open
    const int m0 = blockIdx.x * TM;
    const int g = threadIdx.x & 7;              // which 8-wide m chunk
    const int nr = threadIdx.x >> 3;            // 0..31: this thread reads n rows 4*nr .. 4*nr+3
    const int warp = threadIdx.x >> 5;
    const int m = m0 + g * 8;
    const int cb_first = blockIdx.y * tiles_per_cta;
    const int cb_last = min(cb_first + tiles_per_cta, SEG ? min(nb, *n_tiles) : nb);

    // raw vectors of the next tile are fetched before the current one is converted
    Raw8<T> nxt[4];
    auto fetch = [&](int cb) {
        int src0 = cb * 128, cnt = N_in - cb * 128;
        if constexpr (SEG) {
            if (cb < cb_last) { src0 = tile_src[cb]; cnt = tile_cnt[cb]; }
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int j = nr * 4 + p;
            nxt[p] = (cb < cb_last && j < cnt && m < M) ? load_raw8<T>(x + (int64_t)(src0 + j) * L + m) : zero_raw8<T>();
        }
    };
    fetch(cb_first);
    for (int cb = cb_first, buf = 0; cb < cb_last; ++cb, buf ^= 1) {
        const int n0 = cb * 128;
        float v[4][8];
#pragma unroll
        for (int p = 0; p < 4; ++p) unpack_raw8<T>(nxt[p], v[p]);
        fetch(cb + 1);
        float am[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float a = fmaxf(fmaxf(fabsf(v[0][i]), fabsf(v[1][i])), fmaxf(fabsf(v[2][i]), fabsf(v[3][i])));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
            am[i] = a;
        }
        if ((threadIdx.x & 31) < 8) {
            *reinterpret_cast<float4*>(&s_amax[buf][warp][g * 8]) = make_float4(am[0], am[1], am[2], am[3]);
            *reinterpret_cast<float4*>(&s_amax[buf][warp][g * 8 + 4]) = make_float4(am[4], am[5], am[6], am[7]);
        }
        __syncthreads();                        // (also: everyone is done reading s_out[buf] of two tiles ago)
        float sc[8], dv[8];
        {
            // the eight warps' partial maxima of this thread's eight rows: sixteen 16-byte reads instead of 64 scalar ones
            float4 lo = *reinterpret_cast<const float4*>(&s_amax[buf][0][g * 8]);
            float4 hi = *reinterpret_cast<const float4*>(&s_amax[buf][0][g * 8 + 4]);
#pragma unroll
            for (int w = 1; w < 8; ++w) {
                const float4 a = *reinterpret_cast<const float4*>(&s_amax[buf][w][g * 8]);
                const float4 b = *reinterpret_cast<const float4*>(&s_amax[buf][w][g * 8 + 4]);
                lo.x = fmaxf(lo.x, a.x); lo.y = fmaxf(lo.y, a.y); lo.z = fmaxf(lo.z, a.z); lo.w = fmaxf(lo.w, a.w);
                hi.x = fmaxf(hi.x, b.x); hi.y = fmaxf(hi.y, b.y); hi.z = fmaxf(hi.z, b.z); hi.w = fmaxf(hi.w, b.w);
            }
            const float mx[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sc[i] = scale_from_amax<DIV, ROUND>(mx[i]);
                dv[i] = divisor_of<DIV>(sc[i]);
            }
        }
        if (nr == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (m + i < M) scales[(int64_t)(m + i) * nb + cb] = sc[i];
        }
        // four consecutive n of one logical row -> one 32-bit word
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t word = cvt_e4m3x4(scaled_clamped<DIV>(v[0][i], dv[i]), scaled_clamped<DIV>(v[1][i], dv[i]),
                                             scaled_clamped<DIV>(v[2][i], dv[i]), scaled_clamped<DIV>(v[3][i], dv[i]));
            const int ml = g * 8 + i;
            s_out[buf][ml * 32 + ((((nr >> 2) ^ g) & 7) << 2) + (nr & 3)] = word;
        }
        __syncthreads();
        // 64 rows x 8 chunks of 16 bytes
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int ml = idx >> 3, ch = idx & 7;
            const int mm = m0 + ml, n = n0 + ch * 16;
            if (mm < M && n < N) {
                const uint4 val = *reinterpret_cast<const uint4*>(&s_out[buf][ml * 32 + (((ch ^ (ml >> 3)) & 7) << 2)]);
                __stcs(reinterpret_cast<uint4*>(q + (int64_t)mm * N + n), val);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Both 1x128 quantisations of one matrix in a single pass: tiles along n (what the input
// gradient needs, src/kernels.py:771) and tiles along m of the transpose (what the weight
// gradient needs, src/kernels.py:781-783).  One CTA holds a 128 x 128 piece in registers:
// thread (hw, sub) keeps rows hw*8 .. +7 and columns sub*8 .. +7, so a row tile is reduced
// inside a half-warp and a column tile across the 16 half-warps (one shuffle + shared memory).
// The transposed bytes leave through a 16 KiB staging tile whose 16-byte chunks are XOR-ed
// with (n / 8) so that the 8-byte stores of a warp spread over all banks.
// ---------------------------------------------------------------------------
// One 128 x 128 piece held as v[i][j] = x[mt + i][n + j].  `ok` is this thread's verdict on its input (a
// bounded wait that ran out makes it false); the CTA leaves together when any thread says so.  `after_sync`
// runs once every thread has taken its input out of shared memory.
// SEG: the piece is tile `bm` of a token axis cut into per-expert segments that are padded to whole tiles: its rows
// are the `cnt` source rows from `src0` on (the row-wise bytes and scales go to those rows; the rest of the piece
// counts as zeros), while the transposed bytes and their scales go to the padded position `bm` of an output whose
// token axis is `M` long (`nb_m` tiles).
template <int DIV, bool ROUND, bool SEG = false, typename AfterSync>
__device__ __forceinline__ bool dual_tile(float (&v)[8][8], float (*s_amax)[128], uint8_t* s_out, bool ok,
                                          uint8_t* __restrict__ q_row, float* __restrict__ s_row,
                                          uint8_t* __restrict__ q_col, float* __restrict__ s_col, int M, int N, int nb_n,
                                          int nb_m, int bm, int bn, AfterSync&& after_sync, int src0 = 0, int cnt = 128) {
    const int sub = threadIdx.x & 15, hw = threadIdx.x >> 4, warp = threadIdx.x >> 5;
    const int m0 = bm * 128, n0 = bn * 128;
    const int n = n0 + sub * 8;
    const int mt = SEG ? src0 + hw * 8 : m0 + hw * 8;          // first row of this thread's row-wise outputs
    const int m_rows = SEG ? src0 + cnt : M;                    // one past the last row that is written row-wise
    if constexpr (SEG) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (hw * 8 + i >= cnt) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
            }
    }

    // column tiles first: their reduction needs the barrier, the row tiles fill the wait
    float cam[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float a = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(v[i][j]));
        cam[j] = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
    }
    if ((threadIdx.x & 31) < 16) {
        *reinterpret_cast<float4*>(&s_amax[warp][sub * 8]) = make_float4(cam[0], cam[1], cam[2], cam[3]);
        *reinterpret_cast<float4*>(&s_amax[warp][sub * 8 + 4]) = make_float4(cam[4], cam[5], cam[6], cam[7]);
    }
    if (!__syncthreads_and(ok)) return false;
    after_sync();

    // row tiles: amax inside the half-warp, bytes straight to global memory
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaxf(a, fabsf(v[i][j]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        const float s = scale_from_amax<DIV, ROUND>(a);
        const float d = divisor_of<DIV>(s);
        if (mt + i < m_rows && n < N) {
            uint2 o2;
            o2.x = cvt_e4m3x4(scaled_clamped<DIV>(v[i][0], d), scaled_clamped<DIV>(v[i][1], d),
                              scaled_clamped<DIV>(v[i][2], d), scaled_clamped<DIV>(v[i][3], d));
            o2.y = cvt_e4m3x4(scaled_clamped<DIV>(v[i][4], d), scaled_clamped<DIV>(v[i][5], d),
                              scaled_clamped<DIV>(v[i][6], d), scaled_clamped<DIV>(v[i][7], d));
            __stcs(reinterpret_cast<uint2*>(q_row + (int64_t)(mt + i) * N + n), o2);
            if (sub == 0) s_row[(int64_t)(mt + i) * nb_n + bn] = s;
        }
    }

    // column tiles: every half-warp derives the same 8 scales for its columns
    float sc[8], dv[8];
    {
        float4 lo = *reinterpret_cast<const float4*>(&s_amax[0][sub * 8]);
        float4 hi = *reinterpret_cast<const float4*>(&s_amax[0][sub * 8 + 4]);
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            const float4 a = *reinterpret_cast<const float4*>(&s_amax[w][sub * 8]);
            const float4 b = *reinterpret_cast<const float4*>(&s_amax[w][sub * 8 + 4]);
            lo.x = fmaxf(lo.x, a.x); lo.y = fmaxf(lo.y, a.y); lo.z = fmaxf(lo.z, a.z); lo.w = fmaxf(lo.w, a.w);
            hi.x = fmaxf(hi.x, b.x); hi.y = fmaxf(hi.y, b.y); hi.z = fmaxf(hi.z, b.z); hi.w = fmaxf(hi.w, b.w);
        }
        const float am[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) { sc[j] = scale_from_amax<DIV, ROUND>(am[j]); dv[j] = divisor_of<DIV>(sc[j]); }
    }
    if (hw == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (n + j < N) s_col[(int64_t)(n + j) * nb_m + bm] = sc[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint2 o2;
        o2.x = cvt_e4m3x4(scaled_clamped<DIV>(v[0][j], dv[j]), scaled_clamped<DIV>(v[1][j], dv[j]),
                          scaled_clamped<DIV>(v[2][j], dv[j]), scaled_clamped<DIV>(v[3][j], dv[j]));
        o2.y = cvt_e4m3x4(scaled_clamped<DIV>(v[4][j], dv[j]), scaled_clamped<DIV>(v[5][j], dv[j]),
                          scaled_clamped<DIV>(v[6][j], dv[j]), scaled_clamped<DIV>(v[7][j], dv[j]));
        const int nl = sub * 8 + j;
        *reinterpret_cast<uint2*>(&s_out[nl * 128 + ((((hw >> 1) ^ sub) & 7) << 4) + ((hw & 1) << 3)]) = o2;
    }
    __syncthreads();
    // 128 transposed rows x 8 chunks of 16 bytes (16 consecutive m)
#pragma unroll
    for (int rep = 0; rep < 4; ++rep) {
        const int idx = threadIdx.x + rep * 256;
        const int nl = idx >> 3, ch = idx & 7;
        const int nn = n0 + nl, mm = m0 + ch * 16;
        if (nn < N && mm < M) {
            const uint4 val = *reinterpret_cast<const uint4*>(&s_out[nl * 128 + (((ch ^ (nl >> 3)) & 7) << 4)]);
            __stcs(reinterpret_cast<uint4*>(q_col + (int64_t)nn * M + mm), val);
        }
    }
    return true;
}

// The forward of a trained Linear needs x quantised in 1x128 row tiles (its own GEMM) and, for the weight
// gradient later, those quantised values de-quantised and quantised again in 128x128 blocks
// (src/kernels.py:746 and :784-787).  Same piece layout as above: row tiles are reduced inside half-warps and
// written; the thread then decodes its own bytes, multiplies by the row scale (exactly what
// dequantize_fp8_rowwise yields), and the block's amax is one shuffle tree + shared memory.  Bit-identical to
// quantize_fp8_rowwise followed by the row-to-block re-quantiser, with x read once and its e4m3 copy never re-read.
// TRANS: the block-scaled bytes are written transposed, (N, M) with M contiguous (M a multiple of 16): the layout in
// which the weight-gradient GEMM reads them K-major.  They leave through the staging tile of dual_tile.
template <int DIV, bool ROUND, bool TRANS, typename AfterSync>
__device__ __forceinline__ bool row_block_tile(float (&v)[8][8], float* s_red, uint8_t* s_out, bool ok,
                                               uint8_t* __restrict__ q_row,
                                               float* __restrict__ s_row, uint8_t* __restrict__ q_blk,
                                               float* __restrict__ s_blk, int M, int N, int nb_n, int bm, int bn,
                                               AfterSync&& after_sync) {
    const int sub = threadIdx.x & 15, hw = threadIdx.x >> 4, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = bn * 128 + sub * 8;
    const int mt = bm * 128 + hw * 8;
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaxf(a, fabsf(v[i][j]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        const float s = scale_from_amax<DIV, ROUND>(a);
        const float d = divisor_of<DIV>(s);
        uint2 o2;
        o2.x = cvt_e4m3x4(scaled_clamped<DIV>(v[i][0], d), scaled_clamped<DIV>(v[i][1], d),
                          scaled_clamped<DIV>(v[i][2], d), scaled_clamped<DIV>(v[i][3], d));
        o2.y = cvt_e4m3x4(scaled_clamped<DIV>(v[i][4], d), scaled_clamped<DIV>(v[i][5], d),
                          scaled_clamped<DIV>(v[i][6], d), scaled_clamped<DIV>(v[i][7], d));
        const bool inb = mt + i < M && n < N;
        if (inb) {
            __stcs(reinterpret_cast<uint2*>(q_row + (int64_t)(mt + i) * N + n), o2);
            if (sub == 0) s_row[(int64_t)(mt + i) * nb_n + bn] = s;
        }
        // what the backward would read back: e4m3 value times the row scale (zero outside the matrix)
        const uint32_t w[2] = {o2.x, o2.y};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float2 lo = e4m3x2_to_float2((uint16_t)(w[h] & 0xffff));
            const float2 hi = e4m3x2_to_float2((uint16_t)(w[h] >> 16));
            v[i][4 * h + 0] = inb ? __fmul_rn(lo.x, s) : 0.0f;
            v[i][4 * h + 1] = inb ? __fmul_rn(lo.y, s) : 0.0f;
            v[i][4 * h + 2] = inb ? __fmul_rn(hi.x, s) : 0.0f;
            v[i][4 * h + 3] = inb ? __fmul_rn(hi.y, s) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) bmax = fmaxf(bmax, fabsf(v[i][j]));
    }
    bmax = warp_max(bmax);
    if (lane == 0) s_red[warp] = bmax;
    if (!__syncthreads_and(ok)) return false;
    after_sync();
    bmax = s_red[0];
#pragma unroll
    for (int w8 = 1; w8 < 8; ++w8) bmax = fmaxf(bmax, s_red[w8]);
    const float sb = scale_from_amax<DIV, false>(bmax);
    const float db = divisor_of<DIV>(sb);
    if (threadIdx.x == 0) s_blk[(int64_t)bm * nb_n + bn] = sb;
    if constexpr (!TRANS) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (mt + i < M && n < N) {
                uint2 o2;
                o2.x = cvt_e4m3x4(scaled_clamped<DIV>(v[i][0], db), scaled_clamped<DIV>(v[i][1], db),
                                  scaled_clamped<DIV>(v[i][2], db), scaled_clamped<DIV>(v[i][3], db));
                o2.y = cvt_e4m3x4(scaled_clamped<DIV>(v[i][4], db), scaled_clamped<DIV>(v[i][5], db),
                                  scaled_clamped<DIV>(v[i][6], db), scaled_clamped<DIV>(v[i][7], db));
                __stcs(reinterpret_cast<uint2*>(q_blk + (int64_t)(mt + i) * N + n), o2);
            }
        }
        __syncthreads();                      // s_red is free for the next piece
    } else {
        // eight rows of one column per 8-byte store into the staging tile (elements outside the matrix are zeros)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint2 o2;
            o2.x = cvt_e4m3x4(scaled_clamped<DIV>(v[0][j], db), scaled_clamped<DIV>(v[1][j], db),
                              scaled_clamped<DIV>(v[2][j], db), scaled_clamped<DIV>(v[3][j], db));
            o2.y = cvt_e4m3x4(scaled_clamped<DIV>(v[4][j], db), scaled_clamped<DIV>(v[5][j], db),
                              scaled_clamped<DIV>(v[6][j], db), scaled_clamped<DIV>(v[7][j], db));
            const int nl = sub * 8 + j;
            *reinterpret_cast<uint2*>(&s_out[nl * 128 + ((((hw >> 1) ^ sub) & 7) << 4) + ((hw & 1) << 3)]) = o2;
        }
        __syncthreads();
        const int m0 = bm * 128, n0 = bn * 128;
#pragma unroll
        for (int rep = 0; rep < 4; ++rep) {
            const int idx = threadIdx.x + rep * 256;
            const int nl = idx >> 3, ch = idx & 7;
            const int nn = n0 + nl, mm = m0 + ch * 16;
            if (nn < N && mm < M) {
                const uint4 val = *reinterpret_cast<const uint4*>(&s_out[nl * 128 + (((ch ^ (nl >> 3)) & 7) << 4)]);
                __stcs(reinterpret_cast<uint4*>(q_blk + (int64_t)nn * M + mm), val);
            }
        }
        // the staging tile and s_red are next written after the next piece's block-wide barrier
    }
    return true;
}

// One CTA per piece, loads straight into registers (4-byte inputs, and rows whose pitch a tensor map cannot take).
// MODE 0: q_col / s_col are the quantisation along the rows of the transpose; MODE 1: the 128x128 block re-quantisation;
// MODE 2: the same with its bytes written transposed.
template <typename T, int DIV, bool ROUND, int MODE = 0>
__global__ void __launch_bounds__(256, 2)
quant_row_dual_kernel(const T* __restrict__ x, int64_t ld, uint8_t* __restrict__ q_row, float* __restrict__ s_row,
                      uint8_t* __restrict__ q_col, float* __restrict__ s_col, int M, int N, int nb_n, int nb_m) {
    __shared__ __align__(16) float s_amax[8][128];
    __shared__ __align__(16) uint8_t s_out[128 * 128];
    const int sub = threadIdx.x & 15, hw = threadIdx.x >> 4;
    const int n = blockIdx.x * 128 + sub * 8;
    const int mt = blockIdx.y * 128 + hw * 8;
    Raw8<T> raw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        raw[i] = (mt + i < M && n < N) ? load_raw8<T>(x + (int64_t)(mt + i) * ld + n) : zero_raw8<T>();
    float v[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) unpack_raw8<T>(raw[i], v[i]);
    if constexpr (MODE == 0)
        dual_tile<DIV, ROUND>(v, s_amax, s_out, true, q_row, s_row, q_col, s_col, M, N, nb_n, nb_m, (int)blockIdx.y,
                              (int)blockIdx.x, [] {});
    else
        row_block_tile<DIV, ROUND, MODE == 2>(v, &s_amax[0][0], s_out, true, q_row, s_row, q_col, s_col, M, N, nb_n,
                                              (int)blockIdx.y, (int)blockIdx.x, [] {});
}

// Persistent CTAs fed by TMA (2-byte inputs): the 128 x 128 pieces arrive in a ring of shared-memory stages
// (out-of-range elements arrive as zeros, which is the reference's mask), so the loads of the next pieces are
// in flight while this one is converted.  A stage is handed back to the TMA unit right after every thread has
// copied its part into registers.
constexpr int DUAL_STAGES = 2;
constexpr int DUAL_GROUP_M = 8;
constexpr int DUAL_STAGE_BYTES = 128 * 128 * 2;
constexpr int DUAL_SMEM_BYTES = DUAL_STAGES * DUAL_STAGE_BYTES + 128 * 128 + 8 * 128 * 4 + 64;
constexpr long long QUANT_WAIT_LIMIT_CYCLES = 4000000000LL;   // about two seconds

__device__ int g_quant_status = 0;     // 0 = fine, otherwise (4 << 8) | reason

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 0 && clock64() - t0 > QUANT_WAIT_LIMIT_CYCLES) return false;
    }
}

template <typename T, int DIV, bool ROUND, int MODE = 0>
__global__ void __launch_bounds__(256, 2)
quant_row_dual_tma_kernel(const __grid_constant__ CUtensorMap tmX, uint8_t* __restrict__ q_row, float* __restrict__ s_row,
                          uint8_t* __restrict__ q_col, float* __restrict__ s_col, int M, int N, int nb_n, int nb_m,
                          int total) {
    static_assert(sizeof(T) == 2, "the TMA-fed path takes 2-byte inputs");
    extern __shared__ __align__(128) uint8_t dsm[];
    uint8_t* stages = dsm;
    uint8_t* s_out = dsm + DUAL_STAGES * DUAL_STAGE_BYTES;
    float (*s_amax)[128] = reinterpret_cast<float (*)[128]>(s_out + 128 * 128);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_out + 128 * 128 + 8 * 128 * 4);
    const uint32_t full0 = smem_u32(bars);
    const int sub = threadIdx.x & 15, hw = threadIdx.x >> 4;
    const int stride = gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < DUAL_STAGES; ++s) mbar_init(full0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Pieces are walked in bands of DUAL_GROUP_M row blocks, down the band first: the CTAs running at one time
    // then touch long runs of every input row and DUAL_GROUP_M neighbouring 128-byte pieces of every transposed
    // output row, so both sides keep DRAM pages open.
    auto coords = [&](int t, int& bm, int& bn) {
        const int band = t / (DUAL_GROUP_M * nb_n);
        const int r = t - band * (DUAL_GROUP_M * nb_n);
        const int rows = min(DUAL_GROUP_M, nb_m - band * DUAL_GROUP_M);
        bn = r / rows;
        bm = band * DUAL_GROUP_M + (r - bn * rows);
    };
    auto issue = [&](int t, int s) {                     // one elected thread
        int bm, bn;
        coords(t, bm, bn);
        mbar_expect_tx(full0 + 8 * s, DUAL_STAGE_BYTES);
        tma_load_2d(&tmX, full0 + 8 * s, smem_u32(stages + s * DUAL_STAGE_BYTES), bn * 128, bm * 128);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < DUAL_STAGES; ++s)
            if ((int)blockIdx.x + s * stride < total) issue(blockIdx.x + s * stride, s);
    }
    int k = 0;
    int t = blockIdx.x;
    bool alive = true;
    for (; t < total; t += stride, ++k) {
        const int s = k % DUAL_STAGES;
        const bool ok = mbar_wait_bounded(full0 + 8 * s, (k / DUAL_STAGES) & 1);
        const uint8_t* src = stages + s * DUAL_STAGE_BYTES + (hw * 8) * 256 + sub * 16;
        float v[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            Raw8<T> r;
            r.a = *reinterpret_cast<const uint4*>(src + i * 256);
            unpack_raw8<T>(r, v[i]);
        }
        const int tn = t + DUAL_STAGES * stride;
        int bm, bn;
        coords(t, bm, bn);
        if constexpr (MODE == 0)
            alive = dual_tile<DIV, ROUND>(v, s_amax, s_out, ok, q_row, s_row, q_col, s_col, M, N, nb_n, nb_m, bm, bn,
                                          [&] { if (threadIdx.x == 0 && tn < total) issue(tn, s); });
        else
            alive = row_block_tile<DIV, ROUND, MODE == 2>(v, &s_amax[0][0], s_out, ok, q_row, s_row, q_col, s_col, M, N, nb_n,
                                                          bm, bn, [&] { if (threadIdx.x == 0 && tn < total) issue(tn, s); });
        if (!alive) break;
    }
    if (!alive && threadIdx.x == 0) {
        atomicCAS(&g_quant_status, 0, (4 << 8) | 1);
        // loads still in flight target this CTA's shared memory: give them their (bounded) time before leaving
        for (int j = 1; j < DUAL_STAGES; ++j)
            if (t + j * stride < total) mbar_wait_bounded(full0 + 8 * ((k + j) % DUAL_STAGES), ((k + j) / DUAL_STAGES) & 1);
    }
}

// The dual quantiser over a token axis cut into per-expert segments (the backward of the grouped expert GEMM): one
// pass over dY yields its row-wise quantisation (what the grouped input gradient reads, in place of the rows) and the
// quantisation of dY^T along the tokens of each segment, padded to whole tiles (what the grouped weight gradient
// reads).  Tile y of the padded axis holds tile_cnt[y] rows from tile_src[y] on; only the first *n_tiles tiles exist.
// Same TMA ring as the dense kernel; the elected thread leaves each stage's (first row, row count) beside the barriers.
template <typename T, int DIV>
__global__ void __launch_bounds__(256, 2)
quant_row_dual_seg_kernel(const __grid_constant__ CUtensorMap tmX, uint8_t* __restrict__ q_row, float* __restrict__ s_row,
                          uint8_t* __restrict__ q_col, float* __restrict__ s_col, int M_pad, int N, int nb_n, int nb_m,
                          const int* __restrict__ tile_src, const int* __restrict__ tile_cnt, const int* __restrict__ n_tiles) {
    static_assert(sizeof(T) == 2, "the TMA-fed path takes 2-byte inputs");
    extern __shared__ __align__(128) uint8_t dsm[];
    uint8_t* stages = dsm;
    uint8_t* s_out = dsm + DUAL_STAGES * DUAL_STAGE_BYTES;
    float (*s_amax)[128] = reinterpret_cast<float (*)[128]>(s_out + 128 * 128);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_out + 128 * 128 + 8 * 128 * 4);
    volatile int* s_meta = reinterpret_cast<volatile int*>(bars + DUAL_STAGES);      // (src0, cnt) per stage
    const uint32_t full0 = smem_u32(bars);
    const int sub = threadIdx.x & 15, hw = threadIdx.x >> 4;
    const int stride = gridDim.x;
    const int total = *n_tiles * nb_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < DUAL_STAGES; ++s) mbar_init(full0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](int t, int s) {                     // one elected thread
        const int bm = t / nb_n, bn = t - bm * nb_n;
        const int src0 = tile_src[bm];
        s_meta[2 * s] = src0;
        s_meta[2 * s + 1] = tile_cnt[bm];
        mbar_expect_tx(full0 + 8 * s, DUAL_STAGE_BYTES);
        tma_load_2d(&tmX, full0 + 8 * s, smem_u32(stages + s * DUAL_STAGE_BYTES), bn * 128, src0);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < DUAL_STAGES; ++s)
            if ((int)blockIdx.x + s * stride < total) issue(blockIdx.x + s * stride, s);
    }
    int k = 0;
    int t = blockIdx.x;
    bool alive = true;
    for (; t < total; t += stride, ++k) {
        const int s = k % DUAL_STAGES;
        const bool ok = mbar_wait_bounded(full0 + 8 * s, (k / DUAL_STAGES) & 1);
        const int src0 = s_meta[2 * s], cnt = s_meta[2 * s + 1];
        const uint8_t* src = stages + s * DUAL_STAGE_BYTES + (hw * 8) * 256 + sub * 16;
        float v[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            Raw8<T> r;
            r.a = *reinterpret_cast<const uint4*>(src + i * 256);
            unpack_raw8<T>(r, v[i]);
        }
        const int tn = t + DUAL_STAGES * stride;
        const int bm = t / nb_n, bn = t - bm * nb_n;
        alive = dual_tile<DIV, false, true>(v, s_amax, s_out, ok, q_row, s_row, q_col, s_col, M_pad, N, nb_n, nb_m, bm, bn,
                                            [&] { if (threadIdx.x == 0 && tn < total) issue(tn, s); }, src0, cnt);
        if (!alive) break;
    }
    if (!alive && threadIdx.x == 0) {
        atomicCAS(&g_quant_status, 0, (4 << 8) | 1);
        for (int j = 1; j < DUAL_STAGES; ++j)
            if (t + j * stride < total) mbar_wait_bounded(full0 + 8 * ((k + j) % DUAL_STAGES), ((k + j) / DUAL_STAGES) & 1);
    }
}

// ---------------------------------------------------------------------------
// Block-wise 128x128, vector path: one CTA per block, 8 warps x 16 rows,
// each lane 4 consecutive columns; the whole block stays in registers between
// the amax and the cast, so the input is read exactly once.
// ---------------------------------------------------------------------------
template <typename T, int DIV, bool ROUND>
__global__ void __launch_bounds__(256)
quant_block_vec_kernel(const T* __restrict__ x, int64_t ld, uint8_t* __restrict__ q, float* __restrict__ scales,
                       int M, int N, int nb) {
    __shared__ float s_red[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.y * 128, c = blockIdx.x * 128 + lane * 4;
    float v[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int r = r0 + warp + i * 8;
        if (r < M && c < N) {
            Elem<T>::load4(x + (int64_t)r * ld + c, v[i]);
        } else {
            v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.0f;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    amax = warp_max(amax);
    if (lane == 0) s_red[warp] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
    const float s = scale_from_amax<DIV, ROUND>(amax);
    const float d = divisor_of<DIV>(s);
    if (threadIdx.x == 0) scales[(int64_t)blockIdx.y * nb + blockIdx.x] = s;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int r = r0 + warp + i * 8;
        if (r < M && c < N) {
            const uint32_t o = cvt_e4m3x4(scaled_clamped<DIV>(v[i][0], d), scaled_clamped<DIV>(v[i][1], d),
                                          scaled_clamped<DIV>(v[i][2], d), scaled_clamped<DIV>(v[i][3], d));
            *reinterpret_cast<uint32_t*>(q + (int64_t)r * N + c) = o;
        }
    }
}

// 4 x 4 byte transpose in registers: r[i] holds bytes (row i, columns 0..3); c[j] receives (rows 0..3, column j).
__device__ __forceinline__ void transpose4x4_bytes(const uint32_t (&r)[4], uint32_t (&c)[4]) {
    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[2], r[3], 0x5140);
    const uint32_t t2 = __byte_perm(r[0], r[1], 0x7362), t3 = __byte_perm(r[2], r[3], 0x7362);
    c[0] = __byte_perm(t0, t1, 0x5410);
    c[1] = __byte_perm(t0, t1, 0x7632);
    c[2] = __byte_perm(t2, t3, 0x5410);
    c[3] = __byte_perm(t2, t3, 0x7632);
}

// A 128 x 128 byte tile written transposed.  `blk[a]` (a < 4) holds this thread's 4 x 4 block of rows
// 16 * warp + 4 * a .. + 3 and columns 4 * lane .. + 3, already transposed (word j = four rows of column 4 * lane + j).
// Staging: 128 transposed rows of 32 words; word position XOR-ed with (transposed row / 4) so that both the stores
// (lanes = columns) and the loads (lanes = words of one row) touch 32 different banks.  Output rows of pitch
// `pitch` bytes (a multiple of 4), 4 bytes per lane, 128 contiguous bytes per warp store.
__device__ __forceinline__ void store_tile_transposed(const uint32_t (&blk)[4][4], uint32_t* s_t, uint8_t* __restrict__ out,
                                                      int64_t pitch, int r0, int c0, int R, int C) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int j = 0; j < 4; ++j) s_t[(lane * 4 + j) * 32 + ((warp * 4 + a) ^ lane)] = blk[a][j];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const int n = warp * 16 + k;                       // transposed row = input column
        const uint32_t w = s_t[n * 32 + (lane ^ (n >> 2))];
        if (c0 + n < C && r0 + lane * 4 < R) *reinterpret_cast<uint32_t*>(out + (int64_t)(c0 + n) * pitch + r0 + lane * 4) = w;
    }
}

// The block-wise quantiser with a second, byte-transposed copy of its output: q (M, N) and q_t (N, M), one set of
// scales (a 128 x 128 block and its transpose share their scale).  The transposed copy is the weight as the input
// gradient's GEMM wants it: reduction axis innermost.  Rows are dealt to warps in runs of 16 here, so that a thread
// holds 4 x 4 byte blocks it can transpose in registers.  M must be a multiple of 4.
template <typename T, int DIV, bool ROUND>
__global__ void __launch_bounds__(256)
quant_block_vec_t_kernel(const T* __restrict__ x, int64_t ld, uint8_t* __restrict__ q, uint8_t* __restrict__ q_t,
                         float* __restrict__ scales, int M, int N, int nb) {
    __shared__ float s_red[8];
    __shared__ uint32_t s_t[128 * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.y * 128, c = blockIdx.x * 128 + lane * 4;
    float v[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int r = r0 + warp * 16 + i;
        if (r < M && c < N) {
            Elem<T>::load4(x + (int64_t)r * ld + c, v[i]);
        } else {
            v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.0f;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    amax = warp_max(amax);
    if (lane == 0) s_red[warp] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
    const float s = scale_from_amax<DIV, ROUND>(amax);
    const float d = divisor_of<DIV>(s);
    if (threadIdx.x == 0) scales[(int64_t)blockIdx.y * nb + blockIdx.x] = s;
    uint32_t blk[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        uint32_t rows[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + warp * 16 + a * 4 + i;
            rows[i] = cvt_e4m3x4(scaled_clamped<DIV>(v[a * 4 + i][0], d), scaled_clamped<DIV>(v[a * 4 + i][1], d),
                                 scaled_clamped<DIV>(v[a * 4 + i][2], d), scaled_clamped<DIV>(v[a * 4 + i][3], d));
            if (r < M && c < N) *reinterpret_cast<uint32_t*>(q + (int64_t)r * N + c) = rows[i];
        }
        transpose4x4_bytes(rows, blk[a]);
    }
    store_tile_transposed(blk, s_t, q_t, M, r0, blockIdx.x * 128, M, N);
}

// Block-wise, arbitrary strides / block sizes: one CTA per block, two passes.
template <typename T, int DIV, bool ROUND>
__global__ void __launch_bounds__(256)
quant_block_generic_kernel(const T* __restrict__ x, int64_t ld_m, int64_t ld_n, uint8_t* __restrict__ q,
                           float* __restrict__ scales, int M, int N, int bm, int bn, int nb) {
    __shared__ float s_red[8];
    const int r0 = blockIdx.y * bm, c0 = blockIdx.x * bn;
    const int rows = min(bm, M - r0), cols = min(bn, N - c0);
    const int count = rows * cols;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < count; i += 256) {
        const int r = r0 + i / cols, c = c0 + i % cols;
        amax = fmaxf(amax, fabsf(Elem<T>::to_f(x[(int64_t)r * ld_m + (int64_t)c * ld_n])));
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
    const float s = scale_from_amax<DIV, ROUND>(amax);
    const float d = divisor_of<DIV>(s);
    if (threadIdx.x == 0) scales[(int64_t)blockIdx.y * nb + blockIdx.x] = s;
    for (int i = threadIdx.x; i < count; i += 256) {
        const int r = r0 + i / cols, c = c0 + i % cols;
        const float y = scaled_clamped<DIV>(Elem<T>::to_f(x[(int64_t)r * ld_m + (int64_t)c * ld_n]), d);
        q[(int64_t)r * N + c] = (uint8_t)(cvt_e4m3x2(y, 0.0f) & 0xff);
    }
}

// ---------------------------------------------------------------------------
// Re-quantise row-scaled e4m3 to block-scaled e4m3 in one pass: the weight-
// gradient path de-quantises x row-wise to fp32 and quantises it again in
// 128x128 blocks (src/kernels.py:784-787).  Here the fp32 product lives only
// in registers.  Optionally the block-scaled bytes are written transposed
// (K x M), so that the token axis is contiguous.
// ---------------------------------------------------------------------------
// SEG: row block blockIdx.y reads tile_cnt[y] source rows starting at tile_src[y] (per-expert segments padded to
// whole blocks, see quant_row_transposed_kernel); blocks at or past *n_tiles do not exist.
template <int DIV, bool TRANSPOSE_OUT, bool SEG = false>
__global__ void __launch_bounds__(256)
requant_row_to_block_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, int nkb_in,
                            uint8_t* __restrict__ out, float* __restrict__ scales, int M, int K, int nb, int M_in,
                            const int* __restrict__ tile_src = nullptr, const int* __restrict__ tile_cnt = nullptr,
                            const int* __restrict__ n_tiles = nullptr) {
    // M_in <= M: rows at or past M_in are not read and count as zeros (and are written as zeros)
    __shared__ float s_red[8];
    __shared__ __align__(16) uint8_t s_t[TRANSPOSE_OUT ? 128 * (128 + 16) : 16];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane & 7;                      // 16-byte chunk within the 128-byte row
    const int r0 = blockIdx.y * 128, c = blockIdx.x * 128 + sub * 16;
    int src0 = r0, cnt = M_in - r0;
    if constexpr (SEG) {
        if ((int)blockIdx.y >= *n_tiles) return;
        src0 = tile_src[blockIdx.y];
        cnt = tile_cnt[blockIdx.y];
    }
    float v[4][16];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int rl_in = p * 32 + warp * 4 + (lane >> 3);
        const int r = src0 + rl_in;
        if (rl_in < cnt && c < K) {
            const uint4 raw = *reinterpret_cast<const uint4*>(xq + (int64_t)r * K + c);
            const float rs = xs[(int64_t)r * nkb_in + blockIdx.x];
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = e4m3x2_to_float2((uint16_t)(w[j] & 0xffff));
                const float2 b = e4m3x2_to_float2((uint16_t)(w[j] >> 16));
                v[p][4 * j + 0] = __fmul_rn(a.x, rs); v[p][4 * j + 1] = __fmul_rn(a.y, rs);
                v[p][4 * j + 2] = __fmul_rn(b.x, rs); v[p][4 * j + 3] = __fmul_rn(b.y, rs);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[p][j] = 0.0f;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[p][j]));
    amax = warp_max(amax);
    if (lane == 0) s_red[warp] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
    const float s = scale_from_amax<DIV, false>(amax);
    const float d = divisor_of<DIV>(s);
    if (threadIdx.x == 0) scales[(int64_t)blockIdx.y * nb + blockIdx.x] = s;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int rl = p * 32 + warp * 4 + (lane >> 3);
        const int r = r0 + rl;
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = cvt_e4m3x4(scaled_clamped<DIV>(v[p][4 * j], d), scaled_clamped<DIV>(v[p][4 * j + 1], d),
                              scaled_clamped<DIV>(v[p][4 * j + 2], d), scaled_clamped<DIV>(v[p][4 * j + 3], d));
        if constexpr (!TRANSPOSE_OUT) {
            if (r < M && c < K) *reinterpret_cast<uint4*>(out + (int64_t)r * K + c) = make_uint4(o[0], o[1], o[2], o[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                s_t[(sub * 16 + j) * (128 + 16) + rl] = (uint8_t)((o[j >> 2] >> (8 * (j & 3))) & 0xff);
        }
    }
    if constexpr (TRANSPOSE_OUT) {
        __syncthreads();
        // out is (K, M): row k holds 128 consecutive tokens of this block
#pragma unroll
        for (int rep = 0; rep < 4; ++rep) {
            const int idx = threadIdx.x + rep * 256;
            const int kl = idx >> 3, ch = idx & 7;
            const int k = blockIdx.x * 128 + kl, m = r0 + ch * 16;
            if (k < K && m < M)
                *reinterpret_cast<uint4*>(out + (int64_t)k * M + m) =
                    *reinterpret_cast<const uint4*>(&s_t[kl * (128 + 16) + ch * 16]);
        }
    }
}

// The segmented, transposing re-quantiser as a persistent kernel: every CTA walks tiles (row block y, K block x; x
// fastest) and keeps the raw bytes and row scales of its NEXT tile in flight (cp.async into the other half of a
// double buffer) while it converts the current one.  A CTA that loads, converts and stores one tile at a time leaves
// the memory system idle for most of its life (the loads of a tile all wait on one round trip); with the copy of the
// next tile under the arithmetic of this one the pass runs three times as fast.  Rows at or past a tile's count
// arrive as zeros (cp.async with a source size of 0).  Rows are dealt to warps in runs of 16 and a thread holds
// 4 bytes of each, so that it owns 4 x 4 byte blocks it can transpose in registers before the staged, transposed store.
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool live) {
    const int n = live ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4_zfill(uint32_t dst, const void* src, bool live) {
    const int n = live ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

template <int DIV>
__global__ void __launch_bounds__(256, 2)
requant_seg_t_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, uint8_t* __restrict__ out,
                     float* __restrict__ scales, int M, int K, int nb, const int* __restrict__ tile_src,
                     const int* __restrict__ tile_cnt, const int* __restrict__ n_tiles) {
    __shared__ __align__(16) uint8_t s_raw[2][128 * 128];
    __shared__ float s_rs[2][128];
    __shared__ float s_red[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total = *n_tiles * nb;
    // issue the copies of one tile (rows src0 .. src0 + cnt of K block x) into buffer b
    auto fetch = [&](int x, int src0, int cnt, int b) {
        const uint32_t raw0 = (uint32_t)__cvta_generic_to_shared(&s_raw[b][0]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = threadIdx.x + k * 256, row = c >> 3, part = c & 7;
            const bool live = row < cnt;
            const uint8_t* src = xq + (int64_t)(src0 + (live ? row : 0)) * K + x * 128 + part * 16;
            cp_async16_zfill(raw0 + row * 128 + part * 16, src, live);
        }
        if (threadIdx.x < 128) {
            const bool live = (int)threadIdx.x < cnt;
            cp_async4_zfill((uint32_t)__cvta_generic_to_shared(&s_rs[b][threadIdx.x]),
                            xs + (int64_t)(src0 + (live ? (int)threadIdx.x : 0)) * nb + x, live);
        }
    };
    int t0 = blockIdx.x;
    if (t0 >= total) return;
    int y0 = t0 / nb, x0 = t0 - y0 * nb;
    fetch(x0, tile_src[y0], tile_cnt[y0], 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    int t1 = t0 + gridDim.x, y1 = 0, x1 = 0, src1 = 0, cnt1 = 0;
    if (t1 < total) { y1 = t1 / nb; x1 = t1 - y1 * nb; src1 = tile_src[y1]; cnt1 = tile_cnt[y1]; }
    for (int b = 0; t0 < total; b ^= 1) {
        if (t1 < total) fetch(x1, src1, cnt1, b ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        // the tile after the next: its row range is on its way while this tile is converted
        const int t2 = t1 + gridDim.x;
        int y2 = 0, x2 = 0, src2 = 0, cnt2 = 0;
        if (t2 < total) { y2 = t2 / nb; x2 = t2 - y2 * nb; src2 = tile_src[y2]; cnt2 = tile_cnt[y2]; }
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        float v[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int row = warp * 16 + i;
            const uint32_t raw = *reinterpret_cast<const uint32_t*>(&s_raw[b][row * 128 + lane * 4]);
            const float rs = s_rs[b][row];
            const float2 a = e4m3x2_to_float2((uint16_t)(raw & 0xffff));
            const float2 c = e4m3x2_to_float2((uint16_t)(raw >> 16));
            v[i][0] = __fmul_rn(a.x, rs); v[i][1] = __fmul_rn(a.y, rs);
            v[i][2] = __fmul_rn(c.x, rs); v[i][3] = __fmul_rn(c.y, rs);
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
        amax = warp_max(amax);
        if (lane == 0) s_red[warp] = amax;
        __syncthreads();
        amax = s_red[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
        const float sc = scale_from_amax<DIV, false>(amax);
        const float d = divisor_of<DIV>(sc);
        if (threadIdx.x == 0) scales[(int64_t)y0 * nb + x0] = sc;
        uint32_t blk[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            uint32_t rows[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                rows[i] = cvt_e4m3x4(scaled_clamped<DIV>(v[a * 4 + i][0], d), scaled_clamped<DIV>(v[a * 4 + i][1], d),
                                     scaled_clamped<DIV>(v[a * 4 + i][2], d), scaled_clamped<DIV>(v[a * 4 + i][3], d));
            transpose4x4_bytes(rows, blk[a]);
        }
        // the tile's raw bytes are in registers by now (barrier above): its buffer doubles as the transposing stage
        store_tile_transposed(blk, reinterpret_cast<uint32_t*>(&s_raw[b][0]), out, M, y0 * 128, x0 * 128, M, K);
        __syncthreads();            // s_red and buffer b are free again
        t0 = t1; y0 = y1; x0 = x1;
        t1 = t2; y1 = y2; x1 = x2; src1 = src2; cnt1 = cnt2;
    }
}

// ---------------------------------------------------------------------------
// SwiGLU + row-wise quantisation in one pass: h12 is (T, 2*I) with the gate half first
// (GroupedExperts keeps w12 = [w1; w2], src/layers.py:47-49, 71-73); h = silu(h1) * h2 is
// formed in fp32, rounded to the activation dtype as the reference does before its second
// grouped GEMM (src/layers.py:74), and quantised in 1x128 tiles.  The fp32 h never reaches HBM.
// A half-warp owns one 128-wide tile.
// ---------------------------------------------------------------------------
template <typename T, int DIV>
__global__ void __launch_bounds__(256)
swiglu_quant_row_kernel(const T* __restrict__ h12, uint8_t* __restrict__ q, float* __restrict__ scales,
                        int I, int nb, int64_t total_tiles, int step_rows, int step_cols,
                        const int64_t* __restrict__ n_rows_dev) {
    // optional row count that only the device knows (an expert-parallel rank's received rows): rows past it are skipped
    if (n_rows_dev != nullptr) total_tiles = min(total_tiles, max(n_rows_dev[0], (int64_t)0) * nb);
    // the n-th tile of this half-warp is hw + n * n_hw; (step_rows, step_cols) = divmod(n_hw, nb): tile
    // coordinates advance without a division in the loop
    const int sub = threadIdx.x & 15;
    const int64_t hw = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);
    const int64_t n_hw = (int64_t)gridDim.x * 16;
    int64_t t = hw;                                  // next tile to FETCH
    int row = (int)(hw / nb);
    int cb = (int)(hw - (int64_t)row * nb);
    // the raw vectors of the next tile are in flight while this one is converted
    Raw8<T> na = zero_raw8<T>(), nb8 = zero_raw8<T>();
    int64_t n_off = -1, n_tile = -1;
    auto fetch = [&]() {
        const int col = cb * 128 + sub * 8;
        const bool live = t < total_tiles;
        const bool inb = live && col < I;
        if (inb) {
            const T* p = h12 + (int64_t)row * 2 * I + col;
            na = load_raw8<T>(p);
            nb8 = load_raw8<T>(p + I);
        }
        n_off = inb ? (int64_t)row * I + col : -1;
        n_tile = live ? t : -1;
        t += n_hw;
        row += step_rows;
        cb += step_cols;
        if (cb >= nb) { cb -= nb; row += 1; }
    };
    fetch();
    for (int64_t tw = hw & ~(int64_t)1; tw < total_tiles; tw += n_hw) {
        const Raw8<T> ca = na, cb_raw = nb8;
        const int64_t off = n_off, tile = n_tile;
        fetch();
        float a[8], b[8], v[8];
        if (off >= 0) {
            unpack_raw8<T>(ca, a);
            unpack_raw8<T>(cb_raw, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                // 16-bit activations: silu to a few fp32 ulp (ex2.approx and div.approx), far inside the rounding to
                // the activation type that follows; the IEEE sequences would make this pass instruction-bound
                // instead of HBM-bound.  fp32 activations are not rounded afterwards and take the exact sequences.
                float h;
                if constexpr (sizeof(T) == 4) h = (a[i] / (1.0f + expf(-a[i]))) * b[i];
                else h = __fdividef(a[i], 1.0f + __expf(-a[i])) * b[i];
                if constexpr (std::is_same<T, __nv_bfloat16>::value) v[i] = __bfloat162float(__float2bfloat16_rn(h));
                else if constexpr (std::is_same<T, __half>::value) v[i] = __half2float(__float2half_rn(h));
                else v[i] = h;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float s = scale_from_amax<DIV, false>(amax);
        const float d = divisor_of<DIV>(s);
        if (off >= 0) {
            uint2 o2;
            o2.x = cvt_e4m3x4(scaled_clamped<DIV>(v[0], d), scaled_clamped<DIV>(v[1], d), scaled_clamped<DIV>(v[2], d), scaled_clamped<DIV>(v[3], d));
            o2.y = cvt_e4m3x4(scaled_clamped<DIV>(v[4], d), scaled_clamped<DIV>(v[5], d), scaled_clamped<DIV>(v[6], d), scaled_clamped<DIV>(v[7], d));
            __stcs(reinterpret_cast<uint2*>(q + off), o2);
        }
        if (sub == 0 && tile >= 0) scales[tile] = s;
    }
}

// ---------------------------------------------------------------------------
// De-quantisers
// ---------------------------------------------------------------------------
// out[r, c] = e4m3(q[r, c]) * scales[(r / bm) * ncb + c / bn]; OUT = bf16 or fp32.
template <typename OUT>
__global__ void __launch_bounds__(256)
dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales, OUT* __restrict__ out,
               int64_t M, int N, int bm, int bn, int ncb) {
    const int64_t total = M * (int64_t)N;
    for (int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4; i < total; i += (int64_t)gridDim.x * 1024) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t e = i + j;
            if (e < total) {
                const int64_t r = e / N;
                const int c = (int)(e - r * N);
                const float2 f = e4m3x2_to_float2((uint16_t)q[e]);
                const float y = __fmul_rn(f.x, scales[(r / bm) * ncb + c / bn]);
                if constexpr (sizeof(OUT) == 2) out[e] = __float2bfloat16_rn(y); else out[e] = y;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// byte transpose (used when a caller hands fp8_matmul an operand whose
// reduction axis is not the contiguous one)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
transpose_bytes_kernel(const uint8_t* __restrict__ in, int64_t ld_in, uint8_t* __restrict__ out, int R, int C) {
    // in: R x C (row pitch ld_in) -> out: C x R contiguous; 64 x 64 tiles, byte by byte (any alignment)
    __shared__ uint8_t t[64][64 + 4];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int r = i >> 6, c = i & 63;
        if (r0 + r < R && c0 + c < C) t[r][c] = in[(int64_t)(r0 + r) * ld_in + c0 + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int c = i >> 6, r = i & 63;
        if (r0 + r < R && c0 + c < C) out[(int64_t)(c0 + c) * R + r0 + r] = t[r][c];
    }
}

// The same for 4-byte aligned shapes (R, C, ld_in multiples of 4, 4-byte aligned pointers): 128 x 128 tiles,
// 4-byte loads (128 contiguous bytes per warp), 4 x 4 blocks transposed in registers, 4-byte stores.
__global__ void __launch_bounds__(256)
transpose_bytes_vec_kernel(const uint8_t* __restrict__ in, int64_t ld_in, uint8_t* __restrict__ out, int R, int C) {
    __shared__ uint32_t s_t[128 * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 128;
    uint32_t blk[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        uint32_t rows[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + warp * 16 + a * 4 + i;
            rows[i] = (r < R && c0 + lane * 4 < C) ? __ldg(reinterpret_cast<const uint32_t*>(in + (int64_t)r * ld_in + c0 + lane * 4)) : 0u;
        }
        transpose4x4_bytes(rows, blk[a]);
    }
    store_tile_transposed(blk, s_t, out, R, r0, c0, R, C);
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, int DIV, bool ROUND>
static int launch_rowwise(const T* x, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, uint8_t* q, float* scales,
                          int block, cudaStream_t st) {
    const int nb = (int)((N + block - 1) / block);
    const int64_t tiles = M * nb;
    if (tiles == 0) return CINN_OK;
    const int sms = sm_count();
    if (block == 128 && ld_n == 1 && N % 8 == 0 && ld_m % 8 == 0 && aligned16(x) && aligned16(q)) {
        constexpr int UNROLL = 2;
        int64_t blocks = (tiles + 16 * UNROLL - 1) / (16 * UNROLL);
        const int64_t cap = (int64_t)sms * 8;
        if (blocks > cap) blocks = cap;
        const int64_t n_hw = blocks * 16;
        quant_row_vec_kernel<T, DIV, ROUND, UNROLL><<<(unsigned)blocks, 256, 0, st>>>(
            x, ld_m, q, scales, (int)N, nb, tiles, (int)(n_hw / nb), (int)(n_hw % nb));
    } else if (block == 128 && ld_m == 1 && ld_n >= M && M % 8 == 0 && ld_n % 8 == 0 && N % 16 == 0 && aligned16(x) &&
               aligned16(q) && M > 1) {
        // enough CTAs to fill the GPU several times over, each walking a few tiles with prefetch
        const int64_t slabs = (M + 63) / 64;
        int per = 4;
        while (per > 1 && slabs * ((nb + per - 1) / per) < (int64_t)sms * 8) per >>= 1;
        CINN_CHECK_ARG((nb + per - 1) / per <= 65535, "row-wise quantiser: too many tiles along the strided axis");
        dim3 grid((unsigned)slabs, (unsigned)((nb + per - 1) / per));
        quant_row_transposed_kernel<T, DIV, ROUND><<<grid, 256, 0, st>>>(x, ld_n, q, scales, (int)M, (int)N, nb, per, (int)N);
    } else {
        int64_t blocks = (tiles + 7) / 8;
        const int64_t cap = (int64_t)sms * 16;
        if (blocks > cap) blocks = cap;
        quant_row_generic_kernel<T, DIV, ROUND><<<(unsigned)blocks, 256, 0, st>>>(x, ld_m, ld_n, q, scales, (int)N, nb, block, tiles);
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

template <typename T, int DIV, bool ROUND>
static int launch_blockwise(const T* x, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, uint8_t* q, float* scales,
                            int bm, int bn, cudaStream_t st) {
    const int mb = (int)((M + bm - 1) / bm), nb = (int)((N + bn - 1) / bn);
    if (mb == 0 || nb == 0) return CINN_OK;
    CINN_CHECK_ARG(mb <= 65535, "block-wise quantiser: more than 65535 row blocks (%d)", mb);
    dim3 grid((unsigned)nb, (unsigned)mb);
    const bool a = sizeof(T) == 4 ? aligned16(x) : ((reinterpret_cast<uintptr_t>(x) & 7) == 0);
    if (bm == 128 && bn == 128 && ld_n == 1 && N % 4 == 0 && ld_m % 4 == 0 && a && (reinterpret_cast<uintptr_t>(q) & 3) == 0) {
        quant_block_vec_kernel<T, DIV, ROUND><<<grid, 256, 0, st>>>(x, ld_m, q, scales, (int)M, (int)N, nb);
    } else {
        quant_block_generic_kernel<T, DIV, ROUND><<<grid, 256, 0, st>>>(x, ld_m, ld_n, q, scales, (int)M, (int)N, bm, bn, nb);
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

template <typename T>
static int dispatch_block_t(const T* x, int64_t M, int64_t N, int64_t ld, uint8_t* q, uint8_t* q_t, float* scales,
                            int round_scale, int div_mode, cudaStream_t st) {
    const int mb = (int)((M + 127) / 128), nb = (int)((N + 127) / 128);
    CINN_CHECK_ARG(mb <= 65535, "block-wise quantiser: more than 65535 row blocks (%d)", mb);
    dim3 grid((unsigned)nb, (unsigned)mb);
#define CINN_B(DIV, RND) quant_block_vec_t_kernel<T, DIV, RND><<<grid, 256, 0, st>>>(x, ld, q, q_t, scales, (int)M, (int)N, nb)
    if (div_mode == CINN_DIV_FULL) { if (round_scale) CINN_B(CINN_DIV_FULL, true); else CINN_B(CINN_DIV_FULL, false); }
    else                           { if (round_scale) CINN_B(CINN_DIV_RN, true);   else CINN_B(CINN_DIV_RN, false); }
#undef CINN_B
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int quantize_block_t(const void* x, int dtype, int64_t M, int64_t N, int64_t ld, void* q, void* q_t, float* scales,
                     int round_scale, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M >= 0 && N >= 0, "block quantiser (+ transposed copy): negative shape");
    if (M == 0 || N == 0) return CINN_OK;
    CINN_CHECK_ARG(x && q && q_t && scales, "block quantiser (+ transposed copy): null pointer");
    CINN_CHECK_ARG(N < (1LL << 31) && M < (1LL << 31), "block quantiser (+ transposed copy): dimension too large");
    CINN_CHECK_ARG(M % 4 == 0 && N % 4 == 0 && ld % 4 == 0 && ld >= N,
                   "block quantiser (+ transposed copy): M (%lld), N (%lld) and the row pitch (%lld) must be multiples of 4",
                   (long long)M, (long long)N, (long long)ld);
    CINN_CHECK_ARG(aligned16(x) && aligned16(q) && aligned16(q_t), "block quantiser (+ transposed copy): pointers must be 16-byte aligned");
    CINN_CHECK_ARG(div_mode == CINN_DIV_FULL || div_mode == CINN_DIV_RN, "block quantiser (+ transposed copy): unknown div_mode %d", div_mode);
    switch (dtype) {
        case CINN_BF16: return dispatch_block_t((const __nv_bfloat16*)x, M, N, ld, (uint8_t*)q, (uint8_t*)q_t, scales, round_scale, div_mode, st);
        case CINN_F16:  return dispatch_block_t((const __half*)x, M, N, ld, (uint8_t*)q, (uint8_t*)q_t, scales, round_scale, div_mode, st);
        case CINN_F32:  return dispatch_block_t((const float*)x, M, N, ld, (uint8_t*)q, (uint8_t*)q_t, scales, round_scale, div_mode, st);
        default: set_error("block quantiser (+ transposed copy): unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

template <typename T>
static int dispatch_quant(bool blockwise, const T* x, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, uint8_t* q,
                          float* scales, int bm, int bn, int round_scale, int div_mode, cudaStream_t st) {
#define CINN_Q(DIV, RND)                                                                              \
    return blockwise ? launch_blockwise<T, DIV, RND>(x, M, N, ld_m, ld_n, q, scales, bm, bn, st)      \
                     : launch_rowwise<T, DIV, RND>(x, M, N, ld_m, ld_n, q, scales, bn, st)
    if (div_mode == CINN_DIV_FULL) { if (round_scale) { CINN_Q(CINN_DIV_FULL, true); } else { CINN_Q(CINN_DIV_FULL, false); } }
    else                           { if (round_scale) { CINN_Q(CINN_DIV_RN, true); }   else { CINN_Q(CINN_DIV_RN, false); } }
#undef CINN_Q
}

int quantize(bool blockwise, const void* x, int dtype, int64_t M, int64_t N, int64_t ld_m, int64_t ld_n, void* q,
             float* scales, int bm, int bn, int round_scale, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M >= 0 && N >= 0, "quantise: negative shape (%lld, %lld)", (long long)M, (long long)N);
    if (M == 0 || N == 0) return CINN_OK;
    CINN_CHECK_ARG(x && q && scales, "quantise: null pointer");
    CINN_CHECK_ARG(N < (1LL << 31) && M < (1LL << 31), "quantise: dimension too large");
    CINN_CHECK_ARG(bm >= 1 && bn >= 1 && bn <= 65536 && bm <= 65536, "quantise: bad tile %dx%d", bm, bn);
    CINN_CHECK_ARG(div_mode == CINN_DIV_FULL || div_mode == CINN_DIV_RN, "quantise: unknown div_mode %d", div_mode);
    CINN_CHECK_ARG(ld_m >= 0 && ld_n >= 0, "quantise: negative strides are not supported");
    switch (dtype) {
        case CINN_BF16: return dispatch_quant(blockwise, (const __nv_bfloat16*)x, M, N, ld_m, ld_n, (uint8_t*)q, scales, bm, bn, round_scale, div_mode, st);
        case CINN_F16:  return dispatch_quant(blockwise, (const __half*)x, M, N, ld_m, ld_n, (uint8_t*)q, scales, bm, bn, round_scale, div_mode, st);
        case CINN_F32:  return dispatch_quant(blockwise, (const float*)x, M, N, ld_m, ld_n, (uint8_t*)q, scales, bm, bn, round_scale, div_mode, st);
        default: set_error("quantise: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

template <typename T>
static int dispatch_dual(const T* x, int64_t M, int64_t N, int64_t ld, uint8_t* q_row, float* s_row, uint8_t* q_col,
                         float* s_col, int round_scale, int div_mode, cudaStream_t st) {
    const int nb_n = (int)((N + 127) / 128), nb_m = (int)((M + 127) / 128);
    const bool fused = M % 16 == 0 && N % 8 == 0 && ld % 8 == 0 && nb_m <= 65535 && aligned16(x) && aligned16(q_row) &&
                       aligned16(q_col);
    if (!fused) {
        // ragged shapes: the two single-output quantisers, reading x twice
        int rc = dispatch_quant(false, x, M, N, ld, (int64_t)1, q_row, s_row, 1, 128, round_scale, div_mode, st);
        if (rc) return rc;
        return dispatch_quant(false, x, N, M, (int64_t)1, ld, q_col, s_col, 1, 128, round_scale, div_mode, st);
    }
    if constexpr (sizeof(T) == 2) {
        // 2-byte inputs: persistent CTAs fed by TMA
        CUtensorMap tm;
        int rc = encode_map_2d(&tm, x, (uint64_t)N, (uint64_t)M, (uint64_t)ld * 2, 128, 128, CU_TENSOR_MAP_DATA_TYPE_UINT16,
                               CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        const int64_t total = (int64_t)nb_n * nb_m;
        CINN_CHECK_ARG(total < (1LL << 31), "dual quantiser: too many tiles");
        const int grid = (int)(total < 2 * (int64_t)sm_count() ? total : 2 * (int64_t)sm_count());
#define CINN_D(DIV, RND)                                                                                              \
    do {                                                                                                              \
        auto kern = quant_row_dual_tma_kernel<T, DIV, RND>;                                                           \
        static std::once_flag once;                                                                                   \
        static cudaError_t attr_err = cudaSuccess;                                                                    \
        std::call_once(once, [&] {                                                                                    \
            attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);      \
        });                                                                                                           \
        CINN_CHECK_CUDA(attr_err);                                                                                    \
        kern<<<grid, 256, DUAL_SMEM_BYTES, st>>>(tm, q_row, s_row, q_col, s_col, (int)M, (int)N, nb_n, nb_m, (int)total); \
    } while (0)
        if (div_mode == CINN_DIV_FULL) { if (round_scale) CINN_D(CINN_DIV_FULL, true); else CINN_D(CINN_DIV_FULL, false); }
        else                           { if (round_scale) CINN_D(CINN_DIV_RN, true);   else CINN_D(CINN_DIV_RN, false); }
#undef CINN_D
    } else {
        dim3 grid((unsigned)nb_n, (unsigned)nb_m);
#define CINN_D(DIV, RND) quant_row_dual_kernel<T, DIV, RND><<<grid, 256, 0, st>>>(x, ld, q_row, s_row, q_col, s_col, (int)M, (int)N, nb_n, nb_m)
        if (div_mode == CINN_DIV_FULL) { if (round_scale) CINN_D(CINN_DIV_FULL, true); else CINN_D(CINN_DIV_FULL, false); }
        else                           { if (round_scale) CINN_D(CINN_DIV_RN, true);   else CINN_D(CINN_DIV_RN, false); }
#undef CINN_D
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int requant_row_to_block(const void* xq, const float* xs, int64_t M, int64_t K, void* out, float* scales,
                         int transpose_out, int div_mode, cudaStream_t st);

// Row-wise 1x128 quantisation plus the 128x128 re-quantisation of its result, one pass over x.
template <typename T>
static int dispatch_row_block(const T* x, int64_t M, int64_t N, int64_t ld, uint8_t* q_row, float* s_row, uint8_t* q_blk,
                              float* s_blk, int round_scale, int div_mode, cudaStream_t st, int transpose_block = 0) {
    const int nb_n = (int)((N + 127) / 128), nb_m = (int)((M + 127) / 128);
    const bool fused = N % 16 == 0 && ld % 8 == 0 && nb_m <= 65535 && aligned16(x) && aligned16(q_row) && aligned16(q_blk);
    if (!fused) {
        int rc = dispatch_quant(false, x, M, N, ld, (int64_t)1, q_row, s_row, 1, 128, round_scale, div_mode, st);
        if (rc) return rc;
        return requant_row_to_block(q_row, s_row, M, N, q_blk, s_blk, transpose_block, div_mode, st);
    }
    if constexpr (sizeof(T) == 2) {
        CUtensorMap tm;
        int rc = encode_map_2d(&tm, x, (uint64_t)N, (uint64_t)M, (uint64_t)ld * 2, 128, 128, CU_TENSOR_MAP_DATA_TYPE_UINT16,
                               CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        const int64_t total = (int64_t)nb_n * nb_m;
        CINN_CHECK_ARG(total < (1LL << 31), "row + block quantiser: too many tiles");
        const int grid = (int)(total < 2 * (int64_t)sm_count() ? total : 2 * (int64_t)sm_count());
#define CINN_D(DIV, RND)                                                                                              \
    do {                                                                                                              \
        auto kern = transpose_block ? quant_row_dual_tma_kernel<T, DIV, RND, 2> : quant_row_dual_tma_kernel<T, DIV, RND, 1>; \
        static std::once_flag once;                                                                                   \
        static cudaError_t attr_err = cudaSuccess;                                                                    \
        std::call_once(once, [&] {                                                                                    \
            attr_err = cudaFuncSetAttribute(quant_row_dual_tma_kernel<T, DIV, RND, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES); \
            if (attr_err == cudaSuccess)                                                                              \
                attr_err = cudaFuncSetAttribute(quant_row_dual_tma_kernel<T, DIV, RND, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES); \
        });                                                                                                           \
        CINN_CHECK_CUDA(attr_err);                                                                                    \
        kern<<<grid, 256, DUAL_SMEM_BYTES, st>>>(tm, q_row, s_row, q_blk, s_blk, (int)M, (int)N, nb_n, nb_m, (int)total); \
    } while (0)
        if (div_mode == CINN_DIV_FULL) { if (round_scale) CINN_D(CINN_DIV_FULL, true); else CINN_D(CINN_DIV_FULL, false); }
        else                           { if (round_scale) CINN_D(CINN_DIV_RN, true);   else CINN_D(CINN_DIV_RN, false); }
#undef CINN_D
    } else {
        dim3 grid((unsigned)nb_n, (unsigned)nb_m);
#define CINN_D(DIV, RND)                                                                                              \
    do {                                                                                                              \
        if (transpose_block) quant_row_dual_kernel<T, DIV, RND, 2><<<grid, 256, 0, st>>>(x, ld, q_row, s_row, q_blk, s_blk, (int)M, (int)N, nb_n, nb_m); \
        else quant_row_dual_kernel<T, DIV, RND, 1><<<grid, 256, 0, st>>>(x, ld, q_row, s_row, q_blk, s_blk, (int)M, (int)N, nb_n, nb_m); \
    } while (0)
        if (div_mode == CINN_DIV_FULL) { if (round_scale) CINN_D(CINN_DIV_FULL, true); else CINN_D(CINN_DIV_FULL, false); }
        else                           { if (round_scale) CINN_D(CINN_DIV_RN, true);   else CINN_D(CINN_DIV_RN, false); }
#undef CINN_D
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int quantize_row_block(const void* x, int dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row, void* q_blk,
                       float* s_blk, int round_scale, int div_mode, cudaStream_t st, int transpose_block) {
    CINN_CHECK_ARG(!transpose_block || M % 16 == 0,
                   "row + block quantiser: a transposed block copy needs a row count (%lld) that is a multiple of 16", (long long)M);
    CINN_CHECK_ARG(M >= 0 && N >= 0, "row + block quantiser: negative shape (%lld, %lld)", (long long)M, (long long)N);
    if (M == 0 || N == 0) return CINN_OK;
    CINN_CHECK_ARG(x && q_row && s_row && q_blk && s_blk, "row + block quantiser: null pointer");
    CINN_CHECK_ARG(N < (1LL << 31) && M < (1LL << 31), "row + block quantiser: dimension too large");
    CINN_CHECK_ARG(ld >= N, "row + block quantiser: row pitch %lld below the row length %lld", (long long)ld, (long long)N);
    CINN_CHECK_ARG(N % 16 == 0, "row + block quantiser: the row length (%lld) must be a multiple of 16", (long long)N);
    CINN_CHECK_ARG(div_mode == CINN_DIV_FULL || div_mode == CINN_DIV_RN, "row + block quantiser: unknown div_mode %d", div_mode);
    switch (dtype) {
        case CINN_BF16: return dispatch_row_block((const __nv_bfloat16*)x, M, N, ld, (uint8_t*)q_row, s_row, (uint8_t*)q_blk, s_blk, round_scale, div_mode, st, transpose_block);
        case CINN_F16:  return dispatch_row_block((const __half*)x, M, N, ld, (uint8_t*)q_row, s_row, (uint8_t*)q_blk, s_blk, round_scale, div_mode, st, transpose_block);
        case CINN_F32:  return dispatch_row_block((const float*)x, M, N, ld, (uint8_t*)q_row, s_row, (uint8_t*)q_blk, s_blk, round_scale, div_mode, st, transpose_block);
        default: set_error("row + block quantiser: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

// ---------------------------------------------------------------------------
// Self-check of the hoisted reciprocal: for every positive 16-bit amax pattern (bf16 and fp16, infinity
// included) and both kinds of scale (amax / 448 and its power-of-two rounding), compares
// div.full.f32(x, s) with x * rcp.approx(s) for all 65536 16-bit x of that type and for 65536 fp32 bit
// patterns spread over the whole range, and counts the pairs whose bits differ (two NaNs count as equal:
// the clamp that follows maps both to -448).
// ---------------------------------------------------------------------------
__device__ unsigned long long g_div_mismatches;

__global__ void __launch_bounds__(256)
selfcheck_division_kernel(int fp16) {
    const uint32_t abits = blockIdx.x + 1;
    float amax = fp16 ? __half2float(__ushort_as_half((unsigned short)abits)) : __uint_as_float(abits << 16);
    unsigned long long bad = 0;
    for (int kind = 0; kind < 2; ++kind) {
        const float s = kind == 0 ? scale_from_amax<CINN_DIV_FULL, false>(amax) : scale_from_amax<CINN_DIV_FULL, true>(amax);
        const float d = divisor_of<CINN_DIV_FULL>(s);
        for (uint32_t i = threadIdx.x; i < 2 * 65536u; i += 256) {
            float x;
            if (i < 65536u) x = fp16 ? __half2float(__ushort_as_half((unsigned short)i)) : __uint_as_float(i << 16);
            else x = __uint_as_float((i - 65536u) * 65537u + abits * 40503u);
            const float a = div_f32<CINN_DIV_FULL>(x, s);
            const float b = __fmul_rn(x, d);
            if (__float_as_uint(a) != __float_as_uint(b) && !(a != a && b != b)) ++bad;
        }
    }
    if (bad) atomicAdd(&g_div_mismatches, bad);
}

int selfcheck_division(unsigned long long* mismatches, cudaStream_t st) {
    CINN_CHECK_ARG(mismatches != nullptr, "selfcheck_division: null pointer");
    const unsigned long long zero = 0;
    CINN_CHECK_CUDA(cudaMemcpyToSymbolAsync(g_div_mismatches, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
    selfcheck_division_kernel<<<0x7f80, 256, 0, st>>>(0);      // bf16: patterns 0x0001 .. 0x7f80 (+inf)
    CINN_CHECK_LAUNCH();
    selfcheck_division_kernel<<<0x7c00, 256, 0, st>>>(1);      // fp16: patterns 0x0001 .. 0x7c00 (+inf)
    CINN_CHECK_LAUNCH();
    CINN_CHECK_CUDA(cudaMemcpyFromSymbolAsync(mismatches, g_div_mismatches, sizeof(zero), 0, cudaMemcpyDeviceToHost, st));
    CINN_CHECK_CUDA(cudaStreamSynchronize(st));
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// Padded variants for ragged expert ranges (per-expert weight gradient): the logical tile axis has N_in (resp.
// M_in) real positions and is padded with zeros to N (resp. M), a multiple of 16, without a padded copy of the input.
// ---------------------------------------------------------------------------
template <typename T>
static int transposed_padded_typed(const T* x, int64_t M, int64_t N_in, int64_t N, int64_t L, uint8_t* q, float* scales,
                                   int div_mode, cudaStream_t st) {
    const int nb = (int)((N + 127) / 128);
    const int64_t slabs = (M + 63) / 64;
    int per = 4;
    while (per > 1 && slabs * ((nb + per - 1) / per) < (int64_t)sm_count() * 8) per >>= 1;
    CINN_CHECK_ARG((nb + per - 1) / per <= 65535, "transposed quantiser: too many tiles along the strided axis");
    dim3 grid((unsigned)slabs, (unsigned)((nb + per - 1) / per));
    if (div_mode == CINN_DIV_FULL)
        quant_row_transposed_kernel<T, CINN_DIV_FULL, false><<<grid, 256, 0, st>>>(x, L, q, scales, (int)M, (int)N, nb, per, (int)N_in);
    else
        quant_row_transposed_kernel<T, CINN_DIV_RN, false><<<grid, 256, 0, st>>>(x, L, q, scales, (int)M, (int)N, nb, per, (int)N_in);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// x: element (m, n) at x[m + n * L] for m < M, n < N_in; q: (M, N) e4m3, scales (M, ceil(N / 128)); 1 x 128 tiles along n
int quantize_transposed_padded(const void* x, int dtype, int64_t M, int64_t N_in, int64_t N, int64_t L, void* q,
                               float* scales, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M > 1 && N_in >= 0 && N >= N_in && N % 16 == 0 && M % 8 == 0 && L % 8 == 0 && L >= M,
                   "padded transposed quantiser: needs M %% 8 == 0, a pitch that is a multiple of 8 and N %% 16 == 0");
    if (N == 0) return CINN_OK;
    CINN_CHECK_ARG(x && q && scales && aligned16(x) && aligned16(q), "padded transposed quantiser: null or unaligned pointer");
    CINN_CHECK_ARG(M < (1LL << 31) && N < (1LL << 31), "padded transposed quantiser: dimension too large");
    switch (dtype) {
        case CINN_BF16: return transposed_padded_typed((const __nv_bfloat16*)x, M, N_in, N, L, (uint8_t*)q, scales, div_mode, st);
        case CINN_F16: return transposed_padded_typed((const __half*)x, M, N_in, N, L, (uint8_t*)q, scales, div_mode, st);
        case CINN_F32: return transposed_padded_typed((const float*)x, M, N_in, N, L, (uint8_t*)q, scales, div_mode, st);
        default: set_error("padded transposed quantiser: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

// xq (M_in, K) e4m3 with row scales xs (M_in, ceil(K / 128)) -> out (M, K) block-scaled, scales (ceil(M/128), ceil(K/128))
int requant_row_to_block_padded(const void* xq, const float* xs, int64_t M_in, int64_t M, int64_t K, void* out, float* scales,
                                int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M_in >= 0 && M >= M_in && K >= 0, "padded requant: bad shape");
    if (M == 0 || K == 0) return CINN_OK;
    CINN_CHECK_ARG(xq && xs && out && scales, "padded requant: null pointer");
    CINN_CHECK_ARG(K % 16 == 0 && aligned16(xq) && aligned16(out), "padded requant: K must be a multiple of 16 and buffers 16-byte aligned");
    CINN_CHECK_ARG(M < (1LL << 31) && K < (1LL << 31), "padded requant: dimension too large");
    const int nb = (int)((K + 127) / 128), mb = (int)((M + 127) / 128);
    CINN_CHECK_ARG(mb <= 65535, "padded requant: too many row blocks");
    dim3 grid((unsigned)nb, (unsigned)mb);
    if (div_mode == CINN_DIV_FULL)
        requant_row_to_block_kernel<CINN_DIV_FULL, false><<<grid, 256, 0, st>>>((const uint8_t*)xq, xs, nb, (uint8_t*)out, scales, (int)M, (int)K, nb, (int)M_in);
    else
        requant_row_to_block_kernel<CINN_DIV_RN, false><<<grid, 256, 0, st>>>((const uint8_t*)xq, xs, nb, (uint8_t*)out, scales, (int)M, (int)K, nb, (int)M_in);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// ---------------------------------------------------------------------------
// Per-expert segments padded to whole 128-row tiles, for the grouped weight gradient: from the experts' device-side
// row ranges, kb_start[e] = first tile of expert e (kb_start[E] = number of tiles), and per tile its first source row
// and its number of valid rows.  One CTA.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
segment_tiles_kernel(const int64_t* __restrict__ starts, const int64_t* __restrict__ ends, int E, int64_t T,
                     int* __restrict__ kb_start, int* __restrict__ tile_src, int* __restrict__ tile_cnt, int max_tiles) {
    __shared__ int s_first[1025];
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            long long s = starts[e], t = ends[e];
            if (s < 0) s = 0;
            if (t > T) t = T;
            const int n = t > s ? (int)(t - s) : 0;
            s_first[e] = run;
            run += (n + 127) / 128;
            if (run > max_tiles) run = max_tiles;           // cannot happen for disjoint ranges; keeps every index in range
        }
        s_first[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += 256) kb_start[e] = s_first[e];
    for (int e = 0; e < E; ++e) {
        long long s = starts[e], t = ends[e];
        if (s < 0) s = 0;
        if (t > T) t = T;
        const int n = t > s ? (int)(t - s) : 0;
        const int first = s_first[e], cnt = s_first[e + 1] - first;
        for (int g = threadIdx.x; g < cnt; g += 256) {
            tile_src[first + g] = (int)s + g * 128;
            tile_cnt[first + g] = min(128, n - g * 128);
        }
    }
}

int segment_tiles(const int64_t* starts, const int64_t* ends, int E, int64_t T, int* kb_start, int* tile_src, int* tile_cnt,
                  int max_tiles, cudaStream_t st) {
    CINN_CHECK_ARG(E >= 1 && E <= 1024 && T >= 0 && T < (1LL << 31) && max_tiles >= 1, "segment_tiles: 1 <= experts <= 1024");
    segment_tiles_kernel<<<1, 256, 0, st>>>(starts, ends, E, T, kb_start, tile_src, tile_cnt, max_tiles);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// dY (T, M = d_out; row pitch L) -> (M, max_tiles * 128) e4m3, tiles along the tokens of each expert's segment
template <typename T>
static int transposed_segmented_typed(const T* x, int64_t M, int64_t L, uint8_t* q, float* scales, int max_tiles,
                                      const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode, cudaStream_t st) {
    const int64_t slabs = (M + 63) / 64;
    int per = 4;
    while (per > 1 && slabs * ((max_tiles + per - 1) / per) < (int64_t)sm_count() * 8) per >>= 1;
    CINN_CHECK_ARG((max_tiles + per - 1) / per <= 65535, "segmented transposed quantiser: too many tiles");
    dim3 grid((unsigned)slabs, (unsigned)((max_tiles + per - 1) / per));
    const int N = max_tiles * 128;
    if (div_mode == CINN_DIV_FULL)
        quant_row_transposed_kernel<T, CINN_DIV_FULL, false, true><<<grid, 256, 0, st>>>(x, L, q, scales, (int)M, N, max_tiles, per, 0,
                                                                                          tile_src, tile_cnt, n_tiles);
    else
        quant_row_transposed_kernel<T, CINN_DIV_RN, false, true><<<grid, 256, 0, st>>>(x, L, q, scales, (int)M, N, max_tiles, per, 0,
                                                                                        tile_src, tile_cnt, n_tiles);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int quantize_transposed_segmented(const void* x, int dtype, int64_t M, int64_t L, void* q, float* scales, int max_tiles,
                                  const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M > 1 && M % 8 == 0 && L % 8 == 0 && L >= M && max_tiles >= 1, "segmented transposed quantiser: bad shape");
    CINN_CHECK_ARG(x && q && scales && tile_src && tile_cnt && n_tiles && aligned16(x) && aligned16(q),
                   "segmented transposed quantiser: null or unaligned pointer");
    switch (dtype) {
        case CINN_BF16: return transposed_segmented_typed((const __nv_bfloat16*)x, M, L, (uint8_t*)q, scales, max_tiles, tile_src, tile_cnt, n_tiles, div_mode, st);
        case CINN_F16: return transposed_segmented_typed((const __half*)x, M, L, (uint8_t*)q, scales, max_tiles, tile_src, tile_cnt, n_tiles, div_mode, st);
        case CINN_F32: return transposed_segmented_typed((const float*)x, M, L, (uint8_t*)q, scales, max_tiles, tile_src, tile_cnt, n_tiles, div_mode, st);
        default: set_error("segmented transposed quantiser: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

// dY (T, N) of a 2-byte type -> q_row (T, N) + s_row (T, N / 128) for the rows inside segments, and the transposed,
// segment-padded quantisation q_col (N, max_tiles * 128) + s_col (N, max_tiles); one pass (quant_row_dual_seg_kernel).
int quantize_dual_segmented(const void* x, int dtype, int64_t T, int64_t N, void* q_row, float* s_row, void* q_col, float* s_col,
                            int max_tiles, const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode,
                            cudaStream_t st) {
    CINN_CHECK_ARG((dtype == CINN_BF16 || dtype == CINN_F16) && T >= 1 && T < (1LL << 31) && N >= 128 && N % 128 == 0 &&
                   max_tiles >= 1 && max_tiles <= 65535, "segmented dual quantiser: 2-byte input, N a multiple of 128");
    CINN_CHECK_ARG(x && q_row && s_row && q_col && s_col && tile_src && tile_cnt && n_tiles && aligned16(x) && aligned16(q_row) &&
                   aligned16(q_col), "segmented dual quantiser: null or unaligned pointer");
    CUtensorMap tm;
    int rc = encode_map_2d(&tm, x, (uint64_t)N, (uint64_t)T, (uint64_t)N * 2, 128, 128, CU_TENSOR_MAP_DATA_TYPE_UINT16,
                           CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const int nb_n = (int)(N / 128);
    const int64_t total = (int64_t)nb_n * max_tiles;
    const int grid = (int)(total < 2 * (int64_t)sm_count() ? total : 2 * (int64_t)sm_count());
#define CINN_DS(TT, DIV)                                                                                              \
    do {                                                                                                              \
        auto kern = quant_row_dual_seg_kernel<TT, DIV>;                                                               \
        static std::once_flag once;                                                                                   \
        static cudaError_t attr_err = cudaSuccess;                                                                    \
        std::call_once(once, [&] {                                                                                    \
            attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DUAL_SMEM_BYTES);      \
        });                                                                                                           \
        CINN_CHECK_CUDA(attr_err);                                                                                    \
        kern<<<grid, 256, DUAL_SMEM_BYTES, st>>>(tm, (uint8_t*)q_row, s_row, (uint8_t*)q_col, s_col, max_tiles * 128, (int)N, \
                                                 nb_n, max_tiles, tile_src, tile_cnt, n_tiles);                       \
    } while (0)
    if (dtype == CINN_BF16) { if (div_mode == CINN_DIV_FULL) CINN_DS(__nv_bfloat16, CINN_DIV_FULL); else CINN_DS(__nv_bfloat16, CINN_DIV_RN); }
    else                    { if (div_mode == CINN_DIV_FULL) CINN_DS(__half, CINN_DIV_FULL);        else CINN_DS(__half, CINN_DIV_RN); }
#undef CINN_DS
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

// x_q (T, K) e4m3 + row scales -> block-scaled, transposed: (K, max_tiles * 128), scales (max_tiles, ceil(K/128))
int requant_row_to_block_segmented(const void* xq, const float* xs, int64_t K, void* out, float* scales, int max_tiles,
                                   const int* tile_src, const int* tile_cnt, const int* n_tiles, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(K > 0 && K % 16 == 0 && max_tiles >= 1 && max_tiles <= 65535, "segmented requant: bad shape");
    CINN_CHECK_ARG(xq && xs && out && scales && tile_src && tile_cnt && n_tiles && aligned16(xq) && aligned16(out),
                   "segmented requant: null or unaligned pointer");
    const int nb = (int)((K + 127) / 128);
    const int M = max_tiles * 128;
    if (K % 128 == 0) {
        // persistent, double-buffered, two CTAs per SM
        const int64_t tiles = (int64_t)nb * max_tiles;
        const int grid = (int)(tiles < (int64_t)sm_count() * 2 ? tiles : (int64_t)sm_count() * 2);
        if (div_mode == CINN_DIV_FULL)
            requant_seg_t_kernel<CINN_DIV_FULL><<<grid, 256, 0, st>>>((const uint8_t*)xq, xs, (uint8_t*)out, scales, M, (int)K, nb, tile_src, tile_cnt, n_tiles);
        else
            requant_seg_t_kernel<CINN_DIV_RN><<<grid, 256, 0, st>>>((const uint8_t*)xq, xs, (uint8_t*)out, scales, M, (int)K, nb, tile_src, tile_cnt, n_tiles);
        CINN_CHECK_LAUNCH();
        return CINN_OK;
    }
    dim3 grid((unsigned)nb, (unsigned)max_tiles);
    if (div_mode == CINN_DIV_FULL)
        requant_row_to_block_kernel<CINN_DIV_FULL, true, true><<<grid, 256, 0, st>>>((const uint8_t*)xq, xs, nb, (uint8_t*)out, scales, M, (int)K, nb, M,
                                                                                    tile_src, tile_cnt, n_tiles);
    else
        requant_row_to_block_kernel<CINN_DIV_RN, true, true><<<grid, 256, 0, st>>>((const uint8_t*)xq, xs, nb, (uint8_t*)out, scales, M, (int)K, nb, M,
                                                                                  tile_src, tile_cnt, n_tiles);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int read_quant_status(int* out, int reset) {
    int v = 0;
    CINN_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_quant_status, sizeof(int)));
    if (reset && v != 0) {
        int z = 0;
        CINN_CHECK_CUDA(cudaMemcpyToSymbol(g_quant_status, &z, sizeof(int)));
    }
    *out = v;
    return CINN_OK;
}

int quantize_dual(const void* x, int dtype, int64_t M, int64_t N, int64_t ld, void* q_row, float* s_row, void* q_col,
                  float* s_col, int round_scale, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M >= 0 && N >= 0, "dual quantiser: negative shape (%lld, %lld)", (long long)M, (long long)N);
    if (M == 0 || N == 0) return CINN_OK;
    CINN_CHECK_ARG(x && q_row && s_row && q_col && s_col, "dual quantiser: null pointer");
    CINN_CHECK_ARG(N < (1LL << 31) && M < (1LL << 31), "dual quantiser: dimension too large");
    CINN_CHECK_ARG(ld >= N, "dual quantiser: row pitch %lld below the row length %lld", (long long)ld, (long long)N);
    CINN_CHECK_ARG(div_mode == CINN_DIV_FULL || div_mode == CINN_DIV_RN, "dual quantiser: unknown div_mode %d", div_mode);
    switch (dtype) {
        case CINN_BF16: return dispatch_dual((const __nv_bfloat16*)x, M, N, ld, (uint8_t*)q_row, s_row, (uint8_t*)q_col, s_col, round_scale, div_mode, st);
        case CINN_F16:  return dispatch_dual((const __half*)x, M, N, ld, (uint8_t*)q_row, s_row, (uint8_t*)q_col, s_col, round_scale, div_mode, st);
        case CINN_F32:  return dispatch_dual((const float*)x, M, N, ld, (uint8_t*)q_row, s_row, (uint8_t*)q_col, s_col, round_scale, div_mode, st);
        default: set_error("dual quantiser: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

int requant_row_to_block(const void* xq, const float* xs, int64_t M, int64_t K, void* out, float* scales,
                         int transpose_out, int div_mode, cudaStream_t st) {
    CINN_CHECK_ARG(M >= 0 && K >= 0, "requant: negative shape");
    if (M == 0 || K == 0) return CINN_OK;
    CINN_CHECK_ARG(xq && xs && out && scales, "requant: null pointer");
    CINN_CHECK_ARG(K % 16 == 0 && aligned16(xq) && aligned16(out), "requant: K must be a multiple of 16 and buffers 16-byte aligned");
    CINN_CHECK_ARG(!transpose_out || M % 16 == 0, "requant: transposed output needs M %% 16 == 0");
    CINN_CHECK_ARG(M < (1LL << 31) && K < (1LL << 31), "requant: dimension too large");
    const int nb = (int)((K + 127) / 128), mb = (int)((M + 127) / 128);
    CINN_CHECK_ARG(mb <= 65535, "requant: too many row blocks");
    dim3 grid((unsigned)nb, (unsigned)mb);
    const uint8_t* in = (const uint8_t*)xq;
    uint8_t* o = (uint8_t*)out;
    if (div_mode == CINN_DIV_FULL) {
        if (transpose_out) requant_row_to_block_kernel<CINN_DIV_FULL, true><<<grid, 256, 0, st>>>(in, xs, nb, o, scales, (int)M, (int)K, nb, (int)M);
        else requant_row_to_block_kernel<CINN_DIV_FULL, false><<<grid, 256, 0, st>>>(in, xs, nb, o, scales, (int)M, (int)K, nb, (int)M);
    } else {
        if (transpose_out) requant_row_to_block_kernel<CINN_DIV_RN, true><<<grid, 256, 0, st>>>(in, xs, nb, o, scales, (int)M, (int)K, nb, (int)M);
        else requant_row_to_block_kernel<CINN_DIV_RN, false><<<grid, 256, 0, st>>>(in, xs, nb, o, scales, (int)M, (int)K, nb, (int)M);
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int dequantize(const void* q, const float* scales, void* out, int out_dtype, int64_t M, int64_t N, int bm, int bn,
               cudaStream_t st) {
    CINN_CHECK_ARG(M >= 0 && N >= 0, "dequantise: negative shape");
    if (M == 0 || N == 0) return CINN_OK;
    CINN_CHECK_ARG(q && scales && out, "dequantise: null pointer");
    CINN_CHECK_ARG(bm >= 1 && bn >= 1, "dequantise: bad tile");
    CINN_CHECK_ARG(N < (1LL << 31), "dequantise: N too large");
    const int ncb = (int)((N + bn - 1) / bn);
    int64_t blocks = (M * N + 1023) / 1024;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (out_dtype == CINN_BF16)
        dequant_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)q, scales, (__nv_bfloat16*)out, M, (int)N, bm, bn, ncb);
    else if (out_dtype == CINN_F32)
        dequant_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)q, scales, (float*)out, M, (int)N, bm, bn, ncb);
    else { set_error("dequantise: output dtype must be bf16 or fp32"); return CINN_ERR_INVALID; }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

template <typename T>
static int launch_swiglu(const T* h12, int64_t T_rows, int64_t I, uint8_t* q, float* scales, int div_mode, cudaStream_t st,
                         const int64_t* n_rows_dev) {
    const int nb = (int)((I + 127) / 128);
    const int64_t tiles = T_rows * nb;
    int64_t blocks = (tiles + 15) / 16;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    const int64_t n_hw = blocks * 16;
    const int sr = (int)(n_hw / nb), sc = (int)(n_hw % nb);
    if (div_mode == CINN_DIV_FULL) swiglu_quant_row_kernel<T, CINN_DIV_FULL><<<(unsigned)blocks, 256, 0, st>>>(h12, q, scales, (int)I, nb, tiles, sr, sc, n_rows_dev);
    else swiglu_quant_row_kernel<T, CINN_DIV_RN><<<(unsigned)blocks, 256, 0, st>>>(h12, q, scales, (int)I, nb, tiles, sr, sc, n_rows_dev);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int swiglu_quant_rowwise(const void* h12, int dtype, int64_t T_rows, int64_t I, void* q, float* scales, int div_mode,
                         cudaStream_t st, const int64_t* n_rows_dev) {
    CINN_CHECK_ARG(T_rows >= 0 && I >= 0, "swiglu_quant: negative shape");
    if (T_rows == 0 || I == 0) return CINN_OK;
    CINN_CHECK_ARG(h12 && q && scales, "swiglu_quant: null pointer");
    CINN_CHECK_ARG(I % 8 == 0 && I < (1LL << 30), "swiglu_quant: the hidden width (%lld) must be a multiple of 8", (long long)I);
    CINN_CHECK_ARG(aligned16(h12) && (reinterpret_cast<uintptr_t>(q) & 7) == 0, "swiglu_quant: buffers must be 16-byte aligned");
    CINN_CHECK_ARG(div_mode == CINN_DIV_FULL || div_mode == CINN_DIV_RN, "swiglu_quant: unknown div_mode %d", div_mode);
    switch (dtype) {
        case CINN_BF16: return launch_swiglu((const __nv_bfloat16*)h12, T_rows, I, (uint8_t*)q, scales, div_mode, st, n_rows_dev);
        case CINN_F16: return launch_swiglu((const __half*)h12, T_rows, I, (uint8_t*)q, scales, div_mode, st, n_rows_dev);
        case CINN_F32: return launch_swiglu((const float*)h12, T_rows, I, (uint8_t*)q, scales, div_mode, st, n_rows_dev);
        default: set_error("swiglu_quant: unknown dtype tag %d", dtype); return CINN_ERR_INVALID;
    }
}

int transpose_bytes(const void* in, int64_t ld_in, void* out, int64_t R, int64_t C, cudaStream_t st) {
    if (R == 0 || C == 0) return CINN_OK;
    CINN_CHECK_ARG(in && out, "transpose: null pointer");
    CINN_CHECK_ARG(R < (1LL << 31) && C < (1LL << 31) && (R + 63) / 64 <= 65535, "transpose: shape too large");
    const bool vec = R % 4 == 0 && C % 4 == 0 && ld_in % 4 == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 3) == 0 &&
                     (R + 127) / 128 <= 65535;
    if (vec) {
        dim3 grid((unsigned)((C + 127) / 128), (unsigned)((R + 127) / 128));
        transpose_bytes_vec_kernel<<<grid, 256, 0, st>>>((const uint8_t*)in, ld_in, (uint8_t*)out, (int)R, (int)C);
    } else {
        dim3 grid((unsigned)((C + 63) / 64), (unsigned)((R + 63) / 64));
        transpose_bytes_kernel<<<grid, 256, 0, st>>>((const uint8_t*)in, ld_in, (uint8_t*)out, (int)R, (int)C);
    }
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

}  // namespace cinn
