// Block-scaled FP8 GEMM for sm_100a: tcgen05 MMAs on e4m3 tiles that TMA stages in
// shared memory, fp32 partial sums in tensor memory (TMEM), and a CUDA-core
// "promotion" of every 128-deep K block: partial * sA[row, kb] * sB[kb, nb] is
// added to fp32 registers.  Semantics of cinnamon's fp8_gemm_kernel
// (src/kernels.py:618-664); the grouped variant follows grouped_gemm_kernel
// (src/kernels.py:466-523) with the same e4m3 operands and scales.
//
// One persistent CTA per SM, 11 warps:
//   warps 0-7   promotion + epilogue: tcgen05.ld a K block's partial tile, scale, accumulate; a finished tile leaves
//               through TMA stores (2-byte outputs, whole tiles) or staged 16-byte stores with row/column predicates
//               (fp32 outputs, ragged expert tails, rows scattered to per-row addresses)
//   warp  8     TMA producer (one lane): A 128x128 B and B 256x128 B tiles, 128-byte swizzle, 4-stage ring
//   warps 9-10  MMA issuers (one lane each) on alternate K blocks: four 128x256x32 MMAs per block into one of two
//               256-column TMEM buffers, so block i+1 runs while block i is promoted; warp 9 owns the TMEM allocation
// Every wait is bounded: when one runs out the kernel records a code in a device status
// word, every role leaves its loop, TMEM is freed and the kernel returns.
#include "common.cuh"
#include "tma.cuh"
#include <cuda.h>
#include <mutex>
#include <atomic>
#include <cstdlib>

namespace cinn {

constexpr int BM = 128;            // tile rows
constexpr int BN = 256;            // tile columns (two 128-column scale blocks)
constexpr int BK = 128;            // bytes (= e4m3 elements) per K block: one scale block, one swizzle row
constexpr int STAGES = 4;             // even: each of the two MMA issuers then always meets the same stages, so it
                                      // sees every phase of their barriers (a parity wait cannot skip a phase)
constexpr int C_SLOT_BYTES = BM * 128;   // one TMA-store box: 128 rows x 64 columns of a 2-byte type
constexpr int C_STAGE_BYTES = 2 * C_SLOT_BYTES;   // one slot per column group of promotion warps
constexpr int A_BYTES = BM * BK;   // 16 KiB
constexpr int B_BYTES = BN * BK;   // 32 KiB
constexpr int EPI_WARPS = 8;                    // four TMEM lane quarters x two column groups
constexpr int WCOLS = BN / (EPI_WARPS / 4);     // accumulator columns per epilogue warp
constexpr int THREADS = (EPI_WARPS + 3) * 32;     // + TMA producer + two MMA issuers
constexpr int TMEM_COLS = 512;
constexpr int MAX_EXPERTS = 384;      // bounded by the shared memory left for the per-expert prefix sums
constexpr int GROUP_M = 16;        // rasterisation: m-tiles per L2 group (dense)

// device status word: 0 = fine, otherwise (role << 8) | reason
__device__ int g_device_status = 0;

struct GemmParams {
    const float* sA; int64_t sa_stride_m, sa_stride_k;
    const float* sB; int64_t sb_stride_k, sb_stride_n, sb_stride_e;
    void* C; int64_t ldc;          // scatter variant: C is a table of byte addresses, one per output row (0 = drop the row)
    int M, N, K;                   // dense: A is (M, K); grouped: M = total rows T
    const int64_t* starts; const int64_t* ends; int E; int b_rows_per_expert;
    int tma_out;                   // 1: finished tiles leave through TMA stores (2-byte outputs, N % 8 == 0)
};

// ---------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;   // about two seconds

// Bounded wait.  Returns false when the kernel is being abandoned.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(&g_device_status, 0, code);
                return false;
            }
        }
    }
}

// The same wait taken by a whole warp, with one verdict for all its lanes: the promotion warps execute
// warp-collective tcgen05.ld next, so no lane may leave the wait on its own.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    const bool ok = mbar_wait(bar, parity, abort_flag, code);
    return __all_sync(0xffffffffu, ok);
}

// fp32 load through the read-only path, pinned in program order
__device__ __forceinline__ float ld_scale(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], e4m3 x e4m3 -> fp32
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 16 consecutive fp32 columns: thread i receives TMEM lane (base lane + i)
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell descriptor version 1.
// lbo / sbo in bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;     // descriptor version
    d |= (uint64_t)2 << 61;     // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f8f6f4: fp32 accumulate, e4m3 x e4m3, A K-major.
__host__ __device__ constexpr uint32_t make_idesc(bool b_mn_major) {
    return (1u << 4)                              // D format: fp32
           | (0u << 7) | (0u << 10)               // A, B format: e4m3
           | (0u << 15)                           // A major: K
           | ((b_mn_major ? 1u : 0u) << 16)       // B major
           | ((uint32_t)(BN >> 3) << 17)          // N
           | ((uint32_t)(BM >> 4) << 24);         // M
}

// ---------------------------------------------------------------------------
// tile schedule shared by all roles
// ---------------------------------------------------------------------------
struct TileInfo {
    int m0;        // first row of A / C
    int m_end;     // one past the last valid row for this tile
    int n0;        // first output column
    int expert;
};

template <bool GROUPED>
__device__ __forceinline__ int total_tiles(const GemmParams& p, const int* cum) {
    const int n_tiles = (p.N + BN - 1) / BN;
    if constexpr (GROUPED) return cum[p.E] * n_tiles;
    else return ((p.M + BM - 1) / BM) * n_tiles;
}

template <bool GROUPED>
__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, const int* cum, int t) {
    TileInfo ti;
    const int n_tiles = (p.N + BN - 1) / BN;
    if constexpr (GROUPED) {
        const int mt = t / n_tiles;
        ti.n0 = (t - mt * n_tiles) * BN;
        int lo = 0, hi = p.E;                      // largest e with cum[e] <= mt
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (cum[mid] <= mt) lo = mid; else hi = mid;
        }
        ti.expert = lo;
        const long long s = p.starts[lo], e = p.ends[lo];
        ti.m0 = (int)s + (mt - cum[lo]) * BM;
        ti.m_end = (int)(e < (long long)p.M ? e : (long long)p.M);
    } else {
        const int m_tiles = (p.M + BM - 1) / BM;
        const int per_group = GROUP_M * n_tiles;
        const int g = t / per_group;
        const int first_m = g * GROUP_M;
        const int gsize = min(GROUP_M, m_tiles - first_m);
        const int r = t - g * per_group;
        ti.m0 = (first_m + r % gsize) * BM;
        ti.n0 = (r / gsize) * BN;
        ti.m_end = p.M;
        ti.expert = 0;
    }
    return ti;
}

template <int OUT> struct OutT;
template <> struct OutT<CINN_BF16> { using type = __nv_bfloat16; };
template <> struct OutT<CINN_F16> { using type = __half; };
template <> struct OutT<CINN_F32> { using type = float; };
template <> struct OutT<CINN_F32_BF16> { using type = float; };   // fp32 storage of the bf16-rounded value

template <int OUT>
__device__ __forceinline__ void store8(void* C, int64_t off, const float* a, bool vec, int ncols) {
    using T = typename OutT<OUT>::type;
    T* dst = reinterpret_cast<T*>(C) + off;
    float b[8];
    if constexpr (OUT == CINN_F32_BF16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = __bfloat162float(__float2bfloat16_rn(a[i]));
        a = b;
    }
    if (vec && ncols >= 8) {
        if constexpr (OUT == CINN_F32 || OUT == CINN_F32_BF16) {
            reinterpret_cast<float4*>(dst)[0] = make_float4(a[0], a[1], a[2], a[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(a[4], a[5], a[6], a[7]);
        } else if constexpr (OUT == CINN_BF16) {
            uint4 v;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(a[0], a[1]), t1 = __floats2bfloat162_rn(a[2], a[3]);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(a[4], a[5]), t3 = __floats2bfloat162_rn(a[6], a[7]);
            v.x = *reinterpret_cast<uint32_t*>(&t0); v.y = *reinterpret_cast<uint32_t*>(&t1);
            v.z = *reinterpret_cast<uint32_t*>(&t2); v.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(dst) = v;
        } else {
            uint4 v;
            __half2 t0 = __floats2half2_rn(a[0], a[1]), t1 = __floats2half2_rn(a[2], a[3]);
            __half2 t2 = __floats2half2_rn(a[4], a[5]), t3 = __floats2half2_rn(a[6], a[7]);
            v.x = *reinterpret_cast<uint32_t*>(&t0); v.y = *reinterpret_cast<uint32_t*>(&t1);
            v.z = *reinterpret_cast<uint32_t*>(&t2); v.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(dst) = v;
        }
    } else {
        for (int i = 0; i < 8 && i < ncols; ++i) {
            if constexpr (OUT == CINN_F32 || OUT == CINN_F32_BF16) dst[i] = a[i];
            else if constexpr (OUT == CINN_BF16) dst[i] = __float2bfloat16_rn(a[i]);
            else dst[i] = __float2half_rn(a[i]);
        }
    }
}

// Tile store through shared memory.  Each promotion thread owns one output row; storing it directly would
// make every warp-wide store touch 32 different rows (32 cache lines per instruction).  Instead the warp
// stages 64 bytes of each of its 32 rows (XOR-swizzled 16-byte slots, conflict-free both ways) and writes
// them back out as 8 rows x 64 contiguous bytes per instruction.  `stage` is this warp's 2 KiB.
template <int OUT>
__device__ __forceinline__ uint4 pack16(const float* a) {
    uint4 v;
    if constexpr (OUT == CINN_F32) {
        v = make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
    } else if constexpr (OUT == CINN_F32_BF16) {
        // two packed conversions, then each half widened again by a shift / a mask
        __nv_bfloat162 t0 = __floats2bfloat162_rn(a[0], a[1]), t1 = __floats2bfloat162_rn(a[2], a[3]);
        const uint32_t p0 = *reinterpret_cast<uint32_t*>(&t0), p1 = *reinterpret_cast<uint32_t*>(&t1);
        v = make_uint4(p0 << 16, p0 & 0xffff0000u, p1 << 16, p1 & 0xffff0000u);
    } else if constexpr (OUT == CINN_BF16) {
        __nv_bfloat162 t0 = __floats2bfloat162_rn(a[0], a[1]), t1 = __floats2bfloat162_rn(a[2], a[3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(a[4], a[5]), t3 = __floats2bfloat162_rn(a[6], a[7]);
        v = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1), *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
    } else {
        __half2 t0 = __floats2half2_rn(a[0], a[1]), t1 = __floats2half2_rn(a[2], a[3]);
        __half2 t2 = __floats2half2_rn(a[4], a[5]), t3 = __floats2half2_rn(a[6], a[7]);
        v = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1), *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
    }
    return v;
}

template <int OUT, int NCOLS, bool SCATTER = false>
__device__ __forceinline__ void store_rows_staged(const float* acc, uint8_t* stage, void* C, int64_t ldc, int row0, int m_end,
                                                  int col0, int N, int lane) {
    using T = typename OutT<OUT>::type;
    constexpr int PER16 = 16 / (int)sizeof(T);      // elements per 16-byte slot
    constexpr int PER64 = 4 * PER16;                // elements per staged row piece
#pragma unroll
    for (int ps = 0; ps < NCOLS / PER64; ++ps) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(stage + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)) = pack16<OUT>(&acc[ps * PER64 + c * PER16]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = i * 8 + (lane >> 2), c = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
            const int grow = row0 + r, gcol = col0 + ps * PER64 + c * PER16;
            if constexpr (SCATTER) {
                // C is a table of byte addresses, one per row; the rows may live in another GPU's memory
                if (grow < m_end && gcol < N) {
                    T* dst = reinterpret_cast<T*>(reinterpret_cast<const long long*>(C)[grow]);
                    if (dst) *reinterpret_cast<uint4*>(dst + gcol) = v;
                }
            } else {
                if (grow < m_end && gcol < N) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(C) + (int64_t)grow * ldc + gcol) = v;
            }
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <bool B_MN, bool GROUPED, int OUT, bool SCATTER = false>
__global__ void __launch_bounds__(THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // layout: operand stages | output staging (32 KiB, 1024-aligned) | barriers and flags (256 B) | expert prefix sums
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint8_t* c_stage = smem + STAGES * (A_BYTES + B_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(c_stage + C_STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem full, [2S+2..2S+4) tmem empty, then slot free / slot full x 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* store_stage = c_stage;                                        // 2 KiB per promotion warp (non-TMA path)
    int* cum = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);   // grouped: E + 1 prefix counts of m-tiles

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
    const uint32_t gfree0 = smem_u32(bars + 2 * STAGES + 4), gfull0 = smem_u32(bars + 2 * STAGES + 6);

    if (threadIdx.x == 0) *abort_flag = 0;
    if (warp == EPI_WARPS && lane == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, EPI_WARPS); }
        for (int g = 0; g < 2; ++g) { mbar_init(gfree0 + 8 * g, 4); mbar_init(gfull0 + 8 * g, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == EPI_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if constexpr (GROUPED) {
        if (warp == 0) {                           // prefix sum of per-expert m-tile counts
            int carry = 0;
            for (int base = 0; base < p.E; base += 32) {
                const int e = base + lane;
                int cnt = 0;
                if (e < p.E) {
                    long long s = p.starts[e], t = p.ends[e];
                    if (t > (long long)p.M) t = p.M;
                    if (s < 0) s = 0;
                    if (t > s) cnt = (int)((t - s + BM - 1) / BM);
                }
                int incl = cnt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                if (e < p.E) cum[e] = carry + incl - cnt;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) cum[p.E] = carry;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int KB = (p.K + BK - 1) / BK;
    const int n_total = total_tiles<GROUPED>(p, cum);

    if (warp >= EPI_WARPS) {
      if (warp == EPI_WARPS) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < n_total && alive; t += gridDim.x) {
                const TileInfo ti = tile_info<GROUPED>(p, cum, t);
                const int b_row0 = GROUPED ? ti.expert * p.b_rows_per_expert : 0;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, (1 << 8) | 1)) { alive = false; break; }
                    const uint32_t fb = full0 + 8 * s;
                    mbar_expect_tx(fb, A_BYTES + B_BYTES);
                    tma_load_2d(&tmA, fb, smem_u32(smem_a + s * A_BYTES), kb * BK, ti.m0);
                    if constexpr (!B_MN) {
                        tma_load_2d(&tmB, fb, smem_u32(smem_b + s * B_BYTES), kb * BK, b_row0 + ti.n0);
                    } else {
                        tma_load_2d(&tmB, fb, smem_u32(smem_b + s * B_BYTES), ti.n0, b_row0 + kb * BK);
                        tma_load_2d(&tmB, fb, smem_u32(smem_b + s * B_BYTES + B_BYTES / 2), ti.n0 + 128, b_row0 + kb * BK);
                    }
                }
            }
            if (!alive) {
                // abandoned: let the copies already issued land before shared memory is given up
                const uint32_t issued = it;
                for (uint32_t j = (issued > STAGES ? issued - STAGES : 0); j < issued; ++j) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
                    }
                }
            }
        }
    } else {
        // ------------------------------ MMA issuers ------------------------------
        // Two warps take alternate K blocks (one TMEM buffer each).  Issuing a block's MMAs blocks the
        // issuing thread for about as long as they execute, and every barrier probe costs a few
        // hundred cycles next to a busy tensor pipe; with two issuers one probes while the other feeds.
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(B_MN);
            const uint32_t mine = (uint32_t)(warp - (EPI_WARPS + 1));
            uint32_t it = 0, last = 0xffffffffu;
            bool alive = true;
            for (int t = blockIdx.x; t < n_total && alive; t += gridDim.x) {
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    if ((it & 1u) != mine) continue;
                    last = it;
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const uint32_t b = it & 1, bph = (it >> 1) & 1;
                    // operands first (they landed long ago: this costs one barrier probe, taken while
                    // the epilogue still works on the buffer), then the TMEM buffer
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, (2 << 8) | 1)) { alive = false; break; }
                    if (!mbar_wait(tempty0 + 8 * b, bph ^ 1, abort_flag, (2 << 8) | 2)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + s * A_BYTES);
                    const uint32_t b_addr = smem_u32(smem_b + s * B_BYTES);
                    const uint32_t d = tmem_base + b * BN;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 32 * 128, B_BYTES / 2, 1024)
                                                 : make_smem_desc(b_addr + k * 32, 16, 1024);
                        tc_mma_f8(d, ad, bd, idesc, k > 0 ? 1u : 0u);
                    }
                    tc_commit(empty0 + 8 * s);      // the stage may be refilled once these MMAs retire
                    tc_commit(tfull0 + 8 * b);      // and the partial tile is ready for promotion
                }
            }
            // every MMA issued above must have retired before tensor memory is freed
            if (alive && last != 0xffffffffu) mbar_wait(tfull0 + 8 * (last & 1), (last >> 1) & 1, abort_flag, (2 << 8) | 3);
        }
      }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3, h = warp >> 2;
        uint32_t it = 0;
        bool alive = true;
        const bool vec_ok = (OUT == CINN_F32 || OUT == CINN_F32_BF16) ? (p.ldc % 4 == 0) : (p.ldc % 8 == 0);
        // The first three scale pairs of a tile are fetched while the previous tile is being stored, so that
        // a tile does not start with an exposed round trip to L2 (it matters when K is only a few blocks).
        uint32_t n_rounds = 0;                   // staging rounds of this column group so far (two per TMA tile)
        float sa0 = 0.f, sb0 = 0.f, sa1 = 0.f, sb1 = 0.f, sa2 = 0.f, sb2 = 0.f;
        auto scale_ptrs = [&](const TileInfo& ti, const float*& sa_ptr, const float*& sb_ptr) {
            const int row = ti.m0 + q * 32 + lane;
            const int col0 = ti.n0 + h * WCOLS;
            sa_ptr = p.sA + (int64_t)(row < ti.m_end ? row : ti.m0) * p.sa_stride_m;
            sb_ptr = p.sB + (int64_t)ti.expert * p.sb_stride_e + (int64_t)(col0 < p.N ? col0 / 128 : 0) * p.sb_stride_n;
        };
        auto prefetch_scales = [&](const TileInfo& ti) {
            const float *sa_ptr, *sb_ptr;
            scale_ptrs(ti, sa_ptr, sb_ptr);
            sa0 = ld_scale(sa_ptr); sb0 = ld_scale(sb_ptr);
            if (KB > 1) { sa1 = ld_scale(sa_ptr + p.sa_stride_k); sb1 = ld_scale(sb_ptr + p.sb_stride_k); }
            if (KB > 2) { sa2 = ld_scale(sa_ptr + 2 * p.sa_stride_k); sb2 = ld_scale(sb_ptr + 2 * p.sb_stride_k); }
        };
        if ((int)blockIdx.x < n_total) prefetch_scales(tile_info<GROUPED>(p, cum, blockIdx.x));
        for (int t = blockIdx.x; t < n_total && alive; t += gridDim.x) {
            const TileInfo ti = tile_info<GROUPED>(p, cum, t);
            const int row = ti.m0 + q * 32 + lane;
            const bool rvalid = row < ti.m_end;
            const int col0 = ti.n0 + h * WCOLS;
            const bool cvalid = col0 < p.N;
            const float *sa_ptr, *sb_ptr;
            scale_ptrs(ti, sa_ptr, sb_ptr);
            float acc[WCOLS];
#pragma unroll
            for (int i = 0; i < WCOLS; ++i) acc[i] = 0.0f;
            // within a tile scales are fetched three K blocks ahead with loads the compiler may not move
            // (a load sunk to its use would expose a full L2 round trip in every K block)
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const float s = sa0 * sb0;
                sa0 = sa1; sb0 = sb1; sa1 = sa2; sb1 = sb2;
                if (kb + 3 < KB) {
                    sa2 = ld_scale(sa_ptr + (int64_t)(kb + 3) * p.sa_stride_k);
                    sb2 = ld_scale(sb_ptr + (int64_t)(kb + 3) * p.sb_stride_k);
                }
                const uint32_t b = it & 1, bph = (it >> 1) & 1;
                if (!mbar_wait_warp(tfull0 + 8 * b, bph, abort_flag, (3 << 8) | 1)) { alive = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * BN + h * WCOLS;
                // packed fp32x2 FMAs: half the issue slots of 128 scalar ones, the same IEEE result in every lane
                uint64_t s2;
                asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "f"(s));
#pragma unroll
                for (int c = 0; c < WCOLS / 16; ++c) {
                    float v[16];
                    tc_ld16(taddr + c * 16, v);
#pragma unroll
                    for (int j = 0; j < 16; j += 2)
                        asm("{\n\t.reg .b64 a, x;\n\t"
                            "mov.b64 a, {%0, %1};\n\t"
                            "mov.b64 x, {%2, %3};\n\t"
                            "fma.rn.f32x2 a, x, %4, a;\n\t"
                            "mov.b64 {%0, %1}, a;\n\t}"
                            : "+f"(acc[c * 16 + j]), "+f"(acc[c * 16 + j + 1]) : "f"(v[j]), "f"(v[j + 1]), "l"(s2));
                }
                // (Measured alternatives, all slower on B200: wider TMEM loads with a larger register budget,
                // double-buffered loads, sixteen promotion warps.  Packed FMAs are worth 1 - 2 %.)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * b);
            }
            if (alive && t + (int)gridDim.x < n_total) prefetch_scales(tile_info<GROUPED>(p, cum, t + gridDim.x));
            constexpr bool TMA_OUT = (OUT == CINN_BF16 || OUT == CINN_F16);
            // A tile whose 128 rows all belong to it leaves through TMA stores.  Each column group of four
            // promotion warps owns one 16 KiB slot: its threads drop 64 columns of their rows into it (16-byte
            // chunks, 128-byte swizzle), one thread hands the box to the TMA unit, and the group repeats for its
            // other 64 columns once the unit has read the slot.  Storing one row per thread straight from
            // registers costs thousands of cycles per tile, and so do shared-memory round trips next to a busy
            // tensor pipe.
            const bool whole = !GROUPED || ti.m0 + BM <= ti.m_end;
            if (TMA_OUT && alive && p.tma_out && whole) {
                const bool elected = (warp == h * 4) && lane == 0;
                const uint32_t slot = smem_u32(c_stage) + h * C_SLOT_BYTES;
                const int rl = q * 32 + lane;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t par = n_rounds & 1u;
                    if (elected) tma_store_wait_read();               // the unit has finished reading this slot
                    __syncwarp();
                    if (lane == 0) mbar_arrive(gfree0 + 8 * h);
                    if (!mbar_wait_warp(gfree0 + 8 * h, par, abort_flag, (3 << 8) | 2)) { alive = false; break; }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 v = pack16<OUT>(&acc[r * 64 + j * 8]);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(slot + rl * 128 + ((j ^ (rl & 7)) << 4)),
                                     "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(gfull0 + 8 * h);
                    if (elected) {
                        const int col = col0 + r * 64;
                        if (mbar_wait(gfull0 + 8 * h, par, abort_flag, (3 << 8) | 3)) {
                            if (col < p.N) tma_store_2d(&tmC, slot, col, ti.m0);
                            tma_store_commit();
                        }
                    }
                    __syncwarp();   // the elected lane rejoins its warp before the next warp-collective instruction
                    ++n_rounds;
                }
                if (!alive) break;
            } else if (alive && vec_ok && !(TMA_OUT && p.tma_out)) {
                // warp-uniform: every lane takes part in the staging even if its own row is past the end
                if (cvalid) store_rows_staged<OUT, WCOLS, SCATTER>(acc, store_stage + warp * 2048, p.C, p.ldc, ti.m0 + q * 32, ti.m_end, col0, p.N, lane);
            } else if (alive && rvalid && cvalid) {
                const int64_t base = (int64_t)row * p.ldc + col0;
#pragma unroll
                for (int j = 0; j < WCOLS / 8; ++j) {
                    const int ncols = p.N - (col0 + j * 8);
                    if (ncols > 0) store8<OUT>(p.C, base + j * 8, &acc[j * 8], vec_ok, ncols);
                }
            }
        }
        if (lane == 0 && (warp & 3) == 0) tma_store_wait_all();      // this group's boxes have reached global memory
    }

    tc_fence_before();
    __syncthreads();
    if (warp == EPI_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

#include "gemm_pair.cuh"
#include "gemm16.cuh"

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    });
    return fn;
}

int encode_map_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                  uint32_t box_inner, uint32_t box_rows, CUtensorMapDataType dtype, CUtensorMapSwizzle swizzle) {
    EncodeFn enc = get_encode();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the CUDA driver"); return CINN_ERR_CUDA; }
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
        // a thread that has made no runtime call yet (an autograd worker, say) has no context bound:
        // let the runtime bind the device's primary context, then encode again
        cudaFree(nullptr);
        r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (base %p inner %llu rows %llu pitch %llu)", (int)r, base,
                  (unsigned long long)inner, (unsigned long long)rows, (unsigned long long)pitch_bytes);
        return CINN_ERR_CUDA;
    }
    return CINN_OK;
}

// GEMM operands and outputs: 128-byte swizzle; `pitch` in BYTES
static int make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8) {
    return encode_map_2d(map, base, inner, rows, pitch, box_inner, box_rows, dtype, CU_TENSOR_MAP_SWIZZLE_128B);
}

static size_t smem_bytes(int E) {
    size_t n = (size_t)STAGES * (A_BYTES + B_BYTES) + C_STAGE_BYTES + 1024 + 256 + 4 * (size_t)(E + 2);
    return n;
}

// Output map for the TMA-store epilogue: (rows, N) of a 2-byte type, boxes of 64 columns x 128 rows, 128-byte swizzle.
// Sets p.tma_out; when the output cannot go through TMA the (unused) operand map is passed in its place.
static int make_out_map(CUtensorMap* tc, const CUtensorMap& fallback, GemmParams& p, int out_dtype, int64_t rows,
                        bool fp32_boxes = false) {
    p.tma_out = 0;
    *tc = fallback;
    if (((uintptr_t)p.C & 15) != 0) return CINN_OK;               // TMA wants a 16-byte aligned base; plain stores otherwise
    if (fp32_boxes && (out_dtype == CINN_F32 || out_dtype == CINN_F32_BF16) && p.N % 4 == 0) {
        // the two-SM kernel also sends 4-byte outputs through TMA: boxes of 32 columns x 128 rows
        int rc = make_map(tc, p.C, (uint64_t)p.N, (uint64_t)rows, (uint64_t)p.ldc * 4, 32, BM, CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
        if (rc) return rc;
        p.tma_out = 1;
        return CINN_OK;
    }
    if ((out_dtype == CINN_BF16 || out_dtype == CINN_F16) && p.N % 8 == 0) {
        int rc = make_map(tc, p.C, (uint64_t)p.N, (uint64_t)rows, (uint64_t)p.ldc * 2, 64, BM,
                          out_dtype == CINN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
        if (rc) return rc;
        p.tma_out = 1;
    }
    return CINN_OK;
}

template <bool B_MN, bool GROUPED, int OUT, bool SCATTER = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int grid,
                  cudaStream_t st) {
    auto kern = fp8_gemm_kernel<B_MN, GROUPED, OUT, SCATTER>;
    const size_t smem = smem_bytes(GROUPED ? p.E : 0);
    static thread_local size_t configured[64] = {};   // per instantiation, per thread, per device
    int dev = 0;
    CINN_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        CINN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    kern<<<grid, THREADS, smem, st>>>(ta, tb, tc, p);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

template <bool B_MN, bool GROUPED>
static int launch_out(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int out_dtype, int grid,
                      cudaStream_t st) {
    CUtensorMap tc;
    int rc = make_out_map(&tc, ta, p, out_dtype, p.M);
    if (rc) return rc;
    switch (out_dtype) {
        case CINN_BF16: return launch<B_MN, GROUPED, CINN_BF16>(ta, tb, tc, p, grid, st);
        case CINN_F32: return launch<B_MN, GROUPED, CINN_F32>(ta, tb, tc, p, grid, st);
        case CINN_F16: return launch<B_MN, GROUPED, CINN_F16>(ta, tb, tc, p, grid, st);
        case CINN_F32_BF16: return launch<B_MN, GROUPED, CINN_F32_BF16>(ta, tb, tc, p, grid, st);
        default: set_error("GEMM: unknown output dtype tag %d", out_dtype); return CINN_ERR_INVALID;
    }
}

template <bool B_MN, int OUT>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int clusters,
                       cudaStream_t st) {
    auto kern = pair::fp8_gemm_pair_kernel<B_MN, OUT>;
    const size_t smem = pair::PSMEM_BYTES;
    static thread_local bool configured[64] = {};
    int dev = 0;
    CINN_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        CINN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters, 1, 1);
    cfg.blockDim = dim3(pair::PTHREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CINN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, p));
    return CINN_OK;
}

template <bool B_MN>
static int launch_pair_out(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int out_dtype, int clusters,
                           cudaStream_t st) {
    CUtensorMap tc;
    int rc = make_out_map(&tc, ta, p, out_dtype, p.M, true);
    if (rc) return rc;
    switch (out_dtype) {
        case CINN_BF16: return launch_pair<B_MN, CINN_BF16>(ta, tb, tc, p, clusters, st);
        case CINN_F32: return launch_pair<B_MN, CINN_F32>(ta, tb, tc, p, clusters, st);
        case CINN_F16: return launch_pair<B_MN, CINN_F16>(ta, tb, tc, p, clusters, st);
        case CINN_F32_BF16: return launch_pair<B_MN, CINN_F32_BF16>(ta, tb, tc, p, clusters, st);
        default: set_error("GEMM: unknown output dtype tag %d", out_dtype); return CINN_ERR_INVALID;
    }
}

// Two-SM pairs serve dense problems with at least one 256 x 256 tile per pair of SMs (about 4 % faster than
// the one-SM kernel there); CINN_GEMM_PAIR=0 keeps every problem on the one-SM kernel.
static int pair_mode() {
    static int mode = -1;
    if (mode < 0) {
        const char* e = getenv("CINN_GEMM_PAIR");
        mode = (e && e[0] == '0') ? 0 : (e && e[0] == '2') ? 2 : 1;     // 2 = pairs for every layout (tests)
    }
    return mode;
}

// The persistent GEMM kernels normally take every SM.  A caller that wants other kernels to run beside them
// (the send/receive kernels of an all-to-all on another stream) can cap the number of SMs they occupy.
static std::atomic<int> g_gemm_sm_limit{0};
static inline int gemm_sms() {
    const int lim = g_gemm_sm_limit.load(std::memory_order_relaxed), all = sm_count();
    return (lim > 0 && lim < all) ? lim : all;
}
int set_gemm_sm_limit(int n) { return g_gemm_sm_limit.exchange(n < 0 ? 0 : n); }

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int fp8_gemm(const void* A, const float* sA, int64_t ld_sa, const void* B, const float* sB, int64_t sbk, int64_t sbn,
             void* C, int64_t M, int64_t N, int64_t K, int b_layout, int out_dtype, cudaStream_t st) {
    CINN_CHECK_ARG(M >= 0 && N >= 0 && K >= 0, "fp8_gemm: negative shape");
    if (M == 0 || N == 0) return CINN_OK;
    CINN_CHECK_ARG(A && sA && B && sB && C, "fp8_gemm: null pointer");
    CINN_CHECK_ARG(K > 0, "fp8_gemm: K must be positive");
    CINN_CHECK_ARG(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), "fp8_gemm: dimension too large");
    CINN_CHECK_ARG(K % 16 == 0, "fp8_gemm: K (%lld) must be a multiple of 16", (long long)K);
    CINN_CHECK_ARG(al16(A) && al16(B) && al16(C), "fp8_gemm: A, B and C must be 16-byte aligned");
    CINN_CHECK_ARG(b_layout == 0 || b_layout == 1, "fp8_gemm: unknown B layout %d", b_layout);
    CINN_CHECK_ARG(b_layout == 0 || N % 16 == 0, "fp8_gemm: B stored (K, N) needs N %% 16 == 0");
    const int64_t pair_tiles = ((M + pair::PM - 1) / pair::PM) * ((N + pair::PN - 1) / pair::PN);
    // measured on B200: the pair kernel wins with B K-major (forward), the one-SM kernel with B MN-major
    const int pm = pair_mode();
    const bool use_pair = pair_tiles >= sm_count() / 2 && (pm == 2 || (pm == 1 && b_layout == 0));
    CUtensorMap ta, tb;
    int rc = make_map(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM);
    if (rc) return rc;
    if (b_layout == 0) rc = make_map(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, use_pair ? 128 : BN);
    else rc = make_map(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)N, 128, BK);
    if (rc) return rc;
    GemmParams p{};
    p.sA = sA; p.sa_stride_m = ld_sa; p.sa_stride_k = 1;
    p.sB = sB; p.sb_stride_k = sbk; p.sb_stride_n = sbn; p.sb_stride_e = 0;
    p.C = C; p.ldc = N; p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.starts = nullptr; p.ends = nullptr; p.E = 1; p.b_rows_per_expert = 0;
    if (use_pair) {
        const int clusters = (int)(pair_tiles < gemm_sms() / 2 ? pair_tiles : gemm_sms() / 2);
        return b_layout == 0 ? launch_pair_out<false>(ta, tb, p, out_dtype, clusters, st)
                             : launch_pair_out<true>(ta, tb, p, out_dtype, clusters, st);
    }
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = (int)(tiles < gemm_sms() ? tiles : gemm_sms());
    return b_layout == 0 ? launch_out<false, false>(ta, tb, p, out_dtype, grid, st)
                         : launch_out<true, false>(ta, tb, p, out_dtype, grid, st);
}

int fp8_grouped_gemm(const void* A, const float* sA, const void* W, const float* sW, const int64_t* starts,
                     const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* C, int out_dtype,
                     cudaStream_t st, const long long* row_dst) {
    CINN_CHECK_ARG(E >= 0 && T >= 0 && d_in >= 0 && d_out >= 0, "grouped_gemm: negative shape");
    if (E == 0 || T == 0 || d_out == 0) return CINN_OK;
    CINN_CHECK_ARG(A && sA && W && sW && starts && ends && (C || row_dst), "grouped_gemm: null pointer");
    CINN_CHECK_ARG(row_dst == nullptr || (d_out % 8 == 0 && (out_dtype == CINN_BF16 || out_dtype == CINN_F16)),
                   "grouped_gemm: scattered output rows need a 2-byte output type and d_out %% 8 == 0");
    CINN_CHECK_ARG(E <= MAX_EXPERTS, "grouped_gemm: at most %d experts are supported (got %lld)", MAX_EXPERTS, (long long)E);
    CINN_CHECK_ARG(d_in > 0 && d_in % 16 == 0, "grouped_gemm: d_in (%lld) must be a positive multiple of 16", (long long)d_in);
    CINN_CHECK_ARG(T < (1LL << 31) && d_out < (1LL << 31) && d_in < (1LL << 31) && E * d_out < (1LL << 31),
                   "grouped_gemm: dimension too large");
    CINN_CHECK_ARG(al16(A) && al16(W) && al16(C), "grouped_gemm: A, W and C must be 16-byte aligned");
    CUtensorMap ta, tb;
    int rc = make_map(&ta, A, (uint64_t)d_in, (uint64_t)T, (uint64_t)d_in, BK, BM);
    if (rc) return rc;
    rc = make_map(&tb, W, (uint64_t)d_in, (uint64_t)(E * d_out), (uint64_t)d_in, BK, BN);
    if (rc) return rc;
    const int64_t nkb = (d_in + 127) / 128, nnb = (d_out + 127) / 128;
    GemmParams p{};
    p.sA = sA; p.sa_stride_m = nkb; p.sa_stride_k = 1;
    p.sB = sW; p.sb_stride_k = 1; p.sb_stride_n = nkb; p.sb_stride_e = nnb * nkb;
    p.C = C; p.ldc = d_out; p.M = (int)T; p.N = (int)d_out; p.K = (int)d_in;
    p.starts = starts; p.ends = ends; p.E = (int)E; p.b_rows_per_expert = (int)d_out;
    if (row_dst != nullptr) {
        // scattered rows: the table travels in the C slot of the parameters, tiles leave through staged 16-byte stores
        p.C = const_cast<long long*>(row_dst);
        p.tma_out = 0;
        return out_dtype == CINN_BF16 ? launch<false, true, CINN_BF16, true>(ta, tb, ta, p, gemm_sms(), st)
                                      : launch<false, true, CINN_F16, true>(ta, tb, ta, p, gemm_sms(), st);
    }
    return launch_out<false, true>(ta, tb, p, out_dtype, gemm_sms(), st);
}

// Input gradient of the grouped GEMM: dX[starts[e]:ends[e], :] = dY[starts[e]:ends[e], :] @ W[e]
// (W[e] is (d_out, d_in); its bytes are read MN-major, exactly as the dense dgrad reads a weight).
int fp8_grouped_gemm_dgrad(const void* dY, const float* sdY, const void* W, const float* sW, const int64_t* starts,
                           const int64_t* ends, int64_t E, int64_t T, int64_t d_in, int64_t d_out, void* dX, int out_dtype,
                           cudaStream_t st) {
    CINN_CHECK_ARG(E >= 0 && T >= 0 && d_in >= 0 && d_out >= 0, "grouped_gemm_dgrad: negative shape");
    if (E == 0 || T == 0 || d_in == 0) return CINN_OK;
    CINN_CHECK_ARG(dY && sdY && W && sW && starts && ends && dX, "grouped_gemm_dgrad: null pointer");
    CINN_CHECK_ARG(E <= MAX_EXPERTS, "grouped_gemm_dgrad: at most %d experts are supported (got %lld)", MAX_EXPERTS, (long long)E);
    CINN_CHECK_ARG(d_out > 0 && d_out % 16 == 0 && d_in % 16 == 0,
                   "grouped_gemm_dgrad: d_out (%lld) and d_in (%lld) must be multiples of 16", (long long)d_out, (long long)d_in);
    CINN_CHECK_ARG(T < (1LL << 31) && d_out < (1LL << 31) && d_in < (1LL << 31) && E * d_out < (1LL << 31),
                   "grouped_gemm_dgrad: dimension too large");
    CINN_CHECK_ARG(al16(dY) && al16(W) && al16(dX), "grouped_gemm_dgrad: dY, W and dX must be 16-byte aligned");
    CUtensorMap ta, tb;
    int rc = make_map(&ta, dY, (uint64_t)d_out, (uint64_t)T, (uint64_t)d_out, BK, BM);
    if (rc) return rc;
    // W viewed as (E * d_out) reduction rows of d_in output bytes: boxes of 128 output columns x 128 reduction rows.
    // A K block that runs past an expert's d_out rows meets zero-filled columns of dY, so the neighbour's bytes it
    // reads contribute nothing (quantised weights hold no NaN codes).
    rc = make_map(&tb, W, (uint64_t)d_in, (uint64_t)(E * d_out), (uint64_t)d_in, 128, BK);
    if (rc) return rc;
    const int64_t nkb_in = (d_in + 127) / 128, nob = (d_out + 127) / 128;
    GemmParams p{};
    p.sA = sdY; p.sa_stride_m = nob; p.sa_stride_k = 1;
    p.sB = sW; p.sb_stride_k = nkb_in; p.sb_stride_n = 1; p.sb_stride_e = nob * nkb_in;
    p.C = dX; p.ldc = d_in; p.M = (int)T; p.N = (int)d_in; p.K = (int)d_out;
    p.starts = starts; p.ends = ends; p.E = (int)E; p.b_rows_per_expert = (int)d_out;
    return launch_out<true, true>(ta, tb, p, out_dtype, gemm_sms(), st);
}

// Weight gradients of all experts in one launch (the GK instantiation of the pair kernel): dW (E, d_out, d_in) with
// A = dY^T quantised per expert segment, (d_out, max_tiles * 128), and B = x block-quantised per segment and
// transposed, (d_in, max_tiles * 128); kb_start (E + 1 ints, device) gives every expert's K blocks.
template <int OUT>
static int launch_pair_gk(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int clusters,
                          cudaStream_t st) {
    auto kern = pair::fp8_gemm_pair_kernel<false, OUT, true>;
    const size_t smem = pair::PSMEM_BYTES;
    static thread_local bool configured[64] = {};
    int dev = 0;
    CINN_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        CINN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters, 1, 1);
    cfg.blockDim = dim3(pair::PTHREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CINN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, p));
    return CINN_OK;
}

int fp8_gemm_grouped_k(const void* A, const float* sA, const void* B, const float* sB, const int* kb_start, int64_t E,
                       int64_t M, int64_t N, int64_t max_tiles, void* C, int out_dtype, cudaStream_t st) {
    CINN_CHECK_ARG(E >= 1 && M > 0 && N > 0 && max_tiles >= 1, "grouped-K GEMM: bad shape");
    CINN_CHECK_ARG(M % pair::PM == 0 && N % pair::PN == 0, "grouped-K GEMM: M (%lld) and N (%lld) must be multiples of 256",
                   (long long)M, (long long)N);
    CINN_CHECK_ARG(A && sA && B && sB && kb_start && C && al16(A) && al16(B) && al16(C), "grouped-K GEMM: null or unaligned pointer");
    CINN_CHECK_ARG(E * M < (1LL << 31) && N < (1LL << 31) && max_tiles * 128 < (1LL << 31), "grouped-K GEMM: dimension too large");
    const int64_t Kp = max_tiles * 128;
    CUtensorMap ta, tb;
    int rc = make_map(&ta, A, (uint64_t)Kp, (uint64_t)M, (uint64_t)Kp, BK, BM);
    if (rc) return rc;
    rc = make_map(&tb, B, (uint64_t)Kp, (uint64_t)N, (uint64_t)Kp, BK, 128);
    if (rc) return rc;
    const int64_t nnb = (N + 127) / 128;
    GemmParams p{};
    p.sA = sA; p.sa_stride_m = max_tiles; p.sa_stride_k = 1;
    p.sB = sB; p.sb_stride_k = nnb; p.sb_stride_n = 1; p.sb_stride_e = 0;
    p.C = C; p.ldc = N; p.M = (int)M; p.N = (int)N; p.K = 0;
    p.starts = reinterpret_cast<const int64_t*>(kb_start); p.ends = nullptr; p.E = (int)E; p.b_rows_per_expert = 0;
    CUtensorMap tc;
    rc = make_out_map(&tc, ta, p, out_dtype, E * M, true);
    if (rc) return rc;
    const int64_t tiles = E * (M / pair::PM) * (N / pair::PN);
    const int clusters = (int)(tiles < gemm_sms() / 2 ? tiles : gemm_sms() / 2);
    switch (out_dtype) {
        case CINN_BF16: return launch_pair_gk<CINN_BF16>(ta, tb, tc, p, clusters, st);
        case CINN_F32: return launch_pair_gk<CINN_F32>(ta, tb, tc, p, clusters, st);
        case CINN_F32_BF16: return launch_pair_gk<CINN_F32_BF16>(ta, tb, tc, p, clusters, st);
        default: set_error("grouped-K GEMM: the gradient is fp32 (optionally holding bf16-rounded values) or bf16"); return CINN_ERR_INVALID;
    }
}

// Grouped GEMM on 16-bit operands: C[starts[e]:ends[e]] = A[starts[e]:ends[e]] @ W[e]^T with A (T, d_in) and
// W (E, d_out, d_in) both bf16 or both fp16, fp32 accumulation (the reference's grouped_gemm_kernel arithmetic).
template <bool BF16_IN, int OUT>
static int launch16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int grid,
                    cudaStream_t st) {
    auto kern = g16::grouped_gemm16_kernel<BF16_IN, OUT>;
    const size_t smem = smem_bytes(p.E);
    static thread_local size_t configured[64] = {};
    int dev = 0;
    CINN_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        CINN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    kern<<<grid, g16::GTHREADS, smem, st>>>(ta, tb, tc, p);
    CINN_CHECK_LAUNCH();
    return CINN_OK;
}

int grouped_gemm_16bit(const void* A, const void* W, int in_dtype, const int64_t* starts, const int64_t* ends, int64_t E,
                       int64_t T, int64_t d_in, int64_t d_out, void* C, int out_dtype, cudaStream_t st) {
    CINN_CHECK_ARG(E >= 0 && T >= 0 && d_in >= 0 && d_out >= 0, "grouped_gemm_16bit: negative shape");
    if (E == 0 || T == 0 || d_out == 0) return CINN_OK;
    CINN_CHECK_ARG(A && W && starts && ends && C, "grouped_gemm_16bit: null pointer");
    CINN_CHECK_ARG(in_dtype == CINN_BF16 || in_dtype == CINN_F16, "grouped_gemm_16bit: operands must be bf16 or fp16 (tag %d)", in_dtype);
    CINN_CHECK_ARG(E <= MAX_EXPERTS, "grouped_gemm_16bit: at most %d experts are supported (got %lld)", MAX_EXPERTS, (long long)E);
    CINN_CHECK_ARG(d_in > 0 && d_in % 8 == 0, "grouped_gemm_16bit: d_in (%lld) must be a positive multiple of 8", (long long)d_in);
    CINN_CHECK_ARG(T < (1LL << 31) && d_out < (1LL << 31) && d_in < (1LL << 30) && E * d_out < (1LL << 31),
                   "grouped_gemm_16bit: dimension too large");
    CINN_CHECK_ARG(al16(A) && al16(W) && al16(C), "grouped_gemm_16bit: A, W and C must be 16-byte aligned");
    const CUtensorMapDataType dt = in_dtype == CINN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ta, tb;
    int rc = make_map(&ta, A, (uint64_t)d_in, (uint64_t)T, (uint64_t)d_in * 2, BK / 2, BM, dt);
    if (rc) return rc;
    rc = make_map(&tb, W, (uint64_t)d_in, (uint64_t)(E * d_out), (uint64_t)d_in * 2, BK / 2, BN, dt);
    if (rc) return rc;
    GemmParams p{};
    p.sA = nullptr; p.sB = nullptr;
    p.C = C; p.ldc = d_out; p.M = (int)T; p.N = (int)d_out; p.K = (int)d_in;
    p.starts = starts; p.ends = ends; p.E = (int)E; p.b_rows_per_expert = (int)d_out;
    CUtensorMap tc;
    rc = make_out_map(&tc, ta, p, out_dtype, p.M);
    if (rc) return rc;
    const int grid = gemm_sms();
#define CINN_G16(BF, O) return launch16<BF, O>(ta, tb, tc, p, grid, st)
    if (in_dtype == CINN_BF16) {
        switch (out_dtype) {
            case CINN_BF16: CINN_G16(true, CINN_BF16);
            case CINN_F16: CINN_G16(true, CINN_F16);
            case CINN_F32: CINN_G16(true, CINN_F32);
        }
    } else {
        switch (out_dtype) {
            case CINN_BF16: CINN_G16(false, CINN_BF16);
            case CINN_F16: CINN_G16(false, CINN_F16);
            case CINN_F32: CINN_G16(false, CINN_F32);
        }
    }
#undef CINN_G16
    set_error("grouped_gemm_16bit: unknown output dtype tag %d", out_dtype);
    return CINN_ERR_INVALID;
}

int read_quant_status(int* out, int reset);
int read_moe_status(int* out, int reset);

// One word for the caller: the GEMM's code if it has one, else the quantisers', else the exchange kernels'.
int read_device_status(int* out, int reset) {
    int v = 0, q = 0, m = 0;
    CINN_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (reset && v != 0) {
        int z = 0;
        CINN_CHECK_CUDA(cudaMemcpyToSymbol(g_device_status, &z, sizeof(int)));
    }
    int rc = read_quant_status(&q, reset);
    if (rc) return rc;
    rc = read_moe_status(&m, reset);
    if (rc) return rc;
    *out = v != 0 ? v : (q != 0 ? q : m);
    return CINN_OK;
}

}  // namespace cinn

