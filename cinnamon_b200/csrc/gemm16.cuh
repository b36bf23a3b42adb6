// Grouped GEMM on 16-bit operands (included by gemm.cu): the arithmetic of the reference's grouped_gemm_kernel
// (src/kernels.py:440-523) - 16-bit operands, fp32 accumulation, 16-bit result - for callers that want the routed
// experts in the reference's own precision instead of e4m3.
//
// Same tile (128 x 256), same operand ring (TMA, 128-byte swizzle: a stage holds 64 K elements of 2 bytes), same
// device-side walk over the experts' ragged row ranges and the same stores as the FP8 kernel; what differs is the
// middle: tcgen05.mma kind::f16 accumulates the whole K extent of a tile in one TMEM buffer (there are no scales
// to apply per K block), and the epilogue warps read a finished tile once while the issuer fills the other buffer.
//
// Roles (10 warps): 0-7 epilogue, 8 TMA producer (one lane), 9 MMA issuer (one lane) and owner of the TMEM
// allocation.  Every wait is bounded as in the FP8 kernel.
#pragma once

namespace g16 {

constexpr int GTHREADS = (EPI_WARPS + 2) * 32;

// kind::f16 instruction descriptor: fp32 accumulate, A and B of the same 16-bit type, both K-major
__host__ __device__ constexpr uint32_t make_idesc16(bool bf16) {
    return (1u << 4)                                   // D format: fp32
           | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10)   // A, B format: 0 = fp16, 1 = bf16
           | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <bool BF16_IN, int OUT>
__global__ void __launch_bounds__(GTHREADS, 1)
grouped_gemm16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint8_t* c_stage = smem + STAGES * (A_BYTES + B_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(c_stage + C_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* store_stage = c_stage;
    int* cum = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);

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
    if (warp == 0) {                               // prefix sum of per-expert m-tile counts
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
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int KB = (p.K * 2 + BK - 1) / BK;            // K blocks of 128 bytes = 64 elements
    const int n_total = total_tiles<true>(p, cum);

    if (warp == EPI_WARPS) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < n_total && alive; t += gridDim.x) {
                const TileInfo ti = tile_info<true>(p, cum, t);
                const int b_row0 = ti.expert * p.b_rows_per_expert;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, (1 << 8) | 1)) { alive = false; break; }
                    const uint32_t fb = full0 + 8 * s;
                    mbar_expect_tx(fb, A_BYTES + B_BYTES);
                    tma_load_2d(&tmA, fb, smem_u32(smem_a + s * A_BYTES), kb * (BK / 2), ti.m0);
                    tma_load_2d(&tmB, fb, smem_u32(smem_b + s * B_BYTES), kb * (BK / 2), b_row0 + ti.n0);
                }
            }
            if (!alive) {
                const uint32_t issued = it;
                for (uint32_t j = (issued > STAGES ? issued - STAGES : 0); j < issued; ++j) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
                    }
                }
            }
        }
    } else if (warp == EPI_WARPS + 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc16(BF16_IN);
            uint32_t it = 0, tile_no = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < n_total && alive; t += gridDim.x, ++tile_no) {
                const uint32_t b = tile_no & 1, bph = (tile_no >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * b, bph ^ 1, abort_flag, (2 << 8) | 2)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + b * BN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, (2 << 8) | 1)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + s * A_BYTES);
                    const uint32_t b_addr = smem_u32(smem_b + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)          // 16 elements = 32 bytes per instruction
                        tc_mma_f16(d, make_smem_desc(a_addr + k * 32, 16, 1024), make_smem_desc(b_addr + k * 32, 16, 1024), idesc,
                                   (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);
                }
                if (!alive) break;
                tc_commit(tfull0 + 8 * b);
            }
            // every MMA issued above must have retired before tensor memory is freed
            if (alive && tile_no > 0) {
                const uint32_t last = tile_no - 1;
                mbar_wait(tfull0 + 8 * (last & 1), (last >> 1) & 1, abort_flag, (2 << 8) | 3);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3, h = warp >> 2;
        uint32_t tile_no = 0, n_rounds = 0;
        bool alive = true;
        const bool vec_ok = (OUT == CINN_F32) ? (p.ldc % 4 == 0) : (p.ldc % 8 == 0);
        for (int t = blockIdx.x; t < n_total && alive; t += gridDim.x, ++tile_no) {
            const TileInfo ti = tile_info<true>(p, cum, t);
            const int row = ti.m0 + q * 32 + lane;
            const bool rvalid = row < ti.m_end;
            const int col0 = ti.n0 + h * WCOLS;
            const bool cvalid = col0 < p.N;
            const uint32_t b = tile_no & 1, bph = (tile_no >> 1) & 1;
            if (!mbar_wait_warp(tfull0 + 8 * b, bph, abort_flag, (3 << 8) | 1)) { alive = false; break; }
            tc_fence_after();
            float acc[WCOLS];
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * BN + h * WCOLS;
#pragma unroll
            for (int c = 0; c < WCOLS / 16; ++c) {
                float v[16];
                tc_ld16(taddr + c * 16, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c * 16 + j] = v[j];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * b);        // the issuer may refill this buffer
            constexpr bool TMA_OUT = (OUT == CINN_BF16 || OUT == CINN_F16);
            const bool whole = ti.m0 + BM <= ti.m_end;
            if (TMA_OUT && p.tma_out && whole) {
                const bool elected = (warp == h * 4) && lane == 0;
                const uint32_t slot = smem_u32(c_stage) + h * C_SLOT_BYTES;
                const int rl = q * 32 + lane;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t par = n_rounds & 1u;
                    if (elected) tma_store_wait_read();
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
                    __syncwarp();
                    ++n_rounds;
                }
                if (!alive) break;
            } else if (vec_ok && !(TMA_OUT && p.tma_out)) {
                if (cvalid) store_rows_staged<OUT, WCOLS>(acc, store_stage + warp * 2048, p.C, p.ldc, ti.m0 + q * 32, ti.m_end, col0, p.N, lane);
            } else if (rvalid && cvalid) {
                const int64_t base = (int64_t)row * p.ldc + col0;
#pragma unroll
                for (int j = 0; j < WCOLS / 8; ++j) {
                    const int ncols = p.N - (col0 + j * 8);
                    if (ncols > 0) store8<OUT>(p.C, base + j * 8, &acc[j * 8], vec_ok, ncols);
                }
            }
        }
        if (lane == 0 && (warp & 3) == 0) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == EPI_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace g16
