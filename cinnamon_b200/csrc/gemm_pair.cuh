// Two-SM variant of the dense block-scaled FP8 GEMM (included by gemm.cu).
//
// A cluster of two CTAs on neighbouring SMs computes a 256 x 256 output tile with
// tcgen05.mma.cta_group::2: CTA r holds rows [128 r, 128 r + 128) of A and columns
// [128 r, 128 r + 128) of B in its own shared memory and the 128 x 256 accumulator rows
// in its own tensor memory.  Each SM therefore stages 32 KiB per K block instead of 48 KiB
// and the tensor pipe reads a third less shared memory per MMA.  One thread of the even
// (leader) CTA issues the MMAs for the pair; completion is signalled to a barrier in each
// CTA.  TMA loads are plain per-CTA loads: each CTA fetches only its own halves and reports
// the bytes to the leader's "operands landed" barrier.
//
// Roles per CTA (11 warps): 0-7 promotion/epilogue, 8 TMA producer, 9 TMEM allocation;
// warps 9 and 10 of the leader issue the MMAs of alternate K blocks.  All waits are bounded exactly as in the one-SM kernel.
#pragma once

namespace pair {

constexpr int PM = 256;                 // rows of the pair's tile
constexpr int PN = 256;                 // columns of the pair's tile
constexpr int PSTAGES = 4;               // even (see the one-SM kernel); leaves room for a whole output tile
constexpr int PA_BYTES = 128 * BK;      // A rows of this CTA: 16 KiB
constexpr int PB_BYTES = 128 * BK;      // B columns of this CTA: 16 KiB
constexpr int PTHREADS = 11 * 32;
// dynamic shared memory: operand stages | four 16 KiB output slots = the CTA's whole 128 x 256 tile of a 2-byte type
// (TMA-store boxes; also the 2 KiB-per-warp staging of the non-TMA path) | 256 B of barriers and flags, plus 1 KiB of
// slack to align the stages to 1024 bytes
constexpr int PSTAGE_OFF = PSTAGES * (PA_BYTES + PB_BYTES);
constexpr int PC_BYTES = 4 * C_SLOT_BYTES;
constexpr size_t PSMEM_BYTES = (size_t)PSTAGE_OFF + PC_BYTES + 256 + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier of the other CTA.  Relaxed: the barrier hands over a tensor-memory buffer whose reads
// are already complete (tcgen05.wait::ld + tcgen05.fence), no generic-memory data is published by it, and a
// cluster-scope release here costs over a thousand cycles per K block.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose byte count is reported to a barrier that may live in
// the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint32_t bar_cluster, uint32_t dst, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
// Completion of the pair's MMAs issued so far is reported to the barrier at the same offset in BOTH CTAs:
// one commit per CTA, each naming that CTA's barrier by its cluster address.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint32_t own = mapa(bar, 0), peer = mapa(bar, 1);
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(own) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(peer) : "memory");
}
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_pair(bool b_mn_major) {
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);
}

struct PairTile { int m0, n0; };

__device__ __forceinline__ int pair_total(const GemmParams& p) {
    return ((p.M + PM - 1) / PM) * ((p.N + PN - 1) / PN);
}
__device__ __forceinline__ PairTile pair_tile(const GemmParams& p, int t) {
    const int m_tiles = (p.M + PM - 1) / PM, n_tiles = (p.N + PN - 1) / PN;
    constexpr int GROUP = 16;                      // 16 x 256 rows per L2 group
    const int per_group = GROUP * n_tiles;
    const int g = t / per_group;
    const int first_m = g * GROUP;
    const int gsize = min(GROUP, m_tiles - first_m);
    const int r = t - g * per_group;
    PairTile ti;
    ti.m0 = (first_m + r % gsize) * PM;
    ti.n0 = (r / gsize) * PN;
    return ti;
}

// GK ("grouped K"): E independent problems of the same M x N whose reduction ranges differ - the weight gradients
// of the experts, dW[e] = dY[rows of e]^T @ x[rows of e].  Both operands are K-major over one padded token axis on
// which expert e owns the K blocks [kb_start[e], kb_start[e + 1]) (p.starts holds that int array, p.E = E); tile t
// belongs to expert t / (tiles per expert) and is stored at rows e * M + ... of the (E * M, N) output.  An expert
// without rows gets zeros.  M and N are multiples of 256 here, so every tile is whole.
template <bool B_MN, int OUT, bool GK = false>
__global__ void __launch_bounds__(PTHREADS, 1)
fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + PSTAGES * PA_BYTES;
    uint8_t* c_stage = smem + PSTAGE_OFF;
    uint64_t* bars = reinterpret_cast<uint64_t*>(c_stage + PC_BYTES);
    // [0, S) full (used in the leader), [S, 2S) empty, [2S, 2S+2) tmem full, [2S+2, 2S+4) tmem empty (leader)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* store_stage = c_stage;                                             // 2 KiB per promotion warp (non-TMA path)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();           // 0 = leader
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + PSTAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * PSTAGES), tempty0 = smem_u32(bars + 2 * PSTAGES + 2);
    const uint32_t gfree0 = smem_u32(bars + 2 * PSTAGES + 4), gfull0 = smem_u32(bars + 2 * PSTAGES + 6);

    if (threadIdx.x == 0) *abort_flag = 0;
    if (warp == 8 && lane == 0) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 16); }
        for (int g = 0; g < 2; ++g) { mbar_init(gfree0 + 8 * g, 4); mbar_init(gfull0 + 8 * g, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                    // both CTAs' barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int KB_dense = (p.K + BK - 1) / BK;
    const int per_expert = pair_total(p);
    const int n_total = GK ? per_expert * p.E : per_expert;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int* kb_start = reinterpret_cast<const int*>(p.starts);
    // tile t -> its coordinates inside one problem, the expert it belongs to, its K blocks
    auto locate = [&](int t, PairTile& ti, int& e, int& kb0, int& KB) {
        if constexpr (GK) {
            e = t / per_expert;
            ti = pair_tile(p, t - e * per_expert);
            kb0 = kb_start[e];
            KB = kb_start[e + 1] - kb0;
        } else {
            e = 0; kb0 = 0; KB = KB_dense;
            ti = pair_tile(p, t);
        }
    };

    if (warp == 8) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            const uint32_t full_leader = mapa(full0, 0);
            uint32_t it = 0;
            bool alive = true;
            for (int t = cluster_id; t < n_total && alive; t += n_clusters) {
                PairTile ti; int e, kb0, KB;
                locate(t, ti, e, kb0, KB);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % PSTAGES;
                    const uint32_t ph = (it / PSTAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, (1 << 8) | 1)) { alive = false; break; }
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * (PA_BYTES + PB_BYTES));
                    const uint32_t fb = full_leader + 8 * s;
                    tma_load_2d_pair(&tmA, fb, smem_u32(smem_a + s * PA_BYTES), (kb0 + kb) * BK, ti.m0 + 128 * (int)rank);
                    if constexpr (!B_MN) tma_load_2d_pair(&tmB, fb, smem_u32(smem_b + s * PB_BYTES), (kb0 + kb) * BK, ti.n0 + 128 * (int)rank);
                    else tma_load_2d_pair(&tmB, fb, smem_u32(smem_b + s * PB_BYTES), ti.n0 + 128 * (int)rank, (kb0 + kb) * BK);
                }
            }
            if (!alive) {
                // abandoned: the barrier that counts this CTA's copies may live in the other CTA, so just give
                // the copies already issued ample time to land before shared memory is given up
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) { }
            }
        }
    } else if (warp >= 9) {
        // ------------------------------ MMA issuers (leader only) ------------------------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_pair(B_MN);
            const uint32_t mine = (uint32_t)(warp - 9);
            uint32_t it = 0, last = 0xffffffffu;
            bool alive = true;
            for (int t = cluster_id; t < n_total && alive; t += n_clusters) {
                PairTile ti_; int e_, kb0_, KB;
                locate(t, ti_, e_, kb0_, KB);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    if ((it & 1u) != mine) continue;
                    last = it;
                    const int s = it % PSTAGES;
                    const uint32_t ph = (it / PSTAGES) & 1;
                    const uint32_t b = it & 1, bph = (it >> 1) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, (2 << 8) | 1)) { alive = false; break; }
                    if (!mbar_wait(tempty0 + 8 * b, bph ^ 1, abort_flag, (2 << 8) | 2)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + s * PA_BYTES);
                    const uint32_t b_addr = smem_u32(smem_b + s * PB_BYTES);
                    const uint32_t d = tmem_base + b * PN;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 32 * 128, 16, 1024)
                                                 : make_smem_desc(b_addr + k * 32, 16, 1024);
                        tc_mma_f8_pair(d, ad, bd, idesc, k > 0 ? 1u : 0u);
                    }
                    tc_commit_pair(empty0 + 8 * s);
                    tc_commit_pair(tfull0 + 8 * b);
                }
            }
            if (alive && last != 0xffffffffu) mbar_wait(tfull0 + 8 * (last & 1), (last >> 1) & 1, abort_flag, (2 << 8) | 3);
        }
    } else {
        // ------------------------------ promotion / epilogue (both CTAs) ------------------------------
        const int q = warp & 3, h = warp >> 2;
        const uint32_t tempty_leader = mapa(tempty0, 0);
        uint32_t it = 0, n_rounds = 0;
        bool alive = true;
        const bool vec_ok = (OUT == CINN_F32 || OUT == CINN_F32_BF16) ? (p.ldc % 4 == 0) : (p.ldc % 8 == 0);
        for (int t = cluster_id; t < n_total && alive; t += n_clusters) {
            PairTile ti; int e, kb0, KB;
            locate(t, ti, e, kb0, KB);
            const int row = ti.m0 + 128 * (int)rank + q * 32 + lane;
            const bool rvalid = row < p.M;
            const int col0 = ti.n0 + h * 128;
            const bool cvalid = col0 < p.N;
            const float* sa_ptr = p.sA + (int64_t)(rvalid ? row : 0) * p.sa_stride_m + (int64_t)kb0 * p.sa_stride_k;
            const float* sb_ptr = p.sB + (int64_t)(cvalid ? col0 / 128 : 0) * p.sb_stride_n + (int64_t)kb0 * p.sb_stride_k;
            const int out_row0 = e * p.M;                      // GK: the expert's slice of the (E * M, N) output
            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
            float sa0 = ld_scale(sa_ptr), sb0 = ld_scale(sb_ptr);
            float sa1 = 0.f, sb1 = 0.f, sa2 = 0.f, sb2 = 0.f;
            if (KB > 1) { sa1 = ld_scale(sa_ptr + p.sa_stride_k); sb1 = ld_scale(sb_ptr + p.sb_stride_k); }
            if (KB > 2) { sa2 = ld_scale(sa_ptr + 2 * p.sa_stride_k); sb2 = ld_scale(sb_ptr + 2 * p.sb_stride_k); }
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
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * PN + h * 128;
                // packed fp32x2 FMAs: half the issue slots of 128 scalar ones, the same IEEE result in every lane
                uint64_t s2;
                asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "f"(s));
#pragma unroll
                for (int c = 0; c < 8; ++c) {
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
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(tempty_leader + 8 * b);
            }
            if (alive && p.tma_out) {
                // The tile leaves through TMA stores.  Each column group of four promotion warps owns two 16 KiB slots
                // (boxes of 128 rows x 128 bytes, 128-byte swizzle): its threads drop their rows into them in 16-byte
                // chunks and one thread hands the boxes to the TMA unit.  A 2-byte output fits the group's 128 columns
                // in one round; a 4-byte output takes two rounds of 64 columns.  Nobody waits for the unit until the
                // slots are needed again.
                using T = typename OutT<OUT>::type;
                constexpr int EPR = 128 / (int)sizeof(T);          // elements per 128-byte box row
                constexpr int PER16 = 16 / (int)sizeof(T);
                constexpr int ROUNDS = 128 / (2 * EPR);
                const bool elected = (warp == h * 4) && lane == 0;
                const uint32_t slot = smem_u32(c_stage) + h * 2 * C_SLOT_BYTES;
                const int rl = q * 32 + lane;
#pragma unroll
                for (int r = 0; r < ROUNDS; ++r) {
                    const uint32_t par = n_rounds & 1u;
                    if (elected) tma_store_wait_read();               // the previous boxes have left the slots
                    __syncwarp();
                    if (lane == 0) mbar_arrive(gfree0 + 8 * h);
                    if (!mbar_wait_warp(gfree0 + 8 * h, par, abort_flag, (3 << 8) | 2)) { alive = false; break; }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint4 v = pack16<OUT>(&acc[r * 2 * EPR + (j >> 3) * EPR + (j & 7) * PER16]);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(slot + (j >> 3) * C_SLOT_BYTES + rl * 128 + (((j & 7) ^ (rl & 7)) << 4)),
                                       "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(gfull0 + 8 * h);
                    if (elected) {
                        if (mbar_wait(gfull0 + 8 * h, par, abort_flag, (3 << 8) | 3)) {
#pragma unroll
                            for (int sl = 0; sl < 2; ++sl) {
                                const int col = col0 + r * 2 * EPR + sl * EPR;
                                if (col < p.N) tma_store_2d(&tmC, slot + sl * C_SLOT_BYTES, col, out_row0 + ti.m0 + 128 * (int)rank);
                            }
                            tma_store_commit();
                        }
                    }
                    __syncwarp();       // the elected lane rejoins its warp before the next warp-collective instruction
                    ++n_rounds;
                }
                if (!alive) break;
            } else if (alive && vec_ok) {
                if (cvalid) store_rows_staged<OUT, 128>(acc, store_stage + warp * 2048, p.C, p.ldc,
                                                        out_row0 + ti.m0 + 128 * (int)rank + q * 32, out_row0 + p.M, col0, p.N, lane);
            } else if (alive && rvalid && cvalid) {
                const int64_t base = (int64_t)(out_row0 + row) * p.ldc + col0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int ncols = p.N - (col0 + j * 8);
                    if (ncols > 0) store8<OUT>(p.C, base + j * 8, &acc[j * 8], false, ncols);
                }
            }
        }
        if (lane == 0 && (warp & 3) == 0) tma_store_wait_all();      // this group's boxes have reached global memory
    }

    // nobody leaves while the other CTA may still read this CTA's shared memory or signal its barriers
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pair
