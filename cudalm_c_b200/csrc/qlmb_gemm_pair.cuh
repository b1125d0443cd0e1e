// Two-SM form of the GEMM engine (included by qlmb_gemm.cu).
//
// A cluster of two CTAs on neighbouring SMs computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own
// 128 columns of B (expanding only that half of the weights), the leader CTA
// issues one M=256 instruction per 16-deep step that reads both halves, and each
// CTA's TMEM holds its 128 rows x 256 columns of the result.  Per SM and step the
// tensor core therefore reads half as much shared memory and the dequant warps
// expand half as many weights as in the one-SM form.
//
// Hand-shakes across the pair (all waits bounded, as everywhere in this file):
//   full[s]        leader   one barrier per stage collects everything the MMA needs: the
//                           byte counts of both CTAs' bulk tensor loads (the peer's loads
//                           name the leader's barrier, cta_group::2 form) and one arrival
//                           per dequant warp of either CTA (the peer's arrive remotely)
//   empty[s]       both     released by one tcgen05.commit that arrives in both CTAs
//   tmem_full[a]   both     committed the same way after a tile's last step
//   tmem_empty[a]  leader   8 local + 8 remote epilogue warps
//   full_c/empty_c local    ring of packed-code tiles between the loader and the dequant warps
// No bulk copy in this file has more than one destination CTA.
#pragma once

namespace qlmb {

constexpr int P_BN = 256;                 // accumulator columns of the pair tile
constexpr int P_A_STAGE = BM * BK * 2;    // per CTA: 128 rows
constexpr int P_B_STAGE = 128 * BK * 2;   // per CTA: 128 columns of B
constexpr int P_C_STAGE = 128 * BK / 2;   // per CTA: codes of those columns
constexpr int P_S_STAGE = 128 * 4;        // per CTA: the stage's group scales (up to 128 floats)
constexpr int P_S_RING = 4096;            // the scale slots together, padded so that what follows stays 1 KiB aligned
constexpr int P_NSC = 7;                  // depth of the code / scale ring

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
// (default semantics: a cluster-scope release here costs a full memory fence per call, which
// throttled the relay to one stage per microsecond)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr)
{ asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory"); }
__device__ __forceinline__ uint32_t mbar_try_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *errword, int site)
{
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_cluster(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    if (!*abort_flag) {
        *abort_flag = 1;
        if (errword && atomicCAS(errword, 0, 201) == 0) { errword[1] = site; errword[2] = (int)blockIdx.x; errword[3] = (int)parity; }
    }
    return false;
}
// bulk tensor load into this CTA's shared memory whose byte count is reported to a barrier
// of either CTA of the pair (cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
// 4-byte asynchronous copy global -> shared, and an mbarrier arrival that fires when all
// earlier asynchronous copies of the calling thread have landed (the barrier's expected count
// must include one such arrival per calling thread)
__device__ __forceinline__ void cp_async4(void *dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols)
{ asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory"); }
__device__ __forceinline__ void tmem_relinquish2()
{ asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols)
{ asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory"); }
// completion of all MMAs issued so far -> one arrival on the barrier at this cluster address
__device__ __forceinline__ void tc_commit2(uint32_t cluster_bar)
{ asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory"); }
// one commit that arrives on the barrier at this shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit2_both(uint32_t local_bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(local_bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate),
                   "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}

// Pair tile: 256 rows starting at m0 (CTA r owns rows m0 + 128 r ...), 256 output columns
// starting at n_t * 256 (CTA r expands columns + 128 r); with the SwiGLU epilogue the pair
// tile is 128 gate + 128 up columns of the same 128 activation columns.
template <int SCHED>
__device__ __forceinline__ TileInfo decode_pair_tile(const GemmParams &p, int tile, int ntr)
{
    TileInfo t;
    if (SCHED == SCHED_DENSE) {
        t.m0 = (tile % p.tiles_m) * 256; t.n_t = tile / p.tiles_m; t.e = 0; t.ksteps = p.ksteps; t.row0 = 0;
        t.halves = (t.m0 + BM < p.M) ? 2 : 1;
    } else if (SCHED == SCHED_ROWS) {
        // column tiles fastest: the pairs that run side by side share a row tile of A (which can be
        // far larger than L2 in total: 113 MB for dX) and differ in the weight slice (40 MB in total)
        int rt = tile / p.tiles_n;
        int info = p.tile_info[rt];
        t.m0 = (info & 0xFFFFF) * BM; t.e = (info >> 20) & 0x1FF; t.halves = ((info >> 30) & 1) + 1;
        t.n_t = tile % p.tiles_n; t.ksteps = p.ksteps; t.row0 = 0;
    } else {
        int per = p.tiles_m * p.tiles_n;
        t.e = tile / per;
        int r = tile % per;
        t.m0 = (r % p.tiles_m) * 256; t.n_t = r / p.tiles_m;
        t.row0 = p.off[t.e];
        t.ksteps = (p.off[t.e + 1] - p.off[t.e]) / BK;
        t.halves = (t.m0 + BM < p.M) ? 2 : 1;
    }
    return t;
}

template <int BMODE, int EPI, int SCHED, int DQG>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((BMODE == B_DEQ_MN || BMODE == B_DEQ_K) ? 576 : 320, 1)
k_gemm_pair(const __grid_constant__ GemmParams p)
{
    constexpr bool DEQ = (BMODE == B_DEQ_MN || BMODE == B_DEQ_K);
    constexpr bool DUAL = (EPI == EPI_SWIGLU);           // CTA 0 expands W1 (gate), CTA 1 expands W3 (up)
    constexpr int NS = DEQ ? (EPI == EPI_SWIGLU_BWD ? 4 : 5) : 6, NSC = P_NSC;
    constexpr int GW = DQ_WARPS / DQG;                   // dequant warps per stage group
    // group scales: codes [K][N] need 64 new scales per stage, fetched by the producer warp into the
    // stage's slot; codes [N][K] reuse a row's scale for two stages, each lane keeps its own in registers
    constexpr bool S_SMEM = (BMODE == B_DEQ_MN);
    constexpr uint32_t IDESC = make_idesc(256, P_BN, BMODE == AB_TMA_MN ? 1 : 0, (BMODE == B_DEQ_MN || BMODE == AB_TMA_MN) ? 1 : 0);
    constexpr uint32_t TMEM_COLS = 2 * P_BN;
    constexpr uint32_t TX_BYTES = 2u * (P_A_STAGE + (DEQ ? 0 : P_B_STAGE));   // both CTAs' loads of a stage

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem;
    uint8_t *sB = sA + NS * P_A_STAGE;
    uint8_t *sC = sB + NS * P_B_STAGE;
    float *sS = reinterpret_cast<float *>(sC + (DEQ ? NSC * P_C_STAGE : 0));      // [NSC][128] group scales
    uint8_t *sE = sC + (DEQ ? NSC * P_C_STAGE + P_S_RING : 0);
    static_assert((P_C_STAGE % 1024) == 0 && (P_S_RING % 1024) == 0 && P_NSC * P_S_STAGE <= P_S_RING,
                  "the epilogue staging blocks are bulk-tensor boxes with a 128-byte swizzle: 1 KiB alignment");
    uint64_t *bars = reinterpret_cast<uint64_t *>(sE + EPI_WARPS * epi_stage_bytes(EPI));
    uint64_t *full = bars, *empty = full + NS;
    uint64_t *full_c = empty + NS, *empty_c = full_c + NSC;
    uint64_t *tmem_full = empty_c + NSC, *tmem_empty = tmem_full + 2, *spare = tmem_empty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(spare + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; i++) { mbar_init(smem_u32(&full[i]), 1 + (DEQ ? 2 * GW : 0)); mbar_init(smem_u32(&empty[i]), 1); }
        for (int i = 0; i < NSC; i++) { mbar_init(smem_u32(&full_c[i]), S_SMEM ? 33 : 1); mbar_init(smem_u32(&empty_c[i]), GW); }
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&tmem_full[i]), 1); mbar_init(smem_u32(&tmem_empty[i]), 2 * EPI_WARPS); }
        mbar_init(smem_u32(spare), 1);
        for (int i = 0; i < 2 * EPI_WARPS; i++) mbar_init(smem_u32(bars + 48 + i), 1);   // epilogue input rings
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc2(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish2(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int npairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    const int ntr = (SCHED == SCHED_ROWS) ? *p.ntiles_dev : 0;
    const int total = (SCHED == SCHED_DENSE) ? p.tiles_m * p.tiles_n
                    : (SCHED == SCHED_ROWS) ? ntr * p.tiles_n : p.E * p.tiles_m * p.tiles_n;
    const int my_m = (int)rank * BM;                     // this CTA's row offset inside the pair tile
    const int my_n = (int)rank * 128;                    // and its column offset

    if (warp == 0) {
        // =============================== TMA producer (both CTAs) ===============================
        Ring rs = {0, 0}, rc = {0, 0};
        bool ok = true;
        // group scales of a stage (codes [K][N]): every lane copies its rows' scales into the stage's slot with
        // 4-byte asynchronous copies and lets full_c[s] count their completion, so full_c[s]
        // completes when the code bytes (expect_tx arrival of lane 0) and all 32 lanes' scales landed
        const int gpr = p.w_cols / 128;
        for (int tile = pair; ok && tile < total; tile += npairs) {
            TileInfo t = decode_pair_tile<SCHED>(p, tile, ntr);
            for (int seg = 0; ok && seg < p.nseg; seg++) {
                for (int ks = 0; ks < t.ksteps; ks++) {
                    ok = mbar_wait_idle(smem_u32(&empty[rs.idx]), rs.phase ^ 1u, abort_flag, p.errword, 11);
                    if (!ok) break;
                    if (lane == 0) {
                        if (leader) mbar_expect_tx(smem_u32(&full[rs.idx]), TX_BYTES);
                        const uint32_t bar = map_to_cta(smem_u32(&full[rs.idx]), 0);
                        const uint32_t dstA = smem_u32(sA + rs.idx * P_A_STAGE);
                        const uint32_t dstB = smem_u32(sB + rs.idx * P_B_STAGE);
                        if (BMODE == AB_TMA_MN) {
                            const int row = t.row0 + ks * BK;
                            tma_load_2d_pair(dstA, &p.a_map[0], bar, t.m0 + my_m, row);
                            tma_load_2d_pair(dstA + 8192, &p.a_map[0], bar, t.m0 + my_m + 64, row);
                            tma_load_2d_pair(dstB, &p.w_map[0], bar, t.n_t * P_BN + my_n, row);
                            tma_load_2d_pair(dstB + 8192, &p.w_map[0], bar, t.n_t * P_BN + my_n + 64, row);
                        } else {
                            tma_load_2d_pair(dstA, &p.a_map[seg], bar, ks * BK, t.m0 + my_m);
                            if (BMODE == B_TMA_K) tma_load_2d_pair(dstB, &p.w_map[seg], bar, ks * BK, t.n_t * P_BN + my_n);
                        }
                    }
                    __syncwarp();
                    rs.next(NS);
                    if (DEQ) {
                        ok = mbar_wait_idle(smem_u32(&empty_c[rc.idx]), rc.phase ^ 1u, abort_flag, p.errword, 12);
                        if (!ok) break;
                        if (lane == 0) {
                            uint32_t bar = smem_u32(&full_c[rc.idx]);
                            uint32_t dstC = smem_u32(sC + rc.idx * P_C_STAGE);
                            mbar_expect_tx(bar, P_C_STAGE);
                            if (BMODE == B_DEQ_MN) {
                                int row = t.e * p.w_rows + ks * BK;
                                if (DUAL) tma_load_2d(dstC, &p.w_map[rank], bar, t.n_t * 64, row);
                                else tma_load_2d(dstC, &p.w_map[seg], bar, (t.n_t * P_BN + my_n) / 2, row);
                            } else {
                                tma_load_2d(dstC, &p.w_map[seg], bar, ks * (BK / 2), t.e * p.w_rows + t.n_t * P_BN + my_n);
                            }
                        }
                        if (S_SMEM) {
                            const float *sp = DUAL ? p.scales[rank] : p.scales[seg];
                            float *sdst = sS + rc.idx * 128;
                            const size_t b0 = (size_t)(t.e * p.w_rows + ks * BK) * gpr + (DUAL ? t.n_t * 128 : t.n_t * P_BN + my_n) / 128;
#pragma unroll
                            for (int i = 0; i < 2; i++) cp_async4(sdst + lane + 32 * i, sp + b0 + (size_t)(lane + 32 * i) * gpr);
                            cp_async_arrive(smem_u32(&full_c[rc.idx]));
                        }
                        __syncwarp();
                        rc.next(NSC);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (leader) {
            // =============================== MMA issuer (leader CTA) ===============================
            Ring rs = {0, 0};
            bool ok = true;
            int it = 0;
            for (int tile = pair; ok && tile < total; tile += npairs, it++) {
                TileInfo t = decode_pair_tile<SCHED>(p, tile, ntr);
                const int acc = it & 1;
                ok = mbar_wait_cluster(smem_u32(&tmem_empty[acc]), (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag, p.errword, 13);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * P_BN;
                uint32_t accumulate = 0;
                for (int seg = 0; ok && seg < p.nseg; seg++) {
                    for (int ks = 0; ks < t.ksteps; ks++) {
                        ok = mbar_wait_cluster(smem_u32(&full[rs.idx]), rs.phase, abort_flag, p.errword, 14);
                        if (!ok) break;
                        tc_fence_after();
                        if (lane == 0) {
                            const uint32_t a0 = smem_u32(sA + rs.idx * P_A_STAGE);
                            const uint32_t b0 = smem_u32(sB + rs.idx * P_B_STAGE);
#pragma unroll
                            for (int k16 = 0; k16 < BK / 16; k16++) {
                                uint64_t ad = (BMODE == AB_TMA_MN) ? make_desc(a0 + k16 * 2048, 8192, 1024) : make_desc(a0 + k16 * 32, 16, 1024);
                                uint64_t bd = (BMODE == B_DEQ_MN || BMODE == AB_TMA_MN) ? make_desc(b0 + k16 * 2048, 8192, 1024)
                                                                                        : make_desc(b0 + k16 * 32, 16, 1024);
                                tc_mma2_bf16(tmem_d, ad, bd, IDESC, accumulate);
                                accumulate = 1;
                            }
                            tc_commit2_both(smem_u32(&empty[rs.idx]));
                        }
                        __syncwarp();
                        accumulate = 1;
                        rs.next(NS);
                    }
                }
                if (ok) {
                    if (lane == 0) tc_commit2_both(smem_u32(&tmem_full[acc]));
                    __syncwarp();
                }
            }
            if (*abort_flag) {
                if (lane == 0) tc_commit2(smem_u32(spare));
                __syncwarp();
                for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(smem_u32(spare), 0); i++) {}
            }
        }
    } else if (warp < 2 + EPI_WARPS) {
        // =============================== epilogue (both CTAs) ===============================
        // warp (q, h): q = TMEM lane quarter (= warp id mod 4), h = which 128 of the 256 columns
        const int q = warp & 3, h = (warp - 2) >> 2;
        uint8_t *stage = sE + (warp - 2) * epi_stage_bytes(EPI);
        EpiCtx ec = {bars + 48 + 2 * (warp - 2), 0u};
        bool ok = true;
        int it = 0;
        for (int tile = pair; ok && tile < total; tile += npairs, it++) {
            TileInfo t = decode_pair_tile<SCHED>(p, tile, ntr);
            const int acc = it & 1;
            const long long row0 = (long long)t.m0 + my_m + q * 32;
            int valid = 32;
            if (SCHED == SCHED_ROWS) valid = ((int)rank < t.halves) ? 32 : 0;
            else { long long left = (long long)p.M - row0; valid = left < 0 ? 0 : (left < 32 ? (int)left : 32); }
            const long long rbase = (SCHED == SCHED_GROUPK) ? ((long long)t.e * p.M + row0) : row0;
            const long long col0 = (EPI == EPI_SWIGLU) ? (long long)t.n_t * 128 + h * 64 : (long long)t.n_t * P_BN + h * 128;
            if (valid > 0) epilogue_prefetch<EPI>(p, stage, ec, lane, rbase, col0, valid);
            ok = mbar_wait_idle(smem_u32(&tmem_full[acc]), ((uint32_t)it >> 1) & 1u, abort_flag, p.errword, 19);
            if (!ok) break;
            tc_fence_after();
            if (valid > 0) {
                const bool have_acc = (SCHED != SCHED_GROUPK) || t.ksteps > 0;
                const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * P_BN;
                if (EPI == EPI_SWIGLU)
                    epilogue_rows<EPI, BMODE == B_DEQ_MN>(p, stage, ec, lane, tbase + (uint32_t)h * 64, rbase, col0, valid, have_acc, 128);
                else
                    epilogue_rows<EPI, BMODE == B_DEQ_MN>(p, stage, ec, lane, tbase + (uint32_t)h * 128, rbase, col0, valid, have_acc, 0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                const uint32_t te = smem_u32(&tmem_empty[acc]);
                if (leader) mbar_arrive(te); else mbar_arrive_remote(map_to_cta(te, 0));
            }
        }
        if (lane == 0) bulk_wait_all();                  // outstanding bulk stores of this warp
    } else if (DEQ) {
        // =============================== dequant warps (both CTAs) ===============================
        // The warps form DQG groups; group g expands the stages whose running index is g modulo
        // DQG, so one stage's chain (code read, expand, store, proxy fence, arrive) may take DQG
        // MMA stage times before it limits the tensor pipe.
        const int dw = warp - (2 + EPI_WARPS);
        constexpr int ITERS = (P_C_STAGE / 4) / (GW * 32);           // code words per lane and stage
        const int g = dw / GW, gw = dw % GW;
        // word i of a lane sits ROWS_I rows below word i-1; the swizzle term repeats every PER words
        constexpr int ROWS_I = (BMODE == B_DEQ_MN) ? 2 * GW : 4 * GW;
        constexpr int PER = ROWS_I >= 8 ? 1 : 8 / ROWS_I;
        const int r0 = (BMODE == B_DEQ_MN) ? gw * 2 + (lane >> 4) : gw * 4 + (lane >> 3);   // row of word 0
        const int c0 = (BMODE == B_DEQ_MN) ? (lane & 15) : (lane & 7);
        uint32_t dst0[PER];
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int r = r0 + i * ROWS_I;
            if (BMODE == B_DEQ_MN) dst0[i] = (uint32_t)((c0 / 8) * 8192 + (r >> 3) * 1024 + (r & 7) * 128 + (((c0 & 7) ^ (r & 7)) << 4));
            else dst0[i] = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c0 ^ (r & 7)) << 4));
        }
        constexpr uint32_t DST_STEP = (uint32_t)(PER * ROWS_I / 8) * 1024u;      // bytes per PER words
        Ring rc = {0, 0}, rb = {0, 0};
        bool ok = true;
        const uint32_t full0 = map_to_cta(smem_u32(&full[0]), 0);    // the leader's stage barriers
        const int gpr = p.w_cols / 128;
        int kc = 0;                                                  // running stage index of this CTA
        for (int tile = pair; ok && tile < total; tile += npairs) {
            TileInfo t = decode_pair_tile<SCHED>(p, tile, ntr);
            for (int seg = 0; ok && seg < p.nseg; seg++) {
                int ks = (g - kc % DQG + DQG) % DQG;                 // first stage of this group in the tile
                for (int i = 0; i < ks && i < t.ksteps; i++) { rc.next(NSC); rb.next(NS); }
                // codes [N][K]: scale of word i at stage ks is sp[sb + i * rstep + ks * 64 / 128]
                const float *sp = p.scales[seg];
                const int sb = (t.e * p.w_rows + t.n_t * P_BN + my_n + r0) * gpr, rstep = ROWS_I * gpr;
                float cur[ITERS], nxt[ITERS];
                if (!S_SMEM && ks < t.ksteps) {
#pragma unroll
                    for (int i = 0; i < ITERS; i++) cur[i] = __ldg(sp + sb + i * rstep + (ks * BK) / 128);
                }
                for (; ks < t.ksteps; ks += DQG) {
                    if (!S_SMEM && ks + DQG < t.ksteps) {
#pragma unroll
                        for (int i = 0; i < ITERS; i++) nxt[i] = __ldg(sp + sb + i * rstep + ((ks + DQG) * BK) / 128);
                    }
                    ok = mbar_wait_idle(smem_u32(&full_c[rc.idx]), rc.phase, abort_flag, p.errword, 20);
                    if (!ok) break;
                    const uint32_t *cw = reinterpret_cast<const uint32_t *>(sC + rc.idx * P_C_STAGE);
                    uint32_t w[ITERS];
#pragma unroll
                    for (int i = 0; i < ITERS; i++) w[i] = cw[(i * GW + gw) * 32 + lane];
                    if (S_SMEM) {
                        const float *sc = sS + rc.idx * 128 + r0;    // scale of word i: sc[i * ROWS_I]
#pragma unroll
                        for (int i = 0; i < ITERS; i++) cur[i] = sc[i * ROWS_I];
                    }
                    ok = mbar_wait_idle(smem_u32(&empty[rb.idx]), rb.phase ^ 1u, abort_flag, p.errword, 21);
                    if (!ok) break;
                    uint8_t *bdst = sB + rb.idx * P_B_STAGE;
#pragma unroll
                    for (int i = 0; i < ITERS; i++)
                        *reinterpret_cast<uint4 *>(bdst + dst0[i % PER] + (uint32_t)(i / PER) * DST_STEP) = (BMODE == B_DEQ_MN) ? dequant8_perm(w[i], __float2bfloat162_rn(cur[i])) : dequant8(w[i], __float2bfloat162_rn(cur[i]));
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive_remote(full0 + (uint32_t)rb.idx * 8u); mbar_arrive(smem_u32(&empty_c[rc.idx])); }
                    const int adv = ks + DQG <= t.ksteps ? DQG : t.ksteps - ks;
                    for (int i = 0; i < adv; i++) { rc.next(NSC); rb.next(NS); }
                    if (!S_SMEM) {
#pragma unroll
                        for (int i = 0; i < ITERS; i++) cur[i] = nxt[i];
                    }
                }
                kc += t.ksteps;
            }
        }
    }

    // =============================== teardown ===============================
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                      // the peer's shared memory stays alive until the leader's MMAs are done
    if (warp == 1) { tc_fence_after(); tmem_dealloc2(tmem_base, TMEM_COLS); }
}

}  // namespace qlmb
