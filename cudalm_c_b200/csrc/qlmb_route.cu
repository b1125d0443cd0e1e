// Top-k router and the stable expert-grouping permutation.
//
// Built with --fmad=false: the softmax uses the reference CPU build's
// polynomial exp and its sequential summation order so probabilities, gates
// and expert choices match that build bit for bit on the same logits.
#include "qlmb_common.cuh"
#include "qlmb_internal.h"

namespace qlmb {

// exp as the reference CPU build computes it (cpu_kern.h:28-34): clamp,
// two-part ln2 reduction, degree-6 polynomial, exponent by bit shift.
__device__ __forceinline__ float exp_poly(float x)
{
    x = x < -87.0f ? -87.0f : (x > 88.0f ? 88.0f : x);
    float k = rintf(x * 1.44269504089f);
    float r = x - k * 0.693145751953125f;
    r -= k * 1.428606765330187e-06f;
    float p = 1.0f / 720;
    p = 1.0f / 120 + r * p;
    p = 1.0f / 24 + r * p;
    p = 1.0f / 6 + r * p;
    p = 0.5f + r * p;
    p = 1.0f + r * p;
    p = 1.0f + r * p;
    return p * __uint_as_float((uint32_t)((int)k + 127) << 23);
}

// Same arithmetic with one warp per token and lane = expert (E <= 32): the
// maximum is order-free, the softmax sum is still taken in expert order (every
// lane adds the 32 shuffled terms sequentially) and the K selection rounds are
// warp arg-max reductions with the lowest index winning ties, so the outputs are
// bit-identical to the thread-per-token form above.
// the softmax and the K selection rounds of token n by one warp; lg = the logit of expert `lane` (0 beyond E)
__device__ __forceinline__ void router_topk_row(float lg, int n, int lane, float *rprobs, int *assign, float *gate, int N,
                                                int E, int K, const float *bias, int bs)
{
    const bool live = lane < E;
    float top = (live && lg > -1e30f) ? lg : -1e30f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float p = live ? exp_poly(lg - top) : 0.0f;
    float sum = 0.0f;
    for (int e = 0; e < E; e++) sum += __shfl_sync(0xffffffffu, p, e);
    float inv = 1.0f / sum;
    float pr = p * inv;
    if (live) rprobs[(size_t)n * E + lane] = pr;
    bool taken = false;
    for (int k = 0; k < K; k++) {
        float sc = pr + (bias && live ? bias[k * bs + lane] : 0.0f);
        bool ok = live && !taken && (sc > -1e30f);
        int idx = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float osc = __shfl_xor_sync(0xffffffffu, sc, o);
            int oidx = __shfl_xor_sync(0xffffffffu, idx, o);
            bool ook = __shfl_xor_sync(0xffffffffu, (int)ok, o) != 0;
            bool take = ook && (!ok || osc > sc || (osc == sc && oidx < idx));
            if (take) { sc = osc; idx = oidx; ok = true; }
        }
        int pick = ok ? idx : k;                    // NaN scores: stay in range
        float g = __shfl_sync(0xffffffffu, pr, pick);
        if (lane == 0) { assign[(size_t)k * N + n] = pick; gate[(size_t)k * N + n] = g; }
        taken = taken || (lane == pick);
    }
}
// More than 32 experts (up to 256): still one warp per token, lane l holds experts l, l + 32, ... (EPT per lane).
// The softmax sum runs over the experts in ascending order (the term of expert e is fetched from lane e % 32), as the
// reference's CPU kernel adds them (cpu_kern.h:413-425); each selection round takes every lane's best unused expert
// (lowest index on ties) and then the best over the lanes, again with the lowest index winning.
template <int EPT>
__global__ void __launch_bounds__(256) k_router_topk_wide(const float *rt, float *rprobs, int *assign, float *gate, int N,
                                                          int E, int K, const float *bias, int bs)
{
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    float lg[EPT], pr[EPT];
    float top = -1e30f;
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        const int e = j * 32 + lane;
        lg[j] = e < E ? rt[(size_t)n * E + e] : -1e30f;
        if (lg[j] > top) top = lg[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        pr[j] = (j * 32 + lane < E) ? exp_poly(lg[j] - top) : 0.0f;
        const int live = E - j * 32 < 32 ? E - j * 32 : 32;           // experts of this slice
        for (int l = 0; l < live; l++) sum += __shfl_sync(0xffffffffu, pr[j], l);
    }
    const float inv = 1.0f / sum;
    unsigned used = 0u;                                               // bit j: this lane's expert j * 32 + lane was picked
#pragma unroll
    for (int j = 0; j < EPT; j++) {
        pr[j] *= inv;
        if (j * 32 + lane < E) rprobs[(size_t)n * E + j * 32 + lane] = pr[j];
    }
    for (int k = 0; k < K; k++) {
        float sc = 0.0f; int idx = 0x7fffffff; bool ok = false;
#pragma unroll
        for (int j = 0; j < EPT; j++) {
            const int e = j * 32 + lane;
            if (e >= E || ((used >> j) & 1u)) continue;
            const float v = pr[j] + (bias ? bias[k * bs + e] : 0.0f);
            if (v > -1e30f && (!ok || v > sc)) { sc = v; idx = e; ok = true; }      // ascending e: the first best stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float osc = __shfl_xor_sync(0xffffffffu, sc, o);
            const int oidx = __shfl_xor_sync(0xffffffffu, idx, o);
            const bool ook = __shfl_xor_sync(0xffffffffu, (int)ok, o) != 0;
            if (ook && (!ok || osc > sc || (osc == sc && oidx < idx))) { sc = osc; idx = oidx; ok = true; }
        }
        const int pick = ok ? idx : k;                                // NaN scores: stay in range
        float g = 0.0f;
#pragma unroll
        for (int j = 0; j < EPT; j++) {
            const float v = __shfl_sync(0xffffffffu, pr[j], pick & 31);
            if ((pick >> 5) == j) g = v;
        }
        if (lane == 0) { assign[(size_t)k * N + n] = pick; gate[(size_t)k * N + n] = g; }
        if ((pick & 31) == lane) used |= 1u << (pick >> 5);
    }
}

__global__ void __launch_bounds__(256) k_router_topk_warp(const float *rt, float *rprobs, int *assign,
                                                          float *gate, int N, int E, int K,
                                                          const float *bias, int bs)
{
    int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    router_topk_row(lane < E ? rt[(size_t)n * E + lane] : 0.0f, n, lane, rprobs, assign, gate, N, E, K, bias, bs);
}

// A decode step's few rows: logits and selection in one launch, one block per token.  The logits are those of
// k_router_logits_small (lane = expert, eight warps each sum one eighth of the features in ascending order with fused
// multiply-adds, the eight partial sums added in warp order); warp 0 then runs the selection above on them.
// With perm != NULL (at most 256 routed slots) the block that finishes last also groups the K*N slots by expert in
// stable order (what k_perm_cluster does in a launch of its own): perm[off[e] ..] = the slots of expert e ascending,
// off[0..E], counts[0..E), *bad = an expert id out of range.  The blocks take tickets after a fence, so the last one sees
// every block's choices; the result does not depend on which block that is.
__device__ unsigned g_router_ticket;
__global__ void __launch_bounds__(256) k_router_small(float *rt, const void *X, int x_dtype, const float *Wr, float *rprobs,
                                                      int *assign, float *gate, int N, int D, int E, int K,
                                                      const float *bias, int bs, int *perm, int *off, int *counts, int *bad)
{
    extern __shared__ float rs_x[];                      // D activations
    __shared__ float part[8][32];
    const int n = blockIdx.x, warp = threadIdx.x >> 5, e = threadIdx.x & 31;
    const int per = (D + 7) / 8, j0 = warp * per, j1 = j0 + per < D ? j0 + per : D;
    // 32 rows of Wr in flight per lane (the loads depend neither on the sum nor on the activations: the first batch is
    // requested before the row is staged); the sum itself stays in ascending order
    float w[32];
    pdl_trigger();
    if (e < E) {
#pragma unroll
        for (int u = 0; u < 32; u++) w[u] = j0 + u < j1 ? __ldg(Wr + (size_t)(j0 + u) * E + e) : 0.0f;
    }
    pdl_wait();                                          // the router matrix above is no kernel's output; the row below is
    for (int j = threadIdx.x; j < D; j += 256)
        rs_x[j] = x_dtype == QLMB_BF16 ? __bfloat162float(((const bf16 *)X)[(size_t)n * D + j]) : ((const float *)X)[(size_t)n * D + j];
    __syncthreads();
    float acc = 0.0f;
    if (e < E) {
        for (int j = j0; j < j1; j += 32) {
            if (j > j0) {
#pragma unroll
                for (int u = 0; u < 32; u++) w[u] = j + u < j1 ? __ldg(Wr + (size_t)(j + u) * E + e) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 32; u++)
                if (j + u < j1) acc = __fmaf_rn(rs_x[j + u], w[u], acc);
        }
    }
    part[warp][e] = acc;
    __syncthreads();
    if (warp == 0) {
        float lg = 0.0f;
        if (e < E) {
            lg = part[0][e];
#pragma unroll
            for (int w = 1; w < 8; w++) lg += part[w][e];
            rt[(size_t)n * E + e] = lg;
        }
        router_topk_row(lg, n, e, rprobs, assign, gate, N, E, K, bias, bs);
        __threadfence();                                 // this token's choices are visible before its ticket is
    }
    if (!perm) return;
    __shared__ int s_last, s_asn[256], s_off[33], s_bad;
    __syncthreads();
    if (threadIdx.x == 0) { s_last = atomicAdd(&g_router_ticket, 1u) == (unsigned)(N - 1); s_bad = 0; }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int R = K * N, t = threadIdx.x;
    int my = -1;
    if (t < R) {
        my = __ldcg(assign + t);
        if (my < 0 || my >= E) { atomicMax(&s_bad, 1); my = -1; }
        s_asn[t] = my;
    }
    __syncthreads();
    if (warp == 0) {                                     // lane = expert: count, exclusive scan, offsets
        int c = 0;
        if (e < E) for (int i = 0; i < R; i++) c += s_asn[i] == e;
        int incl = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, d); if (e >= d) incl += v; }
        if (e < E) { s_off[e] = incl - c; off[e] = incl - c; if (counts) counts[e] = c; }
        if (e == E - 1) { s_off[E] = incl; off[E] = incl; }
    }
    __syncthreads();
    if (my >= 0) {
        int rank = 0;
        for (int i = 0; i < t; i++) rank += s_asn[i] == my;
        perm[s_off[my] + rank] = t;
    }
    if (t == 0) { if (bad) *bad = s_bad; g_router_ticket = 0u; }
}

// ------------------------------------------------------------- permutation
// Stable grouping of `len` slots by expert in ONE launch (the reference takes a histogram, a scan and a scatter
// kernel with a host-visible scratch between them, cudalm.cu:3504-3530).  A thread-block cluster of C CTAs of
// 1024 threads owns one sort; CTA c owns a contiguous range of slots and warp w of it a contiguous piece of that
// range, so "stable" means: slots are placed in (CTA, warp, row of 32, lane) order.  Every thread keeps its slots'
// expert ids in registers (at most PERM_RPT), so the input is read once.
//   count    warp-private histograms in shared memory (shared-memory atomics, order irrelevant)
//   scan     per expert: exclusive prefix of the 32 warp counts by warp shuffles (lane = warp), the CTA totals are
//            exchanged through distributed shared memory after one cluster barrier, and every CTA derives the
//            padded expert offsets itself (an exclusive scan of at most 256 totals by one warp)
//   place    row by row: the lanes holding the same expert are found with one ballot per bit of the expert id,
//            a lane's position is offset + CTA base + warp base + running count + its rank among those lanes
// CTA 0 also writes what depends only on the totals: offsets, counts, filler slots (-1), the row-tile table of the
// grouped GEMMs, the per-rank send counts of the expert-parallel exchange and the out-of-range flag.
#define PERM_THREADS 1024
#define PERM_RPT 16                 // rows (slots per thread) a CTA can hold: 16384 slots per CTA, 131072 per cluster of 8
#define PERM_EMAX 256

struct PermArgs {
    const int *asn; int len, E, pad, plen;
    int *perm, *inv, *off, *counts, *tile_info, *ntiles, *bad, *errword;
    int e_lo, skip;
    int *rank_counts; int experts_per_rank;      // optional: slots per destination rank (experts_per_rank experts each)
};

__device__ __forceinline__ uint32_t perm_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t perm_cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void perm_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void perm_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// store into the same shared-memory location of CTA `rank` of the cluster
__device__ __forceinline__ void perm_st_remote(int *local, uint32_t rank, int v)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(r), "r"(v) : "memory");
}

// RPT = rows of 32 slots per warp (slots per thread kept in registers)
template <int RPT>
__global__ void __launch_bounds__(PERM_THREADS) k_perm_cluster(const PermArgs a0, int sorts_stride_asn)
{
    extern __shared__ int psm[];
    PermArgs a = a0;
    const int E = a.E, sort = blockIdx.y;
    int *wh = psm;                          // [32][E] warp histograms, then exclusive warp prefixes
    int *tot = wh + 32 * E;                 // [E] this CTA's totals
    int *rtot = tot + E;                    // [8][E] every CTA's totals, written by their owners (remote stores)
    int *base = rtot + 8 * E;               // [E] slots of the CTAs before this one
    int *gtot = base + E;                   // [E] totals of the sort
    int *po = gtot + E;                     // [E + 1] padded offsets
    int *rbad = po + E + 1;                 // [8] every CTA's out-of-range finding
    int *sbad = rbad + 8;                   // [1]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t crank = perm_cluster_rank(), csize = perm_cluster_size();
    perm_cluster_arrive();                  // phase 0: "this CTA runs"; waited for just before the first remote store
    a.asn += (size_t)sort * sorts_stride_asn;
    a.perm += (size_t)sort * a.plen;
    if (a.inv) a.inv += (size_t)sort * a.len;
    a.off += (size_t)sort * (E + 1);
    if (a.counts) a.counts += (size_t)sort * E;

    // slots of this CTA and of this warp (rows of 32 slots, whole rows per warp)
    const int rows_total = (a.len + 31) / 32;
    const int rows_cta = (rows_total + (int)csize - 1) / (int)csize;
    const int row0 = (int)crank * rows_cta + warp * RPT;
    int row1 = row0 + RPT;
    int cta_end = ((int)crank + 1) * rows_cta;
    if (cta_end > rows_total) cta_end = rows_total;
    if (row1 > cta_end) row1 = cta_end;

    // ---- count: the slots are requested first, the histograms zeroed while they travel
    int ex[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int i = (row0 + r) * 32 + lane;
        ex[r] = (row0 + r < row1 && i < a.len) ? a.asn[i] - a.e_lo : -0x40000000;
    }
    for (int i = tid; i < 32 * E; i += PERM_THREADS) wh[i] = 0;
    if (tid == 0) *sbad = 0;
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int e = ex[r];
        if ((unsigned)e < (unsigned)E) atomicAdd(&wh[warp * E + e], 1);
        else {
            if (e != -0x40000000 && !a.skip) atomicMax(reinterpret_cast<unsigned *>(sbad), (unsigned)((e + a.e_lo) | 0x40000000));
            ex[r] = -1;
        }
    }
    __syncthreads();
    // ---- scan over the warps: warp v takes experts v, v + 32, ...; lane = the warp whose count it holds
    for (int e = warp; e < E; e += 32) {
        const int c = wh[lane * E + e];
        int x = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        wh[lane * E + e] = x - c;
        if (lane == 31) tot[e] = x;
    }
    __syncthreads();
    perm_cluster_wait();                    // phase 0 complete: every CTA of the cluster has started
    for (int i = tid; i < E * (int)csize; i += PERM_THREADS) perm_st_remote(&rtot[crank * E + i % E], (uint32_t)(i / E), tot[i % E]);
    if (tid < (int)csize) perm_st_remote(&rbad[crank], (uint32_t)tid, *sbad);
    perm_cluster_arrive();
    perm_cluster_wait();                    // phase 1: all totals have landed; nothing remote is touched after this
    for (int e = tid; e < E; e += PERM_THREADS) {
        int before = 0, all = 0;
        for (int c = 0; c < (int)csize; c++) { const int t = rtot[c * E + e]; if (c < (int)crank) before += t; all += t; }
        base[e] = before; gtot[e] = all;
    }
    __syncthreads();
    if (warp == 0) {                        // padded offsets: lane l scans experts 8l .. 8l + 7
        int v[8], s = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) { const int e = lane * 8 + k; v[k] = e < E ? (gtot[e] + a.pad - 1) / a.pad * a.pad : 0; s += v[k]; }
        int x = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        int run = x - s;
#pragma unroll
        for (int k = 0; k < 8; k++) { const int e = lane * 8 + k; if (e < E) po[e] = run; run += v[k]; }
        if (lane == 31) po[E] = x;
    }
    __syncthreads();
    // ---- place
    const int nbits = 32 - __clz(E - 1 > 0 ? E - 1 : 1);
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        if (row0 + r < row1) {              // the same for every lane of the warp
            const int e = ex[r];
            unsigned same = __ballot_sync(0xffffffffu, e >= 0);
            for (int b = 0; b < nbits; b++) {
                const unsigned m = __ballot_sync(0xffffffffu, (e >> b) & 1);
                same &= ((e >> b) & 1) ? m : ~m;
            }
            const int i = (row0 + r) * 32 + lane;
            if (e >= 0) {
                const int pos = po[e] + base[e] + wh[warp * E + e] + __popc(same & ((1u << lane) - 1u));
                a.perm[pos] = i;
                if (a.inv) a.inv[i] = pos;
            } else if (a.inv && i < a.len) a.inv[i] = -1;
            __syncwarp();
            if (e >= 0 && (same >> lane) >> 1 == 0) wh[warp * E + e] += __popc(same);     // the highest lane of each expert advances the run
            __syncwarp();
        }
    }
    // ---- what depends only on the totals (CTA 0)
    if (crank != 0) return;
    for (int e = tid; e <= E; e += PERM_THREADS) a.off[e] = po[e];
    if (a.counts) for (int e = tid; e < E; e += PERM_THREADS) a.counts[e] = gtot[e];
    if (a.pad > 1)
        for (int i = tid; i < E * (a.pad - 1); i += PERM_THREADS) {
            const int e = i / (a.pad - 1), p = po[e] + gtot[e] + i % (a.pad - 1);
            if (p < po[e + 1]) a.perm[p] = -1;
        }
    if (a.rank_counts && sort == 0 && a.experts_per_rank > 0)
        for (int r = tid; r * a.experts_per_rank < E; r += PERM_THREADS) {
            int s = 0;
            for (int e = r * a.experts_per_rank; e < (r + 1) * a.experts_per_rank && e < E; e++) s += gtot[e];
            a.rank_counts[r] = s;
        }
    // row tiles of the grouped GEMMs (pad = 128): up to 256 rows of one expert each, packed as
    // first row / 128 | expert << 20 | (halves - 1) << 30, in expert order; one thread per (expert, tile)
    if (a.tile_info && sort == 0) {
        if (warp == 1) {
            int v[8], s = 0;
#pragma unroll
            for (int k = 0; k < 8; k++) { const int e = lane * 8 + k; v[k] = e < E ? ((po[e + 1] - po[e]) / 128 + 1) / 2 : 0; s += v[k]; }
            int x = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
            int nt = x - s;
#pragma unroll
            for (int k = 0; k < 8; k++) { const int e = lane * 8 + k; if (e < E) base[e] = nt; nt += v[k]; }     // base is free now: first tile of e
            if (lane == 31) *a.ntiles = x;
        }
        __syncthreads();
        for (int e = warp; e < E; e += 32) {
            const int n128 = (po[e + 1] - po[e]) / 128;
            for (int t = lane; 2 * t < n128; t += 32)
                a.tile_info[base[e] + t] = (po[e] / 128 + 2 * t) | (e << 20) | ((2 * t + 1 < n128 ? 1 : 0) << 30);
        }
    }
    if (tid == 0) {
        unsigned b = 0u;
        for (int c = 0; c < (int)csize; c++) { const unsigned t = (unsigned)rbad[c]; b = t > b ? t : b; }
        // one sort: this thread is the flag's only writer; several sorts: the flag was zeroed before the launch
        if (gridDim.y == 1) *a.bad = (int)b; else if (b) atomicMax(reinterpret_cast<unsigned *>(a.bad), b);
        if (b && a.errword) { a.errword[0] = 100; a.errword[1] = (int)b & ~0x40000000; }
    }
}

int perm_build(const int *assign, int N, int E, int K, int merged, int pad, int *perm, int *inv,
               int *off, int *counts, int *bad_flag, int *tile_info, int *ntiles,
               int *chunk_scratch, cudaStream_t st, int e_lo, int skip, int *rank_counts, int experts_per_rank)
{
    (void)chunk_scratch;
    const int sorts = merged ? 1 : K, len = merged ? K * N : N;
    QLMB_REQUIRE(E >= 1 && E <= PERM_EMAX, "perm_build: %d experts (at most %d)", E, PERM_EMAX);
    const int rows = (len + 31) / 32;
    int C = 1;
    while (C < 8 && (rows + C - 1) / C > 2 * 32) C *= 2;             // two rows per warp while the cluster may grow
    const int rpw = ((rows + C - 1) / C + 31) / 32;                  // rows per warp
    QLMB_REQUIRE(rpw <= PERM_RPT, "perm_build: %d slots exceed one cluster's capacity (%d)", len, 8 * PERM_RPT * 1024);
    PermArgs a = {assign, len, E, pad, len + E * (pad - 1), perm, inv, off, counts, tile_info, ntiles, bad_flag,
                  device_error_word(), e_lo, skip, rank_counts, experts_per_rank};
    const size_t smem = ((size_t)32 * E + 12 * (size_t)E + 1 + 9) * sizeof(int);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(C, sorts, 1); cfg.blockDim = dim3(PERM_THREADS, 1, 1); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (sorts > 1) QLMB_CUDA(cudaMemsetAsync(bad_flag, 0, sizeof(int), st));
    cudaError_t le;
    if (rpw <= 1) le = cudaLaunchKernelEx(&cfg, k_perm_cluster<1>, a, len);
    else if (rpw <= 2) le = cudaLaunchKernelEx(&cfg, k_perm_cluster<2>, a, len);
    else if (rpw <= 4) le = cudaLaunchKernelEx(&cfg, k_perm_cluster<4>, a, len);
    else if (rpw <= 8) le = cudaLaunchKernelEx(&cfg, k_perm_cluster<8>, a, len);
    else le = cudaLaunchKernelEx(&cfg, k_perm_cluster<16>, a, len);
    QLMB_CUDA(le);
    QLMB_LAUNCH_CHECK("perm_build");
    return QLMB_OK;
}

// the permutation needs no scratch any more; callers that carve one out of their arena get a token size
size_t perm_scratch_ints(int N, int E, int K, int merged)
{
    (void)N; (void)E; (void)K; (void)merged;
    return 64;
}

int router_topk(const float *rt, float *rprobs, int *assign, float *gate, int N, int E, int K,
                const float *bias, int bs, cudaStream_t st)
{
    if (E <= 32) k_router_topk_warp<<<(N + 7) / 8, 256, 0, st>>>(rt, rprobs, assign, gate, N, E, K, bias, bs);
    else if (E <= 64) k_router_topk_wide<2><<<(N + 7) / 8, 256, 0, st>>>(rt, rprobs, assign, gate, N, E, K, bias, bs);
    else if (E <= 128) k_router_topk_wide<4><<<(N + 7) / 8, 256, 0, st>>>(rt, rprobs, assign, gate, N, E, K, bias, bs);
    else k_router_topk_wide<8><<<(N + 7) / 8, 256, 0, st>>>(rt, rprobs, assign, gate, N, E, K, bias, bs);
    QLMB_LAUNCH_CHECK("k_router_topk");
    return QLMB_OK;
}

int router_small(float *rt, const void *X, int x_dtype, const float *Wr, float *rprobs, int *assign, float *gate, int N, int D,
                 int E, int K, const float *bias, int bs, cudaStream_t st, int *perm, int *off, int *counts, int *bad, int *perm_done)
{
    if (perm_done) *perm_done = 0;
    if (N > 64 || E > 32 || D > 8192) {
        int rc = router_logits_small(rt, X, x_dtype, Wr, N, D, E, st);
        return rc ? rc : router_topk(rt, rprobs, assign, gate, N, E, K, bias, bs, st);
    }
    const bool fuse = perm && off && perm_done && K * N <= 256;      // the last block also groups the slots by expert
    if (fuse) *perm_done = 1;
    QLMB_CUDA(pdl_launch(N > 4, k_router_small, dim3(N), dim3(256), (size_t)D * sizeof(float), st, rt, X, x_dtype, Wr, rprobs, assign, gate, N, D, E, K, bias, bs,
                         fuse ? perm : (int *)nullptr, off, counts, bad));
    QLMB_LAUNCH_CHECK("k_router_small");
    return QLMB_OK;
}

// ---------------------------------------------------------------- selection bias
// mbias_upd (cudalm.cu:3791-3802): aux-free balancing.  After routing, the selection-only bias of expert e moves
// towards the target load m: b += u * (m - count_e) / m (proportional form) or b += u * sign(m - count_e).
// With one bias row per top-k pass (the reference's default) block k counts pass k's assignments, otherwise one
// block counts all K*N.  The counts are integer histograms in shared memory, so the result does not depend on
// scheduling; the reference copies the counts to the host and the bias back, here nothing leaves the device.
__global__ void __launch_bounds__(256) k_bias_update(float *bias, const int *assign, int N, int E, int K, int per_slot,
                                                     float u, int proportional)
{
    __shared__ int hist[256];
    const int s = blockIdx.x;
    for (int e = threadIdx.x; e < E; e += 256) hist[e] = 0;
    __syncthreads();
    const int *a = per_slot ? assign + (size_t)s * N : assign;
    const int n = per_slot ? N : K * N;
    for (int i = threadIdx.x; i < n; i += 256) {
        const int e = a[i];
        if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    const float m = per_slot ? (float)N / (float)E : (float)K * (float)N / (float)E;
    for (int e = threadIdx.x; e < E; e += 256) {
        const float c = (float)hist[e];
        const float d = proportional ? (m - c) / m : (c < m ? 1.0f : c > m ? -1.0f : 0.0f);
        bias[(size_t)s * E + e] += u * d;
    }
}

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_perm_build(const int *assign, int N, int E, int K, int merged, int pad, int *perm,
                               int *inv, int *off, int *counts, int *bad_flag, void *stream)
{
    QLMB_REQUIRE(assign && perm && off && bad_flag, "qlmb_perm_build: NULL argument");
    QLMB_REQUIRE(N > 0 && E > 0 && E <= 256 && K > 0 && K <= 8 && pad >= 1, "qlmb_perm_build: N=%d E=%d K=%d pad=%d", N, E, K, pad);
    return perm_build(assign, N, E, K, merged, pad, perm, inv, off, counts, bad_flag, nullptr, nullptr, nullptr, as_stream(stream));
}

extern "C" int qlmb_router_bias_update(float *bias, const int *assign, int N, int E, int K, int per_slot, float u,
                                       int proportional, void *stream)
{
    QLMB_REQUIRE(bias && assign, "qlmb_router_bias_update: NULL argument");
    QLMB_REQUIRE(N > 0 && E > 0 && E <= 256 && K > 0 && K <= 8, "qlmb_router_bias_update: N=%d E=%d K=%d", N, E, K);
    if (u == 0.0f) return QLMB_OK;
    k_bias_update<<<per_slot ? K : 1, 256, 0, as_stream(stream)>>>(bias, assign, N, E, K, per_slot, u, proportional);
    QLMB_LAUNCH_CHECK("k_bias_update");
    return QLMB_OK;
}
