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

// One thread per token (reference cudalm.cu:2515-2534).  The probabilities
// live in rprobs (global, L1-resident) so any E up to 256 needs no local array.
__global__ void __launch_bounds__(128) k_router_topk(const float *rt, float *rprobs, int *assign,
                                                     float *gate, int N, int E, int K,
                                                     const float *bias, int bs)
{
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const float *lg = rt + (size_t)n * E;
    float *pr = rprobs + (size_t)n * E;
    float top = -1e30f;
    for (int e = 0; e < E; e++) { float v = lg[e]; if (v > top) top = v; }
    float sum = 0.0f;
    for (int e = 0; e < E; e++) { float p = exp_poly(lg[e] - top); pr[e] = p; sum += p; }
    float inv = 1.0f / sum;
    for (int e = 0; e < E; e++) pr[e] *= inv;
    int took[8];
    for (int k = 0; k < K; k++) {
        int pick = -1; float best = -1e30f;
        for (int e = 0; e < E; e++) {
            bool used = false;
            for (int j = 0; j < k; j++) used |= (took[j] == e);
            if (used) continue;
            float sc = pr[e] + (bias ? bias[k * bs + e] : 0.0f);
            if (sc > best) { best = sc; pick = e; }
        }
        if (pick < 0) pick = k;                     // NaN scores: stay in range
        took[k] = pick;
        assign[(size_t)k * N + n] = pick;
        gate[(size_t)k * N + n] = pr[pick];
    }
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
__global__ void __launch_bounds__(256) k_router_small(float *rt, const void *X, int x_dtype, const float *Wr, float *rprobs,
                                                      int *assign, float *gate, int N, int D, int E, int K,
                                                      const float *bias, int bs)
{
    extern __shared__ float rs_x[];                      // D activations
    __shared__ float part[8][32];
    const int n = blockIdx.x, warp = threadIdx.x >> 5, e = threadIdx.x & 31;
    const int per = (D + 7) / 8, j0 = warp * per, j1 = j0 + per < D ? j0 + per : D;
    // 32 rows of Wr in flight per lane (the loads depend neither on the sum nor on the activations: the first batch is
    // requested before the row is staged); the sum itself stays in ascending order
    float w[32];
    if (e < E) {
#pragma unroll
        for (int u = 0; u < 32; u++) w[u] = j0 + u < j1 ? __ldg(Wr + (size_t)(j0 + u) * E + e) : 0.0f;
    }
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
    if (warp != 0) return;
    float lg = 0.0f;
    if (e < E) {
        lg = part[0][e];
#pragma unroll
        for (int w = 1; w < 8; w++) lg += part[w][e];
        rt[(size_t)n * E + e] = lg;
    }
    router_topk_row(lg, n, e, rprobs, assign, gate, N, E, K, bias, bs);
}

// ------------------------------------------------------------- permutation
// Stable counting sort in three launches (chunks of 1024 entries):
//   hist    : per-chunk expert histogram
//   scan    : expert offsets (each segment rounded up to `pad`), per-chunk
//             bases, filler entries (-1), the row-tile table for the grouped
//             GEMMs and the unpadded counts
//   scatter : in-chunk stable rank (warp match + per-warp prefix) -> perm, inv
#define PERM_CHUNK 1024

// e_lo / skip: expert ids are taken relative to e_lo; with skip != 0 a slot whose id falls outside
// [e_lo, e_lo + E) is left out (inv = -1) instead of being reported as an error
__global__ void __launch_bounds__(PERM_CHUNK) k_perm_hist(const int *asn, int len, int E, int NC,
                                                          int *ch, int *bad, int e_lo, int skip)
{
    extern __shared__ int h[];
    int c = blockIdx.x, k = blockIdx.y, i = c * PERM_CHUNK + threadIdx.x;
    for (int e = threadIdx.x; e < E; e += blockDim.x) h[e] = 0;
    __syncthreads();
    if (i < len) {
        int e = asn[(size_t)k * len + i] - e_lo;
        if ((unsigned)e >= (unsigned)E) { if (!skip) atomicExch(bad, (e + e_lo) | 0x40000000); }
        else atomicAdd(&h[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) ch[((size_t)k * E + e) * NC + c] = h[e];
}

__global__ void __launch_bounds__(256) k_perm_scan(int *ch, int E, int NC, int pad, int plen,
                                                   int *off, int *counts, int *perm,
                                                   int *tile_info, int *ntiles,
                                                   const int *bad, int *errword)
{
    extern __shared__ int sm[];           // [E] totals, [E+1] padded offsets, then (when it fits) the E*NC chunk counts
    int *tot = sm, *po = sm + E, *cs = sm + 2 * E + 1;
    const int k = blockIdx.x;
    int *cp = ch + (size_t)k * E * NC;
    const bool staged = (size_t)E * NC <= 8192;          // chunk counts through shared memory: no dependent global accesses
    if (staged) {
        for (int i = threadIdx.x; i < E * NC; i += blockDim.x) cs[i] = cp[i];
        __syncthreads();
    }
    const int *src = staged ? cs : cp;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int s = 0;
        for (int c = 0; c < NC; c++) s += src[(size_t)e * NC + c];
        tot[e] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int e = 0; e < E; e++) {
            po[e] = s;
            s += (tot[e] + pad - 1) / pad * pad;
        }
        po[E] = s;
        if (*bad && errword) { errword[0] = 100; errword[1] = *bad & ~0x40000000; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) off[(size_t)k * (E + 1) + e] = po[e];
    if (counts) for (int e = threadIdx.x; e < E; e += blockDim.x) counts[(size_t)k * E + e] = tot[e];
    // chunk bases
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int s = po[e];
        if (staged) {
            for (int c = 0; c < NC; c++) { int t = cs[e * NC + c]; cs[e * NC + c] = s; s += t; }
        } else {
            for (int c = 0; c < NC; c++) { int t = cp[(size_t)e * NC + c]; cp[(size_t)e * NC + c] = s; s += t; }
        }
    }
    if (staged) {
        __syncthreads();
        for (int i = threadIdx.x; i < E * NC; i += blockDim.x) cp[i] = cs[i];
    }
    // filler rows: the padded tail of every expert segment, all experts at once
    if (pad > 1)
        for (int i = threadIdx.x; i < E * (pad - 1); i += blockDim.x) {
            const int e = i / (pad - 1), p = po[e] + tot[e] + i % (pad - 1);
            if (p < po[e + 1]) perm[(size_t)k * plen + p] = -1;
        }
    // row tiles of the grouped GEMMs (pad must be 128): up to 256 rows of one expert each,
    // packed as first row / 128 | expert << 20 | (halves - 1) << 30; expert e's tiles start
    // at the number of tiles of the experts before it
    if (tile_info && k == 0) {
        __shared__ int tbase[257];
        if (threadIdx.x == 0) {
            int nt = 0;
            for (int e = 0; e < E; e++) { tbase[e] = nt; nt += ((po[e + 1] - po[e]) / 128 + 1) / 2; }
            tbase[E] = nt;
            *ntiles = nt;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            const int n128 = (po[e + 1] - po[e]) / 128;
            int nt = tbase[e];
            for (int i = 0; i < n128; i += 2)
                tile_info[nt++] = (po[e] / 128 + i) | (e << 20) | ((i + 1 < n128 ? 1 : 0) << 30);
        }
    }
}

__global__ void __launch_bounds__(PERM_CHUNK) k_perm_scatter(const int *asn, int len, int E, int NC,
                                                             const int *base, int *perm, int plen,
                                                             int *inv, int e_lo)
{
    extern __shared__ int wc[];           // [32 warps][E] counts of the chunk
    int c = blockIdx.x, k = blockIdx.y, i = c * PERM_CHUNK + threadIdx.x;
    int w = threadIdx.x >> 5, ln = threadIdx.x & 31;
    for (int j = threadIdx.x; j < 32 * E; j += blockDim.x) wc[j] = 0;
    __syncthreads();
    int e = -1;
    if (i < len) { e = asn[(size_t)k * len + i] - e_lo; if ((unsigned)e >= (unsigned)E) e = -1; }
    unsigned peers = __match_any_sync(0xffffffffu, e);
    int rank = __popc(peers & ((1u << ln) - 1u));
    if (e >= 0 && rank == 0) wc[w * E + e] = __popc(peers);
    __syncthreads();
    if (e < 0) { if (inv && i < len) inv[(size_t)k * len + i] = -1; return; }
    int pos = base[((size_t)k * E + e) * NC + c] + rank;
    for (int j = 0; j < w; j++) pos += wc[j * E + e];
    perm[(size_t)k * plen + pos] = i;
    if (inv) inv[(size_t)k * len + i] = pos;
}

int perm_build(const int *assign, int N, int E, int K, int merged, int pad, int *perm, int *inv,
               int *off, int *counts, int *bad_flag, int *tile_info, int *ntiles,
               int *chunk_scratch, cudaStream_t st, int e_lo, int skip)
{
    int sorts = merged ? 1 : K, len = merged ? K * N : N;
    int NC = (len + PERM_CHUNK - 1) / PERM_CHUNK;
    int plen = len + E * (pad - 1);
    QLMB_CUDA(cudaMemsetAsync(bad_flag, 0, sizeof(int), st));
    k_perm_hist<<<dim3(NC, sorts), PERM_CHUNK, E * sizeof(int), st>>>(assign, len, E, NC, chunk_scratch, bad_flag, e_lo, skip);
    k_perm_scan<<<sorts, 256, (2 * E + 1 + ((size_t)E * NC <= 8192 ? (size_t)E * NC : 0)) * sizeof(int), st>>>(chunk_scratch, E, NC, pad, plen, off, counts, perm,
                                                             tile_info, ntiles, bad_flag,
                                                             device_error_word());
    k_perm_scatter<<<dim3(NC, sorts), PERM_CHUNK, 32 * E * sizeof(int), st>>>(assign, len, E, NC, chunk_scratch, perm,
                                                                            plen, inv, e_lo);
    QLMB_LAUNCH_CHECK("perm_build");
    return QLMB_OK;
}

size_t perm_scratch_ints(int N, int E, int K, int merged)
{
    int sorts = merged ? 1 : K, len = merged ? K * N : N;
    int NC = (len + PERM_CHUNK - 1) / PERM_CHUNK;
    return (size_t)sorts * E * NC;
}

int router_topk(const float *rt, float *rprobs, int *assign, float *gate, int N, int E, int K,
                const float *bias, int bs, cudaStream_t st)
{
    if (E <= 32) k_router_topk_warp<<<(N + 7) / 8, 256, 0, st>>>(rt, rprobs, assign, gate, N, E, K, bias, bs);
    else k_router_topk<<<(N + 127) / 128, 128, 0, st>>>(rt, rprobs, assign, gate, N, E, K, bias, bs);
    QLMB_LAUNCH_CHECK("k_router_topk");
    return QLMB_OK;
}

int router_small(float *rt, const void *X, int x_dtype, const float *Wr, float *rprobs, int *assign, float *gate, int N, int D,
                 int E, int K, const float *bias, int bs, cudaStream_t st)
{
    if (N > 64 || E > 32 || D > 8192) {
        int rc = router_logits_small(rt, X, x_dtype, Wr, N, D, E, st);
        return rc ? rc : router_topk(rt, rprobs, assign, gate, N, E, K, bias, bs, st);
    }
    k_router_small<<<N, 256, (size_t)D * sizeof(float), st>>>(rt, X, x_dtype, Wr, rprobs, assign, gate, N, D, E, K, bias, bs);
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

// lazily grown per-device scratch for the public perm entry point
static int *g_perm_scratch[64];
static size_t g_perm_cap[64];

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_perm_build(const int *assign, int N, int E, int K, int merged, int pad, int *perm,
                               int *inv, int *off, int *counts, int *bad_flag, void *stream)
{
    QLMB_REQUIRE(assign && perm && off && bad_flag, "qlmb_perm_build: NULL argument");
    QLMB_REQUIRE(N > 0 && E > 0 && E <= 256 && K > 0 && K <= 8 && pad >= 1, "qlmb_perm_build: N=%d E=%d K=%d pad=%d", N, E, K, pad);
    int dev = 0;
    QLMB_CUDA(cudaGetDevice(&dev));
    QLMB_REQUIRE(dev >= 0 && dev < 64, "qlmb_perm_build: device index %d", dev);
    size_t need = perm_scratch_ints(N, E, K, merged);
    if (g_perm_cap[dev] < need) {
        if (g_perm_scratch[dev]) QLMB_CUDA(cudaFree(g_perm_scratch[dev]));
        g_perm_scratch[dev] = nullptr; g_perm_cap[dev] = 0;
        QLMB_CUDA(cudaMalloc(&g_perm_scratch[dev], need * sizeof(int)));
        g_perm_cap[dev] = need;
    }
    return perm_build(assign, N, E, K, merged, pad, perm, inv, off, counts, bad_flag, nullptr, nullptr,
                      g_perm_scratch[dev], as_stream(stream));
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
