// Causal (optionally windowed) flash attention for sm_100a, head dimension 64, bf16 operands.
//
// Forward, one CTA per (sequence, head, tile of 128 queries), two CTAs per SM:
//
//   warp 0      TMA producer   Q tile once; K and V tiles of 128 keys through a two-stage ring
//   warp 1      MMA issuer     S = Q K^T (128 x 128 x 64) and PV = P V (128 x 64 x 128) with
//                              tcgen05.mma, fp32 results in TMEM (S: 128 columns, PV: 64 columns)
//   warps 2-9   softmax        two threads per query row (64 keys and 32 output dimensions each):
//                              tcgen05.ld of the S row, running max / sum in the exp2 domain, P as
//                              bf16 into shared memory in the 128-byte-swizzled K-major layout the
//                              PV MMA reads, and O = O * corr + PV in registers
//
// The MMA warp issues PV(t) and S(t+1) back to back as soon as P(t) is in shared memory, so the
// tensor core works on the next scores while the softmax warps fold PV(t) into O; the second CTA
// of the SM fills the rest.  Every mbarrier wait is bounded (qlmb_tc.cuh): a wait that runs out
// raises the CTA's abort flag, records its site in the device error word and all roles leave.
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>
#include "qlmb_common.cuh"
#include "qlmb_gemm.cuh"
#include "qlmb_tc.cuh"

namespace qlmb {

constexpr int AT_BM = 128;                    // queries per CTA
constexpr int AT_BN = 128;                    // keys per step
constexpr int AT_HD = 64;
constexpr int AT_TILE = AT_BM * AT_HD * 2;    // bytes of a Q, K or V tile
constexpr int AT_P_BYTES = AT_BM * AT_BN * 2;
constexpr int AT_FWD_SMEM = AT_TILE + 4 * AT_TILE + AT_P_BYTES + 768;   // + barriers (256 B) + one exchange word per query row

struct AttnFwdParams {
    alignas(64) CUtensorMap q_map, k_map, v_map;
    bf16 *O;
    float *lse;
    int B, T, H, KV, win, nqt;
    float scale_log2;                         // log2(e) / sqrt(hd)
    int *errword;
};

// Bounded wait of the attention kernels: a tile step takes microseconds, so a wait that has polled
// for about a second is broken; it raises the CTA's abort flag and records its site.  CTAs that
// start after an error was recorded leave at once (at_error_seen), so a broken pipeline ends the
// launch quickly instead of timing out CTA by CTA.
constexpr uint32_t AT_WAIT_LIMIT = 1u << 21;               // polls of the drain loops on the abort path
constexpr unsigned long long AT_WAIT_NS = 1000000000ull;    // one second of wall clock per wait
__device__ __forceinline__ unsigned long long at_now()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t at_test(uint32_t bar, uint32_t parity)     // non-blocking probe
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ bool at_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *errword, int site)
{
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = at_now();
    for (uint32_t i = 0;; i++) {
        if (at_test(bar, parity)) return true;
        if ((i & 1023u) == 1023u) {
            if (*abort_flag) return false;
            if (at_now() - t0 > AT_WAIT_NS) break;
        }
    }
    if (!*abort_flag) {
        *abort_flag = 1;
        if (errword && atomicCAS(errword, 0, 200) == 0) { errword[1] = site; errword[2] = (int)blockIdx.x; errword[3] = (int)parity; }
    }
    return false;
}
__device__ __forceinline__ bool at_error_seen(const int *errword) { return errword && *reinterpret_cast<const volatile int *>(errword) != 0; }

// 2^x on the special-function unit (ex2.approx: 2 ulp, flushes denormal results to zero, -inf -> 0)
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ bool attn_valid(int key, int i, int T, int win)
{
    return key <= i && key < T && (win <= 0 || key > i - win);
}

__global__ void __launch_bounds__(320, 2) k_attn_fwd(const __grid_constant__ AttnFwdParams p)
{
    extern __shared__ __align__(1024) uint8_t at_smem[];
    uint8_t *sQ = at_smem, *sK = sQ + AT_TILE, *sV = sK + 2 * AT_TILE, *sP = sV + 2 * AT_TILE;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sP + AT_P_BYTES);
    uint64_t *q_full = bars, *kv_full = bars + 1, *kv_empty = bars + 3, *s_full = bars + 5, *p_full = bars + 6,
             *o_full = bars + 7, *spare = bars + 8;
    uint64_t *pair_bar = bars + 10;           // one per TMEM lane quarter: the two warps that share a query row meet here
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 14);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *xrow = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(bars) + 256);   // 128 words: running row maximum, then row sum
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (smem_u32(at_smem) & 1023u) {          // the swizzled tiles need a 1 KiB-aligned base
        if (threadIdx.x == 0 && p.errword && atomicCAS(p.errword, 0, 201) == 0) { p.errword[1] = 100; p.errword[2] = (int)blockIdx.x; }
        return;
    }
    if (__syncthreads_or(threadIdx.x == 0 && at_error_seen(p.errword))) return;   // uniform over the CTA
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&kv_full[i]), 1); mbar_init(smem_u32(&kv_empty[i]), 1); }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(p_full), 8);
        for (int i = 0; i < 4; i++) mbar_init(smem_u32(&pair_bar[i]), 2);
        mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(spare), 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (threadIdx.x >= 64 && threadIdx.x < 192) xrow[threadIdx.x - 64] = (int)0x80000000;      // below every encoded maximum
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 256); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tPV = tmem_base + 128;

    // heaviest query tiles first
    const int BH = p.B * p.H;
    const int qt = p.nqt - 1 - (int)blockIdx.x / BH, bh = (int)blockIdx.x % BH;
    const int b = bh / p.H, h = bh % p.H, kvh = h / (p.H / p.KV);
    const int q0 = qt * AT_BM;
    int kt_lo = 0;
    if (p.win > 0) { int lo = q0 - p.win + 1; kt_lo = lo > 0 ? lo / AT_BN : 0; }
    const int kt_hi = (q0 + AT_BM - 1 < p.T ? q0 + AT_BM - 1 : p.T - 1) / AT_BN;     // inclusive
    const int nt = kt_hi - kt_lo + 1;

    if (warp == 0) {
        // =============================== TMA producer ===============================
        bool ok = true;
        int issued = 0;
        if (lane == 0) {
            mbar_expect_tx(smem_u32(q_full), AT_TILE);
            tma_load_2d(smem_u32(sQ), &p.q_map, smem_u32(q_full), h * AT_HD, b * p.T + q0);
        }
        for (int t = 0; ok && t < nt; t++) {
            const int st = t & 1;
            ok = at_wait(smem_u32(&kv_empty[st]), (((uint32_t)t >> 1) & 1u) ^ 1u, abort_flag, p.errword, 101);
            if (!ok) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&kv_full[st]);
                const int row = b * p.T + (kt_lo + t) * AT_BN;
                mbar_expect_tx(bar, 2 * AT_TILE);
                tma_load_2d(smem_u32(sK + st * AT_TILE), &p.k_map, bar, kvh * AT_HD, row);
                tma_load_2d(smem_u32(sV + st * AT_TILE), &p.v_map, bar, kvh * AT_HD, row);
            }
            __syncwarp();
            issued = t + 1;
        }
        if (*abort_flag) {
            // aborting: the copies this warp started must land before the CTA gives its shared memory back
            for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(q_full), 0); i++) {}
            for (int t = issued > 2 ? issued - 2 : 0; t < issued; t++)
                for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(&kv_full[t & 1]), ((uint32_t)t >> 1) & 1u); i++) {}
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        constexpr uint32_t IDESC_S = make_idesc(AT_BM, AT_BN, 0, 0);
        constexpr uint32_t IDESC_PV = make_idesc(AT_BM, AT_HD, 0, 1);
        auto issue_s = [&](int st) {
            const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK + st * AT_TILE);
#pragma unroll
            for (int k16 = 0; k16 < AT_HD / 16; k16++)
                tc_mma_bf16(tS, make_desc(a0 + k16 * 32, 16, 1024), make_desc(b0 + k16 * 32, 16, 1024), IDESC_S, k16 > 0);
            tc_commit(smem_u32(s_full));
        };
        bool ok = at_wait(smem_u32(q_full), 0, abort_flag, p.errword, 110);
        if (ok) ok = at_wait(smem_u32(&kv_full[0]), 0, abort_flag, p.errword, 111);
        if (ok) {
            tc_fence_after();
            if (lane == 0) issue_s(0);
            __syncwarp();
        }
        for (int t = 0; ok && t < nt; t++) {
            const int st = t & 1;
            ok = at_wait(smem_u32(p_full), (uint32_t)t & 1u, abort_flag, p.errword, 112);
            if (!ok) break;
            tc_fence_after();
            // the next scores first (the S columns are free once P is written): the softmax warps start on them while
            // this step's PV runs; they fold PV(t) after their first pass and only then overwrite P
            if (t + 1 < nt) {
                ok = at_wait(smem_u32(&kv_full[st ^ 1]), ((uint32_t)(t + 1) >> 1) & 1u, abort_flag, p.errword, 113);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) issue_s(st ^ 1);
                __syncwarp();
            }
            if (lane == 0) {
                const uint32_t a0 = smem_u32(sP), b0 = smem_u32(sV + st * AT_TILE);
#pragma unroll
                for (int kk = 0; kk < AT_BN / 16; kk++)
                    tc_mma_bf16(tPV, make_desc(a0 + (kk >> 2) * (AT_BM * 128) + (kk & 3) * 32, 16, 1024),
                                make_desc(b0 + kk * 2048, 8192, 1024), IDESC_PV, kk > 0);
                tc_commit(smem_u32(o_full));
                tc_commit(smem_u32(&kv_empty[st]));
            }
            __syncwarp();
        }
        if (*abort_flag) {                    // let issued MMAs retire (bounded) before TMEM is released
            if (lane == 0) tc_commit(smem_u32(spare));
            __syncwarp();
            for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(spare), 0); i++) {}
        }
    } else {
        // =============================== softmax + output ===============================
        // Two threads per query row: warps w and w + 4 share a TMEM lane quarter; thread (r, hf) takes keys
        // [64 hf, 64 hf + 64) of every step and output dimensions [32 hf, 32 hf + 32).  The row maximum is a running
        // atomicMax on one shared word per row (order-preserving integer image of the float): both threads add their
        // half's maximum, meet on the quarter's mbarrier and read the same value.  No reset is needed: the running
        // maximum only grows, and the next step's atomicMax cannot come before the partner has read this step's value,
        // because the next scores are only issued after both warps arrived on p_full.
        const int q = warp & 3, hf = (warp - 2) >> 2, r = q * 32 + lane, i = q0 + r;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        const uint32_t pb = smem_u32(&pair_bar[q]);
        uint32_t pphase = 0;
        float m = -1e30f, l = 0.0f, corr_pend = 1.0f;
        float o[32];
#pragma unroll
        for (int d = 0; d < 32; d++) o[d] = 0.0f;
        bool ok = true;
        auto pair_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(pb);
            const bool got = at_wait(pb, pphase, abort_flag, p.errword, 123);
            pphase ^= 1u;
            return got;
        };
        auto enc = [](float f) { const int b = __float_as_int(f); return b >= 0 ? b : b ^ 0x7fffffff; };
        auto dec = [](int b) { return __int_as_float(b >= 0 ? b : b ^ 0x7fffffff); };
        auto fold_pv = [&]() {                 // O = O * corr + PV for this thread's 32 output dimensions
            uint32_t v[32];
            tmem_ld32(tPV + lane_base + hf * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j++) o[j] = o[j] * corr_pend + __uint_as_float(v[j]);
        };
        for (int t = 0; ok && t < nt; t++) {
            const int k0 = (kt_lo + t) * AT_BN + hf * 64;               // first key of this thread's half
            const bool masked = (k0 + 63 > q0) || p.win > 0 || (k0 + 64 > p.T);
            ok = at_wait(smem_u32(s_full), (uint32_t)t & 1u, abort_flag, p.errword, 120);
            if (!ok) break;
            tc_fence_after();
            // pass 1: maximum of this half of the row
            float mx = -1e30f;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tmem_ld32(tS + lane_base + hf * 64 + c * 32, v);
                tmem_ld_wait();
                if (masked) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (attn_valid(k0 + c * 32 + j, i, p.T, p.win)) mx = fmaxf(mx, __uint_as_float(v[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(v[j]));
                }
            }
            atomicMax(&xrow[r], enc(fmaxf(mx * p.scale_log2, -1e30f)));
            ok = pair_sync();
            if (!ok) break;
            const float m_new = dec(*reinterpret_cast<volatile int *>(&xrow[r]));
            const float corr = ex2(m - m_new);
            // the previous step's PV: its MMA was issued before this step's S, so it has completed
            if (t > 0) {
                ok = at_wait(smem_u32(o_full), (uint32_t)(t - 1) & 1u, abort_flag, p.errword, 121);
                if (!ok) break;
                tc_fence_after();
                fold_pv();
            }
            corr_pend = corr;
            // pass 2: P = exp2(s - m) as bf16 into this half's swizzled K-major sub-tile, partial row sum
            float rs = 0.0f;
            uint8_t *rowp = sP + hf * (AT_BM * 128) + r * 128;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tmem_ld32(tS + lane_base + hf * 64 + c * 32, v);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float p0 = ex2(__uint_as_float(v[j]) * p.scale_log2 - m_new);
                    float p1 = ex2(__uint_as_float(v[j + 1]) * p.scale_log2 - m_new);
                    if (masked) {
                        if (!attn_valid(k0 + c * 32 + j, i, p.T, p.win)) p0 = 0.0f;
                        if (!attn_valid(k0 + c * 32 + j + 1, i, p.T, p.win)) p1 = 0.0f;
                    }
                    rs += p0 + p1;
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                    pk[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int unit = (c * 4 + u) ^ (r & 7);
                    *reinterpret_cast<uint4 *>(rowp + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
                }
            }
            l = l * corr + rs;
            m = m_new;
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(p_full));
        }
        if (ok) ok = at_wait(smem_u32(o_full), (uint32_t)(nt - 1) & 1u, abort_flag, p.errword, 122);
        if (ok) {
            tc_fence_after();
            fold_pv();
            // the row sum: the upper half hands its partial sum over, the lower half returns the total
            float *xl = reinterpret_cast<float *>(xrow);
            if (hf == 1) xl[r] = l;
            ok = pair_sync();
            if (ok) {
                if (hf == 0) { l += *reinterpret_cast<volatile float *>(&xl[r]); xl[r] = l; }
                ok = pair_sync();
            }
            if (ok) {
                if (hf == 1) l = *reinterpret_cast<volatile float *>(&xl[r]);
                if (i < p.T) {
                    const float inv = 1.0f / l;
                    bf16 *orow = p.O + ((size_t)b * p.T + i) * ((size_t)p.H * AT_HD) + (size_t)h * AT_HD + hf * 32;
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[u * 8 + 2 * k] * inv, o[u * 8 + 2 * k + 1] * inv);
                            w[k] = *reinterpret_cast<uint32_t *>(&h2);
                        }
                        *reinterpret_cast<uint4 *>(orow + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    if (hf == 0) p.lse[((size_t)b * p.H + h) * p.T + i] = (m + log2f(l)) * 0.6931471805599453f;
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}


// ------------------------------------------------------------------ backward
// Two kernels, so that every output element has one writer and a fixed summation order:
//   k_attn_bwd_dkv  one CTA per (sequence, K/V head, tile of 128 keys), walks the heads of the
//                   group and the query tiles that see these keys; dK and dV accumulate in TMEM.
//   k_attn_bwd_dq   one CTA per (sequence, head, tile of 128 queries), walks the key tiles;
//                   dQ accumulates in TMEM.
// Both recompute the scores from Q, K and the saved log-sum-exp:  P = exp(S/sqrt(hd) - lse),
// dS = P * (dP - D) / sqrt(hd) with dP = dA V^T and D = rowsum(dA * O) (k_attn_drow).
//
//   warp 0      TMA producer   resident tiles once, the walked tiles through a two-stage ring
//   warp 1      MMA issuer     scores and dP (two 128 x 128 x 64 MMAs into TMEM), then the two
//                              accumulating products from P / dS in shared memory
//   warps 2-17  element-wise   thread = one TMEM lane (a key for dkv, a query for dq) x 32 of the
//                              128 columns: P and dS as bf16 into swizzled K-major tiles
constexpr int AT_BWD_THREADS = 576;             // TMA warp, MMA warp, 16 element-wise warps
constexpr int AT_DKV_SMEM = 2 * AT_TILE + 4 * AT_TILE + 2 * AT_P_BYTES + 2 * 2 * 128 * 4 + 256;
constexpr int AT_DQ_SMEM = 2 * AT_TILE + 4 * AT_TILE + AT_P_BYTES + 256;

struct AttnBwdParams {
    alignas(64) CUtensorMap q_map, k_map, v_map, da_map;
    const float *lse, *drow;
    bf16 *dQ, *dK, *dV;
    int B, T, H, KV, win, nqt;
    float scale, scale_log2;
    int *errword;
};

__global__ void __launch_bounds__(256) k_attn_drow(float *drow, const bf16 *dA, const bf16 *O, int B, int T, int H)
{
    const size_t g = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (g >= (size_t)B * T * H) return;
    const int h = (int)(g % H);
    const size_t bt = g / H;
    const uint4 *a = reinterpret_cast<const uint4 *>(dA + bt * (size_t)H * AT_HD + (size_t)h * AT_HD);
    const uint4 *o = reinterpret_cast<const uint4 *>(O + bt * (size_t)H * AT_HD + (size_t)h * AT_HD);
    float acc = 0.0f;
#pragma unroll
    for (int u = 0; u < 8; u++) {
        const uint4 x = __ldg(a + u), y = __ldg(o + u);
        const __nv_bfloat162 *xh = reinterpret_cast<const __nv_bfloat162 *>(&x), *yh = reinterpret_cast<const __nv_bfloat162 *>(&y);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 xf = __bfloat1622float2(xh[k]), yf = __bfloat1622float2(yh[k]);
            acc += xf.x * yf.x + xf.y * yf.y;
        }
    }
    const int b = (int)(bt / T), t = (int)(bt % T);
    drow[((size_t)b * H + h) * T + t] = acc;
}

// 32 fp32 TMEM columns of this thread's lane -> 64 bytes of bf16 in global memory (the load runs in every lane)
__device__ __forceinline__ void attn_store_row32(bf16 *dst, uint32_t taddr, bool live)
{
    uint32_t v[32];
    tmem_ld32(taddr, v);
    tmem_ld_wait();
#pragma unroll
    for (int u = 0; u < 4; u++) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2 * k]), __uint_as_float(v[u * 8 + 2 * k + 1]));
            w[k] = *reinterpret_cast<uint32_t *>(&h2);
        }
        if (live) *reinterpret_cast<uint4 *>(dst + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}
// 64 fp32 TMEM columns of this thread's lane -> one 128-byte row of bf16 in global memory
// (tcgen05.ld is warp-collective: every lane runs it, only live lanes store)
__device__ __forceinline__ void attn_store_row64(bf16 *dst, uint32_t taddr, bool live)
{
#pragma unroll
    for (int c = 0; c < 2; c++) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 4; u++) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2 * k]), __uint_as_float(v[u * 8 + 2 * k + 1]));
                w[k] = *reinterpret_cast<uint32_t *>(&h2);
            }
            if (live) *reinterpret_cast<uint4 *>(dst + c * 32 + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

__global__ void __launch_bounds__(AT_BWD_THREADS, 1) k_attn_bwd_dkv(const __grid_constant__ AttnBwdParams p)
{
    extern __shared__ __align__(1024) uint8_t at_smem[];
    uint8_t *sK = at_smem, *sV = sK + AT_TILE, *sQ = sV + AT_TILE, *sA = sQ + 2 * AT_TILE;
    uint8_t *sPt = sA + 2 * AT_TILE, *sSt = sPt + AT_P_BYTES;
    float *sL = reinterpret_cast<float *>(sSt + AT_P_BYTES), *sD = sL + 2 * 128;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sD + 2 * 128);
    uint64_t *kv_full = bars, *qd_full = bars + 1, *qd_empty = bars + 3, *s_full = bars + 5, *pds_full = bars + 6,
             *acc_done = bars + 7, *spare = bars + 8;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 10);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (smem_u32(at_smem) & 1023u) {
        if (threadIdx.x == 0 && p.errword && atomicCAS(p.errword, 0, 201) == 0) { p.errword[1] = 200; p.errword[2] = (int)blockIdx.x; }
        return;
    }
    if (__syncthreads_or(threadIdx.x == 0 && at_error_seen(p.errword))) return;   // uniform over the CTA
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(kv_full), 1);
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&qd_full[i]), 2); mbar_init(smem_u32(&qd_empty[i]), 1); }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(pds_full), 16);
        mbar_init(smem_u32(acc_done), 1);
        mbar_init(smem_u32(spare), 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 320;

    // key tiles that see the most queries first
    const int BK_ = p.B * p.KV, grp = p.H / p.KV;
    const int kt = (int)blockIdx.x / BK_, bk = (int)blockIdx.x % BK_;
    const int b = bk / p.KV, kvh = bk % p.KV;
    const int k0 = kt * AT_BN;
    int qt_hi = p.nqt - 1;
    if (p.win > 0) { int hi = (k0 + AT_BN - 1 + p.win - 1) / AT_BM; if (hi < qt_hi) qt_hi = hi; }
    const int nq = qt_hi - kt + 1, nit = nq * grp;        // iteration it: head kvh*grp + it / nq, query tile kt + it % nq

    if (warp == 0) {
        // =============================== producer ===============================
        bool ok = true;
        int issued = 0;
        if (lane == 0) {
            mbar_expect_tx(smem_u32(kv_full), 2 * AT_TILE);
            tma_load_2d(smem_u32(sK), &p.k_map, smem_u32(kv_full), kvh * AT_HD, b * p.T + k0);
            tma_load_2d(smem_u32(sV), &p.v_map, smem_u32(kv_full), kvh * AT_HD, b * p.T + k0);
        }
        for (int it = 0; ok && it < nit; it++) {
            const int st = it & 1, h = kvh * grp + it / nq, q0 = (kt + it % nq) * AT_BM;
            ok = at_wait(smem_u32(&qd_empty[st]), (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag, p.errword, 201);
            if (!ok) break;
            const uint32_t bar = smem_u32(&qd_full[st]);
            if (lane == 0) {
                mbar_expect_tx(bar, 2 * AT_TILE);
                tma_load_2d(smem_u32(sQ + st * AT_TILE), &p.q_map, bar, h * AT_HD, b * p.T + q0);
                tma_load_2d(smem_u32(sA + st * AT_TILE), &p.da_map, bar, h * AT_HD, b * p.T + q0);
            }
            // log-sum-exp (log2 domain) and D of the 128 queries; queries past the sequence get +huge, so P = 0
            const size_t rowb = ((size_t)b * p.H + h) * p.T;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int c = lane + 32 * k, qi = q0 + c;
                sL[st * 128 + c] = qi < p.T ? p.lse[rowb + qi] * 1.4426950408889634f : 1e30f;
                sD[st * 128 + c] = qi < p.T ? p.drow[rowb + qi] : 0.0f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
            issued = it + 1;
        }
        if (*abort_flag) {
            for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(kv_full), 0); i++) {}
            for (int it = issued > 2 ? issued - 2 : 0; it < issued; it++)
                for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(&qd_full[it & 1]), ((uint32_t)it >> 1) & 1u); i++) {}
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        constexpr uint32_t IDESC_S = make_idesc(AT_BN, AT_BM, 0, 0);
        constexpr uint32_t IDESC_ACC = make_idesc(AT_BN, AT_HD, 0, 1);
        auto issue_scores = [&](int st) {      // S^T = K Q^T, dP^T = V dA^T
            const uint32_t k_ = smem_u32(sK), v_ = smem_u32(sV), q_ = smem_u32(sQ + st * AT_TILE), a_ = smem_u32(sA + st * AT_TILE);
#pragma unroll
            for (int k16 = 0; k16 < AT_HD / 16; k16++)
                tc_mma_bf16(tS, make_desc(k_ + k16 * 32, 16, 1024), make_desc(q_ + k16 * 32, 16, 1024), IDESC_S, k16 > 0);
#pragma unroll
            for (int k16 = 0; k16 < AT_HD / 16; k16++)
                tc_mma_bf16(tP, make_desc(v_ + k16 * 32, 16, 1024), make_desc(a_ + k16 * 32, 16, 1024), IDESC_S, k16 > 0);
            tc_commit(smem_u32(s_full));
        };
        bool ok = at_wait(smem_u32(kv_full), 0, abort_flag, p.errword, 210);
        if (ok) ok = at_wait(smem_u32(&qd_full[0]), 0, abort_flag, p.errword, 211);
        if (ok) {
            tc_fence_after();
            if (lane == 0) issue_scores(0);
            __syncwarp();
        }
        for (int it = 0; ok && it < nit; it++) {
            const int st = it & 1;
            ok = at_wait(smem_u32(pds_full), (uint32_t)it & 1u, abort_flag, p.errword, 212);
            if (!ok) break;
            tc_fence_after();
            // the next step's scores first (their TMEM columns are free once P / dS are written), so that the
            // element-wise warps work on them while the two accumulating products of this step run
            if (it + 1 < nit) {
                ok = at_wait(smem_u32(&qd_full[st ^ 1]), ((uint32_t)(it + 1) >> 1) & 1u, abort_flag, p.errword, 213);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) issue_scores(st ^ 1);
                __syncwarp();
            }
            if (lane == 0) {
                const uint32_t pt = smem_u32(sPt), dst = smem_u32(sSt), q_ = smem_u32(sQ + st * AT_TILE), a_ = smem_u32(sA + st * AT_TILE);
#pragma unroll
                for (int kk = 0; kk < AT_BM / 16; kk++)       // dV += P^T dA
                    tc_mma_bf16(tdV, make_desc(pt + (kk >> 2) * (AT_BN * 128) + (kk & 3) * 32, 16, 1024),
                                make_desc(a_ + kk * 2048, 8192, 1024), IDESC_ACC, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < AT_BM / 16; kk++)       // dK += dS^T Q
                    tc_mma_bf16(tdK, make_desc(dst + (kk >> 2) * (AT_BN * 128) + (kk & 3) * 32, 16, 1024),
                                make_desc(q_ + kk * 2048, 8192, 1024), IDESC_ACC, (it > 0 || kk > 0) ? 1u : 0u);
                tc_commit(smem_u32(acc_done));
                tc_commit(smem_u32(&qd_empty[st]));
            }
            __syncwarp();
        }
        if (*abort_flag) {
            if (lane == 0) tc_commit(smem_u32(spare));
            __syncwarp();
            for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(spare), 0); i++) {}
        }
    } else {
        // =============================== element-wise ===============================
        // warp = (TMEM lane quarter qr, 32-column chunk cq of the 128): hf = which 64-column sub-tile, c = chunk in it
        const int qr = warp & 3, cq = (warp - 2) >> 2, hf = cq >> 1, c = cq & 1, r = qr * 32 + lane, key = k0 + r;
        const uint32_t lane_base = (uint32_t)(qr * 32) << 16;
        bool ok = true;
        for (int it = 0; ok && it < nit; it++) {
            const int st = it & 1, q0 = (kt + it % nq) * AT_BM;
            const bool masked = (q0 < k0 + AT_BN - 1) || p.win > 0;
            ok = at_wait(smem_u32(&qd_full[st]), ((uint32_t)it >> 1) & 1u, abort_flag, p.errword, 220);      // lse / D in shared memory
            if (ok) ok = at_wait(smem_u32(s_full), (uint32_t)it & 1u, abort_flag, p.errword, 221);
            if (!ok) break;
            tc_fence_after();
            const float *L2 = sL + st * 128 + hf * 64, *Dq = sD + st * 128 + hf * 64;
            uint32_t sv[32], dv[32];                 // both TMEM loads of the step in flight: one round trip
            tmem_ld32(tS + lane_base + cq * 32, sv);
            tmem_ld32(tP + lane_base + cq * 32, dv);
            tmem_ld_wait();
            {
                uint32_t pp[16], ds[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float pv[2], dsv[2];
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int col = c * 32 + j + e, qi = q0 + hf * 64 + col;
                        float pe = ex2(__uint_as_float(sv[j + e]) * p.scale_log2 - L2[col]);
                        if (masked && !(key <= qi && (p.win <= 0 || key > qi - p.win))) pe = 0.0f;
                        pv[e] = pe;
                        dsv[e] = pe * (__uint_as_float(dv[j + e]) - Dq[col]) * p.scale;
                    }
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(pv[0], pv[1]);
                    pp[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                    h2 = __floats2bfloat162_rn(dsv[0], dsv[1]);
                    ds[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                }
                // the previous step's products must have read the P / dS tiles before they are overwritten
                if (it > 0) ok = at_wait(smem_u32(acc_done), (uint32_t)(it - 1) & 1u, abort_flag, p.errword, 222);
                uint8_t *prow = sPt + hf * (AT_BN * 128) + r * 128, *srow = sSt + hf * (AT_BN * 128) + r * 128;
                if (ok) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int unit = (c * 4 + u) ^ (r & 7);
                        *reinterpret_cast<uint4 *>(prow + unit * 16) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
                        *reinterpret_cast<uint4 *>(srow + unit * 16) = make_uint4(ds[4 * u], ds[4 * u + 1], ds[4 * u + 2], ds[4 * u + 3]);
                    }
                }
            }
            if (!ok) break;
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(pds_full));
        }
        if (ok) ok = at_wait(smem_u32(acc_done), (uint32_t)(nit - 1) & 1u, abort_flag, p.errword, 223);
        if (ok) {
            tc_fence_after();
            // chunks 0, 1: the two halves of the dV row; chunks 2, 3: of the dK row
            bf16 *dst = (hf ? p.dK : p.dV) + ((size_t)b * p.T + key) * ((size_t)p.KV * AT_HD) + (size_t)kvh * AT_HD + c * 32;
            attn_store_row32(dst, (hf ? tdK : tdV) + lane_base + c * 32, key < p.T);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

__global__ void __launch_bounds__(AT_BWD_THREADS, 1) k_attn_bwd_dq(const __grid_constant__ AttnBwdParams p)
{
    extern __shared__ __align__(1024) uint8_t at_smem[];
    uint8_t *sQ = at_smem, *sA = sQ + AT_TILE, *sK = sA + AT_TILE, *sV = sK + 2 * AT_TILE, *sS = sV + 2 * AT_TILE;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sS + AT_P_BYTES);
    uint64_t *qa_full = bars, *kv_full = bars + 1, *kv_empty = bars + 3, *s_full = bars + 5, *ds_full = bars + 6,
             *acc_done = bars + 7, *spare = bars + 8;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 10);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (smem_u32(at_smem) & 1023u) {
        if (threadIdx.x == 0 && p.errword && atomicCAS(p.errword, 0, 201) == 0) { p.errword[1] = 300; p.errword[2] = (int)blockIdx.x; }
        return;
    }
    if (__syncthreads_or(threadIdx.x == 0 && at_error_seen(p.errword))) return;   // uniform over the CTA
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(qa_full), 1);
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&kv_full[i]), 1); mbar_init(smem_u32(&kv_empty[i]), 1); }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(ds_full), 16);
        mbar_init(smem_u32(acc_done), 1);
        mbar_init(smem_u32(spare), 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tP = tmem_base + 128, tdQ = tmem_base + 256;

    const int BH = p.B * p.H;
    const int qt = p.nqt - 1 - (int)blockIdx.x / BH, bh = (int)blockIdx.x % BH;
    const int b = bh / p.H, h = bh % p.H, kvh = h / (p.H / p.KV);
    const int q0 = qt * AT_BM;
    int kt_lo = 0;
    if (p.win > 0) { int lo = q0 - p.win + 1; kt_lo = lo > 0 ? lo / AT_BN : 0; }
    const int kt_hi = (q0 + AT_BM - 1 < p.T ? q0 + AT_BM - 1 : p.T - 1) / AT_BN;
    const int nt = kt_hi - kt_lo + 1;

    if (warp == 0) {
        bool ok = true;
        int issued = 0;
        if (lane == 0) {
            mbar_expect_tx(smem_u32(qa_full), 2 * AT_TILE);
            tma_load_2d(smem_u32(sQ), &p.q_map, smem_u32(qa_full), h * AT_HD, b * p.T + q0);
            tma_load_2d(smem_u32(sA), &p.da_map, smem_u32(qa_full), h * AT_HD, b * p.T + q0);
        }
        for (int t = 0; ok && t < nt; t++) {
            const int st = t & 1;
            ok = at_wait(smem_u32(&kv_empty[st]), (((uint32_t)t >> 1) & 1u) ^ 1u, abort_flag, p.errword, 301);
            if (!ok) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&kv_full[st]);
                const int row = b * p.T + (kt_lo + t) * AT_BN;
                mbar_expect_tx(bar, 2 * AT_TILE);
                tma_load_2d(smem_u32(sK + st * AT_TILE), &p.k_map, bar, kvh * AT_HD, row);
                tma_load_2d(smem_u32(sV + st * AT_TILE), &p.v_map, bar, kvh * AT_HD, row);
            }
            __syncwarp();
            issued = t + 1;
        }
        if (*abort_flag) {
            for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(qa_full), 0); i++) {}
            for (int t = issued > 2 ? issued - 2 : 0; t < issued; t++)
                for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(&kv_full[t & 1]), ((uint32_t)t >> 1) & 1u); i++) {}
        }
    } else if (warp == 1) {
        constexpr uint32_t IDESC_S = make_idesc(AT_BM, AT_BN, 0, 0);
        constexpr uint32_t IDESC_ACC = make_idesc(AT_BM, AT_HD, 0, 1);
        auto issue_scores = [&](int st) {      // S = Q K^T, dP = dA V^T
            const uint32_t q_ = smem_u32(sQ), a_ = smem_u32(sA), k_ = smem_u32(sK + st * AT_TILE), v_ = smem_u32(sV + st * AT_TILE);
#pragma unroll
            for (int k16 = 0; k16 < AT_HD / 16; k16++)
                tc_mma_bf16(tS, make_desc(q_ + k16 * 32, 16, 1024), make_desc(k_ + k16 * 32, 16, 1024), IDESC_S, k16 > 0);
#pragma unroll
            for (int k16 = 0; k16 < AT_HD / 16; k16++)
                tc_mma_bf16(tP, make_desc(a_ + k16 * 32, 16, 1024), make_desc(v_ + k16 * 32, 16, 1024), IDESC_S, k16 > 0);
            tc_commit(smem_u32(s_full));
        };
        bool ok = at_wait(smem_u32(qa_full), 0, abort_flag, p.errword, 310);
        if (ok) ok = at_wait(smem_u32(&kv_full[0]), 0, abort_flag, p.errword, 311);
        if (ok) {
            tc_fence_after();
            if (lane == 0) issue_scores(0);
            __syncwarp();
        }
        for (int t = 0; ok && t < nt; t++) {
            const int st = t & 1;
            ok = at_wait(smem_u32(ds_full), (uint32_t)t & 1u, abort_flag, p.errword, 312);
            if (!ok) break;
            tc_fence_after();
            if (t + 1 < nt) {                                 // next scores first, see k_attn_bwd_dkv
                ok = at_wait(smem_u32(&kv_full[st ^ 1]), ((uint32_t)(t + 1) >> 1) & 1u, abort_flag, p.errword, 313);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) issue_scores(st ^ 1);
                __syncwarp();
            }
            if (lane == 0) {
                const uint32_t s_ = smem_u32(sS), k_ = smem_u32(sK + st * AT_TILE);
#pragma unroll
                for (int kk = 0; kk < AT_BN / 16; kk++)       // dQ += dS K
                    tc_mma_bf16(tdQ, make_desc(s_ + (kk >> 2) * (AT_BM * 128) + (kk & 3) * 32, 16, 1024),
                                make_desc(k_ + kk * 2048, 8192, 1024), IDESC_ACC, (t > 0 || kk > 0) ? 1u : 0u);
                tc_commit(smem_u32(acc_done));
                tc_commit(smem_u32(&kv_empty[st]));
            }
            __syncwarp();
        }
        if (*abort_flag) {
            if (lane == 0) tc_commit(smem_u32(spare));
            __syncwarp();
            for (uint32_t i = 0; i < AT_WAIT_LIMIT && !mbar_try(smem_u32(spare), 0); i++) {}
        }
    } else {
        const int qr = warp & 3, cq = (warp - 2) >> 2, hf = cq >> 1, c = cq & 1, r = qr * 32 + lane, i = q0 + r;
        const uint32_t lane_base = (uint32_t)(qr * 32) << 16;
        const size_t rowb = ((size_t)b * p.H + h) * p.T;
        const float L2 = i < p.T ? p.lse[rowb + i] * 1.4426950408889634f : 1e30f;
        const float Dq = i < p.T ? p.drow[rowb + i] : 0.0f;
        bool ok = true;
        for (int t = 0; ok && t < nt; t++) {
            const int k0 = (kt_lo + t) * AT_BN;
            const bool masked = (k0 + AT_BN - 1 > q0) || p.win > 0 || (k0 + AT_BN > p.T);
            ok = at_wait(smem_u32(s_full), (uint32_t)t & 1u, abort_flag, p.errword, 321);
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[32], dv[32];                 // both TMEM loads of the step in flight: one round trip
            tmem_ld32(tS + lane_base + cq * 32, sv);
            tmem_ld32(tP + lane_base + cq * 32, dv);
            tmem_ld_wait();
            {
                uint32_t ds[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float dsv[2];
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int key = k0 + hf * 64 + c * 32 + j + e;
                        float pe = ex2(__uint_as_float(sv[j + e]) * p.scale_log2 - L2);
                        if (masked && !attn_valid(key, i, p.T, p.win)) pe = 0.0f;
                        dsv[e] = pe * (__uint_as_float(dv[j + e]) - Dq) * p.scale;
                    }
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(dsv[0], dsv[1]);
                    ds[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                }
                if (t > 0) ok = at_wait(smem_u32(acc_done), (uint32_t)(t - 1) & 1u, abort_flag, p.errword, 322);   // dS tile free again
                uint8_t *srow = sS + hf * (AT_BM * 128) + r * 128;
                if (ok) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int unit = (c * 4 + u) ^ (r & 7);
                        *reinterpret_cast<uint4 *>(srow + unit * 16) = make_uint4(ds[4 * u], ds[4 * u + 1], ds[4 * u + 2], ds[4 * u + 3]);
                    }
                }
            }
            if (!ok) break;
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(ds_full));
        }
        if (ok) ok = at_wait(smem_u32(acc_done), (uint32_t)(nt - 1) & 1u, abort_flag, p.errword, 323);
        if (ok) {
            tc_fence_after();
            {                                  // each of the row's four threads stores 16 of its 64 columns
                bf16 *dst = p.dQ + ((size_t)b * p.T + i) * ((size_t)p.H * AT_HD) + (size_t)h * AT_HD + cq * 16;
                uint32_t v[16];
                tmem_ld16(tdQ + lane_base + cq * 16, v);          // warp-collective: all lanes, also those past the sequence
                tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    uint32_t w[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2 * k]), __uint_as_float(v[u * 8 + 2 * k + 1]));
                        w[k] = *reinterpret_cast<uint32_t *>(&h2);
                    }
                    if (i < p.T) *reinterpret_cast<uint4 *>(dst + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_attn_fwd(void *O, float *lse, const void *Q, const void *K, const void *V, int B, int T, int H,
                             int KV, int hd, int win, void *stream)
{
    QLMB_REQUIRE(O && lse && Q && K && V, "qlmb_attn_fwd: NULL argument");
    QLMB_REQUIRE(hd == AT_HD, "qlmb_attn_fwd: head dimension %d (only 64 is built)", hd);
    QLMB_REQUIRE(B > 0 && T > 0 && H > 0 && KV > 0 && H % KV == 0, "qlmb_attn_fwd: bad shape B %d T %d H %d KV %d", B, T, H, KV);
    AttnFwdParams p;
    memset(&p, 0, sizeof p);
    const unsigned long long rows = (unsigned long long)B * T;
    int rc = make_map(&p.q_map, Q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (unsigned long long)H * hd, rows, (unsigned long long)H * hd * 2, AT_HD, AT_BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_map(&p.k_map, K, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (unsigned long long)KV * hd, rows, (unsigned long long)KV * hd * 2, AT_HD, AT_BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_map(&p.v_map, V, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (unsigned long long)KV * hd, rows, (unsigned long long)KV * hd * 2, AT_HD, AT_BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    p.O = (bf16 *)O; p.lse = lse;
    p.B = B; p.T = T; p.H = H; p.KV = KV; p.win = win;
    p.nqt = (T + AT_BM - 1) / AT_BM;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
    p.errword = device_error_word();
    // the attribute belongs to a device's copy of the kernel: set it once per device of this process
    static bool configured_dev[64];
    int dev_ = 0;
    QLMB_CUDA(cudaGetDevice(&dev_));
    QLMB_REQUIRE(dev_ >= 0 && dev_ < 64, "device index %d", dev_);
    if (!configured_dev[dev_]) {
        QLMB_CUDA(cudaFuncSetAttribute(k_attn_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_FWD_SMEM));
        configured_dev[dev_] = true;
    }
    k_attn_fwd<<<(unsigned)(p.nqt * B * H), 320, AT_FWD_SMEM, as_stream(stream)>>>(p);
    QLMB_LAUNCH_CHECK("k_attn_fwd");
    return QLMB_OK;
}

extern "C" int qlmb_attn_bwd(void *dQ, void *dK, void *dV, float *drow, const void *Q, const void *K, const void *V,
                             const void *O, const void *dA, const float *lse, int B, int T, int H, int KV, int hd,
                             int win, void *stream)
{
    QLMB_REQUIRE(dQ && dK && dV && drow && Q && K && V && O && dA && lse, "qlmb_attn_bwd: NULL argument");
    QLMB_REQUIRE(hd == AT_HD, "qlmb_attn_bwd: head dimension %d (only 64 is built)", hd);
    QLMB_REQUIRE(B > 0 && T > 0 && H > 0 && KV > 0 && H % KV == 0, "qlmb_attn_bwd: bad shape B %d T %d H %d KV %d", B, T, H, KV);
    AttnBwdParams p;
    memset(&p, 0, sizeof p);
    const unsigned long long rows = (unsigned long long)B * T, qw = (unsigned long long)H * hd, kw = (unsigned long long)KV * hd;
    int rc = make_map(&p.q_map, Q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, qw, rows, qw * 2, AT_HD, AT_BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_map(&p.da_map, dA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, qw, rows, qw * 2, AT_HD, AT_BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_map(&p.k_map, K, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kw, rows, kw * 2, AT_HD, AT_BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_map(&p.v_map, V, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kw, rows, kw * 2, AT_HD, AT_BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    p.lse = lse; p.drow = drow;
    p.dQ = (bf16 *)dQ; p.dK = (bf16 *)dK; p.dV = (bf16 *)dV;
    p.B = B; p.T = T; p.H = H; p.KV = KV; p.win = win;
    p.nqt = (T + AT_BM - 1) / AT_BM;
    p.scale = 1.0f / sqrtf((float)hd);
    p.scale_log2 = 1.4426950408889634f * p.scale;
    p.errword = device_error_word();
    // the attribute belongs to a device's copy of the kernel: set it once per device of this process
    static bool configured_dev[64];
    int dev_ = 0;
    QLMB_CUDA(cudaGetDevice(&dev_));
    QLMB_REQUIRE(dev_ >= 0 && dev_ < 64, "device index %d", dev_);
    if (!configured_dev[dev_]) {
        QLMB_CUDA(cudaFuncSetAttribute(k_attn_bwd_dkv, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_DKV_SMEM));
        QLMB_CUDA(cudaFuncSetAttribute(k_attn_bwd_dq, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_DQ_SMEM));
        configured_dev[dev_] = true;
    }
    cudaStream_t st = as_stream(stream);
    const size_t nrow = (size_t)B * T * H;
    k_attn_drow<<<(unsigned)((nrow + 255) / 256), 256, 0, st>>>(drow, (const bf16 *)dA, (const bf16 *)O, B, T, H);
    k_attn_bwd_dkv<<<(unsigned)(p.nqt * B * KV), AT_BWD_THREADS, AT_DKV_SMEM, st>>>(p);
    k_attn_bwd_dq<<<(unsigned)(p.nqt * B * H), AT_BWD_THREADS, AT_DQ_SMEM, st>>>(p);
    QLMB_LAUNCH_CHECK("k_attn_bwd");
    return QLMB_OK;
}
