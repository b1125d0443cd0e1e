// Causal (optionally windowed) flash attention for sm_100a, head dimension 64, bf16 operands.
//
// Forward, one CTA per (sequence, head, tile of 128 queries), two CTAs per SM:
//
//   warp 0      TMA producer   Q tile once; K and V tiles of 128 keys through a two-stage ring
//   warp 1      MMA issuer     S = Q K^T (128 x 128 x 64) and PV = P V (128 x 64 x 128) with
//                              tcgen05.mma, fp32 results in TMEM (S: 128 columns, PV: 64 columns)
//   warps 2-5   softmax        a thread owns one query row: tcgen05.ld of its S row, running
//                              max / sum in the exp2 domain, P as bf16 into shared memory in the
//                              128-byte-swizzled K-major layout the PV MMA reads, and
//                              O = O * corr + PV in registers
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
constexpr int AT_FWD_SMEM = AT_TILE + 4 * AT_TILE + AT_P_BYTES + 256;

struct AttnFwdParams {
    alignas(64) CUtensorMap q_map, k_map, v_map;
    bf16 *O;
    float *lse;
    int B, T, H, KV, win, nqt;
    float scale_log2;                         // log2(e) / sqrt(hd)
    int *errword;
};

__device__ __forceinline__ bool attn_valid(int key, int i, int T, int win)
{
    return key <= i && key < T && (win <= 0 || key > i - win);
}

__global__ void __launch_bounds__(192, 2) k_attn_fwd(const __grid_constant__ AttnFwdParams p)
{
    extern __shared__ __align__(1024) uint8_t at_smem[];
    uint8_t *sQ = at_smem, *sK = sQ + AT_TILE, *sV = sK + 2 * AT_TILE, *sP = sV + 2 * AT_TILE;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sP + AT_P_BYTES);
    uint64_t *q_full = bars, *kv_full = bars + 1, *kv_empty = bars + 3, *s_full = bars + 5, *p_full = bars + 6,
             *o_full = bars + 7, *spare = bars + 8;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 10);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (smem_u32(at_smem) & 1023u) {          // the swizzled tiles need a 1 KiB-aligned base
        if (threadIdx.x == 0 && p.errword && atomicCAS(p.errword, 0, 201) == 0) { p.errword[1] = 100; p.errword[2] = (int)blockIdx.x; }
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&kv_full[i]), 1); mbar_init(smem_u32(&kv_empty[i]), 1); }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(p_full), 4);
        mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(spare), 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
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
            ok = mbar_wait_idle(smem_u32(&kv_empty[st]), (((uint32_t)t >> 1) & 1u) ^ 1u, abort_flag, p.errword, 101);
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
            for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(smem_u32(q_full), 0); i++) {}
            for (int t = issued > 2 ? issued - 2 : 0; t < issued; t++)
                for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(smem_u32(&kv_full[t & 1]), ((uint32_t)t >> 1) & 1u); i++) {}
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
        bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.errword, 110);
        if (ok) ok = mbar_wait(smem_u32(&kv_full[0]), 0, abort_flag, p.errword, 111);
        if (ok) {
            tc_fence_after();
            if (lane == 0) issue_s(0);
            __syncwarp();
        }
        for (int t = 0; ok && t < nt; t++) {
            const int st = t & 1;
            ok = mbar_wait(smem_u32(p_full), (uint32_t)t & 1u, abort_flag, p.errword, 112);
            if (!ok) break;
            tc_fence_after();
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
            if (t + 1 < nt) {
                ok = mbar_wait(smem_u32(&kv_full[st ^ 1]), ((uint32_t)(t + 1) >> 1) & 1u, abort_flag, p.errword, 113);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) issue_s(st ^ 1);
                __syncwarp();
            }
        }
        if (*abort_flag) {                    // let issued MMAs retire (bounded) before TMEM is released
            if (lane == 0) tc_commit(smem_u32(spare));
            __syncwarp();
            for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(smem_u32(spare), 0); i++) {}
        }
    } else {
        // =============================== softmax + output ===============================
        const int q = warp & 3, r = q * 32 + lane, i = q0 + r;       // tile row = TMEM lane, query index
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        float m = -1e30f, l = 0.0f, corr_pend = 1.0f;
        float o[AT_HD];
#pragma unroll
        for (int d = 0; d < AT_HD; d++) o[d] = 0.0f;
        bool ok = true;
        auto fold_pv = [&]() {                 // O = O * corr + PV for the tile whose PV just completed
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tmem_ld32(tPV + lane_base + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) o[c * 32 + j] = o[c * 32 + j] * corr_pend + __uint_as_float(v[j]);
            }
        };
        for (int t = 0; ok && t < nt; t++) {
            const int k0 = (kt_lo + t) * AT_BN;
            const bool masked = (k0 + AT_BN - 1 > q0) || p.win > 0 || (k0 + AT_BN > p.T);
            ok = mbar_wait(smem_u32(s_full), (uint32_t)t & 1u, abort_flag, p.errword, 120);
            if (!ok) break;
            tc_fence_after();
            // pass 1: row maximum
            float mx = -1e30f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tS + lane_base + c * 32, v);
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
            const float m_new = fmaxf(m, mx * p.scale_log2);
            const float corr = exp2f(m - m_new);
            // the previous tile's PV: its MMA was issued before this tile's S, so it has completed
            if (t > 0) {
                ok = mbar_wait(smem_u32(o_full), (uint32_t)(t - 1) & 1u, abort_flag, p.errword, 121);
                if (!ok) break;
                tc_fence_after();
                fold_pv();
            }
            corr_pend = corr;
            // pass 2: P = exp2(s - m) as bf16 into the swizzled K-major tile, row sum
            float rs = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tS + lane_base + c * 32, v);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float p0 = exp2f(__uint_as_float(v[j]) * p.scale_log2 - m_new);
                    float p1 = exp2f(__uint_as_float(v[j + 1]) * p.scale_log2 - m_new);
                    if (masked) {
                        if (!attn_valid(k0 + c * 32 + j, i, p.T, p.win)) p0 = 0.0f;
                        if (!attn_valid(k0 + c * 32 + j + 1, i, p.T, p.win)) p1 = 0.0f;
                    }
                    rs += p0 + p1;
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                    pk[j >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                }
                uint8_t *rowp = sP + (c >> 1) * (AT_BM * 128) + r * 128;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int unit = ((c & 1) * 4 + u) ^ (r & 7);
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
        if (ok) ok = mbar_wait(smem_u32(o_full), (uint32_t)(nt - 1) & 1u, abort_flag, p.errword, 122);
        if (ok) {
            tc_fence_after();
            fold_pv();
            if (i < p.T) {
                const float inv = 1.0f / l;
                bf16 *orow = p.O + ((size_t)b * p.T + i) * ((size_t)p.H * AT_HD) + (size_t)h * AT_HD;
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    uint32_t w[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(o[u * 8 + 2 * k] * inv, o[u * 8 + 2 * k + 1] * inv);
                        w[k] = *reinterpret_cast<uint32_t *>(&h2);
                    }
                    *reinterpret_cast<uint4 *>(orow + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                p.lse[((size_t)b * p.H + h) * p.T + i] = (m + log2f(l)) * 0.6931471805599453f;
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
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
    static bool configured = false;
    if (!configured) {
        QLMB_CUDA(cudaFuncSetAttribute(k_attn_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_FWD_SMEM));
        configured = true;
    }
    k_attn_fwd<<<(unsigned)(p.nqt * B * H), 192, AT_FWD_SMEM, as_stream(stream)>>>(p);
    QLMB_LAUNCH_CHECK("k_attn_fwd");
    return QLMB_OK;
}
