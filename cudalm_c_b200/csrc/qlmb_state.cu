// QLM integer state kernels: encode, render, integer AdamW step, scale servo,
// global-norm clip and the bf16-moment AdamW for unquantised spans.
//
// THIS TRANSLATION UNIT IS BUILT WITH --fmad=false.  The integer state is only
// reproducible against the reference's CPU build when no a*b+c is fused
// (the reference documents the same for its own no-FMA flavour, build.py:253);
// division and sqrt are the IEEE-rounded defaults (-prec-div/-prec-sqrt).
//
// Thread mapping of the hot kernel (step_fast): a TEAM of 8 lanes owns one
// 128-element group, each lane 16 consecutive elements, so every global access
// is a 128-bit (G, r, m8, v8) or 64-bit (packed digits) vector and a warp
// covers 4 groups = 2 KiB of gradient per load instruction.  Group maxima are
// 3-step shuffles inside the team; nibble pairs never leave a lane.
#include <stdlib.h>
#include <string.h>
#include "qlmb_common.cuh"

namespace qlmb {

// ---------------------------------------------------------------- rounding
// floor(v) + [24-bit draw < frac(v)]  (reference qlm.cuh:83-87); key = the
// pre-multiplied element term plus the per-launch step term.
__device__ __forceinline__ int sround_key(float v, uint64_t key)
{
    float fl = floorf(v);
    uint32_t h = hash_u32(key);
    float u = (float)(h >> 8) * (1.0f / 16777216.0f);
    return (int)fl + (u < (v - fl) ? 1 : 0);
}

struct StepArgs {
    float *P; const float *G; int8_t *d; int8_t *r; const float *s; int8_t *m8; float *m8s;
    uint8_t *v8; float *v8s; const qlmb_span *sp; int nspan; int group; int dmax;
    float lr, b1, b2, wd, gscale; const float *gsp; float inv_bc1, inv_sqrt_bc2;
    int lrmode; uint64_t t; int adam; unsigned long long *stat; int packed; int gi_base, ng;
    int v4;       // QLM_V4 (qlm.cuh:62-67): v8 holds the fourth root of the second moment instead of its square root
    // sparse form (k_ng_q4_step, cudalm.cu:4476-4530): group w of the launch is touched[w], its gradients are the w-th
    // row of a compact buffer; only the first *touched_count entries are live
    const int *touched; const int *touched_count;
    unsigned long long *skipped;    // device counter of launches that found a non-finite norm and wrote nothing
    qlmb_span inl; int use_inl;     // one span carried in the launch arguments (the n-gram table) instead of a table in memory
    float one;                      // 1.0f, as a run-time value (see pk_add)
};

// gpu_adam returns without stepping when the gradient norm is not finite (cudalm.cu:6446-6447; the caller prints
// "[nan] ... step skipped", 8651-8656).  The reference reads the norm back to the host for that; here every step
// kernel looks at the norm word that follows the clip multiplier (gs[1], as k_gnorm leaves it) and returns before
// its first store, so a bad step costs no host round trip and leaves every state byte as it was.
__device__ __forceinline__ bool step_is_skipped(const StepArgs &a)
{
    if (!a.gsp) return false;
    const float gn = a.gsp[1];
    if (isfinite(gn)) return false;
    if (blockIdx.x == 0 && threadIdx.x == 0 && a.skipped) atomicAdd(a.skipped, 1ULL);
    return true;
}

// Per-element update shared by both paths (reference qlm.cuh:206-242).
// Returns the new digit; writes mn / rv (the un-quantised new moments).
struct ElemOut { int dd; int rr; float mn; float rv; int idl; int c; };
__device__ __forceinline__ ElemOut elem_update(float g, int m8v, int v8v, int dd, int rold,
                                               float gs, float ms_old, float vs_old, float b1,
                                               float b2, float omb1, float omb2, float inv_bc1,
                                               float inv_sqrt_bc2, float L, float dec, int dmax,
                                               int adam, uint64_t key_t, int v4 = 0)
{
    ElemOut o;
    float gr = g * gs;
    float mv = (float)m8v * ms_old;
    float u;
    o.rv = 0.0f;
    if (adam) {
        float sv = (float)v8v * vs_old;
        if (v4) sv = sv * sv;                            // qv_dec
        float vv = sv * sv;
        o.mn = b1 * mv + omb1 * gr;
        vv = b2 * vv + omb2 * gr * gr;
        o.rv = sqrtf(vv);
        float veps = fmaxf(v4 ? vs_old * vs_old : vs_old, 1e-8f);
        u = (o.mn * inv_bc1) / (o.rv * inv_sqrt_bc2 + veps);
        u = fmaxf(-8.0f, fminf(8.0f, u));
        if (v4) o.rv = sqrtf(o.rv);                      // qv_enc: what is quantised and maximised
    } else {
        float cc = b1 * mv + omb1 * gr;
        u = (float)((cc > 0.0f) - (cc < 0.0f));
        o.mn = b2 * mv + omb2 * gr;
    }
    o.idl = sround_key(-(L * u + dec * (float)dd), key_t);
    int rr = rold + o.idl;
    int c = 0;
    if (rr > 64) c = ((rr - 65) >> 7) + 1;
    else if (rr < -64) c = -((((-rr) - 65) >> 7) + 1);
    o.c = c;
    o.rr = rr - 128 * c;
    o.dd = clampi(dd + c, -dmax, dmax);
    return o;
}

// ------------------------------------------------- generic team-per-group step
// T lanes (team) walk one group two elements (= one packed byte) at a time.
// Pass 1 updates digits/residuals and finds the group maxima; pass 2 recomputes
// the new moments from the still-unmodified m8/v8/G and re-quantises them, so
// no per-lane arrays are needed for any group size up to 256.
template <int T>
__device__ void step_group_team(const StepArgs &a, int gi, int tl, unsigned tmask, long long g_row = -1)
{
    uint64_t j0; int n;
    int si = locate_group(a.sp, a.nspan, gi, a.group, j0, n);
    const qlmb_span &S = a.sp[si];
    uint64_t q0 = S.qi0 + j0, p0 = S.pof + j0, g0 = g_row >= 0 ? (uint64_t)g_row * (uint64_t)a.group : S.gof + j0;
    float gs = a.gsp ? *a.gsp : a.gscale;
    float sg = a.s[gi];
    float L = a.lr * 128.0f / (a.lrmode ? sg : S.sref);
    float dec = a.lr * a.wd * 128.0f;
    float ms_old = a.m8s[gi], vs_old = a.v8s ? a.v8s[gi] : 0.0f;
    float omb1 = 1.0f - a.b1, omb2 = 1.0f - a.b2;
    uint64_t kt = a.t * QLMB_HASH_T;
    float am = 0.0f, vm = 0.0f;
    unsigned long long st0 = 0, st1 = 0, st2 = 0, st3 = 0;
    for (int p = tl; 2 * p < n; p += T) {
        int dig[2] = {0, 0};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int j = 2 * p + h;
            if (j >= n) break;
            uint64_t qi = q0 + j;
            int dd = digit_at(a.d, qi, a.packed);
            ElemOut o = elem_update(a.G[g0 + j], a.m8[qi], a.adam ? a.v8[qi] : 0, dd, a.r[qi], gs,
                                    ms_old, vs_old, a.b1, a.b2, omb1, omb2, a.inv_bc1,
                                    a.inv_sqrt_bc2, L, dec, a.dmax, a.adam, qi * QLMB_HASH_I + kt, a.v4);
            dig[h] = o.dd;
            a.r[qi] = (int8_t)o.rr;
            if (a.P) a.P[p0 + j] = sg * (float)o.dd;
            if (!a.packed) a.d[qi] = (int8_t)o.dd;
            am = fmaxf(am, fabsf(o.mn));
            vm = fmaxf(vm, o.rv);
            if (a.stat) {
                unsigned long long ai = (unsigned long long)(o.idl < 0 ? -o.idl : o.idl);
                st3 = ai > st3 ? ai : st3;
                st0 += (unsigned long long)(o.c < 0 ? -o.c : o.c);
                st1 += (o.dd == a.dmax) | (o.dd == -a.dmax);
                st2 += (o.dd == 0);
            }
        }
        if (a.packed) a.d[(q0 >> 1) + p] = (int8_t)(((dig[1] & 15) << 4) | (dig[0] & 15));
    }
#pragma unroll
    for (int o = T / 2; o > 0; o >>= 1) {
        am = fmaxf(am, __shfl_xor_sync(tmask, am, o));
        vm = fmaxf(vm, __shfl_xor_sync(tmask, vm, o));
    }
    float ms = am > 0.0f ? am / 127.0f : 1e-12f;
    float vs = vm > 0.0f ? vm / 255.0f : 1e-12f;
    // pass 2: every lane re-derives the moments of the elements it owns
    for (int p = tl; 2 * p < n; p += T) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int j = 2 * p + h;
            if (j >= n) break;
            uint64_t qi = q0 + j;
            float gr = a.G[g0 + j] * gs;
            float mv = (float)a.m8[qi] * ms_old, mn, rv = 0.0f;
            if (a.adam) {
                float sv = (float)a.v8[qi] * vs_old;
                if (a.v4) sv = sv * sv;
                float vv = sv * sv;
                mn = a.b1 * mv + omb1 * gr;
                vv = a.b2 * vv + omb2 * gr * gr;
                rv = sqrtf(vv);
                if (a.v4) rv = sqrtf(rv);
            } else {
                mn = a.b2 * mv + omb2 * gr;
            }
            a.m8[qi] = (int8_t)clampi(sround_key(mn / ms, qi * QLMB_HASH_I + (a.t + 0x5EEDULL) * QLMB_HASH_T), -127, 127);
            if (a.adam) {
                int vq = clampi(sround_key(rv / vs, qi * QLMB_HASH_I + (a.t + 0xBEEFULL) * QLMB_HASH_T), 0, 255);
                if (vq == 0 && rv > 0.0f) vq = 1;
                a.v8[qi] = (uint8_t)vq;
            }
        }
    }
    // the scales are read by pass 2 of no other team, so they can be stored last
    __syncwarp(tmask);
    if (tl == 0) { a.m8s[gi] = ms; if (a.adam) a.v8s[gi] = vs; }
    if (a.stat) {
        atomicAdd(&a.stat[0], st0); atomicAdd(&a.stat[1], st1); atomicAdd(&a.stat[2], st2);
        atomicMax(&a.stat[3], st3);
    }
}

__global__ void __launch_bounds__(256) k_step_generic(const __grid_constant__ StepArgs a0)
{
    if (step_is_skipped(a0)) return;
    StepArgs a = a0;
    if (a0.use_inl) a.sp = &a0.inl;
    int w = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (w >= a.ng) return;
    if (a.touched) {
        if (w >= *a.touched_count) return;
        step_group_team<32>(a, a.touched[w], threadIdx.x & 31, 0xffffffffu, w);
        return;
    }
    step_group_team<32>(a, a.gi_base + w, threadIdx.x & 31, 0xffffffffu);
}

// ------------------------------------------------ sparse table update: touched groups and their compact gradients
// (ng_build_touched + k_ng_scatter_compact, cudalm.cu:4465-4475, 4673-4700.)  The reference claims slots with a CAS
// and an atomic counter and adds gradients with float atomics; here every step has a fixed order: groups are marked,
// compacted in ascending group order by one block, and each gradient element is summed by one warp over the keys
// in ascending position -- the order of the reference's CPU build.
__global__ void __launch_bounds__(256) k_ng_mark(int *flag, const int *key, int NK, int De, int group)
{
    const int n = blockIdx.x * 256 + threadIdx.x;
    if (n >= NK) return;
    const int r = key[n];
    if (r >= 0) flag[(int)(((long long)r * De) / group)] = 1;
}
// one block: tgi[0..count) = the marked groups in ascending order; the flags are cleared for the next step
__global__ void __launch_bounds__(1024) k_ng_compact(int *tgi, int *count, int *flag, int ngrp)
{
    __shared__ int wsum[32];
    __shared__ int base;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) base = 0;
    __syncthreads();
    for (int g0 = 0; g0 < ngrp; g0 += 1024) {
        const int gi = g0 + tid;
        const int f = gi < ngrp ? flag[gi] : 0;
        if (f) flag[gi] = 0;
        int x = f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        if (lane == 31) wsum[warp] = x;
        __syncthreads();
        if (warp == 0) {
            int v = wsum[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += y; }
            wsum[lane] = v;                              // inclusive sums of the warps
        }
        __syncthreads();
        const int before = base + (warp ? wsum[warp - 1] : 0) + x - f;
        if (f) tgi[before] = gi;
        __syncthreads();
        if (tid == 0) base += wsum[31];
        __syncthreads();
    }
    if (tid == 0) *count = base;
}
// Gc[c*group + o] = sum over positions n (ascending) whose key is the row of element o: warp = (slot c, row of the group)
// the gradient row of key position n is dbuf + (n % Nd) * ld + (n / Nd) * sub: ld = De, sub = 0 for the n-gram table (every
// key set of a position reads the same row), ld = S * De, sub = De for the engram's S sub-tables (k_eg_scatter_c)
__global__ void __launch_bounds__(256) k_ng_scatter_compact(float *Gc, const int *key, const int *tgi, const int *count,
                                                            const float *dbuf, int NK, int De, int group, int Nd, int ld, int sub)
{
    __shared__ int skey[2048];
    const int rpg = group / De;                          // rows per group (group % De == 0)
    const int w = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int c = w / rpg, rr = w % rpg;
    const int cnt = *count;
    if (blockIdx.x * 8 / rpg >= cnt) return;             // the whole block is past the live slots
    const bool live = c < cnt;
    const int row = live ? (int)(((long long)tgi[c] * group) / De) + rr : -2;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] = 0.0f;
    for (int n0 = 0; n0 < NK; n0 += 2048) {
        __syncthreads();
        for (int i = threadIdx.x; i < 2048; i += 256) skey[i] = n0 + i < NK ? key[n0 + i] : -1;
        __syncthreads();
        const int lim = NK - n0 < 2048 ? NK - n0 : 2048;
        for (int q = 0; q < lim; q += 32) {
            unsigned m = __ballot_sync(0xffffffffu, skey[q + lane] == row);
            while (m) {
                const int n = n0 + q + __ffs(m) - 1;
                m &= m - 1;
                const float *src = dbuf + (size_t)(n % Nd) * ld + (size_t)(n / Nd) * sub;
#pragma unroll
                for (int k = 0; k < 8; k++) { const int e = lane + 32 * k; if (e < De) acc[k] += src[e]; }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < 8; k++) { const int e = lane + 32 * k; if (e < De) Gc[(size_t)c * group + rr * De + e] = acc[k]; }
    }
}

// ------------------------------------------------------- fast step, group 128
// A TEAM of 128/EPL lanes owns one group, each lane EPL consecutive elements
// (EPL = 4, 8 or 16), so a warp covers EPL/4 groups and every access is a
// vector of EPL*4 (gradient), EPL (r, m8, v8) or EPL/2 (digits) bytes.  Fewer
// elements per lane mean a smaller fully unrolled body (instruction cache)
// at the price of two more shuffle steps per reduction.
// Requirements checked per group at run time (else the team falls back to the
// generic walk): 128 full elements, digit offset a multiple of 16, P and G
// offsets multiples of 4; base pointers are 16-byte aligned (checked on host).
template <int BYTES> struct VecOf;
template <> struct VecOf<2> { typedef unsigned short T; };
template <> struct VecOf<4> { typedef uint32_t T; };
template <> struct VecOf<8> { typedef uint2 T; };
template <> struct VecOf<16> { typedef uint4 T; };
template <int BYTES>
__device__ __forceinline__ void ld_vec(uint32_t *dst, const void *src)
{
    typename VecOf<BYTES>::T v = *reinterpret_cast<const typename VecOf<BYTES>::T *>(src);
    if (BYTES == 2) dst[0] = *reinterpret_cast<unsigned short *>(&v);
    else memcpy(dst, &v, BYTES);
}
template <int BYTES>
__device__ __forceinline__ void st_vec(void *dst, const uint32_t *src)
{
    typename VecOf<BYTES>::T v;
    if (BYTES == 2) { unsigned short h = (unsigned short)src[0]; memcpy(&v, &h, 2); }
    else memcpy(&v, src, BYTES);
    *reinterpret_cast<typename VecOf<BYTES>::T *>(dst) = v;
}

template <bool WRITE_P, int EPL>
__global__ void __launch_bounds__(256) k_step_fast(StepArgs a)
{
    constexpr int TEAM = 128 / EPL;                      // lanes per group
    constexpr int GPW = 32 / TEAM;                       // groups per warp
    if (step_is_skipped(a)) return;
    const int lane = threadIdx.x & 31, tl = lane % TEAM, team = lane / TEAM;
    const unsigned tmask = (TEAM == 32) ? 0xffffffffu : (((1u << TEAM) - 1u) << (team * TEAM));
    long long w = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * GPW + team;
    if (w >= a.ng) return;
    int gi = a.gi_base + (int)w;
    uint64_t j0; int n;
    int si = locate_group(a.sp, a.nspan, gi, 128, j0, n);
    const qlmb_span &S = a.sp[si];
    uint64_t q0 = S.qi0 + j0, p0 = S.pof + j0, g0 = S.gof + j0;
    if (n != 128 || (q0 & 15) || (g0 & 3) || (WRITE_P && (p0 & 3))) {
        step_group_team<TEAM>(a, gi, tl, tmask);
        return;
    }
    const uint64_t qe = q0 + (uint64_t)tl * EPL;         // first element of this lane
    const float4 *gp = reinterpret_cast<const float4 *>(a.G + g0 + tl * EPL);
    float4 gv[EPL / 4];
#pragma unroll
    for (int i = 0; i < EPL / 4; i++) gv[i] = __ldcs(gp + i);
    uint32_t rw[(EPL + 3) / 4], mw[(EPL + 3) / 4], vw[(EPL + 3) / 4], dw[(EPL + 7) / 8];
    ld_vec<EPL>(rw, a.r + qe);
    ld_vec<EPL>(mw, a.m8 + qe);
    ld_vec<EPL>(vw, a.v8 + qe);
    ld_vec<EPL / 2>(dw, a.d + (qe >> 1));
    float gs = a.gsp ? *a.gsp : a.gscale;
    float sg = a.s[gi];
    float L = a.lr * 128.0f / (a.lrmode ? sg : S.sref);
    float dec = a.lr * a.wd * 128.0f;
    float ms_old = a.m8s[gi], vs_old = a.v8s[gi];
    float omb1 = 1.0f - a.b1, omb2 = 1.0f - a.b2;
    const uint64_t kt = a.t * QLMB_HASH_T;
    uint64_t key = qe * QLMB_HASH_I;                     // advanced by one multiplier per element

    const float *gf = reinterpret_cast<const float *>(gv);
    float mn[EPL], rv[EPL], am = 0.0f, vm = 0.0f;
    uint32_t rout[(EPL + 3) / 4], dout[(EPL + 7) / 8];
#pragma unroll
    for (int i = 0; i < (EPL + 3) / 4; i++) rout[i] = 0;
#pragma unroll
    for (int i = 0; i < (EPL + 7) / 8; i++) dout[i] = 0;
    float pv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) {
        int rold = (int)(int8_t)((rw[e >> 2] >> ((e & 3) * 8)) & 0xff);
        int m8v = (int)(int8_t)((mw[e >> 2] >> ((e & 3) * 8)) & 0xff);
        int v8v = (int)((vw[e >> 2] >> ((e & 3) * 8)) & 0xff);
        int nib = (int)((dw[e >> 3] >> ((e & 7) * 4)) & 15u);
        int dd = nib > 7 ? nib - 16 : nib;
        ElemOut o = elem_update(gf[e], m8v, v8v, dd, rold, gs, ms_old, vs_old, a.b1, a.b2, omb1,
                                omb2, a.inv_bc1, a.inv_sqrt_bc2, L, dec, a.dmax, 1, key + kt);
        key += QLMB_HASH_I;
        mn[e] = o.mn; rv[e] = o.rv;
        am = fmaxf(am, fabsf(o.mn));
        vm = fmaxf(vm, o.rv);
        rout[e >> 2] |= ((uint32_t)(o.rr & 0xff)) << ((e & 3) * 8);
        dout[e >> 3] |= ((uint32_t)(o.dd & 15)) << ((e & 7) * 4);
        if (WRITE_P) pv[e] = sg * (float)o.dd;
    }
    st_vec<EPL>(a.r + qe, rout);
    st_vec<EPL / 2>(a.d + (qe >> 1), dout);
    if (WRITE_P) {
        float4 *pp = reinterpret_cast<float4 *>(a.P + p0 + tl * EPL);
#pragma unroll
        for (int i = 0; i < EPL / 4; i++) pp[i] = make_float4(pv[4 * i], pv[4 * i + 1], pv[4 * i + 2], pv[4 * i + 3]);
    }
#pragma unroll
    for (int o = TEAM / 2; o > 0; o >>= 1) {
        am = fmaxf(am, __shfl_xor_sync(tmask, am, o));
        vm = fmaxf(vm, __shfl_xor_sync(tmask, vm, o));
    }
    float ms = am > 0.0f ? am / 127.0f : 1e-12f;
    float vs = vm > 0.0f ? vm / 255.0f : 1e-12f;
    if (tl == 0) { a.m8s[gi] = ms; a.v8s[gi] = vs; }
    uint32_t mo[(EPL + 3) / 4], vo[(EPL + 3) / 4];
#pragma unroll
    for (int i = 0; i < (EPL + 3) / 4; i++) { mo[i] = 0; vo[i] = 0; }
    const uint64_t ktm = (a.t + 0x5EEDULL) * QLMB_HASH_T, ktv = (a.t + 0xBEEFULL) * QLMB_HASH_T;
    key = qe * QLMB_HASH_I;
#pragma unroll
    for (int e = 0; e < EPL; e++) {
        int mq = clampi(sround_key(mn[e] / ms, key + ktm), -127, 127);
        int vq = clampi(sround_key(rv[e] / vs, key + ktv), 0, 255);
        if (vq == 0 && rv[e] > 0.0f) vq = 1;
        key += QLMB_HASH_I;
        mo[e >> 2] |= ((uint32_t)(mq & 0xff)) << ((e & 3) * 8);
        vo[e >> 2] |= ((uint32_t)vq) << ((e & 3) * 8);
    }
    st_vec<EPL>(a.m8 + qe, mo);
    st_vec<EPL>(a.v8 + qe, vo);
}

// ------------------------------------------------------- packed step, group 128
// The same arithmetic as k_step_fast, operation for operation and rounding for rounding, written for the
// instruction-issue limit that bounds this kernel (it is not the memory system: the update needs three 64-bit
// hashes, three stochastic roundings, three divisions and a square root per element).  What changes is only how
// many instructions carry the work:
//  * floating-point work runs on PAIRS of elements with the sm_100 two-wide fp32 instructions (add / mul / fma .rn.f32x2: each lane of a pair is an IEEE round-to-nearest operation, so results are those
//    of the scalar sequence);
//  * small integers live in floats (exactly representable), so bytes and nibbles are unpacked and packed with
//    byte permutes and a magic-number add instead of integer<->float conversions;
//  * x / ms and x / vs (one denominator per group) use the correctly rounded reciprocal r = RN(1 / y) computed
//    once per group: q0 = x*r, two residual corrections q <- q + (x - q*y)*r.  With r correctly rounded and q
//    faithful after the first correction, the second one returns RN(x / y) (Markstein's theorem), as long as no
//    intermediate underflows: the path is taken only for y in [2^-40, 1]; below |x| = 2^-100 the quotient is so
//    small that only its sign and whether it is zero reach the rounding, and both are preserved.  Any other
//    group divides with the IEEE operator;
//  * the carry c with rr - 128c in [-64, 64] (rr = +-64 does not carry) is RN((rr -+ 1/2) / 128), which has no
//    ties, taken with the magic-number add;
//  * the hash is written on 32-bit halves (one widening multiply and two multiply-adds per 64-bit product).
// Element values that cannot take this path (|L*8 + dec*7| >= 2^20, a short or unaligned group) go through the
// generic team walk.
__device__ __forceinline__ uint32_t mix32(uint64_t x)
{
    // x already holds key + 0x9E3779B97F4A7C15; returns the low 32 bits of the splitmix64 finaliser (qlm.cuh:78-82).
    // (Taking the shifts as widening multiplies by a power of two, to move them off the half-rate integer pipe,
    // was measured 22 % slower: 0.926 ms against 0.757 ms per 125.8 M parameters.)
    uint32_t lo = (uint32_t)x, hi = (uint32_t)(x >> 32);
    lo ^= __funnelshift_r(lo, hi, 30); hi ^= hi >> 30;
    uint64_t p = (uint64_t)lo * 0x1CE4E5B9u;
    hi = (uint32_t)(p >> 32) + lo * 0xBF58476Du + hi * 0x1CE4E5B9u;
    lo = (uint32_t)p;
    lo ^= __funnelshift_r(lo, hi, 27); hi ^= hi >> 27;
    p = (uint64_t)lo * 0x133111EBu;
    hi = (uint32_t)(p >> 32) + lo * 0x94D049BBu + hi * 0x133111EBu;
    lo = (uint32_t)p;
    return lo ^ __funnelshift_r(lo, hi, 31);
}
__device__ __forceinline__ float2 bc2(float x) { return make_float2(x, x); }
// Two-wide fp32 arithmetic.  ptxas contracts a two-wide multiply that feeds a two-wide add into a fused multiply-add
// even under --fmad=false and with explicit .rn instructions (measured: the scales came out as fma(b1, mv, .)), which
// the integer state's reproducibility cannot tolerate.  A sum of products is therefore written as
// fma(p, one, q) with `one` a kernel argument equal to 1.0f: RN(p * 1 + q) = RN(p + q), and a multiply cannot be
// folded into an existing fma.
__device__ __forceinline__ float2 pk_add(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 pk_mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 pk_fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
// floor(v) + [24-bit draw < frac(v)] for a pair, as floats (qsri, qlm.cuh:83-87)
__device__ __forceinline__ float2 sround_pair(float2 v, uint32_t h0, uint32_t h1)
{
    const float2 fl = make_float2(floorf(v.x), floorf(v.y));
    const float2 fr = pk_fma(fl, bc2(-1.0f), v);                  // v - fl, one rounding
    const float2 y = pk_mul(fr, bc2(16777216.0f));                // u * 2^-24 < fr  <=>  (h >> 8) < fr * 2^24 (both exact)
    const float p0 = (float)(h0 >> 8) < y.x ? 1.0f : 0.0f, p1 = (float)(h1 >> 8) < y.y ? 1.0f : 0.0f;
    return pk_add(fl, make_float2(p0, p1));
}
// x / y for a pair with one denominator; r = RN(1 / y)
__device__ __forceinline__ float2 div_pair(float2 x, float y, float r, bool fast)
{
    if (!fast) return make_float2(x.x / y, x.y / y);
    const float2 ny = bc2(-y), rr = bc2(r);
    float2 q = pk_mul(x, rr);
    q = pk_fma(pk_fma(q, ny, x), rr, q);
    q = pk_fma(pk_fma(q, ny, x), rr, q);
    return q;
}
// byte-permute selector that replaces byte j of the first operand by the low byte of the second
__host__ __device__ constexpr uint32_t ins_sel(int j) { return j == 0 ? 0x3214u : j == 1 ? 0x3240u : j == 2 ? 0x3410u : 0x4210u; }
#define QLMB_MAGIC_RN 12582912.0f        // 1.5 * 2^23: adding it leaves the integer nearest to x in the low mantissa bits
#define QLMB_MAGIC_U 8388608.0f          // 2^23 under a byte: as_float(0x4B000000 | b) = 2^23 + b

template <bool WRITE_P>
__global__ void __launch_bounds__(256) k_step_pk(const __grid_constant__ StepArgs a)
{
    constexpr int EPL = 8, TEAM = 16, NP = EPL / 2;
    constexpr bool CVT = true;      // bytes -> floats by conversion instructions (0.7455 ms) or by byte permutes and a magic add (0.7569 ms)
#define MIX(x) mix32(x)
    if (step_is_skipped(a)) return;
    const int lane = threadIdx.x & 31, tl = lane % TEAM, team = lane / TEAM;
    const unsigned tmask = 0xffffu << (team * TEAM);
    const long long w = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * 2 + team;
    if (w >= a.ng) return;
    const int gi = a.gi_base + (int)w;
    uint64_t j0; int n;
    const int si = locate_group(a.sp, a.nspan, gi, 128, j0, n);
    const qlmb_span &S = a.sp[si];
    const uint64_t q0 = S.qi0 + j0, p0 = S.pof + j0, g0 = S.gof + j0;
    const float sg = a.s[gi];
    const float L = a.lr * 128.0f / (a.lrmode ? sg : S.sref);
    const float dec = a.lr * a.wd * 128.0f;
    if (n != 128 || (q0 & 15) || (g0 & 3) || (WRITE_P && (p0 & 3)) || !(fabsf(L) * 8.0f + fabsf(dec) * 7.0f < 1048576.0f)) {
        step_group_team<TEAM>(a, gi, tl, tmask);
        return;
    }
    const uint64_t qe = q0 + (uint64_t)tl * EPL;
    const float4 *gp = reinterpret_cast<const float4 *>(a.G + g0 + tl * EPL);
    const float4 ga = __ldcs(gp), gb = __ldcs(gp + 1);
    const uint2 rw = *reinterpret_cast<const uint2 *>(a.r + qe);
    const uint2 mw = *reinterpret_cast<const uint2 *>(a.m8 + qe);
    const uint2 vw = *reinterpret_cast<const uint2 *>(a.v8 + qe);
    const uint32_t dw = *reinterpret_cast<const uint32_t *>(a.d + (qe >> 1));
    const float gs = a.gsp ? *a.gsp : a.gscale;
    const float ms_old = a.m8s[gi], vs_old = a.v8s[gi];
    const float omb1 = 1.0f - a.b1, omb2 = 1.0f - a.b2;
    const float veps = fmaxf(vs_old, 1e-8f), dmaxf = (float)a.dmax;
    // keys: element index term of this lane + the three step terms (the finaliser's first add is folded in)
    const uint64_t kbase = qe * QLMB_HASH_I + 0x9E3779B97F4A7C15ULL;
    const uint64_t kd = kbase + a.t * QLMB_HASH_T, km = kbase + (a.t + 0x5EEDULL) * QLMB_HASH_T,
                   kv = kbase + (a.t + 0xBEEFULL) * QLMB_HASH_T;

    const float2 one2 = bc2(a.one);
    const float2 g2[NP] = {make_float2(ga.x, ga.y), make_float2(ga.z, ga.w), make_float2(gb.x, gb.y), make_float2(gb.z, gb.w)};
    // bytes -> floats: signed bytes are biased by 128 first, nibbles by 8
    const uint32_t rx[2] = {rw.x ^ 0x80808080u, rw.y ^ 0x80808080u}, mx[2] = {mw.x ^ 0x80808080u, mw.y ^ 0x80808080u};
    const uint32_t vx[2] = {vw.x, vw.y};
    const uint32_t dx = dw ^ 0x88888888u, dev = dx & 0x0F0F0F0Fu, dod = (dx >> 4) & 0x0F0F0F0Fu;
    float2 mn[NP], rv[NP];
    float am = 0.0f, vm = 0.0f;
    uint32_t rout[2] = {0u, 0u}, dout = 0u;
    float4 pv[2];
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int e0 = 2 * p, wd_ = e0 >> 2, b0 = e0 & 3;            // word and byte of the pair's first element
        auto byte2 = [&](const uint32_t *src, float bias) {
            const float x0 = __uint_as_float(__byte_perm(src[wd_], 0x4B000000u, 0x7440 + b0));
            const float x1 = __uint_as_float(__byte_perm(src[wd_], 0x4B000000u, 0x7441 + b0));
            return pk_add(make_float2(x0, x1), bc2(bias));
        };
        float2 rold, m8f, v8f;
        if (CVT) {
            const uint32_t rs = wd_ ? rw.y : rw.x, ms_ = wd_ ? mw.y : mw.x, vs_ = wd_ ? vw.y : vw.x;
            rold = make_float2((float)(int8_t)(rs >> (8 * b0)), (float)(int8_t)(rs >> (8 * b0 + 8)));
            m8f = make_float2((float)(int8_t)(ms_ >> (8 * b0)), (float)(int8_t)(ms_ >> (8 * b0 + 8)));
            v8f = make_float2((float)(uint8_t)(vs_ >> (8 * b0)), (float)(uint8_t)(vs_ >> (8 * b0 + 8)));
        } else {
            rold = byte2(rx, -(QLMB_MAGIC_U + 128.0f)); m8f = byte2(mx, -(QLMB_MAGIC_U + 128.0f)); v8f = byte2(vx, -QLMB_MAGIC_U);
        }
        const float2 ddf = pk_add(make_float2(__uint_as_float(__byte_perm(dev, 0x4B000000u, 0x7440 + p)),
                                                  __uint_as_float(__byte_perm(dod, 0x4B000000u, 0x7440 + p))), bc2(-(QLMB_MAGIC_U + 8.0f)));
        // moments (qlm.cuh:206-222)
        const float2 gr = pk_mul(g2[p], bc2(gs));
        const float2 mv = pk_mul(m8f, bc2(ms_old));
        const float2 sv = pk_mul(v8f, bc2(vs_old));
        float2 vv = pk_mul(sv, sv);
        mn[p] = pk_fma(pk_mul(bc2(a.b1), mv), one2, pk_mul(bc2(omb1), gr));
        vv = pk_fma(pk_mul(bc2(a.b2), vv), one2, pk_mul(pk_mul(bc2(omb2), gr), gr));
        rv[p] = make_float2(sqrtf(vv.x), sqrtf(vv.y));
        const float2 num = pk_mul(mn[p], bc2(a.inv_bc1));
        const float2 den = pk_fma(pk_mul(rv[p], bc2(a.inv_sqrt_bc2)), one2, bc2(veps));
        float2 u = make_float2(num.x / den.x, num.y / den.y);
        u.x = fmaxf(-8.0f, fminf(8.0f, u.x)); u.y = fmaxf(-8.0f, fminf(8.0f, u.y));
        am = fmaxf(am, fmaxf(fabsf(mn[p].x), fabsf(mn[p].y)));
        vm = fmaxf(vm, fmaxf(rv[p].x, rv[p].y));
        // digit and residual (qlm.cuh:231-242): -(L*u + dec*d), rounded stochastically, added to the residual
        const float2 v = pk_fma(pk_mul(bc2(-L), u), one2, pk_mul(bc2(-dec), ddf));
        const float2 idl = sround_pair(v, MIX(kd + (uint64_t)e0 * QLMB_HASH_I), MIX(kd + (uint64_t)(e0 + 1) * QLMB_HASH_I));
        const float2 rr = pk_add(rold, idl);
        const float2 half = make_float2(__uint_as_float(0xBB800000u ^ (__float_as_uint(rr.x) & 0x80000000u)),
                                        __uint_as_float(0xBB800000u ^ (__float_as_uint(rr.y) & 0x80000000u)));   // -+ 2^-8
        const float2 c = pk_add(pk_add(pk_fma(rr, bc2(0.0078125f), half), bc2(QLMB_MAGIC_RN)), bc2(-QLMB_MAGIC_RN));
        const float2 rnew = pk_fma(c, bc2(-128.0f), rr);
        float2 dn = pk_add(ddf, c);
        dn.x = fminf(fmaxf(dn.x, -dmaxf), dmaxf); dn.y = fminf(fmaxf(dn.y, -dmaxf), dmaxf);
        const float2 rb = pk_add(rnew, bc2(QLMB_MAGIC_RN)), db = pk_add(dn, bc2(QLMB_MAGIC_RN));
        rout[wd_] = __byte_perm(rout[wd_], __float_as_uint(rb.x), ins_sel(b0));
        rout[wd_] = __byte_perm(rout[wd_], __float_as_uint(rb.y), ins_sel(b0 + 1));
        const uint32_t nb = (__float_as_uint(db.x) & 15u) | (__float_as_uint(db.y) << 4);
        dout = __byte_perm(dout, nb, ins_sel(p));
        if (WRITE_P) {
            const float2 pp = pk_mul(bc2(sg), dn);
            if (p & 1) { pv[p >> 1].z = pp.x; pv[p >> 1].w = pp.y; } else { pv[p >> 1].x = pp.x; pv[p >> 1].y = pp.y; }
        }
    }
    *reinterpret_cast<uint2 *>(a.r + qe) = make_uint2(rout[0], rout[1]);
    *reinterpret_cast<uint32_t *>(a.d + (qe >> 1)) = dout;
    if (WRITE_P) {
        float4 *pp = reinterpret_cast<float4 *>(a.P + p0 + tl * EPL);
        pp[0] = pv[0]; pp[1] = pv[1];
    }
#pragma unroll
    for (int o = TEAM / 2; o > 0; o >>= 1) {
        am = fmaxf(am, __shfl_xor_sync(tmask, am, o));
        vm = fmaxf(vm, __shfl_xor_sync(tmask, vm, o));
    }
    const float ms = am > 0.0f ? am / 127.0f : 1e-12f;
    const float vs = vm > 0.0f ? vm / 255.0f : 1e-12f;
    if (tl == 0) { a.m8s[gi] = ms; a.v8s[gi] = vs; }
    // 2^-40 <= y <= 1: the reciprocal path is exact there (see above); NaN fails both comparisons
    const bool fm = ms >= 9.094947e-13f && ms <= 1.0f, fv = vs >= 9.094947e-13f && vs <= 1.0f;
    const float rms = 1.0f / ms, rvs = 1.0f / vs;
    uint32_t mo[2] = {0u, 0u}, vo[2] = {0u, 0u};
#pragma unroll
    for (int p = 0; p < NP; p++) {
        const int e0 = 2 * p, wd_ = e0 >> 2, b0 = e0 & 3;
        const uint64_t ei = (uint64_t)e0 * QLMB_HASH_I, ej = (uint64_t)(e0 + 1) * QLMB_HASH_I;
        float2 mq = sround_pair(div_pair(mn[p], ms, rms, fm), MIX(km + ei), MIX(km + ej));
        mq.x = fminf(fmaxf(mq.x, -127.0f), 127.0f); mq.y = fminf(fmaxf(mq.y, -127.0f), 127.0f);
        float2 vq = sround_pair(div_pair(rv[p], vs, rvs, fv), MIX(kv + ei), MIX(kv + ej));
        // clamp to [0, 255]; a value that rounded to 0 while rv > 0 becomes 1 (qlm.cuh:275-277)
        vq.x = fminf(fmaxf(vq.x, rv[p].x > 0.0f ? 1.0f : 0.0f), 255.0f); vq.y = fminf(fmaxf(vq.y, rv[p].y > 0.0f ? 1.0f : 0.0f), 255.0f);
        const float2 mb = pk_add(mq, bc2(QLMB_MAGIC_RN)), vb = pk_add(vq, bc2(QLMB_MAGIC_U));
        mo[wd_] = __byte_perm(mo[wd_], __float_as_uint(mb.x), ins_sel(b0));
        mo[wd_] = __byte_perm(mo[wd_], __float_as_uint(mb.y), ins_sel(b0 + 1));
        vo[wd_] = __byte_perm(vo[wd_], __float_as_uint(vb.x), ins_sel(b0));
        vo[wd_] = __byte_perm(vo[wd_], __float_as_uint(vb.y), ins_sel(b0 + 1));
    }
    *reinterpret_cast<uint2 *>(a.m8 + qe) = make_uint2(mo[0], mo[1]);
    *reinterpret_cast<uint2 *>(a.v8 + qe) = make_uint2(vo[0], vo[1]);
#undef MIX
}

// ------------------------------------------------------------------ encode
// One warp per group, lanes walk byte pairs (reference qlm.cuh:136-167).
__global__ void __launch_bounds__(256) k_encode(const float *P, int8_t *d, int8_t *r, float *s,
                                                const qlmb_span *sp, int nspan, int ngrp, int group,
                                                int dmax, int packed)
{
    int gi = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (gi >= ngrp) return;
    uint64_t j0; int n;
    int si = locate_group(sp, nspan, gi, group, j0, n);
    const float *p = P + sp[si].pof + j0;
    uint64_t q0 = sp[si].qi0 + j0;
    float amax = 0.0f;
    for (int j = lane; j < n; j += 32) amax = fmaxf(amax, fabsf(p[j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc = amax / (float)dmax;
    if (!(sc > 0.0f)) sc = 1e-8f;
    if (lane == 0) s[gi] = sc;
    for (int b = lane; 2 * b < n; b += 32) {
        int dig[2] = {0, 0};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int j = 2 * b + h;
            if (j >= n) break;
            float t = p[j] / sc;
            int dd = clampi((int)rintf(t), -dmax, dmax);
            int rr = clampi((int)rintf((t - (float)dd) * 128.0f), -64, 64);
            dig[h] = dd;
            r[q0 + j] = (int8_t)rr;
            if (!packed) d[q0 + j] = (int8_t)dd;
        }
        if (packed) d[(q0 >> 1) + b] = (int8_t)(((dig[1] & 15) << 4) | (dig[0] & 15));
    }
}

// ------------------------------------------------------------------ render
__global__ void __launch_bounds__(256) k_render(float *P, const int8_t *d, const float *s,
                                                const qlmb_span *sp, int nspan, int group,
                                                int packed, int gi_base, int ng)
{
    int w = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= ng) return;
    int gi = gi_base + w, n; uint64_t j0;
    int si = locate_group(sp, nspan, gi, group, j0, n);
    float sc = s[gi];
    float *p = P + sp[si].pof + j0;
    uint64_t q0 = sp[si].qi0 + j0;
    for (int j = lane; j < n; j += 32) p[j] = sc * (float)digit_at(d, q0 + j, packed);
}

// ------------------------------------------------------------------- servo
// One warp per group (reference qlm.cuh:404-441).
__global__ void __launch_bounds__(256) k_servo(int8_t *d, int8_t *r, float *s, const qlmb_span *sp,
                                               int nspan, int ngrp, int group, int dmax, float f_hi,
                                               float f_lo, int packed)
{
    int gi = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (gi >= ngrp) return;
    uint64_t j0; int n;
    int si = locate_group(sp, nspan, gi, group, j0, n);
    uint64_t q0 = sp[si].qi0 + j0;
    int railed = 0;
    for (int j = lane; j < n; j += 32) {
        int dd = digit_at(d, q0 + j, packed);
        railed += (dd == dmax) | (dd == -dmax);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) railed += __shfl_xor_sync(0xffffffffu, railed, o);
    float f = (float)railed / (float)n, old = s[gi], nw;
    if (f > f_hi) nw = old * 1.09051f;
    else if (f < f_lo) nw = old / 1.09051f;
    else return;
    float conv = old / nw;
    __syncwarp();
    if (lane == 0) s[gi] = nw;
    for (int b = lane; 2 * b < n; b += 32) {
        int dig[2] = {0, 0};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int j = 2 * b + h;
            if (j >= n) break;
            uint64_t qi = q0 + j;
            float t = ((float)digit_at(d, qi, packed) + (float)r[qi] * (1.0f / 128.0f)) * conv;
            int dd = clampi((int)rintf(t), -dmax, dmax);
            int rr = clampi((int)rintf((t - (float)dd) * 128.0f), -64, 64);
            dig[h] = dd;
            r[qi] = (int8_t)rr;
            if (!packed) d[qi] = (int8_t)dd;
        }
        if (packed) d[(q0 >> 1) + b] = (int8_t)(((dig[1] & 15) << 4) | (dig[0] & 15));
    }
}

// -------------------------------------------------------------- grad norm
// Stage 1: chunk c of 64 covers [n*c/64, n*(c+1)/64) (reference CPU build,
// cpu_kern.h:533-540); each chunk is split over SUB blocks whose double sums
// are combined in a fixed order by stage 2, so the result does not depend on
// scheduling.  Double accumulation makes the float rounding of each chunk sum
// agree with the CPU's double loop.
#define GN_SUB 16
__global__ void __launch_bounds__(256) k_sq_partial(const float *G, size_t n, double *sub)
{
    __shared__ double sh[8];
    int c = blockIdx.y, b = blockIdx.x;
    size_t i0 = n * (size_t)c / 64, i1 = n * (size_t)(c + 1) / 64;
    size_t len = i1 - i0, per = (len + GN_SUB - 1) / GN_SUB;
    size_t lo = i0 + per * (size_t)b, hi = lo + per < i1 ? lo + per : i1;
    double acc = 0.0;
    for (size_t i = lo + threadIdx.x; i < hi; i += 256) { double g = (double)G[i]; acc += g * g; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < 8; i++) t += sh[i];
        sub[(size_t)c * GN_SUB + b] = t;
    }
}
// Stage 2 (reference cudalm.cu:2807-2812): part[64*(1+nside)] -> gs[0..1].
__global__ void k_gnorm_final(const double *sub, int nside, int clip_side, float *gs)
{
    double ss = 0.0, sd = 0.0;
    for (int i = 0; i < 64 * (1 + nside); i++) {
        double t = 0.0;
        for (int b = 0; b < GN_SUB; b++) t += sub[(size_t)i * GN_SUB + b];
        float part = (float)t;
        if (i < 64) ss += part; else sd += part;
    }
    float gn = (float)sqrt(clip_side ? ss + sd : ss);
    if (!isfinite(sd)) gn = __int_as_float(0x7fc00000);
    gs[0] = gn > 1.0f ? 1.0f / gn : 1.0f;
    gs[1] = gn;
}

// The fused per-layer update (reference qlm_fused_layer / qlm_fused_tail, cudalm.cu:6105-6187)
// keeps one slice of 64 float partial sums per layer and closes the norm once per step.
__global__ void k_sq_fold(const double *sub, float *part64)
{
    const int c = threadIdx.x;
    double t = 0.0;
    for (int b = 0; b < GN_SUB; b++) t += sub[(size_t)c * GN_SUB + b];
    part64[c] = (float)t;
}
// Close-out: all partials added in ascending order in double, as the reference's host loop does
// (cudalm.cu:6182-6186); one thread, a few thousand additions once per step.
__global__ void k_gnorm_close(const float *part, int n, float *gs)
{
    double ss = 0.0;
    for (int i = 0; i < n; i++) ss += (double)part[i];
    const float gn = (float)sqrt(ss);
    gs[0] = gn > 1.0f ? 1.0f / gn : 1.0f;
    gs[1] = gn;
}

// ------------------------------------------------------ float-span AdamW
__device__ __forceinline__ float bf_to_f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ uint16_t f_to_bf(float f)
{
    uint32_t x = __float_as_uint(f);
    return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}
// reference cudalm.cu:2855-2870 in the CPU build's operation order
// (cpu_kern.h:552-561): (m/bc1) / (sqrt(v/bc2) + 1e-8)
__global__ void __launch_bounds__(256) k_adamw_bf16(float *P, const float *G, uint16_t *M,
                                                    uint16_t *V, size_t n, float lr, float b1,
                                                    float b2, float wd, float bc1, float bc2,
                                                    const float *gs)
{
    size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    if (gs && !isfinite(gs[1])) return;                  // the step is skipped on a non-finite norm (cudalm.cu:6446-6447)
    float g = gs ? G[i] * gs[0] : G[i];
    float m = b1 * bf_to_f(M[i]) + (1.0f - b1) * g;
    float v = b2 * bf_to_f(V[i]) + (1.0f - b2) * g * g;
    M[i] = f_to_bf(m);
    V[i] = f_to_bf(v);
    float p = P[i];
    P[i] = p - lr * ((m / bc1) / (sqrtf(v / bc2) + 1e-8f) + wd * p);
}

// per-device scratch for the partial sums, grown on demand
static double *g_gn_scratch[64];
static size_t g_gn_cap[64];

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_encode(const float *P, int8_t *d, int8_t *r, float *s, const qlmb_span *sp,
                           int nspan, int ngrp, int group, int dmax, int packed, void *stream)
{
    QLMB_REQUIRE(P && d && r && s && sp && nspan > 0, "qlmb_encode: NULL argument");
    QLMB_REQUIRE(group >= 32 && group <= 256 && (!packed || (group % 2) == 0), "qlmb_encode: group %d", group);
    QLMB_REQUIRE(dmax >= 1 && dmax <= 127 && (!packed || dmax <= 7), "qlmb_encode: dmax %d", dmax);
    if (ngrp <= 0) return QLMB_OK;
    k_encode<<<(ngrp + 7) / 8, 256, 0, as_stream(stream)>>>(P, d, r, s, sp, nspan, ngrp, group, dmax, packed);
    QLMB_LAUNCH_CHECK("k_encode");
    return QLMB_OK;
}

extern "C" int qlmb_render(float *P, const int8_t *d, const float *s, const qlmb_span *sp, int nspan,
                           int group, int packed, int gi_base, int ng, void *stream)
{
    QLMB_REQUIRE(P && d && s && sp && nspan > 0, "qlmb_render: NULL argument");
    QLMB_REQUIRE(group >= 32 && group <= 256, "qlmb_render: group %d", group);
    if (ng <= 0) return QLMB_OK;
    k_render<<<(ng + 7) / 8, 256, 0, as_stream(stream)>>>(P, d, s, sp, nspan, group, packed, gi_base, ng);
    QLMB_LAUNCH_CHECK("k_render");
    return QLMB_OK;
}

// the count of skipped step launches lives behind the per-device error word (ints 8..9 of its 16)
static unsigned long long *skip_counter(void)
{
    int *w = device_error_word();
    return w ? reinterpret_cast<unsigned long long *>(w + 8) : nullptr;
}
extern "C" int qlmb_skipped_steps(unsigned long long *count, int reset, void *stream)
{
    QLMB_REQUIRE(count, "qlmb_skipped_steps: NULL argument");
    unsigned long long *c = skip_counter();
    if (!c) return cuda_fail(cudaGetLastError(), "device_error_word");
    QLMB_CUDA(cudaMemcpyAsync(count, c, sizeof *count, cudaMemcpyDeviceToHost, as_stream(stream)));
    QLMB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    if (reset) QLMB_CUDA(cudaMemsetAsync(c, 0, sizeof *c, as_stream(stream)));
    return QLMB_OK;
}

// QLM_V4 is a process-wide switch in the reference too (device global d_qv4, set from the environment by
// qlm_v4_init, qlm.cuh:68-72)
static int g_qv4 = 0;
extern "C" int qlmb_set_v4(int on) { g_qv4 = on ? 1 : 0; return QLMB_OK; }

extern "C" int qlmb_step(float *P, const float *G, int8_t *d, int8_t *r, const float *s, int8_t *m8,
                         float *m8s, uint8_t *v8, float *v8s, const qlmb_span *sp, int nspan,
                         int group, int dmax, float lr, float b1, float b2, float wd, float gscale,
                         const float *gsp, float inv_bc1, float inv_sqrt_bc2, int lrmode, uint64_t t,
                         int adam, int64_t *stat, int packed, int gi_base, int ng, void *stream)
{
    QLMB_REQUIRE(G && d && r && s && m8 && m8s && sp && nspan > 0, "qlmb_step: NULL argument");
    QLMB_REQUIRE(!adam || (v8 && v8s), "qlmb_step: adam needs v8 and v8s");
    QLMB_REQUIRE(group >= 32 && group <= 256 && (!packed || (group % 2) == 0), "qlmb_step: group %d", group);
    QLMB_REQUIRE(dmax >= 1 && dmax <= 127 && (!packed || dmax <= 7), "qlmb_step: dmax %d", dmax);
    if (ng <= 0) return QLMB_OK;
    StepArgs a = {P, G, d, r, s, m8, m8s, v8, v8s, sp, nspan, group, dmax, lr, b1, b2, wd, gscale, gsp,
                  inv_bc1, inv_sqrt_bc2, lrmode, t, adam, (unsigned long long *)stat, packed, gi_base, ng, g_qv4, nullptr, nullptr,
                  skip_counter(), {}, 0, 1.0f};
    auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    bool fast = group == 128 && packed && adam && !stat && !g_qv4 && al16(G) && al16(d) && al16(r) && al16(m8) &&
                al16(v8) && (!P || al16(P));
    cudaStream_t st = as_stream(stream);
    static int impl = -1;
    if (impl < 0) { const char *e = getenv("QLMB_STEP_IMPL"); impl = (e && !strcmp(e, "scalar")) ? 0 : 1; }
    if (fast && impl == 1) {
        // the packed form (two-wide fp32 instructions, reciprocal divisions); QLMB_STEP_IMPL=scalar keeps the older kernels
        unsigned nb = (unsigned)((ng + 15) / 16);
        if (P) k_step_pk<true><<<nb, 256, 0, st>>>(a); else k_step_pk<false><<<nb, 256, 0, st>>>(a);
    } else if (fast) {
        // elements per lane: 8 by default (measured fastest); QLMB_STEP_EPL=4|16 selects the other forms
        static int epl = 0;
        if (!epl) { const char *e = getenv("QLMB_STEP_EPL"); epl = e ? atoi(e) : 8; if (epl != 4 && epl != 16) epl = 8; }
        unsigned gpb = 8u * (unsigned)(epl / 4);          // groups per block
        unsigned nb = (unsigned)((ng + gpb - 1) / gpb);
        if (epl == 4) { if (P) k_step_fast<true, 4><<<nb, 256, 0, st>>>(a); else k_step_fast<false, 4><<<nb, 256, 0, st>>>(a); }
        else if (epl == 8) { if (P) k_step_fast<true, 8><<<nb, 256, 0, st>>>(a); else k_step_fast<false, 8><<<nb, 256, 0, st>>>(a); }
        else { if (P) k_step_fast<true, 16><<<nb, 256, 0, st>>>(a); else k_step_fast<false, 16><<<nb, 256, 0, st>>>(a); }
    } else {
        k_step_generic<<<(ng + 7) / 8, 256, 0, st>>>(a);
    }
    QLMB_LAUNCH_CHECK("k_step");
    return QLMB_OK;
}

extern "C" int qlmb_servo(int8_t *d, int8_t *r, float *s, const qlmb_span *sp, int nspan, int ngrp,
                          int group, int dmax, float f_hi, float f_lo, int packed, void *stream)
{
    QLMB_REQUIRE(d && r && s && sp && nspan > 0, "qlmb_servo: NULL argument");
    QLMB_REQUIRE(group >= 32 && group <= 256 && (!packed || (group % 2) == 0), "qlmb_servo: group %d", group);
    if (ngrp <= 0) return QLMB_OK;
    k_servo<<<(ngrp + 7) / 8, 256, 0, as_stream(stream)>>>(d, r, s, sp, nspan, ngrp, group, dmax, f_hi, f_lo, packed);
    QLMB_LAUNCH_CHECK("k_servo");
    return QLMB_OK;
}

extern "C" int qlmb_gnorm(const float *G, size_t n, const float *const *side, const size_t *side_n,
                          int nside, int clip_side, float *gs, void *stream)
{
    QLMB_REQUIRE(G && gs && nside >= 0 && nside <= 62, "qlmb_gnorm: bad argument");
    QLMB_REQUIRE(nside == 0 || (side && side_n), "qlmb_gnorm: side arrays missing");
    int dev = 0;
    QLMB_CUDA(cudaGetDevice(&dev));
    QLMB_REQUIRE(dev >= 0 && dev < 64, "qlmb_gnorm: device index %d", dev);
    size_t need = (size_t)64 * (1 + nside) * GN_SUB;
    if (g_gn_cap[dev] < need) {
        if (g_gn_scratch[dev]) QLMB_CUDA(cudaFree(g_gn_scratch[dev]));
        g_gn_scratch[dev] = nullptr; g_gn_cap[dev] = 0;
        QLMB_CUDA(cudaMalloc(&g_gn_scratch[dev], need * sizeof(double)));
        g_gn_cap[dev] = need;
    }
    double *sub = g_gn_scratch[dev];
    cudaStream_t st = as_stream(stream);
    k_sq_partial<<<dim3(GN_SUB, 64), 256, 0, st>>>(G, n, sub);
    for (int i = 0; i < nside; i++)
        k_sq_partial<<<dim3(GN_SUB, 64), 256, 0, st>>>(side[i], side_n[i], sub + (size_t)64 * GN_SUB * (1 + i));
    k_gnorm_final<<<1, 1, 0, st>>>(sub, nside, clip_side, gs);
    QLMB_LAUNCH_CHECK("k_gnorm");
    return QLMB_OK;
}

extern "C" int qlmb_adamw(float *P, const float *G, uint16_t *M, uint16_t *V, size_t n, float lr,
                          float b1, float b2, float wd, float bc1, float bc2, const float *gs,
                          void *stream)
{
    QLMB_REQUIRE(P && G && M && V, "qlmb_adamw: NULL argument");
    if (n == 0) return QLMB_OK;
    k_adamw_bf16<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(P, G, M, V, n, lr, b1, b2, wd, bc1, bc2, gs);
    QLMB_LAUNCH_CHECK("k_adamw");
    return QLMB_OK;
}

// ------------------------------------------------- grad-norm clip without allocation
// Some hosts cannot let a library allocate device memory: a training job that
// has handed every spare byte to its own pool, or a serving loop that must not
// meet the device-wide synchronisation cudaMalloc/cudaFree imply in the middle
// of a step.  For them the partial sums of the norm live in this fixed array,
// which exists once per GPU from the moment the library is loaded until the
// process ends: 64 chunks x 16 sub-blocks x (1 gradient + up to 7 side buffers)
// doubles = 64 KiB.
#define QLMB_NOALLOC_MAX_SIDES 7
static __device__ __align__(256) double g_gnorm_static_partials[64 * GN_SUB * (1 + QLMB_NOALLOC_MAX_SIDES)];
// The array's name is only a handle on the host; the kernels need its device
// address, looked up once per device (with that device current) and kept here.
static double *g_gnorm_static_addr[64];

// Same result as qlmb_gnorm, with no cudaMalloc/cudaFree and no other allocating
// call on any path.  The first call on each device resolves the address of the
// static array; make that call before starting any stream capture.  All calls on
// a device share the one array: two calls whose kernels may overlap on the GPU
// (different streams, no ordering between them) race on it.  Nothing in it has to
// be cleared beforehand: every slot the final kernel reads is written earlier in
// the same call, so what an earlier call left behind is never seen.
extern "C" int qlmb_gnorm_noalloc(const float *G, size_t n, const float *const *side, const size_t *side_n,
                                  int nside, int clip_side, float *gs, void *stream)
{
    QLMB_REQUIRE(G && gs && nside >= 0, "qlmb_gnorm_noalloc: bad argument");
    QLMB_REQUIRE(nside == 0 || (side && side_n), "qlmb_gnorm_noalloc: side arrays missing");
    if (nside > QLMB_NOALLOC_MAX_SIDES) {
        set_error("qlmb_gnorm_noalloc: %d side buffers exceed the fixed scratch (at most %d; use qlmb_gnorm for more)",
                  nside, QLMB_NOALLOC_MAX_SIDES);
        return QLMB_E_ARG;
    }
    int dev = 0;
    QLMB_CUDA(cudaGetDevice(&dev));
    QLMB_REQUIRE(dev >= 0 && dev < 64, "qlmb_gnorm_noalloc: device index %d", dev);
    if (!g_gnorm_static_addr[dev]) {
        double *p = nullptr;
        QLMB_CUDA(cudaGetSymbolAddress((void **)&p, g_gnorm_static_partials));
        g_gnorm_static_addr[dev] = p;
    }
    double *sub = g_gnorm_static_addr[dev];
    cudaStream_t st = as_stream(stream);
    k_sq_partial<<<dim3(GN_SUB, 64), 256, 0, st>>>(G, n, sub);
    for (int i = 0; i < nside; i++)
        k_sq_partial<<<dim3(GN_SUB, 64), 256, 0, st>>>(side[i], side_n[i], sub + (size_t)64 * GN_SUB * (1 + i));
    k_gnorm_final<<<1, 1, 0, st>>>(sub, nside, clip_side, gs);
    QLMB_LAUNCH_CHECK("qlmb_gnorm_noalloc");
    return QLMB_OK;
}

// ------------------------------------------------- fused per-layer update: the norm in slices
static __device__ __align__(256) double g_sqsum_static_partials[64 * GN_SUB];
static double *g_sqsum_static_addr[64];

extern "C" int qlmb_sqsum(const float *G, size_t n, float *part64, void *stream)
{
    QLMB_REQUIRE(G && part64, "qlmb_sqsum: NULL argument");
    int dev = 0;
    QLMB_CUDA(cudaGetDevice(&dev));
    QLMB_REQUIRE(dev >= 0 && dev < 64, "qlmb_sqsum: device index %d", dev);
    if (!g_sqsum_static_addr[dev]) {
        double *p = nullptr;
        QLMB_CUDA(cudaGetSymbolAddress((void **)&p, g_sqsum_static_partials));
        g_sqsum_static_addr[dev] = p;
    }
    cudaStream_t st = as_stream(stream);
    k_sq_partial<<<dim3(GN_SUB, 64), 256, 0, st>>>(G, n, g_sqsum_static_addr[dev]);
    k_sq_fold<<<1, 64, 0, st>>>(g_sqsum_static_addr[dev], part64);
    QLMB_LAUNCH_CHECK("qlmb_sqsum");
    return QLMB_OK;
}

extern "C" int qlmb_gnorm_close(const float *part, int nslice, float *gs, void *stream)
{
    QLMB_REQUIRE(part && gs && nslice > 0, "qlmb_gnorm_close: bad argument");
    k_gnorm_close<<<1, 1, 0, as_stream(stream)>>>(part, 64 * nslice, gs);
    QLMB_LAUNCH_CHECK("qlmb_gnorm_close");
    return QLMB_OK;
}

// ------------------------------------------------- 4-bit n-gram / engram table: sparse integer AdamW
extern "C" int qlmb_ng_touched(int *tgi, int *count, int *flag, const int *key, int NK, int De, int group, int ngrp,
                               void *stream)
{
    QLMB_REQUIRE(tgi && count && flag && key, "qlmb_ng_touched: NULL argument");
    QLMB_REQUIRE(NK >= 0 && De > 0 && group > 0 && group % De == 0 && ngrp > 0, "qlmb_ng_touched: NK %d De %d group %d ngrp %d", NK, De, group, ngrp);
    cudaStream_t st = as_stream(stream);
    if (NK > 0) k_ng_mark<<<(NK + 255) / 256, 256, 0, st>>>(flag, key, NK, De, group);
    k_ng_compact<<<1, 1024, 0, st>>>(tgi, count, flag, ngrp);
    QLMB_LAUNCH_CHECK("qlmb_ng_touched");
    return QLMB_OK;
}

extern "C" int qlmb_ng_scatter_compact(float *Gc, const int *key, const int *tgi, const int *count, const float *dbuf,
                                       int NK, int De, int group, int Nd, int max_touched, void *stream)
{
    QLMB_REQUIRE(Gc && key && tgi && count && dbuf, "qlmb_ng_scatter_compact: NULL argument");
    QLMB_REQUIRE(De > 0 && De <= 256 && group > 0 && group % De == 0 && Nd > 0 && max_touched >= 0, "qlmb_ng_scatter_compact: De %d group %d", De, group);
    if (max_touched == 0 || NK <= 0) return QLMB_OK;
    const long long warps = (long long)max_touched * (group / De);
    k_ng_scatter_compact<<<(unsigned)((warps + 7) / 8), 256, 0, as_stream(stream)>>>(Gc, key, tgi, count, dbuf, NK, De, group, Nd, De, 0);
    QLMB_LAUNCH_CHECK("k_ng_scatter_compact");
    return QLMB_OK;
}

// ---- sparse engram: S hashed sub-tables inside the one 4-bit table (cudalm.cu:4963-5098, CPU twins cpu_kern.h:665-688)
// k_eg_key: key s*N + n = row of sub-table s for the last ord[s] token ids at position n (-1 without enough history)
__global__ void __launch_bounds__(256) k_eg_key(int *key, const int *tok, const unsigned short *canon, const int *ord, const int *prime,
                                                const unsigned long long *mult, int N, int T, int S, int Rp)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)S * N) return;
    const int sidx = (int)(i / N), n = (int)(i % N), o = ord[sidx];
    if (n % T < o - 1) { key[i] = -1; return; }
    unsigned long long m = 0;
    for (int k = 0; k < o; k++) {
        unsigned t = (unsigned)tok[n - k];
        if (canon) t = canon[t];
        m ^= (unsigned long long)t * mult[sidx * 4 + k];
    }
    key[i] = (int)(m % (unsigned long long)prime[sidx]) + sidx * Rp;
}
// k_eg_gather: buf[n][s][:] = table row key[s*N + n] (zeros where the key is -1)
__global__ void __launch_bounds__(256) k_eg_gather(float *buf, const float *tbl, const int *key, int N, int S, int De)
{
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x, SD = (size_t)S * De;
    if (i >= (size_t)N * SD) return;
    const int n = (int)(i / SD), r = (int)(i % SD), sidx = r / De, e = r % De, k = key[(size_t)sidx * N + n];
    buf[i] = k >= 0 ? tbl[(size_t)k * De + e] : 0.0f;
}
extern "C" int qlmb_eg_key(int *key, const int *tok, const unsigned short *canon, const int *ord, const int *prime,
                           const unsigned long long *mult, int N, int T, int S, int Rp, void *stream)
{
    QLMB_REQUIRE(key && tok && ord && prime && mult, "qlmb_eg_key: NULL argument");
    QLMB_REQUIRE(N > 0 && T > 0 && S > 0 && S <= 32 && Rp > 0, "qlmb_eg_key: N %d T %d S %d Rp %d", N, T, S, Rp);
    k_eg_key<<<(unsigned)(((long long)S * N + 255) / 256), 256, 0, as_stream(stream)>>>(key, tok, canon, ord, prime, mult, N, T, S, Rp);
    QLMB_LAUNCH_CHECK("k_eg_key");
    return QLMB_OK;
}
extern "C" int qlmb_eg_gather(float *buf, const float *tbl, const int *key, int N, int S, int De, void *stream)
{
    QLMB_REQUIRE(buf && tbl && key && N > 0 && S > 0 && De > 0, "qlmb_eg_gather: bad argument");
    k_eg_gather<<<(unsigned)(((size_t)N * S * De + 255) / 256), 256, 0, as_stream(stream)>>>(buf, tbl, key, N, S, De);
    QLMB_LAUNCH_CHECK("k_eg_gather");
    return QLMB_OK;
}
// k_eg_scatter_c: the compact gradient rows of the touched groups from db [N][S][De]; per element the positions are added
// in ascending order (the reference's CPU build; its GPU kernel uses float atomics)
extern "C" int qlmb_eg_scatter_compact(float *Gc, const int *key, const int *tgi, const int *count, const float *db, int N, int S,
                                       int De, int group, int max_touched, void *stream)
{
    QLMB_REQUIRE(Gc && key && tgi && count && db, "qlmb_eg_scatter_compact: NULL argument");
    QLMB_REQUIRE(N > 0 && S > 0 && De > 0 && De <= 256 && group > 0 && group % De == 0 && max_touched >= 0, "qlmb_eg_scatter_compact: N %d S %d De %d group %d", N, S, De, group);
    if (max_touched == 0) return QLMB_OK;
    const long long warps = (long long)max_touched * (group / De);
    k_ng_scatter_compact<<<(unsigned)((warps + 7) / 8), 256, 0, as_stream(stream)>>>(Gc, key, tgi, count, db, S * N, De, group, N, S * De, De);
    QLMB_LAUNCH_CHECK("qlmb_eg_scatter_compact");
    return QLMB_OK;
}

extern "C" int qlmb_ng_step(float *P, const float *Gc, int8_t *d, int8_t *r, const float *s, int8_t *m8, float *m8s,
                            uint8_t *v8, float *v8s, const int *tgi, const int *count, int max_touched, int group,
                            int dmax, float lr, float b1, float b2, float wd, float sref, float inv_bc1,
                            float inv_sqrt_bc2, uint64_t t, uint64_t nt, const float *gs, void *stream)
{
    QLMB_REQUIRE(Gc && d && r && s && m8 && m8s && v8 && v8s && tgi && count, "qlmb_ng_step: NULL argument");
    QLMB_REQUIRE(group >= 32 && group <= 256 && (group % 2) == 0 && dmax >= 1 && dmax <= 7 && nt > 0, "qlmb_ng_step: group %d dmax %d", group, dmax);
    if (max_touched <= 0) return QLMB_OK;
    // the table is one packed span that starts at element 0 (ngram_q4_setup, cudalm.cu:4541-4543); it travels in the
    // launch arguments, so tables stepped on different streams share nothing and the call can be captured
    qlmb_span h;
    memset(&h, 0, sizeof h);
    h.pof = 0; h.gof = 0; h.qi0 = 0; h.n = nt; h.gi0 = 0; h.ngrp = (int)((nt + group - 1) / group); h.sref = sref;
    cudaStream_t st = as_stream(stream);
    StepArgs a = {P, Gc, d, r, s, m8, m8s, v8, v8s, nullptr, 1, group, dmax, lr, b1, b2, wd, 1.0f, gs,
                  inv_bc1, inv_sqrt_bc2, 0, t, 1, nullptr, 1, 0, max_touched, g_qv4, tgi, count, skip_counter(), h, 1, 1.0f};
    k_step_generic<<<(max_touched + 7) / 8, 256, 0, st>>>(a);
    QLMB_LAUNCH_CHECK("qlmb_ng_step");
    return QLMB_OK;
}
