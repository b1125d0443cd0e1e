// Decode path: Y[B,N] = X[B,K] * deq(W) for B <= 64 live slots (the reference's
// dec_step calls g_ab with M = slots on the rendered fp32 weights,
// cudalm.cu:7178-7198).  Weight streaming kernels: every code byte is read once
// from HBM per call, activations sit in shared memory, accumulation is fp32.
// Results do not depend on scheduling: partial sums are combined in a fixed order.
#include <stdlib.h>
#include "qlmb_common.cuh"
#include "qlmb_internal.h"

namespace qlmb {

int workspace(size_t bytes, void **out);       // qlmb_linear.cu


__device__ __forceinline__ float ld_x(const void *X, int dtype, size_t i)
{
    return dtype == QLMB_BF16 ? __bfloat162float(((const bf16 *)X)[i]) : ((const float *)X)[i];
}
// eight nibbles of a code word as exact floats (two's complement, element 0 in the low nibble):
// byte b in 0..15 under the exponent of 2^23 is 8388608 + b; (nibble ^ 8) - 8 is the value.
__device__ __forceinline__ void unpack8(uint32_t w, float d[8])
{
    w ^= 0x88888888u;
    uint32_t ev = w & 0x0F0F0F0Fu, od = (w >> 4) & 0x0F0F0F0Fu;
    const uint32_t magic = 0x4B000000u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        d[2 * i] = __uint_as_float(__byte_perm(ev, magic, 0x7440 + i)) - 8388616.0f;
        d[2 * i + 1] = __uint_as_float(__byte_perm(od, magic, 0x7440 + i)) - 8388616.0f;
    }
}

// ---- codes W[K][N] (groups along N).  Block: 256 output columns x a K slice; warp w takes rows
// k0+w, k0+w+8, ..., eight of them in flight per step; lane = 8 consecutive columns (one code word).
// BT activation rows are multiplied per pass (BT = 1, 2, 4 or 8: no arithmetic on absent rows);
// part[ks][b][n] receives the slice sums.
// NB batches of four rows in flight per lane: 2 (four blocks per SM for up to two rows) when the grid fills the device,
// 4 (two blocks per SM) for the small grids of a decode step, where the latency of each round of loads is what counts
template <int BT, int NB = 2>
__global__ void __launch_bounds__(256, NB == 4 ? 2 : (BT <= 2 ? 4 : 2)) k_gemv_kn(float *part, const void *X, int dtype, const uint8_t *codes,
                                                 const float *scales, int B, int K, int N, int kslice,
                                                 const int *row_expert = nullptr, size_t e_codes = 0, size_t e_scales = 0,
                                                 int ntok = 1, const float *gamma = nullptr, int dual_rows = 0,
                                                 const uint8_t *codes2 = nullptr, const float *scales2 = nullptr)
{
    pdl_trigger();
    if (row_expert) pdl_wait();                 // the expert choice is the work of a kernel before this one
    // routed form: blockIdx.z is an output row, it reads activation row z % ntok and one matrix of a stack; B must be 1 then
    size_t xrow = 0, prow = 0;
    int PB = B;
    if (e_codes) {
        // the matrix of a row: looked up (experts of a step), or z / ntok for a stack of matrices applied to the same ntok rows
        // dual_rows: rows dual_rows.. repeat the first dual_rows rows on a second stack of matrices (gate and up of an expert)
        int zr = blockIdx.z;
        if (dual_rows && zr >= dual_rows) { zr -= dual_rows; codes = codes2; scales = scales2; }
        const int e = row_expert ? row_expert[zr] : zr / ntok;
        codes += (size_t)e * e_codes; scales += (size_t)e * e_scales;
        xrow = zr % ntok; prow = blockIdx.z; PB = gridDim.z;
    }
    extern __shared__ float xs[];               // [BT][kslice]
    constexpr bool PAR = BT <= 2;               // every warp parks its sums, one pass adds them in warp order
    __shared__ float red[PAR ? 8 * BT : BT][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 256 + lane * 8;
    const int k0 = blockIdx.y * kslice, k1 = k0 + kslice < K ? k0 + kslice : K;
    const int gpr = N / 128;
    const bool live = n0 < N;
    const uint8_t *cp = codes + (size_t)n0 / 2;
    const float *sp = scales + n0 / 128;
    // four rows per batch (k, k+8, k+16, k+24), NB batches in flight; the first NB are requested before the
    // activations are staged (the weights do not depend on them)
    uint32_t w[NB][4];
    float sc[NB][4];
    auto fetch = [&](int buf, int k) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int kk = k + 8 * u;
            w[buf][u] = 0u; sc[buf][u] = 0.0f;
            if (kk < k1) {
                w[buf][u] = __ldcs(reinterpret_cast<const uint32_t *>(cp + (size_t)kk * N / 2));
                sc[buf][u] = __ldg(sp + (size_t)kk * gpr);
            }
        }
    };
    if (live) {
#pragma unroll
        for (int u = 0; u < NB; u++) fetch(u, k0 + warp + 32 * u);
    }
    if (!row_expert) pdl_wait();                // the weights above do not depend on the kernels before; the rows below do
    // gamma (routed form, one activation row per block): the row is normalised on the way in, x * rinv * gamma rounded
    // to bf16 as the separate norm kernel stores it (e_rmsf in front of the q, k, v projections, cudalm.cu:7176)
    float rinv = 1.0f;
    if (gamma) {
        float ss = 0.0f;
        for (int k = threadIdx.x; k < K; k += 256) { const float x = ld_x(X, dtype, xrow * K + k); ss += x * x; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[0][warp] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < 8; w8++) tot += red[0][w8];
        rinv = 1.0f / sqrtf(tot / (float)K + 1e-5f);
    }
    for (int b0 = 0; b0 < B; b0 += BT) {
        __syncthreads();
        for (int i = threadIdx.x; i < BT * kslice; i += 256) {
            const int b = b0 + i / kslice, k = k0 + i % kslice;
            float x = (b < B && k < k1) ? ld_x(X, dtype, ((size_t)b + xrow) * K + k) : 0.0f;
            if (gamma && k < k1) x = __bfloat162float(__float2bfloat16_rn(x * rinv * gamma[k]));
            xs[i] = x;
        }
        if (!PAR) for (int i = threadIdx.x; i < BT * 256; i += 256) red[i / 256][i % 256] = 0.0f;
        __syncthreads();
        float acc[BT][8];
#pragma unroll
        for (int b = 0; b < BT; b++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[b][j] = 0.0f;
        if (live) {
            auto use = [&](int buf, int k) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int kk = k + 8 * u;
                    if (kk < k1) {
                        float d[8];
                        unpack8(w[buf][u], d);
#pragma unroll
                        for (int b = 0; b < BT; b++) {
                            const float xv = xs[b * kslice + (kk - k0)] * sc[buf][u];
#pragma unroll
                            for (int j = 0; j < 8; j++) acc[b][j] += xv * d[j];
                        }
                    }
                }
            };
            int k = k0 + warp;
            if (b0 > 0) {
#pragma unroll
                for (int u = 0; u < NB; u++) fetch(u, k + 32 * u);
            }
            for (; k < k1; k += 32 * NB) {
#pragma unroll
                for (int u = 0; u < NB; u++) { use(u, k + 32 * u); fetch(u, k + 32 * u + 32 * NB); }
            }
        }
        // fixed-order combination of the 8 warps
        if (PAR) {
#pragma unroll
            for (int b = 0; b < BT; b++)
#pragma unroll
                for (int j = 0; j < 8; j++) red[warp * BT + b][lane * 8 + j] = acc[b][j];
            __syncthreads();
            for (int i = threadIdx.x; i < BT * 256; i += 256) {
                const int bb = i / 256, c = i % 256, b = b0 + bb, n = blockIdx.x * 256 + c;
                float v = 0.0f;
#pragma unroll
                for (int w8 = 0; w8 < 8; w8++) v += red[w8 * BT + bb][c];
                if (b < B && n < N) part[((size_t)blockIdx.y * PB + b + prow) * N + n] = v;
            }
        } else {
            for (int w8 = 0; w8 < 8; w8++) {
                if (warp == w8 && live) {
#pragma unroll
                    for (int b = 0; b < BT; b++)
#pragma unroll
                        for (int j = 0; j < 8; j++) red[b][lane * 8 + j] += acc[b][j];
                }
                __syncthreads();
            }
            for (int i = threadIdx.x; i < BT * 256; i += 256) {
                const int b = b0 + i / 256, n = blockIdx.x * 256 + i % 256;
                if (b < B && n < N) part[((size_t)blockIdx.y * PB + b + prow) * N + n] = red[i / 256][i % 256];
            }
        }
    }
}

// k_gemv_kn as a programmatic dependent launch, with the kernel's default arguments
template <int BT, int NB>
static cudaError_t launch_kn(bool early, dim3 grid, size_t smem, cudaStream_t st, float *part, const void *X, int dtype, const uint8_t *codes,
                             const float *scales, int B, int K, int N, int kslice, const int *row_expert = nullptr,
                             size_t e_codes = 0, size_t e_scales = 0, int ntok = 1, const float *gamma = nullptr,
                             int dual_rows = 0, const uint8_t *codes2 = nullptr, const float *scales2 = nullptr)
{
    return pdl_launch(early, k_gemv_kn<BT, NB>, grid, dim3(256), smem, st, part, X, dtype, codes, scales, B, K, N, kslice, row_expert,
                      e_codes, e_scales, ntok, gamma, dual_rows, codes2, scales2);
}

// ---- streaming form for codes W[K][N] and up to four activation rows: the whole product in one launch.
// Block = 32 * CPL output columns (a lane owns CPL = 8 or 16 consecutive columns, one 4- or 8-byte load per row, so a
// lane's columns share a scale group) x a K slice; warp w takes rows k0 + w, k0 + w + 8, ..., eight of them
// requested ahead of the eight being multiplied.  The eight warps' sums are combined by a fixed tree in shared
// memory; with several K slices every block leaves its sums in `part`, takes a ticket for its column block, and the
// block that draws the last ticket adds the slices in ascending order and writes Y (no second launch, and the order
// of the additions does not depend on which block came last).
// Nibbles become floats without a conversion and with few integer-pipe instructions: one three-input logic
// operation turns two nibbles i and i+4 of a code word into the two bf16 patterns of 136 + d (as the GEMM engine's
// expansion does); read as ONE fp32 that word is 136 + d_hi + (0x4308 + d_lo) / 65536, and shifted left by 16 it is
// 136 + d_lo exactly.  Both are multiplied as they are; the constants and the small cross term are taken out of the
// finished sums with the sum of the multipliers: y_lo = acc_lo - 136 S, y_hi = acc_hi - (136 + 0x4308 / 65536) S -
// y_lo / 65536, S = sum over the rows of x * scale.  The shift is written as a multiply by a run-time 65536 so that
// it runs on the multiply-add pipe rather than on the half-rate integer pipe.
__device__ unsigned g_gemv_ticket[2048];

__device__ __forceinline__ uint32_t nib_pair_f(uint32_t w)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43084308, 0x6A;" : "=r"(r) : "r"(w));
    return r;
}

template <int BT, int CPL, int U = 4>
__global__ void __launch_bounds__(256, BT <= 2 ? 3 : 2) k_gemv_stream(void *Y, int dtype, float *part, const void *X, const uint8_t *codes,
                                                     const float *scales, int B, int K, int N, int kslice, uint32_t k65536)
{
    // kslice is a multiple of 64 that divides K: every warp owns kslice / 8 rows, a whole number of batches
    constexpr int WPL = CPL / 8, CW = 32 * CPL;
    extern __shared__ float gsm[];                       // activations [BT][kslice]; later the reduction tree [4][BT][CW]
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n0 = blockIdx.x * CW + lane * CPL;
    const bool live = n0 < N;
    if (!live) n0 = N - CPL;                             // lanes past the last column repeat valid loads and store nothing
    const int k0 = blockIdx.y * kslice;
    const size_t cstep = (size_t)8 * (N / 2), sstep = (size_t)8 * (N / 128);
    const uint8_t *cp = codes + (size_t)(k0 + warp) * (N / 2) + n0 / 2;
    const float *sp = scales + (size_t)(k0 + warp) * (N / 128) + n0 / 128;
    uint32_t w[2][U][WPL];
    float sc[2][U];
    auto fetch = [&](int buf) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (WPL == 2) { const uint2 t = __ldcs(reinterpret_cast<const uint2 *>(cp)); w[buf][u][0] = t.x; w[buf][u][WPL - 1] = t.y; }
            else w[buf][u][0] = __ldcs(reinterpret_cast<const uint32_t *>(cp));
            sc[buf][u] = __ldg(sp);
            cp += cstep; sp += sstep;
        }
    };
    fetch(0);                                            // the weights do not depend on the activations: request them first
    for (int i = threadIdx.x; i < BT * kslice; i += 256) {
        const int b = i / kslice, k = k0 + i % kslice;
        gsm[i] = b < B ? ld_x(X, dtype, (size_t)b * K + k) : 0.0f;
    }
    __syncthreads();
    float acc[BT][CPL], s0[BT];
#pragma unroll
    for (int b = 0; b < BT; b++) {
        s0[b] = 0.0f;
#pragma unroll
        for (int j = 0; j < CPL; j++) acc[b][j] = 0.0f;
    }
    const float *xr = gsm + warp;                        // this warp's activation of the batch's first row
    auto use = [&](int buf) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            float xv[BT];
#pragma unroll
            for (int b = 0; b < BT; b++) { xv[b] = xr[b * kslice + 8 * u] * sc[buf][u]; s0[b] += xv[b]; }
#pragma unroll
            for (int i = 0; i < WPL; i++) {
                const uint32_t ww = w[buf][u][i];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t qq = nib_pair_f(ww >> (4 * j));
                    const float vlo = __uint_as_float(qq * k65536), vhi = __uint_as_float(qq);
#pragma unroll
                    for (int b = 0; b < BT; b++) {
                        acc[b][8 * i + j] = fmaf(xv[b], vlo, acc[b][8 * i + j]);
                        acc[b][8 * i + j + 4] = fmaf(xv[b], vhi, acc[b][8 * i + j + 4]);
                    }
                }
            }
        }
        xr += 8 * U;
    };
    for (int r = 0; r < kslice / 8; r += 2 * U) {        // two batches per round: the buffer indices stay compile-time constants
        fetch(1);
        use(0);
        if (r + 2 * U < kslice / 8) fetch(0);
        use(1);
    }
    float y[BT][CPL];
#pragma unroll
    for (int b = 0; b < BT; b++)
#pragma unroll
        for (int i = 0; i < WPL; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float lo = acc[b][8 * i + j] - 136.0f * s0[b];
                y[b][8 * i + j] = lo;
                y[b][8 * i + j + 4] = acc[b][8 * i + j + 4] - 136.26184082031250f * s0[b] - lo * (1.0f / 65536.0f);
            }
    // the eight warps' sums: 4..7 -> 0..3, 2..3 -> 0..1, 1 -> 0 (fixed pairs)
    __syncthreads();                                     // the activations are no longer needed
    float *red = gsm;
#pragma unroll
    for (int half = 4; half >= 1; half >>= 1) {
        if (warp >= half && warp < 2 * half) {
#pragma unroll
            for (int b = 0; b < BT; b++)
#pragma unroll
                for (int c = 0; c < CPL; c++) red[((warp - half) * BT + b) * CW + c * 32 + lane] = y[b][c];
        }
        __syncthreads();
        if (warp < half) {
#pragma unroll
            for (int b = 0; b < BT; b++)
#pragma unroll
                for (int c = 0; c < CPL; c++) y[b][c] += red[(warp * BT + b) * CW + c * 32 + lane];
        }
        __syncthreads();
    }
    const int nslice = gridDim.y;
    if (warp == 0 && live) {
#pragma unroll
        for (int b = 0; b < BT; b++) {
            if (b >= B) break;
            if (nslice == 1) {
#pragma unroll
                for (int c = 0; c < CPL; c++) {
                    if (dtype == QLMB_BF16) ((bf16 *)Y)[(size_t)b * N + n0 + c] = __float2bfloat16_rn(y[b][c]);
                    else ((float *)Y)[(size_t)b * N + n0 + c] = y[b][c];
                }
            } else {
                float *dst = part + ((size_t)blockIdx.y * B + b) * N + n0;
#pragma unroll
                for (int c = 0; c < CPL; c += 4) __stcg(reinterpret_cast<float4 *>(dst + c), make_float4(y[b][c], y[b][c + 1], y[b][c + 2], y[b][c + 3]));
            }
        }
    }
    if (nslice == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&g_gemv_ticket[blockIdx.x], 1u) == (unsigned)(nslice - 1));
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < BT * CW; i += 256) {
        const int b = i / CW, n = blockIdx.x * CW + i % CW;
        if (b < B && n < N) {
            float v = 0.0f;
            for (int s = 0; s < nslice; s++) v += __ldcg(part + ((size_t)s * B + b) * N + n);
            if (dtype == QLMB_BF16) ((bf16 *)Y)[(size_t)b * N + n] = __float2bfloat16_rn(v);
            else ((float *)Y)[(size_t)b * N + n] = v;
        }
    }
    if (threadIdx.x == 0) g_gemv_ticket[blockIdx.x] = 0u;     // ready for the next call on this stream
}

// ---- up to 64 rows against one pass over the weights: groups of eight rows.
// A decode step with more than four live slots used to send every output row to its own blocks (each re-reading the
// matrix from L2) or, for the experts, through the 256-row tensor-core tiles (a few routed rows per expert in a
// 128-row tile).  Here a block owns 256 output columns x a K slice x a GROUP of up to eight rows that share a
// matrix: the weights are expanded once per group and multiplied with eight activation values (64 fp32 multiply-adds
// per code word), the same arithmetic as k_gemv_stream.  Two ways to form the groups:
//   dense   rows b of a batch B against a stack of nmat matrices of one shape (q, k, v; wo): group z = (m, g),
//           rows 8g .. 8g+7, output row m * B + b
//   routed  the K*N routed slots of a decode step sorted by expert (perm / off of the permutation kernel): expert e's
//           slots in groups of eight; a slot s reads activation row s % ntok (gate, up) or s (down) and writes
//           partial row s (+ R for the second stack of matrices: gate and up in one launch)
// part[ks][row][n] receives the slice sums; the finish kernels are the ones of the one-row path.

// Which rows does group blockIdx.z hold?  Dense: rows g*GR.. of matrix m.  Routed: the z-th group of GR slots in
// expert order (perm sorted by expert, off = expert offsets).  Run by warp 0: the lanes read the expert offsets
// side by side (one round of loads instead of one per expert), a shuffle scan finds the expert, then lane i reads slot i.
template <int GR>
__device__ __forceinline__ void group_lookup(const Rows8 &a, int lane, int *s_n, int *s_mat, int *s_x, int *s_o)
{
    int n = 0, mat = 0;
    if (!a.perm) {
        const int G = (a.B + GR - 1) / GR;
        const int m = blockIdx.z / G, gg = blockIdx.z % G;
        n = a.B - gg * GR < GR ? a.B - gg * GR : GR;
        mat = m;
        for (int i = lane; i < n; i += 32) { s_x[i] = gg * GR + i; s_o[i] = m * a.B + gg * GR + i; }
    } else {
        int z = blockIdx.z, second = 0;
        if (a.zdual && z >= a.zdual) { z -= a.zdual; second = 1; }
        int base_groups = 0, found = -1, first = 0, cnt = 0;
        for (int e0 = 0; e0 < a.E && found < 0; e0 += 32) {
            const int e = e0 + lane;
            const int o0 = e < a.E ? a.off[e] : 0, o1 = e < a.E ? a.off[e + 1] : 0;
            const int c = o1 - o0, ng = (c + GR - 1) / GR;
            int incl = ng;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += v; }
            const unsigned hit = __ballot_sync(0xffffffffu, z < base_groups + incl);
            if (hit) {
                const int l = __ffs(hit) - 1;
                const int excl = __shfl_sync(0xffffffffu, incl - ng, l);
                found = e0 + l;
                first = __shfl_sync(0xffffffffu, o0, l) + (z - base_groups - excl) * GR;
                cnt = __shfl_sync(0xffffffffu, o1, l) - first;
            }
            base_groups += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (found >= 0) {
            n = cnt < GR ? cnt : GR;
            mat = found | (second << 16);
            for (int i = lane; i < n; i += 32) {
                const int sl = a.perm[first + i];
                s_x[i] = a.x_by_token ? sl % a.ntok : sl;
                s_o[i] = sl + second * a.R;
            }
        }
    }
    if (lane == 0) { *s_n = n; *s_mat = mat; }
}

__global__ void __launch_bounds__(256, 2) k_gemv_rows8(const __grid_constant__ Rows8 a)
{
    constexpr int BT = 8, CPL = 8, CW = 256, U = 4;
    extern __shared__ float gsm[];                       // activations [BT][kslice]; later the reduction tree [4][BT][CW]
    __shared__ int s_n, s_mat, s_x[BT], s_o[BT];
    __shared__ float s_rinv[BT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kslice = a.kslice, K = a.K, N = a.N;
    pdl_trigger();
    if (a.perm) pdl_wait();                              // the slot order is the work of a kernel before this one
    if (warp == 0) group_lookup<BT>(a, lane, &s_n, &s_mat, s_x, s_o);
    __syncthreads();
    const int nrow = s_n;
    if (nrow == 0) { if (!a.perm) pdl_wait(); return; }
    const int mat = s_mat & 0xffff, second = s_mat >> 16;
    const uint8_t *codes = (second ? a.codes2 : a.codes) + (size_t)mat * a.e_codes;
    const float *scales = (second ? a.scales2 : a.scales) + (size_t)mat * a.e_scales;
    int n0 = blockIdx.x * CW + lane * CPL;
    const bool live = n0 < N;
    if (!live) n0 = N - CPL;
    const int k0 = blockIdx.y * kslice;
    const size_t cstep = (size_t)8 * (N / 2), sstep = (size_t)8 * (N / 128);
    const uint8_t *cp = codes + (size_t)(k0 + warp) * (N / 2) + n0 / 2;
    const float *sp = scales + (size_t)(k0 + warp) * (N / 128) + n0 / 128;
    uint32_t w[2][U];
    float sc[2][U];
    auto fetch = [&](int buf) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            w[buf][u] = __ldg(reinterpret_cast<const uint32_t *>(cp));
            sc[buf][u] = __ldg(sp);
            cp += cstep; sp += sstep;
        }
    };
    fetch(0);
    if (!a.perm) pdl_wait();                             // the weights above do not depend on the kernels before; the rows below do
    if (a.gamma) {                                       // warp w: 1 / rms of row w over the whole K
        if (warp < nrow) {
            float ss = 0.0f;
            for (int k = lane; k < K; k += 32) { const float x = ld_x(a.X, a.x_dtype, (size_t)s_x[warp] * K + k); ss += x * x; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) s_rinv[warp] = 1.0f / sqrtf(ss / (float)K + 1e-5f);
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < BT * kslice; i += 256) {
        const int b = i / kslice, k = k0 + i % kslice;
        float x = 0.0f;
        if (b < nrow) {
            x = ld_x(a.X, a.x_dtype, (size_t)s_x[b] * K + k);
            if (a.gamma) x = __bfloat162float(__float2bfloat16_rn(x * s_rinv[b] * a.gamma[k]));
        }
        gsm[i] = x;
    }
    __syncthreads();
    float acc[BT][CPL], s0[BT];
#pragma unroll
    for (int b = 0; b < BT; b++) {
        s0[b] = 0.0f;
#pragma unroll
        for (int j = 0; j < CPL; j++) acc[b][j] = 0.0f;
    }
    const float *xr = gsm + warp;
    const uint32_t k65536 = a.k65536;
    auto use = [&](int buf) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            float xv[BT];
#pragma unroll
            for (int b = 0; b < BT; b++) { xv[b] = xr[b * kslice + 8 * u] * sc[buf][u]; s0[b] += xv[b]; }
            const uint32_t ww = w[buf][u];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t qq = nib_pair_f(ww >> (4 * j));
                const float vlo = __uint_as_float(qq * k65536), vhi = __uint_as_float(qq);
#pragma unroll
                for (int b = 0; b < BT; b++) {
                    acc[b][j] = fmaf(xv[b], vlo, acc[b][j]);
                    acc[b][j + 4] = fmaf(xv[b], vhi, acc[b][j + 4]);
                }
            }
        }
        xr += 8 * U;
    };
    for (int r = 0; r < kslice / 8; r += 2 * U) {
        fetch(1);
        use(0);
        if (r + 2 * U < kslice / 8) fetch(0);
        use(1);
    }
#pragma unroll
    for (int b = 0; b < BT; b++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float lo = acc[b][j] - 136.0f * s0[b];
            acc[b][j] = lo;
            acc[b][j + 4] = acc[b][j + 4] - 136.26184082031250f * s0[b] - lo * (1.0f / 65536.0f);
        }
    __syncthreads();
    float *red = gsm;
#pragma unroll
    for (int half = 4; half >= 1; half >>= 1) {
        if (warp >= half && warp < 2 * half) {
#pragma unroll
            for (int b = 0; b < BT; b++)
#pragma unroll
                for (int c = 0; c < CPL; c++) red[((warp - half) * BT + b) * CW + c * 32 + lane] = acc[b][c];
        }
        __syncthreads();
        if (warp < half) {
#pragma unroll
            for (int b = 0; b < BT; b++)
#pragma unroll
                for (int c = 0; c < CPL; c++) acc[b][c] += red[(warp * BT + b) * CW + c * 32 + lane];
        }
        __syncthreads();
    }
    if (warp == 0 && live) {
#pragma unroll
        for (int b = 0; b < BT; b++) {
            if (b < nrow) {
                float *dst = a.part + ((size_t)blockIdx.y * a.rows_out + s_o[b]) * N + n0;
                *reinterpret_cast<float4 *>(dst) = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
                *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[b][4], acc[b][5], acc[b][6], acc[b][7]);
            }
        }
    }
}

// ---- the same groups with the multiplies on the warp-level tensor-core instruction (mma.sync m16n8k16, bf16 operands,
// fp32 accumulators), operands straight from registers.  k_gemv_rows8 spends 64 fp32 multiply-adds per code word
// on eight rows; here a group holds sixteen (or thirty-two) rows and a code word costs the expansion plus a quarter
// of eight MMAs.  tcgen05.mma takes its operands from shared memory, which for a kernel that streams every weight
// exactly once would add a store, a proxy fence and a barrier round trip per stage; the register form needs none.
// Warp = 64 output columns x the K slice; lane (g = lane / 4, t = lane % 4) loads the code word of columns 8g .. 8g+7
// for the rows 2t, 2t+1, 2t+8, 2t+9 of every 16-row step, expands it to exact bf16 digits (d = (136 + d) - 136),
// and pairs the rows with byte permutes into the B fragments of eight MMAs: MMA c uses column 8q + c of the tile
// for q = 0..7.  The group scale of a row (one per row for the 64 columns, which lie in one group of 128) multiplies
// the activations: A = bf16(x * bf16(s)), the rounding the GEMM engine applies to its rendered weights.
__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four registers of exact bf16 digit pairs (elements j and j + 4 of the word in register j)
__device__ __forceinline__ void digits_bf16(uint32_t w, uint32_t q[4])
{
    const uint32_t k136 = 0x43084308u;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t x = nib_pair_f(w >> (4 * j));
        __nv_bfloat162 v = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&x), *reinterpret_cast<const __nv_bfloat162 *>(&k136));
        q[j] = *reinterpret_cast<uint32_t *>(&v);
    }
}

template <int MT>
__global__ void __launch_bounds__(256, MT == 1 ? 2 : 1) k_gemv_mma(const __grid_constant__ Rows8 a)
{
    constexpr int GR = 16 * MT, CW = 512, PADK = 8;
    extern __shared__ __align__(16) uint8_t msm[];       // activations bf16 [GR][kslice + PADK], then scales [kslice][4]
    __shared__ int s_n, s_mat, s_x[GR], s_o[GR];
    __shared__ float s_rinv[GR];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kslice = a.kslice, K = a.K, N = a.N, ldx = kslice + PADK;
    bf16 *xs = reinterpret_cast<bf16 *>(msm);
    pdl_trigger();
    if (a.perm) pdl_wait();                              // the slot order is the work of a kernel before this one
    if (warp == 0) group_lookup<GR>(a, lane, &s_n, &s_mat, s_x, s_o);
    __syncthreads();
    const int nrow = s_n;
    if (nrow == 0) { if (!a.perm) pdl_wait(); return; }
    const int mat = s_mat & 0xffff, second = s_mat >> 16;
    const uint8_t *codes = (second ? a.codes2 : a.codes) + (size_t)mat * a.e_codes;
    const float *scales = (second ? a.scales2 : a.scales) + (size_t)mat * a.e_scales;
    const int c0 = blockIdx.x * CW + warp * 64;          // this warp's 64 columns
    const bool live = c0 < N;
    const int cc = live ? c0 : N - 64;
    const int k0 = blockIdx.y * kslice;
    const size_t crow = (size_t)(N / 2), srow = (size_t)(N / 128);
    // lane's rows of a step: 2t, 2t+1, 2t+8, 2t+9; four steps (sixteen code words) are kept in flight per lane
    const uint8_t *cp = codes + (size_t)(k0 + 2 * t) * crow + (cc + 8 * g) / 2;
    uint32_t w[4][4];
    auto fetch = [&](int slot) {
        w[slot][0] = __ldg(reinterpret_cast<const uint32_t *>(cp));
        w[slot][1] = __ldg(reinterpret_cast<const uint32_t *>(cp + crow));
        w[slot][2] = __ldg(reinterpret_cast<const uint32_t *>(cp + 8 * crow));
        w[slot][3] = __ldg(reinterpret_cast<const uint32_t *>(cp + 9 * crow));
        cp += 16 * crow;
    };
    const int steps = kslice / 16;                       // a multiple of four: kslice is a multiple of 64
#pragma unroll
    for (int u = 0; u < 4; u++) fetch(u);
    // the slice's group scales for the block's four column groups: [kslice][4] floats behind the activations
    float *ssc = reinterpret_cast<float *>(msm + (size_t)GR * ldx * sizeof(bf16));
    {
        const int g0 = blockIdx.x * (CW / 128), gmax = N / 128 - 1;
        if (g0 + 3 <= gmax && (srow & 3) == 0) {                  // four neighbouring scales of a row in one load
            for (int i = threadIdx.x; i < kslice; i += 256)
                reinterpret_cast<float4 *>(ssc)[i] = __ldg(reinterpret_cast<const float4 *>(scales + (size_t)(k0 + i) * srow + g0));
        } else {
            for (int i = threadIdx.x; i < kslice * 4; i += 256) {
                const int gq = g0 + (i & 3) < gmax ? g0 + (i & 3) : gmax;
                ssc[i] = __ldg(scales + (size_t)(k0 + (i >> 2)) * srow + gq);
            }
        }
    }
    if (!a.perm) pdl_wait();                             // codes and scales above do not depend on the kernels before; the rows below do
    const bool vec = a.x_dtype == QLMB_BF16;                     // bf16 rows are staged in 16-byte pieces, four loads in flight
    if (a.gamma) {                                       // 1 / rms of every row over the whole K: warp w takes rows w, w + 8, ...
        for (int r = warp; r < nrow; r += 8) {
            float ss = 0.0f;
            if (vec) {
                const uint4 *xr = reinterpret_cast<const uint4 *>(reinterpret_cast<const bf16 *>(a.X) + (size_t)s_x[r] * K);
                for (int kc = lane; kc < K / 8; kc += 32) {
                    const uint4 v = __ldg(xr + kc);
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
                    for (int j = 0; j < 4; j++) { const float2 f = __bfloat1622float2(h[j]); ss += f.x * f.x; ss += f.y * f.y; }
                }
            } else {
                for (int k = lane; k < K; k += 32) { const float x = ld_x(a.X, a.x_dtype, (size_t)s_x[r] * K + k); ss += x * x; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) s_rinv[r] = 1.0f / sqrtf(ss / (float)K + 1e-5f);
        }
        __syncthreads();
    }
    if (vec) {
        const int cpr = kslice / 8, total = GR * cpr;
        for (int i0 = threadIdx.x; i0 < total; i0 += 4 * 256) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int i = i0 + j * 256, b = i / cpr, kc = i - b * cpr;
                v[j] = make_uint4(0u, 0u, 0u, 0u);
                if (i < total && b < nrow)
                    v[j] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const bf16 *>(a.X) + (size_t)s_x[b] * K + k0 + kc * 8));
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int i = i0 + j * 256, b = i / cpr, kc = i - b * cpr;
                if (i >= total) continue;
                if (a.gamma && b < nrow) {
                    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&v[j]);
                    const float ri = s_rinv[b];
                    const float *gm = a.gamma + k0 + kc * 8;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float2 f = __bfloat1622float2(h[q]);
                        h[q] = __floats2bfloat162_rn(f.x * ri * gm[2 * q], f.y * ri * gm[2 * q + 1]);
                    }
                }
                *reinterpret_cast<uint4 *>(xs + b * ldx + kc * 8) = v[j];
            }
        }
    } else {
        for (int i = threadIdx.x; i < GR * kslice; i += 256) {
            const int b = i / kslice, kk = i % kslice;
            float x = 0.0f;
            if (b < nrow) {
                x = ld_x(a.X, a.x_dtype, (size_t)s_x[b] * K + k0 + kk);
                if (a.gamma) x = x * s_rinv[b] * a.gamma[k0 + kk];
            }
            xs[b * ldx + kk] = __float2bfloat16_rn(x);
        }
    }
    __syncthreads();
    float acc[MT][8][4];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int c = 0; c < 8; c++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[m][c][i] = 0.0f;
    const bf16 *xa = xs + g * ldx + 2 * t;               // A fragment of step 0: rows g, g + 8 (per 16-row tile), columns 2t.., 2t + 8..
    const float *sl = ssc + (2 * t) * 4 + (warp >> 1);   // scale of the lane's first row of step 0 for this warp's column group
    auto use = [&](int slot) {
        uint32_t q[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++) digits_bf16(w[slot][r], q[r]);
        const __nv_bfloat162 s01 = __floats2bfloat162_rn(sl[0], sl[4]), s23 = __floats2bfloat162_rn(sl[32], sl[36]);
        sl += 64;
        uint32_t af[MT][4];
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const bf16 *p = xa + m * 16 * ldx;
            __nv_bfloat162 a0 = *reinterpret_cast<const __nv_bfloat162 *>(p), a1 = *reinterpret_cast<const __nv_bfloat162 *>(p + 8 * ldx);
            __nv_bfloat162 a2 = *reinterpret_cast<const __nv_bfloat162 *>(p + 8), a3 = *reinterpret_cast<const __nv_bfloat162 *>(p + 8 * ldx + 8);
            a0 = __hmul2(a0, s01); a1 = __hmul2(a1, s01); a2 = __hmul2(a2, s23); a3 = __hmul2(a3, s23);
            af[m][0] = *reinterpret_cast<uint32_t *>(&a0); af[m][1] = *reinterpret_cast<uint32_t *>(&a1);
            af[m][2] = *reinterpret_cast<uint32_t *>(&a2); af[m][3] = *reinterpret_cast<uint32_t *>(&a3);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // column j: the low halves of rows (2t, 2t+1) and (2t+8, 2t+9); column j + 4: the high halves
            const uint32_t b0l = __byte_perm(q[0][j], q[1][j], 0x5410), b1l = __byte_perm(q[2][j], q[3][j], 0x5410);
            const uint32_t b0h = __byte_perm(q[0][j], q[1][j], 0x7632), b1h = __byte_perm(q[2][j], q[3][j], 0x7632);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                mma_bf16_16816(acc[m][j], af[m], b0l, b1l);
                mma_bf16_16816(acc[m][j + 4], af[m], b0h, b1h);
            }
        }
        xa += 16;
    };
    for (int i = 0; i < steps; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            use(u);
            if (i + u + 4 < steps) fetch(u);
        }
    }
    if (!live) return;
    // acc[m][c][0..1]: row 16m + g, columns c0 + 8 (2t) + c and c0 + 8 (2t + 1) + c; [2..3]: row 16m + g + 8
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int r = 16 * m + g + 8 * h;
            if (r < nrow) {
                float *dst = a.part + ((size_t)blockIdx.y * a.rows_out + s_o[r]) * N + c0 + 16 * t;
#pragma unroll
                for (int v = 0; v < 2; v++) {
                    *reinterpret_cast<float4 *>(dst + 8 * v) = make_float4(acc[m][0][2 * h + v], acc[m][1][2 * h + v], acc[m][2][2 * h + v], acc[m][3][2 * h + v]);
                    *reinterpret_cast<float4 *>(dst + 8 * v + 4) = make_float4(acc[m][4][2 * h + v], acc[m][5][2 * h + v], acc[m][6][2 * h + v], acc[m][7][2 * h + v]);
                }
            }
        }
}

// K slices of a k_gemv_rows8 launch with nz groups: a divisor of K / 64, about three blocks per SM in total
static int rows8_slices(int K, int N, int nz)
{
    const int nb = (N + 255) / 256, units = K / 64;
    int want = (3 * sm_count() + nb * nz / 2) / (nb * nz), ns = 1;
    if (want < 1) want = 1;
    for (int d = 1; d <= units; d++)
        if (units % d == 0 && d <= want) ns = d;
    while ((size_t)8 * (K / ns) * sizeof(float) > 48 * 1024 && ns < units) { ns++; while (units % ns) ns++; }
    return ns;
}
// launches k_gemv_rows8 over nz groups (grid.z) and ns K slices; a.part holds ns * a.rows_out * N floats
static int rows8_launch(Rows8 a, int nz, int ns, cudaStream_t st)
{
    const int nb = (a.N + 255) / 256;
    a.kslice = a.K / ns;
    a.k65536 = 65536u;
    size_t sm_b = (size_t)8 * a.kslice * sizeof(float), red_b = (size_t)4 * 8 * 256 * sizeof(float);
    if (red_b > sm_b) sm_b = red_b;
    static bool attr_done[64];
    int dv = 0;
    QLMB_CUDA(cudaGetDevice(&dv));
    if (dv >= 0 && dv < 64 && !attr_done[dv]) {
        QLMB_CUDA(cudaFuncSetAttribute(k_gemv_rows8, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        attr_done[dv] = true;
    }
    QLMB_CUDA(pdl_launch(true, k_gemv_rows8, dim3(nb, ns, nz), dim3(256), sm_b, st, a));
    QLMB_LAUNCH_CHECK("k_gemv_rows8");
    return QLMB_OK;
}

// K slices of a k_gemv_mma launch with nz groups of 16 * mt rows: a divisor of K / 64 such that the activation tile
// fits 64 KiB of shared memory, about two blocks per SM in total
static int mma_slices(int K, int N, int nz, int mt)
{
    const int nb = (N + 511) / 512, units = K / 64, kmax = mt == 1 ? 1024 : 512;
    int want = (2 * sm_count() + nb * nz / 2) / (nb * nz), best = 0, smallest = 0;
    if (want < 1) want = 1;
    for (int d = 1; d <= units; d++) {
        if (units % d || K / d > kmax) continue;
        if (!smallest) smallest = d;
        if (d <= want) best = d;
    }
    return best ? best : smallest;
}
static int mma_launch(Rows8 a, int nz, int ns, int mt, cudaStream_t st)
{
    const int nb = (a.N + 511) / 512;
    a.kslice = a.K / ns;
    a.k65536 = 65536u;
    const size_t sm_b = (size_t)16 * mt * (a.kslice + 8) * sizeof(bf16) + (size_t)a.kslice * 4 * sizeof(float);
    static bool attr_done[64];
    int dv = 0;
    QLMB_CUDA(cudaGetDevice(&dv));
    if (dv >= 0 && dv < 64 && !attr_done[dv]) {
        QLMB_CUDA(cudaFuncSetAttribute(k_gemv_mma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        QLMB_CUDA(cudaFuncSetAttribute(k_gemv_mma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        attr_done[dv] = true;
    }
    if (mt == 1) QLMB_CUDA(pdl_launch(true, k_gemv_mma<1>, dim3(nb, ns, nz), dim3(256), sm_b, st, a));
    else QLMB_CUDA(pdl_launch(true, k_gemv_mma<2>, dim3(nb, ns, nz), dim3(256), sm_b, st, a));
    QLMB_LAUNCH_CHECK("k_gemv_mma");
    return QLMB_OK;
}

// ---- codes W[N][K] (groups along K).  A warp owns 4 consecutive output columns (rows of W) and a
// K slice; lanes stride over the code words of the slice, 4 words (one per column) per step share the
// activation values; the scale multiplies the 8-element partial dot product of each word.
template <int BT>
__global__ void __launch_bounds__(256, BT <= 2 ? 4 : 2) k_gemv_nk(float *part, const void *X, int dtype, const uint8_t *codes,
                                                 const float *scales, int B, int K, int N, int kslice)
{
    extern __shared__ float xs[];               // [BT][kslice]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * 8 + warp) * 4;
    const int k0 = blockIdx.y * kslice, k1 = k0 + kslice < K ? k0 + kslice : K;
    const int gpr = K / 128, nw = (k1 - k0) / 8;             // code words of the slice
    for (int b0 = 0; b0 < B; b0 += BT) {
        __syncthreads();
        for (int i = threadIdx.x; i < BT * kslice; i += 256) {
            const int b = b0 + i / kslice, k = k0 + i % kslice;
            xs[i] = (b < B && k < k1) ? ld_x(X, dtype, (size_t)b * K + k) : 0.0f;
        }
        __syncthreads();
        if (n0 >= N) continue;
        float acc[4][BT];
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int b = 0; b < BT; b++) acc[c][b] = 0.0f;
#pragma unroll 2
        for (int kw = lane; kw < nw; kw += 32) {
            uint32_t w[4];
            float sc[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                w[c] = 0u; sc[c] = 0.0f;
                if (n0 + c < N) {
                    w[c] = __ldcs(reinterpret_cast<const uint32_t *>(codes + ((size_t)(n0 + c) * K + k0) / 2) + kw);
                    sc[c] = __ldg(scales + (size_t)(n0 + c) * gpr + (k0 + kw * 8) / 128);
                }
            }
            float d[4][8];
#pragma unroll
            for (int c = 0; c < 4; c++) unpack8(w[c], d[c]);
#pragma unroll
            for (int b = 0; b < BT; b++) {
                const float4 x0 = *reinterpret_cast<const float4 *>(&xs[b * kslice + kw * 8]);
                const float4 x1 = *reinterpret_cast<const float4 *>(&xs[b * kslice + kw * 8 + 4]);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const float t = x0.x * d[c][0] + x0.y * d[c][1] + x0.z * d[c][2] + x0.w * d[c][3] +
                                    x1.x * d[c][4] + x1.y * d[c][5] + x1.z * d[c][6] + x1.w * d[c][7];
                    acc[c][b] += sc[c] * t;
                }
            }
        }
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int b = 0; b < BT; b++) {
                float v = acc[c][b];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && b0 + b < B && n0 + c < N) part[((size_t)blockIdx.y * B + b0 + b) * N + n0 + c] = v;
            }
    }
}

// Y[b,n] = sum over K slices (ascending) of part[ks][b][n]
__global__ void __launch_bounds__(256) k_gemv_finish(void *Y, int dtype, const float *part, int nslice, size_t BN_)
{
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= BN_) return;
    float s = 0.0f;
    for (int k = 0; k < nslice; k++) s += part[(size_t)k * BN_ + i];
    if (dtype == QLMB_BF16) ((bf16 *)Y)[i] = __float2bfloat16_rn(s);
    else ((float *)Y)[i] = s;
}

// The finish of a decode step's output projection (dec_step, cudalm.cu:7188-7190: wo, the residual add and the norm in
// front of the FFN) in one launch, one block per slot: F[b,:] = bf16(slice sums) + res[b,:] (rounded to bf16 as the
// separate kernels do), Fn[b,:] = F * rinv * gamma with rinv = 1/sqrt(mean(F^2) + 1e-5).  N <= 2048.
__global__ void __launch_bounds__(256) k_gemv_finish_res_norm(bf16 *F, bf16 *Fn, const float *part, int nslice, int B, int N,
                                                              const bf16 *res, const float *gamma)
{
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float v[8], rs[8], gm[8], ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 8; c++) {                        // residual and gain are requested together with the slices
        const int n = threadIdx.x + 256 * c;
        v[c] = 0.0f; rs[c] = 0.0f; gm[c] = 0.0f;
        if (n < N) { rs[c] = __bfloat162float(res[(size_t)b * N + n]); gm[c] = gamma[n]; }
    }
    for (int k = 0; k < nslice; k++) {                   // slice order ascending per column, the columns' loads independent
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int n = threadIdx.x + 256 * c;
            if (n < N) v[c] += part[((size_t)k * B + b) * N + n];
        }
    }
#pragma unroll
    for (int c = 0; c < 8; c++) {
        const int n = threadIdx.x + 256 * c;
        if (n < N) {
            float y = v[c];
            v[c] = 0.0f;
            y = __bfloat162float(__float2bfloat16_rn(y));
            const bf16 f = __float2bfloat16_rn(y + rs[c]);
            F[(size_t)b * N + n] = f;
            v[c] = __bfloat162float(f);
            ss += v[c] * v[c];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float rinv = 1.0f / sqrtf(tot / (float)N + 1e-5f);
#pragma unroll
    for (int c = 0; c < 8; c++) {
        const int n = threadIdx.x + 256 * c;
        if (n < N) Fn[(size_t)b * N + n] = __float2bfloat16_rn(v[c] * rinv * gm[c]);
    }
}

// The finish of a decode step's stacked q, k, v projections with what follows them (dec_step, cudalm.cu:7181-7183):
// rows [3][B][N] of slice sums -> bf16; the q and k rows are rotated by the angle of their slot's position
// (k_dec_rope: pairs (i, i + hd/2) of every head), the k and v rows go to position pos[b] of the slot's cache
// (k_dec_kv).  One thread per pair; Y receives all three rows as the separate kernels would leave them.
__global__ void __launch_bounds__(256) k_gemv_finish_qkv(bf16 *Y, bf16 *Kc, bf16 *Vc, const float *part, int nslice, int B, int N,
                                                         int hd, const float *cosb, const float *sinb, const int *pos, int Tm,
                                                         int *errword)
{
    pdl_trigger();
    pdl_wait();
    const int hf = hd / 2, nh = N / hd;
    const size_t g = (size_t)blockIdx.x * 256 + threadIdx.x, RN = (size_t)3 * B * N;
    if (g >= RN / 2) return;
    const int i = (int)(g % hf);
    const size_t r = g / hf;
    const int row = (int)(r / nh), h = (int)(r % nh), m = row / B, b = row % B, t = pos[b];
    // a slot past its cache (or past the rotation tables, which cover the cache): no table read, no cache write
    if (t < 0 || t >= Tm) { if (i == 0 && h == 0 && m == 0) report_bad_index(errword, 303, b, t); return; }
    const size_t o = (size_t)row * N + (size_t)h * hd + i;
    float x = 0.0f, y = 0.0f;
    for (int k = 0; k < nslice; k++) { x += part[(size_t)k * RN + o]; y += part[(size_t)k * RN + o + hf]; }
    x = __bfloat162float(__float2bfloat16_rn(x)); y = __bfloat162float(__float2bfloat16_rn(y));
    if (m < 2) {
        const float c = cosb[(size_t)t * hf + i], sn = sinb[(size_t)t * hf + i];
        const float xr = x * c - y * sn, yr = y * c + x * sn;
        x = xr; y = yr;
    }
    const bf16 xo = __float2bfloat16_rn(x), yo = __float2bfloat16_rn(y);
    Y[o] = xo; Y[o + hf] = yo;
    if (m >= 1) {
        bf16 *cache = m == 1 ? Kc : Vc;
        const size_t co = ((size_t)b * Tm + t) * N + (size_t)h * hd + i;
        cache[co] = xo; cache[co + hf] = yo;
    }
}

// act[r,f] = silu(g) * u with g, u the K-slice sums (ascending) of the gate and up partials
__global__ void __launch_bounds__(256) k_gemv_finish_swiglu(bf16 *act, const float *pg, const float *pu, int nslice, size_t RN,
                                                            size_t slice_stride)
{
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= RN) return;
    float g = 0.0f, u = 0.0f;
    for (int k = 0; k < nslice; k++) { g += pg[(size_t)k * slice_stride + i]; u += pu[(size_t)k * slice_stride + i]; }
    // the stash of the training path holds g and u as bf16; round the same way before the product
    g = __bfloat162float(__float2bfloat16_rn(g)); u = __bfloat162float(__float2bfloat16_rn(u));
    act[i] = __float2bfloat16_rn(g * __fdividef(1.0f, 1.0f + __expf(-g)) * u);
}
// out[n,j] = f_in[n,j] + sum_k gate[k,n] * y[k*ntok+n, j]   (k ascending, cudalm.cu:4027), y = slice sums of the down partials
__global__ void __launch_bounds__(256) k_gemv_finish_combine(bf16 *out, const bf16 *f_in, const float *part, const float *gate,
                                                             int nslice, int ntok, int Kk, int D)
{
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (size_t)ntok * D) return;
    const int n = (int)(i / D), j = (int)(i % D);
    const size_t RN = (size_t)Kk * ntok * D;
    float acc = __bfloat162float(f_in[i]);
    for (int k = 0; k < Kk; k++) {
        const size_t o = ((size_t)k * ntok + n) * D + j;
        float y = 0.0f;
        for (int s = 0; s < nslice; s++) y += part[(size_t)s * RN + o];
        y = __bfloat162float(__float2bfloat16_rn(y));
        acc += gate[(size_t)k * ntok + n] * y;
    }
    out[i] = __float2bfloat16_rn(acc);
}

// Experts of a decode step with at most 128 routed rows: three routed GEMVs that read only the chosen experts'
// codes (W1, W3: [E][D][F]; W2: [E][F][D]), SwiGLU and the gate-weighted combination in the slice-sum kernels.
int moe_decode_experts(const qlmb_moe_layer *L, void *out, const void *f_in, const void *f_norm, const int *assign,
                       const float *gate, cudaStream_t st, int *perm, int *off, int *counts, int *bad, int perm_ready)
{
    const int N = L->N, D = L->D, F = L->F, K = L->K, R = K * N;
    if (R > 16 && perm && off && bad) {
        // many routed rows: sort the slots by expert once, then every expert's matrices are read once per group of
        // sixteen of its slots instead of once per slot
        int rc = perm_ready ? 0 : perm_build(assign, N, L->E, K, 1, 1, perm, nullptr, off, counts, bad, nullptr, nullptr, nullptr, st);
        if (rc) return rc;
        const int zmax = L->E + R / 16;                  // sum over the experts of ceil(count / 16) never exceeds this
        const int ns1 = mma_slices(D, F, 2 * L->E, 1), ns2 = mma_slices(F, D, L->E, 1);
        const size_t pg_n = (size_t)ns1 * 2 * R * F, pd_n = (size_t)ns2 * R * D;
        void *ws = nullptr;
        if ((rc = workspace((pg_n + pd_n) * sizeof(float) + (size_t)R * F * sizeof(bf16) + 256, &ws))) return rc;
        float *pg = (float *)ws, *pd = pg + pg_n;
        bf16 *act = (bf16 *)(pd + pd_n);
        Rows8 a = {};
        a.part = pg; a.X = f_norm; a.x_dtype = QLMB_BF16; a.K = D; a.N = F;
        a.codes = (const uint8_t *)L->w1_codes; a.scales = L->w1_scales; a.codes2 = (const uint8_t *)L->w3_codes; a.scales2 = L->w3_scales;
        a.e_codes = (size_t)D * F / 2; a.e_scales = (size_t)D * F / 128;
        a.rows_out = 2 * R; a.perm = perm; a.off = off; a.E = L->E; a.ntok = N; a.x_by_token = 1; a.zdual = zmax; a.R = R;
        if ((rc = mma_launch(a, 2 * zmax, ns1, 1, st))) return rc;
        pdl_launch(N > 4, k_gemv_finish_swiglu, dim3((unsigned)(((size_t)R * F + 255) / 256)), dim3(256), 0, st, act, pg, pg + (size_t)R * F, ns1, (size_t)R * F, (size_t)2 * R * F);
        Rows8 b = {};
        b.part = pd; b.X = act; b.x_dtype = QLMB_BF16; b.K = F; b.N = D;
        b.codes = (const uint8_t *)L->w2_codes; b.scales = L->w2_scales; b.e_codes = (size_t)D * F / 2; b.e_scales = (size_t)D * F / 128;
        b.rows_out = R; b.perm = perm; b.off = off; b.E = L->E; b.ntok = N; b.x_by_token = 0; b.zdual = 0; b.R = R;
        if ((rc = mma_launch(b, zmax, ns2, 1, st))) return rc;
        pdl_launch(N > 4, k_gemv_finish_combine, dim3((unsigned)(((size_t)N * D + 255) / 256)), dim3(256), 0, st, (bf16 *)out, (const bf16 *)f_in, pd, gate, ns2, N, K, D);
        QLMB_LAUNCH_CHECK("moe_decode_experts");
        return QLMB_OK;
    }
    auto slices = [](int Kdim, int Ncols, int rows, int &kslice, int &nslice) {
        const int nblk = (Ncols + 255) / 256;
        nslice = (4 * sm_count()) / (nblk * rows);
        if (nslice > Kdim / 64) nslice = Kdim / 64;
        if (nslice < 1) nslice = 1;
        kslice = ((Kdim + nslice - 1) / nslice + 127) / 128 * 128;
        nslice = (Kdim + kslice - 1) / kslice;
    };
    int ks1, ns1, ks2, ns2;
    slices(D, F, 2 * R, ks1, ns1);
    slices(F, D, R, ks2, ns2);
    const size_t pg_n = (size_t)ns1 * R * F, pd_n = (size_t)ns2 * R * D;
    void *ws = nullptr;
    int rc = workspace((2 * pg_n + pd_n) * sizeof(float) + (size_t)R * F * sizeof(bf16) + 256, &ws);
    if (rc) return rc;
    // gate and up share one launch: rows 0..R-1 of a slice are the gate partials, rows R..2R-1 the up partials
    float *pg = (float *)ws, *pu = pg + (size_t)R * F, *pd = pg + 2 * pg_n;
    bf16 *act = (bf16 *)(pd + pd_n);
    const size_t ec = (size_t)D * F / 2, es = (size_t)D * F / 128;
    const dim3 g1((F + 255) / 256, ns1, 2 * R), g2((D + 255) / 256, ns2, R);
    const size_t small_grid = (size_t)2 * sm_count();
    if ((size_t)g1.x * g1.y * g1.z <= small_grid)
        launch_kn<1, 4>(N > 4, g1, (size_t)ks1 * sizeof(float), st, pg, f_norm, QLMB_BF16, (const uint8_t *)L->w1_codes, L->w1_scales, 1, D, F, ks1, assign, ec, es, N, nullptr, R,
            (const uint8_t *)L->w3_codes, L->w3_scales);
    else
        launch_kn<1, 2>(N > 4, g1, (size_t)ks1 * sizeof(float), st, pg, f_norm, QLMB_BF16, (const uint8_t *)L->w1_codes, L->w1_scales, 1, D, F, ks1, assign, ec, es, N, nullptr, R,
            (const uint8_t *)L->w3_codes, L->w3_scales);
    pdl_launch(N > 4, k_gemv_finish_swiglu, dim3((unsigned)(((size_t)R * F + 255) / 256)), dim3(256), 0, st, act, pg, pu, ns1, (size_t)R * F, (size_t)2 * R * F);
    if ((size_t)g2.x * g2.y * g2.z <= small_grid)
        launch_kn<1, 4>(N > 4, g2, (size_t)ks2 * sizeof(float), st, pd, act, QLMB_BF16, (const uint8_t *)L->w2_codes, L->w2_scales, 1, F, D, ks2, assign, ec, es, R);
    else
        launch_kn<1, 2>(N > 4, g2, (size_t)ks2 * sizeof(float), st, pd, act, QLMB_BF16, (const uint8_t *)L->w2_codes, L->w2_scales, 1, F, D, ks2, assign, ec, es, R);
    pdl_launch(N > 4, k_gemv_finish_combine, dim3((unsigned)(((size_t)N * D + 255) / 256)), dim3(256), 0, st, (bf16 *)out, (const bf16 *)f_in, pd, gate, ns2, N, K, D);
    QLMB_LAUNCH_CHECK("moe_decode_experts");
    return QLMB_OK;
}

}  // namespace qlmb

using namespace qlmb;

// the fused finish of the output projection: F (written through Y), Fn, the residual and the norm's gain
struct FinishResNorm { void *Fn; const void *res; const float *gamma; };

static int gemv_decode_impl(void *Y, const void *X, const int8_t *codes, const float *scales, int layout, int B, int K, int N,
                            int dtype, void *stream, const FinishResNorm *fr)
{
    QLMB_REQUIRE(layout == QLMB_KN || layout == QLMB_NK, "qlmb_gemv_decode: layout %d", layout);
    QLMB_REQUIRE(dtype == QLMB_F32 || dtype == QLMB_BF16, "qlmb_gemv_decode: dtype %d", dtype);
    QLMB_REQUIRE(B >= 0 && B <= 64 && K > 0 && N > 0, "qlmb_gemv_decode: B=%d (at most 64 slots) K=%d N=%d", B, K, N);
    if ((K % 128) || (N % 128)) {
        set_error("qlmb_gemv_decode: K=%d and N=%d must be multiples of the 128-element scale group", K, N);
        return QLMB_E_UNSUPPORTED;
    }
    if (B == 0) return QLMB_OK;
    QLMB_REQUIRE(Y && X && codes && scales, "qlmb_gemv_decode: NULL argument");
    cudaStream_t st = as_stream(stream);
    // more than 4 live slots with bf16 activations: the tensor-core engine streams the weights
    // faster than fp32 FMAs can consume them (fp32 activations keep the exact fp32 path)
    // many rows on a large matrix: the 256-row tensor-core tiles of the training engine read the weights once
    // (940 GB/s at 4096 x 16384 with 64 rows, against 520 for two passes of 32-row groups)
    if (!fr && layout == QLMB_KN && B > 32 && dtype == QLMB_BF16 && (K % 64) == 0 && (size_t)K * N >= ((size_t)16 << 20))
        return qlmb_linear_fwd(Y, X, codes, scales, layout, B, K, N, nullptr, dtype, stream);
    if (layout == QLMB_KN && B > 4) {
        // groups of eight rows per pass over the weights (fp32 multiply-adds; the 256-row tensor-core tiles would be
        // seven eighths padding for a handful of rows)
        const bool tc = dtype == QLMB_BF16 && (N % 64) == 0;
        const int mt = B > 16 ? 2 : 1;
        const int nz = tc ? (B + 16 * mt - 1) / (16 * mt) : (B + 7) / 8, ns = tc ? mma_slices(K, N, nz, mt) : rows8_slices(K, N, nz);
        void *wsr = nullptr;
        int rcr = workspace((size_t)ns * B * N * sizeof(float), &wsr);
        if (rcr) return rcr;
        Rows8 a = {};
        a.part = (float *)wsr; a.X = X; a.x_dtype = dtype; a.K = K; a.N = N;
        a.codes = (const uint8_t *)codes; a.scales = scales; a.B = B; a.nmat = 1; a.rows_out = B;
        if ((rcr = tc ? mma_launch(a, nz, ns, mt, st) : rows8_launch(a, nz, ns, st))) return rcr;
        if (fr) pdl_launch(B > 4, k_gemv_finish_res_norm, dim3(B), dim3(256), 0, st, (bf16 *)Y, (bf16 *)fr->Fn, a.part, ns, B, N, (const bf16 *)fr->res, fr->gamma);
        else pdl_launch(B > 4, k_gemv_finish, dim3((unsigned)(((size_t)B * N + 255) / 256)), dim3(256), 0, st, Y, dtype, a.part, ns, (size_t)B * N);
        QLMB_LAUNCH_CHECK("qlmb_gemv_decode");
        return QLMB_OK;
    }
    if (!fr && B > 4 && dtype == QLMB_BF16 && (K % 64) == 0)
        return qlmb_linear_fwd(Y, X, codes, scales, layout, B, K, N, nullptr, dtype, stream);
    const int bt = B <= 1 ? 1 : B <= 2 ? 2 : B <= 4 ? 4 : 8;
    static int stream_on = -1;
    if (stream_on < 0) { const char *e = getenv("QLMB_GEMV_STREAM"); stream_on = (e && atoi(e) == 0) ? 0 : 1; }
    if (stream_on && !fr && layout == QLMB_KN && bt <= 4) {
        // one launch: streaming kernel with the slice sums combined by the last block of every column block
        const int cpl = N >= 8192 ? 16 : 8, cw = 32 * cpl;
        const int nb = (N + cw - 1) / cw;
        QLMB_REQUIRE(nb <= 2048, "qlmb_gemv_decode: N=%d", N);
        // K slices: a divisor of K / 64 (slices are whole multiples of 64 rows), about three blocks per SM in total
        const int units = K / 64;
        // (measured at 4096 x 16384, one row: 3 blocks per SM in total 14.3 us, 6: 16.4 us, 12: 18.6 us -- the staging,
        // the warp tree and the ticket are a fixed cost per block; a ring of bulk copies per row into shared memory
        // instead of register prefetch was slower, 29 us)
        int want = (3 * sm_count() + nb / 2) / nb, ns = 1;
        for (int d = 1; d <= units; d++)
            if (units % d == 0 && d <= want && (size_t)bt * (K / d) * sizeof(float) <= 64 * 1024) ns = d;
        while ((size_t)bt * (K / ns) * sizeof(float) > 64 * 1024 && ns < units) { ns++; while (units % ns) ns++; }
        const int ksl = K / ns;
        void *ws2 = nullptr;
        int rc2 = workspace((size_t)ns * B * N * sizeof(float), &ws2);
        if (rc2) return rc2;
        size_t sm_b = (size_t)bt * ksl * sizeof(float), red_b = (size_t)4 * bt * cw * sizeof(float);
        if (red_b > sm_b) sm_b = red_b;
        const dim3 g(nb, ns);
#define GS_LAUNCH(BT_, CPL_) \
        do { \
            static bool attr_done[64]; int dv = 0; QLMB_CUDA(cudaGetDevice(&dv)); \
            if (dv >= 0 && dv < 64 && !attr_done[dv]) { QLMB_CUDA(cudaFuncSetAttribute(k_gemv_stream<BT_, CPL_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)); attr_done[dv] = true; } \
            k_gemv_stream<BT_, CPL_><<<g, 256, sm_b, st>>>(Y, dtype, (float *)ws2, X, (const uint8_t *)codes, scales, B, K, N, ksl, 65536u); \
        } while (0)
        if (cpl == 16) { if (bt == 1) GS_LAUNCH(1, 16); else if (bt == 2) GS_LAUNCH(2, 16); else GS_LAUNCH(4, 16); }
        else { if (bt == 1) GS_LAUNCH(1, 8); else if (bt == 2) GS_LAUNCH(2, 8); else GS_LAUNCH(4, 8); }
#undef GS_LAUNCH
        QLMB_LAUNCH_CHECK("k_gemv_stream");
        return QLMB_OK;
    }
    // K slices: enough blocks to fill the device once, at least 64 rows each,
    // a multiple of 8 rows, and small enough for the activation tile in shared memory
    const int nblk = layout == QLMB_KN ? (N + 255) / 256 : (N + 31) / 32;
    // K slices for 4 (bt <= 2) or 2 blocks per SM
    int nslice = ((bt <= 2 ? 4 : 2) * sm_count()) / nblk;
    if (nslice > K / 64) nslice = K / 64;
    if (nslice < 1) nslice = 1;
    int kslice = ((K + nslice - 1) / nslice + 127) / 128 * 128;
    while ((size_t)bt * kslice * sizeof(float) > 32 * 1024) kslice = (kslice / 2 + 127) / 128 * 128;
    nslice = (K + kslice - 1) / kslice;
    void *ws = nullptr;
    int rc = workspace((size_t)nslice * B * N * sizeof(float), &ws);
    if (rc) return rc;
    float *part = (float *)ws;
    const size_t smem = (size_t)bt * kslice * sizeof(float);
    const dim3 grid(nblk, nslice);
#define GV_LAUNCH(KERN) \
    do { \
        if (bt == 1) KERN<1><<<grid, 256, smem, st>>>(part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice); \
        else if (bt == 2) KERN<2><<<grid, 256, smem, st>>>(part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice); \
        else if (bt == 4) KERN<4><<<grid, 256, smem, st>>>(part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice); \
        else KERN<8><<<grid, 256, smem, st>>>(part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice); \
    } while (0)
    if (layout == QLMB_KN && bt == 1 && (size_t)nblk * nslice <= (size_t)2 * sm_count())
        launch_kn<1, 4>(B > 4, grid, smem, st, part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice);
    else if (layout == QLMB_KN) {
        if (bt == 1) launch_kn<1, 2>(B > 4, grid, smem, st, part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice);
        else if (bt == 2) launch_kn<2, 2>(B > 4, grid, smem, st, part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice);
        else if (bt == 4) launch_kn<4, 2>(B > 4, grid, smem, st, part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice);
        else launch_kn<8, 2>(B > 4, grid, smem, st, part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice);
    }
    else GV_LAUNCH(k_gemv_nk);
#undef GV_LAUNCH
    if (fr) pdl_launch(B > 4, k_gemv_finish_res_norm, dim3(B), dim3(256), 0, st, (bf16 *)Y, (bf16 *)fr->Fn, part, nslice, B, N, (const bf16 *)fr->res, fr->gamma);
    else pdl_launch(B > 4, k_gemv_finish, dim3((unsigned)(((size_t)B * N + 255) / 256)), dim3(256), 0, st, Y, dtype, part, nslice, (size_t)B * N);
    QLMB_LAUNCH_CHECK("qlmb_gemv_decode");
    return QLMB_OK;
}

extern "C" int qlmb_gemv_decode(void *Y, const void *X, const int8_t *codes, const float *scales, int layout,
                                int B, int K, int N, int dtype, void *stream)
{
    return gemv_decode_impl(Y, X, codes, scales, layout, B, K, N, dtype, stream, nullptr);
}

// Y[m*B + b, :] = X[b, :] deq(W_m) for nmat equally shaped matrices stored one after the other (codes W_m[K][N]):
// the q, k and v projections of a decode step in one launch pair (cudalm.cu:7178-7180) when KD = D.
// fq: the q, k, v finish (rotation tables, positions, the slot caches)
struct FinishQkv { void *Kc; void *Vc; const float *cosb; const float *sinb; const int *pos; int hd; int Tm; };
static int gemv_stack_impl(void *Y, const void *X, const int8_t *codes, const float *scales, int nmat, int B, int K, int N,
                           int dtype, void *stream, const FinishResNorm *fr, const float *gamma = nullptr,
                           const FinishQkv *fq = nullptr)
{
    QLMB_REQUIRE(Y && X && codes && scales, "qlmb_gemv_decode_stack: NULL argument");
    QLMB_REQUIRE(dtype == QLMB_F32 || dtype == QLMB_BF16, "qlmb_gemv_decode_stack: dtype %d", dtype);
    QLMB_REQUIRE(nmat > 0 && B > 0 && nmat * B <= 256 && K > 0 && N > 0 && (K % 128) == 0 && (N % 128) == 0,
                 "qlmb_gemv_decode_stack: nmat=%d B=%d K=%d N=%d", nmat, B, K, N);
    cudaStream_t st = as_stream(stream);
    const int R = nmat * B, nblk = (N + 255) / 256;
    int nslice = (4 * sm_count()) / (nblk * R);
    if (nslice > K / 64) nslice = K / 64;
    if (nslice < 1) nslice = 1;
    int kslice = ((K + nslice - 1) / nslice + 127) / 128 * 128;
    nslice = (K + kslice - 1) / kslice;
    const bool groups = B > 4;                           // more than four rows: groups share one pass over a matrix
    const bool tc = groups && dtype == QLMB_BF16 && (N % 64) == 0;   // bf16 rows: warp-level MMAs, 16 or 32 rows per group
    const int mt = B > 16 ? 2 : 1;
    const int nz = tc ? nmat * ((B + 16 * mt - 1) / (16 * mt)) : nmat * ((B + 7) / 8);
    if (groups) nslice = tc ? mma_slices(K, N, nz, mt) : rows8_slices(K, N, nz);
    void *ws = nullptr;
    int rc = workspace((size_t)nslice * R * N * sizeof(float), &ws);
    if (rc) return rc;
    float *part = (float *)ws;
    if (groups) {
        Rows8 a = {};
        a.part = part; a.X = X; a.x_dtype = dtype; a.K = K; a.N = N;
        a.codes = (const uint8_t *)codes; a.scales = scales; a.e_codes = (size_t)K * N / 2; a.e_scales = (size_t)K * N / 128;
        a.B = B; a.nmat = nmat; a.rows_out = R; a.gamma = gamma;
        if ((rc = tc ? mma_launch(a, nz, nslice, mt, st) : rows8_launch(a, nz, nslice, st))) return rc;
    } else if ((size_t)nblk * nslice * R <= (size_t)2 * sm_count())
        launch_kn<1, 4>(B > 4, dim3(nblk, nslice, R), (size_t)kslice * sizeof(float), st, part, X, dtype, (const uint8_t *)codes, scales, 1, K, N, kslice, nullptr, (size_t)K * N / 2, (size_t)K * N / 128, B, gamma);
    else
        launch_kn<1, 2>(B > 4, dim3(nblk, nslice, R), (size_t)kslice * sizeof(float), st, part, X, dtype, (const uint8_t *)codes, scales, 1, K, N, kslice, nullptr, (size_t)K * N / 2, (size_t)K * N / 128, B, gamma);
    if (fr) pdl_launch(B > 4, k_gemv_finish_res_norm, dim3(R), dim3(256), 0, st, (bf16 *)Y, (bf16 *)fr->Fn, part, nslice, R, N, (const bf16 *)fr->res, fr->gamma);
    else if (fq) pdl_launch(B > 4, k_gemv_finish_qkv, dim3((unsigned)(((size_t)R * N / 2 + 255) / 256)), dim3(256), 0, st, (bf16 *)Y, (bf16 *)fq->Kc, (bf16 *)fq->Vc, part, nslice, B, N, fq->hd, fq->cosb, fq->sinb, fq->pos, fq->Tm, device_error_word());
    else pdl_launch(B > 4, k_gemv_finish, dim3((unsigned)(((size_t)R * N + 255) / 256)), dim3(256), 0, st, Y, dtype, part, nslice, (size_t)R * N);
    QLMB_LAUNCH_CHECK("qlmb_gemv_decode_stack");
    return QLMB_OK;
}

extern "C" int qlmb_gemv_decode_stack(void *Y, const void *X, const int8_t *codes, const float *scales, int nmat, int B,
                                      int K, int N, int dtype, void *stream)
{
    return gemv_stack_impl(Y, X, codes, scales, nmat, B, K, N, dtype, stream, nullptr);
}

extern "C" int qlmb_gemv_decode_norm_stack(void *Y, const void *X, const float *gamma, const int8_t *codes, const float *scales,
                                          int nmat, int B, int K, int N, int dtype, void *stream)
{
    QLMB_REQUIRE(gamma, "qlmb_gemv_decode_norm_stack: NULL argument");
    return gemv_stack_impl(Y, X, codes, scales, nmat, B, K, N, dtype, stream, nullptr, gamma);
}

extern "C" int qlmb_dec_qkv(void *Y, void *Kc, void *Vc, const void *X, const float *gamma, const int8_t *codes,
                            const float *scales, const float *cosb, const float *sinb, const int *pos, int B, int D, int hd,
                            int Tm, void *stream)
{
    QLMB_REQUIRE(Y && Kc && Vc && X && gamma && cosb && sinb && pos, "qlmb_dec_qkv: NULL argument");
    QLMB_REQUIRE(hd > 0 && hd % 2 == 0 && D % hd == 0 && Tm > 0, "qlmb_dec_qkv: D=%d hd=%d Tm=%d", D, hd, Tm);
    const FinishQkv fq = {Kc, Vc, cosb, sinb, pos, hd, Tm};
    return gemv_stack_impl(Y, X, codes, scales, 3, B, D, D, QLMB_BF16, stream, nullptr, gamma, &fq);
}

extern "C" int qlmb_gemv_decode_res_norm(void *F, void *Fn, const void *X, const int8_t *codes, const float *scales,
                                         const void *res, const float *gamma, int B, int K, int N, void *stream)
{
    QLMB_REQUIRE(F && Fn && X && codes && scales && res && gamma, "qlmb_gemv_decode_res_norm: NULL argument");
    QLMB_REQUIRE(B > 0 && B <= 256 && K > 0 && N > 0 && N <= 2048 && (K % 128) == 0 && (N % 128) == 0,
                 "qlmb_gemv_decode_res_norm: B=%d K=%d N=%d", B, K, N);
    const FinishResNorm fr = {Fn, res, gamma};
    if (B <= 4) return gemv_decode_impl(F, X, codes, scales, QLMB_KN, B, K, N, QLMB_BF16, stream, &fr);
    return gemv_stack_impl(F, X, codes, scales, 1, B, K, N, QLMB_BF16, stream, &fr);
}
