// Memory-bound row kernels around the expert GEMMs: router logits, token
// gather into expert order, gated combine, the backward's gate/dy pass,
// router backward and the un-permute of input gradients.  All of them read
// and write 16-byte vectors along the feature dimension.
#include "qlmb_common.cuh"
#include "qlmb_internal.h"

namespace qlmb {

__device__ __forceinline__ float ld_act(const void *p, int dtype, size_t i)
{
    return dtype == QLMB_BF16 ? __bfloat162float(((const bf16 *)p)[i]) : ((const float *)p)[i];
}
__device__ __forceinline__ void st_act(void *p, int dtype, size_t i, float v)
{
    if (dtype == QLMB_BF16) ((bf16 *)p)[i] = __float2bfloat16_rn(v);
    else ((float *)p)[i] = v;
}
// 8 consecutive activations as fp32 (16 B of bf16 or 32 B of fp32); i is a multiple of 8
__device__ __forceinline__ void ld_act8(const void *p, int dtype, size_t i, float v[8])
{
    if (dtype == QLMB_BF16) {
        uint4 q = *reinterpret_cast<const uint4 *>((const bf16 *)p + i);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
        for (int k = 0; k < 4; k++) { float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
    } else {
        float4 a = *reinterpret_cast<const float4 *>((const float *)p + i);
        float4 b = *reinterpret_cast<const float4 *>((const float *)p + i + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float v[8])
{
    uint4 q;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
    for (int k = 0; k < 4; k++) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    return q;
}
__device__ __forceinline__ void st_act8(void *p, int dtype, size_t i, const float v[8])
{
    if (dtype == QLMB_BF16) {
        *reinterpret_cast<uint4 *>((bf16 *)p + i) = pack_bf16x8(v);
    } else {
        *reinterpret_cast<float4 *>((float *)p + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>((float *)p + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// ------------------------------------------------------------ router logits
// rt[n,e] = sum_j X[n,j] * Wr[j,e]  (reference cudalm.cu:4158, g_ab with N = E), fp32.
// A warp owns 8 tokens, lane = expert; Wr rows (128 B) and the token rows (broadcast
// vector loads) come through L1, which holds all of Wr.
template <int XBF16>
__global__ void __launch_bounds__(512) k_router_logits_warp(float *rt, const void *X, const float *Wr, int N, int D, int E)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * 16 + warp) * 8;
    if (n0 >= N) return;
    const int e = lane < E ? lane : E - 1;
    float acc[8];
#pragma unroll
    for (int t = 0; t < 8; t++) acc[t] = 0.0f;
#pragma unroll 2
    for (int j = 0; j < D; j += 4) {
        float w[4];
#pragma unroll
        for (int jj = 0; jj < 4; jj++) w[jj] = __ldg(Wr + (size_t)(j + jj) * E + e);
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const int n = n0 + t < N ? n0 + t : N - 1;
            float x0, x1, x2, x3;
            if (XBF16) {
                uint2 q = __ldg(reinterpret_cast<const uint2 *>((const bf16 *)X + (size_t)n * D + j));
                float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&q.x));
                float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&q.y));
                x0 = a.x; x1 = a.y; x2 = b.x; x3 = b.y;
            } else {
                float4 q = __ldg(reinterpret_cast<const float4 *>((const float *)X + (size_t)n * D + j));
                x0 = q.x; x1 = q.y; x2 = q.z; x3 = q.w;
            }
            acc[t] += x0 * w[0]; acc[t] += x1 * w[1]; acc[t] += x2 * w[2]; acc[t] += x3 * w[3];
        }
    }
    if (lane < E) {
#pragma unroll
        for (int t = 0; t < 8; t++) if (n0 + t < N) rt[(size_t)(n0 + t) * E + lane] = acc[t];
    }
}

// General shape (E > 32 or Wr too large for shared memory): a block owns 32 tokens,
// the token tile is staged 256 features at a time.
#define RL_TOK 32
#define RL_DCH 256
__global__ void __launch_bounds__(256) k_router_logits(float *rt, const void *X, int x_dtype,
                                                       const float *Wr, int N, int D, int E)
{
    __shared__ float xs[RL_TOK][RL_DCH];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n0 = blockIdx.x * RL_TOK;
    for (int e0 = 0; e0 < E; e0 += 32) {
        int e = e0 + lane;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int d0 = 0; d0 < D; d0 += RL_DCH) {
            int dn = D - d0 < RL_DCH ? D - d0 : RL_DCH;
            __syncthreads();
            for (int i = threadIdx.x; i < RL_TOK * RL_DCH; i += 256) {
                int t = i / RL_DCH, j = i % RL_DCH, n = n0 + t;
                xs[t][j] = (n < N && j < dn) ? ld_act(X, x_dtype, (size_t)n * D + d0 + j) : 0.0f;
            }
            __syncthreads();
            if (e < E) {
                for (int j = 0; j < dn; j++) {
                    float w = Wr[(size_t)(d0 + j) * E + e];
#pragma unroll
                    for (int t = 0; t < 4; t++) acc[t] += xs[warp * 4 + t][j] * w;
                }
            }
        }
        if (e < E) {
#pragma unroll
            for (int t = 0; t < 4; t++) {
                int n = n0 + warp * 4 + t;
                if (n < N) rt[(size_t)n * E + e] = acc[t];
            }
        }
    }
}

int router_logits(float *rt, const void *X, int x_dtype, const float *Wr, int N, int D, int E, cudaStream_t st)
{
    if (E <= 32 && (D % 4) == 0) {
        int blocks = (N + 127) / 128;               // 16 warps x 8 tokens per block
        if (x_dtype == QLMB_BF16) k_router_logits_warp<1><<<blocks, 512, 0, st>>>(rt, X, Wr, N, D, E);
        else k_router_logits_warp<0><<<blocks, 512, 0, st>>>(rt, X, Wr, N, D, E);
    } else {
        k_router_logits<<<(N + RL_TOK - 1) / RL_TOK, 256, 0, st>>>(rt, X, x_dtype, Wr, N, D, E);
    }
    QLMB_LAUNCH_CHECK("k_router_logits");
    return QLMB_OK;
}

// ------------------------------------------------------------------ gather
// One warp per permuted row, 16-byte chunks (reference k_gather_bf, cudalm.cu:3892).
__global__ void __launch_bounds__(256) k_gather_rows(bf16 *Xp, const void *src, int dtype,
                                                     const int *perm, const int *nrows_dev, int nrows_host, int N, int D)
{
    int rows = nrows_dev ? *nrows_dev : nrows_host;
    int lane = threadIdx.x & 31;
    for (int j = blockIdx.x * 8 + (threadIdx.x >> 5); j < rows; j += gridDim.x * 8) {
        int np = perm[j];
        uint4 *o = reinterpret_cast<uint4 *>(Xp + (size_t)j * D);
        if (np < 0) {
            for (int c = lane; c < D / 8; c += 32) o[c] = make_uint4(0, 0, 0, 0);
            continue;
        }
        size_t base = (size_t)(np % N) * D;
        if (dtype == QLMB_BF16) {
            const uint4 *s = reinterpret_cast<const uint4 *>((const bf16 *)src + base);
            for (int c = lane; c < D / 8; c += 32) o[c] = s[c];
        } else {
            for (int c = lane; c < D / 8; c += 32) {
                float v[8];
                ld_act8(src, QLMB_F32, base + (size_t)c * 8, v);
                o[c] = pack_bf16x8(v);
            }
        }
    }
}

int gather_rows(bf16 *Xp, const void *src, int dtype, const int *perm, const int *nrows_dev, int max_rows,
                int N, int D, cudaStream_t st)
{
    int blocks = (max_rows + 7) / 8;
    int cap = sm_count() * 8;
    if (blocks > cap) blocks = cap;
    k_gather_rows<<<blocks, 256, 0, st>>>(Xp, src, dtype, perm, nrows_dev, max_rows, N, D);
    QLMB_LAUNCH_CHECK("k_gather_rows");
    return QLMB_OK;
}

// ----------------------------------------------------------------- combine
// out[n] = f_in[n] + sum_k gate[k,n] * yp[inv[k,n]], k ascending (reference
// k_combine_bf, cudalm.cu:4028-4034).  One warp per token.
__global__ void __launch_bounds__(256) k_combine_rows(void *out, const void *f_in, int dtype,
                                                      const bf16 *yp, const int *inv, const float *gate,
                                                      int N, int D, int K)
{
    int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    for (int c = lane; c < D / 8; c += 32) {
        float acc[8];
        ld_act8(f_in, dtype, (size_t)n * D + (size_t)c * 8, acc);
        for (int k = 0; k < K; k++) {
            size_t slot = (size_t)k * N + n;
            float g = gate[slot];
            float y[8];
            ld_act8(yp, QLMB_BF16, (size_t)inv[slot] * D + (size_t)c * 8, y);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += g * y[i];
        }
        st_act8(out, dtype, (size_t)n * D + (size_t)c * 8, acc);
    }
}

int combine_rows(void *out, const void *f_in, int dtype, const bf16 *yp, const int *inv, const float *gate,
                 int N, int D, int K, cudaStream_t st)
{
    k_combine_rows<<<(N + 7) / 8, 256, 0, st>>>(out, f_in, dtype, yp, inv, gate, N, D, K);
    QLMB_LAUNCH_CHECK("k_combine_rows");
    return QLMB_OK;
}

// ------------------------------------------------------------------- dgate
// Per permuted row j with slot n' = perm[j]: d_gate[n'] = dout[n].yp[j],
// dyp[j] = gate[n'] * dout[n]; filler rows are zeroed so they contribute
// nothing to the weight gradients (reference k_moe_dgate4, cudalm.cu:2569-2584).
__global__ void __launch_bounds__(256) k_dgate_rows(bf16 *dyp, float *d_gate, const void *dout, int dtype,
                                                    const bf16 *yp, const int *perm, const float *gate,
                                                    const int *nrows_dev, int nrows_host, int N, int D)
{
    int rows = nrows_dev ? *nrows_dev : nrows_host;
    int lane = threadIdx.x & 31;
    for (int j = blockIdx.x * 8 + (threadIdx.x >> 5); j < rows; j += gridDim.x * 8) {
        int np = perm[j];
        uint4 *o = reinterpret_cast<uint4 *>(dyp + (size_t)j * D);
        if (np < 0) {
            for (int c = lane; c < D / 8; c += 32) o[c] = make_uint4(0, 0, 0, 0);
            continue;
        }
        size_t base = (size_t)(np % N) * D;
        float g = gate[np], dot = 0.0f;
        for (int c = lane; c < D / 8; c += 32) {
            float dv[8], y[8];
            ld_act8(dout, dtype, base + (size_t)c * 8, dv);
            ld_act8(yp, QLMB_BF16, (size_t)j * D + (size_t)c * 8, y);
#pragma unroll
            for (int i = 0; i < 8; i++) { dot += dv[i] * y[i]; dv[i] *= g; }
            o[c] = pack_bf16x8(dv);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
        if (lane == 0) d_gate[np] = dot;
    }
}

int dgate_rows(bf16 *dyp, float *d_gate, const void *dout, int dtype, const bf16 *yp, const int *perm,
               const float *gate, const int *nrows_dev, int max_rows, int N, int D, cudaStream_t st)
{
    int blocks = (max_rows + 7) / 8;
    int cap = sm_count() * 8;
    if (blocks > cap) blocks = cap;
    k_dgate_rows<<<blocks, 256, 0, st>>>(dyp, d_gate, dout, dtype, yp, perm, gate, nrows_dev, max_rows, N, D);
    QLMB_LAUNCH_CHECK("k_dgate_rows");
    return QLMB_OK;
}

// ---------------------------------------------------------- router backward
// drt[n,:] = softmax Jacobian of (aux weights + gate gradients)
// (reference k_router_bwd_topk, cudalm.cu:2621-2629, with the aux weights
// w[e] = aux*E*(cnt[e]/(K*N))/N of cudalm.cu:4382 built on the device).
// One warp per token, lane = expert (E <= 32); the thread-per-token form below
// covers larger E.
__global__ void __launch_bounds__(256) k_router_bwd_warp(float *drt, const float *rprobs, const int *assign,
                                                         const float *d_gate, const int *counts, int N, int E,
                                                         int K, float aux)
{
    int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    float invN = 1.0f / N, invKN = 1.0f / ((float)K * N);
    float pr = lane < E ? rprobs[(size_t)n * E + lane] : 0.0f;
    float d = lane < E ? aux * E * ((float)counts[lane] * invKN) * invN : 0.0f;
    for (int k = 0; k < K; k++)
        if (assign[(size_t)k * N + n] == lane) d += d_gate[(size_t)k * N + n];
    float dot = pr * d;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane < E) drt[(size_t)n * E + lane] = pr * (d - dot);
}
__global__ void __launch_bounds__(128) k_router_bwd(float *drt, const float *rprobs, const int *assign,
                                                    const float *d_gate, const int *counts, int N, int E,
                                                    int K, float aux)
{
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const float *pr = rprobs + (size_t)n * E;
    float *d = drt + (size_t)n * E;
    float invN = 1.0f / N, invKN = 1.0f / ((float)K * N), dot = 0.0f;
    for (int e = 0; e < E; e++) d[e] = aux * E * ((float)counts[e] * invKN) * invN;
    for (int k = 0; k < K; k++) d[assign[(size_t)k * N + n]] += d_gate[(size_t)k * N + n];
    for (int e = 0; e < E; e++) dot += pr[e] * d[e];
    for (int e = 0; e < E; e++) d[e] = pr[e] * (d[e] - dot);
}

int router_bwd(float *drt, const float *rprobs, const int *assign, const float *d_gate, const int *counts,
               int N, int E, int K, float aux, cudaStream_t st)
{
    if (E <= 32) k_router_bwd_warp<<<(N + 7) / 8, 256, 0, st>>>(drt, rprobs, assign, d_gate, counts, N, E, K, aux);
    else k_router_bwd<<<(N + 127) / 128, 128, 0, st>>>(drt, rprobs, assign, d_gate, counts, N, E, K, aux);
    QLMB_LAUNCH_CHECK("k_router_bwd");
    return QLMB_OK;
}

// --------------------------------------------------------------- unpermute
// dfnorm[n,j] = sum_k dXp[inv[k,n], j] + sum_e drt[n,e] * Wr[j,e]
// (reference k_scatter_add + g_abt_b(drt, Wr), cudalm.cu:4368-4390).
// WrT is Wr transposed ([E][D], written by k_transpose_wr into scratch), so a
// lane's 8 consecutive features are two 16-byte loads that hit L1; a warp owns a
// token, a lane 8 consecutive features per pass.
__global__ void __launch_bounds__(256) k_transpose_wr(float *WrT, const float *Wr, int D, int E)
{
    int i = blockIdx.x * 256 + threadIdx.x;
    if (i < D * E) { int j = i / E, e = i % E; WrT[(size_t)e * D + j] = Wr[i]; }
}
__global__ void __launch_bounds__(256) k_unpermute_rows_warp(void *dfnorm, int dtype, const bf16 *dXp, const int *inv,
                                                             const float *drt, const float *WrT, int N, int D, int E, int K)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    float dr = lane < E ? drt[(size_t)n * E + lane] : 0.0f;
    int slot = lane < K ? inv[(size_t)lane * N + n] : 0;
    for (int j = lane * 8; j < D; j += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < K; k++) {
            int row = __shfl_sync(0xffffffffu, slot, k);
            float y[8];
            ld_act8(dXp, QLMB_BF16, (size_t)row * D + j, y);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] += y[i];
        }
#pragma unroll 4
        for (int e = 0; e < E; e++) {
            float dv = __shfl_sync(0xffffffffu, dr, e);
            float4 w0 = __ldg(reinterpret_cast<const float4 *>(WrT + (size_t)e * D + j));
            float4 w1 = __ldg(reinterpret_cast<const float4 *>(WrT + (size_t)e * D + j + 4));
            acc[0] += dv * w0.x; acc[1] += dv * w0.y; acc[2] += dv * w0.z; acc[3] += dv * w0.w;
            acc[4] += dv * w1.x; acc[5] += dv * w1.y; acc[6] += dv * w1.z; acc[7] += dv * w1.w;
        }
        st_act8(dfnorm, dtype, (size_t)n * D + j, acc);
    }
}

// General shape: a block owns 8 tokens; a thread owns feature columns j = tid, tid+256, ...
#define UP_TOK 8
__global__ void __launch_bounds__(256) k_unpermute_rows(void *dfnorm, int dtype, const bf16 *dXp,
                                                        const int *inv, const float *drt, const float *Wr,
                                                        int N, int D, int E, int K)
{
    extern __shared__ float sh[];         // drt tile [UP_TOK][E] then slot table [UP_TOK][K]
    float *dr = sh;
    int *slot = reinterpret_cast<int *>(sh + UP_TOK * E);
    int n0 = blockIdx.x * UP_TOK;
    for (int i = threadIdx.x; i < UP_TOK * E; i += 256) {
        int n = n0 + i / E;
        dr[i] = n < N ? drt[(size_t)n * E + i % E] : 0.0f;
    }
    for (int i = threadIdx.x; i < UP_TOK * K; i += 256) {
        int n = n0 + i / K, k = i % K;
        slot[i] = n < N ? inv[(size_t)k * N + n] : 0;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < D; j += 256) {
        float acc[UP_TOK];
#pragma unroll
        for (int t = 0; t < UP_TOK; t++) acc[t] = 0.0f;
        const float *w = Wr + (size_t)j * E;
        for (int e = 0; e < E; e++) {
            float wv = w[e];
#pragma unroll
            for (int t = 0; t < UP_TOK; t++) acc[t] += dr[t * E + e] * wv;
        }
#pragma unroll
        for (int t = 0; t < UP_TOK; t++) {
            int n = n0 + t;
            if (n >= N) break;
            float x = 0.0f;
            for (int k = 0; k < K; k++) x += __bfloat162float(dXp[(size_t)slot[t * K + k] * D + j]);
            st_act(dfnorm, dtype, (size_t)n * D + j, x + acc[t]);
        }
    }
}

int unpermute_rows(void *dfnorm, int dtype, const bf16 *dXp, const int *inv, const float *drt, const float *Wr,
                   float *wrt_scratch, int N, int D, int E, int K, cudaStream_t st)
{
    if (E <= 32 && (D % 8) == 0 && wrt_scratch) {
        k_transpose_wr<<<(D * E + 255) / 256, 256, 0, st>>>(wrt_scratch, Wr, D, E);
        k_unpermute_rows_warp<<<(N + 7) / 8, 256, 0, st>>>(dfnorm, dtype, dXp, inv, drt, wrt_scratch, N, D, E, K);
    } else {
        size_t smem = (size_t)UP_TOK * E * sizeof(float) + (size_t)UP_TOK * K * sizeof(int);
        k_unpermute_rows<<<(N + UP_TOK - 1) / UP_TOK, 256, smem, st>>>(dfnorm, dtype, dXp, inv, drt, Wr, N, D, E, K);
    }
    QLMB_LAUNCH_CHECK("k_unpermute_rows");
    return QLMB_OK;
}

// ------------------------------------------------------------ router wgrad
// dWr[j,e] = beta*dWr[j,e] + sum_n fnorm[n,j]*drt[n,e]  (reference g_atb,
// cudalm.cu:4391).  Stage 1: block (c, jb) sums token chunk c for the 256
// features of block jb in registers (warp = 32 features, lane = expert); stage 2
// adds the chunks in a fixed order, so the result is run-to-run identical.
#define RW_CHUNKS 192
__global__ void __launch_bounds__(256) k_router_wgrad_part(float *part, const void *fnorm, int dtype,
                                                           const float *drt, int N, int D, int E, int e0)
{
    const int c = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j0 = blockIdx.y * 256 + warp * 32;
    const int per = (N + RW_CHUNKS - 1) / RW_CHUNKS;
    const int n_lo = c * per, n_hi = n_lo + per < N ? n_lo + per : N;
    const int e = e0 + lane;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; i++) acc[i] = 0.0f;
    if (j0 < D) {
#pragma unroll 2
        for (int n = n_lo; n < n_hi; n++) {
            float dv = e < E ? drt[(size_t)n * E + e] : 0.0f;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                float x[8];
                if (j0 + i + 8 <= D) ld_act8(fnorm, dtype, (size_t)n * D + j0 + i, x);
                else {
#pragma unroll
                    for (int k = 0; k < 8; k++) x[k] = j0 + i + k < D ? ld_act(fnorm, dtype, (size_t)n * D + j0 + i + k) : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < 8; k++) acc[i + k] += x[k] * dv;
            }
        }
        if (e < E) {
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (j0 + i < D) part[((size_t)c * D + j0 + i) * E + e] = acc[i];
        }
    }
}
__global__ void __launch_bounds__(256) k_router_wgrad_sum(float *dWr, const float *part, int nchunk, int DE, float beta)
{
    int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= DE) return;
    float s = 0.0f;
    for (int c = 0; c < nchunk; c++) s += part[(size_t)c * DE + i];
    dWr[i] = (beta != 0.0f ? beta * dWr[i] : 0.0f) + s;
}

int router_wgrad(float *dWr, const void *fnorm, int dtype, const float *drt, float *scratch, int N, int D, int E,
                 float beta, cudaStream_t st)
{
    for (int e0 = 0; e0 < E; e0 += 32)
        k_router_wgrad_part<<<dim3(RW_CHUNKS, (D + 255) / 256), 256, 0, st>>>(scratch, fnorm, dtype, drt, N, D, E, e0);
    k_router_wgrad_sum<<<(D * E + 255) / 256, 256, 0, st>>>(dWr, scratch, RW_CHUNKS, D * E, beta);
    QLMB_LAUNCH_CHECK("router_wgrad");
    return QLMB_OK;
}

// ----------------------------------------------------------- conversions
__global__ void __launch_bounds__(256) k_f32_to_bf16(bf16 *dst, const float *src, size_t n8, size_t n)
{
    size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    size_t stride = (size_t)gridDim.x * 256;
    for (size_t c = i; c < n8; c += stride) {
        float v[8];
        ld_act8(src, QLMB_F32, c * 8, v);
        *reinterpret_cast<uint4 *>(dst + c * 8) = pack_bf16x8(v);
    }
    for (size_t k = n8 * 8 + i; k < n; k += stride) dst[k] = __float2bfloat16_rn(src[k]);
}
int convert_f32_to_bf16(bf16 *dst, const float *src, size_t n, cudaStream_t st)
{
    if (n == 0) return QLMB_OK;
    size_t n8 = n / 8;
    size_t blocks = (n8 + 255) / 256;
    size_t cap = (size_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    k_f32_to_bf16<<<(unsigned)blocks, 256, 0, st>>>(dst, src, n8, n);
    QLMB_LAUNCH_CHECK("k_f32_to_bf16");
    return QLMB_OK;
}

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_router_topk(const float *rt_in, float *rt_out, const void *X, int x_dtype, const float *Wr,
                                const float *bias, int bias_stride, float *rprobs, int *assign, float *gate,
                                int N, int D, int E, int K, void *stream)
{
    QLMB_REQUIRE(rprobs && assign && gate, "qlmb_router_topk: NULL output");
    QLMB_REQUIRE(N > 0 && E > 0 && E <= 256 && K > 0 && K <= 8 && K <= E, "qlmb_router_topk: N=%d E=%d K=%d", N, E, K);
    const float *rt = rt_in;
    if (!rt) {
        QLMB_REQUIRE(X && Wr && rt_out && D > 0, "qlmb_router_topk: logits need X, Wr and rt_out");
        QLMB_REQUIRE(x_dtype == QLMB_F32 || x_dtype == QLMB_BF16, "qlmb_router_topk: dtype %d", x_dtype);
        int rc = router_logits(rt_out, X, x_dtype, Wr, N, D, E, as_stream(stream));
        if (rc) return rc;
        rt = rt_out;
    }
    return router_topk(rt, rprobs, assign, gate, N, E, K, bias, bias_stride, as_stream(stream));
}
