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
// Register-tiled: a block of 256 threads owns 64 tokens, a thread 2 tokens (32 apart) x 4 experts.
// The token tile and Wr move through a ring of shared-memory stages, 32 features per stage,
// filled by cp.async three (bf16) or two (fp32) stages ahead of the multiply.  Each output is
// summed over the features in ascending order.
#define RLT_TOK 64
#define RLT_CH 32
__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool live)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = live ? 16 : 0;                         // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

template <int XBF16>
__global__ void __launch_bounds__(256) k_router_logits_tile(float *rt, const void *X, const float *Wr, int N, int D, int E)
{
    constexpr int NST = XBF16 ? 4 : 3;                   // stages
    constexpr int XROW = XBF16 ? 80 : 144;               // bytes per token row of a stage (64 / 128 + pad)
    __shared__ __align__(16) uint8_t xs[NST][RLT_TOK * XROW];
    __shared__ __align__(16) float ws[NST][RLT_CH][32];
    const int tid = threadIdx.x, n0 = blockIdx.x * RLT_TOK;
    const int tg = tid >> 3, eg = tid & 7;
    float acc[2][4];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[t][i] = 0.0f;
    const int nch = (D + RLT_CH - 1) / RLT_CH;
    auto fill = [&](int c) {
        if (c < nch) {
            const int st = c % NST, j0 = c * RLT_CH;
            // token tile: 16-byte pieces (8 bf16 or 4 fp32 features)
            constexpr int PPR = XBF16 ? 4 : 8;           // pieces per token row
#pragma unroll
            for (int i = 0; i < RLT_TOK * PPR / 256; i++) {
                const int p = tid + i * 256, tok = p / PPR, part = p % PPR;
                const int n = n0 + tok, j = j0 + part * (XBF16 ? 8 : 4);
                const bool live = n < N && j < D;
                const uint8_t *src = (const uint8_t *)X + (live ? ((size_t)n * D + j) * (XBF16 ? 2 : 4) : 0);
                cp_async16(&xs[st][tok * XROW + part * 16], src, live);
            }
            if (E == 32) {
                const int row = tid >> 3, c4 = tid & 7;
                const bool live = j0 + row < D;
                cp_async16(&ws[st][row][c4 * 4], Wr + (live ? (size_t)(j0 + row) * 32 + c4 * 4 : 0), live);
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int q = tid + i * 256, row = q >> 5, e = q & 31;
                    ws[st][row][e] = (e < E && j0 + row < D) ? __ldg(Wr + (size_t)(j0 + row) * E + e) : 0.0f;
                }
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int c = 0; c < NST - 1; c++) fill(c);
    for (int c = 0; c < nch; c++) {
        cp_async_wait<NST - 2>();
        __syncthreads();
        fill(c + NST - 1);
        const int st = c % NST;
#pragma unroll
        for (int kk = 0; kk < RLT_CH; kk += 4) {
            float xv[2][4];
#pragma unroll
            for (int t = 0; t < 2; t++) {
                const uint8_t *row = &xs[st][(tg + 32 * t) * XROW];
                if (XBF16) {
                    const uint2 q = *reinterpret_cast<const uint2 *>(row + kk * 2);
                    xv[t][0] = __uint_as_float(q.x << 16); xv[t][1] = __uint_as_float(q.x & 0xffff0000u);
                    xv[t][2] = __uint_as_float(q.y << 16); xv[t][3] = __uint_as_float(q.y & 0xffff0000u);
                } else {
                    const float4 q = *reinterpret_cast<const float4 *>(row + kk * 4);
                    xv[t][0] = q.x; xv[t][1] = q.y; xv[t][2] = q.z; xv[t][3] = q.w;
                }
            }
#pragma unroll
            for (int k4 = 0; k4 < 4; k4++) {
                const float4 w = *reinterpret_cast<const float4 *>(&ws[st][kk + k4][eg * 4]);
#pragma unroll
                for (int t = 0; t < 2; t++) {
                    const float x = xv[t][k4];
                    acc[t][0] += x * w.x; acc[t][1] += x * w.y; acc[t][2] += x * w.z; acc[t][3] += x * w.w;
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const int n = n0 + tg + 32 * t;
        if (n >= N) continue;
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (eg * 4 + i < E) rt[(size_t)n * E + eg * 4 + i] = acc[t][i];
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

// A handful of rows (a decode step): one block per token, lane = expert, eight warps each sum one eighth of the
// features in ascending order (loads of Wr rows are independent of the running sums, so they pipeline), and the
// eight partial sums are added in warp order.  Deterministic, but a different summation order than the tiled
// kernel, hence only used where no backward pass reads the logits.
__global__ void __launch_bounds__(256) k_router_logits_small(float *rt, const void *X, int x_dtype, const float *Wr, int D, int E)
{
    extern __shared__ float rl_x[];                      // D activations
    __shared__ float part[8][32];
    const int n = blockIdx.x, warp = threadIdx.x >> 5, e = threadIdx.x & 31;
    for (int j = threadIdx.x; j < D; j += 256) rl_x[j] = ld_act(X, x_dtype, (size_t)n * D + j);
    __syncthreads();
    const int per = (D + 7) / 8, j0 = warp * per, j1 = j0 + per < D ? j0 + per : D;
    float acc = 0.0f;
    if (e < E) {
#pragma unroll 8
        for (int j = j0; j < j1; j++) acc += rl_x[j] * __ldg(Wr + (size_t)j * E + e);
    }
    part[warp][e] = acc;
    __syncthreads();
    if (warp == 0 && e < E) {
        float s = part[0][e];
#pragma unroll
        for (int w = 1; w < 8; w++) s += part[w][e];
        rt[(size_t)n * E + e] = s;
    }
}
int router_logits_small(float *rt, const void *X, int x_dtype, const float *Wr, int N, int D, int E, cudaStream_t st)
{
    if (N > 64 || E > 32 || D > 8192) return router_logits(rt, X, x_dtype, Wr, N, D, E, st);
    k_router_logits_small<<<N, 256, (size_t)D * sizeof(float), st>>>(rt, X, x_dtype, Wr, D, E);
    QLMB_LAUNCH_CHECK("k_router_logits_small");
    return QLMB_OK;
}

int router_logits(float *rt, const void *X, int x_dtype, const float *Wr, int N, int D, int E, cudaStream_t st)
{
    if (E <= 32 && (D % 8) == 0 && (((uintptr_t)X | (uintptr_t)Wr) & 15) == 0) {
        int blocks = (N + RLT_TOK - 1) / RLT_TOK;
        if (x_dtype == QLMB_BF16) k_router_logits_tile<1><<<blocks, 256, 0, st>>>(rt, X, Wr, N, D, E);
        else k_router_logits_tile<0><<<blocks, 256, 0, st>>>(rt, X, Wr, N, D, E);
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
            ld_act8(yp, QLMB_BF16, (size_t)(inv ? inv[slot] : (int)slot) * D + (size_t)c * 8, y);
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
// WrT is Wr transposed ([E][D], written by k_transpose_wr into scratch), so that a
// feature slice of it is staged with 16-byte copies.
__global__ void __launch_bounds__(256) k_transpose_wr(float *WrT, const float *Wr, int D, int E)
{
    int i = blockIdx.x * 256 + threadIdx.x;
    if (i < D * E) { int j = i / E, e = i % E; WrT[(size_t)e * D + j] = Wr[i]; }
}
// Register-tiled: a block owns 256 features and walks over tiles of 32 tokens; warp = 4 tokens,
// lane = features [4*lane, 4*lane+4) and [128+4*lane, ...) of the block's slice.  The slice of WrT
// is staged in shared memory once per block, the tokens' drt rows and row indices per tile.
// With PEER the permuted rows live in the arena of the rank that owns the slot's expert
// (rows = that arena's row index per slot, read through the peer pointers).
#define UPT_TOK 32
#define UPT_F 256
template <bool PEER>
__global__ void __launch_bounds__(256, 3) k_unpermute_rows_tile(void *dfnorm, int dtype, const bf16 *dXp, PeerPtrs dXpP,
                                                                const int *rows, const int *assign, int el, const float *drt,
                                                                const float *WrT, int N, int D, int E, int K)
{
    __shared__ __align__(16) float ws[32][UPT_F];
    __shared__ __align__(16) float drs[UPT_TOK][32];
    __shared__ int srow[UPT_TOK][8], sown[UPT_TOK][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int j0 = blockIdx.y * UPT_F;
    const int jA = j0 + lane * 4, jB = jA + 128;
    for (int i = tid; i < 32 * (UPT_F / 4); i += 256) {
        const int e = i / (UPT_F / 4), c = i % (UPT_F / 4), j = j0 + c * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < E && j < D) v = __ldg(reinterpret_cast<const float4 *>(WrT + (size_t)e * D + j));
        *reinterpret_cast<float4 *>(&ws[e][c * 4]) = v;
    }
    const int ntiles = (N + UPT_TOK - 1) / UPT_TOK;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int n0 = tile * UPT_TOK;
        __syncthreads();                                 // the previous tile's reads of drs / srow are done
        for (int i = tid; i < UPT_TOK * K; i += 256) {
            const int t = i / K, k = i % K, n = n0 + t;
            int row = -1, own = 0;
            if (n < N) {
                const size_t slot = (size_t)k * N + n;
                row = rows ? __ldg(rows + slot) : (int)slot;
                if (PEER) own = __ldg(assign + slot) / el;
            }
            srow[t][k] = row; sown[t][k] = own;
        }
        for (int i = tid; i < UPT_TOK * 32; i += 256) {
            const int n = n0 + (i >> 5), e = i & 31;
            drs[i >> 5][e] = (n < N && e < E) ? drt[(size_t)n * E + e] : 0.0f;
        }
        __syncthreads();
        // the K permuted rows of the warp's 4 tokens: all loads of one k are in flight together
        float acc[4][8];
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int i = 0; i < 8; i++) acc[t][i] = 0.0f;
        for (int k = 0; k < K; k++) {
            uint2 qa[4], qb[4];
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const int row = srow[warp * 4 + t][k];
                qa[t] = qb[t] = make_uint2(0u, 0u);
                if (row >= 0) {
                    const bf16 *src = (PEER ? (const bf16 *)dXpP.p[sown[warp * 4 + t][k]] : dXp) + (size_t)row * D;
                    if (jA < D) qa[t] = *reinterpret_cast<const uint2 *>(src + jA);
                    if (jB < D) qb[t] = *reinterpret_cast<const uint2 *>(src + jB);
                }
            }
#pragma unroll
            for (int t = 0; t < 4; t++) {
                float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&qa[t].x));
                float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&qa[t].y));
                acc[t][0] += a.x; acc[t][1] += a.y; acc[t][2] += b.x; acc[t][3] += b.y;
                a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&qb[t].x));
                b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&qb[t].y));
                acc[t][4] += a.x; acc[t][5] += a.y; acc[t][6] += b.x; acc[t][7] += b.y;
            }
        }
#pragma unroll 2
        for (int e4 = 0; e4 < 32; e4 += 4) {
            float4 dv[4];
#pragma unroll
            for (int t = 0; t < 4; t++) dv[t] = *reinterpret_cast<const float4 *>(&drs[warp * 4 + t][e4]);
#pragma unroll
            for (int k4 = 0; k4 < 4; k4++) {
                const float4 wa = *reinterpret_cast<const float4 *>(&ws[e4 + k4][lane * 4]);
                const float4 wb = *reinterpret_cast<const float4 *>(&ws[e4 + k4][128 + lane * 4]);
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const float d = k4 == 0 ? dv[t].x : k4 == 1 ? dv[t].y : k4 == 2 ? dv[t].z : dv[t].w;
                    acc[t][0] += d * wa.x; acc[t][1] += d * wa.y; acc[t][2] += d * wa.z; acc[t][3] += d * wa.w;
                    acc[t][4] += d * wb.x; acc[t][5] += d * wb.y; acc[t][6] += d * wb.z; acc[t][7] += d * wb.w;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const int n = n0 + warp * 4 + t;
            if (n >= N) continue;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int j = h ? jB : jA;
                if (j >= D) continue;
                const float *v = &acc[t][h * 4];
                if (dtype == QLMB_BF16) {
                    uint2 q;
                    *reinterpret_cast<__nv_bfloat162 *>(&q.x) = __floats2bfloat162_rn(v[0], v[1]);
                    *reinterpret_cast<__nv_bfloat162 *>(&q.y) = __floats2bfloat162_rn(v[2], v[3]);
                    *reinterpret_cast<uint2 *>((bf16 *)dfnorm + (size_t)n * D + j) = q;
                } else {
                    *reinterpret_cast<float4 *>((float *)dfnorm + (size_t)n * D + j) = make_float4(v[0], v[1], v[2], v[3]);
                }
            }
        }
    }
}
static dim3 unpermute_grid(int N, int D)
{
    const int ny = (D + UPT_F - 1) / UPT_F, ntiles = (N + UPT_TOK - 1) / UPT_TOK;
    int gx = 3 * sm_count() / ny;
    if (gx < 1) gx = 1;
    if (gx > ntiles) gx = ntiles;
    const int per = (ntiles + gx - 1) / gx;              // whole tiles per block, evenly
    gx = (ntiles + per - 1) / per;
    return dim3(gx, ny);
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
        PeerPtrs none = {};
        k_unpermute_rows_tile<false><<<unpermute_grid(N, D), 256, 0, st>>>(dfnorm, dtype, dXp, none, inv, nullptr, 1, drt, wrt_scratch, N, D, E, K);
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
// Register-tiled stage 1 for E <= 32: block (c, jb) owns token chunk c and 128 features; a
// thread 4 features x 4 experts.  Tokens are staged 32 at a time (fp32 in shared memory,
// next sub-chunk prefetched into registers during the multiply).
#define RWT_F 128
#define RWT_SUB 32
template <int XBF16>
__global__ void __launch_bounds__(256) k_router_wgrad_tile(float *part, const void *fnorm, const float *drt,
                                                           int N, int D, int E, int per)
{
    __shared__ __align__(16) float xs[2][RWT_SUB][RWT_F];
    __shared__ __align__(16) float ds[2][RWT_SUB][32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, j0 = blockIdx.y * RWT_F;
    const int n_lo = c * per, n_hi = n_lo + per < N ? n_lo + per : N;
    const int eg = lane & 7, fg = warp * 4 + (lane >> 3);
    float acc[4][4];
#pragma unroll
    for (int f = 0; f < 4; f++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[f][i] = 0.0f;
    float xr[2][8], dr[4];
    auto fetch = [&](int nb) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int p = tid + i * 256, n = nb + (p >> 4), j = j0 + (p & 15) * 8;
            if (n < n_hi && j < D) ld_act8(fnorm, XBF16 ? QLMB_BF16 : QLMB_F32, (size_t)n * D + j, xr[i]);
            else {
#pragma unroll
                for (int k = 0; k < 8; k++) xr[i][k] = 0.0f;
            }
        }
        const int n = nb + (tid >> 3);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = (tid & 7) * 4 + i;
            dr[i] = (n < n_hi && e < E) ? drt[(size_t)n * E + e] : 0.0f;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int p = tid + i * 256;
            float *o = &xs[buf][p >> 4][(p & 15) * 8];
            *reinterpret_cast<float4 *>(o) = make_float4(xr[i][0], xr[i][1], xr[i][2], xr[i][3]);
            *reinterpret_cast<float4 *>(o + 4) = make_float4(xr[i][4], xr[i][5], xr[i][6], xr[i][7]);
        }
        *reinterpret_cast<float4 *>(&ds[buf][tid >> 3][(tid & 7) * 4]) = make_float4(dr[0], dr[1], dr[2], dr[3]);
    };
    fetch(n_lo);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int nb = n_lo; nb < n_hi; nb += RWT_SUB, buf ^= 1) {
        const bool more = nb + RWT_SUB < n_hi;
        if (more) fetch(nb + RWT_SUB);
#pragma unroll 8
        for (int t = 0; t < RWT_SUB; t++) {
            const float4 x = *reinterpret_cast<const float4 *>(&xs[buf][t][fg * 4]);
            const float4 d = *reinterpret_cast<const float4 *>(&ds[buf][t][eg * 4]);
            acc[0][0] += x.x * d.x; acc[0][1] += x.x * d.y; acc[0][2] += x.x * d.z; acc[0][3] += x.x * d.w;
            acc[1][0] += x.y * d.x; acc[1][1] += x.y * d.y; acc[1][2] += x.y * d.z; acc[1][3] += x.y * d.w;
            acc[2][0] += x.z * d.x; acc[2][1] += x.z * d.y; acc[2][2] += x.z * d.z; acc[2][3] += x.z * d.w;
            acc[3][0] += x.w * d.x; acc[3][1] += x.w * d.y; acc[3][2] += x.w * d.z; acc[3][3] += x.w * d.w;
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int f = 0; f < 4; f++) {
        const int j = j0 + fg * 4 + f;
        if (j >= D) continue;
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (eg * 4 + i < E) part[((size_t)c * D + j) * E + eg * 4 + i] = acc[f][i];
    }
}
// four lanes per output: each adds one quarter of the chunks in ascending order, then the quarters
// are combined as (q0 + q1) + (q2 + q3) -- a fixed order, so the result is run-to-run identical
__global__ void __launch_bounds__(256) k_router_wgrad_sum(float *dWr, const float *part, int nchunk, int DE, float beta)
{
    const int gid = blockIdx.x * 256 + threadIdx.x, i = gid >> 2, q = gid & 3;
    const int per = (nchunk + 3) / 4, c0 = q * per, c1 = c0 + per < nchunk ? c0 + per : nchunk;
    float s = 0.0f;
    if (i < DE)
        for (int c = c0; c < c1; c++) s += part[(size_t)c * DE + i];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (i < DE && q == 0) dWr[i] = (beta != 0.0f ? beta * dWr[i] : 0.0f) + s;
}

int router_wgrad(float *dWr, const void *fnorm, int dtype, const float *drt, float *scratch, int N, int D, int E,
                 float beta, cudaStream_t st)
{
    int nchunk = RW_CHUNKS;
    if (E <= 32 && (D % 8) == 0) {
        const int fblocks = (D + RWT_F - 1) / RWT_F;
        int want = 4 * sm_count() / fblocks;
        if (want < 1) want = 1;
        if (want > RW_CHUNKS) want = RW_CHUNKS;
        int per = ((N + want - 1) / want + RWT_SUB - 1) / RWT_SUB * RWT_SUB;
        nchunk = (N + per - 1) / per;
        if (dtype == QLMB_BF16) k_router_wgrad_tile<1><<<dim3(nchunk, fblocks), 256, 0, st>>>(scratch, fnorm, drt, N, D, E, per);
        else k_router_wgrad_tile<0><<<dim3(nchunk, fblocks), 256, 0, st>>>(scratch, fnorm, drt, N, D, E, per);
    } else {
        for (int e0 = 0; e0 < E; e0 += 32)
            k_router_wgrad_part<<<dim3(RW_CHUNKS, (D + 255) / 256), 256, 0, st>>>(scratch, fnorm, dtype, drt, N, D, E, e0);
    }
    k_router_wgrad_sum<<<(4 * D * E + 255) / 256, 256, 0, st>>>(dWr, scratch, nchunk, D * E, beta);
    QLMB_LAUNCH_CHECK("router_wgrad");
    return QLMB_OK;
}

// ------------------------------------------------- expert parallelism by peer loads
// Rows that belong to another GPU are read through peer pointers (plain loads over NVLink)
// inside the row kernels themselves, so no separate exchange step exists.  Global slot
// g = s * KN + k * Nh + n names copy k of token n of rank s (Nh tokens per rank, KN = K * Nh).
// A PeerPtrs holds, per rank, the address of the same buffer in that rank's window.

// expert side: Xp[j] = f_norm of rank s, token n, for perm[j] = g (zero rows where perm[j] < 0)
__global__ void __launch_bounds__(256) k_gather_rows_peer(bf16 *Xp, PeerPtrs src, int dtype, const int *perm,
                                                          const int *nrows_dev, int Nh, int KN, int D)
{
    const int rows = *nrows_dev, lane = threadIdx.x & 31;
    for (int j = blockIdx.x * 8 + (threadIdx.x >> 5); j < rows; j += gridDim.x * 8) {
        const int g = perm[j];
        uint4 *o = reinterpret_cast<uint4 *>(Xp + (size_t)j * D);
        if (g < 0) {
            for (int c = lane; c < D / 8; c += 32) o[c] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int s = g / KN, n = (g % KN) % Nh;
        const size_t base = (size_t)n * D;
        if (dtype == QLMB_BF16) {
            const uint4 *r = reinterpret_cast<const uint4 *>((const bf16 *)src.p[s] + base);
            for (int c = lane; c < D / 8; c += 32) o[c] = r[c];
        } else {
            for (int c = lane; c < D / 8; c += 32) {
                float v[8];
                ld_act8(src.p[s], QLMB_F32, base + (size_t)c * 8, v);
                o[c] = pack_bf16x8(v);
            }
        }
    }
}

// The same gather with bulk copies: a warp moves whole rows (D bf16) peer -> shared -> local global
// memory, two rows in flight per warp, so NVLink sees large requests and no row passes through
// registers.  Waits are bounded; a timeout sets the device error word and leaves.
__device__ __forceinline__ uint32_t rk_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool rk_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < (1u << 22); i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__global__ void __launch_bounds__(256) k_gather_rows_peer_bulk(bf16 *Xp, PeerPtrs src, const int *perm, const int *nrows_dev,
                                                               int Nh, int KN, int D, int *errword)
{
    extern __shared__ __align__(128) uint8_t rowbuf[];         // [8 warps][2][D * 2 bytes]
    __shared__ __align__(8) uint64_t bars[8][2];
    const int rows = *nrows_dev, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rb = (uint32_t)D * 2u;
    uint8_t *buf = rowbuf + (size_t)warp * 2 * rb;
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rk_smem(&bars[warp][0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rk_smem(&bars[warp][1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const int stride = gridDim.x * 8;
    int it = 0;
    uint32_t ph[2] = {0u, 0u};
    // issue(j, b): start fetching row j into buffer b (or nothing for a filler row)
    auto issue = [&](int j, int b) {
        if (lane == 0 && j < rows) {
            const int g = perm[j];
            if (g >= 0) {
                // the buffer's previous store must have finished reading it
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                const int s = g / KN, n = (g % KN) % Nh;
                const uint32_t bar = rk_smem(&bars[warp][b]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(rb) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(rk_smem(buf + (size_t)b * rb)), "l"((const bf16 *)src.p[s] + (size_t)n * D), "r"(rb), "r"(bar) : "memory");
            }
        }
    };
    int j = blockIdx.x * 8 + warp;
    issue(j, 0);
    for (; j < rows; j += stride, it++) {
        const int b = it & 1;
        issue(j + stride, b ^ 1);
        const int g = perm[j];
        if (g < 0) {
            uint4 *o = reinterpret_cast<uint4 *>(Xp + (size_t)j * D);
            for (int c = lane; c < D / 8; c += 32) o[c] = make_uint4(0, 0, 0, 0);
            continue;
        }
        if (!rk_wait(rk_smem(&bars[warp][b]), ph[b])) {
            if (lane == 0 && errword && atomicCAS(errword, 0, 210) == 0) { errword[1] = j; errword[2] = (int)blockIdx.x; }
            break;
        }
        ph[b] ^= 1u;
        if (lane == 0) {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(Xp + (size_t)j * D), "r"(rk_smem(buf + (size_t)b * rb)), "r"(rb) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        __syncwarp();
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// home side: d_gate[slot] = dout[n] . y[slot], y = the row copies kept by the combine (one warp per slot)
__global__ void __launch_bounds__(256) k_dgate_dot_peer(float *d_gate, const void *dout, int dtype, const bf16 *ykeep,
                                                        int N, int D, int KN)
{
    const int slot = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (slot >= KN) return;
    const int n = slot % N;
    const void *y = ykeep;
    const size_t yb = (size_t)slot * D, db = (size_t)n * D;
    float dot = 0.0f;
    for (int c = lane; c < D / 8; c += 32) {
        float dv[8], yv[8];
        ld_act8(dout, dtype, db + (size_t)c * 8, dv);
        ld_act8(y, QLMB_BF16, yb + (size_t)c * 8, yv);
#pragma unroll
        for (int i = 0; i < 8; i++) dot += dv[i] * yv[i];
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
    if (lane == 0) d_gate[slot] = dot;
}

// expert side: dyp[j] = gate_s[slot] * dout_s[n] for perm[j] = s * KN + slot (zero filler rows)
__global__ void __launch_bounds__(256) k_dyp_rows_peer(bf16 *dyp, PeerPtrs dout, PeerPtrs gate, int dtype, const int *perm,
                                                       const int *nrows_dev, int Nh, int KN, int D)
{
    const int rows = *nrows_dev, lane = threadIdx.x & 31;
    for (int j = blockIdx.x * 8 + (threadIdx.x >> 5); j < rows; j += gridDim.x * 8) {
        const int g = perm[j];
        uint4 *o = reinterpret_cast<uint4 *>(dyp + (size_t)j * D);
        if (g < 0) {
            for (int c = lane; c < D / 8; c += 32) o[c] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int s = g / KN, slot = g % KN, n = slot % Nh;
        const float gv = ((const float *)gate.p[s])[slot];
        for (int c = lane; c < D / 8; c += 32) {
            float dv[8];
            ld_act8(dout.p[s], dtype, (size_t)n * D + (size_t)c * 8, dv);
#pragma unroll
            for (int i = 0; i < 8; i++) dv[i] *= gv;
            o[c] = pack_bf16x8(dv);
        }
    }
}

// counts[e] = how many of the K*N slots chose expert e (integer atomics: order independent);
// a block counts in shared memory first, so the global array sees E adds per block
__global__ void __launch_bounds__(256) k_count_assign(int *counts, const int *assign, int KN, int E)
{
    __shared__ int h[256];
    for (int e = threadIdx.x; e < E; e += 256) h[e] = 0;
    __syncthreads();
    for (int i = blockIdx.x * 256 + threadIdx.x; i < KN; i += gridDim.x * 256) {
        const int e = assign[i];
        if ((unsigned)e < (unsigned)E) atomicAdd(&h[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += 256) if (h[e]) atomicAdd(&counts[e], h[e]);
}

int gather_rows_peer(bf16 *Xp, const PeerPtrs &src, int dtype, const int *perm, const int *nrows_dev, int max_rows,
                     int Nh, int KN, int D, cudaStream_t st)
{
    int blocks = (max_rows + 7) / 8, cap = sm_count() * 8;
    if (blocks > cap) blocks = cap;
    static int bulk = -1;
    if (bulk < 0) { const char *e = getenv("QLMB_PEER_BULK"); bulk = (e && atoi(e) == 0) ? 0 : 1; }
    if (bulk && dtype == QLMB_BF16 && (D % 8) == 0 && (size_t)D * 2 * 16 <= 48 * 1024) {
        k_gather_rows_peer_bulk<<<blocks, 256, (size_t)D * 2 * 16, st>>>(Xp, src, perm, nrows_dev, Nh, KN, D, device_error_word());
        QLMB_LAUNCH_CHECK("k_gather_rows_peer_bulk");
        return QLMB_OK;
    }
    k_gather_rows_peer<<<blocks, 256, 0, st>>>(Xp, src, dtype, perm, nrows_dev, Nh, KN, D);
    QLMB_LAUNCH_CHECK("k_gather_rows_peer");
    return QLMB_OK;
}
int dgate_dot_peer(float *d_gate, const void *dout, int dtype, const bf16 *ykeep, int N, int D, int K, cudaStream_t st)
{
    k_dgate_dot_peer<<<(K * N + 7) / 8, 256, 0, st>>>(d_gate, dout, dtype, ykeep, N, D, K * N);
    QLMB_LAUNCH_CHECK("k_dgate_dot_peer");
    return QLMB_OK;
}
int dyp_rows_peer(bf16 *dyp, const PeerPtrs &dout, const PeerPtrs &gate, int dtype, const int *perm, const int *nrows_dev,
                  int max_rows, int Nh, int KN, int D, cudaStream_t st)
{
    int blocks = (max_rows + 7) / 8, cap = sm_count() * 8;
    if (blocks > cap) blocks = cap;
    k_dyp_rows_peer<<<blocks, 256, 0, st>>>(dyp, dout, gate, dtype, perm, nrows_dev, Nh, KN, D);
    QLMB_LAUNCH_CHECK("k_dyp_rows_peer");
    return QLMB_OK;
}
int count_assign(int *counts, const int *assign, int KN, int E, cudaStream_t st)
{
    QLMB_CUDA(cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int), st));
    int cb = (KN + 1023) / 1024;
    if (cb > 64) cb = 64;
    k_count_assign<<<cb, 256, 0, st>>>(counts, assign, KN, E);
    QLMB_LAUNCH_CHECK("k_count_assign");
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
