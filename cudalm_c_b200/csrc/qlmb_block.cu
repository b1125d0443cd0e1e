// The memory-bound operators around the GEMMs of a transformer block: embedding gather and its
// gradient, RMSNorm forward / backward / gain gradient, rotary embedding, softmax + cross-entropy.
// Activations are fp32 or bf16 (a dtype argument per tensor); all arithmetic is fp32.  Every
// kernel gives run-to-run identical results: no floating-point atomics, fixed summation orders.
#include <cuda_bf16.h>
#include <math.h>
#include "qlmb_common.cuh"

namespace qlmb {

typedef __nv_bfloat16 bf16_t;

__device__ __forceinline__ float blk_ld(const void *p, int dtype, size_t i)
{
    return dtype == QLMB_BF16 ? __bfloat162float(((const bf16_t *)p)[i]) : ((const float *)p)[i];
}
__device__ __forceinline__ void blk_st(void *p, int dtype, size_t i, float v)
{
    if (dtype == QLMB_BF16) ((bf16_t *)p)[i] = __float2bfloat16_rn(v);
    else ((float *)p)[i] = v;
}
// four consecutive elements (i a multiple of 4, rows 16-byte aligned for fp32 / 8-byte for bf16)
__device__ __forceinline__ float4 blk_ld4(const void *p, int dtype, size_t i)
{
    if (dtype == QLMB_BF16) {
        const uint2 q = *reinterpret_cast<const uint2 *>((const bf16_t *)p + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&q.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&q.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return *reinterpret_cast<const float4 *>((const float *)p + i);
}
__device__ __forceinline__ void blk_st4(void *p, int dtype, size_t i, float4 v)
{
    if (dtype == QLMB_BF16) {
        uint2 q;
        *reinterpret_cast<__nv_bfloat162 *>(&q.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162 *>(&q.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2 *>((bf16_t *)p + i) = q;
    } else {
        *reinterpret_cast<float4 *>((float *)p + i) = v;
    }
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------ embedding
// X[n,:] = emb[tok[n],:]  (k_embed, cpu_kern.h:87-90).  One warp per token row.
__global__ void __launch_bounds__(256) k_embed(void *X, int x_dtype, const float *emb, const int *tok, int N, int D)
{
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    const float *src = emb + (size_t)tok[n] * D;
    for (int j = lane * 4; j < D; j += 128) blk_st4(X, x_dtype, (size_t)n * D + j, *reinterpret_cast<const float4 *>(src + j));
}
// G[tok[n],:] += dout[n,:] with the rows of one token added in ascending n (k_embed_bwd,
// cpu_kern.h:92-98; the reference's GPU kernel uses atomics, its CPU twin this fixed order).
// One warp per vocabulary row: it scans the token list 32 positions at a time and adds the rows
// that match, so a row of G has one writer.  Work is V*N/32 warp steps -- sized for vocabularies
// and batches of tens of thousands.
template <int NV>
__global__ void __launch_bounds__(256) k_embed_bwd(float *G, const void *dout, int dtype, const int *tok, int N, int D, int V)
{
    __shared__ int stok[2048];
    const int v = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    float4 acc[NV];
#pragma unroll
    for (int k = 0; k < NV; k++) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    bool any = false;
    for (int n0 = 0; n0 < N; n0 += 2048) {
        __syncthreads();
        for (int i = threadIdx.x; i < 2048; i += 256) stok[i] = n0 + i < N ? tok[n0 + i] : -1;
        __syncthreads();
        const int lim = N - n0 < 2048 ? N - n0 : 2048;
        for (int c = 0; c < lim; c += 32) {
            unsigned m = __ballot_sync(0xffffffffu, stok[c + lane] == v);
            while (m) {
                const int n = n0 + c + __ffs(m) - 1;
                m &= m - 1;
                any = true;
#pragma unroll
                for (int k = 0; k < NV; k++) {
                    const int j = lane * 4 + k * 128;
                    if (j < D) {
                        const float4 d = blk_ld4(dout, dtype, (size_t)n * D + j);
                        acc[k].x += d.x; acc[k].y += d.y; acc[k].z += d.z; acc[k].w += d.w;
                    }
                }
            }
        }
    }
    if (v < V && any) {
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int j = lane * 4 + k * 128;
            if (j < D) {
                float4 g = *reinterpret_cast<float4 *>(G + (size_t)v * D + j);
                g.x += acc[k].x; g.y += acc[k].y; g.z += acc[k].z; g.w += acc[k].w;
                *reinterpret_cast<float4 *>(G + (size_t)v * D + j) = g;
            }
        }
    }
}

// ------------------------------------------------------------------ RMSNorm
// O = X * rinv * gamma, rinv = 1/sqrt(mean(x^2) + 1e-5)  (k_rmsnorm, cpu_kern.h:103-109).  Warp per row.
__global__ void __launch_bounds__(256) k_rmsnorm_fwd(void *O, int o_dtype, float *rinv, const void *X, int x_dtype,
                                                     const float *gamma, int N, int D)
{
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    float ss = 0.0f;
    for (int j = lane * 4; j < D; j += 128) {
        const float4 x = blk_ld4(X, x_dtype, (size_t)n * D + j);
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    ss = warp_sum(ss);
    const float s = 1.0f / sqrtf(ss / (float)D + 1e-5f);
    if (lane == 0) rinv[n] = s;
    for (int j = lane * 4; j < D; j += 128) {
        const float4 x = blk_ld4(X, x_dtype, (size_t)n * D + j);
        const float4 g = *reinterpret_cast<const float4 *>(gamma + j);
        blk_st4(O, o_dtype, (size_t)n * D + j, make_float4(x.x * s * g.x, x.y * s * g.y, x.z * s * g.z, x.w * s * g.w));
    }
}
// dx (+)= s*g*dy - (s^3/D * sum(x*g*dy)) * x   (k_rmsnorm_bwd, cpu_kern.h:110-119)
__global__ void __launch_bounds__(256) k_rmsnorm_bwd(void *dx, int dx_dtype, int accumulate, const void *X, int x_dtype,
                                                     const float *gamma, const float *rinv, const void *dy, int dy_dtype,
                                                     int N, int D)
{
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    float c = 0.0f;
    for (int j = lane * 4; j < D; j += 128) {
        const float4 x = blk_ld4(X, x_dtype, (size_t)n * D + j), d = blk_ld4(dy, dy_dtype, (size_t)n * D + j);
        const float4 g = *reinterpret_cast<const float4 *>(gamma + j);
        c += x.x * g.x * d.x + x.y * g.y * d.y + x.z * g.z * d.z + x.w * g.w * d.w;
    }
    c = warp_sum(c);
    const float s = rinv[n], cf = s * s * s / (float)D * c;
    for (int j = lane * 4; j < D; j += 128) {
        const float4 x = blk_ld4(X, x_dtype, (size_t)n * D + j), d = blk_ld4(dy, dy_dtype, (size_t)n * D + j);
        const float4 g = *reinterpret_cast<const float4 *>(gamma + j);
        float4 r = make_float4(s * g.x * d.x - cf * x.x, s * g.y * d.y - cf * x.y, s * g.z * d.z - cf * x.z, s * g.w * d.w - cf * x.w);
        if (accumulate) {
            const float4 o = blk_ld4(dx, dx_dtype, (size_t)n * D + j);
            r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w;
        }
        blk_st4(dx, dx_dtype, (size_t)n * D + j, r);
    }
}
// Gain gradient in two deterministic stages (k_gamma_part / k_gamma_sum, cudalm.cu:927-940,
// cpu_kern.h:128-138): 128 fixed row chunks, each summed over its rows in ascending order, then the
// chunks in ascending order, added to G.
#define GAMMA_CH 128
__global__ void __launch_bounds__(128) k_gamma_part(float *part, const void *X, int x_dtype, const float *rinv, const void *dy,
                                                    int dy_dtype, int N, int D)
{
    const int c = blockIdx.y, j = blockIdx.x * 128 + threadIdx.x;
    if (j >= D) return;
    const int r0 = (int)((long long)N * c / GAMMA_CH), r1 = (int)((long long)N * (c + 1) / GAMMA_CH);
    float acc = 0.0f;
    int n = r0;
    for (; n + 8 <= r1; n += 8) {                        // eight rows of loads in flight, added in row order
        float x[8], d[8], r[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            x[k] = blk_ld(X, x_dtype, (size_t)(n + k) * D + j); d[k] = blk_ld(dy, dy_dtype, (size_t)(n + k) * D + j); r[k] = __ldg(rinv + n + k);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) acc += x[k] * r[k] * d[k];
    }
    for (; n < r1; n++) acc += blk_ld(X, x_dtype, (size_t)n * D + j) * rinv[n] * blk_ld(dy, dy_dtype, (size_t)n * D + j);
    part[(size_t)c * D + j] = acc;
}
__global__ void __launch_bounds__(128) k_gamma_sum(float *G, const float *part, int D)
{
    const int j = blockIdx.x * 128 + threadIdx.x;
    if (j >= D) return;
    float a = 0.0f;
    for (int c = 0; c < GAMMA_CH; c++) a += part[(size_t)c * D + j];
    G[j] += a;
}

// ------------------------------------------------------------------ rotary embedding
// In place on buf[N, nh, hd]; position of row n is n % T; pairs (i, i + hd/2)  (k_rope, cpu_kern.h:139-152).
__global__ void __launch_bounds__(256) k_rope(void *buf, int dtype, const float *cosb, const float *sinb, size_t total, int nh,
                                              int hd, int T, int back)
{
    const size_t g = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (g >= total) return;
    const int hf = hd / 2, i = (int)(g % hf);
    const size_t vh = g / hf;                            // (row, head)
    const size_t n = vh / nh;
    const float cs = cosb[(size_t)(n % T) * hf + i], sn = sinb[(size_t)(n % T) * hf + i];
    const size_t o = vh * hd + i;
    const float a = blk_ld(buf, dtype, o), b = blk_ld(buf, dtype, o + hf);
    float ra, rb;
    if (back) { ra = a * cs + b * sn; rb = -a * sn + b * cs; }
    else { ra = a * cs - b * sn; rb = b * cs + a * sn; }
    blk_st(buf, dtype, o, ra);
    blk_st(buf, dtype, o + hf, rb);
}

// hd/2 a multiple of 8: a thread rotates 8 consecutive pairs with 16-byte accesses
__global__ void __launch_bounds__(256) k_rope8(void *buf, int dtype, const float *cosb, const float *sinb, size_t total, int nh,
                                               int hd, int T, int back)
{
    const size_t g = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (g >= total) return;
    const int hf = hd / 2, per = hf / 8, i = (int)(g % per) * 8;
    const size_t vh = g / per, n = vh / nh, o = vh * hd + i;
    const float *cp = cosb + (size_t)(n % T) * hf + i, *sp = sinb + (size_t)(n % T) * hf + i;
    float a[8], b[8], cs[8], sn[8];
    *reinterpret_cast<float4 *>(cs) = *reinterpret_cast<const float4 *>(cp);
    *reinterpret_cast<float4 *>(cs + 4) = *reinterpret_cast<const float4 *>(cp + 4);
    *reinterpret_cast<float4 *>(sn) = *reinterpret_cast<const float4 *>(sp);
    *reinterpret_cast<float4 *>(sn + 4) = *reinterpret_cast<const float4 *>(sp + 4);
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const float4 x = blk_ld4(buf, dtype, o + 4 * k), y = blk_ld4(buf, dtype, o + hf + 4 * k);
        a[4 * k] = x.x; a[4 * k + 1] = x.y; a[4 * k + 2] = x.z; a[4 * k + 3] = x.w;
        b[4 * k] = y.x; b[4 * k + 1] = y.y; b[4 * k + 2] = y.z; b[4 * k + 3] = y.w;
    }
    float ra[8], rb[8];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        if (back) { ra[k] = a[k] * cs[k] + b[k] * sn[k]; rb[k] = -a[k] * sn[k] + b[k] * cs[k]; }
        else { ra[k] = a[k] * cs[k] - b[k] * sn[k]; rb[k] = b[k] * cs[k] + a[k] * sn[k]; }
    }
#pragma unroll
    for (int k = 0; k < 2; k++) {
        blk_st4(buf, dtype, o + 4 * k, make_float4(ra[4 * k], ra[4 * k + 1], ra[4 * k + 2], ra[4 * k + 3]));
        blk_st4(buf, dtype, o + hf + 4 * k, make_float4(rb[4 * k], rb[4 * k + 1], rb[4 * k + 2], rb[4 * k + 3]));
    }
}

// ------------------------------------------------------------------ softmax + cross-entropy
// Per row: loss = -log(p[tgt] + 1e-12), dl = (p - onehot) / n_all; rows with tgt < 0 give loss 0 and a
// zero gradient row  (k_softmax_ce, cpu_kern.h:489-503, without per-token weights).  Block per row.
__global__ void __launch_bounds__(256) k_softmax_ce(const void *lg, int lg_dtype, const int *tgt, float *loss, void *dl,
                                                    int dl_dtype, int V, int n_all)
{
    __shared__ float red[8];
    __shared__ float bc;
    const size_t row = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, tg = tgt[row];
    if (tg < 0) {
        for (int i = tid; i < V; i += 256) blk_st(dl, dl_dtype, row * V + i, 0.0f);
        if (tid == 0) loss[row] = 0.0f;
        return;
    }
    float mx = -1e30f;
    for (int i = tid; i < V; i += 256) mx = fmaxf(mx, blk_ld(lg, lg_dtype, row * V + i));
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (tid == 0) { float m = red[0]; for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]); bc = m; }
    __syncthreads();
    mx = bc;
    float sum = 0.0f;
    for (int i = tid; i < V; i += 256) sum += expf(blk_ld(lg, lg_dtype, row * V + i) - mx);
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (tid == 0) { float s = 0.0f; for (int w = 0; w < 8; w++) s += red[w]; bc = s; }
    __syncthreads();
    const float inv = 1.0f / bc, iN = 1.0f / (float)n_all;
    for (int i = tid; i < V; i += 256) {
        const float p = expf(blk_ld(lg, lg_dtype, row * V + i) - mx) * inv;
        blk_st(dl, dl_dtype, row * V + i, (p - (i == tg ? 1.0f : 0.0f)) * iN);
        if (i == tg) loss[row] = -logf(p + 1e-12f);
    }
}


// ------------------------------------------------------------------ decoder (one new token per live slot)
// k_dec_rope (cudalm.cu:7023-7027): rotate the single row of slot b by the angle of its position pos[b]
__global__ void __launch_bounds__(256) k_dec_rope(void *buf, int dtype, const float *cosb, const float *sinb, const int *pos,
                                                  int B, int nh, int hd, int Tm, int *errword)
{
    const int hf = hd / 2;
    const size_t g = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (g >= (size_t)B * nh * hf) return;
    const int i = (int)(g % hf);
    const size_t r = g / hf;
    const int b = (int)(r / nh), t = pos[b];
    // a position outside the rotation tables: reported, the row is left as it is (no table read)
    if (t < 0 || t >= Tm) { if (i == 0 && r % nh == 0) report_bad_index(errword, 304, b, t); return; }
    const size_t o = r * hd + i;
    const float c = cosb[(size_t)t * hf + i], sn = sinb[(size_t)t * hf + i];
    const float x = blk_ld(buf, dtype, o), y = blk_ld(buf, dtype, o + hf);
    blk_st(buf, dtype, o, x * c - y * sn);
    blk_st(buf, dtype, o + hf, y * c + x * sn);
}
// k_dec_kv (cudalm.cu:7028-7030): the new key / value rows go to position pos[b] of slot b's cache [B, Tm, KD] (bf16)
__global__ void __launch_bounds__(256) k_dec_kv(bf16_t *Kc, bf16_t *Vc, const bf16_t *k, const bf16_t *v, const int *pos, int B,
                                                int Tm, int KD, int *errword)
{
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (size_t)B * KD) return;
    const int b = (int)(i / KD), j = (int)(i % KD);
    const int t = pos[b];
    if (t < 0 || t >= Tm) { if (j == 0) report_bad_index(errword, 301, b, t); return; }   // the slot ran past its cache: nothing is written
    const size_t o = ((size_t)b * Tm + t) * KD + j;
    Kc[o] = k[i]; Vc[o] = v[i];
}
// k_dec_attn (cudalm.cu:7031-7047): one block of four warps per (slot, head) over the cached keys lo..pos[b].
// Pass 1: a thread takes every 128th key and computes its whole 64-wide dot product (16-byte loads), scores
// go to shared memory, block-wide max and sum.  Pass 2: a lane owns two of the 64 output dimensions, each warp
// walks a quarter of the keys (four value rows in flight, each one coalesced 128-byte line), and the four
// partial outputs are added in warp order.  Head dimension 64, bf16 cache.
#define DEC_TM_MAX 4096
__global__ void __launch_bounds__(128) k_dec_attn(bf16_t *O, const bf16_t *Q, const bf16_t *Kc, const bf16_t *Vc, const int *pos,
                                                  int win, int B, int Tm, int H, int KV, float scale, int *errword)
{
    extern __shared__ float dec_sc[];                    // Tm scores
    __shared__ float red[4], part[4][64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int g = blockIdx.x;
    pdl_trigger();
    pdl_wait();                                          // positions, query and cache rows are written by the kernels before
    const int b = g / H, h = g % H, kvh = h / (H / KV), t = pos[b], KD = KV * 64, D = H * 64;
    if (t < 0 || t >= Tm) { if (tid == 0 && h == 0) report_bad_index(errword, 302, b, t); return; }   // whole block: no score past the cache
    float *sc = dec_sc;
    const int lo = (win > 0 && t >= win) ? t - win + 1 : 0;
    float q[64];
    {
        const uint4 *qp = reinterpret_cast<const uint4 *>(Q + (size_t)b * D + h * 64);
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint4 x = __ldg(qp + u);
            const __nv_bfloat162 *xh = reinterpret_cast<const __nv_bfloat162 *>(&x);
#pragma unroll
            for (int k = 0; k < 4; k++) { const float2 f = __bfloat1622float2(xh[k]); q[u * 8 + 2 * k] = f.x; q[u * 8 + 2 * k + 1] = f.y; }
        }
    }
    float mx = -1e30f;
    for (int s = lo + tid; s <= t; s += 128) {
        const uint4 *kp = reinterpret_cast<const uint4 *>(Kc + ((size_t)b * Tm + s) * KD + kvh * 64);
        float dot = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint4 x = kp[u];
            const __nv_bfloat162 *xh = reinterpret_cast<const __nv_bfloat162 *>(&x);
#pragma unroll
            for (int k = 0; k < 4; k++) { const float2 f = __bfloat1622float2(xh[k]); dot += q[u * 8 + 2 * k] * f.x + q[u * 8 + 2 * k + 1] * f.y; }
        }
        dot *= scale;
        sc[s] = dot;
        mx = fmaxf(mx, dot);
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float l = 0.0f;
    for (int s = lo + tid; s <= t; s += 128) { const float p = __expf(sc[s] - mx); sc[s] = p; l += p; }
    l = warp_sum(l);
    if (lane == 0) red[warp] = l;
    __syncthreads();
    l = (red[0] + red[1]) + (red[2] + red[3]);
    // pass 2: warp w takes keys lo + w, lo + w + 4, ...
    float a0 = 0.0f, a1 = 0.0f;
    const bf16_t *vb = Vc + (size_t)b * Tm * KD + kvh * 64 + 2 * lane;
    int s = lo + warp;
    for (; s + 60 <= t; s += 64) {                       // sixteen value rows in flight, added in the same ascending order
        float2 f[16]; float p[16];
#pragma unroll
        for (int k = 0; k < 16; k++) {
            f[k] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(vb + (size_t)(s + 4 * k) * KD));
            p[k] = sc[s + 4 * k];
        }
#pragma unroll
        for (int k = 0; k < 16; k++) { a0 += p[k] * f[k].x; a1 += p[k] * f[k].y; }
    }
    for (; s + 12 <= t; s += 16) {
        float2 f[4]; float p[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            f[k] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(vb + (size_t)(s + 4 * k) * KD));
            p[k] = sc[s + 4 * k];
        }
#pragma unroll
        for (int k = 0; k < 4; k++) { a0 += p[k] * f[k].x; a1 += p[k] * f[k].y; }
    }
    for (; s <= t; s += 4) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(vb + (size_t)s * KD));
        const float p = sc[s];
        a0 += p * f.x; a1 += p * f.y;
    }
    part[warp][2 * lane] = a0; part[warp][2 * lane + 1] = a1;
    __syncthreads();
    if (warp == 0) {
        const float inv = 1.0f / l;
        const float o0 = (part[0][2 * lane] + part[1][2 * lane]) + (part[2][2 * lane] + part[3][2 * lane]);
        const float o1 = (part[0][2 * lane + 1] + part[1][2 * lane + 1]) + (part[2][2 * lane + 1] + part[3][2 * lane + 1]);
        *reinterpret_cast<__nv_bfloat162 *>(O + (size_t)b * D + h * 64 + 2 * lane) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
    }
}
// Greedy pick of k_dec_sample (cudalm.cu:7078-7093: temp <= 0): arg-max with the lowest index on ties and the
// log-probability of the pick.  One block per slot.
__global__ void __launch_bounds__(256) k_dec_greedy(int *out, float *lp, const float *logits, int V)
{
    __shared__ float rv[8], rs[8];
    __shared__ int ri[8];
    const int s = blockIdx.x, tid = threadIdx.x, w = tid >> 5, ln = tid & 31;
    const float *lg = logits + (size_t)s * V;
    float mx = -INFINITY; int mi = 0;
    for (int i = tid; i < V; i += 256) { const float v = lg[i]; if (v > mx) { mx = v; mi = i; } }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(~0u, mx, o); const int oi = __shfl_xor_sync(~0u, mi, o);
        if (ov > mx || (ov == mx && oi < mi)) { mx = ov; mi = oi; }
    }
    if (!ln) { rv[w] = mx; ri[w] = mi; }
    __syncthreads();
    mx = rv[0]; mi = ri[0];
    for (int k = 1; k < 8; k++) if (rv[k] > mx || (rv[k] == mx && ri[k] < mi)) { mx = rv[k]; mi = ri[k]; }
    float z = 0.0f;
    for (int i = tid; i < V; i += 256) z += __expf(lg[i] - mx);
    z = warp_sum(z);
    if (!ln) rs[w] = z;
    __syncthreads();
    if (!tid) {
        float t = 0.0f;
        for (int k = 0; k < 8; k++) t += rs[k];
        out[s] = mi; lp[s] = -logf(t);
    }
}


// The sampling branch of k_dec_sample (cudalm.cu:7078-7108): top_k -> top_p -> temperature.
// One block of 1024 threads per slot.  (1) arg-max and log-sum-exp as in the greedy pick; (2) a value
// threshold, starting 30 below the maximum and halving its distance to it until at most DEC_SCAP
// logits pass; (3) the passing (value, index) pairs are compacted into shared memory and sorted by
// value descending, index ascending (bitonic network; the index as tie-break makes the order, and
// with it the pick, independent of the order the compaction's counter handed out slots);
// (4) thread 0 cuts the list at top_k, then at the first prefix whose probability reaches top_p,
// and draws from exp((v - v0) / temp) with a uniform number hashed from (seed, step).
#define DEC_SCAP 2048
__device__ __forceinline__ bool samp_before(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }
__global__ void __launch_bounds__(1024) k_dec_sample(int *out, float *lp, const float *logits, const qlmb_dec_sampling *sp, int V)
{
    __shared__ float sv[DEC_SCAP];
    __shared__ int si[DEC_SCAP];
    __shared__ float rv[32], rz[32];
    __shared__ int ri[32];
    __shared__ int cnt;
    __shared__ float sth;
    const int s = blockIdx.x, t = threadIdx.x, w = t >> 5, ln = t & 31;
    const float *lg = logits + (size_t)s * V;
    const qlmb_dec_sampling prm = sp[s];
    float mx = -INFINITY; int mi = 0;
    for (int i = t; i < V; i += 1024) { const float v = lg[i]; if (v > mx) { mx = v; mi = i; } }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(~0u, mx, o); const int oi = __shfl_xor_sync(~0u, mi, o);
        if (samp_before(ov, oi, mx, mi)) { mx = ov; mi = oi; }
    }
    if (!ln) { rv[w] = mx; ri[w] = mi; }
    __syncthreads();
    mx = rv[0]; mi = ri[0];
    for (int k = 1; k < 32; k++) if (samp_before(rv[k], ri[k], mx, mi)) { mx = rv[k]; mi = ri[k]; }
    const float M = mx;
    float z = 0.0f;
    for (int i = t; i < V; i += 1024) z += __expf(lg[i] - M);
    z = warp_sum(z);
    if (!ln) rz[w] = z;
    __syncthreads();
    float ssum = 0.0f;
    for (int k = 0; k < 32; k++) ssum += rz[k];
    const float ls = M + logf(ssum);
    if (prm.temp <= 0.0f || prm.top_k == 1) {
        if (!t) { out[s] = mi; lp[s] = M - ls; }
        return;
    }
    // (2) threshold
    float th = M - 30.0f;
    for (int round = 0; round < 64; round++) {
        __syncthreads();
        if (!t) cnt = 0;
        __syncthreads();
        int c = 0;
        for (int i = t; i < V; i += 1024) c += lg[i] >= th;
        c = (int)warp_sum((float)c);
        if (!ln && c) atomicAdd(&cnt, c);
        __syncthreads();
        if (cnt <= DEC_SCAP) break;
        th = 0.5f * (th + M);
    }
    // (3) compaction and sort
    __syncthreads();
    if (!t) cnt = 0;
    __syncthreads();
    for (int i = t; i < V; i += 1024) {
        const float v = lg[i];
        if (v >= th) { const int k = atomicAdd(&cnt, 1); if (k < DEC_SCAP) { sv[k] = v; si[k] = i; } }
    }
    __syncthreads();
    const int n = cnt < DEC_SCAP ? cnt : DEC_SCAP;
    int P2 = 1;
    while (P2 < n) P2 <<= 1;
    for (int i = n + t; i < P2; i += 1024) { sv[i] = -INFINITY; si[i] = 0x7fffffff; }
    __syncthreads();
    for (int k = 2; k <= P2; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = t; i < P2; i += 1024) {
                const int ij = i ^ j;
                if (ij > i) {
                    const float a = sv[i], b = sv[ij]; const int ia = si[i], ib = si[ij];
                    const bool up = (i & k) == 0;              // this pair sorts towards "best first"
                    if (up ? samp_before(b, ib, a, ia) : samp_before(a, ia, b, ib)) { sv[i] = b; sv[ij] = a; si[i] = ib; si[ij] = ia; }
                }
            }
            __syncthreads();
        }
    if (t) return;
    // (4) cut and draw
    int k = prm.top_k > 0 ? (prm.top_k < n ? prm.top_k : n) : n;
    float zz = 0.0f;
    for (int i = 0; i < k; i++) zz += __expf(sv[i] - sv[0]);
    if (prm.top_p < 1.0f) {
        float c = 0.0f;
        for (int i = 0; i < k; i++) { c += __expf(sv[i] - sv[0]) / zz; if (c >= prm.top_p) { k = i + 1; break; } }
    }
    const float it = 1.0f / prm.temp;
    zz = 0.0f;
    for (int i = 0; i < k; i++) zz += __expf((sv[i] - sv[0]) * it);
    unsigned long long h = prm.seed * 0x9E3779B97F4A7C15ull + (unsigned long long)(prm.step + 1) * 0xD1B54A32D192ED03ull;
    h ^= h >> 30; h *= 0xBF58476D1CE4E5B9ull; h ^= h >> 27; h *= 0x94D049BB133111EBull; h ^= h >> 31;
    float u = (float)(h >> 40) * (1.0f / 16777216.0f) * zz;
    int pick = k - 1;
    for (int i = 0; i < k; i++) { u -= __expf((sv[i] - sv[0]) * it); if (u <= 0.0f) { pick = i; break; } }
    out[s] = si[pick]; lp[s] = sv[pick] - ls;
}


// ------------------------------------------------------------------ n-gram table: keys and gather
// k_ngram_key (cudalm.cu:4438-4445): the table row of position n from the hash of its last `order` tokens
// (FNV-1a over the token ids, folded, modulo R, plus base); -1 for the first order-1 positions of a sequence.
__global__ void __launch_bounds__(256) k_ngram_key(int *key, const int *tok, int N, int T, int R, int order, int base)
{
    const int n = blockIdx.x * 256 + threadIdx.x;
    if (n >= N) return;
    if (n % T < order - 1) { key[n] = -1; return; }
    unsigned h = 2166136261u;
    for (int j = order - 1; j >= 0; j--) h = (h ^ (unsigned)tok[n - j]) * 16777619u;
    h ^= h >> 15;
    key[n] = base + (int)(h % (unsigned)R);
}
// k_dec_ngkey (cudalm.cu:7056-7062): the same key for a decoder slot from its window of last tokens tokw[b*4 .. b*4+3]
__global__ void __launch_bounds__(256) k_dec_ngkey(int *key, const int *tokw, const int *pos, int B, int R, int order, int base)
{
    const int b = blockIdx.x * 256 + threadIdx.x;
    if (b >= B) return;
    if (pos[b] < order - 1) { key[b] = -1; return; }
    unsigned h = 2166136261u;
    for (int j = order - 1; j >= 0; j--) h = (h ^ (unsigned)tokw[b * 4 + 3 - j]) * 16777619u;
    h ^= h >> 15;
    key[b] = base + (int)(h % (unsigned)R);
}
// k_ngram_gather (cudalm.cu:4446-4451): buf[n,:] = sum over the nk key sets (ascending) of the table rows, masked keys skipped
__global__ void __launch_bounds__(256) k_ngram_gather(float *buf, const float *tbl, const int *key, int N, int De, int nk)
{
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (size_t)N * De) return;
    const int n = (int)(i / De), e = (int)(i % De);
    int k = key[n];
    float s = k >= 0 ? tbl[(size_t)k * De + e] : 0.0f;
    for (int j = 1; j < nk; j++) { k = key[(size_t)j * N + n]; if (k >= 0) s += tbl[(size_t)k * De + e]; }
    buf[i] = s;
}


// ---------------------------------------------------------------- n-gram context gate
// k_nggate_f (cudalm.cu:3362-3368): per row, g = sigmoid(<rms(h), rms(k)> / sqrt(D)); h += g * v.  Leaves rms(h) in hn,
// rms(k) in k (in place) and g, 1/rms(h), 1/rms(k) per row for the backward pass.  Warp per row, three sums in one pass.
__global__ void __launch_bounds__(256) k_nggate_fwd(void *h, const void *v, void *k, void *hn, int dtype, float *g, float *rh,
                                                    float *rk, int N, int D)
{
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    const size_t o = (size_t)n * D;
    float a = 0.0f, b = 0.0f, c = 0.0f;
    for (int j = lane * 4; j < D; j += 128) {
        const float4 x = blk_ld4(h, dtype, o + j), y = blk_ld4(k, dtype, o + j);
        a += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        b += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
        c += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
    }
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    const float r1 = 1.0f / sqrtf(a / (float)D + 1e-6f), r2 = 1.0f / sqrtf(b / (float)D + 1e-6f);
    const float gg = 1.0f / (1.0f + expf(-(c * r1 * r2 / sqrtf((float)D))));
    for (int j = lane * 4; j < D; j += 128) {
        const float4 x = blk_ld4(h, dtype, o + j), y = blk_ld4(k, dtype, o + j), w = blk_ld4(v, dtype, o + j);
        blk_st4(hn, dtype, o + j, make_float4(x.x * r1, x.y * r1, x.z * r1, x.w * r1));
        blk_st4(k, dtype, o + j, make_float4(y.x * r2, y.y * r2, y.z * r2, y.w * r2));
        blk_st4(h, dtype, o + j, make_float4(x.x + gg * w.x, x.y + gg * w.y, x.z + gg * w.z, x.w + gg * w.w));
    }
    if (lane == 0) { g[n] = gg; rh[n] = r1; rk[n] = r2; }
}
// k_nggate_b (cudalm.cu:3370-3378): dv = g * dy; dk and the part of dh that flows through the gate's logit; dy += that
// part in place.
__global__ void __launch_bounds__(256) k_nggate_bwd(void *dy, const void *v, const void *hn, const void *kn, int dtype,
                                                    const float *g, const float *rh, const float *rk, void *dv, void *dk,
                                                    int N, int D)
{
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    const size_t o = (size_t)n * D;
    float a = 0.0f, b = 0.0f;
    for (int j = lane * 4; j < D; j += 128) {
        const float4 d = blk_ld4(dy, dtype, o + j), w = blk_ld4(v, dtype, o + j);
        const float4 x = blk_ld4(hn, dtype, o + j), y = blk_ld4(kn, dtype, o + j);
        a += d.x * w.x + d.y * w.y + d.z * w.z + d.w * w.w;
        b += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
    }
    a = warp_sum(a); b = warp_sum(b);
    const float gg = g[n], cz = a * gg * (1.0f - gg) / sqrtf((float)D), m = b / (float)D, r1 = rh[n], r2 = rk[n];
    for (int j = lane * 4; j < D; j += 128) {
        const float4 d = blk_ld4(dy, dtype, o + j), x = blk_ld4(hn, dtype, o + j), y = blk_ld4(kn, dtype, o + j);
        blk_st4(dv, dtype, o + j, make_float4(gg * d.x, gg * d.y, gg * d.z, gg * d.w));
        blk_st4(dk, dtype, o + j, make_float4(cz * (x.x - y.x * m) * r2, cz * (x.y - y.y * m) * r2, cz * (x.z - y.z * m) * r2,
                                              cz * (x.w - y.w * m) * r2));
        blk_st4(dy, dtype, o + j, make_float4(d.x + cz * (y.x - x.x * m) * r1, d.y + cz * (y.y - x.y * m) * r1,
                                              d.z + cz * (y.z - x.z * m) * r1, d.w + cz * (y.w - x.w * m) * r1));
    }
}
}  // namespace qlmb

using namespace qlmb;

static bool dtype_ok(int d) { return d == QLMB_F32 || d == QLMB_BF16; }

extern "C" int qlmb_embed(void *X, int x_dtype, const float *emb, const int *tok, int N, int D, void *stream)
{
    QLMB_REQUIRE(X && emb && tok && dtype_ok(x_dtype), "qlmb_embed: bad argument");
    QLMB_REQUIRE(D > 0 && D % 4 == 0, "qlmb_embed: D %d must be a multiple of 4", D);
    if (N <= 0) return QLMB_OK;
    k_embed<<<(N + 7) / 8, 256, 0, as_stream(stream)>>>(X, x_dtype, emb, tok, N, D);
    QLMB_LAUNCH_CHECK("k_embed");
    return QLMB_OK;
}

extern "C" int qlmb_embed_bwd(float *G, const void *dout, int dtype, const int *tok, int N, int D, int V, void *stream)
{
    QLMB_REQUIRE(G && dout && tok && dtype_ok(dtype), "qlmb_embed_bwd: bad argument");
    QLMB_REQUIRE(D > 0 && D % 4 == 0 && D <= 2048, "qlmb_embed_bwd: D %d must be a multiple of 4, at most 2048", D);
    if (N <= 0 || V <= 0) return QLMB_OK;
    const unsigned grid = (unsigned)((V + 7) / 8);
    cudaStream_t st = as_stream(stream);
    if (D <= 512) k_embed_bwd<4><<<grid, 256, 0, st>>>(G, dout, dtype, tok, N, D, V);
    else if (D <= 1024) k_embed_bwd<8><<<grid, 256, 0, st>>>(G, dout, dtype, tok, N, D, V);
    else k_embed_bwd<16><<<grid, 256, 0, st>>>(G, dout, dtype, tok, N, D, V);
    QLMB_LAUNCH_CHECK("k_embed_bwd");
    return QLMB_OK;
}

extern "C" int qlmb_rmsnorm_fwd(void *O, int o_dtype, float *rinv, const void *X, int x_dtype, const float *gamma, int N,
                                int D, void *stream)
{
    QLMB_REQUIRE(O && rinv && X && gamma && dtype_ok(o_dtype) && dtype_ok(x_dtype), "qlmb_rmsnorm_fwd: bad argument");
    QLMB_REQUIRE(D > 0 && D % 4 == 0 && ((uintptr_t)gamma & 15) == 0, "qlmb_rmsnorm_fwd: D %d must be a multiple of 4, gamma 16-byte aligned", D);
    if (N <= 0) return QLMB_OK;
    k_rmsnorm_fwd<<<(N + 7) / 8, 256, 0, as_stream(stream)>>>(O, o_dtype, rinv, X, x_dtype, gamma, N, D);
    QLMB_LAUNCH_CHECK("k_rmsnorm_fwd");
    return QLMB_OK;
}

extern "C" int qlmb_rmsnorm_bwd(void *dx, int dx_dtype, int accumulate, float *dgamma, float *part, const void *X, int x_dtype,
                                const float *gamma, const float *rinv, const void *dy, int dy_dtype, int N, int D,
                                void *stream)
{
    QLMB_REQUIRE(dx && X && gamma && rinv && dy && dtype_ok(dx_dtype) && dtype_ok(x_dtype) && dtype_ok(dy_dtype), "qlmb_rmsnorm_bwd: bad argument");
    QLMB_REQUIRE(D > 0 && D % 4 == 0 && ((uintptr_t)gamma & 15) == 0, "qlmb_rmsnorm_bwd: D %d must be a multiple of 4, gamma 16-byte aligned", D);
    QLMB_REQUIRE(!dgamma || part, "qlmb_rmsnorm_bwd: the gain gradient needs the 128 x D scratch");
    if (N <= 0) return QLMB_OK;
    cudaStream_t st = as_stream(stream);
    k_rmsnorm_bwd<<<(N + 7) / 8, 256, 0, st>>>(dx, dx_dtype, accumulate, X, x_dtype, gamma, rinv, dy, dy_dtype, N, D);
    if (dgamma) {
        k_gamma_part<<<dim3((D + 127) / 128, GAMMA_CH), 128, 0, st>>>(part, X, x_dtype, rinv, dy, dy_dtype, N, D);
        k_gamma_sum<<<(D + 127) / 128, 128, 0, st>>>(dgamma, part, D);
    }
    QLMB_LAUNCH_CHECK("k_rmsnorm_bwd");
    return QLMB_OK;
}

extern "C" int qlmb_rope(void *buf, int dtype, const float *cosb, const float *sinb, int N, int nh, int hd, int T, int back,
                         void *stream)
{
    QLMB_REQUIRE(buf && cosb && sinb && dtype_ok(dtype), "qlmb_rope: bad argument");
    QLMB_REQUIRE(nh > 0 && hd > 0 && hd % 2 == 0 && T > 0, "qlmb_rope: bad shape nh %d hd %d T %d", nh, hd, T);
    if (N <= 0) return QLMB_OK;
    if ((hd / 2) % 8 == 0 && (((uintptr_t)buf | (uintptr_t)cosb | (uintptr_t)sinb) & 15) == 0) {
        const size_t total = (size_t)N * nh * (hd / 16);
        k_rope8<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(buf, dtype, cosb, sinb, total, nh, hd, T, back);
    } else {
        const size_t total = (size_t)N * nh * (hd / 2);
        k_rope<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(buf, dtype, cosb, sinb, total, nh, hd, T, back);
    }
    QLMB_LAUNCH_CHECK("k_rope");
    return QLMB_OK;
}

extern "C" int qlmb_softmax_ce(const void *logits, int lg_dtype, const int *tgt, float *loss, void *dlogits, int dl_dtype,
                               int rows, int V, int n_all, void *stream)
{
    QLMB_REQUIRE(logits && tgt && loss && dlogits && dtype_ok(lg_dtype) && dtype_ok(dl_dtype), "qlmb_softmax_ce: bad argument");
    QLMB_REQUIRE(V > 0 && n_all > 0, "qlmb_softmax_ce: bad shape V %d n_all %d", V, n_all);
    if (rows <= 0) return QLMB_OK;
    k_softmax_ce<<<(unsigned)rows, 256, 0, as_stream(stream)>>>(logits, lg_dtype, tgt, loss, dlogits, dl_dtype, V, n_all);
    QLMB_LAUNCH_CHECK("k_softmax_ce");
    return QLMB_OK;
}

// ---- decoder operators (dec_step, cudalm.cu:7166-7212) ----
extern "C" int qlmb_dec_rope(void *buf, int dtype, const float *cosb, const float *sinb, const int *pos, int B, int nh, int hd,
                             int Tm, void *stream)
{
    QLMB_REQUIRE(buf && cosb && sinb && pos && dtype_ok(dtype) && nh > 0 && hd > 0 && hd % 2 == 0 && Tm > 0, "qlmb_dec_rope: bad argument");
    if (B <= 0) return QLMB_OK;
    const size_t total = (size_t)B * nh * (hd / 2);
    k_dec_rope<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(buf, dtype, cosb, sinb, pos, B, nh, hd, Tm, device_error_word());
    QLMB_LAUNCH_CHECK("k_dec_rope");
    return QLMB_OK;
}

extern "C" int qlmb_dec_kv(void *Kc, void *Vc, const void *k, const void *v, const int *pos, int B, int Tm, int KD, void *stream)
{
    QLMB_REQUIRE(Kc && Vc && k && v && pos && Tm > 0 && KD > 0, "qlmb_dec_kv: bad argument");
    if (B <= 0) return QLMB_OK;
    const size_t total = (size_t)B * KD;
    k_dec_kv<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>((bf16_t *)Kc, (bf16_t *)Vc, (const bf16_t *)k,
                                                                              (const bf16_t *)v, pos, B, Tm, KD, device_error_word());
    QLMB_LAUNCH_CHECK("k_dec_kv");
    return QLMB_OK;
}

extern "C" int qlmb_dec_attn(void *O, const void *Q, const void *Kc, const void *Vc, const int *pos, int win, int B, int Tm,
                             int H, int KV, int hd, void *stream)
{
    QLMB_REQUIRE(O && Q && Kc && Vc && pos, "qlmb_dec_attn: NULL argument");
    QLMB_REQUIRE(hd == 64 && H > 0 && KV > 0 && H % KV == 0 && Tm > 0 && Tm <= DEC_TM_MAX, "qlmb_dec_attn: hd %d H %d KV %d Tm %d", hd, H, KV, Tm);
    if (B <= 0) return QLMB_OK;
    const size_t smem = (size_t)Tm * sizeof(float);
    // the attribute belongs to a device's copy of the kernel: set it once per device of this process
    static bool configured_dev[64];
    int dev_ = 0;
    QLMB_CUDA(cudaGetDevice(&dev_));
    QLMB_REQUIRE(dev_ >= 0 && dev_ < 64, "device index %d", dev_);
    if (!configured_dev[dev_]) {
        QLMB_CUDA(cudaFuncSetAttribute(k_dec_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_TM_MAX * (int)sizeof(float)));
        configured_dev[dev_] = true;
    }
    QLMB_CUDA(pdl_launch(B > 4, k_dec_attn, dim3((unsigned)(B * H)), dim3(128), smem, as_stream(stream), (bf16_t *)O, (const bf16_t *)Q,
                         (const bf16_t *)Kc, (const bf16_t *)Vc, pos, win, B, Tm, H, KV, 1.0f / sqrtf((float)hd), device_error_word()));
    QLMB_LAUNCH_CHECK("k_dec_attn");
    return QLMB_OK;
}

extern "C" int qlmb_dec_greedy(int *out, float *lp, const float *logits, int B, int V, void *stream)
{
    QLMB_REQUIRE(out && lp && logits && V > 0, "qlmb_dec_greedy: bad argument");
    if (B <= 0) return QLMB_OK;
    k_dec_greedy<<<(unsigned)B, 256, 0, as_stream(stream)>>>(out, lp, logits, V);
    QLMB_LAUNCH_CHECK("k_dec_greedy");
    return QLMB_OK;
}

extern "C" int qlmb_dec_sample(int *out, float *lp, const float *logits, const qlmb_dec_sampling *params, int B, int V,
                               void *stream)
{
    QLMB_REQUIRE(out && lp && logits && params && V > 0, "qlmb_dec_sample: bad argument");
    if (B <= 0) return QLMB_OK;
    k_dec_sample<<<(unsigned)B, 1024, 0, as_stream(stream)>>>(out, lp, logits, params, V);
    QLMB_LAUNCH_CHECK("k_dec_sample");
    return QLMB_OK;
}

// ---- n-gram table forward (ngram_forward, cudalm.cu:4701-4716) ----
extern "C" int qlmb_ngram_key(int *key, const int *tok, int N, int T, int R, int order, int base, void *stream)
{
    QLMB_REQUIRE(key && tok && T > 0 && R > 0 && order >= 1, "qlmb_ngram_key: bad argument");
    if (N <= 0) return QLMB_OK;
    k_ngram_key<<<(N + 255) / 256, 256, 0, as_stream(stream)>>>(key, tok, N, T, R, order, base);
    QLMB_LAUNCH_CHECK("k_ngram_key");
    return QLMB_OK;
}
extern "C" int qlmb_dec_ngkey(int *key, const int *tokw, const int *pos, int B, int R, int order, int base, void *stream)
{
    QLMB_REQUIRE(key && tokw && pos && R > 0 && order >= 1 && order <= 4, "qlmb_dec_ngkey: bad argument");
    if (B <= 0) return QLMB_OK;
    k_dec_ngkey<<<(B + 255) / 256, 256, 0, as_stream(stream)>>>(key, tokw, pos, B, R, order, base);
    QLMB_LAUNCH_CHECK("k_dec_ngkey");
    return QLMB_OK;
}
extern "C" int qlmb_ngram_gather(float *buf, const float *tbl, const int *key, int N, int De, int nk, void *stream)
{
    QLMB_REQUIRE(buf && tbl && key && De > 0 && nk >= 1, "qlmb_ngram_gather: bad argument");
    if (N <= 0) return QLMB_OK;
    const size_t total = (size_t)N * De;
    k_ngram_gather<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(buf, tbl, key, N, De, nk);
    QLMB_LAUNCH_CHECK("k_ngram_gather");
    return QLMB_OK;
}

extern "C" int qlmb_nggate_fwd(void *h, const void *v, void *k, void *hn, int dtype, float *g, float *rh, float *rk, int N,
                               int D, void *stream)
{
    QLMB_REQUIRE(h && v && k && hn && g && rh && rk && dtype_ok(dtype), "qlmb_nggate_fwd: bad argument");
    QLMB_REQUIRE(D > 0 && D % 4 == 0, "qlmb_nggate_fwd: D %d must be a multiple of 4", D);
    if (N <= 0) return QLMB_OK;
    k_nggate_fwd<<<(N + 7) / 8, 256, 0, as_stream(stream)>>>(h, v, k, hn, dtype, g, rh, rk, N, D);
    QLMB_LAUNCH_CHECK("k_nggate_fwd");
    return QLMB_OK;
}

extern "C" int qlmb_nggate_bwd(void *dy, const void *v, const void *hn, const void *kn, int dtype, const float *g,
                               const float *rh, const float *rk, void *dv, void *dk, int N, int D, void *stream)
{
    QLMB_REQUIRE(dy && v && hn && kn && g && rh && rk && dv && dk && dtype_ok(dtype), "qlmb_nggate_bwd: bad argument");
    QLMB_REQUIRE(D > 0 && D % 4 == 0, "qlmb_nggate_bwd: D %d must be a multiple of 4", D);
    if (N <= 0) return QLMB_OK;
    k_nggate_bwd<<<(N + 7) / 8, 256, 0, as_stream(stream)>>>(dy, v, hn, kn, dtype, g, rh, rk, dv, dk, N, D);
    QLMB_LAUNCH_CHECK("k_nggate_bwd");
    return QLMB_OK;
}
