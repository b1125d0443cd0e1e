// Decode path: Y[B,N] = X[B,K] * deq(W) for B <= 64 live slots (the reference's
// dec_step calls g_ab with M = slots on the rendered fp32 weights,
// cudalm.cu:7178-7198).  Weight streaming kernels: every code byte is read once
// from HBM per call, activations sit in shared memory, accumulation is fp32.
// Results do not depend on scheduling: partial sums are combined in a fixed order.
#include "qlmb_common.cuh"
#include "qlmb_internal.h"

namespace qlmb {

int workspace(size_t bytes, void **out);       // qlmb_linear.cu

#define GV_BT 8                                 // activation rows processed per pass

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

// ---- codes W[K][N] (groups along N).  Block: 256 output columns x a K slice; warp w takes
// rows k0+w, k0+w+8, ...; lane = 8 consecutive columns.  part[ks][b][n] receives the slice sums.
__global__ void __launch_bounds__(256) k_gemv_kn(float *part, const void *X, int dtype, const uint8_t *codes,
                                                 const float *scales, int B, int K, int N, int kslice)
{
    extern __shared__ float xs[];               // [GV_BT][kslice]
    __shared__ float red[GV_BT][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 256 + lane * 8;
    const int k0 = blockIdx.y * kslice, k1 = k0 + kslice < K ? k0 + kslice : K;
    const int gpr = N / 128;
    const bool live = n0 < N;
    for (int b0 = 0; b0 < B; b0 += GV_BT) {
        __syncthreads();
        for (int i = threadIdx.x; i < GV_BT * kslice; i += 256) {
            int b = b0 + i / kslice, k = k0 + i % kslice;
            xs[i] = (b < B && k < k1) ? ld_x(X, dtype, (size_t)b * K + k) : 0.0f;
        }
        for (int i = threadIdx.x; i < GV_BT * 256; i += 256) red[i / 256][i % 256] = 0.0f;
        __syncthreads();
        float acc[GV_BT][8];
#pragma unroll
        for (int b = 0; b < GV_BT; b++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[b][j] = 0.0f;
        if (live) {
#pragma unroll 4
            for (int k = k0 + warp; k < k1; k += 8) {
                uint32_t w = __ldcs(reinterpret_cast<const uint32_t *>(codes + ((size_t)k * N + n0) / 2));
                float s = __ldg(scales + (size_t)k * gpr + n0 / 128);
                float d[8];
                unpack8(w, d);
#pragma unroll
                for (int b = 0; b < GV_BT; b++) {
                    float xv = xs[b * kslice + (k - k0)] * s;
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[b][j] += xv * d[j];
                }
            }
        }
        // fixed-order combination of the 8 warps
        for (int w8 = 0; w8 < 8; w8++) {
            if (warp == w8 && live) {
#pragma unroll
                for (int b = 0; b < GV_BT; b++)
#pragma unroll
                    for (int j = 0; j < 8; j++) red[b][lane * 8 + j] += acc[b][j];
            }
            __syncthreads();
        }
        for (int i = threadIdx.x; i < GV_BT * 256; i += 256) {
            int b = b0 + i / 256, n = blockIdx.x * 256 + i % 256;
            if (b < B && n < N) part[((size_t)blockIdx.y * B + b) * N + n] = red[i / 256][i % 256];
        }
    }
}

// ---- codes W[N][K] (groups along K).  One warp per output column n; lanes stride over the
// row's code words; the scale multiplies the 8-element partial dot product of each word.
__global__ void __launch_bounds__(256) k_gemv_nk(float *part, const void *X, int dtype, const uint8_t *codes,
                                                 const float *scales, int B, int K, int N)
{
    extern __shared__ float xs[];               // [GV_BT][K]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    const int gpr = K / 128;
    for (int b0 = 0; b0 < B; b0 += GV_BT) {
        __syncthreads();
        for (int i = threadIdx.x; i < GV_BT * K; i += 256) {
            int b = b0 + i / K;
            xs[i] = b < B ? ld_x(X, dtype, (size_t)b * K + i % K) : 0.0f;
        }
        __syncthreads();
        if (n >= N) continue;
        float acc[GV_BT];
#pragma unroll
        for (int b = 0; b < GV_BT; b++) acc[b] = 0.0f;
#pragma unroll 2
        for (int k = lane * 8; k < K; k += 256) {
            uint32_t w = __ldcs(reinterpret_cast<const uint32_t *>(codes + ((size_t)n * K + k) / 2));
            float s = __ldg(scales + (size_t)n * gpr + k / 128);
            float d[8];
            unpack8(w, d);
#pragma unroll
            for (int b = 0; b < GV_BT; b++) {
                const float4 x0 = *reinterpret_cast<const float4 *>(&xs[b * K + k]);
                const float4 x1 = *reinterpret_cast<const float4 *>(&xs[b * K + k + 4]);
                float t = x0.x * d[0] + x0.y * d[1] + x0.z * d[2] + x0.w * d[3] + x1.x * d[4] + x1.y * d[5] + x1.z * d[6] + x1.w * d[7];
                acc[b] += s * t;
            }
        }
#pragma unroll
        for (int b = 0; b < GV_BT; b++) {
            float v = acc[b];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && b0 + b < B) part[(size_t)(b0 + b) * N + n] = v;
        }
    }
}

// Y[b,n] = sum over K slices (ascending) of part[ks][b][n]
__global__ void __launch_bounds__(256) k_gemv_finish(void *Y, int dtype, const float *part, int nslice, size_t BN_)
{
    size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= BN_) return;
    float s = 0.0f;
    for (int k = 0; k < nslice; k++) s += part[(size_t)k * BN_ + i];
    if (dtype == QLMB_BF16) ((bf16 *)Y)[i] = __float2bfloat16_rn(s);
    else ((float *)Y)[i] = s;
}

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_gemv_decode(void *Y, const void *X, const int8_t *codes, const float *scales, int layout,
                                int B, int K, int N, int dtype, void *stream)
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
    int nslice = 1, kslice = K;
    if (layout == QLMB_KN) {
        // enough K slices to give every SM a few blocks, at least 64 rows each
        int nchunks = (N + 255) / 256;
        int want = (4 * sm_count() + nchunks - 1) / nchunks;
        nslice = want < 1 ? 1 : want;
        if (nslice > K / 64) nslice = K / 64;
        if (nslice < 1) nslice = 1;
        kslice = ((K + nslice - 1) / nslice + 7) / 8 * 8;
        nslice = (K + kslice - 1) / kslice;
    }
    void *ws = nullptr;
    int rc = workspace((size_t)nslice * B * N * sizeof(float), &ws);
    if (rc) return rc;
    float *part = (float *)ws;
    if (layout == QLMB_KN) {
        size_t smem = (size_t)GV_BT * kslice * sizeof(float);
        QLMB_REQUIRE(smem <= 40 * 1024, "qlmb_gemv_decode: K slice of %d rows does not fit shared memory", kslice);
        k_gemv_kn<<<dim3((N + 255) / 256, nslice), 256, smem, st>>>(part, X, dtype, (const uint8_t *)codes, scales, B, K, N, kslice);
    } else {
        size_t smem = (size_t)GV_BT * K * sizeof(float);
        static bool cfg = false;
        if (smem > 48 * 1024) {
            QLMB_REQUIRE(smem <= 200 * 1024, "qlmb_gemv_decode: K=%d too large for the shared-memory activation tile", K);
            if (!cfg) { QLMB_CUDA(cudaFuncSetAttribute(k_gemv_nk, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); cfg = true; }
        }
        k_gemv_nk<<<(N + 7) / 8, 256, smem, st>>>(part, X, dtype, (const uint8_t *)codes, scales, B, K, N);
    }
    k_gemv_finish<<<(unsigned)(((size_t)B * N + 255) / 256), 256, 0, st>>>(Y, dtype, part, nslice, (size_t)B * N);
    QLMB_LAUNCH_CHECK("qlmb_gemv_decode");
    return QLMB_OK;
}
