// Quantised linear entry points (the reference's g_ab / g_abt / g_abt_b / g_atb
// call sites, cudalm.cu:3133-3202) on top of the tcgen05 GEMM engine.
#include "qlmb_common.cuh"
#include "qlmb_gemm.cuh"

namespace qlmb {

// per-device scratch for the bf16 copies of fp32 operands, grown on demand
static void *g_ws[64];
static size_t g_ws_cap[64];
int workspace(size_t bytes, void **out)
{
    int dev = 0;
    QLMB_CUDA(cudaGetDevice(&dev));
    QLMB_REQUIRE(dev >= 0 && dev < 64, "workspace: device index %d", dev);
    if (g_ws_cap[dev] < bytes) {
        if (g_ws[dev]) { QLMB_CUDA(cudaDeviceSynchronize()); QLMB_CUDA(cudaFree(g_ws[dev])); }
        g_ws[dev] = nullptr; g_ws_cap[dev] = 0;
        size_t cap = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        QLMB_CUDA(cudaMalloc(&g_ws[dev], cap));
        g_ws_cap[dev] = cap;
    }
    *out = g_ws[dev];
    return QLMB_OK;
}

// bf16 view of an activation matrix: the matrix itself, or a converted copy in `slot`
static int as_bf16(const void *x, int dtype, size_t n, bf16 *slot, const bf16 **out, cudaStream_t st)
{
    if (dtype == QLMB_BF16) { *out = (const bf16 *)x; return QLMB_OK; }
    int rc = convert_f32_to_bf16(slot, (const float *)x, n, st);
    *out = slot;
    return rc;
}

static int check_linear(const char *who, int layout, int M, int K, int N, int dtype)
{
    QLMB_REQUIRE(layout == QLMB_KN || layout == QLMB_NK, "%s: layout %d", who, layout);
    QLMB_REQUIRE(dtype == QLMB_F32 || dtype == QLMB_BF16, "%s: dtype %d", who, dtype);
    QLMB_REQUIRE(M >= 0 && K > 0 && N > 0, "%s: M=%d K=%d N=%d", who, M, K, N);
    if ((K % 128) || (N % 128)) {
        set_error("%s: K=%d and N=%d must be multiples of the 128-element scale group", who, K, N);
        return QLMB_E_UNSUPPORTED;
    }
    return QLMB_OK;
}

// row offsets of S equal slices (the `off` table of the grouped weight-gradient schedule)
__global__ void k_slice_offsets(int *off, int S, int rows)
{
    if ((int)threadIdx.x <= S) off[threadIdx.x] = (int)threadIdx.x * rows;
}
// dW = beta * dW + part[0] + part[1] + ... in ascending slice order; n is a multiple of 4
__global__ void __launch_bounds__(256) k_sum_slices(float *dW, const float *part, int S, size_t n, float beta)
{
    const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 4;
    if (i >= n) return;
    float4 a = *reinterpret_cast<const float4 *>(part + i);
    for (int s = 1; s < S; s++) {
        const float4 b = *reinterpret_cast<const float4 *>(part + (size_t)s * n + i);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    if (beta != 0.0f) {
        const float4 o = *reinterpret_cast<const float4 *>(dW + i);
        a.x += beta * o.x; a.y += beta * o.y; a.z += beta * o.z; a.w += beta * o.w;
    }
    *reinterpret_cast<float4 *>(dW + i) = a;
}

}  // namespace qlmb

using namespace qlmb;

extern "C" int qlmb_linear_fwd(void *Y, const void *X, const int8_t *codes, const float *scales, int layout,
                               int M, int K, int N, const void *R, int dtype, void *stream)
{
    int rc = check_linear("qlmb_linear_fwd", layout, M, K, N, dtype);
    if (rc) return rc;
    if (M == 0) return QLMB_OK;
    QLMB_REQUIRE(Y && X && codes && scales, "qlmb_linear_fwd: NULL argument");
    cudaStream_t st = as_stream(stream);
    void *ws = nullptr;
    if (dtype == QLMB_F32) { rc = workspace((size_t)M * K * 2, &ws); if (rc) return rc; }
    const bf16 *xb;
    rc = as_bf16(X, dtype, (size_t)M * K, (bf16 *)ws, &xb, st);
    if (rc) return rc;
    GemmLaunch g = {};
    g.bmode = layout == QLMB_KN ? B_DEQ_MN : B_DEQ_K;
    g.epi = EPI_STORE; g.sched = SCHED_DENSE;
    g.a[0] = xb; g.a_rows = M; g.a_cols = K;
    g.w[0] = codes; g.scales[0] = scales;
    g.w_rows = layout == QLMB_KN ? K : N; g.w_cols = layout == QLMB_KN ? N : K;
    g.nseg = 1; g.ksteps = K / 64; g.M = M; g.N = N; g.E = 1;
    g.out = Y; g.out_dtype = dtype; g.ldo = N; g.resid = R; g.beta = 0.0f;
    return gemm_launch(g, st);
}

extern "C" int qlmb_linear_dgrad(void *dX, const void *dY, const int8_t *codes, const float *scales, int layout,
                                 int M, int K, int N, float beta, int dtype, void *stream)
{
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_linear_dgrad: beta %g", beta);
    int rc = check_linear("qlmb_linear_dgrad", layout, M, K, N, dtype);
    if (rc) return rc;
    if (M == 0) return QLMB_OK;
    QLMB_REQUIRE(dX && dY && codes && scales, "qlmb_linear_dgrad: NULL argument");
    cudaStream_t st = as_stream(stream);
    void *ws = nullptr;
    if (dtype == QLMB_F32) { rc = workspace((size_t)M * N * 2, &ws); if (rc) return rc; }
    const bf16 *gb;
    rc = as_bf16(dY, dtype, (size_t)M * N, (bf16 *)ws, &gb, st);
    if (rc) return rc;
    GemmLaunch g = {};
    // the contraction now runs over N: codes W[K][N] are K-major for it, W[N][K] MN-major
    g.bmode = layout == QLMB_KN ? B_DEQ_K : B_DEQ_MN;
    g.epi = EPI_STORE; g.sched = SCHED_DENSE;
    g.a[0] = gb; g.a_rows = M; g.a_cols = N;
    g.w[0] = codes; g.scales[0] = scales;
    g.w_rows = layout == QLMB_KN ? K : N; g.w_cols = layout == QLMB_KN ? N : K;
    g.nseg = 1; g.ksteps = N / 64; g.M = M; g.N = K; g.E = 1;
    g.out = dX; g.out_dtype = dtype; g.ldo = K; g.resid = nullptr; g.beta = beta;
    return gemm_launch(g, st);
}

extern "C" int qlmb_linear_wgrad(float *dW, const void *dY, const void *X, int layout, int M, int K, int N,
                                 float beta, int dtype, void *stream)
{
    QLMB_REQUIRE(dW && (M == 0 || (dY && X)), "qlmb_linear_wgrad: NULL argument");
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_linear_wgrad: beta %g", beta);
    int rc = check_linear("qlmb_linear_wgrad", layout, M, K, N, dtype);
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    if (M == 0) {
        if (beta == 0.0f) QLMB_CUDA(cudaMemsetAsync(dW, 0, (size_t)K * N * sizeof(float), st));
        return QLMB_OK;
    }
    // dW[K,N] = X^T dY (KN)   or   dW[N,K] = dY^T X (NK)
    const int Md = layout == QLMB_KN ? K : N, Nd = layout == QLMB_KN ? N : K;
    // A small weight matrix gives few output tiles (768 x 768: 9 tiles of 256 x 256 for 74 SM pairs) over a
    // long contraction (the M rows).  Then the rows are cut into S slices that run as the "experts" of the
    // grouped weight-gradient schedule, each into its own partial, and the partials are added in ascending
    // slice order: every element still has one writer and a fixed order.
    int S = 1;
    {
        const int tiles = ((Md + 255) / 256) * ((Nd + 255) / 256), pairs = sm_count() / 2;
        while (S < 16 && tiles * S * 2 <= pairs && M % (256 * S) == 0 && M / (2 * S) >= 512) S *= 2;
    }
    const size_t conv = dtype == QLMB_F32 ? ((((size_t)M * K * 2 + 255) & ~(size_t)255) + (((size_t)M * N * 2 + 255) & ~(size_t)255)) : 0;
    const size_t part_bytes = S > 1 ? (size_t)S * Md * Nd * sizeof(float) + 256 : 0;
    void *ws = nullptr;
    if (conv + part_bytes) { rc = workspace(conv + part_bytes, &ws); if (rc) return rc; }
    const bf16 *xb, *gb;
    bf16 *slot2 = conv ? (bf16 *)((uint8_t *)ws + (((size_t)M * K * 2 + 255) & ~(size_t)255)) : nullptr;
    rc = as_bf16(X, dtype, (size_t)M * K, (bf16 *)ws, &xb, st);
    if (rc) return rc;
    rc = as_bf16(dY, dtype, (size_t)M * N, slot2, &gb, st);
    if (rc) return rc;
    GemmLaunch g = {};
    g.bmode = AB_TMA_MN; g.epi = EPI_ACCUM; g.sched = SCHED_DENSE;
    g.a[0] = layout == QLMB_KN ? xb : gb; g.a_rows = M; g.a_cols = Md;
    g.w[0] = layout == QLMB_KN ? gb : xb; g.w_cols = Nd; g.w_rows = 0;
    if (S > 1) {
        float *part = (float *)((uint8_t *)ws + conv);
        int *off = (int *)((uint8_t *)part + (size_t)S * Md * Nd * sizeof(float));
        k_slice_offsets<<<1, 32, 0, st>>>(off, S, M / S);
        g.sched = SCHED_GROUPK;
        g.nseg = 1; g.M = Md; g.N = Nd; g.E = S; g.off = off;
        g.out = part; g.out_dtype = QLMB_F32; g.ldo = Nd; g.beta = 0.0f; g.name = "gemm_wgrad_slices";
        rc = gemm_launch(g, st);
        if (rc) return rc;
        const size_t n = (size_t)Md * Nd;
        k_sum_slices<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(dW, part, S, n, beta);
        QLMB_LAUNCH_CHECK("k_sum_slices");
        return QLMB_OK;
    }
    g.nseg = 1; g.ksteps = (M + 63) / 64; g.M = Md; g.N = Nd; g.E = 1;
    g.out = dW; g.out_dtype = QLMB_F32; g.ldo = Nd; g.beta = beta;
    return gemm_launch(g, st);
}

// Engine check (not part of the reference's operator surface): C[M,N] (fp32) =
// A[M,K] * B[N,K]^T with both bf16 operands delivered by TMA, i.e. the same
// pipeline as the quantised kernels minus the dequant warps.
extern "C" int qlmb_selftest_gemm_bf16(float *C, const void *A, const void *B, int M, int K, int N, void *stream)
{
    QLMB_REQUIRE(C && A && B && M > 0 && K > 0 && N > 0 && K % 64 == 0 && N % 128 == 0, "qlmb_selftest_gemm_bf16: bad shape");
    GemmLaunch g = {};
    g.bmode = B_TMA_K; g.epi = EPI_STORE; g.sched = SCHED_DENSE;
    g.a[0] = A; g.a_rows = M; g.a_cols = K;
    g.w[0] = B; g.w_rows = N; g.w_cols = K;
    g.nseg = 1; g.ksteps = K / 64; g.M = M; g.N = N; g.E = 1;
    g.out = C; g.out_dtype = QLMB_F32; g.ldo = N;
    return gemm_launch(g, as_stream(stream));
}

// ---- unquantised operands (lm_head over the tied embedding, cudalm.cu:5832-5858) ----
// C[M,N] = A[M,K] B[N,K]^T (+ beta * C): both operands bf16, delivered by TMA; C is fp32 or bf16.
extern "C" int qlmb_gemm_nt(void *C, int c_dtype, const void *A, const void *B, int M, int K, int N, float beta, void *stream)
{
    QLMB_REQUIRE(C && A && B, "qlmb_gemm_nt: NULL argument");
    QLMB_REQUIRE(c_dtype == QLMB_F32 || c_dtype == QLMB_BF16, "qlmb_gemm_nt: dtype %d", c_dtype);
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_gemm_nt: beta %g", beta);
    QLMB_REQUIRE(M >= 0 && K > 0 && N > 0 && K % 64 == 0 && N % 128 == 0, "qlmb_gemm_nt: M=%d K=%d N=%d (K %% 64, N %% 128)", M, K, N);
    if (M == 0) return QLMB_OK;
    GemmLaunch g = {};
    g.bmode = B_TMA_K; g.epi = EPI_STORE; g.sched = SCHED_DENSE;
    g.a[0] = A; g.a_rows = M; g.a_cols = K;
    g.w[0] = B; g.w_rows = N; g.w_cols = K;
    g.nseg = 1; g.ksteps = K / 64; g.M = M; g.N = N; g.E = 1;
    g.out = C; g.out_dtype = c_dtype; g.ldo = N; g.beta = beta;
    return gemm_launch(g, as_stream(stream));
}

namespace qlmb {
// dst[c][r] = bf16(src[r][c]) through a padded 32 x 32 shared-memory tile
__global__ void __launch_bounds__(256) k_cast_transpose(bf16 *dst, const float *src, int R, int Cc)
{
    __shared__ float t[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32, tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int i = ty; i < 32; i += 8) t[i][tx] = (r0 + i < R && c0 + tx < Cc) ? src[(size_t)(r0 + i) * Cc + c0 + tx] : 0.0f;
    __syncthreads();
    for (int i = ty; i < 32; i += 8)
        if (c0 + i < Cc && r0 + tx < R) dst[(size_t)(c0 + i) * R + r0 + tx] = __float2bfloat16_rn(t[tx][i]);
}
}  // namespace qlmb

// bf16 copies of an fp32 matrix src[R][C]: plain (dst, may be NULL) and transposed (dst_t [C][R], may be NULL).
// The tied embedding is a float span; the head GEMMs read these copies (the reference casts it once per
// step as well, cudalm.cu:5822-5829).
extern "C" int qlmb_cast_bf16(void *dst, void *dst_t, const float *src, int R, int Cc, void *stream)
{
    QLMB_REQUIRE(src && (dst || dst_t) && R > 0 && Cc > 0, "qlmb_cast_bf16: bad argument");
    cudaStream_t st = as_stream(stream);
    if (dst) { int rc = convert_f32_to_bf16((bf16 *)dst, src, (size_t)R * Cc, st); if (rc) return rc; }
    if (dst_t) {
        k_cast_transpose<<<dim3((Cc + 31) / 32, (R + 31) / 32), 256, 0, st>>>((bf16 *)dst_t, src, R, Cc);
        QLMB_LAUNCH_CHECK("k_cast_transpose");
    }
    return QLMB_OK;
}
