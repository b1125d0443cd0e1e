// Internal (non-ABI) interfaces shared between the translation units of
// libqlm_b200.  All pointers are device pointers unless noted.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stddef.h>
#include <stdint.h>

namespace qlmb {

typedef __nv_bfloat16 bf16;

// ---- grouped decode GEMVs (qlmb_gemv.cu): rows in groups share one pass over the codes W[K][N] ----
struct Rows8 {
    float *part; const void *X; int x_dtype; int K, N, kslice;
    const uint8_t *codes; const float *scales; size_t e_codes, e_scales;
    const uint8_t *codes2; const float *scales2;         // routed: second stack for groups z >= zdual
    int B, nmat, rows_out;                               // dense: batch and stack; rows_out = rows of `part` per slice
    const int *perm, *off; int E, ntok, x_by_token, zdual, R;   // routed (perm != nullptr)
    const float *gamma;                                  // dense: rows are normalised on the way in (rinv * gamma, bf16)
    uint32_t k65536;
};
// ---- routing (qlmb_route.cu) ----
int router_topk(const float *rt, float *rprobs, int *assign, float *gate, int N, int E, int K,
                const float *bias, int bs, cudaStream_t st);
size_t perm_scratch_ints(int N, int E, int K, int merged);
int perm_build(const int *assign, int N, int E, int K, int merged, int pad, int *perm, int *inv,
               int *off, int *counts, int *bad_flag, int *tile_info, int *ntiles,
               int *chunk_scratch, cudaStream_t st, int e_lo = 0, int skip = 0, int *rank_counts = nullptr,
               int experts_per_rank = 0);

// ---- row kernels (qlmb_dispatch.cu) ----
int router_logits(float *rt, const void *X, int x_dtype, const float *Wr, int N, int D, int E,
                  cudaStream_t st);
// Xp[j,:] = src[perm[j] % N,:] as bf16 (zero rows where perm[j] < 0); rows = *nrows_dev, or
// max_rows when nrows_dev is NULL
int gather_rows(bf16 *Xp, const void *src, int dtype, const int *perm, const int *nrows_dev,
                int max_rows, int N, int D, cudaStream_t st);
// out[n,:] = f_in[n,:] + sum_k gate[k*N+n] * yp[inv[k*N+n],:]   (k ascending)
int combine_rows(void *out, const void *f_in, int dtype, const bf16 *yp, const int *inv,
                 const float *gate, int N, int D, int K, cudaStream_t st);
// per permuted row j: d_gate[slot] = dout[n].yp[j]; dyp[j] = gate[slot]*dout[n]; zero filler rows
int dgate_rows(bf16 *dyp, float *d_gate, const void *dout, int dtype, const bf16 *yp,
               const int *perm, const float *gate, const int *nrows_dev, int max_rows, int N, int D,
               cudaStream_t st);
// router backward pieces (reference cudalm.cu:4372-4391)
int router_bwd(float *drt, const float *rprobs, const int *assign, const float *d_gate,
               const int *counts, int N, int E, int K, float aux, cudaStream_t st);
// dfnorm[n,:] = sum_k dXp[inv[k*N+n],:] + drt[n,:] * Wr^T
int unpermute_rows(void *dfnorm, int dtype, const bf16 *dXp, const int *inv, const float *drt,
                   const float *Wr, float *wrt_scratch /* D*E floats */, int N, int D, int E, int K,
                   cudaStream_t st);
// dWr[D,E] = beta*dWr + fnorm^T drt ; scratch holds 192*D*E floats
int router_wgrad(float *dWr, const void *fnorm, int dtype, const float *drt, float *scratch, int N,
                 int D, int E, float beta, cudaStream_t st);
// ---- expert parallelism by peer loads (qlmb_dispatch.cu) ----
#define QLMB_EP_MAX_WORLD 8
struct PeerPtrs { const void *p[QLMB_EP_MAX_WORLD]; };   // the same buffer in every rank's window
int gather_rows_peer(bf16 *Xp, const PeerPtrs &src, int dtype, const int *perm, const int *nrows_dev, int max_rows,
                     int Nh, int KN, int D, cudaStream_t st);
int dgate_dot_peer(float *d_gate, const void *dout, int dtype, const bf16 *ykeep, int N, int D, int K, cudaStream_t st);
int dyp_rows_peer(bf16 *dyp, const PeerPtrs &dout, const PeerPtrs &gate, int dtype, const int *perm, const int *nrows_dev,
                  int max_rows, int Nh, int KN, int D, cudaStream_t st);
int count_assign(int *counts, const int *assign, int KN, int E, cudaStream_t st);
// fp32 <-> bf16 row conversion helpers
int convert_f32_to_bf16(bf16 *dst, const float *src, size_t n, cudaStream_t st);

// ---- tensor-core GEMMs (qlmb_gemm.cu) ----
struct GemmProblem;   // see qlmb_gemm.cuh

// router logits of a few rows (decode): deterministic, not the tiled kernel's summation order
int router_logits_small(float *rt, const void *X, int x_dtype, const float *Wr, int N, int D, int E, cudaStream_t st);
// the same logits and the selection in one launch (qlmb_route.cu); larger shapes fall back to the two kernels
// perm / off / counts / bad (optional): with at most 256 routed slots the same launch groups the slots by expert;
// *perm_done tells the caller whether it did
int router_small(float *rt, const void *X, int x_dtype, const float *Wr, float *rprobs, int *assign, float *gate, int N, int D,
                 int E, int K, const float *bias, int bs, cudaStream_t st, int *perm = nullptr, int *off = nullptr,
                 int *counts = nullptr, int *bad = nullptr, int *perm_done = nullptr);
// experts of a decode step with at most 64 routed rows (qlmb_gemv.cu): routed GEMVs over the chosen experts' codes
// perm / off / counts / bad: scratch of the permutation (K*N, E + 1, E and 1 ints) for steps with more than 16 routed rows
int moe_decode_experts(const qlmb_moe_layer *L, void *out, const void *f_in, const void *f_norm, const int *assign,
                       const float *gate, cudaStream_t st, int *perm = nullptr, int *off = nullptr, int *counts = nullptr,
                       int *bad = nullptr, int perm_ready = 0);

}  // namespace qlmb
