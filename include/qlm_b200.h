/* qlm_b200.h -- C ABI of libqlm_b200.so: the QLM hot path of Dsg2/cudalm-c
 * (4-bit pack/quantise, integer AdamW, dequant-fused linears, top-k routed
 * expert FFN, decode GEMV) as hand-written sm_100a kernels.
 *
 * The reference has no FFI layer: its operators are `static` functions of one
 * translation unit that take raw device pointers, run on the default stream
 * and exit() on error.  Each entry point below replaces one of those
 * operators (cited as file:line of the reference project) with the same
 * argument meaning, plus an explicit stream, and returns a status instead of
 * exiting.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer into caller-owned memory unless the
 *     parameter comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *     calls are asynchronous with respect to the host;
 *   - return value: 0 = QLMB_OK, otherwise a QLMB_E_* code; the message of the
 *     last failure on the calling thread is qlmb_last_error();
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point returns QLMB_E_CUDA.
 *   - matrices are row-major; 4-bit codes are two's-complement nibbles, element
 *     i in byte i>>1, even i in the low nibble (qlm.cuh:96-101); one fp32 scale
 *     per 128 consecutive elements of the flat row-major span (qlm.cuh:28-29).
 */
#ifndef QLM_B200_H
#define QLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    QLMB_OK = 0,
    QLMB_E_ARG = 1,      /* bad argument (shape, alignment, NULL)            */
    QLMB_E_CUDA = 2,     /* CUDA runtime / driver error                      */
    QLMB_E_UNSUPPORTED = 3,
    QLMB_E_DEVICE = 4    /* a kernel reported a bounded wait that ran out    */
};

/* element type of activation / gradient tensors */
enum { QLMB_F32 = 0, QLMB_BF16 = 1 };
/* storage orientation of a quantised weight relative to Y = X * W:
 * KN: codes are W[K,N] (the reference's own layout, applied with g_ab);
 * NK: codes are W[N,K] (applied with g_abt, BASELINE config 1).            */
enum { QLMB_KN = 0, QLMB_NK = 1 };

/* One quantised span; binary-compatible with the reference's QSpanD
 * (qlm.cuh:30-38). */
typedef struct {
    uint64_t pof;    /* offset of the span in P                         */
    uint64_t gof;    /* offset of the span in G                         */
    uint64_t qi0;    /* offset of the span in d / r / m8 / v8           */
    uint64_t n;      /* elements                                        */
    int32_t gi0;     /* first group index                               */
    int32_t ngrp;    /* groups in the span (the last may be short)      */
    float sref;      /* frozen reference scale (relative-LR mode)       */
} qlmb_span;

const char *qlmb_last_error(void);
int qlmb_version(void);
/* Reads and clears the per-device error word kernels set when a bounded
 * wait expires (QLMB_E_DEVICE); synchronises `stream`. */
int qlmb_check_device(void *stream);
/* No counterpart in the reference (its kernels have no waits).  Runs the give-up path of the library's
 * bounded waits on purpose and harmlessly: one warp polls an mbarrier that nothing arrives at `polls`
 * times (1..65536), records error code 200 / site 9999 in the device error word and returns.  The next
 * qlmb_check_device reports QLMB_E_DEVICE and clears the word; later launches run as usual. */
int qlmb_selftest_wait_expires(int polls, void *stream);
/* No counterpart in the reference.  Calibration for the decode GEMV's roofline: a kernel that only LOADS a matrix of
 * `rows` rows of `row_bytes` bytes (a multiple of 256) once, in the grid shape of the streaming GEMV (256-byte column
 * blocks x kslices row slices, 16 rows in flight per lane), and does no arithmetic.  Its duration is what launch,
 * first-load latency and the tail cost at that size; bench.py reports it beside the GEMV's. */
int qlmb_selftest_stream_read(const void *W, unsigned long long row_bytes, int rows, int kslices, void *stream);

/* Work that does not depend on each other inside one call (the three expert weight-gradient GEMMs
 * of the MoE backward against d(act) and dX, the router's backward chain against all of them) runs on
 * library-owned side streams (two per device) and is joined back into the caller's stream before the
 * call returns.  on = 0 keeps everything on the
 * caller's stream (also: environment QLMB_SIDE_STREAM=0, and always while the stream is being
 * captured).  No reference counterpart (the reference uses the default stream only). */
int qlmb_side_stream_enable(int on);

/* Per-operator timing, the counterpart of the reference's CUDALM_PROF=3 event
 * timers (cudalm.cu:806-825): while enabled, every kernel launch of the MoE
 * and linear entry points is bracketed by CUDA events on its stream.
 * qlmb_prof_read synchronises the device, fills up to `max` names (64 bytes
 * each) and milliseconds, clears the record and returns the count. */
int qlmb_prof_enable(int on);
int qlmb_prof_read(char *names, float *ms, int max);

/* ------------------------------------------------------------------ QLM state */

/* k_qlm_encode (qlm.cuh:136-167): P -> digits d, residuals r, scales s for
 * all `ngrp` groups of the span table. */
int qlmb_encode(const float *P, int8_t *d, int8_t *r, float *s, const qlmb_span *sp, int nspan,
                int ngrp, int group, int dmax, int packed, void *stream);

/* k_qlm_render (qlm.cuh:170-178): P = s*d for groups [gi_base, gi_base+ng). */
int qlmb_render(float *P, const int8_t *d, const float *s, const qlmb_span *sp, int nspan,
                int group, int packed, int gi_base, int ng, void *stream);

/* qlm_step_launch (qlm.cuh:377-397): one integer-AdamW step over groups
 * [gi_base, gi_base+ng).  P may be NULL (no fp32 view is written); gsp, when
 * not NULL, points at the TWO device floats k_gnorm writes (qlmb_gnorm,
 * qlmb_gnorm_close): gsp[0] replaces gscale (the clip multiplier), gsp[1] is
 * the gradient norm.  When that norm is not finite the launch writes nothing
 * and counts itself in qlmb_skipped_steps: gpu_adam's "step skipped"
 * (cudalm.cu:6446-6447, 8651-8656) without its copy to the host.
 * stat may be NULL.  Element indices in the rounding hash are global, so a
 * step split over several calls / GPUs gives the same bytes as one call. */
int qlmb_step(float *P, const float *G, int8_t *d, int8_t *r, const float *s, int8_t *m8,
              float *m8s, uint8_t *v8, float *v8s, const qlmb_span *sp, int nspan, int group,
              int dmax, float lr, float b1, float b2, float wd, float gscale, const float *gsp,
              float inv_bc1, float inv_sqrt_bc2, int lrmode, uint64_t t, int adam, int64_t *stat,
              int packed, int gi_base, int ng, void *stream);

/* Number of qlmb_step / qlmb_ng_step launches on the current device that found a non-finite norm
 * in gsp[1] and left the state untouched (the reference prints "[nan] ... step skipped" and counts
 * them in a row, cudalm.cu:8651-8656).  count is a HOST pointer; synchronises `stream`;
 * reset != 0 clears the counter afterwards. */
int qlmb_skipped_steps(unsigned long long *count, int reset, void *stream);

/* QLM_V4 (qlm.cuh:62-72, qv_dec / qv_enc): v8 stores the fourth root of the second moment instead of its square
 * root, so that small-gradient elements of a group do not sit on the uint8 floor.  A process-wide switch, as in
 * the reference (its device global d_qv4); affects qlmb_step. */
int qlmb_set_v4(int on);

/* ---- 4-bit n-gram / engram table: sparse integer AdamW over the groups a step touched
 * (NGRAM_Q4_FOLD: ng_build_touched, k_ng_scatter_compact, k_ng_q4_step; cudalm.cu:4465-4530, 4673-4745).
 * The table is one packed span of nt elements starting at element 0; key[n] is the table row of position n
 * (-1: masked), a row has De elements, group % De == 0.  Nothing is copied to the host: the number of touched
 * groups stays in *count (device) and the launches are sized by max_touched (an upper bound, e.g. min(NK, ngrp)).
 * Every step has a fixed order (no atomics on floats, no CAS race for slots), so results are run-to-run identical.
 *
 * qlmb_ng_touched: tgi[0..*count) = the groups some key falls into, ascending (the reference's slot order is
 * arbitrary).  flag is a scratch of ngrp ints that must be zero on entry and is zero again on exit. */
int qlmb_ng_touched(int *tgi, int *count, int *flag, const int *key, int NK, int De, int group, int ngrp, void *stream);
/* Gc[c*group + o] = sum over positions n (ascending) with key[n] = row of element o of group tgi[c], of
 * dbuf[(n % Nd)*De + e]; every element of the first *count rows of Gc is written (no memset needed). */
int qlmb_ng_scatter_compact(float *Gc, const int *key, const int *tgi, const int *count, const float *dbuf, int NK,
                            int De, int group, int Nd, int max_touched, void *stream);
/* k_ng_q4_step: the integer AdamW step of qlmb_step (packed, adam, relative learning rate against the frozen
 * sref, gradient multiplier gs[0] when gs is not NULL, skipped like qlmb_step when gs[1] is not finite) on groups
 * tgi[0..*count), gradients from Gc. */
int qlmb_ng_step(float *P, const float *Gc, int8_t *d, int8_t *r, const float *s, int8_t *m8, float *m8s, uint8_t *v8,
                 float *v8s, const int *tgi, const int *count, int max_touched, int group, int dmax, float lr, float b1,
                 float b2, float wd, float sref, float inv_bc1, float inv_sqrt_bc2, uint64_t t, uint64_t nt,
                 const float *gs, void *stream);

/* Sparse engram (cudalm.cu:4963-5098): S = orders x heads hashed sub-tables share the one 4-bit table (sub-table s owns rows
 * [s*Rp, s*Rp + prime[s])), so its update is the three calls above with NK = S*N keys.  k_eg_key (5077-5083): key[s*N + n] =
 * s*Rp + (xor over the last ord[s] token ids of tok * mult[s*4 + k]) mod prime[s], -1 for the first ord[s]-1 positions of a
 * sequence of T; canon (may be NULL) maps token ids first.  ord, prime [S] and mult [S*4] are DEVICE arrays the caller fills
 * (engram_setup's primes below the row count and splitmix64 multipliers, 5040-5047).  k_eg_gather (5084-5087): buf[n][s][:] =
 * the table row of key[s*N + n] (zeros for -1).  k_eg_scatter_c (5092-5097): compact gradient rows of the touched groups from
 * db [N][S][De], each element's positions added in ascending order. */
int qlmb_eg_key(int *key, const int *tok, const unsigned short *canon, const int *ord, const int *prime,
                const unsigned long long *mult, int N, int T, int S, int Rp, void *stream);
int qlmb_eg_gather(float *buf, const float *tbl, const int *key, int N, int S, int De, void *stream);
int qlmb_eg_scatter_compact(float *Gc, const int *key, const int *tgi, const int *count, const float *db, int N, int S, int De,
                            int group, int max_touched, void *stream);

/* The table's forward (ngram_forward, cudalm.cu:4701-4716).  k_ngram_key (4438-4445): key[n] = base + hash of the
 * last `order` token ids of position n, modulo R; -1 for the first order-1 positions of a sequence of T.
 * k_dec_ngkey (7056-7062): the same from a decoder slot's window of its last four tokens and its position.
 * k_ngram_gather (4446-4451): buf[n,:] = sum over the nk key sets (key[j*N + n], ascending j) of the table rows. */
int qlmb_ngram_key(int *key, const int *tok, int N, int T, int R, int order, int base, void *stream);
int qlmb_dec_ngkey(int *key, const int *tokw, const int *pos, int B, int R, int order, int base, void *stream);
int qlmb_ngram_gather(float *buf, const float *tbl, const int *key, int N, int De, int nk, void *stream);
/* The table's context gate (k_nggate_f / k_nggate_b, cudalm.cu:3362-3378; ngram_forward 4717-4718, ngram_backward 4725).
 * Forward, per row of D: g = sigmoid(<rms(h), rms(k)> / sqrt(D)); hn = rms(h); k = rms(k) in place; h += g * v in place;
 * g, rh = 1/rms(h), rk = 1/rms(k) are kept per row.  Backward: dv = g * dy; dk and the gate's share of dh from the
 * logit's gradient; dy += that share in place.  h, v, k, hn, dy, dv, dk share one element type (QLMB_F32 / QLMB_BF16). */
int qlmb_nggate_fwd(void *h, const void *v, void *k, void *hn, int dtype, float *g, float *rh, float *rk, int N, int D,
                    void *stream);
int qlmb_nggate_bwd(void *dy, const void *v, const void *hn, const void *kn, int dtype, const float *g, const float *rh,
                    const float *rk, void *dv, void *dk, int N, int D, void *stream);

/* k_qlm_servo (qlm.cuh:404-441). */
int qlmb_servo(int8_t *d, int8_t *r, float *s, const qlmb_span *sp, int nspan, int ngrp, int group,
               int dmax, float f_hi, float f_lo, int packed, void *stream);

/* k_sqsum + k_gnorm (cudalm.cu:2794-2812, 6442-6444): gs[0] = clip multiplier,
 * gs[1] = global gradient norm.  side/side_n are HOST arrays of nside device
 * pointers / lengths.  Partial sums follow the reference CPU build
 * (cpu_kern.h:533-540): 64 contiguous chunks, double accumulation.  Uses a
 * lazily grown per-device scratch buffer (cudaMalloc on first use). */
int qlmb_gnorm(const float *G, size_t n, const float *const *side, const size_t *side_n, int nside,
               int clip_side, float *gs, void *stream);

/* No counterpart in the reference.  qlmb_gnorm for hosts that cannot let a
 * library allocate device memory (all of it already belongs to their own pool,
 * or a cudaMalloc's device-wide synchronisation is not acceptable inside a
 * step): identical arguments and result, but the partial sums sit in a fixed
 * 64 KiB array inside the library, so no allocation happens on any path.
 * Limit: nside <= 7, more is rejected with QLMB_E_ARG.  The first call on a
 * device looks up the array's address -- make it before any stream capture.
 * Calls on one device share the array; calls that can overlap on the GPU race. */
int qlmb_gnorm_noalloc(const float *G, size_t n, const float *const *side, const size_t *side_n,
                       int nside, int clip_side, float *gs, void *stream);

/* Fused per-layer update (qlm_fused_layer / qlm_fused_tail, cudalm.cu:6105-6187): the optimizer
 * consumes a layer's gradients as soon as backward has produced them, so the gradient block of
 * one layer can be reused by the next, and the clip multiplier comes from the PREVIOUS step's norm.
 * A layer is: qlmb_sqsum of its gradient block into slice l of a caller-owned float[64 * nslice]
 * array (k_sqsum overwrites its 64 partials, cudalm.cu:6122), qlmb_step over the layer's groups
 * [gi0, gi0 + ng) with gsp = the gs word of the previous step, qlmb_adamw on its float spans.
 * After the last layer qlmb_gnorm_close adds all partials in ascending order in double
 * (cudalm.cu:6182-6186) and writes gs[0] = clip multiplier for the next step, gs[1] = norm --
 * on the device, where the reference copies the partials to the host.  qlmb_sqsum uses a fixed
 * 8 KiB array inside the library (no allocation); calls on one device must be stream-ordered. */
int qlmb_sqsum(const float *G, size_t n, float *part64, void *stream);
int qlmb_gnorm_close(const float *part, int nslice, float *gs, void *stream);

/* k_adamw (cudalm.cu:2855-2870) for the unquantised spans: bf16 moments,
 * gs (device, may be NULL) = the two floats k_gnorm writes: gs[0] is the clip
 * multiplier applied on load; a non-finite norm in gs[1] leaves P, M, V as they
 * were (the skipped step of cudalm.cu:6446-6447). */
int qlmb_adamw(float *P, const float *G, uint16_t *M, uint16_t *V, size_t n, float lr, float b1,
               float b2, float wd, float bc1, float bc2, const float *gs, void *stream);

/* ------------------------------------------------------- dequant-fused linears */

/* g_ab / g_abt / g_ab_res (cudalm.cu:3133-3172) on 4-bit codes instead of the
 * rendered fp32 view: Y[M,N] = X[M,K] * deq(W) (+ R).  X, Y, R have element
 * type `dtype` (QLMB_F32 or QLMB_BF16); the contraction runs on tcgen05 with
 * bf16 operands and fp32 accumulation.  K and N must be multiples of 128. */
int qlmb_linear_fwd(void *Y, const void *X, const int8_t *codes, const float *scales, int layout,
                    int M, int K, int N, const void *R, int dtype, void *stream);

/* g_abt_b / g_ab (cudalm.cu:3174-3186): dX[M,K] = dY[M,N] * deq(W)^T for the
 * same (codes, layout) as the forward; beta in {0,1} adds into dX. */
int qlmb_linear_dgrad(void *dX, const void *dY, const int8_t *codes, const float *scales,
                      int layout, int M, int K, int N, float beta, int dtype, void *stream);

/* g_atb (cudalm.cu:3190-3202): dW (fp32, the shape of W for `layout`)
 * = beta*dW + X^T dY resp. dY^T X; beta in {0,1} (the reference is always 1). */
int qlmb_linear_wgrad(float *dW, const void *dY, const void *X, int layout, int M, int K, int N,
                      float beta, int dtype, void *stream);

/* Decode path (cudalm.cu:7178-7198, g_ab with M = live slots <= 64):
 * Y[B,N] = X[B,K] * deq(W), weight-streaming kernel. */
int qlmb_gemv_decode(void *Y, const void *X, const int8_t *codes, const float *scales, int layout,
                     int B, int K, int N, int dtype, void *stream);

/* ------------------------------------------------------- router + permutation */

/* g_ab(f_norm, Wr) + k_router_topk (cudalm.cu:4158, 2515-2534).  If rt_in is
 * not NULL the logits are read from it (then X, Wr may be NULL); otherwise
 * they are computed as X[N,D] * Wr[D,E] in fp32 into rt_out (required then).  exp() is the reference CPU build's polynomial
 * (cpu_kern.h:28-34) so probabilities match the oracle bit for bit. */
int qlmb_router_topk(const float *rt_in, float *rt_out, const void *X, int x_dtype, const float *Wr,
                     const float *bias, int bias_stride, float *rprobs, int *assign, float *gate,
                     int N, int D, int E, int K, void *stream);

/* mbias_upd (cudalm.cu:3791-3802): the selection-only bias the router adds to its probabilities (qlmb_router_topk's
 * `bias`, [K][E] with per_slot, else [E]) moves towards the target load m after a step's routing:
 * b += u * (m - count) / m (proportional) or u * sign(m - count); m = N/E per pass, K*N/E combined.  assign is the
 * [K][N] table the router wrote.  The reference counts on the host and copies the bias back; this stays on the device. */
int qlmb_router_bias_update(float *bias, const int *assign, int N, int E, int K, int per_slot, float u, int proportional,
                            void *stream);

/* moe_perm_all / moe_gperm (cudalm.cu:3537-3602): stable grouping of token
 * slots by expert.  merged=0: K sorts of N entries, off[K*(E+1)], perm[k*N+pos];
 * merged=1: one sort of the K*N entries n' = k*N+n, off[E+1].
 * pad >= 1 rounds every expert's segment up to a multiple of `pad` rows; the
 * filler entries of perm are -1 (the reference's capacity-padded form,
 * cudalm.cu:3597-3599) and off holds the padded offsets.  inv (may be NULL)
 * receives the position of every entry.  perm must hold
 * len + E*(pad-1) ints per sort.  bad_flag (device int) is set to
 * 0x40000000|e when an expert index e is out of range (cudalm.cu:3507).
 * counts (may be NULL) receives the unpadded per-expert counts. */
int qlmb_perm_build(const int *assign, int N, int E, int K, int merged, int pad, int *perm, int *inv,
                    int *off, int *counts, int *bad_flag, void *stream);

/* ------------------------------------------------------------- MoE expert FFN */

typedef struct {
    int N, D, F, E, K;        /* tokens, d_model, d_ff, experts, top-k            */
    int dtype;                /* element type of f_in / f_norm / out / dout / dfnorm */
    const int8_t *w1_codes, *w3_codes, *w2_codes; /* [E][D][F], [E][D][F], [E][F][D]  */
    const float *w1_scales, *w3_scales, *w2_scales;
    const float *wr;          /* router weights [D][E], fp32                      */
    const float *bias;        /* selection-only bias [K][bias_stride] or NULL     */
    int bias_stride;
    float aux;                /* load-balance coefficient (cudalm.cu:3334)        */
} qlmb_moe_layer;

/* Bytes of the per-layer activation arena the two calls below share (the MoE
 * members of the reference's GA, cudalm.cu:3308-3333, with the stash on). */
size_t qlmb_moe_arena_bytes(int N, int D, int F, int E, int K);
/* Device pointer of a named arena member ("rt","rprobs","assign","gate",
 * "perm","inv","off","counts","Xp","gp","up","ap","yp","d_gate","drt","dyp",
 * "dgp","dup","dXp","ntiles","bad") or NULL. rows_out receives its row capacity. */
void *qlmb_moe_arena_member(void *arena, int N, int D, int F, int E, int K, const char *name);

/* The same forward for a decode step (dec_step, cudalm.cu:7199): nothing is stashed for a backward pass.
 * With K*N <= 128 routed rows and bf16 activations the experts run as GEMVs over the chosen experts' codes
 * only; otherwise this is qlmb_moe_forward.  The arena's "assign", "gate", "rprobs" members are filled. */
int qlmb_moe_decode(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in, const void *f_norm,
                    void *stream);
/* moe_forward (cudalm.cu:4151-4229): out = f_in + sum_k gate_k * FFN_e(f_norm). */
int qlmb_moe_forward(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in,
                     const void *f_norm, void *stream);

/* qlmb_moe_forward with the router's logits supplied by the caller instead of computed from f_norm
 * (rt_in [N][E] fp32, the `rt_in` of qlmb_router_topk); everything after the logits is the same code, and
 * qlmb_moe_backward works on the result as usual.  The reference has no such switch: it exists so that this
 * library and the reference's CPU build can be compared on identical expert choices (a near-tie of two
 * logits is decided differently by bf16 and fp32 activations). */
int qlmb_moe_forward_routed(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in,
                            const void *f_norm, const float *rt_in, void *stream);

/* moe_backward (cudalm.cu:4233-4393): consumes dout, produces dfnorm and adds
 * the weight gradients into dW1/dW3/dW2/dWr (fp32; beta=1 as the reference,
 * beta=0 overwrites, valid when G was just zeroed). */
int qlmb_moe_backward(const qlmb_moe_layer *L, void *arena, void *dfnorm, const void *dout,
                      const void *f_norm, float *dW1, float *dW3, float *dW2, float *dWr,
                      float beta, void *stream);

/* ----------------------------------------------------- expert parallelism (new)
 * The reference runs on one GPU.  These six calls are moe_forward / moe_backward
 * (cudalm.cu:4151-4393) cut where rows cross GPUs when the experts are sharded:
 * the home rank of a token routes and packs (route), the expert's rank computes
 * (experts_forward / experts_backward) and the home rank finishes (combine,
 * dgate, route_backward).  The caller moves the packed rows between ranks
 * (all-to-all) between the calls.  Packed rows are bf16 [K*N][D], grouped by
 * global expert index in stable order, no filler rows; the number of rows per
 * expert is arena member "counts".  qlmb_moe_route needs only L->wr (+bias);
 * the experts_* calls need only the expert weights, with L->E = experts held by
 * the rank, L->N = row capacity of `earena` = qlmb_moe_arena_bytes(N,D,F,E,1). */
int qlmb_moe_route(const qlmb_moe_layer *L, void *arena, void *Xs, const void *f_norm, void *stream);
int qlmb_moe_experts_forward(const qlmb_moe_layer *L, void *earena, void *Y, const void *X,
                             const int *expert_of_row, int R, void *stream);
int qlmb_moe_combine(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in, const void *Ys,
                     void *stream);
int qlmb_moe_dgate(const qlmb_moe_layer *L, void *arena, void *dYs, const void *dout, const void *Ys,
                   void *stream);
int qlmb_moe_experts_backward(const qlmb_moe_layer *L, void *earena, void *dX, const void *dY, int R,
                              float *dW1, float *dW3, float *dW2, float beta, void *stream);
int qlmb_moe_route_backward(const qlmb_moe_layer *L, void *arena, void *dfnorm, const void *dXs,
                            const void *f_norm, float *dWr, float beta, void *stream);

/* ------------------------------------------------------------ QLMH state file
 * The reference's checkpoint of the integer optimizer state (qlm_save / qlm_load,
 * qlm.cuh:703-788), same bytes, on caller-owned HOST arrays: copy the device state to the
 * host, call qlmb_statefile_write; or size the arrays from qlmb_statefile_read_header, call
 * qlmb_statefile_read and upload.  d holds (nq+1)/2 bytes when packed, else nq; v8 / v8s
 * exist only with adam != 0; Mc / Vc are the bf16 moments of the float spans (cudalm.cu:
 * 2855-2870); sref[i] is span i's frozen reference scale (the file's SREF trailer); prev_gn
 * is the previous step's gradient norm (PGN1 trailer).  Reading refuses a file whose
 * dmax/group/adam/packed/nq/ngrp differ from the caller's fields or that holds more
 * float-span moments than the caller (QLMB_E_UNSUPPORTED), like the reference. */
typedef struct qlmb_statefile {
    int dmax, group, adam, nspan, packed, iter;
    unsigned long long nq, ngrp, nfloat;
    unsigned short *Mc, *Vc;
    int8_t *d, *r, *m8;
    uint8_t *v8;
    float *s, *m8s, *v8s;
    float *sref;
    int have_sref;
    float prev_gn;
    int have_prev_gn;
} qlmb_statefile;
int qlmb_statefile_write(const char *path, const qlmb_statefile *v);
int qlmb_statefile_read_header(const char *path, qlmb_statefile *v);
int qlmb_statefile_read(const char *path, qlmb_statefile *v);

/* Model file of the reference (model_save_bundle / model_load_full, cudalm.cu:554-565, 431-466): "TLM4" + 11 ints
 * {V, D, L, H, KV, F, T, eot, tmpl, n_mtp, n_exp} ("TLM5" + 13 ints with {win, full_every} when win > 0), the fp32
 * parameter vector in the reference's layout, the tokenizer blob's length and bytes.  hdr13 always has 13 ints.
 * Written through a temporary file and an atomic rename, like the reference.  A run whose quantised weights exist
 * only as digits writes their rendered values (qlmb_render into a host-bound buffer). */
int qlmb_modelfile_write(const char *path, const int *hdr13, const float *P, unsigned long long n, const void *tok_blob,
                         int tok_bytes);
int qlmb_modelfile_read_header(const char *path, int *hdr13, unsigned long long *n_params, int *tok_bytes);
int qlmb_modelfile_read(const char *path, float *P, unsigned long long n, void *tok_blob, int tok_cap, int *tok_bytes);

/* Exact 4-bit export ("q4n") of a parameter vector and the quantised container file (quantize_params /
 * dequantize_params with qtype 3, cudalm.cu:639-656, 688-695; the quantize command's TLQ1 / TLQ2 writer, 9783-9793, and
 * model_load_full's reader, 438-450).  Per group of `group` values (the reference uses 128): a fp32 scale and ceil(g/2)
 * nibble-pair bytes, or, where no scale puts the group on a 4-bit grid, a NaN scale and the g raw fp32 values.  The scale
 * search is the reference's (amax/k for k = 7..1 with its +-1 and +-2 ulp neighbours), so a vector rendered from 4-bit
 * digits exports without loss and the stream is byte-identical to the reference's.
 *   qlmb_q4n_export   P, out, work on the device; totals (device) receives {stream bytes, raw groups}; nothing is
 *                     written to out when the stream would exceed cap (check totals[0] <= cap after the stream is done).
 *                     out 4-byte aligned; work = qlmb_q4n_work_bytes(n, group) bytes, 8-byte aligned; group % 8 == 0.
 *   qlmb_q4n_index    HOST walk of a stream (host memory) that yields the byte offset of every group, off[groups + 1];
 *                     the position of a group depends on the kind of every group before it.
 *   qlmb_q4n_decode   P[i] = digit * scale (or the raw value) on the device from the stream and its offsets, both on
 *                     the device.
 * qlmb_qfile_*: "TLQ1" + 11 header ints ("TLQ2" + 13 when hdr13[11], the window, is set), qtype, group, the body, the
 * tokenizer blob's length and bytes.  read_header gives the number of bytes after `group`; read copies them to a host
 * buffer, whose body part qlmb_q4n_index measures (off[groups] = body bytes; the tokenizer trailer follows). */
unsigned long long qlmb_q4n_work_bytes(unsigned long long n, int group);
unsigned long long qlmb_q4n_max_bytes(unsigned long long n, int group);
int qlmb_q4n_export(unsigned char *out, unsigned long long cap, unsigned long long *totals, const float *P,
                    unsigned long long n, int group, void *work, void *stream);
int qlmb_q4n_index(const unsigned char *host_stream, unsigned long long len, unsigned long long n, int group,
                   unsigned long long *off);
int qlmb_q4n_decode(float *P, const unsigned char *in, const unsigned long long *off, unsigned long long n, int group,
                    void *stream);
int qlmb_qfile_write(const char *path, const int *hdr13, int qtype, int group, const void *body, unsigned long long body_len,
                     const void *tok_blob, int tok_bytes);
int qlmb_qfile_read_header(const char *path, int *hdr13, int *qtype, int *group, unsigned long long *rest);
int qlmb_qfile_read(const char *path, void *buf, unsigned long long rest);

/* ------------------------- expert parallelism over peer memory (new, no reference counterpart)
 * Same cut of moe_forward / moe_backward (cudalm.cu:4151-4393), but rows never travel in a
 * separate exchange: every rank places its inputs, its Ys / dXs buffers and both arenas in one
 * "window" of device memory that the other ranks of the node map (qlmb_peer_*), all windows have
 * the same layout, and rows cross NVLink inside kernels that exist anyway: the expert side's
 * gather reads token rows (and, in the backward, dout rows and gates) from their home rank with
 * peer loads; the epilogues of its down-projection and dX GEMMs store every output row straight
 * into the Ys / dXs buffer of the row's home rank, at the row's slot k*N + n.
 * The caller provides the stream-ordered synchronisation between the calls with collectives of
 * its own (no kernel of this library waits for another GPU):
 *   qlmb_ep_route            every rank
 *   all-gather of arena member "assign" ([K*N] ints per rank) into assign_all[W][K*N]
 *   qlmb_ep_experts_forward  every rank, for the experts it holds; fills the Ys of all ranks
 *   barrier
 *   qlmb_ep_combine          (forward done)
 *   qlmb_ep_dgate
 *   qlmb_ep_experts_backward fills the dXs of all ranks
 *   barrier
 *   qlmb_ep_route_backward
 * The all-gather of the next step is the barrier that protects Ys, dXs and the arenas from being
 * overwritten while a slower rank still reads them.  Global slot g = s*K*N + k*N + n is copy k
 * of token n of rank s.  `home` describes the router side (N tokens of this rank, E experts in
 * total, K, wr); `loc` the expert side (E = experts held by this rank, rank r holds experts
 * [r*E_loc, (r+1)*E_loc), N = W*K*N_home slots, the capacity of `earena` =
 * qlmb_moe_arena_bytes(loc->N, D, F, loc->E, 1)).  f_norm, dout, Ys, dXs (bf16 [K*N][D] each),
 * harena and earena must lie inside this rank's window; the same offsets are used in the peers'. */
#define QLMB_EP_MAX_WORLD 8
typedef struct qlmb_ep_peers {
    int rank, world;
    void *base[QLMB_EP_MAX_WORLD];   /* window of rank i as mapped into this process; base[rank] = own */
} qlmb_ep_peers;

/* device memory that other processes of the node can map */
int qlmb_peer_alloc(size_t bytes, void **ptr);
int qlmb_peer_free(void *ptr);
int qlmb_peer_export(const void *ptr, unsigned char handle[64]);
int qlmb_peer_open(const unsigned char handle[64], void **ptr);
int qlmb_peer_close(void *ptr);

int qlmb_ep_route(const qlmb_moe_layer *home, void *harena, const void *f_norm, void *stream);
int qlmb_ep_experts_forward(const qlmb_moe_layer *loc, void *earena, const qlmb_ep_peers *peers,
                            const int *assign_all, const void *f_norm, int x_dtype, int tokens_per_rank,
                            int K, void *Ys, void *stream);
int qlmb_ep_combine(const qlmb_moe_layer *home, void *harena, const void *Ys, void *out, const void *f_in,
                    void *stream);
int qlmb_ep_dgate(const qlmb_moe_layer *home, void *harena, const void *Ys, const void *dout, void *stream);
int qlmb_ep_experts_backward(const qlmb_moe_layer *loc, void *earena, const qlmb_moe_layer *home,
                             void *harena, const qlmb_ep_peers *peers, const void *dout, int tokens_per_rank,
                             int K, void *dXs, float *dW1, float *dW3, float *dW2, float beta, void *stream);
int qlmb_ep_route_backward(const qlmb_moe_layer *home, void *harena, const void *dXs, void *dfnorm,
                           const void *f_norm, float *dWr, float beta, void *stream);

/* ------------------------- native multi-GPU host layer (new, no reference counterpart: the reference is single-GPU)
 * One process per GPU.  NCCL is bound at run time (the libnccl.so.2 the process has loaded, else the system's, else
 * the path in QLMB_NCCL_LIB); without it these calls return QLMB_E_UNSUPPORTED and the rest of the library works.
 * Rank 0 makes the 128-byte id (qlmb_comm_unique_id) and hands it to the other ranks by any host channel; every
 * rank then calls qlmb_comm_init with its device current.  All collectives are enqueued on the caller's stream.
 *   qlmb_comm_allreduce_f32   sum (avg = 0) or mean (avg = 1), in place
 *   qlmb_comm_allgather       recv[r*bytes..] = rank r's bytes; send == recv + rank*bytes gathers in place
 *   qlmb_comm_barrier         stream-ordered meeting point (a one-int all-reduce); nothing waits on the host
 *   qlmb_dp_grad_sync         data parallelism: the replicated parameters' gradient becomes the mean over the ranks
 *   qlmb_dp_gnorm_close       qlmb_gnorm_close after the partial sums of rank-local buffers (expert shards),
 *                             slices [first_local, nslice), have been summed over the ranks
 *   qlmb_zero1_step           qlmb_step on this rank's share of the groups (ngrp % world == 0), then an all-gather of
 *                             the new codes: every rank ends with the codes qlmb_step on the whole span gives, bit
 *                             for bit, while residuals and moments of a share never leave its rank
 *   qlmb_zero1_gather_scales  after a servo pass over the share: the scales of all groups on every rank
 *   qlmb_ep_window_open       maps every rank's window (qlmb_peer_alloc) into this process; _close unmaps them
 *   qlmb_ep_layer_forward     qlmb_ep_route, all-gather of the routing table into assign_all [world][K*N],
 *                             qlmb_ep_experts_forward, meeting point, qlmb_ep_combine
 *   qlmb_ep_layer_backward    qlmb_ep_dgate, (meeting point when dout was written this step: inputs_fresh),
 *                             qlmb_ep_experts_backward, meeting point, qlmb_ep_route_backward */
typedef struct qlmb_comm qlmb_comm;
int qlmb_comm_unique_id(unsigned char id[128]);
int qlmb_comm_init(qlmb_comm **comm, const unsigned char id[128], int rank, int world);
int qlmb_comm_destroy(qlmb_comm *comm);
int qlmb_comm_rank(const qlmb_comm *comm);
int qlmb_comm_world(const qlmb_comm *comm);
int qlmb_comm_allreduce_f32(qlmb_comm *comm, float *buf, unsigned long long n, int avg, void *stream);
int qlmb_comm_allgather(qlmb_comm *comm, const void *send, void *recv, unsigned long long bytes, void *stream);
int qlmb_comm_barrier(qlmb_comm *comm, void *stream);
int qlmb_dp_grad_sync(qlmb_comm *comm, float *G, unsigned long long n, void *stream);
int qlmb_dp_gnorm_close(qlmb_comm *comm, float *part, int nslice, int first_local, float *gs, void *stream);
int qlmb_zero1_step(qlmb_comm *comm, float *P, const float *G, int8_t *d, int8_t *r, const float *s, int8_t *m8,
                    float *m8s, uint8_t *v8, float *v8s, const qlmb_span *sp, int nspan, int ngrp, int group,
                    int dmax, float lr, float b1, float b2, float wd, float gscale, const float *gsp,
                    float inv_bc1, float inv_sqrt_bc2, int lrmode, uint64_t t, int adam, int64_t *stat,
                    int packed, void *stream);
int qlmb_zero1_gather_scales(qlmb_comm *comm, float *s, int ngrp, void *stream);
int qlmb_ep_window_open(qlmb_comm *comm, void *window, qlmb_ep_peers *peers, void *stream);
int qlmb_ep_window_close(qlmb_comm *comm, qlmb_ep_peers *peers, void *stream);
int qlmb_ep_layer_forward(qlmb_comm *comm, const qlmb_moe_layer *home, void *harena, const qlmb_moe_layer *loc, void *earena,
                          const qlmb_ep_peers *peers, int *assign_all, const void *f_norm, int x_dtype, const void *f_in,
                          void *Ys, void *out, void *stream);
int qlmb_ep_layer_backward(qlmb_comm *comm, const qlmb_moe_layer *home, void *harena, const qlmb_moe_layer *loc, void *earena,
                           const qlmb_ep_peers *peers, const void *dout, const void *f_norm, const void *Ys, void *dXs,
                           void *dfnorm, float *dW1, float *dW3, float *dW2, float *dWr, float beta, int inputs_fresh,
                           void *stream);

/* g_abt / g_ab on unquantised operands (the lm_head over the tied embedding, cudalm.cu:5832-5858):
 * C[M,N] = A[M,K] B[N,K]^T (+ C when beta = 1); A and B bf16, C fp32 or bf16; K % 64 == 0, N % 128 == 0.
 * logits = fn emb^T uses B = the bf16 copy of emb [V, D]; dfn = dlogits emb uses B = the transposed copy
 * [D, V]; dEmb += dlogits^T fn is qlmb_linear_wgrad (layout NK) into the fp32 gradient. */
int qlmb_gemm_nt(void *C, int c_dtype, const void *A, const void *B, int M, int K, int N, float beta, void *stream);
/* bf16 copies of an fp32 matrix src[R][C]: dst [R][C] and / or dst_t [C][R] (either may be NULL); the
 * reference casts the embedding once per step for its head GEMMs too (cudalm.cu:5822-5829). */
int qlmb_cast_bf16(void *dst, void *dst_t, const float *src, int R, int C, void *stream);

/* ---- the memory-bound operators around the GEMMs of a block ----
 * Activations are QLMB_F32 or QLMB_BF16 per tensor, arithmetic is fp32, D % 4 == 0.  No floating-point
 * atomics: results are run-to-run identical.
 * k_embed (cudalm.cu:5740; cpu_kern.h:87-90): X[n,:] = emb[tok[n],:]. */
int qlmb_embed(void *X, int x_dtype, const float *emb, const int *tok, int N, int D, void *stream);
/* k_embed_bwd (cudalm.cu:6000; cpu_kern.h:92-98): G[tok[n],:] += dout[n,:], the rows of one token in
 * ascending n (the order of the reference's CPU build; its GPU kernel uses atomics).  G is [V, D]. */
int qlmb_embed_bwd(float *G, const void *dout, int dtype, const int *tok, int N, int D, int V, void *stream);
/* e_rmsf / k_rmsnorm (cudalm.cu:3635-3637; cpu_kern.h:103-109): O = X * rinv * gamma,
 * rinv[n] = 1/sqrt(mean(X[n,:]^2) + 1e-5) is saved for the backward pass. */
int qlmb_rmsnorm_fwd(void *O, int o_dtype, float *rinv, const void *X, int x_dtype, const float *gamma, int N, int D,
                     void *stream);
/* e_rmsb (cudalm.cu:3638-3645; cpu_kern.h:110-138): dx = (accumulate ? dx : 0) + rinv*gamma*dy -
 * (rinv^3/D * sum(x*gamma*dy)) * x; when dgamma is not NULL, dgamma[j] += sum_n x*rinv*dy summed over
 * 128 fixed row chunks and then over the chunks (k_gamma_part / k_gamma_sum), with `part` a scratch of
 * 128 * D floats. */
int qlmb_rmsnorm_bwd(void *dx, int dx_dtype, int accumulate, float *dgamma, float *part, const void *X, int x_dtype,
                     const float *gamma, const float *rinv, const void *dy, int dy_dtype, int N, int D, void *stream);
/* e_rope / k_rope (cudalm.cu:3630; cpu_kern.h:139-152): rotate pairs (i, i + hd/2) of every head of
 * buf[N, nh, hd] in place by the angle of position n % T (tables cosb, sinb [T, hd/2]); back = 1 applies
 * the transpose (the gradient). */
int qlmb_rope(void *buf, int dtype, const float *cosb, const float *sinb, int N, int nh, int hd, int T, int back,
              void *stream);
/* k_softmax_ce (cudalm.cu:5838; cpu_kern.h:489-503, without per-token weights): per row
 * loss = -log(p[tgt] + 1e-12) and dlogits = (p - onehot) / n_all; rows with tgt < 0 give 0 and a zero row. */
int qlmb_softmax_ce(const void *logits, int lg_dtype, const int *tgt, float *loss, void *dlogits, int dl_dtype, int rows,
                    int V, int n_all, void *stream);

/* The q, k, v projections of a decode step in one call (cudalm.cu:7178-7180): nmat matrices of the same shape
 * stored one after the other (codes W_m[K][N], groups along N), Y[m*B + b, :] = X[b, :] deq(W_m); nmat*B <= 256.
 * Every output row is computed by its own blocks (the matrices of a projection fit the L2), so this is for small
 * matrices and few rows; nmat = 1 is a plain GEMV without row batching. */
int qlmb_gemv_decode_stack(void *Y, const void *X, const int8_t *codes, const float *scales, int nmat, int B, int K,
                           int N, int dtype, void *stream);
/* qlmb_gemv_decode_stack on the normalised rows: X is multiplied by rinv * gamma (rinv = 1/sqrt(mean(x^2) + 1e-5)) and
 * rounded to bf16 while it is staged, so the norm in front of the q, k, v projections (e_rmsf, cudalm.cu:7176) needs no
 * launch and no buffer of its own. */
int qlmb_gemv_decode_norm_stack(void *Y, const void *X, const float *gamma, const int8_t *codes, const float *scales, int nmat,
                                int B, int K, int N, int dtype, void *stream);
/* The attention input of a decode step in one launch pair (dec_step, cudalm.cu:7176-7183: e_rmsf, g_ab on wq / wk / wv,
 * k_dec_rope on q and k, k_dec_kv) for models whose key width equals D: Y[3][B][D] = the q, k, v rows (q and k rotated
 * by the angle of pos[b]), and the k, v rows are stored at position pos[b] of the bf16 caches Kc, Vc [B][Tm][D].
 * wq, wk, wv are three [D][D] code matrices stored one after the other; bf16 activations; 3 * B <= 256. */
int qlmb_dec_qkv(void *Y, void *Kc, void *Vc, const void *X, const float *gamma, const int8_t *codes, const float *scales,
                 const float *cosb, const float *sinb, const int *pos, int B, int D, int hd, int Tm, void *stream);
/* The output projection of a decode step with what follows it (dec_step, cudalm.cu:7188-7190: g_ab on wo, the
 * residual add, the norm in front of the FFN) in one launch pair: F = bf16(X deq(W)) + res, Fn = F * rinv * gamma with
 * rinv = 1/sqrt(mean(F^2) + 1e-5).  bf16 activations, codes W[K][N], B <= 256 slots, N <= 2048. */
int qlmb_gemv_decode_res_norm(void *F, void *Fn, const void *X, const int8_t *codes, const float *scales, const void *res,
                              const float *gamma, int B, int K, int N, void *stream);

/* ---- decoder: one new token per live slot (dec_step, cudalm.cu:7166-7212) ----
 * The K/V cache of a layer is bf16 [B, Tm, KV*hd]; pos[b] (device) is the position of slot b's new token.
 * k_dec_rope (cudalm.cu:7023-7027): rotate the single row of each slot by the angle of pos[b]; the tables have Tm rows,
 * and a slot whose position lies outside them is reported through the device error word and left unrotated. */
int qlmb_dec_rope(void *buf, int dtype, const float *cosb, const float *sinb, const int *pos, int B, int nh, int hd,
                  int Tm, void *stream);
/* k_dec_kv (cudalm.cu:7028-7030): append the new key / value rows (bf16 [B, KD]) at pos[b]. */
int qlmb_dec_kv(void *Kc, void *Vc, const void *k, const void *v, const int *pos, int B, int Tm, int KD, void *stream);
/* k_dec_attn (cudalm.cu:7031-7047): O[b, h*hd..] = softmax(q k^T / sqrt(hd)) v over cached positions
 * max(0, pos-win+1) .. pos[b] (win <= 0: all); Q, O bf16 [B, H*hd]; hd = 64, Tm <= 4096. */
int qlmb_dec_attn(void *O, const void *Q, const void *Kc, const void *Vc, const int *pos, int win, int B, int Tm, int H,
                  int KV, int hd, void *stream);
/* Per-slot sampling parameters, the layout of the reference's DSP (cudalm.cu:7020). */
typedef struct {
    float temp, top_p;          /* temp <= 0: greedy; top_p >= 1: no nucleus cut */
    int top_k;                  /* 0: no cut; 1: greedy */
    unsigned long long seed;
    int step;                   /* the draw is hashed from (seed, step) */
} qlmb_dec_sampling;
/* k_dec_sample (cudalm.cu:7048-7108): top_k -> top_p -> temperature over logits[b,:], greedy when
 * temp <= 0 or top_k == 1; out[b] = the picked token, lp[b] = its log-probability under the
 * unmodified distribution.  params is a device array of B entries.  Candidates are ordered by value
 * and then by token index, so the pick does not depend on scheduling. */
int qlmb_dec_sample(int *out, float *lp, const float *logits, const qlmb_dec_sampling *params, int B, int V,
                    void *stream);
/* The greedy branch of k_dec_sample (cudalm.cu:7078-7093, temp <= 0): out[b] = arg-max of logits[b,:] (lowest
 * index on ties), lp[b] = its log-probability. */
int qlmb_dec_greedy(int *out, float *lp, const float *logits, int B, int V, void *stream);

/* ---- attention (rows of Q/K/V/O are tokens b*T + t; head h occupies columns [h*hd, (h+1)*hd)) ----
 * e_attn / k_attn_fwd (cudalm.cu:3705-3730; CPU twin cpu_kern.h:166-229): causal attention with an
 * optional window (win > 0: keys t-win+1 .. t), grouped-query heads (head h reads K/V head
 * h / (H/KV)), scores scaled by 1/sqrt(hd); lse[b,h,t] = max + log(sum) of the scaled scores.
 * Q [B*T, H*hd], K and V [B*T, KV*hd], O [B*T, H*hd] are bf16 with RoPE already applied to Q and K;
 * hd must be 64. */
int qlmb_attn_fwd(void *O, float *lse, const void *Q, const void *K, const void *V, int B, int T, int H,
                  int KV, int hd, int win, void *stream);

/* Attention backward (gpu_backward, cudalm.cu:5918-5960: k_attn_drow, then dQ / dK / dV; CPU twins
 * cpu_kern.h:255-322).  drow[b,h,t] = sum_d dA * O is written first (B*H*T floats, also an output);
 * dQ [B*T, H*hd], dK and dV [B*T, KV*hd] are bf16 and are overwritten (the reference zeroes its
 * buffers and accumulates once).  Every element has one writer and a fixed summation order:
 * dK/dV come from one CTA per (sequence, K/V head, key tile) that walks the heads of the group and the
 * query tiles, dQ from one CTA per (sequence, head, query tile). */
int qlmb_attn_bwd(void *dQ, void *dK, void *dV, float *drow, const void *Q, const void *K, const void *V,
                  const void *O, const void *dA, const float *lse, int B, int T, int H, int KV, int hd,
                  int win, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QLM_B200_H */
