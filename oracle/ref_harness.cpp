/* ref_harness.cpp -- C-ABI shim over the UNMODIFIED reference translation unit.
 *
 * TEST INFRASTRUCTURE ONLY (the checker and the timed CPU baseline); the
 * shipped library never links or loads it.  The reference (Dsg2/cudalm-c) is a
 * single translation unit whose operators are `static`; its own CPU build
 * (-DCUDALM_CPU) replaces the CUDA runtime and cuBLAS with host stand-ins.
 * This file includes that translation unit where it lies (the include path is
 * given on the command line by the Makefile; no reference source is copied)
 * and re-exports the operators on the QLM path under extern "C" names.
 *
 * Two flavours are built from this one file:
 *   libcudalm_ref_exact.so  -ffp-contract=off : the parity oracle
 *   libcudalm_ref_fast.so   stock flags       : the timed CPU baseline
 */
#define main cudalm_reference_main
#include "cudalm.cu"
#undef main

extern "C" {

int ref_threads(void) { return omp_get_max_threads(); }
/* a launcher may have exported OMP_NUM_THREADS=1 for its workers: the timed baseline sets its own count */
void ref_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

/* ---- QLM state ops (qlm.cuh:136-178, 377-397, 404-441) ---- */
void ref_encode(const float *P, signed char *d, signed char *r, float *s, const QSpanD *sp,
                int nspan, int ngrp, int group, int dmax, int packed)
{
    KL(k_qlm_encode, (unsigned)ngrp, group, group)(P, d, r, s, sp, nspan, group, dmax, packed);
}
void ref_render(float *P, const signed char *d, const float *s, const QSpanD *sp, int nspan,
                int group, int packed, int gi_base, int ng)
{
    KL(k_qlm_render, (unsigned)ng, group)(P, d, s, sp, nspan, group, packed, gi_base);
}
void ref_step(float *P, const float *G, signed char *d, signed char *r, float *s, signed char *m8,
              float *m8s, unsigned char *v8, float *v8s, const QSpanD *sp, int nspan, int group,
              int dmax, float lr, float b1, float b2, float wd, float gscale, const float *gsp,
              float inv_bc1, float inv_sqrt_bc2, int lrmode, unsigned long long t, int adam,
              long long *stat, int packed, int gi_base, int ng)
{
    qlm_step_launch(P, G, d, r, s, m8, m8s, v8, v8s, sp, nspan, group, dmax, lr, b1, b2, wd,
                    gscale, gsp, inv_bc1, inv_sqrt_bc2, lrmode, t, adam, stat, packed, gi_base, ng);
}
/* QLM_V4: the CPU build's copy of the device global (qlm.cuh:65) */
void ref_set_v4(int on) { d_qv4 = on ? 1 : 0; }
void ref_servo(signed char *d, signed char *r, float *s, const QSpanD *sp, int nspan, int ngrp,
               int group, int dmax, float f_hi, float f_lo, int packed)
{
    KL(k_qlm_servo, (unsigned)ngrp, group, group)(d, r, s, sp, nspan, group, dmax, f_hi, f_lo, packed);
}
unsigned ref_hash(unsigned long long x) { return qhashu(x); }
int ref_sround(float v, unsigned long long i, unsigned long long t) { return qsri(v, i, t); }

/* ---- grad-norm clip (cudalm.cu:6442-6444) and float-span AdamW (2855-2870) ---- */
void ref_gnorm(const float *G, size_t n, const float *const *side, const size_t *side_n, int nside,
               int clip_side, float *gs)
{
    float *part = (float *)malloc(sizeof(float) * 64 * (size_t)(1 + nside));
    KL(k_sqsum, 64, TPB)(G, n, part);
    for (int i = 0; i < nside; i++) KL(k_sqsum, 64, TPB)(side[i], side_n[i], part + 64 * (1 + i));
    KL(k_gnorm, 1, 1)(part, nside, clip_side, gs);
    free(part);
}
/* the 64 partial sums of one buffer, as qlm_fused_layer / qlm_fused_tail take them (cudalm.cu:6122, 6181) */
void ref_sqsum(const float *G, size_t n, float *part64) { KL(k_sqsum, 64, TPB)(G, n, part64); }
void ref_adamw(float *P, const float *G, unsigned short *M, unsigned short *V, size_t n, float lr,
               float b1, float b2, float wd, float bc1, float bc2, const float *gs)
{
    KL(k_adamw, nblk(n, TPB), TPB)(P, G, M, V, n, lr, b1, b2, wd, bc1, bc2, NULL, 0, 0, 0, MU_OFF, gs);
}

/* ---- block operators around the GEMMs (cpu_kern.h:87-152, 489-503; call sites gpu_forward / gpu_backward) ---- */
void ref_embed(const float *emb, const int *tok, float *X, int N, int D) { KL(k_embed, 1, 1)(emb, 0, tok, X, N, D); }
void ref_embed_bwd(const int *tok, const float *dout, float *G, int N, int D) { KL(k_embed_bwd, 1, 1)(tok, dout, G, 0, N, D); }
void ref_rmsnorm(const float *X, const float *gamma, float *O, float *rinv, int N, int D) { KL(k_rmsnorm, N, TPB)(X, gamma, 0, O, rinv, N, D); }
/* e_rmsb (cudalm.cu:3638-3645): dx += ..., then the gain gradient through GG_CH row chunks */
void ref_rmsnorm_bwd(const float *X, const float *gamma, const float *rinv, const float *dy, float *dx, float *dgamma, int N, int D)
{
    KL(k_rmsnorm_bwd, N, TPB)(X, gamma, 0, rinv, dy, dx, N, D);
    float *part = (float *)malloc(sizeof(float) * (size_t)GG_CH * D);
    KL(k_gamma_part, dim3((unsigned)nblk(D, TPB), GG_CH), TPB)(X, rinv, dy, part, N, D);
    KL(k_gamma_sum, nblk(D, TPB), TPB)(part, dgamma, 0, D);
    free(part);
}
void ref_rope(float *buf, const float *cosb, const float *sinb, int N, int nh, int hd, int T, int back)
{
    KL(k_rope, 1, 1)(buf, cosb, sinb, N, nh, hd, hd / 2, T, back);
}
void ref_softmax_ce(const float *lg, const int *tgt, float *loss, float *dl, int rows, int V, int n_all)
{
    KL(k_softmax_ce<float>, rows, TPB)(lg, tgt, loss, dl, (__nv_fp8_e4m3 *)NULL, rows, V, n_all, (const float *)NULL, 0.05f);
}

/* ---- attention (cpu_kern.h:166-229 forward, 255-312 backward; call sites cudalm.cu:3705-3730, 5918-5936) ---- */
void ref_attn_fwd(const float *Q, const float *K, const float *V, float *O, float *lse, int win, int B, int T,
                  int H, int KV, int hd)
{
    KL(k_attn_fwd, 1, 1)(Q, K, V, O, lse, win, B, T, H, KV, hd, H * hd, KV * hd);
}
/* dQ, dK, dV are accumulated into (the caller zeroes them, as gpu_backward does) */
void ref_attn_bwd(const float *Q, const float *K, const float *V, const float *O, const float *dA, const float *lse,
                  float *drow, float *dQ, float *dK, float *dV, int win, int B, int T, int H, int KV, int hd)
{
    KL(k_attn_drow, B * H * T, 32)(dA, O, drow, B, T, H, hd, H * hd, 1.0f);
    cpu_attn_bwd(Q, K, V, dA, lse, drow, dQ, dK, dV, win, B, T, H, KV, hd, H * hd, KV * hd);
}

/* ---- n-gram table forward (cpu_kern.h:598-610) ---- */
void ref_ngram_key(const int *tok, int *key, int N, int T, int R, int order, int base) { KL(k_ngram_key, 1, 1)(tok, key, N, T, R, order, base); }
void ref_ngram_gather(const float *tbl, const int *key, float *buf, int N, int De, int nk) { KL(k_ngram_gather, 1, 1)(tbl, key, buf, N, De, nk); }

/* ---- aux-free balancing: the selection bias after a step's routing (mbias_upd, cudalm.cu:3793-3802) on the caller's
 * rows b[ns][E]; cs = ns count rows, m = target load, u and lmul = CUDALM_MOE_BIAS and the layer's multiplier ---- */
void ref_mbias_upd(float *b, const int *cs, int ns, int E, float m, float u, float lmul, int prop)
{
    float su = g_mbias_u, *sH = g_mbiasH, *sD = g_mbiasD, sl = g_biaslm[0];
    int sp = g_mbias_p, ss = g_mbias_slot, sn = g_biaslm_n, sE = gC.n_exp, sk = g_topk;
    float *dev = (float *)malloc(sizeof(float) * (size_t)ns * E);       /* the CPU build's "device" copy */
    g_mbias_u = u; g_mbias_p = prop; g_mbias_slot = ns > 1; g_topk = ns; gC.n_exp = E; g_biaslm[0] = lmul; g_biaslm_n = 1;
    g_mbiasH = b; g_mbiasD = dev;
    mbias_upd(0, cs, ns, E, m);
    g_mbias_u = su; g_mbiasH = sH; g_mbiasD = sD; g_biaslm[0] = sl;
    g_mbias_p = sp; g_mbias_slot = ss; g_biaslm_n = sn; gC.n_exp = sE; g_topk = sk;
    free(dev);
}

/* ---- the table's context gate (cpu_kern.h:573-589) ---- */
void ref_nggate_f(float *h, const float *v, float *k, float *hn, float *g, float *rh, float *rk, int N, int D) { KL(k_nggate_f, N, 128)(h, v, k, hn, g, rh, rk, D); }
void ref_nggate_b(float *dy, const float *v, const float *hn, const float *kn, const float *g, const float *rh, const float *rk, float *dv, float *dk, int N, int D)
{ KL(k_nggate_b, N, 128)(dy, v, hn, kn, g, rh, rk, dv, dk, D); }

/* ---- 4-bit n-gram table update (cpu_kern.h:615-660; ng_build_touched / ng_tbl_step, cudalm.cu:4673-4745) ---- */
int ref_ng_touched(const int *key, int *slot /* ngrp ints, all -1 */, int *tgi, int *cidx, int N, int De, int grp)
{
    int cnt = 0;
    KL(k_ng_claim, 1, 1)(key, slot, tgi, &cnt, N, De, grp);
    KL(k_ng_cidx, 1, 1)(key, slot, cidx, N, De, grp);
    if (cnt) KL(k_ng_unclaim, 1, 1)(slot, tgi, cnt);
    return cnt;
}
void ref_ng_scatter_compact(float *Gc, const int *key, const int *cidx, const float *dbuf, int N, int De, int group, int Nd)
{
    KL(k_ng_scatter_compact, 1, 1)(Gc, key, cidx, dbuf, N, De, group, Nd);
}
void ref_ng_step(float *P, const float *Gc, signed char *d, signed char *r, float *s, signed char *m8, float *m8s,
                 unsigned char *v8, float *v8s, const int *tgi, int Gt, int group, int dmax, float lr, float b1, float b2,
                 float wd, float sref, float inv_bc1, float inv_sqrt_bc2, unsigned long long t, unsigned long long nt,
                 const float *gs)
{
    if (Gt) KL(k_ng_q4_step, (unsigned)Gt, group, group)(P, Gc, d, r, s, m8, m8s, v8, v8s, tgi, group, dmax, lr, b1, b2, wd, sref,
                                                         inv_bc1, inv_sqrt_bc2, t, nt, gs);
}

/* ---- sparse engram: the sub-tables' primes and multipliers as engram_setup derives them (cudalm.cu:5040-5047), keys,
 * gather and the compact scatter (cpu_kern.h:665-688) ---- */
void ref_eg_tables(int Rraw, int S, const int *ord_of_sub, int *prime, unsigned long long *mult)
{
    int p = Rraw + 1;
    for (int s = 0; s < S; s++) {
        do p--; while (p > 1 && !eg_isprime(p));
        prime[s] = p;
        for (int k = 0; k < 4; k++) mult[s * 4 + k] = splitmix64(0x5EED0E17A11ULL + (unsigned long long)(s * 4 + k)) | 1ULL;
    }
    cudaMemcpyToSymbol(c_eg_ord, ord_of_sub, (size_t)S * 4);
    cudaMemcpyToSymbol(c_eg_prime, prime, (size_t)S * 4);
    cudaMemcpyToSymbol(c_eg_mult, mult, (size_t)S * 32);
}
void ref_eg_key(const int *tok, const unsigned short *cn, int *key, int N, int T, int S, int Rp) { KL(k_eg_key, 1, 1)(tok, cn, key, N, T, S, Rp); }
void ref_eg_gather(const float *tbl, const int *key, float *buf, int N, int S, int De) { KL(k_eg_gather, 1, 1)(tbl, key, buf, N, S, De); }
void ref_eg_scatter_c(float *Gc, const int *key, const int *cidx, const float *db, int N, int S, int De, int grp)
{ KL(k_eg_scatter_c, 1, 1)(Gc, key, cidx, db, N, S, De, grp); }

/* ---- exact 4-bit export of a rendered parameter vector and its reader (quantize_params / dequantize_params with
 * qtype 3, cudalm.cu:639-656, 688-695) ---- */
unsigned long long ref_q4n_export(const float *P, unsigned long long n, int group, unsigned char *out, unsigned long long cap)
{
    size_t len = 0;
    uint8_t *q = quantize_params(P, (size_t)n, 3, group, &len);
    if (len <= cap) memcpy(out, q, len);
    free(q);
    return (unsigned long long)len;
}

int ref_q4n_decode(const unsigned char *in, unsigned long long len, float *P, unsigned long long n, int group)
{
    Rd r = {in, in + len};
    return dequantize_params(&r, P, (size_t)n, 3, group);
}

/* ---- model file (model_save_bundle / model_load_full, cudalm.cu:554-565, 431-466) ---- */
static void cfg_from_ints(Cfg *c, const int *h) { cfg_from_hdr(c, h, h[11] > 0 ? 5 : 4); }
unsigned long long ref_param_count(const int *hdr13) { Cfg c; cfg_from_ints(&c, hdr13); return (unsigned long long)param_count(&c); }
void ref_model_save(const char *path, const int *hdr13, const float *P, unsigned long long n)
{
    Cfg c; cfg_from_ints(&c, hdr13);
    model_save_bundle(path, &c, P, (size_t)n, NULL, 0);
}
/* returns the parameter count, fills hdr13 and P (capacity cap floats) */
unsigned long long ref_model_load(const char *path, int *hdr13, float *P, unsigned long long cap)
{
    Cfg c; Tok *tk = NULL;
    float *Ph = model_load_full(path, &c, &tk);
    size_t n = param_count(&c);
    int h[13] = {c.V, c.D, c.L, c.H, c.KV, c.F, c.T, c.eot, c.tmpl, c.n_mtp, c.n_exp, c.win, c.full_every};
    memcpy(hdr13, h, sizeof h);
    if (n <= cap) memcpy(P, Ph, n * 4);
    free(Ph);
    return (unsigned long long)n;
}

/* ---- router and permutation (cudalm.cu:2515-2534, 3576-3602) ---- */
void ref_router_topk(const float *rt, float *rprobs, int *assign, float *gate, int N, int E, int K,
                     const float *bias, int bs)
{
    KL(k_router_topk, nblk(N, TPB), TPB)(rt, rprobs, assign, gate, N, E, K, bias, bs);
}

/* ---- fp32 GEMM wrappers on a rendered weight view (cudalm.cu:3133-3202) ---- */
static void gemm_flags_off(void)
{
    g_fp8gemm = g_fp16 = g_fp16gemm = g_h16 = g_lane = g_fwd_tc = g_dq_tc = g_dkv_tc = 0;
    g_moef8 = g_tiled = g_sub = g_moe_sb = 0;
}
void ref_g_ab(const float *A, const float *B, float *C, int M, int K, int N)
{ gemm_flags_off(); g_ab(A, B, C, M, K, N); }
void ref_g_abt(const float *A, const float *B, float *C, int M, int K, int N)
{ gemm_flags_off(); g_abt(A, B, C, M, K, N); }
void ref_g_abt_b(const float *A, const float *B, float *C, int M, int K, int N, float beta)
{ gemm_flags_off(); g_abt_b(A, B, C, M, K, N, beta); }
void ref_g_atb(const float *A, const float *B, float *C, int M, int K, int N)
{ gemm_flags_off(); g_atb(A, B, C, M, K, N); }

/* ---- one MoE layer through moe_forward / moe_backward (cudalm.cu:4151-4393) ---- */
struct RefMoe {
    GA *a; float *P, *G, *out; Off o; size_t np; int N, D, F, E, K;
};

void *ref_moe_new(int N, int D, int F, int E, int K, float aux)
{
    gemm_flags_off();
    memset(&gC, 0, sizeof gC);
    gC.V = 8; gC.D = D; gC.L = 1; gC.F = F; gC.T = N; gC.n_exp = E; gC.rope_base = 10000.0f;
    gC.H = (D % 64 == 0) ? D / 64 : 1; gC.KV = gC.H;
    cfg_derive(&gC);
    g_topk = K; g_mbias_u = 0.0f; g_moe_aux = aux; g_moe_stash = 1; g_moe_train = 0;
    g_prof = 0; g_qlm_on = 0;
    RefMoe *h = (RefMoe *)calloc(1, sizeof(RefMoe));
    h->N = N; h->D = D; h->F = F; h->E = E; h->K = K;
    h->np = calc_offsets(&gC, &h->o);
    h->P = (float *)calloc(h->np, 4);
    h->G = (float *)calloc(h->np, 4);
    h->out = (float *)calloc((size_t)N * D, 4);
    h->a = ga_new(N, 1);
    h->a->tr = 1;
    return h;
}
/* pointer to a named buffer of the layer (host memory in the CPU build) */
void *ref_moe_buf(void *hv, const char *name)
{
    RefMoe *h = (RefMoe *)hv; GA *a = h->a;
    if (!strcmp(name, "P")) return h->P;
    if (!strcmp(name, "G")) return h->G;
    if (!strcmp(name, "out")) return h->out;
    if (!strcmp(name, "f_in")) return a->f_in[0];
    if (!strcmp(name, "f_norm")) return a->f_norm[0];
    if (!strcmp(name, "dout")) return a->dout;
    if (!strcmp(name, "dfnorm")) return a->dfnorm;
    if (!strcmp(name, "rt")) return a->rt;
    if (!strcmp(name, "rprobs")) return a->rprobs[0];
    if (!strcmp(name, "assign")) return a->assign[0];
    if (!strcmp(name, "gate")) return a->gate[0];
    if (!strcmp(name, "perm")) return a->perm[0];
    if (!strcmp(name, "hoff")) return a->hoff;
    if (!strcmp(name, "d_gate")) return a->d_gate;
    if (!strcmp(name, "gpS")) return a->gpS[0];
    if (!strcmp(name, "upS")) return a->upS[0];
    if (!strcmp(name, "ypS")) return a->ypS[0];
    return NULL;
}
/* element offset of a weight block inside P / G */
long long ref_moe_off(void *hv, const char *name)
{
    RefMoe *h = (RefMoe *)hv;
    if (!strcmp(name, "wr")) return (long long)h->o.wr[0];
    if (!strcmp(name, "w1")) return (long long)h->o.w1[0];
    if (!strcmp(name, "w3")) return (long long)h->o.w3[0];
    if (!strcmp(name, "w2")) return (long long)h->o.w2[0];
    if (!strcmp(name, "np")) return (long long)h->np;
    return -1;
}
void ref_moe_forward(void *hv)
{
    RefMoe *h = (RefMoe *)hv;
    moe_forward(h->P, &h->o, h->a, 0, h->out, h->N);
}
void ref_moe_backward(void *hv)
{
    RefMoe *h = (RefMoe *)hv;
    memset(h->G, 0, h->np * 4);
    moe_backward(h->P, h->G, &h->o, h->a, 0, h->N);
}

/* ---- the whole training step: gpu_forward (cudalm.cu:5736-5787), gpu_loss (8834-8847), gpu_head_bwd + gpu_backward
 * (5799-6002), gpu_adam with QLM on (6438-6465 -> qlm_gpu_update 6082-6103), set up the way cmd_train does it
 * (qlm_gpu_init, g_qlm_on = 1, g_muon = 0; 8223-8226, 8301).  One model at a time: the reference keeps the
 * configuration, the rope tables and the Qlm in file-scope globals. ---- */
struct RefModel {
    Cfg c; Off o; size_t np; int N; float *P, *G; GA *a; int *tok, *tgt; int qlm;
};
void *ref_model_new(int V, int D, int L, int H, int KV, int F, int T, int E, int K, int B, float aux)
{
    gemm_flags_off();
    memset(&gC, 0, sizeof gC);
    gC.V = V; gC.D = D; gC.L = L; gC.H = H; gC.KV = KV; gC.F = F; gC.T = T; gC.n_exp = E; gC.rope_base = 10000.0f;
    cfg_derive(&gC);
    g_topk = K; g_mbias_u = 0.0f; g_moe_aux = aux; g_moe_stash = 1; g_moe_train = 0; g_prof = 0;
    g_qlm_on = 0; g_muon = 0; g_fused = 0; g_pscratch = 0; g_nkeep = 0; g_loss_denom = 0;
    RefModel *h = (RefModel *)calloc(1, sizeof(RefModel));
    h->c = gC; h->N = B * T;
    h->np = calc_offsets(&gC, &h->o);
    h->P = (float *)calloc(h->np, 4);
    h->G = (float *)calloc(h->np, 4);
    h->tok = (int *)calloc(h->N, 4); h->tgt = (int *)calloc(h->N, 4);
    rope_tables(&gC);
    h->a = ga_new(h->N, 1);
    h->a->tr = 1;
    return h;
}
unsigned long long ref_model_np(void *hv) { return (unsigned long long)((RefModel *)hv)->np; }
/* named buffers: the parameter and gradient vectors, the Qlm's state arrays, activations of layer l */
void *ref_model_buf(void *hv, const char *name, int l)
{
    RefModel *h = (RefModel *)hv; GA *a = h->a;
    if (!strcmp(name, "P")) return h->P;
    if (!strcmp(name, "G")) return h->G;
    if (!strcmp(name, "fn")) return a->fn;
    if (!strcmp(name, "x_final")) return a->x_final;
    if (!strcmp(name, "lossb")) return a->lossb;
    if (!strcmp(name, "a_in")) return a->a_in[l];
    if (!strcmp(name, "f_in")) return a->f_in[l];
    if (!strcmp(name, "f_norm")) return a->f_norm[l];
    if (!strcmp(name, "att")) return a->att[l];
    if (!strcmp(name, "assign")) return a->assign[l];
    if (!strcmp(name, "gate")) return a->gate[l];
    if (!strcmp(name, "rprobs")) return a->rprobs[l];
    if (!strcmp(name, "q.d")) return QQ.d;
    if (!strcmp(name, "q.r")) return QQ.r;
    if (!strcmp(name, "q.s")) return QQ.s;
    if (!strcmp(name, "q.m8")) return QQ.m8;
    if (!strcmp(name, "q.v8")) return QQ.v8;
    if (!strcmp(name, "q.m8s")) return QQ.m8s;
    if (!strcmp(name, "q.v8s")) return QQ.v8s;
    if (!strcmp(name, "q.span")) return QQ.spanH;
    if (!strcmp(name, "q.Mc")) return QQ.Mc;
    if (!strcmp(name, "q.Vc")) return QQ.Vc;
    return NULL;
}
/* nq, ngrp, nspan, nfloat of the Qlm that ref_model_qlm_init built */
void ref_model_qlm_dims(unsigned long long *out4)
{
    out4[0] = QQ.nq; out4[1] = QQ.ngrp; out4[2] = (unsigned long long)QQ.nspan; out4[3] = QQ.nfloat;
}
/* cmd_train with CUDALM_QLM=1: quantise P in place (P becomes the rendered view s*d) */
void ref_model_qlm_init(void *hv)
{
    RefModel *h = (RefModel *)hv;
    gC = h->c;
    qlm_gpu_init(&QQ, &h->c, &h->o, h->P, h->np);
    g_qlm_on = 1; g_muon = 0; h->qlm = 1;
}
void ref_model_forward(void *hv, const int *tok)
{
    RefModel *h = (RefModel *)hv;
    gC = h->c;
    memcpy(h->tok, tok, (size_t)h->N * 4);
    gpu_forward(h->P, &h->o, h->a, h->tok);
}
/* mean cross-entropy of the last forward (gpu_loss; perpos = N floats or NULL) */
double ref_model_loss(void *hv, const int *tgt, float *perpos)
{
    RefModel *h = (RefModel *)hv;
    memcpy(h->tgt, tgt, (size_t)h->N * 4);
    return gpu_loss(h->P, &h->o, h->a, h->tgt, h->N, perpos);
}
/* gpu_backward after ref_model_forward on the same tokens; returns the mean of the per-row losses the head wrote */
double ref_model_backward(void *hv, const int *tgt)
{
    RefModel *h = (RefModel *)hv;
    memcpy(h->tgt, tgt, (size_t)h->N * 4);
    gpu_backward(h->P, h->G, &h->o, h->a, h->tok, h->tgt);
    double s = 0; for (int i = 0; i < h->N; i++) s += h->a->lossb[i];
    return s / h->N;
}
/* gpu_adam; returns its own return value (0 = step skipped on a non-finite norm); gn = the norm it read back */
int ref_model_adam(void *hv, float lr, int t, float *gn)
{
    RefModel *h = (RefModel *)hv;
    int ok = gpu_adam(h->P, h->G, NULL, NULL, h->np, lr, t);
    if (gn) *gn = g_gn;
    return ok;
}

/* ---- QLMH optimizer-state file (qlm.cuh:703-788), on caller-owned host arrays ---- */
static void fill_qlm(Qlm *q, int dmax, int group, int adam, int packed, QSpanD *spans, int nspan,
                     unsigned long long nq, unsigned long long ngrp, unsigned long long nfloat,
                     signed char *d, signed char *r, signed char *m8, unsigned char *v8, float *s,
                     float *m8s, float *v8s, unsigned short *Mc, unsigned short *Vc)
{
    memset(q, 0, sizeof *q);
    q->dmax = dmax; q->group = group; q->adam = adam; q->packed = packed;
    q->nspan = nspan; q->spanH = spans; q->spanD = spans;
    q->nq = nq; q->ngrp = ngrp; q->nfloat = nfloat;
    q->d = d; q->r = r; q->m8 = m8; q->v8 = v8; q->s = s; q->m8s = m8s; q->v8s = v8s;
    q->Mc = (bf16 *)Mc; q->Vc = (bf16 *)Vc;
}
int ref_qlm_save(const char *path, int iter, float prev_gn, int dmax, int group, int adam, int packed,
                 QSpanD *spans, int nspan, unsigned long long nq, unsigned long long ngrp,
                 unsigned long long nfloat, signed char *d, signed char *r, signed char *m8,
                 unsigned char *v8, float *s, float *m8s, float *v8s, unsigned short *Mc, unsigned short *Vc)
{
    Qlm q;
    fill_qlm(&q, dmax, group, adam, packed, spans, nspan, nq, ngrp, nfloat, d, r, m8, v8, s, m8s, v8s, Mc, Vc);
    g_prev_gn = prev_gn;
    return qlm_save(&q, path, iter);
}
int ref_qlm_load(const char *path, int *iter, float *prev_gn, int dmax, int group, int adam, int packed,
                 QSpanD *spans, int nspan, unsigned long long nq, unsigned long long ngrp,
                 unsigned long long nfloat, signed char *d, signed char *r, signed char *m8,
                 unsigned char *v8, float *s, float *m8s, float *v8s, unsigned short *Mc, unsigned short *Vc)
{
    Qlm q;
    fill_qlm(&q, dmax, group, adam, packed, spans, nspan, nq, ngrp, nfloat, d, r, m8, v8, s, m8s, v8s, Mc, Vc);
    g_prev_gn = 0.0f;
    int ok = qlm_load(&q, path, iter);
    if (prev_gn) *prev_gn = g_prev_gn;
    return ok;
}

} /* extern "C" */
