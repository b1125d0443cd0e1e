/* qlm_oracle.c -- CPU restatement of the QLM hot path of Dsg2/cudalm-c.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against; nothing in the shipped library links, loads or calls it.
 * It is a from-scratch restatement (plain C99, one group / one token at a
 * time) of the arithmetic the reference performs; every function names the
 * reference lines it follows.  It is pinned two ways: against the known-answer
 * vectors under tests/golden/ (produced by running the reference's own CPU
 * build) and, when the compiled reference is available, against
 * oracle/_ref/libcudalm_ref_exact.so on random inputs.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off is part of the contract: the reference's integer state is
 * only reproducible when a*b+c is NOT fused (the reference's own no-FMA build
 * flavour, build.py --cpu-arch x86-64-v2, gives the same bytes).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Same memory layout as the reference's QSpanD (qlm.cuh:30-38). */
typedef struct {
    uint64_t pof, gof, qi0, n;
    int32_t gi0, ngrp;
    float sref;
} QoSpan;

/* ------------------------------------------------------------------ hash */

/* splitmix64 finaliser, low 32 bits (qlm.cuh:78-82). */
uint32_t qo_hash(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return (uint32_t)(x ^ (x >> 31));
}

/* Stochastic rounding keyed on (element, step): floor(v) plus one when a
 * 24-bit uniform draw falls below the fractional part (qlm.cuh:83-87). */
int qo_sround(float v, uint64_t i, uint64_t t)
{
    float fl = floorf(v);
    uint32_t h = qo_hash(i * 0x2545F4914F6CDD1DULL + t * 0x9E3779B97F4A7C15ULL);
    float u = (float)(h >> 8) * (1.0f / 16777216.0f);
    return (int)fl + (u < (v - fl) ? 1 : 0);
}

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* ---------------------------------------------------------------- digits */

/* Digit i of a digit array: packed = two's-complement nibbles, even index in
 * the low half of byte i/2 (qlm.cuh:96-101). */
int qo_digit(const int8_t *d, uint64_t i, int packed)
{
    if (!packed) return d[i];
    unsigned b = (uint8_t)d[i >> 1];
    int v = (i & 1) ? (int)(b >> 4) : (int)(b & 15u);
    return v > 7 ? v - 16 : v;
}

/* Store the n digits of one group; an odd tail leaves the high nibble zero
 * (qlm.cuh:123-132). */
static void put_digits(int8_t *d, uint64_t q0, const int *dig, int n, int packed)
{
    if (!packed) {
        for (int j = 0; j < n; j++) d[q0 + j] = (int8_t)dig[j];
        return;
    }
    for (int b = 0; 2 * b < n; b++) {
        int lo = dig[2 * b] & 15;
        int hi = (2 * b + 1 < n) ? (dig[2 * b + 1] & 15) : 0;
        d[(q0 >> 1) + b] = (int8_t)((hi << 4) | lo);
    }
}

/* Which span owns group gi, where the group starts inside it and how many
 * elements it has (qlm.cuh:113-117, cpu_kern.h:773-776). */
static const QoSpan *locate(const QoSpan *sp, int nspan, int gi, int group,
                            uint64_t *j0, int *n)
{
    const QoSpan *hit = &sp[0];
    for (int i = 0; i < nspan; i++)
        if (gi >= sp[i].gi0 && gi < sp[i].gi0 + sp[i].ngrp) { hit = &sp[i]; break; }
    *j0 = (uint64_t)(gi - hit->gi0) * (uint64_t)group;
    uint64_t left = hit->n - *j0;
    *n = (int)(left < (uint64_t)group ? left : (uint64_t)group);
    return hit;
}

/* ---------------------------------------------------------------- encode */

/* Quantise fp32 weights into (digit, residual, scale) per group: scale =
 * absmax/dmax floored at 1e-8, digit = nearest integer clamped to +-dmax,
 * residual = nearest 1/128th of the remainder clamped to +-64
 * (qlm.cuh:136-167, cpu_kern.h:777-789). */
void qo_encode(const float *P, int8_t *d, int8_t *r, float *s, const QoSpan *sp,
               int nspan, int ngrp, int group, int dmax, int packed)
{
#pragma omp parallel for schedule(static)
    for (int gi = 0; gi < ngrp; gi++) {
        uint64_t j0; int n;
        const QoSpan *o = locate(sp, nspan, gi, group, &j0, &n);
        const float *p = P + o->pof + j0;
        uint64_t q0 = o->qi0 + j0;
        float amax = 0.0f;
        for (int j = 0; j < n; j++) amax = fmaxf(amax, fabsf(p[j]));
        float sc = amax / (float)dmax;
        if (!(sc > 0.0f)) sc = 1e-8f;
        s[gi] = sc;
        int dig[256];
        for (int j = 0; j < n; j++) {
            float t = p[j] / sc;
            int dd = clampi((int)rintf(t), -dmax, dmax);
            int rr = clampi((int)rintf((t - (float)dd) * 128.0f), -64, 64);
            dig[j] = dd;
            r[q0 + j] = (int8_t)rr;
        }
        put_digits(d, q0, dig, n, packed);
    }
}

/* ---------------------------------------------------------------- render */

/* fp32 view P = scale * digit for groups [gi_base, gi_base+ng)
 * (qlm.cuh:170-178, cpu_kern.h:790-796). */
void qo_render(float *P, const int8_t *d, const float *s, const QoSpan *sp,
               int nspan, int group, int packed, int gi_base, int ng)
{
#pragma omp parallel for schedule(static)
    for (int w = 0; w < ng; w++) {
        int gi = gi_base + w, n; uint64_t j0;
        const QoSpan *o = locate(sp, nspan, gi, group, &j0, &n);
        for (int j = 0; j < n; j++)
            P[o->pof + j0 + j] = s[gi] * (float)qo_digit(d, o->qi0 + j0 + j, packed);
    }
}

/* ------------------------------------------------------- integer AdamW step */

/* One optimiser step over groups [gi_base, gi_base+ng).  Per element, in this
 * exact fp32 operation order (qlm.cuh:199-277, cpu_kern.h:798-826):
 *   gr = G*gs;  m = b1*(m8*ms) + (1-b1)*gr;  v = b2*(v8*vs)^2 + (1-b2)*gr*gr;
 *   rv = sqrt(v);  u = clamp((m*inv_bc1)/(rv*inv_sqrt_bc2 + max(vs,1e-8)), +-8)
 *   idl = sround(-(L*u + dec*digit), qi, t);  rr = residual + idl
 *   carry c = the unique integer with rr-128c in [-64,64]  (rr==64 stays)
 *   digit = clamp(digit + c, +-dmax);  residual = rr - 128c
 * then the group's new moment scales ms = max|m|/127, vs = max rv/255 (1e-12
 * when the max is 0) and the re-quantised moments
 *   m8 = clamp(sround(m/ms, qi, t+0x5EED), +-127)
 *   v8 = clamp(sround(rv/vs, qi, t+0xBEEF), 0, 255), kept >= 1 while rv > 0.
 * adam==0 is the sign-momentum variant (qlm.cuh:225-229).  P may be NULL
 * (no fp32 view wanted); stat may be NULL (qlm.cuh:243-250). */
/* QLM_V4 (qlm.cuh:62-72): v8 holds v^(1/4); process-wide switch like the reference's d_qv4 */
static int qo_v4 = 0;
void qo_set_v4(int on) { qo_v4 = on ? 1 : 0; }

void qo_step(float *P, const float *G, int8_t *d, int8_t *r, const float *s,
             int8_t *m8, float *m8s, uint8_t *v8, float *v8s, const QoSpan *sp,
             int nspan, int group, int dmax, float lr, float b1, float b2, float wd,
             float gs, float inv_bc1, float inv_sqrt_bc2, int lrmode, uint64_t t,
             int adam, int64_t *stat, int packed, int gi_base, int ng)
{
    int64_t st0 = 0, st1 = 0, st2 = 0, st3 = 0;
#pragma omp parallel for schedule(static) reduction(+ : st0, st1, st2) reduction(max : st3)
    for (int w = 0; w < ng; w++) {
        int gi = gi_base + w, n; uint64_t j0;
        const QoSpan *o = locate(sp, nspan, gi, group, &j0, &n);
        uint64_t q0 = o->qi0 + j0;
        const float *g = G + o->gof + j0;
        float sc = s[gi];
        float L = lr * 128.0f / (lrmode ? sc : o->sref);
        float dec = lr * wd * 128.0f;
        float ms_old = m8s[gi], vs_old = v8s ? v8s[gi] : 0.0f;
        float mnew[256], rnew[256], amax = 0.0f, vmax = 0.0f;
        int dig[256];
        for (int j = 0; j < n; j++) {
            uint64_t qi = q0 + j;
            float gr = g[j] * gs;
            float mv = (float)m8[qi] * ms_old;
            float u;
            rnew[j] = 0.0f;
            if (adam) {
                float sv = (float)v8[qi] * vs_old;
                if (qo_v4) sv = sv * sv;                 /* qv_dec, qlm.cuh:66 */
                float vv = sv * sv;
                mnew[j] = b1 * mv + (1.0f - b1) * gr;
                vv = b2 * vv + (1.0f - b2) * gr * gr;
                rnew[j] = sqrtf(vv);
                float veps = fmaxf(qo_v4 ? vs_old * vs_old : vs_old, 1e-8f);
                u = (mnew[j] * inv_bc1) / (rnew[j] * inv_sqrt_bc2 + veps);
                u = fmaxf(-8.0f, fminf(8.0f, u));
                if (qo_v4) rnew[j] = sqrtf(rnew[j]);     /* qv_enc, qlm.cuh:67 */
            } else {
                float cc = b1 * mv + (1.0f - b1) * gr;
                u = (float)((cc > 0.0f) - (cc < 0.0f));
                mnew[j] = b2 * mv + (1.0f - b2) * gr;
            }
            int dd = qo_digit(d, qi, packed);
            int idl = qo_sround(-(L * u + dec * (float)dd), qi, t);
            int rr = (int)r[qi] + idl;
            int c = 0;
            if (rr > 64) c = ((rr - 65) >> 7) + 1;
            else if (rr < -64) c = -((((-rr) - 65) >> 7) + 1);
            rr -= 128 * c;
            dd = clampi(dd + c, -dmax, dmax);
            dig[j] = dd;
            r[qi] = (int8_t)rr;
            if (P) P[o->pof + j0 + j] = sc * (float)dd;
            if (stat) {
                int ai = idl < 0 ? -idl : idl;
                if (ai > st3) st3 = ai;
                st0 += c < 0 ? -c : c;
                st1 += (dd == dmax) | (dd == -dmax);
                st2 += (dd == 0);
            }
            amax = fmaxf(amax, fabsf(mnew[j]));
            vmax = fmaxf(vmax, rnew[j]);
        }
        put_digits(d, q0, dig, n, packed);
        float ms = amax > 0.0f ? amax / 127.0f : 1e-12f;
        float vs = vmax > 0.0f ? vmax / 255.0f : 1e-12f;
        m8s[gi] = ms;
        if (adam) v8s[gi] = vs;
        for (int j = 0; j < n; j++) {
            uint64_t qi = q0 + j;
            m8[qi] = (int8_t)clampi(qo_sround(mnew[j] / ms, qi, t + 0x5EEDULL), -127, 127);
            if (adam) {
                int vq = clampi(qo_sround(rnew[j] / vs, qi, t + 0xBEEFULL), 0, 255);
                if (vq == 0 && rnew[j] > 0.0f) vq = 1;
                v8[qi] = (uint8_t)vq;
            }
        }
    }
    if (stat) {
        stat[0] += st0; stat[1] += st1; stat[2] += st2;
        if (st3 > stat[3]) stat[3] = st3;
    }
}

/* ----------------------------------------------------------------- servo */

/* Scale servo: a group whose fraction of railed digits (|digit| == dmax)
 * leaves [f_lo, f_hi] has its scale multiplied / divided by 1.09051 and its
 * digit+residual pair re-derived at the new scale (qlm.cuh:404-441,
 * cpu_kern.h:857-873). */
void qo_servo(int8_t *d, int8_t *r, float *s, const QoSpan *sp, int nspan, int ngrp,
              int group, int dmax, float f_hi, float f_lo, int packed)
{
#pragma omp parallel for schedule(static)
    for (int gi = 0; gi < ngrp; gi++) {
        uint64_t j0; int n;
        const QoSpan *o = locate(sp, nspan, gi, group, &j0, &n);
        uint64_t q0 = o->qi0 + j0;
        int railed = 0;
        for (int j = 0; j < n; j++) {
            int dd = qo_digit(d, q0 + j, packed);
            railed += (dd == dmax) | (dd == -dmax);
        }
        float f = (float)railed / (float)n, old = s[gi], nw;
        if (f > f_hi) nw = old * 1.09051f;
        else if (f < f_lo) nw = old / 1.09051f;
        else continue;
        float conv = old / nw;
        s[gi] = nw;
        int dig[256];
        for (int j = 0; j < n; j++) {
            uint64_t qi = q0 + j;
            float t = ((float)qo_digit(d, qi, packed) + (float)r[qi] * (1.0f / 128.0f)) * conv;
            int dd = clampi((int)rintf(t), -dmax, dmax);
            int rr = clampi((int)rintf((t - (float)dd) * 128.0f), -64, 64);
            dig[j] = dd;
            r[qi] = (int8_t)rr;
        }
        put_digits(d, q0, dig, n, packed);
    }
}

/* ------------------------------------------------------------- grad norm */

/* Global-norm clip multiplier.  The gradient is cut into 64 contiguous chunks
 * [n*c/64, n*(c+1)/64); each chunk's sum of squares is accumulated in double
 * and stored as float; the 64 floats are summed in double; gn = (float)sqrt.
 * Side buffers get 64 partials each: they join the norm when clip_side is set
 * and a non-finite side sum poisons gn either way.  gs[0] = gn>1 ? 1/gn : 1,
 * gs[1] = gn (cpu_kern.h:533-546; cudalm.cu:2807-2812, 6442-6444). */
static void sq_partials(const float *G, size_t n, float *part)
{
#pragma omp parallel for schedule(static)
    for (int c = 0; c < 64; c++) {
        size_t i0 = n * (size_t)c / 64, i1 = n * (size_t)(c + 1) / 64;
        double acc = 0.0;
        for (size_t i = i0; i < i1; i++) acc += (double)G[i] * (double)G[i];
        part[c] = (float)acc;
    }
}

/* the 64 partials of one buffer, as the fused per-layer update keeps them per layer
 * (qlm_fused_layer, cudalm.cu:6122; k_sqsum, cpu_kern.h:533-540) */
void qo_sqsum(const float *G, size_t n, float *part64) { sq_partials(G, n, part64); }

void qo_gnorm(const float *G, size_t n, const float *const *side, const size_t *side_n,
              int nside, int clip_side, float *gs)
{
    float *part = (float *)malloc(sizeof(float) * 64 * (size_t)(1 + nside));
    sq_partials(G, n, part);
    for (int k = 0; k < nside; k++) sq_partials(side[k], side_n[k], part + 64 * (k + 1));
    double ss = 0.0, sd = 0.0;
    for (int i = 0; i < 64; i++) ss += part[i];
    for (int i = 64; i < 64 * (1 + nside); i++) sd += part[i];
    float gn = (float)sqrt(clip_side ? ss + sd : ss);
    if (!isfinite(sd)) gn = NAN;
    gs[0] = gn > 1.0f ? 1.0f / gn : 1.0f;
    gs[1] = gn;
    free(part);
}

/* ------------------------------------------------ float-span AdamW (bf16 m,v) */

static float bf2f(uint16_t h) { uint32_t x = (uint32_t)h << 16; float f; memcpy(&f, &x, 4); return f; }
static uint16_t f2bf(float f)
{
    uint32_t x; memcpy(&x, &f, 4);
    return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}

/* AdamW for the unquantised spans, moments stored as bf16 (round to nearest
 * even), eps 1e-8, decoupled decay (cpu_kern.h:552-561; cudalm.cu:2855-2870). */
void qo_adamw(float *P, const float *G, uint16_t *M, uint16_t *V, size_t n, float lr,
              float b1, float b2, float wd, float bc1, float bc2, const float *gs)
{
#pragma omp parallel for schedule(static)
    for (long j = 0; j < (long)n; j++) {
        float g = gs ? G[j] * gs[0] : G[j];
        float m = b1 * bf2f(M[j]) + (1.0f - b1) * g;
        float v = b2 * bf2f(V[j]) + (1.0f - b2) * g * g;
        M[j] = f2bf(m);
        V[j] = f2bf(v);
        P[j] -= lr * ((m / bc1) / (sqrtf(v / bc2) + 1e-8f) + wd * P[j]);
    }
}

/* ---------------------------------------------------------------- router */

/* The reference CPU build's exp: clamp, Cody-Waite range reduction with a
 * two-part ln2, degree-6 Taylor polynomial, exponent rebuilt by bit shift
 * (cpu_kern.h:28-34). */
float qo_fexp(float x)
{
    if (x < -87.0f) x = -87.0f;
    if (x > 88.0f) x = 88.0f;
    float k = rintf(x * 1.44269504089f);
    float r = x - k * 0.693145751953125f;
    r -= k * 1.428606765330187e-06f;
    float p = 1.0f / 720;
    p = 1.0f / 120 + r * p;
    p = 1.0f / 24 + r * p;
    p = 1.0f / 6 + r * p;
    p = 0.5f + r * p;
    p = 1.0f + r * p;
    p = 1.0f + r * p;
    uint32_t bits = (uint32_t)((int)k + 127) << 23;
    float sc; memcpy(&sc, &bits, 4);
    return p * sc;
}

/* Softmax over E logits per token, then K rounds of "highest prob+bias among
 * the experts not yet taken", first index winning ties; a round that finds
 * nothing (NaN scores) falls back to expert k.  Outputs are pass-major:
 * assign[k*N+n], gate[k*N+n] = the raw softmax probability
 * (cpu_kern.h:413-425; cudalm.cu:2515-2534). */
void qo_router_topk(const float *rt, float *rprobs, int *assign, float *gate, int N, int E,
                    int K, const float *bias, int bs)
{
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const float *lg = rt + (size_t)n * E;
        float *pr = rprobs + (size_t)n * E;
        float top = -1e30f;
        for (int e = 0; e < E; e++) if (lg[e] > top) top = lg[e];
        float sum = 0.0f;
        for (int e = 0; e < E; e++) { pr[e] = qo_fexp(lg[e] - top); sum += pr[e]; }
        float inv = 1.0f / sum;
        for (int e = 0; e < E; e++) pr[e] *= inv;
        int took[8];
        for (int k = 0; k < K; k++) {
            int pick = -1; float best = -1e30f;
            for (int e = 0; e < E; e++) {
                int used = 0;
                for (int j = 0; j < k; j++) used |= (took[j] == e);
                if (used) continue;
                float sc = pr[e] + (bias ? bias[k * bs + e] : 0.0f);
                if (sc > best) { best = sc; pick = e; }
            }
            if (pick < 0) pick = k;
            took[k] = pick;
            assign[(size_t)k * N + n] = pick;
            gate[(size_t)k * N + n] = pr[pick];
        }
    }
}

/* ------------------------------------------------------------ permutation */

/* Stable counting sort of token slots by expert.
 * merged==0: one sort per pass k; off has K*(E+1) entries, perm[k*N + pos] = n
 *            (cudalm.cu:3586-3600 with cap==0).
 * merged==1: one sort over the K*N entries n' = k*N+n; off has E+1 entries and
 *            inv[n'] = pos (cudalm.cu:3532-3552).
 * Returns 0, or 1+the first out-of-range expert index (cudalm.cu:3476-3478). */
int qo_perm_build(const int *assign, int N, int E, int K, int merged, int *perm, int *inv,
                  int *off)
{
    int passes = merged ? 1 : K;
    int len = merged ? K * N : N;
    for (int k = 0; k < passes; k++) {
        const int *a = assign + (size_t)k * len;
        int *o = off + (size_t)k * (E + 1);
        int *p = perm + (size_t)k * len;
        for (int e = 0; e <= E; e++) o[e] = 0;
        for (int i = 0; i < len; i++) {
            if ((unsigned)a[i] >= (unsigned)E) return 1 + a[i];
            o[a[i] + 1]++;
        }
        for (int e = 0; e < E; e++) o[e + 1] += o[e];
        int *cur = (int *)malloc(sizeof(int) * (size_t)E);
        for (int e = 0; e < E; e++) cur[e] = o[e];
        for (int i = 0; i < len; i++) {
            int pos = cur[a[i]]++;
            p[pos] = i;
            if (inv) inv[(size_t)k * len + i] = pos;
        }
        free(cur);
    }
    return 0;
}

/* ----------------------------------------------------- quantised linears */

/* W is the rendered view s*d of a row-major [rows, cols] code matrix whose
 * 128-element groups run along the flat index.  Accumulation in double: the
 * reference accumulates in fp32 with a blocking of its own, and GEMM parity is
 * a tolerance, not bit equality (cudalm.cu:3133-3202). */
static float wval(const int8_t *d, const float *s, size_t idx, int group)
{
    return s[idx / (size_t)group] * (float)qo_digit(d, idx, 1);
}

/* layout 0 ("KN", the reference's g_ab): W is [K,N], Y[M,N] = X[M,K] @ W.
 * layout 1 ("NK", g_abt):                W is [N,K], Y[M,N] = X[M,K] @ W^T. */
void qo_linear_fwd(float *Y, const float *X, const int8_t *d, const float *s, int layout,
                   int M, int K, int N, int group)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        double *acc = (double *)calloc((size_t)N, sizeof(double));
        for (int k = 0; k < K; k++) {
            double x = X[(size_t)m * K + k];
            for (int n = 0; n < N; n++) {
                size_t idx = layout ? (size_t)n * K + k : (size_t)k * N + n;
                acc[n] += x * (double)wval(d, s, idx, group);
            }
        }
        for (int n = 0; n < N; n++) Y[(size_t)m * N + n] = (float)acc[n];
        free(acc);
    }
}

/* dX[M,K] = dY[M,N] @ W^T (layout 0) or dY @ W (layout 1): the input gradient
 * of qo_linear_fwd with the same W (cudalm.cu:3147-3186). */
void qo_linear_dgrad(float *dX, const float *dY, const int8_t *d, const float *s, int layout,
                     int M, int K, int N, int group)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        double *acc = (double *)calloc((size_t)K, sizeof(double));
        for (int n = 0; n < N; n++) {
            double g = dY[(size_t)m * N + n];
            for (int k = 0; k < K; k++) {
                size_t idx = layout ? (size_t)n * K + k : (size_t)k * N + n;
                acc[k] += g * (double)wval(d, s, idx, group);
            }
        }
        for (int k = 0; k < K; k++) dX[(size_t)m * K + k] = (float)acc[k];
        free(acc);
    }
}

/* Weight gradient, accumulated into dW (beta = 1): layout 0 gives
 * dW[K,N] += X^T dY, layout 1 gives dW[N,K] += dY^T X (cudalm.cu:3190-3202). */
void qo_linear_wgrad(float *dW, const float *dY, const float *X, int layout, int M, int K,
                     int N)
{
    int R = layout ? N : K, C = layout ? K : N;
#pragma omp parallel for schedule(static)
    for (int a = 0; a < R; a++)
        for (int b = 0; b < C; b++) {
            double acc = 0.0;
            for (int m = 0; m < M; m++) {
                double x = layout ? X[(size_t)m * K + b] : X[(size_t)m * K + a];
                double g = layout ? dY[(size_t)m * N + a] : dY[(size_t)m * N + b];
                acc += x * g;
            }
            dW[(size_t)a * C + b] += (float)acc;
        }
}

/* ------------------------------------------------------------ MoE layer */

static float sigm(float z) { return 1.0f / (1.0f + expf(-z)); }

/* Expert FFN forward for one MoE layer, token by token
 * (cudalm.cu:4151-4229, the K-pass branch):
 *   rt = fnorm @ Wr;  (assign, gate, rprobs) = router_topk(rt)
 *   out[n] = f_in[n] + sum_k gate[k,n] * (silu(x W1_e) * (x W3_e)) W2_e,  e = assign[k,n]
 * Expert weights are rendered views of 4-bit codes: W1,W3 [E][D][F], W2 [E][F][D].
 * gsave/usave/ysave (each [K*N, .], slot k*N+n) keep the pre-activation and
 * pre-gate values for the backward; any of them may be NULL. */
void qo_moe_fwd(float *out, const float *f_in, const float *fnorm, const float *Wr,
                const int8_t *d1, const float *s1, const int8_t *d3, const float *s3,
                const int8_t *d2, const float *s2, int N, int D, int F, int E, int K,
                float *rt, float *rprobs, int *assign, float *gate, float *gsave,
                float *usave, float *ysave, int group)
{
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++)
        for (int e = 0; e < E; e++) {
            float acc = 0.0f;
            for (int k = 0; k < D; k++) acc += fnorm[(size_t)n * D + k] * Wr[(size_t)k * E + e];
            rt[(size_t)n * E + e] = acc;
        }
    qo_router_topk(rt, rprobs, assign, gate, N, E, K, NULL, 0);
#pragma omp parallel for schedule(dynamic, 8)
    for (int n = 0; n < N; n++) {
        const float *x = fnorm + (size_t)n * D;
        double *gv = (double *)malloc(sizeof(double) * (size_t)(2 * F + D));
        double *uv = gv + F, *yv = uv + F;
        float *act = (float *)malloc(sizeof(float) * (size_t)F);
        for (int j = 0; j < D; j++) out[(size_t)n * D + j] = f_in[(size_t)n * D + j];
        for (int k = 0; k < K; k++) {
            int e = assign[(size_t)k * N + n];
            size_t slot = (size_t)k * N + n, wb = (size_t)e * D * F;
            for (int f = 0; f < F; f++) gv[f] = uv[f] = 0.0;
            for (int j = 0; j < D; j++) {
                double xv = x[j];
                size_t row = wb + (size_t)j * F;
                for (int f = 0; f < F; f++) {
                    gv[f] += xv * (double)wval(d1, s1, row + f, group);
                    uv[f] += xv * (double)wval(d3, s3, row + f, group);
                }
            }
            for (int f = 0; f < F; f++) {
                float z = (float)gv[f], u = (float)uv[f];
                act[f] = z * sigm(z) * u;
                if (gsave) gsave[slot * F + f] = z;
                if (usave) usave[slot * F + f] = u;
            }
            for (int j = 0; j < D; j++) yv[j] = 0.0;
            for (int f = 0; f < F; f++) {
                double a = act[f];
                size_t row = wb + (size_t)f * D;
                for (int j = 0; j < D; j++) yv[j] += a * (double)wval(d2, s2, row + j, group);
            }
            float gt = gate[slot];
            for (int j = 0; j < D; j++) {
                if (ysave) ysave[slot * D + j] = (float)yv[j];
                out[(size_t)n * D + j] += gt * (float)yv[j];
            }
        }
        free(gv); free(act);
    }
}

/* Backward of qo_moe_fwd (cudalm.cu:4278-4391).  Inputs: dout [N,D] and the
 * forward's saved assign/gate/rprobs/gsave/usave/ysave.  Produces
 *   dfnorm [N,D]  (expert path + router path),
 *   dW1,dW3 [E][D][F], dW2 [E][F][D], dWr [D,E]   accumulated (+=),
 *   d_gate [K*N].
 * The load-balance term is w[e] = aux*E*(cnt[e]/(K*N))/N added to every
 * token's probability gradient before the softmax Jacobian. */
void qo_moe_bwd(float *dfnorm, float *dW1, float *dW3, float *dW2, float *dWr, float *d_gate,
                const float *dout, const float *fnorm, const float *Wr, const int8_t *d1,
                const float *s1, const int8_t *d3, const float *s3, const int8_t *d2,
                const float *s2, int N, int D, int F, int E, int K, const float *rprobs,
                const int *assign, const float *gate, const float *gsave, const float *usave,
                const float *ysave, float aux, int group)
{
    memset(dfnorm, 0, sizeof(float) * (size_t)N * D);
    int *cnt = (int *)calloc((size_t)E, sizeof(int));
    for (size_t i = 0; i < (size_t)K * N; i++) cnt[assign[i]]++;
    /* expert path: parallel over experts so weight-gradient rows have one writer */
#pragma omp parallel for schedule(dynamic, 1)
    for (int e = 0; e < E; e++) {
        double *da = (double *)malloc(sizeof(double) * (size_t)(F + D));
        double *dx = da + F;
        float *dg = (float *)malloc(sizeof(float) * (size_t)(3 * F));
        float *du = dg + F, *act = du + F;
        size_t wb = (size_t)e * D * F;
        for (int k = 0; k < K; k++)
            for (int n = 0; n < N; n++) {
                size_t slot = (size_t)k * N + n;
                if (assign[slot] != e) continue;
                const float *x = fnorm + (size_t)n * D, *dro = dout + (size_t)n * D;
                float gt = gate[slot];
                double dot = 0.0;
                for (int j = 0; j < D; j++) dot += (double)dro[j] * (double)ysave[slot * D + j];
                d_gate[slot] = (float)dot;
                for (int f = 0; f < F; f++) {
                    float z = gsave[slot * F + f];
                    act[f] = z * sigm(z) * usave[slot * F + f];
                    da[f] = 0.0;
                }
                for (int f = 0; f < F; f++) {
                    size_t row = wb + (size_t)f * D;
                    double acc = 0.0;
                    for (int j = 0; j < D; j++) {
                        float dy = gt * dro[j];
                        dW2[row + j] += act[f] * dy;
                        acc += (double)dy * (double)wval(d2, s2, row + j, group);
                    }
                    da[f] = acc;
                }
                for (int f = 0; f < F; f++) {
                    float z = gsave[slot * F + f], u = usave[slot * F + f], sg = sigm(z);
                    float silu = z * sg, ds = sg + z * sg * (1.0f - sg);
                    dg[f] = (float)da[f] * u * ds;
                    du[f] = (float)da[f] * silu;
                }
                for (int j = 0; j < D; j++) {
                    size_t row = wb + (size_t)j * F;
                    double acc = 0.0;
                    for (int f = 0; f < F; f++) {
                        dW1[row + f] += x[j] * dg[f];
                        dW3[row + f] += x[j] * du[f];
                        acc += (double)dg[f] * (double)wval(d1, s1, row + f, group)
                             + (double)du[f] * (double)wval(d3, s3, row + f, group);
                    }
                    dx[j] = acc;
                }
#pragma omp critical
                for (int j = 0; j < D; j++) dfnorm[(size_t)n * D + j] += (float)dx[j];
            }
        free(da); free(dg);
    }
    /* router path */
    float *drt = (float *)malloc(sizeof(float) * (size_t)N * E);
    float invN = 1.0f / N, invKN = 1.0f / ((float)K * N);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const float *pr = rprobs + (size_t)n * E;
        float *dr = drt + (size_t)n * E, dot = 0.0f;
        for (int e = 0; e < E; e++) dr[e] = aux * E * ((float)cnt[e] * invKN) * invN;
        for (int k = 0; k < K; k++) dr[assign[(size_t)k * N + n]] += d_gate[(size_t)k * N + n];
        for (int e = 0; e < E; e++) dot += pr[e] * dr[e];
        for (int e = 0; e < E; e++) dr[e] = pr[e] * (dr[e] - dot);
        for (int j = 0; j < D; j++) {
            float acc = 0.0f;
            for (int e = 0; e < E; e++) acc += dr[e] * Wr[(size_t)j * E + e];
            dfnorm[(size_t)n * D + j] += acc;
        }
    }
#pragma omp parallel for schedule(static)
    for (int j = 0; j < D; j++)
        for (int e = 0; e < E; e++) {
            double acc = 0.0;
            for (int n = 0; n < N; n++) acc += (double)fnorm[(size_t)n * D + j] * drt[(size_t)n * E + e];
            dWr[(size_t)j * E + e] += (float)acc;
        }
    free(drt); free(cnt);
}

/* ---- aux-free balancing (mbias_upd, cudalm.cu:3793-3798; call forms at 4385) ----
 * b[ns][E] += u * ((m - c) / m  or  sign(m - c)), c = the count of expert e in row s of cs, all in float. */
void qo_bias_update(float *b, const int *cs, int ns, int E, float m, float u, int prop)
{
    for (int s = 0; s < ns; s++)
        for (int e = 0; e < E; e++) {
            float c = (float)cs[s * E + e];
            float d = prop ? (m - c) / m : (c < m ? 1.0f : c > m ? -1.0f : 0.0f);
            float step = u * d;
            b[s * E + e] = b[s * E + e] + step;
        }
}

/* ---- n-gram context gate (k_nggate_f / k_nggate_b, cudalm.cu:3362-3378; CPU twins cpu_kern.h:573-589) ----
 * Row sums in double (the reference's kernels sum in float in their own orders; the comparison is to 1e-5). */
void qo_nggate_f(float *h, const float *v, float *k, float *hn, float *g, float *rh, float *rk, int N, int D)
{
    for (int r = 0; r < N; r++) {
        size_t o = (size_t)r * D;
        double a = 0, b = 0, c = 0;
        for (int i = 0; i < D; i++) { a += (double)h[o + i] * h[o + i]; b += (double)k[o + i] * k[o + i]; c += (double)h[o + i] * k[o + i]; }
        float r1 = 1.0f / sqrtf((float)a / D + 1e-6f), r2 = 1.0f / sqrtf((float)b / D + 1e-6f);
        float gg = sigm((float)c * r1 * r2 / sqrtf((float)D));
        for (int i = 0; i < D; i++) { hn[o + i] = h[o + i] * r1; k[o + i] *= r2; h[o + i] += gg * v[o + i]; }
        g[r] = gg; rh[r] = r1; rk[r] = r2;
    }
}
void qo_nggate_b(float *dy, const float *v, const float *hn, const float *kn, const float *g, const float *rh,
                 const float *rk, float *dv, float *dk, int N, int D)
{
    for (int r = 0; r < N; r++) {
        size_t o = (size_t)r * D;
        double a = 0, b = 0;
        for (int i = 0; i < D; i++) { a += (double)dy[o + i] * v[o + i]; b += (double)hn[o + i] * kn[o + i]; }
        float gg = g[r], cz = (float)a * gg * (1.0f - gg) / sqrtf((float)D), m = (float)b / D, r1 = rh[r], r2 = rk[r];
        for (int i = 0; i < D; i++) {
            float d = dy[o + i], x = hn[o + i], y = kn[o + i];
            dv[o + i] = gg * d; dk[o + i] = cz * (x - y * m) * r2; dy[o + i] = d + cz * (y - x * m) * r1;
        }
    }
}
