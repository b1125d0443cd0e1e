// MoE expert FFN layer: host-side control flow of the reference's moe_forward /
// moe_backward (cudalm.cu:4151-4393) over the kernels of this library.  Nothing
// here synchronises with the host: expert row counts, the row-tile table and
// the padded offsets stay on the device (the reference reads the offsets back
// once per layer, cudalm.cu:3554-3559).
//
// Row layout: the K*N routed slots n' = k*N+n are grouped by expert in stable
// order ("merged" grouping, cudalm.cu:3532-3535) and every expert's segment is
// padded with zero rows to a multiple of 128, so each 128-row GEMM tile belongs
// to one expert and filler rows contribute exact zeros to the weight gradients.
#include <string.h>
#include "qlmb_common.cuh"
#include "qlmb_gemm.cuh"

namespace qlmb {

struct Arena {
    size_t rows_cap;     // padded row capacity
    float *rt, *rprobs, *gate, *d_gate, *drt, *wr_scratch, *wrt;
    int *assign, *perm, *inv, *off, *counts, *tile_info, *ntiles, *bad, *chunk;
    bf16 *Xp, *gp, *up, *ap, *yp, *dyp, *dgp, *dup, *dXp;
    size_t bytes;
};

static size_t take(size_t &cur, size_t bytes)
{
    size_t at = cur;
    cur += (bytes + 255) & ~(size_t)255;
    return at;
}

// Carves the arena; with base == nullptr only the size is computed.
static Arena carve(void *base, int N, int D, int F, int E, int K)
{
    Arena a;
    memset(&a, 0, sizeof a);
    size_t KN = (size_t)K * N;
    a.rows_cap = (KN + (size_t)E * 127 + 127) / 128 * 128;
    size_t R = a.rows_cap, cur = 0;
    uint8_t *b = (uint8_t *)base;
#define MEMBER(field, type, count) a.field = (type *)(b + take(cur, (size_t)(count) * sizeof(type)))
    MEMBER(rt, float, (size_t)N * E);
    MEMBER(rprobs, float, (size_t)N * E);
    MEMBER(gate, float, KN);
    MEMBER(d_gate, float, KN);
    MEMBER(drt, float, (size_t)N * E);
    MEMBER(wr_scratch, float, (size_t)192 * D * E);
    MEMBER(wrt, float, (size_t)D * E);
    MEMBER(assign, int, KN);
    MEMBER(perm, int, R);
    MEMBER(inv, int, KN);
    MEMBER(off, int, E + 1);
    MEMBER(counts, int, E);
    MEMBER(tile_info, int, R / 256 + E + 1);
    MEMBER(ntiles, int, 1);
    MEMBER(bad, int, 1);
    MEMBER(chunk, int, perm_scratch_ints(N, E, K, 1));
    MEMBER(Xp, bf16, R * D);
    MEMBER(gp, bf16, R * F);
    MEMBER(up, bf16, R * F);
    MEMBER(ap, bf16, R * F);
    MEMBER(yp, bf16, R * D);
    MEMBER(dyp, bf16, R * D);
    MEMBER(dgp, bf16, R * F);
    MEMBER(dup, bf16, R * F);
    MEMBER(dXp, bf16, R * D);
#undef MEMBER
    a.bytes = cur;
    return a;
}

static int check_layer(const char *who, const qlmb_moe_layer *L, bool need_experts = true, bool need_router = true)
{
    QLMB_REQUIRE(L, "%s: NULL layer", who);
    QLMB_REQUIRE(L->N > 0 && L->E > 0 && L->E <= 256 && L->K > 0 && L->K <= 8 && L->K <= L->E, "%s: N=%d E=%d K=%d", who, L->N, L->E, L->K);
    QLMB_REQUIRE(L->dtype == QLMB_F32 || L->dtype == QLMB_BF16, "%s: dtype %d", who, L->dtype);
    QLMB_REQUIRE(!need_experts || (L->w1_codes && L->w3_codes && L->w2_codes && L->w1_scales && L->w3_scales && L->w2_scales), "%s: NULL expert weight pointer", who);
    QLMB_REQUIRE(!need_router || L->wr, "%s: NULL router weight pointer", who);
    if ((L->D % 128) || (L->F % 128)) {
        set_error("%s: D=%d and F=%d must be multiples of 128", who, L->D, L->F);
        return QLMB_E_UNSUPPORTED;
    }
    return QLMB_OK;
}

// Where the rows of an expert-side GEMM output go when they belong to other ranks: row j to row
// (perm[j] % kn) of out[perm[j] / kn] (see GemmLaunch::scatter_perm).  perm == nullptr: the arena.
struct Scatter { const int *perm; int kn; const void *out[8]; };

// gate/up (+SwiGLU) and down projections over the expert-grouped rows of `a` (cudalm.cu:4211-4225)
static int experts_forward_gemms(const qlmb_moe_layer *L, const Arena &a, cudaStream_t st, const Scatter *sc = nullptr)
{
    const int D = L->D, F = L->F, E = L->E, R = (int)a.rows_cap;
    int rc;
    GemmLaunch g = {};
    g.bmode = B_DEQ_MN; g.epi = EPI_SWIGLU; g.sched = SCHED_ROWS;
    g.a[0] = a.Xp; g.a_rows = R; g.a_cols = D;
    g.w[0] = L->w1_codes; g.w[1] = L->w3_codes; g.scales[0] = L->w1_scales; g.scales[1] = L->w3_scales;
    g.w_rows = D; g.w_cols = F; g.nseg = 1; g.ksteps = D / 64; g.M = R; g.N = F; g.E = E;
    g.tile_info = a.tile_info; g.ntiles_dev = a.ntiles; g.max_row_tiles = R / 256 + E / 2 + 1;
    g.gp = a.gp; g.up = a.up; g.ap = a.ap; g.ldo = F; g.name = "gemm_gate_up_swiglu";
    if ((rc = gemm_launch(g, st))) return rc;
    GemmLaunch h = {};
    h.bmode = B_DEQ_MN; h.epi = EPI_STORE; h.sched = SCHED_ROWS;
    h.a[0] = a.ap; h.a_rows = R; h.a_cols = F;
    h.w[0] = L->w2_codes; h.scales[0] = L->w2_scales;
    h.w_rows = F; h.w_cols = D; h.nseg = 1; h.ksteps = F / 64; h.M = R; h.N = D; h.E = E;
    h.tile_info = a.tile_info; h.ntiles_dev = a.ntiles; h.max_row_tiles = R / 256 + E / 2 + 1;
    h.out = a.yp; h.out_dtype = QLMB_BF16; h.ldo = D; h.name = "gemm_down";
    if (sc && sc->perm) { h.scatter_perm = sc->perm; h.scatter_kn = sc->kn; for (int i = 0; i < 8; i++) h.scatter_out[i] = sc->out[i]; }
    return gemm_launch(h, st);
}

// d(act) with the SwiGLU backward, dXp, and the three weight gradients (cudalm.cu:4335-4366).
// The weight gradients run on the device's side stream: dW2 needs only what exists before this
// call, dW1/dW3 need d(act)'s outputs; their tiles fill the SMs that the last, partial wave of
// d(act) and dXp leaves idle.  Everything is joined back into `st` before returning.
static int experts_backward_gemms(const qlmb_moe_layer *L, const Arena &a, float *dW1, float *dW3, float *dW2,
                                  float beta, cudaStream_t st, const Scatter *sc = nullptr)
{
    const int D = L->D, F = L->F, E = L->E, R = (int)a.rows_cap;
    int rc;
    struct { const bf16 *A; int Ma; const bf16 *B; int Nb; float *out; const char *name; } wg[3] = {
        {a.ap, F, a.dyp, D, dW2, "gemm_wgrad_w2"}, {a.Xp, D, a.dgp, F, dW1, "gemm_wgrad_w1"}, {a.Xp, D, a.dup, F, dW3, "gemm_wgrad_w3"}};
    auto wgrad = [&](int i, cudaStream_t s) {
        GemmLaunch w = {};
        w.bmode = AB_TMA_MN; w.epi = EPI_ACCUM; w.sched = SCHED_GROUPK;
        w.a[0] = wg[i].A; w.a_rows = R; w.a_cols = wg[i].Ma;
        w.w[0] = wg[i].B; w.w_cols = wg[i].Nb;
        w.nseg = 1; w.M = wg[i].Ma; w.N = wg[i].Nb; w.E = E; w.off = a.off;
        w.out = wg[i].out; w.out_dtype = QLMB_F32; w.ldo = wg[i].Nb; w.beta = beta; w.name = wg[i].name;
        return gemm_launch(w, s);
    };
    cudaStream_t side = side_fork(st);
    if ((rc = wgrad(0, side))) { side_join(side, st); return rc; }
    GemmLaunch g = {};
    g.bmode = B_DEQ_K; g.epi = EPI_SWIGLU_BWD; g.sched = SCHED_ROWS;
    g.a[0] = a.dyp; g.a_rows = R; g.a_cols = D;
    g.w[0] = L->w2_codes; g.scales[0] = L->w2_scales;
    g.w_rows = F; g.w_cols = D; g.nseg = 1; g.ksteps = D / 64; g.M = R; g.N = F; g.E = E;
    g.tile_info = a.tile_info; g.ntiles_dev = a.ntiles; g.max_row_tiles = R / 256 + E / 2 + 1;
    g.gp = a.gp; g.up = a.up; g.dgp = a.dgp; g.dup = a.dup; g.ldo = F; g.name = "gemm_dact_swiglu_bwd";
    if ((rc = gemm_launch(g, st))) { side_join(side, st); return rc; }
    side_wait_main(side, st);
    GemmLaunch h = {};
    h.bmode = B_DEQ_K; h.epi = EPI_STORE; h.sched = SCHED_ROWS;
    h.a[0] = a.dgp; h.a[1] = a.dup; h.a_rows = R; h.a_cols = F;
    h.w[0] = L->w1_codes; h.w[1] = L->w3_codes; h.scales[0] = L->w1_scales; h.scales[1] = L->w3_scales;
    h.w_rows = D; h.w_cols = F; h.nseg = 2; h.ksteps = F / 64; h.M = R; h.N = D; h.E = E;
    h.tile_info = a.tile_info; h.ntiles_dev = a.ntiles; h.max_row_tiles = R / 256 + E / 2 + 1;
    h.out = a.dXp; h.out_dtype = QLMB_BF16; h.ldo = D; h.name = "gemm_dx";
    if (sc && sc->perm) { h.scatter_perm = sc->perm; h.scatter_kn = sc->kn; for (int i = 0; i < 8; i++) h.scatter_out[i] = sc->out[i]; }
    rc = gemm_launch(h, st);
    if (!rc) rc = wgrad(1, side);
    if (!rc) rc = wgrad(2, side);
    side_join(side, st);
    return rc;
}

}  // namespace qlmb

using namespace qlmb;

extern "C" size_t qlmb_moe_arena_bytes(int N, int D, int F, int E, int K)
{
    if (N <= 0 || D <= 0 || F <= 0 || E <= 0 || K <= 0) return 0;
    return carve(nullptr, N, D, F, E, K).bytes;
}

extern "C" void *qlmb_moe_arena_member(void *arena, int N, int D, int F, int E, int K, const char *name)
{
    if (!arena || !name || N <= 0 || D <= 0 || F <= 0 || E <= 0 || K <= 0) return nullptr;
    Arena a = carve(arena, N, D, F, E, K);
#define NAMED(f) if (!strcmp(name, #f)) return (void *)a.f
    NAMED(rt); NAMED(rprobs); NAMED(gate); NAMED(d_gate); NAMED(drt); NAMED(assign); NAMED(perm); NAMED(inv);
    NAMED(off); NAMED(counts); NAMED(tile_info); NAMED(ntiles); NAMED(bad); NAMED(Xp); NAMED(gp); NAMED(up);
    NAMED(ap); NAMED(yp); NAMED(dyp); NAMED(dgp); NAMED(dup); NAMED(dXp);
#undef NAMED
    return nullptr;
}

static int moe_forward_impl(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in, const void *f_norm,
                            void *stream, bool small_router, const float *rt_in = nullptr);
extern "C" int qlmb_moe_forward(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in,
                                const void *f_norm, void *stream)
{
    return moe_forward_impl(L, arena, out, f_in, f_norm, stream, false);
}
// The same layer with the router's logits given by the caller (rt_in [N][E], as qlmb_router_topk takes them):
// two implementations can then be compared on identical expert choices, which a near-tie of two logits would
// otherwise make differ between bf16 and fp32 activations.
extern "C" int qlmb_moe_forward_routed(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in,
                                       const void *f_norm, const float *rt_in, void *stream)
{
    QLMB_REQUIRE(rt_in, "qlmb_moe_forward_routed: NULL logits");
    return moe_forward_impl(L, arena, out, f_in, f_norm, stream, false, rt_in);
}
// small_router: the logits of a decode step's few rows come from k_router_logits_small (another summation order
// than the tiled kernel; nothing reads them in a backward pass)
static int moe_forward_impl(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in, const void *f_norm,
                            void *stream, bool small_router, const float *rt_in)
{
    int rc = check_layer("qlmb_moe_forward", L);
    if (rc) return rc;
    QLMB_REQUIRE(arena && out && f_in && f_norm, "qlmb_moe_forward: NULL argument");
    QLMB_REQUIRE(((uintptr_t)arena & 255) == 0, "qlmb_moe_forward: arena must be 256-byte aligned");
    const int N = L->N, D = L->D, F = L->F, E = L->E, K = L->K;
    Arena a = carve(arena, N, D, F, E, K);
    cudaStream_t st = as_stream(stream);
    const int R = (int)a.rows_cap;

    // router: logits, softmax top-k (cudalm.cu:4158, 4174)
    if (rt_in) {
        QLMB_CUDA(cudaMemcpyAsync(a.rt, rt_in, (size_t)N * E * sizeof(float), cudaMemcpyDeviceToDevice, st));
        ProfScope ps("router_topk", st);
        if ((rc = router_topk(a.rt, a.rprobs, a.assign, a.gate, N, E, K, L->bias, L->bias_stride, st))) return rc;
    } else if (small_router) {
        if ((rc = router_small(a.rt, f_norm, L->dtype, L->wr, a.rprobs, a.assign, a.gate, N, D, E, K, L->bias, L->bias_stride, st))) return rc;
    } else {
        { ProfScope ps("router_logits", st);
        if ((rc = router_logits(a.rt, f_norm, L->dtype, L->wr, N, D, E, st))) return rc; }
        { ProfScope ps("router_topk", st);
        if ((rc = router_topk(a.rt, a.rprobs, a.assign, a.gate, N, E, K, L->bias, L->bias_stride, st))) return rc; }
    }
    // expert grouping, padded to 128-row tiles (cudalm.cu:4189)
    { ProfScope ps("perm_build", st);
    if ((rc = perm_build(a.assign, N, E, K, 1, 128, a.perm, a.inv, a.off, a.counts, a.bad, a.tile_info, a.ntiles, a.chunk, st))) return rc; }
    { ProfScope ps("gather_rows", st);
    if ((rc = gather_rows(a.Xp, f_norm, L->dtype, a.perm, a.off + E, R, N, D, st))) return rc; }

    // gate/up projections with SwiGLU in the epilogue, down projection (cudalm.cu:4211-4225)
    if ((rc = experts_forward_gemms(L, a, st))) return rc;

    // residual + gated sum over the K passes (cudalm.cu:4177, 4227)
    ProfScope ps("combine_rows", st);
    return combine_rows(out, f_in, L->dtype, a.yp, a.inv, a.gate, N, D, K, st);
}

// Forward of a decode step (dec_step's moe_forward call, cudalm.cu:7199): no stash for a backward pass.  With at
// most 128 routed rows (K * N) and bf16 activations the experts run as routed GEMVs that read only the chosen
// experts' codes; larger batches take qlmb_moe_forward.
extern "C" int qlmb_moe_decode(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in, const void *f_norm,
                               void *stream)
{
    int rc = check_layer("qlmb_moe_decode", L);
    if (rc) return rc;
    QLMB_REQUIRE(arena && out && f_in && f_norm, "qlmb_moe_decode: NULL argument");
    if (L->K * L->N > 128 || L->dtype != QLMB_BF16 || (L->D % 128) || (L->F % 128))
        return moe_forward_impl(L, arena, out, f_in, f_norm, stream, L->N <= 64);
    QLMB_REQUIRE(((uintptr_t)arena & 255) == 0, "qlmb_moe_decode: arena must be 256-byte aligned");
    const int N = L->N, D = L->D, F = L->F, E = L->E, K = L->K;
    Arena a = carve(arena, N, D, F, E, K);
    cudaStream_t st = as_stream(stream);
    // more than 16 routed rows: the experts' GEMVs want the slots grouped by expert, which the router's launch does on the way
    int grouped = 0;
    const bool want = K * N > 16;
    if ((rc = router_small(a.rt, f_norm, L->dtype, L->wr, a.rprobs, a.assign, a.gate, N, D, E, K, L->bias, L->bias_stride, st,
                           want ? a.perm : nullptr, a.off, a.counts, a.bad, want ? &grouped : nullptr))) return rc;
    return moe_decode_experts(L, out, f_in, f_norm, a.assign, a.gate, st, a.perm, a.off, a.counts, a.bad, grouped);
}

extern "C" int qlmb_moe_backward(const qlmb_moe_layer *L, void *arena, void *dfnorm, const void *dout,
                                 const void *f_norm, float *dW1, float *dW3, float *dW2, float *dWr,
                                 float beta, void *stream)
{
    int rc = check_layer("qlmb_moe_backward", L);
    if (rc) return rc;
    QLMB_REQUIRE(arena && dfnorm && dout && f_norm && dW1 && dW3 && dW2 && dWr, "qlmb_moe_backward: NULL argument");
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_moe_backward: beta %g", beta);
    const int N = L->N, D = L->D, F = L->F, E = L->E, K = L->K;
    Arena a = carve(arena, N, D, F, E, K);
    cudaStream_t st = as_stream(stream);
    const int R = (int)a.rows_cap;

    // d_gate and the gated dy (cudalm.cu:4317-4319)
    { ProfScope ps("dgate_rows", st);
    if ((rc = dgate_rows(a.dyp, a.d_gate, dout, L->dtype, a.yp, a.perm, a.gate, a.off + E, R, N, D, st))) return rc; }

    // router backward (cudalm.cu:4372-4391): needs only d_gate, so it and the router weight gradient
    // run on the second side stream next to the expert GEMMs
    cudaStream_t side = side_fork(st, 1);
    { ProfScope ps("router_bwd", side); rc = router_bwd(a.drt, a.rprobs, a.assign, a.d_gate, a.counts, N, E, K, L->aux, side); }
    if (!rc) { ProfScope ps("router_wgrad", side); rc = router_wgrad(dWr, f_norm, L->dtype, a.drt, a.wr_scratch, N, D, E, beta, side); }

    // d(act), dXp and the weight gradients (cudalm.cu:4335-4366)
    if (!rc) rc = experts_backward_gemms(L, a, dW1, dW3, dW2, beta, st);
    side_join(side, st);
    if (rc) return rc;

    ProfScope ps("unpermute_rows", st);
    return unpermute_rows(dfnorm, L->dtype, a.dXp, a.inv, a.drt, L->wr, a.wrt, N, D, E, K, st);
}

// ===================================================================== expert parallelism
// The same layer cut at the two places where rows cross GPUs.  The home rank of a token
// routes it and packs its K copies into expert order (compact, no filler rows) for the
// dispatch all-to-all; the rank that owns an expert runs the FFN on whatever rows arrive,
// tagged with their local expert index; the home rank combines what comes back.  The
// exchanges themselves (NCCL all-to-all) are done by the caller between these calls.

extern "C" int qlmb_moe_route(const qlmb_moe_layer *L, void *arena, void *Xs, const void *f_norm, void *stream)
{
    int rc = check_layer("qlmb_moe_route", L, false, true);
    if (rc) return rc;
    QLMB_REQUIRE(arena && Xs && f_norm, "qlmb_moe_route: NULL argument");
    const int N = L->N, D = L->D, F = L->F, E = L->E, K = L->K;
    Arena a = carve(arena, N, D, F, E, K);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("router_logits", st); if ((rc = router_logits(a.rt, f_norm, L->dtype, L->wr, N, D, E, st))) return rc; }
    { ProfScope ps("router_topk", st); if ((rc = router_topk(a.rt, a.rprobs, a.assign, a.gate, N, E, K, L->bias, L->bias_stride, st))) return rc; }
    { ProfScope ps("perm_build", st);
      if ((rc = perm_build(a.assign, N, E, K, 1, 1, a.perm, a.inv, a.off, a.counts, a.bad, nullptr, nullptr, a.chunk, st))) return rc; }
    ProfScope ps("gather_rows", st);
    return gather_rows((bf16 *)Xs, f_norm, L->dtype, a.perm, nullptr, K * N, N, D, st);
}

extern "C" int qlmb_moe_combine(const qlmb_moe_layer *L, void *arena, void *out, const void *f_in, const void *Ys,
                                void *stream)
{
    int rc = check_layer("qlmb_moe_combine", L, false, false);
    if (rc) return rc;
    QLMB_REQUIRE(arena && out && f_in && Ys, "qlmb_moe_combine: NULL argument");
    Arena a = carve(arena, L->N, L->D, L->F, L->E, L->K);
    ProfScope ps("combine_rows", as_stream(stream));
    return combine_rows(out, f_in, L->dtype, (const bf16 *)Ys, a.inv, a.gate, L->N, L->D, L->K, as_stream(stream));
}

extern "C" int qlmb_moe_dgate(const qlmb_moe_layer *L, void *arena, void *dYs, const void *dout, const void *Ys,
                              void *stream)
{
    int rc = check_layer("qlmb_moe_dgate", L, false, false);
    if (rc) return rc;
    QLMB_REQUIRE(arena && dYs && dout && Ys, "qlmb_moe_dgate: NULL argument");
    Arena a = carve(arena, L->N, L->D, L->F, L->E, L->K);
    ProfScope ps("dgate_rows", as_stream(stream));
    return dgate_rows((bf16 *)dYs, a.d_gate, dout, L->dtype, (const bf16 *)Ys, a.perm, a.gate, nullptr, L->K * L->N,
                      L->N, L->D, as_stream(stream));
}

extern "C" int qlmb_moe_route_backward(const qlmb_moe_layer *L, void *arena, void *dfnorm, const void *dXs,
                                       const void *f_norm, float *dWr, float beta, void *stream)
{
    int rc = check_layer("qlmb_moe_route_backward", L, false, true);
    if (rc) return rc;
    QLMB_REQUIRE(arena && dfnorm && dXs && f_norm && dWr, "qlmb_moe_route_backward: NULL argument");
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_moe_route_backward: beta %g", beta);
    const int N = L->N, D = L->D, E = L->E, K = L->K;
    Arena a = carve(arena, N, D, L->F, E, K);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("router_bwd", st); if ((rc = router_bwd(a.drt, a.rprobs, a.assign, a.d_gate, a.counts, N, E, K, L->aux, st))) return rc; }
    cudaStream_t side = side_fork(st, 1);
    { ProfScope ps("router_wgrad", side); rc = router_wgrad(dWr, f_norm, L->dtype, a.drt, a.wr_scratch, N, D, E, beta, side); }
    if (!rc) { ProfScope ps("unpermute_rows", st); rc = unpermute_rows(dfnorm, L->dtype, (const bf16 *)dXs, a.inv, a.drt, L->wr, a.wrt, N, D, E, K, st); }
    side_join(side, st);
    return rc;
}

// Expert side.  L describes the experts held by this rank (E = local experts, K is ignored,
// N = row capacity of `earena`, which was sized with qlmb_moe_arena_bytes(N, D, F, E, 1)).
// X[R][D] (bf16) are the received rows in arrival order, expert_of_row[R] their local expert
// index; Y[R][D] receives the FFN output of every row, in the same order.
extern "C" int qlmb_moe_experts_forward(const qlmb_moe_layer *L, void *earena, void *Y, const void *X,
                                        const int *expert_of_row, int R, void *stream)
{
    int rc = check_layer("qlmb_moe_experts_forward", L, true, false);
    if (rc) return rc;
    QLMB_REQUIRE(earena && R >= 0 && R <= L->N, "qlmb_moe_experts_forward: %d rows exceed the arena capacity %d", R, L->N);
    if (R == 0) return QLMB_OK;
    QLMB_REQUIRE(Y && X && expert_of_row, "qlmb_moe_experts_forward: NULL argument");
    const int D = L->D, E = L->E;
    Arena a = carve(earena, L->N, D, L->F, E, 1);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("perm_build", st);
      if ((rc = perm_build(expert_of_row, R, E, 1, 1, 128, a.perm, a.inv, a.off, a.counts, a.bad, a.tile_info, a.ntiles, a.chunk, st))) return rc; }
    { ProfScope ps("gather_rows", st);
      if ((rc = gather_rows(a.Xp, X, QLMB_BF16, a.perm, a.off + E, (int)a.rows_cap, R, D, st))) return rc; }
    if ((rc = experts_forward_gemms(L, a, st))) return rc;
    ProfScope ps("gather_rows", st);
    return gather_rows((bf16 *)Y, a.yp, QLMB_BF16, a.inv, nullptr, R, (int)a.rows_cap, D, st);
}

// dY[R][D] (bf16): gradients of the rows' outputs, in arrival order (gate already applied by
// the home rank).  dX[R][D] receives the gradients of the rows' inputs; the weight gradients
// of the local experts are added into (beta = 1) or written to (beta = 0) dW1/dW3/dW2.
extern "C" int qlmb_moe_experts_backward(const qlmb_moe_layer *L, void *earena, void *dX, const void *dY, int R,
                                         float *dW1, float *dW3, float *dW2, float beta, void *stream)
{
    int rc = check_layer("qlmb_moe_experts_backward", L, true, false);
    if (rc) return rc;
    QLMB_REQUIRE(earena && dW1 && dW3 && dW2 && R >= 0 && R <= L->N, "qlmb_moe_experts_backward: bad argument");
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_moe_experts_backward: beta %g", beta);
    QLMB_REQUIRE(R == 0 || (dX && dY), "qlmb_moe_experts_backward: NULL argument");
    const int D = L->D, E = L->E;
    Arena a = carve(earena, L->N, D, L->F, E, 1);
    cudaStream_t st = as_stream(stream);
    if (R == 0) {
        // no rows arrived: the permutation of the forward holds zero rows per expert
        if (beta == 0.0f) {
            QLMB_CUDA(cudaMemsetAsync(dW1, 0, (size_t)E * D * L->F * sizeof(float), st));
            QLMB_CUDA(cudaMemsetAsync(dW3, 0, (size_t)E * D * L->F * sizeof(float), st));
            QLMB_CUDA(cudaMemsetAsync(dW2, 0, (size_t)E * D * L->F * sizeof(float), st));
        }
        return QLMB_OK;
    }
    { ProfScope ps("gather_rows", st);
      if ((rc = gather_rows(a.dyp, dY, QLMB_BF16, a.perm, a.off + E, (int)a.rows_cap, R, D, st))) return rc; }
    if ((rc = experts_backward_gemms(L, a, dW1, dW3, dW2, beta, st))) return rc;
    ProfScope ps("gather_rows", st);
    return gather_rows((bf16 *)dX, a.dXp, QLMB_BF16, a.inv, nullptr, R, (int)a.rows_cap, D, st);
}

// ------------------------------------------------ expert parallelism by peer loads
namespace qlmb {
static int check_peers(const char *who, const qlmb_ep_peers *P)
{
    QLMB_REQUIRE(P && P->world >= 1 && P->world <= QLMB_EP_MAX_WORLD && P->rank >= 0 && P->rank < P->world,
                 "%s: bad peer table", who);
    for (int i = 0; i < P->world; i++) QLMB_REQUIRE(P->base[i], "%s: window of rank %d is not mapped", who, i);
    return QLMB_OK;
}
// the buffer at `local` (inside this rank's window) as seen in every rank's window
static PeerPtrs peer_view(const qlmb_ep_peers *P, const void *local)
{
    PeerPtrs v;
    memset(&v, 0, sizeof v);
    const ptrdiff_t off = (const char *)local - (const char *)P->base[P->rank];
    for (int i = 0; i < P->world; i++) v.p[i] = (const char *)P->base[i] + off;
    return v;
}
static int check_ep_shapes(const char *who, const qlmb_moe_layer *home, const qlmb_moe_layer *loc, const qlmb_ep_peers *P)
{
    QLMB_REQUIRE(home->E == loc->E * P->world, "%s: %d experts in total but %d ranks x %d local", who, home->E, P->world, loc->E);
    QLMB_REQUIRE(loc->N == P->world * home->K * home->N, "%s: expert arena holds %d slots, need %d", who, loc->N,
                 P->world * home->K * home->N);
    QLMB_REQUIRE(home->D == loc->D && home->F == loc->F, "%s: D/F differ between the two layer views", who);
    return QLMB_OK;
}
}  // namespace qlmb

extern "C" int qlmb_ep_route(const qlmb_moe_layer *L, void *harena, const void *f_norm, void *stream)
{
    int rc = check_layer("qlmb_ep_route", L, false, true);
    if (rc) return rc;
    QLMB_REQUIRE(harena && f_norm, "qlmb_ep_route: NULL argument");
    const int N = L->N, D = L->D, E = L->E, K = L->K;
    Arena a = carve(harena, N, D, L->F, E, K);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("router_logits", st); if ((rc = router_logits(a.rt, f_norm, L->dtype, L->wr, N, D, E, st))) return rc; }
    { ProfScope ps("router_topk", st); if ((rc = router_topk(a.rt, a.rprobs, a.assign, a.gate, N, E, K, L->bias, L->bias_stride, st))) return rc; }
    ProfScope ps("count_assign", st);
    return count_assign(a.counts, a.assign, K * N, E, st);
}

extern "C" int qlmb_ep_experts_forward(const qlmb_moe_layer *L, void *earena, const qlmb_ep_peers *P,
                                       const int *assign_all, const void *f_norm, int x_dtype, int tokens_per_rank,
                                       int K, void *Ys, void *stream)
{
    int rc = check_layer("qlmb_ep_experts_forward", L, true, false);
    if (rc) return rc;
    if ((rc = check_peers("qlmb_ep_experts_forward", P))) return rc;
    QLMB_REQUIRE(earena && assign_all && f_norm && Ys, "qlmb_ep_experts_forward: NULL argument");
    QLMB_REQUIRE(x_dtype == QLMB_F32 || x_dtype == QLMB_BF16, "qlmb_ep_experts_forward: dtype %d", x_dtype);
    QLMB_REQUIRE(tokens_per_rank > 0 && K > 0 && L->N == P->world * K * tokens_per_rank,
                 "qlmb_ep_experts_forward: arena holds %d slots, need %d", L->N, P->world * K * tokens_per_rank);
    const int D = L->D, E = L->E, KN = K * tokens_per_rank;
    Arena a = carve(earena, L->N, D, L->F, E, 1);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("perm_build", st);
      if ((rc = perm_build(assign_all, L->N, E, 1, 1, 128, a.perm, a.inv, a.off, a.counts, a.bad, a.tile_info, a.ntiles,
                           a.chunk, st, P->rank * E, 1))) return rc; }
    { ProfScope ps("gather_rows_peer", st);
      if ((rc = gather_rows_peer(a.Xp, peer_view(P, f_norm), x_dtype, a.perm, a.off + E, (int)a.rows_cap, tokens_per_rank, KN, D, st))) return rc; }
    // the down projection's epilogue writes every output row straight into the Ys buffer of the
    // row's home rank, at the row's slot
    Scatter sc;
    sc.perm = a.perm; sc.kn = KN;
    PeerPtrs yv = peer_view(P, Ys);
    for (int i = 0; i < 8; i++) sc.out[i] = i < P->world ? yv.p[i] : nullptr;
    return experts_forward_gemms(L, a, st, &sc);
}

extern "C" int qlmb_ep_combine(const qlmb_moe_layer *H, void *harena, const void *Ys, void *out, const void *f_in,
                               void *stream)
{
    int rc = check_layer("qlmb_ep_combine", H, false, false);
    if (rc) return rc;
    QLMB_REQUIRE(harena && Ys && out && f_in, "qlmb_ep_combine: NULL argument");
    Arena h = carve(harena, H->N, H->D, H->F, H->E, H->K);
    ProfScope ps("combine_rows", as_stream(stream));
    return combine_rows(out, f_in, H->dtype, (const bf16 *)Ys, nullptr, h.gate, H->N, H->D, H->K, as_stream(stream));
}

extern "C" int qlmb_ep_dgate(const qlmb_moe_layer *H, void *harena, const void *Ys, const void *dout, void *stream)
{
    int rc = check_layer("qlmb_ep_dgate", H, false, false);
    if (rc) return rc;
    QLMB_REQUIRE(harena && Ys && dout, "qlmb_ep_dgate: NULL argument");
    Arena h = carve(harena, H->N, H->D, H->F, H->E, H->K);
    ProfScope ps("dgate_dot", as_stream(stream));
    return dgate_dot_peer(h.d_gate, dout, H->dtype, (const bf16 *)Ys, H->N, H->D, H->K, as_stream(stream));
}

extern "C" int qlmb_ep_experts_backward(const qlmb_moe_layer *L, void *earena, const qlmb_moe_layer *H, void *harena,
                                        const qlmb_ep_peers *P, const void *dout, int tokens_per_rank, int K,
                                        void *dXs, float *dW1, float *dW3, float *dW2, float beta, void *stream)
{
    int rc = check_layer("qlmb_ep_experts_backward", L, true, false);
    if (rc) return rc;
    if ((rc = check_peers("qlmb_ep_experts_backward", P))) return rc;
    QLMB_REQUIRE(H && earena && harena && dout && dXs && dW1 && dW3 && dW2, "qlmb_ep_experts_backward: NULL argument");
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_ep_experts_backward: beta %g", beta);
    if ((rc = check_ep_shapes("qlmb_ep_experts_backward", H, L, P))) return rc;
    QLMB_REQUIRE(tokens_per_rank == H->N && K == H->K, "qlmb_ep_experts_backward: tokens_per_rank / K differ from the router view");
    Arena h = carve(harena, H->N, H->D, H->F, H->E, H->K);
    Arena e = carve(earena, L->N, L->D, L->F, L->E, 1);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("dyp_rows_peer", st);
      if ((rc = dyp_rows_peer(e.dyp, peer_view(P, dout), peer_view(P, h.gate), H->dtype, e.perm, e.off + L->E, (int)e.rows_cap,
                              tokens_per_rank, K * tokens_per_rank, L->D, st))) return rc; }
    Scatter sc;                                          // dX rows go straight to their home rank's dXs buffer
    sc.perm = e.perm; sc.kn = K * tokens_per_rank;
    PeerPtrs xv = peer_view(P, dXs);
    for (int i = 0; i < 8; i++) sc.out[i] = i < P->world ? xv.p[i] : nullptr;
    return experts_backward_gemms(L, e, dW1, dW3, dW2, beta, st, &sc);
}

extern "C" int qlmb_ep_route_backward(const qlmb_moe_layer *H, void *harena, const void *dXs, void *dfnorm,
                                      const void *f_norm, float *dWr, float beta, void *stream)
{
    int rc = check_layer("qlmb_ep_route_backward", H, false, true);
    if (rc) return rc;
    QLMB_REQUIRE(harena && dXs && dfnorm && f_norm && dWr, "qlmb_ep_route_backward: NULL argument");
    QLMB_REQUIRE(beta == 0.0f || beta == 1.0f, "qlmb_ep_route_backward: beta %g", beta);
    const int N = H->N, D = H->D, E = H->E, K = H->K;
    Arena h = carve(harena, N, D, H->F, E, K);
    cudaStream_t st = as_stream(stream);
    { ProfScope ps("router_bwd", st); if ((rc = router_bwd(h.drt, h.rprobs, h.assign, h.d_gate, h.counts, N, E, K, H->aux, st))) return rc; }
    cudaStream_t side = side_fork(st, 1);
    { ProfScope ps("router_wgrad", side); rc = router_wgrad(dWr, f_norm, H->dtype, h.drt, h.wr_scratch, N, D, E, beta, side); }
    // dXs is in slot order (k*N + n): no row index needed
    if (!rc) { ProfScope ps("unpermute_rows", st);
               rc = unpermute_rows(dfnorm, H->dtype, (const bf16 *)dXs, nullptr, h.drt, H->wr, h.wrt, N, D, E, K, st); }
    side_join(side, st);
    return rc;
}
