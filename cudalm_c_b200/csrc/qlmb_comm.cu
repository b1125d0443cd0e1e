// Native multi-GPU host layer: one process per GPU, NCCL over NVLink for the exchanges the data-parallel and
// expert-parallel forms of the step need, and the composed calls a C or C++ trainer would make per step.  The
// reference is single-GPU (its ranks do not exist), so nothing here has a reference counterpart; the per-rank
// arithmetic is the library's own entry points (qlmb_step, qlmb_gnorm_*, qlmb_ep_*).
//
// NCCL is bound at run time (dlopen of libnccl.so.2: the copy the process has already loaded, e.g. torch's, else the
// system's), so the library still loads on a machine without NCCL or a GPU.  Only its stable C entry points are used.
#include "qlmb_common.cuh"
#include <dlfcn.h>
#include <string.h>
#include <stdlib.h>
#include <mutex>

namespace qlmb {
namespace {

typedef struct ncclComm *nccl_comm_t;
typedef struct { char internal[128]; } nccl_uid_t;
enum { NC_INT8 = 0, NC_UINT8 = 1, NC_INT32 = 2, NC_FLOAT32 = 7 };     // ncclDataType_t
enum { NC_SUM = 0, NC_MAX = 2, NC_AVG = 4 };                          // ncclRedOp_t

struct Nccl {
    void *so = nullptr;
    int (*GetUniqueId)(nccl_uid_t *) = nullptr;
    int (*CommInitRank)(nccl_comm_t *, int, nccl_uid_t, int) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*GroupStart)(void) = nullptr;
    int (*GroupEnd)(void) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
};
Nccl g_nccl;
std::once_flag g_nccl_once;

void nccl_bind()
{
    Nccl &n = g_nccl;
    const char *names[] = {getenv("QLMB_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    n.so = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);               // share the copy the process already has
    for (int i = 0; i < 3 && !n.so; i++)
        if (names[i] && names[i][0]) n.so = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!n.so) return;
#define QLMB_SYM(field, name) *(void **)(&n.field) = dlsym(n.so, name)
    QLMB_SYM(GetUniqueId, "ncclGetUniqueId");
    QLMB_SYM(CommInitRank, "ncclCommInitRank");
    QLMB_SYM(CommDestroy, "ncclCommDestroy");
    QLMB_SYM(AllReduce, "ncclAllReduce");
    QLMB_SYM(AllGather, "ncclAllGather");
    QLMB_SYM(GroupStart, "ncclGroupStart");
    QLMB_SYM(GroupEnd, "ncclGroupEnd");
    QLMB_SYM(GetErrorString, "ncclGetErrorString");
#undef QLMB_SYM
    n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllReduce && n.AllGather && n.GroupStart && n.GroupEnd;
}

int nccl_ready(const char *who)
{
    std::call_once(g_nccl_once, nccl_bind);
    if (!g_nccl.ok) { set_error("%s: NCCL (libnccl.so.2) could not be loaded; set QLMB_NCCL_LIB to its path", who); return QLMB_E_UNSUPPORTED; }
    return QLMB_OK;
}
int nccl_fail(int rc, const char *what)
{
    set_error("%s: NCCL error %d (%s)", what, rc, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?");
    return QLMB_E_CUDA;
}
#define QLMB_NCCL(call, what)                                                  \
    do {                                                                       \
        int rc__ = (call);                                                     \
        if (rc__ != 0) return nccl_fail(rc__, what);                           \
    } while (0)

} // namespace
} // namespace qlmb

using namespace qlmb;

struct qlmb_comm {
    nccl_comm_t nc;
    int rank, world, device;
    int *flag;               // one device int: the operand of the stream-ordered barrier
    unsigned char *handles;  // world * 64 bytes on the device: IPC handles while windows are opened
};

extern "C" int qlmb_comm_unique_id(unsigned char id[128])
{
    QLMB_REQUIRE(id, "qlmb_comm_unique_id: NULL argument");
    int rc = nccl_ready("qlmb_comm_unique_id");
    if (rc != QLMB_OK) return rc;
    nccl_uid_t u;
    QLMB_NCCL(g_nccl.GetUniqueId(&u), "ncclGetUniqueId");
    memcpy(id, &u, 128);
    return QLMB_OK;
}

extern "C" int qlmb_comm_init(qlmb_comm **out, const unsigned char id[128], int rank, int world)
{
    QLMB_REQUIRE(out && id && world >= 1 && world <= 1024 && rank >= 0 && rank < world, "qlmb_comm_init: rank %d of %d", rank, world);
    int rc = nccl_ready("qlmb_comm_init");
    if (rc != QLMB_OK) return rc;
    qlmb_comm *c = (qlmb_comm *)calloc(1, sizeof(qlmb_comm));
    QLMB_REQUIRE(c, "qlmb_comm_init: out of host memory");
    c->rank = rank; c->world = world;
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc(&c->flag, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->flag, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&c->handles, (size_t)world * 64);
    if (e != cudaSuccess) { cudaFree(c->flag); free(c); return cuda_fail(e, "qlmb_comm_init"); }
    nccl_uid_t u;
    memcpy(&u, id, 128);
    int nrc = g_nccl.CommInitRank(&c->nc, world, u, rank);
    if (nrc != 0) { cudaFree(c->flag); cudaFree(c->handles); free(c); return nccl_fail(nrc, "ncclCommInitRank"); }
    *out = c;
    return QLMB_OK;
}

extern "C" int qlmb_comm_destroy(qlmb_comm *c)
{
    if (!c) return QLMB_OK;
    if (c->nc) g_nccl.CommDestroy(c->nc);
    cudaFree(c->flag);
    cudaFree(c->handles);
    free(c);
    return QLMB_OK;
}

extern "C" int qlmb_comm_rank(const qlmb_comm *c) { return c ? c->rank : -1; }
extern "C" int qlmb_comm_world(const qlmb_comm *c) { return c ? c->world : 0; }

// sum (avg = 0) or mean (avg = 1) of n floats over the ranks, in place
extern "C" int qlmb_comm_allreduce_f32(qlmb_comm *c, float *buf, unsigned long long n, int avg, void *stream)
{
    QLMB_REQUIRE(c && (buf || n == 0), "qlmb_comm_allreduce_f32: NULL argument");
    if (n == 0 || c->world == 1) return QLMB_OK;
    QLMB_NCCL(g_nccl.AllReduce(buf, buf, (size_t)n, NC_FLOAT32, avg ? NC_AVG : NC_SUM, c->nc, as_stream(stream)), "ncclAllReduce");
    return QLMB_OK;
}

// recv[r*bytes ...] = rank r's `bytes` bytes; send == recv + rank*bytes gathers in place
extern "C" int qlmb_comm_allgather(qlmb_comm *c, const void *send, void *recv, unsigned long long bytes, void *stream)
{
    QLMB_REQUIRE(c && send && recv, "qlmb_comm_allgather: NULL argument");
    if (bytes == 0) return QLMB_OK;
    if (c->world == 1) {
        if (send != recv) QLMB_CUDA(cudaMemcpyAsync(recv, send, (size_t)bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
        return QLMB_OK;
    }
    QLMB_NCCL(g_nccl.AllGather(send, recv, (size_t)bytes, NC_UINT8, c->nc, as_stream(stream)), "ncclAllGather");
    return QLMB_OK;
}

// Stream-ordered meeting point: work enqueued after it on any rank starts after the work enqueued before it on
// every rank.  Nothing waits on the host and no kernel of this library waits for another GPU.
extern "C" int qlmb_comm_barrier(qlmb_comm *c, void *stream)
{
    QLMB_REQUIRE(c, "qlmb_comm_barrier: NULL argument");
    if (c->world == 1) return QLMB_OK;
    QLMB_NCCL(g_nccl.AllReduce(c->flag, c->flag, 1, NC_INT32, NC_MAX, c->nc, as_stream(stream)), "ncclAllReduce (barrier)");
    return QLMB_OK;
}

// ---- data parallelism: the gradient of the replicated parameters is the mean over the ranks' batches; the global
// norm then comes from the averaged buffer exactly as on one GPU (k_sqsum + k_gnorm, cudalm.cu:6442-6444).
extern "C" int qlmb_dp_grad_sync(qlmb_comm *c, float *G, unsigned long long n, void *stream)
{
    return qlmb_comm_allreduce_f32(c, G, n, 1, stream);
}
// Global norm and clip multiplier when some gradient buffers are rank-local (the expert shards of an expert-parallel
// model): part holds 64 partial sums of squares per buffer; the slices [first_local, nslice) belong to rank-local
// buffers and are summed over the ranks before qlmb_gnorm_close turns all of them into gs = {multiplier, norm}.
extern "C" int qlmb_dp_gnorm_close(qlmb_comm *c, float *part, int nslice, int first_local, float *gs, void *stream)
{
    QLMB_REQUIRE(c && part && gs && nslice > 0 && first_local >= 0 && first_local <= nslice, "qlmb_dp_gnorm_close: bad argument");
    int rc = qlmb_comm_allreduce_f32(c, part + 64 * (size_t)first_local, 64ull * (unsigned long long)(nslice - first_local), 0, stream);
    if (rc != QLMB_OK) return rc;
    return qlmb_gnorm_close(part, nslice, gs, stream);
}

// ---- ZeRO-1 form of the integer AdamW step: the ngrp groups of the spans are cut into `world` equal shares; this
// rank steps its share (all seven state arrays of the share stay rank-local) and the new codes and nothing else
// travel: ngrp*group/2 bytes in total per step (packed) instead of the fp32 parameters.  The scales do not change in
// a step (the servo pass changes them; call qlmb_zero1_gather_scales after it).  Bit-identical to qlmb_step on the
// whole span, because element and step keys of the rounding hash are global.
extern "C" int qlmb_zero1_step(qlmb_comm *c, float *P, const float *G, int8_t *d, int8_t *r, const float *s, int8_t *m8,
                               float *m8s, uint8_t *v8, float *v8s, const qlmb_span *sp, int nspan, int ngrp, int group,
                               int dmax, float lr, float b1, float b2, float wd, float gscale, const float *gsp,
                               float inv_bc1, float inv_sqrt_bc2, int lrmode, uint64_t t, int adam, int64_t *stat,
                               int packed, void *stream)
{
    QLMB_REQUIRE(c && d && sp, "qlmb_zero1_step: NULL argument");
    QLMB_REQUIRE(ngrp > 0 && ngrp % c->world == 0, "qlmb_zero1_step: %d groups do not divide over %d ranks", ngrp, c->world);
    QLMB_REQUIRE(group % 2 == 0, "qlmb_zero1_step: group %d", group);
    const int per = ngrp / c->world, gi0 = c->rank * per;
    int rc = qlmb_step(P, G, d, r, s, m8, m8s, v8, v8s, sp, nspan, group, dmax, lr, b1, b2, wd, gscale, gsp, inv_bc1,
                       inv_sqrt_bc2, lrmode, t, adam, stat, packed, gi0, per, stream);
    if (rc != QLMB_OK) return rc;
    const size_t bytes = packed ? (size_t)per * group / 2 : (size_t)per * group;
    return qlmb_comm_allgather(c, d + (size_t)c->rank * bytes, d, bytes, stream);
}
extern "C" int qlmb_zero1_gather_scales(qlmb_comm *c, float *s, int ngrp, void *stream)
{
    QLMB_REQUIRE(c && s && ngrp > 0 && ngrp % c->world == 0, "qlmb_zero1_gather_scales: bad argument");
    const size_t bytes = (size_t)(ngrp / c->world) * 4;
    return qlmb_comm_allgather(c, (const char *)s + (size_t)c->rank * bytes, s, bytes, stream);
}

// ---- expert parallelism over peer memory: windows and the per-layer call order
// Opens every rank's window (allocated with qlmb_peer_alloc) in this process: the 64-byte handles travel by one
// all-gather.  peers->base[rank] is this rank's own pointer.  Synchronises the stream once (set-up, not per step).
extern "C" int qlmb_ep_window_open(qlmb_comm *c, void *window, qlmb_ep_peers *peers, void *stream)
{
    QLMB_REQUIRE(c && window && peers, "qlmb_ep_window_open: NULL argument");
    QLMB_REQUIRE(c->world <= QLMB_EP_MAX_WORLD, "qlmb_ep_window_open: %d ranks, at most %d", c->world, QLMB_EP_MAX_WORLD);
    memset(peers, 0, sizeof(*peers));
    peers->rank = c->rank; peers->world = c->world;
    peers->base[c->rank] = window;
    if (c->world == 1) return QLMB_OK;
    unsigned char mine[64], *all = (unsigned char *)malloc((size_t)c->world * 64);
    QLMB_REQUIRE(all, "qlmb_ep_window_open: out of host memory");
    int rc = qlmb_peer_export(window, mine);
    cudaStream_t st = as_stream(stream);
    if (rc == QLMB_OK && cudaMemcpyAsync(c->handles + (size_t)c->rank * 64, mine, 64, cudaMemcpyHostToDevice, st) != cudaSuccess) rc = QLMB_E_CUDA;
    if (rc == QLMB_OK) rc = qlmb_comm_allgather(c, c->handles + (size_t)c->rank * 64, c->handles, 64, stream);
    if (rc == QLMB_OK && (cudaMemcpyAsync(all, c->handles, (size_t)c->world * 64, cudaMemcpyDeviceToHost, st) != cudaSuccess
                          || cudaStreamSynchronize(st) != cudaSuccess)) { set_error("qlmb_ep_window_open: copying the handles failed"); rc = QLMB_E_CUDA; }
    for (int r = 0; rc == QLMB_OK && r < c->world; r++) {
        if (r == c->rank) continue;
        rc = qlmb_peer_open(all + (size_t)r * 64, &peers->base[r]);
    }
    free(all);
    if (rc == QLMB_OK) rc = qlmb_comm_barrier(c, stream);               // every window is mapped before a step reads one
    return rc;
}

// Closes the peers' windows after all ranks have finished their work on them.
extern "C" int qlmb_ep_window_close(qlmb_comm *c, qlmb_ep_peers *peers, void *stream)
{
    QLMB_REQUIRE(c && peers, "qlmb_ep_window_close: NULL argument");
    int rc = qlmb_comm_barrier(c, stream);
    if (cudaStreamSynchronize(as_stream(stream)) != cudaSuccess && rc == QLMB_OK) rc = QLMB_E_CUDA;
    for (int r = 0; r < peers->world; r++) {
        if (r != peers->rank && peers->base[r]) qlmb_peer_close(peers->base[r]);
        if (r != peers->rank) peers->base[r] = nullptr;
    }
    return rc;
}

// One layer's forward in the order the peer-memory design needs: route, all-gather of the routing table, the expert
// side (reads foreign rows, stores into the home ranks' Ys), meeting point, combine.
extern "C" int qlmb_ep_layer_forward(qlmb_comm *c, const qlmb_moe_layer *home, void *harena, const qlmb_moe_layer *loc, void *earena,
                                     const qlmb_ep_peers *peers, int *assign_all, const void *f_norm, int x_dtype, const void *f_in,
                                     void *Ys, void *out, void *stream)
{
    QLMB_REQUIRE(c && home && loc && peers && assign_all, "qlmb_ep_layer_forward: NULL argument");
    const int N = home->N, K = home->K;
    int rc = qlmb_ep_route(home, harena, f_norm, stream);
    if (rc != QLMB_OK) return rc;
    const int *assign = (const int *)qlmb_moe_arena_member((void *)harena, home->N, home->D, home->F, home->E, home->K, "assign");
    QLMB_REQUIRE(assign, "qlmb_ep_layer_forward: the arena has no member 'assign'");
    rc = qlmb_comm_allgather(c, assign, assign_all, (unsigned long long)K * N * 4, stream);
    if (rc != QLMB_OK) return rc;
    rc = qlmb_ep_experts_forward(loc, earena, peers, assign_all, f_norm, x_dtype, N, K, Ys, stream);
    if (rc != QLMB_OK) return rc;
    rc = qlmb_comm_barrier(c, stream);
    if (rc != QLMB_OK) return rc;
    return qlmb_ep_combine(home, harena, Ys, out, f_in, stream);
}

// The layer's backward: gate gradients at home, meeting point when dout was written this step (inputs_fresh), the
// expert side (stores dX rows into the home ranks' dXs), meeting point, router backward at home.
extern "C" int qlmb_ep_layer_backward(qlmb_comm *c, const qlmb_moe_layer *home, void *harena, const qlmb_moe_layer *loc, void *earena,
                                      const qlmb_ep_peers *peers, const void *dout, const void *f_norm, const void *Ys, void *dXs,
                                      void *dfnorm, float *dW1, float *dW3, float *dW2, float *dWr, float beta, int inputs_fresh,
                                      void *stream)
{
    QLMB_REQUIRE(c && home && loc && peers, "qlmb_ep_layer_backward: NULL argument");
    int rc = qlmb_ep_dgate(home, harena, Ys, dout, stream);
    if (rc == QLMB_OK && inputs_fresh) rc = qlmb_comm_barrier(c, stream);
    if (rc != QLMB_OK) return rc;
    rc = qlmb_ep_experts_backward(loc, earena, home, harena, peers, dout, home->N, home->K, dXs, dW1, dW3, dW2, beta, stream);
    if (rc != QLMB_OK) return rc;
    rc = qlmb_comm_barrier(c, stream);
    if (rc != QLMB_OK) return rc;
    return qlmb_ep_route_backward(home, harena, dXs, dfnorm, f_norm, dWr, beta, stream);
}
