// Shared declarations for libqlm_b200: status handling, span lookup, nibble
// access and the rounding hash.  Device code here is integer-only, so it is
// safe to include from translation units built with or without --fmad=false.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "../../include/qlm_b200.h"

namespace qlmb {

// ---- host-side status ------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);          // records + returns QLMB_E_CUDA
int *device_error_word(void);                            // per-device int, lazily allocated
#define QLMB_CUDA(call)                                                        \
    do {                                                                       \
        cudaError_t e__ = (call);                                              \
        if (e__ != cudaSuccess) return qlmb::cuda_fail(e__, #call);            \
    } while (0)
#define QLMB_REQUIRE(cond, ...)                                                \
    do {                                                                       \
        if (!(cond)) { qlmb::set_error(__VA_ARGS__); return QLMB_E_ARG; }      \
    } while (0)
#define QLMB_LAUNCH_CHECK(what)                                                \
    do {                                                                       \
        cudaError_t e__ = cudaGetLastError();                                  \
        if (e__ != cudaSuccess) return qlmb::cuda_fail(e__, what);             \
    } while (0)

static inline cudaStream_t as_stream(void *s) { return (cudaStream_t)s; }
int sm_count(void);                                      // SMs of the current device
// second stream of the device for overlappable work (qlmb_runtime.cu); returns `st` itself when unavailable
cudaStream_t side_fork(cudaStream_t st, int which = 0);   // two side streams per device: which = 0 or 1
void side_wait_main(cudaStream_t side, cudaStream_t st);
void side_join(cudaStream_t side, cudaStream_t st);
// Times the enclosed launches with CUDA events when qlmb_prof_enable(1) was called.
struct ProfScope {
    int slot; cudaStream_t stream;
    ProfScope(const char *name, cudaStream_t st);
    ~ProfScope();
};

// ---- programmatic dependent launch ----------------------------------------
// A kernel launched with pdl_launch may start while the kernel before it in the stream is still running: its blocks
// are scheduled as soon as every block of that kernel has called pdl_trigger() (or exited), and run up to their
// pdl_wait(), which returns once that kernel has completed and its writes are visible.  Rules kept by every such kernel:
// every block executes pdl_wait() exactly once, before its first read of anything a kernel of the stream wrote, before
// its first write, and before any early return; only data that no kernel of the step writes (the weights) is touched
// ahead of it.  The caller decides per launch (`early`): with one to four rows per step the early blocks cost the
// running kernel more than they gain (decode step 0.53 -> 0.56 ms at one slot, 0.85 -> 0.81 ms at eight, CUDA events).
// QLMB_PDL=0 turns the attribute off everywhere (the instructions are then no-ops).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdl_enabled(void);                                  // qlmb_runtime.cu
template <typename... KArgs, typename... Args>
static inline cudaError_t pdl_launch(bool early, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = (early && pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- device helpers --------------------------------------------------------
// splitmix64 finaliser, low 32 bits (reference qlm.cuh:78-82).
__host__ __device__ __forceinline__ uint32_t hash_u32(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return (uint32_t)(x ^ (x >> 31));
}
#define QLMB_HASH_I 0x2545F4914F6CDD1DULL   // element-index multiplier (qlm.cuh:85)
#define QLMB_HASH_T 0x9E3779B97F4A7C15ULL   // step multiplier

__host__ __device__ __forceinline__ int clampi(int v, int lo, int hi)
{
    return v < lo ? lo : (v > hi ? hi : v);
}

// A kernel that finds an argument it must not act on (a cache position outside the cache) records code 201 with the
// site, the slot and the value in the device error word and skips the access; qlmb_check_device reports it.
__device__ __forceinline__ void report_bad_index(int *errword, int site, int slot, int value)
{
    if (errword && atomicCAS(errword, 0, 201) == 0) { errword[1] = site; errword[2] = slot; errword[3] = value; }
}

// digit i of a digit array (qlm.cuh:96-101)
__device__ __forceinline__ int digit_at(const int8_t *d, uint64_t i, int packed)
{
    if (!packed) return d[i];
    unsigned b = (uint8_t)d[i >> 1];
    int v = (i & 1) ? (int)(b >> 4) : (int)(b & 15u);
    return v > 7 ? v - 16 : v;
}

// span that owns group gi (qlm.cuh:113-117): returns index, fills start/len
__device__ __forceinline__ int locate_group(const qlmb_span *sp, int nspan, int gi, int group,
                                            uint64_t &j0, int &n)
{
    // spans are appended in ascending group order (qlm_add_span, qlm.cuh:448-455): bisect for the last
    // span that starts at or before gi; a table that is not ascending falls back to the linear scan
    int lo = 0, hi = nspan - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((int)sp[mid].gi0 <= gi) lo = mid; else hi = mid - 1;
    }
    int si = lo;
    if (!(gi >= sp[si].gi0 && gi < sp[si].gi0 + sp[si].ngrp)) {
        si = 0;
        for (int i = 0; i < nspan; i++)
            if (gi >= sp[i].gi0 && gi < sp[i].gi0 + sp[i].ngrp) { si = i; break; }
    }
    j0 = (uint64_t)(gi - sp[si].gi0) * (uint64_t)group;
    uint64_t left = sp[si].n - j0;
    n = (int)(left < (uint64_t)group ? left : (uint64_t)group);
    return si;
}

}  // namespace qlmb
