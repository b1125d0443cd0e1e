// tcgen05 GEMM engine for sm_100a: persistent, warp-specialised CTAs.
//
// A CTA tile is 256 rows x 128 columns: two M=128 MMAs per 16-deep step share
// one B slice, so every expanded weight element feeds 512 flops.
//
//   warp 0      TMA producer   activations (bf16, 128-byte swizzle) and packed
//                              4-bit code tiles into shared-memory rings
//   warp 1      MMA issuer     tcgen05.mma, fp32 accumulators in TMEM (two
//                              accumulator buffers of 2 x 128 columns, so the
//                              epilogue of tile i overlaps the main loop of i+1)
//   warps 2-9   epilogue       tcgen05.ld -> registers -> fused epilogue ->
//                              swizzled staging -> whole-row stores to HBM
//   warps 10-17 dequant        codes (shared) -> registers -> bf16 x scale ->
//                              UMMA-canonical swizzled B tile (shared)
//
// The weights never exist in HBM as bf16 or fp32: each 64-deep slice of the B
// tile is expanded from its nibbles once per CTA tile and consumed from shared
// memory by the tensor core.  Every mbarrier wait is bounded: when a wait runs
// out the CTA raises an abort flag, records the site in the device error word
// and every role leaves its loop, so a broken pipeline ends the kernel instead
// of hanging the GPU.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <cuda_bf16.h>
#include "qlmb_common.cuh"
#include "qlmb_gemm.cuh"
#include "qlmb_tc.cuh"

namespace qlmb {

constexpr int BM = 128;           // rows per MMA (UMMA M); a CTA tile has MH such halves
constexpr int MH = 2;
constexpr int BN = 128;           // accumulator columns per tile
constexpr int BK = 64;            // contraction elements per pipeline stage (one 128-byte swizzle row)
constexpr int DQ_WARPS = 8;
constexpr int EPI_WARPS = 8;
constexpr int A_STAGE_BYTES = MH * BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int C_STAGE_BYTES = BN * BK / 2;

struct GemmParams {
    alignas(64) CUtensorMap a_map[2];
    alignas(64) CUtensorMap w_map[2];
    alignas(64) CUtensorMap o_map[3];      // bf16 outputs written by bulk tensor stores (boxes of 32 rows x 64 columns)
    alignas(64) CUtensorMap i_map[2];      // SwiGLU backward: stashed gate / up, boxes of 32 rows x 32 columns
    int o_tma;                             // 1: o_map (and i_map) valid
    const float *scales[2];
    int nseg, ksteps;
    int M, N, E;
    int tiles_m, tiles_n;
    int w_rows, w_cols;
    const int *tile_info, *ntiles_dev, *off;
    void *out; int out_dtype; long long ldo;
    const void *resid; float beta;
    bf16 *gp, *up, *ap, *dgp, *dup;
    const int *scatter_perm; int scatter_kn; bf16 *scatter_out[8];
    int *errword;
};

// ------------------------------------------------------------------ dequant
// Eight two's-complement nibbles -> eight bf16 (value * scale), in element order.
// nibble ^ 8 is the value + 8 in 0..15; OR-ing it under the bf16 exponent of 128
// gives 136 + value exactly, so (x - 136) * scale needs no int->float convert.
__device__ __forceinline__ uint4 dequant8(uint32_t w, __nv_bfloat162 s2)
{
    w ^= 0x88888888u;
    uint32_t q[4];
    q[0] = (w & 0x000F000Fu) | 0x43004300u;            // elements (0,4)
    q[1] = ((w >> 4) & 0x000F000Fu) | 0x43004300u;     // (1,5)
    q[2] = ((w >> 8) & 0x000F000Fu) | 0x43004300u;     // (2,6)
    q[3] = ((w >> 12) & 0x000F000Fu) | 0x43004300u;    // (3,7)
    const uint32_t k136 = 0x43084308u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162 *>(&q[i]);
        x = __hmul2(__hsub2(x, *reinterpret_cast<const __nv_bfloat162 *>(&k136)), s2);
        q[i] = *reinterpret_cast<uint32_t *>(&x);
    }
    uint4 o;
    o.x = __byte_perm(q[0], q[1], 0x5410);   // (0,1)
    o.y = __byte_perm(q[2], q[3], 0x5410);   // (2,3)
    o.z = __byte_perm(q[0], q[1], 0x7632);   // (4,5)
    o.w = __byte_perm(q[2], q[3], 0x7632);   // (6,7)
    return o;
}

// The same expansion without the final reordering: the eight results stay in the order
// (0,4,1,5,2,6,3,7), i.e. position c of each group of eight holds element PERM8[c].  Used where the
// eight elements run along the OUTPUT columns (codes [K][N]): the epilogue reads accumulator column
// 8m + c as output column 8m + PERM8[c], which costs nothing, and four PRMTs per word are saved.
// The nibble extraction folds the sign flip and the exponent into one LOP3 per pair:
// bit = mask ? (cst ? ~w : w) : cst, with mask 0x000F000F and cst 0x43084308 (0x4300 | the flipped bit 3).
__device__ __forceinline__ uint32_t nib_pair(uint32_t w)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43084308, 0x6A;" : "=r"(r) : "r"(w));
    return r;
}
__device__ __forceinline__ uint4 dequant8_perm(uint32_t w, __nv_bfloat162 s2)
{
    uint32_t q[4] = {nib_pair(w), nib_pair(w >> 4), nib_pair(w >> 8), nib_pair(w >> 12)};
    const uint32_t k136 = 0x43084308u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162 *>(&q[i]);
        x = __hmul2(__hsub2(x, *reinterpret_cast<const __nv_bfloat162 *>(&k136)), s2);
        q[i] = *reinterpret_cast<uint32_t *>(&x);
    }
    return make_uint4(q[0], q[1], q[2], q[3]);
}
// accumulator column that holds output column i of a tile expanded with dequant8_perm
template <bool NPERM>
__device__ __forceinline__ constexpr int acc_col(int i)
{
    return NPERM ? ((i & ~7) | (((i & 7) >> 2) | ((i & 3) << 1))) : i;
}

// ------------------------------------------------------------------ epilogue staging
// Lane r of a warp owns tile row r and holds VECS 16-byte vectors of it (a row
// piece of 32, 64 or 128 bytes).  The piece goes through a swizzled 4 KiB buffer so
// that each global access instruction covers whole row pieces: 4 rows x 128 B,
// 8 rows x 64 B or 16 rows x 32 B.  Both the lane-per-row and the transposed access pattern are
// free of shared-memory bank conflicts.
template <int VECS>
__device__ __forceinline__ int stage_slot(int r, int c)
{
    return VECS == 8 ? (c ^ (r & 7)) : VECS == 4 ? (c ^ ((r >> 1) & 3)) : (c ^ ((r >> 2) & 1));
}

template <int VECS>
__device__ __forceinline__ void warp_store_rows(uint8_t *stage, const uint4 *v, int lane, uint8_t *g0, long long pitch, int valid_rows)
{
    constexpr int RB = VECS * 16;
#pragma unroll
    for (int c = 0; c < VECS; c++) *reinterpret_cast<uint4 *>(stage + lane * RB + stage_slot<VECS>(lane, c) * 16) = v[c];
    __syncwarp();
    constexpr int RPI = 32 / VECS;
#pragma unroll
    for (int j = 0; j < VECS; j++) {
        const int r = j * RPI + lane / VECS, c = lane % VECS;
        uint4 x = *reinterpret_cast<const uint4 *>(stage + r * RB + stage_slot<VECS>(r, c) * 16);
        if (r < valid_rows) *reinterpret_cast<uint4 *>(g0 + (long long)r * pitch + c * 16) = x;
    }
    __syncwarp();
}

template <int VECS>
__device__ __forceinline__ void warp_load_rows(uint8_t *stage, uint4 *v, int lane, const uint8_t *g0, long long pitch, int valid_rows)
{
    constexpr int RB = VECS * 16;
    constexpr int RPI = 32 / VECS;
#pragma unroll
    for (int j = 0; j < VECS; j++) {
        const int r = j * RPI + lane / VECS, c = lane % VECS;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (r < valid_rows) x = *reinterpret_cast<const uint4 *>(g0 + (long long)r * pitch + c * 16);
        *reinterpret_cast<uint4 *>(stage + r * RB + stage_slot<VECS>(r, c) * 16) = x;
    }
    __syncwarp();
#pragma unroll
    for (int c = 0; c < VECS; c++) v[c] = *reinterpret_cast<const uint4 *>(stage + lane * RB + stage_slot<VECS>(lane, c) * 16);
    __syncwarp();
}

// 32 rows x 128 bytes in a 4 KiB block: 16-byte vector c of row r sits at a swizzled slot, so
// both "lane = row" accesses and "8 lanes = one whole row" accesses are free of bank conflicts.
__device__ __forceinline__ uint4 *blk_vec(uint8_t *blk, int r, int c)
{
    return reinterpret_cast<uint4 *>(blk + r * 128 + ((c ^ (r & 7)) << 4));
}
// the block to / from global rows of 128 bytes: every access instruction covers 4 whole rows
__device__ __forceinline__ void blk_store(uint8_t *blk, int lane, uint8_t *g0, long long pitch, int valid_rows)
{
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int r = j * 4 + (lane >> 3), c = lane & 7;
        const uint4 x = *blk_vec(blk, r, c);
        if (r < valid_rows) *reinterpret_cast<uint4 *>(g0 + (long long)r * pitch + c * 16) = x;
    }
    __syncwarp();
}
__device__ __forceinline__ void blk_load(uint8_t *blk, int lane, const uint8_t *g0, long long pitch, int valid_rows)
{
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int r = j * 4 + (lane >> 3), c = lane & 7;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (r < valid_rows) x = __ldg(reinterpret_cast<const uint4 *>(g0 + (long long)r * pitch + c * 16));
        *blk_vec(blk, r, c) = x;
    }
}
// the block to scattered global rows: lane r's destination row pointer (or nullptr) is `mine`
__device__ __forceinline__ void blk_store_scattered(uint8_t *blk, int lane, bf16 *mine, int col)
{
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int r = j * 4 + (lane >> 3), c = lane & 7;
        const uint4 x = *blk_vec(blk, r, c);
        bf16 *dst = reinterpret_cast<bf16 *>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine), r));
        if (dst) *reinterpret_cast<uint4 *>(dst + col + c * 8) = x;
    }
    __syncwarp();
}
// The block layout is the 128-byte swizzle of a bulk tensor copy, so a staged block can leave as
// one asynchronous store issued by lane 0.  blk_reuse() must precede the next write to the block.
__device__ __forceinline__ void blk_store_bulk(uint8_t *blk, int lane, const CUtensorMap *map, int x, int y)
{
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) { tma_store_2d(map, smem_u32(blk), x, y); bulk_commit(); }
}
__device__ __forceinline__ void blk_reuse(int lane)
{
    if (lane == 0) bulk_wait_read();
    __syncwarp();
}
// staging bytes per epilogue warp
__host__ __device__ constexpr int epi_stage_bytes(int epi) { return epi == EPI_SWIGLU_BWD ? 8192 : 4096; }

struct Ring {
    int idx; uint32_t phase;
    __device__ __forceinline__ void next(int n) { if (++idx == n) { idx = 0; phase ^= 1u; } }
};

// m0: first row of the tile; halves: how many 128-row halves carry rows (1 or 2)
struct TileInfo { int m0, n_t, e, ksteps, row0, halves; };

template <int SCHED>
__device__ __forceinline__ TileInfo decode_tile(const GemmParams &p, int tile, int ntr)
{
    TileInfo t;
    if (SCHED == SCHED_DENSE) {
        t.m0 = (tile % p.tiles_m) * (MH * BM); t.n_t = tile / p.tiles_m; t.e = 0; t.ksteps = p.ksteps; t.row0 = 0;
        t.halves = (t.m0 + BM < p.M) ? 2 : 1;
    } else if (SCHED == SCHED_ROWS) {
        int rt = tile % ntr;
        int info = p.tile_info[rt];
        t.m0 = (info & 0xFFFFF) * BM; t.e = (info >> 20) & 0x1FF; t.halves = ((info >> 30) & 1) + 1;
        t.n_t = tile / ntr; t.ksteps = p.ksteps; t.row0 = 0;
    } else {
        int per = p.tiles_m * p.tiles_n;
        t.e = tile / per;
        int r = tile % per;
        t.m0 = (r % p.tiles_m) * (MH * BM); t.n_t = r / p.tiles_m;
        t.row0 = p.off[t.e];
        t.ksteps = (p.off[t.e + 1] - p.off[t.e]) / BK;
        t.halves = (t.m0 + BM < p.M) ? 2 : 1;
    }
    return t;
}

__device__ __forceinline__ float sigmoid_f(float z) { return __fdividef(1.0f, 1.0f + __expf(-z)); }

struct EpiCtx;
__device__ __forceinline__ bool swiglu_bwd_bulk(const GemmParams &p, uint8_t *stage, EpiCtx &ec, int lane, uint32_t tbase,
                                                long long rbase, long long col0);

// ------------------------------------------------------------------ fused epilogues
// One warp, 32 tile rows (lane = row) x 128 accumulator columns starting at TMEM
// address tbase; rbase = index of the warp's first row in the output, col0 = first
// output column.  EPI_SWIGLU reads 64 gate columns at tbase and 64 up columns at
// tbase + u_off and writes 64 activation columns.
template <int EPI, bool NPERM = false>
__device__ __forceinline__ void epilogue_rows(const GemmParams &p, uint8_t *stage, EpiCtx &ec, int lane, uint32_t tbase,
                                              long long rbase, long long col0, int valid, bool have_acc, uint32_t u_off)
{
    static_assert(!(EPI == EPI_SWIGLU_BWD && NPERM), "the SwiGLU-backward epilogue reads accumulator columns in place");
    if (EPI == EPI_SWIGLU_BWD && p.o_tma) { swiglu_bwd_bulk(p, stage, ec, lane, tbase, rbase, col0); return; }
    if (EPI == EPI_STORE && p.out_dtype == QLMB_BF16 && !p.resid && p.beta == 0.0f) {
        // plain bf16 store: two blocks of 64 columns, each written with whole 128-byte rows
        bf16 *mine = nullptr;                                // scattered form: this lane's row destination
        if (p.scatter_perm && lane < valid) {
            const int g = p.scatter_perm[rbase + lane];
            if (g >= 0) mine = p.scatter_out[g / p.scatter_kn] + (size_t)(g % p.scatter_kn) * p.ldo;
        }
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            if (p.o_tma && !p.scatter_perm) blk_reuse(lane);
#pragma unroll 1
            for (int cc = 0; cc < 2; cc++) {
                uint32_t v[32];
                tmem_ld32(tbase + half * 64 + cc * 32, v);
                tmem_ld_wait();
                uint4 w[4];
                __nv_bfloat162 *hw = reinterpret_cast<__nv_bfloat162 *>(w);
#pragma unroll
                for (int i = 0; i < 16; i++)
                    hw[i] = have_acc ? __floats2bfloat162_rn(__uint_as_float(v[acc_col<NPERM>(2 * i)]), __uint_as_float(v[acc_col<NPERM>(2 * i + 1)])) : __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
                for (int k = 0; k < 4; k++) *blk_vec(stage, lane, cc * 4 + k) = w[k];
            }
            if (p.scatter_perm) blk_store_scattered(stage, lane, mine, (int)(col0 + half * 64));
            else if (p.o_tma) blk_store_bulk(stage, lane, &p.o_map[0], (int)(col0 + half * 64), (int)rbase);
            else blk_store(stage, lane, reinterpret_cast<uint8_t *>((bf16 *)p.out + rbase * p.ldo + col0 + half * 64), p.ldo * 2, valid);
        }
    } else if ((EPI == EPI_STORE || EPI == EPI_ACCUM) && p.out_dtype == QLMB_F32 && p.o_tma) {
        // fp32 output through bulk tensor copies: 32 rows x 32 columns (128-byte rows) per block;
        // beta = 1 adds into the tensor with a bulk reduction, so the old values are never read here
        if (!(p.beta != 0.0f && !have_acc)) {
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tbase + c * 32, v);
                tmem_ld_wait();
                blk_reuse(lane);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    uint4 q = have_acc ? make_uint4(v[acc_col<NPERM>(4 * k)], v[acc_col<NPERM>(4 * k + 1)], v[acc_col<NPERM>(4 * k + 2)], v[acc_col<NPERM>(4 * k + 3)]) : make_uint4(0, 0, 0, 0);
                    *blk_vec(stage, lane, k) = q;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (p.beta != 0.0f) tma_reduce_add_2d(&p.o_map[0], smem_u32(stage), (int)(col0 + c * 32), (int)rbase);
                    else tma_store_2d(&p.o_map[0], smem_u32(stage), (int)(col0 + c * 32), (int)rbase);
                    bulk_commit();
                }
            }
        }
    } else if (EPI == EPI_STORE || EPI == EPI_ACCUM) {
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
            uint32_t v[32];
            tmem_ld32(tbase + c * 32, v);
            tmem_ld_wait();
            const long long o = rbase * p.ldo + col0 + c * 32;
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; i++) f[i] = have_acc ? __uint_as_float(v[acc_col<NPERM>(i)]) : 0.0f;
            if (p.out_dtype == QLMB_F32) {
                if (p.resid) {
                    uint4 r[8];
                    warp_load_rows<8>(stage, r, lane, reinterpret_cast<const uint8_t *>((const float *)p.resid + o), p.ldo * 4, valid);
                    const float *rf = reinterpret_cast<const float *>(r);
#pragma unroll
                    for (int i = 0; i < 32; i++) f[i] += rf[i];
                }
                if (p.beta != 0.0f) {
                    uint4 r[8];
                    warp_load_rows<8>(stage, r, lane, reinterpret_cast<const uint8_t *>((const float *)p.out + o), p.ldo * 4, valid);
                    const float *rf = reinterpret_cast<const float *>(r);
#pragma unroll
                    for (int i = 0; i < 32; i++) f[i] += p.beta * rf[i];
                }
                warp_store_rows<8>(stage, reinterpret_cast<const uint4 *>(f), lane, reinterpret_cast<uint8_t *>((float *)p.out + o), p.ldo * 4, valid);
            } else {
                if (p.resid) {
                    uint4 r[4];
                    warp_load_rows<4>(stage, r, lane, reinterpret_cast<const uint8_t *>((const bf16 *)p.resid + o), p.ldo * 2, valid);
                    const __nv_bfloat162 *hh = reinterpret_cast<const __nv_bfloat162 *>(r);
#pragma unroll
                    for (int i = 0; i < 16; i++) { float2 g = __bfloat1622float2(hh[i]); f[2 * i] += g.x; f[2 * i + 1] += g.y; }
                }
                if (p.beta != 0.0f) {
                    uint4 r[4];
                    warp_load_rows<4>(stage, r, lane, reinterpret_cast<const uint8_t *>((const bf16 *)p.out + o), p.ldo * 2, valid);
                    const __nv_bfloat162 *hh = reinterpret_cast<const __nv_bfloat162 *>(r);
#pragma unroll
                    for (int i = 0; i < 16; i++) { float2 g = __bfloat1622float2(hh[i]); f[2 * i] += p.beta * g.x; f[2 * i + 1] += p.beta * g.y; }
                }
                uint4 w[4];
                __nv_bfloat162 *hw = reinterpret_cast<__nv_bfloat162 *>(w);
#pragma unroll
                for (int i = 0; i < 16; i++) hw[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                warp_store_rows<4>(stage, w, lane, reinterpret_cast<uint8_t *>((bf16 *)p.out + o), p.ldo * 2, valid);
            }
        }
    } else if (EPI == EPI_SWIGLU) {
        // three passes over the warp's 64 activation columns (activation, gate, up), each staged
        // as one block and written with whole 128-byte rows; the accumulators are re-read from
        // TMEM per pass, which costs less than holding them
        const long long o = rbase * p.ldo + col0;
#pragma unroll 1
        for (int pass = 0; pass < 3; pass++) {
            if (p.o_tma) blk_reuse(lane);
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t g[16], u[16];
                uint4 w[2];
                __nv_bfloat162 *hw = reinterpret_cast<__nv_bfloat162 *>(w);
                if (pass == 0) {
                    tmem_ld16(tbase + c * 16, g);
                    tmem_ld16(tbase + u_off + c * 16, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        float g0 = __uint_as_float(g[acc_col<NPERM>(2 * k)]), g1 = __uint_as_float(g[acc_col<NPERM>(2 * k + 1)]);
                        float u0 = __uint_as_float(u[acc_col<NPERM>(2 * k)]), u1 = __uint_as_float(u[acc_col<NPERM>(2 * k + 1)]);
                        hw[k] = __floats2bfloat162_rn(g0 * sigmoid_f(g0) * u0, g1 * sigmoid_f(g1) * u1);
                    }
                } else {
                    tmem_ld16(tbase + (pass == 2 ? u_off : 0u) + c * 16, g);
                    tmem_ld_wait();
#pragma unroll
                    for (int k = 0; k < 8; k++) hw[k] = __floats2bfloat162_rn(__uint_as_float(g[acc_col<NPERM>(2 * k)]), __uint_as_float(g[acc_col<NPERM>(2 * k + 1)]));
                }
                *blk_vec(stage, lane, 2 * c) = w[0];
                *blk_vec(stage, lane, 2 * c + 1) = w[1];
            }
            bf16 *dst = pass == 0 ? p.ap : pass == 1 ? p.gp : p.up;
            if (p.o_tma) blk_store_bulk(stage, lane, &p.o_map[pass], (int)col0, (int)rbase);
            else blk_store(stage, lane, reinterpret_cast<uint8_t *>(dst + o), p.ldo * 2, valid);
        }
    } else {   // EPI_SWIGLU_BWD: accumulator = d(act); dg = da*u*silu'(g), du = da*silu(g)
        // Two groups of 64 columns.  The gate and up pieces of a group are staged as two blocks
        // (whole 128-byte rows), the results overwrite them in place and leave the same way.
        // Group 0 was staged by epilogue_prefetch before the accumulator was ready.
        const long long o0 = rbase * p.ldo + col0;
        const long long pitch = p.ldo * 2;
        uint8_t *bg = stage, *bu = stage + 4096;
#pragma unroll 1
        for (int grp = 0; grp < 2; grp++) {
            if (grp == 1) {
                if (p.o_tma) blk_reuse(lane);
                blk_load(bg, lane, reinterpret_cast<const uint8_t *>(p.gp + o0 + 64), pitch, valid);
                blk_load(bu, lane, reinterpret_cast<const uint8_t *>(p.up + o0 + 64), pitch, valid);
            }
            __syncwarp();
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[16];
                tmem_ld16(tbase + grp * 64 + c * 16, v);
                uint4 rg[2], ru[2], wdg[2], wdu[2];
#pragma unroll
                for (int k = 0; k < 2; k++) { rg[k] = *blk_vec(bg, lane, 2 * c + k); ru[k] = *blk_vec(bu, lane, 2 * c + k); }
                tmem_ld_wait();
                const __nv_bfloat162 *hg = reinterpret_cast<const __nv_bfloat162 *>(rg), *hu = reinterpret_cast<const __nv_bfloat162 *>(ru);
                __nv_bfloat162 *hdg = reinterpret_cast<__nv_bfloat162 *>(wdg), *hdu = reinterpret_cast<__nv_bfloat162 *>(wdu);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    float2 gg = __bfloat1622float2(hg[k]), uu = __bfloat1622float2(hu[k]);
                    float d0 = __uint_as_float(v[2 * k]), d1 = __uint_as_float(v[2 * k + 1]);
                    float s0 = sigmoid_f(gg.x), s1 = sigmoid_f(gg.y);
                    float dg0 = d0 * uu.x * (s0 + gg.x * s0 * (1.0f - s0)), dg1 = d1 * uu.y * (s1 + gg.y * s1 * (1.0f - s1));
                    float du0 = d0 * gg.x * s0, du1 = d1 * gg.y * s1;
                    hdg[k] = __floats2bfloat162_rn(dg0, dg1);
                    hdu[k] = __floats2bfloat162_rn(du0, du1);
                }
#pragma unroll
                for (int k = 0; k < 2; k++) { *blk_vec(bg, lane, 2 * c + k) = wdg[k]; *blk_vec(bu, lane, 2 * c + k) = wdu[k]; }
            }
            if (p.o_tma) {
                blk_store_bulk(bg, lane, &p.o_map[0], (int)(col0 + grp * 64), (int)rbase);
                blk_store_bulk(bu, lane, &p.o_map[1], (int)(col0 + grp * 64), (int)rbase);
            } else {
                blk_store(bg, lane, reinterpret_cast<uint8_t *>(p.dgp + o0 + grp * 64), pitch, valid);
                blk_store(bu, lane, reinterpret_cast<uint8_t *>(p.dup + o0 + grp * 64), pitch, valid);
            }
        }
    }
}

// Per-warp state of the SwiGLU-backward epilogue's input ring: two mbarriers (one per 4 KiB buffer)
// and the parity to wait for next on each.
struct EpiCtx { uint64_t *bar; uint32_t ph; };

// SwiGLU backward over bulk tensor copies: the warp's 128 columns are four groups of 32; a group's
// gate and up pieces (32 rows x 64 bytes each) arrive by TMA in one of two buffers, the results
// overwrite them in place and leave by TMA.  The load of group j+1 is issued before group j is
// computed, the load of the next tile's group 0 before its accumulator is ready.
__device__ __forceinline__ void swiglu_bwd_issue(const GemmParams &p, uint8_t *buf, uint64_t *bar, int lane, int x, int y)
{
    if (lane == 0) bulk_wait_read();                     // stores that still read this buffer
    __syncwarp();
    if (lane == 0) {
        mbar_expect_tx(smem_u32(bar), 4096);
        tma_load_2d(smem_u32(buf), &p.i_map[0], smem_u32(bar), x, y);
        tma_load_2d(smem_u32(buf + 2048), &p.i_map[1], smem_u32(bar), x, y);
    }
}
__device__ __forceinline__ bool swiglu_bwd_bulk(const GemmParams &p, uint8_t *stage, EpiCtx &ec, int lane, uint32_t tbase,
                                                long long rbase, long long col0)
{
#pragma unroll 1
    for (int j = 0; j < 4; j++) {
        const int b = j & 1;
        uint8_t *bg = stage + b * 4096, *bu = bg + 2048;
        if (j < 3) swiglu_bwd_issue(p, stage + (b ^ 1) * 4096, ec.bar + (b ^ 1), lane, (int)(col0 + (j + 1) * 32), (int)rbase);
        bool ok = false;
        for (uint32_t i = 0; i < WAIT_LIMIT && !ok; i++) ok = mbar_try(smem_u32(ec.bar + b), (ec.ph >> b) & 1u);
        if (!ok) { if (p.errword && atomicCAS(p.errword, 0, 202) == 0) { p.errword[1] = 30 + j; p.errword[2] = (int)blockIdx.x; } return false; }
        ec.ph ^= 1u << b;
#pragma unroll 1
        for (int c = 0; c < 2; c++) {
            uint32_t v[16];
            tmem_ld16(tbase + j * 32 + c * 16, v);
            uint4 rg[2], ru[2], wdg[2], wdu[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                rg[k] = *reinterpret_cast<const uint4 *>(bg + lane * 64 + stage_slot<4>(lane, 2 * c + k) * 16);
                ru[k] = *reinterpret_cast<const uint4 *>(bu + lane * 64 + stage_slot<4>(lane, 2 * c + k) * 16);
            }
            tmem_ld_wait();
            const __nv_bfloat162 *hg = reinterpret_cast<const __nv_bfloat162 *>(rg), *hu = reinterpret_cast<const __nv_bfloat162 *>(ru);
            __nv_bfloat162 *hdg = reinterpret_cast<__nv_bfloat162 *>(wdg), *hdu = reinterpret_cast<__nv_bfloat162 *>(wdu);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                float2 gg = __bfloat1622float2(hg[k]), uu = __bfloat1622float2(hu[k]);
                float d0 = __uint_as_float(v[2 * k]), d1 = __uint_as_float(v[2 * k + 1]);
                float s0 = sigmoid_f(gg.x), s1 = sigmoid_f(gg.y);
                float dg0 = d0 * uu.x * (s0 + gg.x * s0 * (1.0f - s0)), dg1 = d1 * uu.y * (s1 + gg.y * s1 * (1.0f - s1));
                float du0 = d0 * gg.x * s0, du1 = d1 * gg.y * s1;
                hdg[k] = __floats2bfloat162_rn(dg0, dg1);
                hdu[k] = __floats2bfloat162_rn(du0, du1);
            }
#pragma unroll
            for (int k = 0; k < 2; k++) {
                *reinterpret_cast<uint4 *>(bg + lane * 64 + stage_slot<4>(lane, 2 * c + k) * 16) = wdg[k];
                *reinterpret_cast<uint4 *>(bu + lane * 64 + stage_slot<4>(lane, 2 * c + k) * 16) = wdu[k];
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(&p.o_map[0], smem_u32(bg), (int)(col0 + j * 32), (int)rbase);
            tma_store_2d(&p.o_map[1], smem_u32(bu), (int)(col0 + j * 32), (int)rbase);
            bulk_commit();
        }
    }
    return true;
}

// Work an epilogue warp can do for its next tile before that tile's accumulator is complete.
template <int EPI>
__device__ __forceinline__ void epilogue_prefetch(const GemmParams &p, uint8_t *stage, EpiCtx &ec, int lane, long long rbase, long long col0, int valid)
{
    if (EPI == EPI_SWIGLU_BWD && p.o_tma) {
        swiglu_bwd_issue(p, stage, ec.bar, lane, (int)col0, (int)rbase);
    } else if (EPI == EPI_SWIGLU_BWD) {
        const long long o0 = rbase * p.ldo + col0;
        if (p.o_tma) blk_reuse(lane);
        blk_load(stage, lane, reinterpret_cast<const uint8_t *>(p.gp + o0), p.ldo * 2, valid);
        blk_load(stage + 4096, lane, reinterpret_cast<const uint8_t *>(p.up + o0), p.ldo * 2, valid);
    }
}

// ------------------------------------------------------------------ the kernel
template <int BMODE, int EPI, int SCHED>
__global__ void __launch_bounds__((BMODE == B_DEQ_MN || BMODE == B_DEQ_K) ? 576 : 320, 1)
k_gemm(const __grid_constant__ GemmParams p)
{
    constexpr bool DEQ = (BMODE == B_DEQ_MN || BMODE == B_DEQ_K);
    constexpr bool DUAL = (EPI == EPI_SWIGLU);           // B tile = [64 W1 columns | 64 W3 columns]
    constexpr int NSA = DEQ ? 3 : 4, NSB = DEQ ? 3 : 4, NSC = 4;
    constexpr uint32_t IDESC = make_idesc(BM, BN, BMODE == AB_TMA_MN ? 1 : 0, (BMODE == B_DEQ_MN || BMODE == AB_TMA_MN) ? 1 : 0);
    constexpr uint32_t ACC_COLS = MH * BN;               // one accumulator buffer
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem;
    uint8_t *sB = sA + NSA * A_STAGE_BYTES;
    uint8_t *sC = sB + NSB * B_STAGE_BYTES;
    uint8_t *sE = sC + (DEQ ? NSC * C_STAGE_BYTES : 0);       // 8 epilogue warps x 4 KiB staging
    uint64_t *bars = reinterpret_cast<uint64_t *>(sE + EPI_WARPS * epi_stage_bytes(EPI));
    uint64_t *full_a = bars, *empty_a = full_a + NSA, *full_b = empty_a + NSA, *empty_b = full_b + NSB;
    uint64_t *full_c = empty_b + NSB, *empty_c = full_c + NSC, *tmem_full = empty_c + NSC, *tmem_empty = tmem_full + 2;
    uint64_t *spare = tmem_empty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(spare + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSA; i++) { mbar_init(smem_u32(&full_a[i]), 1); mbar_init(smem_u32(&empty_a[i]), 1); }
        for (int i = 0; i < NSB; i++) { mbar_init(smem_u32(&full_b[i]), DEQ ? DQ_WARPS : 1); mbar_init(smem_u32(&empty_b[i]), 1); }
        for (int i = 0; i < NSC; i++) { mbar_init(smem_u32(&full_c[i]), 1); mbar_init(smem_u32(&empty_c[i]), DQ_WARPS); }
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&tmem_full[i]), 1); mbar_init(smem_u32(&tmem_empty[i]), EPI_WARPS); }
        mbar_init(smem_u32(spare), 1);
        for (int i = 0; i < 2 * EPI_WARPS; i++) mbar_init(smem_u32(bars + 48 + i), 1);   // epilogue input rings
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int ntr = (SCHED == SCHED_ROWS) ? *p.ntiles_dev : 0;
    const int total = (SCHED == SCHED_DENSE) ? p.tiles_m * p.tiles_n
                    : (SCHED == SCHED_ROWS) ? ntr * p.tiles_n : p.E * p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // =============================== TMA producer ===============================
        Ring ra = {0, 0}, rc = {0, 0};
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            TileInfo t = decode_tile<SCHED>(p, tile, ntr);
            for (int seg = 0; ok && seg < p.nseg; seg++) {
                for (int ks = 0; ks < t.ksteps; ks++) {
                    ok = mbar_wait(smem_u32(&empty_a[ra.idx]), ra.phase ^ 1u, abort_flag, p.errword, 1);
                    if (!ok) break;
                    if (lane == 0) {
                        uint32_t bar = smem_u32(&full_a[ra.idx]);
                        uint32_t dstA = smem_u32(sA + ra.idx * A_STAGE_BYTES);
                        if (BMODE == AB_TMA_MN) {
                            uint32_t dstB = smem_u32(sB + ra.idx * B_STAGE_BYTES);
                            int row = t.row0 + ks * BK;
                            mbar_expect_tx(bar, t.halves * (BM * BK * 2) + B_STAGE_BYTES);
                            for (int i = 0; i < 2 * t.halves; i++)
                                tma_load_2d(dstA + i * 8192, &p.a_map[0], bar, t.m0 + 64 * i, row);
#pragma unroll
                            for (int j = 0; j < BN / 64; j++)
                                tma_load_2d(dstB + j * 8192, &p.w_map[0], bar, t.n_t * BN + 64 * j, row);
                        } else {
                            mbar_expect_tx(bar, t.halves * (BM * BK * 2) + (BMODE == B_TMA_K ? B_STAGE_BYTES : 0));
                            for (int h = 0; h < t.halves; h++)
                                tma_load_2d(dstA + h * (BM * BK * 2), &p.a_map[seg], bar, ks * BK, t.m0 + h * BM);
                            if (BMODE == B_TMA_K)
                                tma_load_2d(smem_u32(sB + ra.idx * B_STAGE_BYTES), &p.w_map[seg], bar, ks * BK, t.n_t * BN);
                        }
                    }
                    __syncwarp();
                    ra.next(NSA);
                    if (DEQ) {
                        ok = mbar_wait(smem_u32(&empty_c[rc.idx]), rc.phase ^ 1u, abort_flag, p.errword, 2);
                        if (!ok) break;
                        if (lane == 0) {
                            uint32_t bar = smem_u32(&full_c[rc.idx]);
                            uint32_t dstC = smem_u32(sC + rc.idx * C_STAGE_BYTES);
                            mbar_expect_tx(bar, C_STAGE_BYTES);
                            if (BMODE == B_DEQ_MN) {
                                int row = t.e * p.w_rows + ks * BK;
                                if (DUAL) {
                                    tma_load_2d(dstC, &p.w_map[0], bar, t.n_t * (BN / 4), row);
                                    tma_load_2d(dstC + C_STAGE_BYTES / 2, &p.w_map[1], bar, t.n_t * (BN / 4), row);
                                } else {
                                    tma_load_2d(dstC, &p.w_map[seg], bar, t.n_t * (BN / 2), row);
                                }
                            } else {
                                tma_load_2d(dstC, &p.w_map[seg], bar, ks * (BK / 2), t.e * p.w_rows + t.n_t * BN);
                            }
                        }
                        __syncwarp();
                        rc.next(NSC);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        Ring ra = {0, 0}, rb = {0, 0};
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x, it++) {
            TileInfo t = decode_tile<SCHED>(p, tile, ntr);
            const int acc = it & 1;
            ok = mbar_wait(smem_u32(&tmem_empty[acc]), (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag, p.errword, 3);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)acc * ACC_COLS;
            uint32_t accumulate = 0;
            for (int seg = 0; ok && seg < p.nseg; seg++) {
                for (int ks = 0; ks < t.ksteps; ks++) {
                    ok = mbar_wait(smem_u32(&full_a[ra.idx]), ra.phase, abort_flag, p.errword, 4);
                    if (!ok) break;
                    const int sb = DEQ ? rb.idx : ra.idx;
                    if (DEQ) {
                        ok = mbar_wait(smem_u32(&full_b[rb.idx]), rb.phase, abort_flag, p.errword, 5);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t a0 = smem_u32(sA + ra.idx * A_STAGE_BYTES);
                        const uint32_t b0 = smem_u32(sB + sb * B_STAGE_BYTES);
#pragma unroll
                        for (int k16 = 0; k16 < BK / 16; k16++) {
                            uint64_t bd = (BMODE == B_DEQ_MN || BMODE == AB_TMA_MN) ? make_desc(b0 + k16 * 2048, 8192, 1024)
                                                                                    : make_desc(b0 + k16 * 32, 16, 1024);
                            for (int h = 0; h < t.halves; h++) {
                                uint64_t ad = (BMODE == AB_TMA_MN) ? make_desc(a0 + h * 16384 + k16 * 2048, 8192, 1024)
                                                                   : make_desc(a0 + h * 16384 + k16 * 32, 16, 1024);
                                tc_mma_bf16(tmem_d + (uint32_t)h * BN, ad, bd, IDESC, accumulate);
                            }
                            accumulate = 1;
                        }
                        tc_commit(smem_u32(&empty_a[ra.idx]));
                        if (DEQ) tc_commit(smem_u32(&empty_b[rb.idx]));
                    }
                    __syncwarp();
                    accumulate = 1;
                    ra.next(NSA);
                    if (DEQ) rb.next(NSB);
                }
            }
            if (ok) {
                if (lane == 0) tc_commit(smem_u32(&tmem_full[acc]));
                __syncwarp();
            }
        }
        if (*abort_flag) {   // aborting: let issued MMAs retire (bounded) before TMEM is released
            if (lane == 0) tc_commit(smem_u32(spare));
            __syncwarp();
            for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(smem_u32(spare), 0); i++) {}
        }
    } else if (warp < 2 + EPI_WARPS) {
        // =============================== epilogue ===============================
        // Warp (q, h): q = TMEM lane quarter it may read (= warp id mod 4), h = which
        // 128-row half of the tile.  A lane holds one tile row; element-wise work runs in
        // registers, then the row pieces go through a swizzled 4 KiB staging buffer so that
        // every global store instruction writes whole row pieces.
        const int q = warp & 3, h = (warp - 2) >> 2;
        uint8_t *stage = sE + (warp - 2) * epi_stage_bytes(EPI);
        EpiCtx ec = {bars + 48 + 2 * (warp - 2), 0u};
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x, it++) {
            TileInfo t = decode_tile<SCHED>(p, tile, ntr);
            const int acc = it & 1;
            const long long row0 = (long long)t.m0 + h * BM + q * 32;                // first row of this warp
            int valid = 32;
            if (SCHED != SCHED_ROWS) { long long left = (long long)p.M - row0; valid = left < 0 ? 0 : (left < 32 ? (int)left : 32); }
            const long long rbase = (SCHED == SCHED_GROUPK) ? ((long long)t.e * p.M + row0) : row0;
            const long long col0 = (long long)t.n_t * (EPI == EPI_SWIGLU ? BN / 2 : BN);
            if (h < t.halves) epilogue_prefetch<EPI>(p, stage, ec, lane, rbase, col0, valid);
            ok = mbar_wait(smem_u32(&tmem_full[acc]), ((uint32_t)it >> 1) & 1u, abort_flag, p.errword, 6);
            if (!ok) break;
            tc_fence_after();
            if (h < t.halves) {
                const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * ACC_COLS + (uint32_t)h * BN;
                const bool have_acc = (SCHED != SCHED_GROUPK) || t.ksteps > 0;
                epilogue_rows<EPI>(p, stage, ec, lane, tbase, rbase, col0, valid, have_acc, BN / 2);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tmem_empty[acc]));
        }
        if (lane == 0) bulk_wait_all();                  // outstanding bulk stores of this warp
    } else if (DEQ) {
        // =============================== dequant warps ===============================
        const int dw = warp - (2 + EPI_WARPS);
        constexpr int ITERS = (C_STAGE_BYTES / 4) / (DQ_WARPS * 32);
        Ring rc = {0, 0}, rb = {0, 0};
        bool ok = true;
        // per-lane constants: where each of its code words lands in a B stage, and which
        // (row, column) of the stored code matrix it comes from (for the scale lookup)
        uint32_t dst_off[ITERS];
        int srow[ITERS], scol[ITERS];
        bool second[ITERS];
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            int wi = (i * DQ_WARPS + dw) * 32 + lane;
            if (BMODE == B_DEQ_MN) {
                int k, c, nb;
                if (DUAL) { int half = wi / (BN * 4); int r = wi % (BN * 4); k = r / (BN / 16); c = r % (BN / 16); nb = half * (BN / 128) + c / 8; second[i] = half != 0; }
                else { constexpr int WPR = BN / 8; k = wi / WPR; c = wi % WPR; nb = c / 8; second[i] = false; }
                dst_off[i] = (uint32_t)(nb * 8192 + (k >> 3) * 1024 + (k & 7) * 128 + (((c & 7) ^ (k & 7)) << 4));
                srow[i] = k; scol[i] = c * 8;
            } else {
                int n = wi / 8, c = wi % 8;
                dst_off[i] = (uint32_t)((n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4));
                srow[i] = n; scol[i] = c * 8; second[i] = false;
            }
        }
        const int gpr = p.w_cols / 128;                  // scale groups per stored row
        const float *sc0 = p.scales[0], *sc1 = p.scales[1];
        for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            TileInfo t = decode_tile<SCHED>(p, tile, ntr);
            for (int seg = 0; ok && seg < p.nseg; seg++) {
                const float *sseg = seg ? sc1 : sc0;
                // index of the scale of word i at step ks = sbase[i] + ks * sstep
                int sbase[ITERS], sstep;
#pragma unroll
                for (int i = 0; i < ITERS; i++) {
                    if (BMODE == B_DEQ_MN) {
                        int ncol = DUAL ? (t.n_t * (BN / 2) + scol[i]) : (t.n_t * BN + scol[i]);
                        sbase[i] = (t.e * p.w_rows + srow[i]) * gpr + ncol / 128;
                    } else {
                        sbase[i] = (t.e * p.w_rows + t.n_t * BN + srow[i]) * gpr;
                    }
                }
                sstep = (BMODE == B_DEQ_MN) ? BK * gpr : 0;
                float cur[ITERS], nxt[ITERS];
#pragma unroll
                for (int i = 0; i < ITERS; i++) {
                    const float *sp = (DUAL && second[i]) ? sc1 : sseg;
                    cur[i] = __ldg(sp + sbase[i]);
                }
                for (int ks = 0; ks < t.ksteps; ks++) {
                    // scales of the next step are requested before this step's tile is awaited
                    if (ks + 1 < t.ksteps) {
#pragma unroll
                        for (int i = 0; i < ITERS; i++) {
                            const float *sp = (DUAL && second[i]) ? sc1 : sseg;
                            int idx = (BMODE == B_DEQ_MN) ? sbase[i] + (ks + 1) * sstep : sbase[i] + ((ks + 1) * BK) / 128;
                            nxt[i] = __ldg(sp + idx);
                        }
                    }
                    ok = mbar_wait(smem_u32(&full_c[rc.idx]), rc.phase, abort_flag, p.errword, 7);
                    if (!ok) break;
                    const uint32_t *cw = reinterpret_cast<const uint32_t *>(sC + rc.idx * C_STAGE_BYTES);
                    uint32_t w[ITERS];
#pragma unroll
                    for (int i = 0; i < ITERS; i++) w[i] = cw[(i * DQ_WARPS + dw) * 32 + lane];
                    ok = mbar_wait(smem_u32(&empty_b[rb.idx]), rb.phase ^ 1u, abort_flag, p.errword, 8);
                    if (!ok) break;
                    uint8_t *bdst = sB + rb.idx * B_STAGE_BYTES;
#pragma unroll
                    for (int i = 0; i < ITERS; i++)
                        *reinterpret_cast<uint4 *>(bdst + dst_off[i]) = dequant8(w[i], __float2bfloat162_rn(cur[i]));
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(smem_u32(&full_b[rb.idx])); mbar_arrive(smem_u32(&empty_c[rc.idx])); }
                    rc.next(NSC);
                    rb.next(NSB);
#pragma unroll
                    for (int i = 0; i < ITERS; i++) cur[i] = nxt[i];
                }
            }
        }
    }

    // =============================== teardown ===============================
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace qlmb

#include "qlmb_gemm_pair.cuh"

namespace qlmb {

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int load_encode(void)
{
    if (g_encode) return QLMB_OK;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (!fn || qres != cudaDriverEntryPointSuccess) { set_error("cuTensorMapEncodeTiled not available from this driver"); return QLMB_E_CUDA; }
    g_encode = (EncodeTiledFn)fn;
    return QLMB_OK;
}

// 2-D row-major tensor [outer][inner] with `pitch` bytes per row and a box of box_inner x box_outer elements.
int make_map(CUtensorMap *m, const void *base, CUtensorMapDataType dt, int esize, unsigned long long inner,
                    unsigned long long outer, unsigned long long pitch, unsigned box_inner, unsigned box_outer,
                    CUtensorMapSwizzle sw)
{
    if (int rc = load_encode()) return rc;
    QLMB_REQUIRE(((uintptr_t)base & 15) == 0, "tensor map: base %p not 16-byte aligned", base);
    QLMB_REQUIRE((pitch & 15) == 0, "tensor map: row pitch %llu not a multiple of 16 bytes", pitch);
    QLMB_REQUIRE(box_inner * (unsigned)esize <= 128u && box_outer <= 256u, "tensor map: box %ux%u too large", box_inner, box_outer);
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with %d (inner %llu outer %llu pitch %llu box %ux%u)", (int)r, inner, outer, pitch, box_inner, box_outer); return QLMB_E_CUDA; }
    return QLMB_OK;
}

template <int BMODE, int EPI, int SCHED>
static int launch_inst(const GemmParams &p, int grid, cudaStream_t st)
{
    constexpr bool DEQ = (BMODE == B_DEQ_MN || BMODE == B_DEQ_K);
    constexpr int NSA = DEQ ? 3 : 4, NSB = DEQ ? 3 : 4, NSC = 4;
    constexpr size_t smem = 1024 + NSA * A_STAGE_BYTES + NSB * B_STAGE_BYTES + (DEQ ? NSC * C_STAGE_BYTES : 0) + EPI_WARPS * epi_stage_bytes(EPI) + 512;
    static bool configured = false;
    auto kfn = k_gemm<BMODE, EPI, SCHED>;
    if (!configured) {
        QLMB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    kfn<<<grid, DEQ ? 576 : 320, smem, st>>>(p);
    QLMB_LAUNCH_CHECK("k_gemm");
    return QLMB_OK;
}

template <int BMODE, int EPI, int SCHED, int DQG>
static int launch_pair_g(const GemmParams &p, long long total, cudaStream_t st)
{
    constexpr bool DEQ = (BMODE == B_DEQ_MN || BMODE == B_DEQ_K);
    constexpr size_t smem = 1024 + (size_t)(DEQ ? (EPI == EPI_SWIGLU_BWD ? 4 : 5) : 6) * (P_A_STAGE + P_B_STAGE) + (DEQ ? P_NSC * P_C_STAGE + P_S_RING : 0) + EPI_WARPS * epi_stage_bytes(EPI) + 512;
    // persistent kernel: every cluster must be resident at once, so the grid is the number of
    // clusters the device can hold at the same time (asked once per kernel instance)
    static int max_clusters = 0;
    auto kfn = k_gemm_pair<BMODE, EPI, SCHED, DQG>;
    if (!max_clusters) {
        QLMB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sm_count() & ~1)); cfg.blockDim = dim3(DEQ ? 576 : 320); cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        QLMB_CUDA(cudaOccupancyMaxActiveClusters(&n, kfn, &cfg));
        QLMB_REQUIRE(n > 0, "gemm: the device cannot hold a two-SM cluster of this kernel");
        max_clusters = n;
    }
    long long clusters = total < max_clusters ? total : max_clusters;
    kfn<<<(unsigned)(2 * clusters), DEQ ? 576 : 320, smem, st>>>(p);
    QLMB_LAUNCH_CHECK("k_gemm_pair");
    return QLMB_OK;
}

template <int BMODE, int EPI, int SCHED>
static int launch_pair(const GemmParams &p, long long total, cudaStream_t st)
{
    return launch_pair_g<BMODE, EPI, SCHED, 2>(p, total, st);     // two dequant stage groups
}

// The two-SM form needs whole 256-column tiles (128 activation columns with the SwiGLU
// epilogue); QLMB_GEMM_PAIR=0 forces the one-SM form.
static bool use_pair(const GemmLaunch &g)
{
    static int enabled = -1;
    if (enabled < 0) { const char *e = getenv("QLMB_GEMM_PAIR"); enabled = (e && atoi(e) == 0) ? 0 : 1; }
    if (!enabled) return false;
    return g.epi == EPI_SWIGLU ? (g.N % 128 == 0) : (g.N % 256 == 0);
}

int gemm_launch(const GemmLaunch &g, cudaStream_t st)
{
    int rc = load_encode();
    if (rc) return rc;
    const bool dual = g.epi == EPI_SWIGLU;
    QLMB_REQUIRE(g.N % (dual ? BN / 2 : BN) == 0, "gemm: N=%d is not a multiple of the %d-column tile", g.N, dual ? BN / 2 : BN);
    QLMB_REQUIRE(g.sched != SCHED_GROUPK || g.M % BM == 0, "gemm: grouped weight gradient needs M=%d to be a multiple of %d", g.M, BM);
    const bool pair = use_pair(g);
    GemmParams p;
    memset(&p, 0, sizeof p);
    p.nseg = g.nseg; p.ksteps = g.ksteps; p.M = g.M; p.N = g.N; p.E = g.E;
    p.tiles_m = (g.M + MH * BM - 1) / (MH * BM);
    p.tiles_n = pair ? (dual ? g.N / 128 : g.N / 256) : (dual ? g.N / (BN / 2) : g.N / BN);
    p.w_rows = g.w_rows; p.w_cols = g.w_cols;
    p.tile_info = g.tile_info; p.ntiles_dev = g.ntiles_dev; p.off = g.off;
    p.out = g.out; p.out_dtype = g.out_dtype; p.ldo = g.ldo; p.resid = g.resid; p.beta = g.beta;
    p.gp = g.gp; p.up = g.up; p.ap = g.ap; p.dgp = g.dgp; p.dup = g.dup;
    p.errword = device_error_word();
    p.scatter_perm = g.scatter_perm; p.scatter_kn = g.scatter_kn;
    for (int i = 0; i < 8; i++) p.scatter_out[i] = (bf16 *)g.scatter_out[i];
    p.scales[0] = g.scales[0]; p.scales[1] = g.scales[1];
    const unsigned long long wrows_total = (unsigned long long)g.E * g.w_rows;
    for (int s = 0; s < (dual ? 2 : g.nseg); s++) {
        if (g.bmode == AB_TMA_MN) {
            if (s > 0) break;
            // Asrc [a_rows][M-dim], Bsrc [a_rows][N]; boxes of 64 columns x 64 rows
            rc = make_map(&p.a_map[0], g.a[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.a_cols, g.a_rows, (unsigned long long)g.a_cols * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
            rc = make_map(&p.w_map[0], g.w[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.w_cols, g.a_rows, (unsigned long long)g.w_cols * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
            continue;
        }
        if (!dual || s == 0) {
            const void *a = g.a[dual ? 0 : s];
            rc = make_map(&p.a_map[s], a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.a_cols, g.a_rows, (unsigned long long)g.a_cols * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
        }
        if (g.bmode == B_TMA_K) {
            rc = make_map(&p.w_map[s], g.w[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.w_cols, wrows_total, (unsigned long long)g.w_cols * 2, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B);
        } else if (g.bmode == B_DEQ_MN) {
            QLMB_REQUIRE(g.w_cols % 128 == 0, "gemm: code matrix width %d is not a multiple of the 128-element group", g.w_cols);
            rc = make_map(&p.w_map[s], g.w[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.w_cols / 2, wrows_total, g.w_cols / 2, (dual && !pair) ? BN / 4 : BN / 2, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
        } else {
            QLMB_REQUIRE(g.w_cols % 128 == 0, "gemm: code matrix width %d is not a multiple of the 128-element group", g.w_cols);
            rc = make_map(&p.w_map[s], g.w[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.w_cols / 2, wrows_total, g.w_cols / 2, 32, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
        }
        if (rc) return rc;
    }
    // bf16 outputs leave through bulk tensor stores when their layout allows a tensor map
    {
        const unsigned long long orows = (g.sched == SCHED_ROWS) ? (unsigned long long)g.a_rows
                                       : (g.sched == SCHED_GROUPK) ? (unsigned long long)g.E * g.M : (unsigned long long)g.M;
        const void *optr[3] = {nullptr, nullptr, nullptr};
        int no = 0;
        const bool f32out = (g.epi == EPI_STORE || g.epi == EPI_ACCUM) && g.out_dtype == QLMB_F32 && !g.resid &&
                            (g.beta == 0.0f || g.beta == 1.0f);
        if (f32out) { optr[0] = g.out; no = 1; }
        else if (g.epi == EPI_STORE && g.out_dtype == QLMB_BF16 && !g.resid && g.beta == 0.0f) { optr[0] = g.out; no = 1; }
        else if (g.epi == EPI_SWIGLU) { optr[0] = g.ap; optr[1] = g.gp; optr[2] = g.up; no = 3; }
        else if (g.epi == EPI_SWIGLU_BWD) { optr[0] = g.dgp; optr[1] = g.dup; no = 2; }
        bool can = no > 0 && (g.ldo % 8) == 0 && (g.sched != SCHED_GROUPK || f32out) && orows > 0;
        for (int i = 0; i < no && can; i++) can = optr[i] && (((uintptr_t)optr[i]) & 15) == 0;
        const bool bwd = g.epi == EPI_SWIGLU_BWD;           // 32-column boxes, 64-byte swizzle
        if (bwd) can = can && g.gp && g.up && ((((uintptr_t)g.gp) | ((uintptr_t)g.up)) & 15) == 0;
        for (int i = 0; i < no && can; i++) {
            if (f32out)
                rc = make_map(&p.o_map[i], optr[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (unsigned long long)g.ldo, orows,
                              (unsigned long long)g.ldo * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
            else
                rc = make_map(&p.o_map[i], optr[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (unsigned long long)g.ldo, orows,
                              (unsigned long long)g.ldo * 2, bwd ? 32 : 64, 32, bwd ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
        }
        for (int i = 0; i < 2 && can && bwd; i++) {
            rc = make_map(&p.i_map[i], i ? (const void *)g.up : (const void *)g.gp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          (unsigned long long)g.ldo, orows, (unsigned long long)g.ldo * 2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
            if (rc) return rc;
        }
        p.o_tma = can ? 1 : 0;
    }
    long long total;
    if (g.sched == SCHED_DENSE) total = (long long)p.tiles_m * p.tiles_n;
    else if (g.sched == SCHED_ROWS) total = (long long)g.max_row_tiles * p.tiles_n;
    else total = (long long)g.E * p.tiles_m * p.tiles_n;
    if (total <= 0) return QLMB_OK;
    int grid = sm_count();
    if (total < grid) grid = (int)total;
    ProfScope prof(g.name ? g.name : "gemm", st);

#define PAIR(BM_, EP_, SC_) if (pair && g.bmode == BM_ && g.epi == EP_ && g.sched == SC_) return launch_pair<BM_, EP_, SC_>(p, total, st)
    PAIR(B_DEQ_MN, EPI_STORE, SCHED_DENSE);
    PAIR(B_DEQ_K, EPI_STORE, SCHED_DENSE);
    PAIR(AB_TMA_MN, EPI_ACCUM, SCHED_DENSE);
    PAIR(B_TMA_K, EPI_STORE, SCHED_DENSE);
    PAIR(B_DEQ_MN, EPI_SWIGLU, SCHED_ROWS);
    PAIR(B_DEQ_MN, EPI_STORE, SCHED_ROWS);
    PAIR(B_DEQ_K, EPI_SWIGLU_BWD, SCHED_ROWS);
    PAIR(B_DEQ_K, EPI_STORE, SCHED_ROWS);
    PAIR(AB_TMA_MN, EPI_ACCUM, SCHED_GROUPK);
#undef PAIR

#define INST(BM_, EP_, SC_) if (g.bmode == BM_ && g.epi == EP_ && g.sched == SC_) return launch_inst<BM_, EP_, SC_>(p, grid, st)
    // dense linears
    INST(B_DEQ_MN, EPI_STORE, SCHED_DENSE);
    INST(B_DEQ_K, EPI_STORE, SCHED_DENSE);
    INST(AB_TMA_MN, EPI_ACCUM, SCHED_DENSE);
    INST(B_TMA_K, EPI_STORE, SCHED_DENSE);
    // expert FFN
    INST(B_DEQ_MN, EPI_SWIGLU, SCHED_ROWS);
    INST(B_DEQ_MN, EPI_STORE, SCHED_ROWS);
    INST(B_DEQ_K, EPI_SWIGLU_BWD, SCHED_ROWS);
    INST(B_DEQ_K, EPI_STORE, SCHED_ROWS);
    INST(AB_TMA_MN, EPI_ACCUM, SCHED_GROUPK);
#undef INST
    set_error("gemm: no kernel instance for bmode %d epi %d sched %d", g.bmode, g.epi, g.sched);
    return QLMB_E_UNSUPPORTED;
}

}  // namespace qlmb
