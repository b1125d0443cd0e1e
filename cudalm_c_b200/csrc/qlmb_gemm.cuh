// Host-side launch interface of the tcgen05 GEMM engine (qlmb_gemm.cu).
#pragma once
#include <cuda.h>
#include "qlmb_internal.h"

namespace qlmb {

// How the B operand (and for AB_TMA_MN also A) reaches shared memory.
enum BMode {
    B_TMA_K = 0,    // bf16 B[N][K] by TMA, K-major          (plain NT GEMM, used for engine tests)
    B_DEQ_MN = 1,   // 4-bit codes W[K][N], expanded by the dequant warps into an MN-major tile
    B_DEQ_K = 2,    // 4-bit codes W[N][K], expanded into a K-major tile
    AB_TMA_MN = 3   // bf16 Asrc[R][Ma], Bsrc[R][Nb] by TMA, both MN-major: C = Asrc^T Bsrc (wgrad)
};
enum Epi {
    EPI_STORE = 0,       // out = acc (+ resid) (+ beta*out), fp32 or bf16
    EPI_SWIGLU = 1,      // accumulator = [g | u] halves: ap = silu(g)*u, gp = g, up = u (bf16)
    EPI_SWIGLU_BWD = 2,  // accumulator = d(act): dgp, dup from stashed gp, up (bf16)
    EPI_ACCUM = 3        // out(fp32) = beta*out + acc
};
enum Sched {
    SCHED_DENSE = 0,   // tiles over [ceil(M/256)] x [N/128]
    SCHED_ROWS = 1,    // row tiles from a device table (one expert per tile) x [N/128]
    SCHED_GROUPK = 2   // per expert: [ceil(Ma/256)] x [Nb/128] tiles, contraction over the expert's rows
};

struct GemmLaunch {
    int bmode, epi, sched;
    // A operand(s): bf16 [a_rows][a_cols] row-major; one per contraction segment
    const void *a[2];
    long long a_rows;
    int a_cols;
    // weights: codes (two nibbles per byte) or bf16, stored [E*w_rows][w_cols] row-major
    const void *w[2];
    const float *scales[2];
    int w_rows, w_cols;
    int nseg;                      // contraction segments (2: dXp = dg W1^T + du W3^T)
    int ksteps;                    // 64-wide contraction steps per segment (DENSE / ROWS)
    int M, N, E;                   // valid rows (DENSE), output columns, experts
    const int *tile_info;          // ROWS: per 256-row tile: first row/128 | expert << 20 | (halves-1) << 30
    const int *ntiles_dev;         // ROWS: number of row tiles (device int)
    const int *off;                // GROUPK: padded row offsets [E+1]
    int max_row_tiles;             // ROWS: upper bound of *ntiles_dev (grid sizing)
    // epilogue
    void *out; int out_dtype; long long ldo;
    const void *resid; float beta;
    bf16 *gp, *up, *ap, *dgp, *dup;
    // bf16 EPI_STORE only: rows leave to where they came from instead of to `out` -- output row j goes to
    // row (scatter_perm[j] % scatter_kn) of the buffer scatter_out[scatter_perm[j] / scatter_kn] (one per
    // rank, possibly peer-mapped); rows with scatter_perm[j] < 0 are not written
    const int *scatter_perm; int scatter_kn; const void *scatter_out[8];
    const char *name;              // label for the optional per-kernel timing
};

int gemm_launch(const GemmLaunch &g, cudaStream_t st);

// 2-D row-major tensor map [outer][inner] with `pitch` bytes per row and a box of box_inner x box_outer elements
int make_map(CUtensorMap *m, const void *base, CUtensorMapDataType dt, int esize, unsigned long long inner,
             unsigned long long outer, unsigned long long pitch, unsigned box_inner, unsigned box_outer,
             CUtensorMapSwizzle sw);

}  // namespace qlmb
