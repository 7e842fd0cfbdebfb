// Shared declarations for the sm_100a kernels behind libpspmm's C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "pspmm.h"

#define PSPMM_FULL_MASK 0xffffffffu
#define PSPMM_MAX_CF 8
#define PSPMM_RPG_MAX 16  // most consecutive segments one lane group owns
#define PSPMM_GAP_MAX 256  // longest run of uncovered rows the SpMM kernel zeroes by itself

// Records the CUDA error text for pspmm_last_cuda_error() and returns PSPMM_E_CUDA.
int pspmm_note_cuda_error(cudaError_t e);

#define PSPMM_CUDA_TRY(expr)                    \
    do {                                        \
        cudaError_t e__ = (expr);               \
        if (e__ != cudaSuccess)                 \
            return pspmm_note_cuda_error(e__);  \
    } while (0)

// One launch of the segment SpMM kernel.  A "segment" is a CSR row, a PCSR row piece, or
// the block-row forms of either.
struct SpmmArgs {
    const int32_t *segPtr;      // [n_seg + 1] entry ranges
    const int32_t *target_row;  // [n_seg] output (block-)row of each segment, or nullptr: row == segment
    const int32_t *colIdx;      // [n_entries]
    const float *val;           // [n_entries * V]
    const float *B;
    float *C;
    int64_t n_seg;
    int64_t n_out;              // output (block-)rows
    int64_t ldB, ldC;
    int32_t nvec;               // dim / VW: vectors per dense row
    int32_t rows_per_group;
    float keep_fraction;        // share of B's lines marked evict-last in L2 (0..1]
    int32_t bucketed;           // target_row carries PSPMM_SEG_* flags, segments come in any order
};

// Flags in target_row of a length-bucketed plan (pspmm_cfg.bucketed): the low 30 bits are the row.
#define PSPMM_SEG_MULTI 0x80000000u  // the row is cut into several segments: every one of them adds with REDs
#define PSPMM_SEG_FIRST 0x40000000u  // the first of them: the pre-pass zeroes the row when it meets this one
#define PSPMM_SEG_ROW_MASK 0x3fffffffu

struct SddmmArgs {
    const int32_t *segPtr;
    const int32_t *target_row;
    const int32_t *colIdx;
    const float *val;  // mask for V > 1, unused for V == 1
    const float *A;
    const float *B;
    float *out;
    int64_t n_seg;
    int64_t n_rows_A;  // rows of A that exist: block forms read rows arow*V + w only below this
    int64_t ldA, ldB;
    int32_t nvec;
    int32_t rows_per_group;
    float keep_fraction;
};

// Resolved launch shape.
struct LaunchShape {
    int lpr, vw, cf, threads, rpg, tiles, mlp;
};

// Per-translation-unit dispatchers (one per vector width so the files compile in parallel).
// Return false when (lpr, cf, V) is not instantiated for that width.
bool pspmm_launch_spmm_vw4(const LaunchShape &s, int V, const SpmmArgs &a, dim3 grid, cudaStream_t st);
bool pspmm_launch_spmm_vw4_acc(const LaunchShape &s, const SpmmArgs &a, dim3 grid, cudaStream_t st);
bool pspmm_launch_spmm_vw2(const LaunchShape &s, int V, const SpmmArgs &a, dim3 grid, cudaStream_t st);
bool pspmm_launch_spmm_vw1(const LaunchShape &s, int V, const SpmmArgs &a, dim3 grid, cudaStream_t st);
bool pspmm_launch_sddmm_vw4(const LaunchShape &s, int V, const SddmmArgs &a, dim3 grid, cudaStream_t st);
bool pspmm_launch_sddmm_vw2(const LaunchShape &s, int V, const SddmmArgs &a, dim3 grid, cudaStream_t st);
bool pspmm_launch_sddmm_vw1(const LaunchShape &s, int V, const SddmmArgs &a, dim3 grid, cudaStream_t st);

// Smallest instantiated coarsening factor >= need (0 when none).
static inline int pspmm_round_cf(int need)
{
    static const int have[] = {1, 2, 3, 4, 6, 8};
    for (int c : have)
        if (c >= need)
            return c;
    return 0;
}

int pspmm_validate_cfg(const pspmm_cfg *cfg, bool sddmm);
int pspmm_resolve_shape(const pspmm_cfg *cfg, int32_t dim, int vw_max, int V, LaunchShape *out);
int pspmm_vw_max(int32_t dim, int64_t ld0, int64_t ld1, const void *p0, const void *p1);
