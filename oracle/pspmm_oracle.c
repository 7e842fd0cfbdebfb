/*
 * CPU oracle for the ParamSpMM sparse hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, what the reference computes on the path
 * CSR/PCSR x dense SpMM, pattern-masked SDDMM, and the PCSR index builders.
 * It exists so the CUDA kernels can be checked against something that is easy
 * to read.  It is never linked into, loaded by, or called from the product
 * library; only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * Every function names the reference location (path within the reference
 * project : lines) whose behaviour it follows.
 *
 * Build: oracle/build_oracle.py::build_oracle (gcc -O2 -fopenmp -shared -fPIC).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* Number of host threads the OpenMP loops will use (1 without OpenMP). */
ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------
 * PCSR partition: cut every row into pieces of at most `gran` entries.
 * Follows SpMM/SpMM.cpp:15-40 (split_csr; split_csr_par :42-75 computes the
 * same arrays in parallel from per-row offsets).
 *
 * Pass 1 (out arrays NULL) returns the number of pieces S.
 * Pass 2 fills rowPtr_split[S+1] and target_row[S].
 * ---------------------------------------------------------------------- */
ORC_API int64_t orc_split_csr(const int32_t *rowPtr, int64_t n_rows, int32_t gran,
                              int32_t *rowPtr_split, int32_t *target_row)
{
    int64_t s = 0;
    if (rowPtr_split)
        rowPtr_split[0] = 0;
    for (int64_t r = 0; r < n_rows; ++r) {
        int32_t end = rowPtr[r + 1];
        for (int32_t at = rowPtr[r]; at < end; at += gran) {
            if (rowPtr_split) {
                int32_t stop = at + gran;
                rowPtr_split[s + 1] = stop > end ? end : stop;
                target_row[s] = (int32_t)r;
            }
            ++s;
        }
    }
    return s;
}

/* ------------------------------------------------------------------------
 * CSR -> block CSR with V x 1 blocks, as scipy.sparse.csr_array.tobsr does
 * (scipy is the third-party code graph_input.py:245-266 relies on; the
 * algorithm restated here is scipy's csr_tobsr: inside one block-row, blocks
 * are created in order of FIRST ENCOUNTER while walking the V member rows
 * top to bottom, so block columns are NOT sorted).  Rows beyond n_rows (when
 * n_rows is not a multiple of V) are treated as empty, which is what the
 * reference's padding of rowPtr achieves (graph_input.py:248-256).
 *
 * Pass 1 (colIdx_b NULL) fills rowPtr_b[nbr+1] and returns the block count.
 * Pass 2 fills colIdx_b[nblk] and val_b[nblk*V] (zero where absent).
 * `scratch` must hold n_cols int32 initialised to -1; it is restored to -1.
 * ---------------------------------------------------------------------- */
ORC_API int64_t orc_bcsr_build(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                               int64_t n_rows, int32_t V, int32_t *scratch,
                               int32_t *rowPtr_b, int32_t *colIdx_b, float *val_b)
{
    int64_t nbr = (n_rows + V - 1) / V;
    int64_t nblk = 0;
    rowPtr_b[0] = 0;
    for (int64_t br = 0; br < nbr; ++br) {
        int64_t first = nblk;
        for (int32_t v = 0; v < V; ++v) {
            int64_t r = br * V + v;
            if (r >= n_rows)
                break;
            for (int32_t k = rowPtr[r]; k < rowPtr[r + 1]; ++k) {
                int32_t c = colIdx[k];
                if (scratch[c] < 0) {
                    scratch[c] = (int32_t)(nblk - first);
                    if (colIdx_b) {
                        colIdx_b[nblk] = c;
                        for (int32_t u = 0; u < V; ++u)
                            val_b[nblk * V + u] = 0.0f;
                    }
                    ++nblk;
                }
                if (colIdx_b)
                    val_b[(first + scratch[c]) * V + v] += val[k];
            }
        }
        for (int32_t v = 0; v < V; ++v) {
            int64_t r = br * V + v;
            if (r >= n_rows)
                break;
            for (int32_t k = rowPtr[r]; k < rowPtr[r + 1]; ++k)
                scratch[colIdx[k]] = -1;
        }
        rowPtr_b[br + 1] = (int32_t)nblk;
    }
    return nblk;
}

/* ------------------------------------------------------------------------
 * CSR-order -> flattened BCSR(2x1) value index ("mask").
 * Follows SDDMM/sddmm_kernel.cu:78-118 (genmask_kernel): per block-row two
 * running cursors start at the CSR row starts of rows 2r and 2r+1; walking
 * the blocks in stored order, every non-zero lane u of block i emits
 * mask[cursor[u]++] = 2*i + u.
 * ---------------------------------------------------------------------- */
ORC_API void orc_genmask(const int32_t *rowPtr_b, const int32_t *rowPtr, const float *val_b,
                         int64_t n_blk_rows, int32_t *mask)
{
    for (int64_t br = 0; br < n_blk_rows; ++br) {
        int32_t lo = rowPtr_b[br], hi = rowPtr_b[br + 1];
        if (lo == hi)
            continue;
        int32_t cur0 = rowPtr[2 * br];
        int32_t cur1 = rowPtr[2 * br + 1];
        for (int32_t i = lo; i < hi; ++i) {
            if (val_b[2 * (int64_t)i] != 0.0f)
                mask[cur0++] = 2 * i;
            if (val_b[2 * (int64_t)i + 1] != 0.0f)
                mask[cur1++] = 2 * i + 1;
        }
    }
}

/* ------------------------------------------------------------------------
 * SpMM, C = A * B with A in CSR.  Follows SpMM/SpMM_kernel.cu:1157-1243
 * (csr_spmm_cuda_kernel): per output element a running sum over the row's
 * entries in stored order; rows without entries stay zero (:136, :1179).
 * acc64 != 0 accumulates in double (tighter truth); acc64 == 0 keeps the
 * reference's fp32 running sum.  C is fully overwritten.
 * ---------------------------------------------------------------------- */
ORC_API void orc_spmm_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                          const float *B, float *C, int64_t n_rows, int32_t dim, int64_t ldB,
                          int64_t ldC, int32_t acc64)
{
#pragma omp parallel
    {
        double *acc = (double *)malloc(sizeof(double) * (size_t)(dim > 0 ? dim : 1));
        float *accf = (float *)acc;
#pragma omp for schedule(dynamic, 256)
        for (int64_t r = 0; r < n_rows; ++r) {
            float *out = C + r * ldC;
            if (acc64) {
                for (int32_t j = 0; j < dim; ++j)
                    acc[j] = 0.0;
                for (int32_t k = rowPtr[r]; k < rowPtr[r + 1]; ++k) {
                    const float *b = B + (int64_t)colIdx[k] * ldB;
                    double a = (double)val[k];
                    for (int32_t j = 0; j < dim; ++j)
                        acc[j] += a * (double)b[j];
                }
                for (int32_t j = 0; j < dim; ++j)
                    out[j] = (float)acc[j];
            } else {
                for (int32_t j = 0; j < dim; ++j)
                    accf[j] = 0.0f;
                for (int32_t k = rowPtr[r]; k < rowPtr[r + 1]; ++k) {
                    const float *b = B + (int64_t)colIdx[k] * ldB;
                    float a = val[k];
                    for (int32_t j = 0; j < dim; ++j)
                        accf[j] += a * b[j];
                }
                for (int32_t j = 0; j < dim; ++j)
                    out[j] = accf[j];
            }
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------------
 * SpMM over a row-split layout.  Follows SpMM/SpMM_kernel.cu:1245-1360
 * (csr_split_spmm_cuda_kernel): every piece s sums its entries and ADDS the
 * result into row target_row[s] of a zero-initialised output (atomicAdd at
 * :1300, :1325).  Serial here, so the result is deterministic.
 * ---------------------------------------------------------------------- */
ORC_API void orc_spmm_csr_split(const int32_t *rowPtr_split, const int32_t *target_row,
                                int64_t n_seg, const int32_t *colIdx, const float *val,
                                const float *B, float *C, int64_t n_rows, int32_t dim, int64_t ldB,
                                int64_t ldC)
{
    for (int64_t r = 0; r < n_rows; ++r)
        memset(C + r * ldC, 0, sizeof(float) * (size_t)dim);
    double *acc = (double *)malloc(sizeof(double) * (size_t)(dim > 0 ? dim : 1));
    for (int64_t s = 0; s < n_seg; ++s) {
        for (int32_t j = 0; j < dim; ++j)
            acc[j] = 0.0;
        for (int32_t k = rowPtr_split[s]; k < rowPtr_split[s + 1]; ++k) {
            const float *b = B + (int64_t)colIdx[k] * ldB;
            double a = (double)val[k];
            for (int32_t j = 0; j < dim; ++j)
                acc[j] += a * (double)b[j];
        }
        float *out = C + (int64_t)target_row[s] * ldC;
        for (int32_t j = 0; j < dim; ++j)
            out[j] = (float)((double)out[j] + acc[j]);
    }
    free(acc);
}

/* ------------------------------------------------------------------------
 * SpMM with V x 1 blocks (V = 2 is the reference's "bcsr", V = 3 its "vec").
 * Follows SpMM/SpMM_kernel.cu:1362-1493 and :1653-1785: block k of block-row
 * r carries column colIdx[k] and V values; lane u adds val[k][u]*B[col] into
 * output row V*r+u, lanes whose value is exactly zero are skipped (:1399,
 * :1405).  The output has V*ceil(n/V) rows (:281-282, :427-428).  With
 * target_row != NULL the block-rows are pieces of a split layout
 * (:1495-1651, :1787-1972) and results are added into block-row
 * target_row[s]; otherwise piece s is block-row s.
 * ---------------------------------------------------------------------- */
ORC_API void orc_spmm_bcsr(const int32_t *rowPtr_b, const int32_t *target_row, int64_t n_seg,
                           const int32_t *colIdx, const float *val_b, int32_t V, const float *B,
                           float *C, int64_t n_out_rows, int32_t dim, int64_t ldB, int64_t ldC)
{
    for (int64_t r = 0; r < n_out_rows; ++r)
        memset(C + r * ldC, 0, sizeof(float) * (size_t)dim);
    double *acc = (double *)malloc(sizeof(double) * (size_t)(dim > 0 ? dim : 1) * (size_t)V);
    for (int64_t s = 0; s < n_seg; ++s) {
        for (int64_t j = 0; j < (int64_t)dim * V; ++j)
            acc[j] = 0.0;
        for (int32_t k = rowPtr_b[s]; k < rowPtr_b[s + 1]; ++k) {
            const float *b = B + (int64_t)colIdx[k] * ldB;
            for (int32_t u = 0; u < V; ++u) {
                float a = val_b[(int64_t)k * V + u];
                if (a == 0.0f)
                    continue;
                for (int32_t j = 0; j < dim; ++j)
                    acc[(int64_t)u * dim + j] += (double)a * (double)b[j];
            }
        }
        int64_t br = target_row ? (int64_t)target_row[s] : s;
        for (int32_t u = 0; u < V; ++u) {
            float *out = C + (br * V + u) * ldC;
            for (int32_t j = 0; j < dim; ++j)
                out[j] = (float)((double)out[j] + acc[(int64_t)u * dim + j]);
        }
    }
    free(acc);
}

/* ------------------------------------------------------------------------
 * SDDMM on a CSR pattern: out[k] = <A[row(k)], B[colIdx[k]]>.
 * Follows SDDMM/sddmm_kernel.cu:917-1057; the stored values are never read
 * (:969-981).  With target_row != NULL the rows are pieces of a split layout
 * and row(k) = target_row[s].
 * ---------------------------------------------------------------------- */
ORC_API void orc_sddmm_csr(const int32_t *rowPtr, const int32_t *target_row, int64_t n_seg,
                           const int32_t *colIdx, const float *A, const float *B, float *out,
                           int32_t dim, int64_t ldA, int64_t ldB)
{
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t s = 0; s < n_seg; ++s) {
        int64_t r = target_row ? (int64_t)target_row[s] : s;
        const float *a = A + r * ldA;
        for (int32_t k = rowPtr[s]; k < rowPtr[s + 1]; ++k) {
            const float *b = B + (int64_t)colIdx[k] * ldB;
            double acc = 0.0;
            for (int32_t j = 0; j < dim; ++j)
                acc += (double)a[j] * (double)b[j];
            out[k] = (float)acc;
        }
    }
}

/* ------------------------------------------------------------------------
 * SDDMM on V x 1 blocks: out[k][u] = <A[V*row+u], B[colIdx[k]]> where the
 * stored value val_b[k][u] is non-zero, zero elsewhere (values act as the
 * mask).  Follows SDDMM/sddmm_kernel.cu:1059-1287 (:1144, :1159) and the
 * intent of the V = 3 kernels at :1289-1468.
 * ---------------------------------------------------------------------- */
ORC_API void orc_sddmm_bcsr(const int32_t *rowPtr_b, const int32_t *target_row, int64_t n_seg,
                            const int32_t *colIdx, const float *val_b, int32_t V, const float *A,
                            const float *B, float *out, int32_t dim, int64_t ldA, int64_t ldB)
{
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t s = 0; s < n_seg; ++s) {
        int64_t br = target_row ? (int64_t)target_row[s] : s;
        for (int32_t k = rowPtr_b[s]; k < rowPtr_b[s + 1]; ++k) {
            const float *b = B + (int64_t)colIdx[k] * ldB;
            for (int32_t u = 0; u < V; ++u) {
                double acc = 0.0;
                if (val_b[(int64_t)k * V + u] != 0.0f) {
                    const float *a = A + (br * V + u) * ldA;
                    for (int32_t j = 0; j < dim; ++j)
                        acc += (double)a[j] * (double)b[j];
                }
                out[(int64_t)k * V + u] = (float)acc;
            }
        }
    }
}
