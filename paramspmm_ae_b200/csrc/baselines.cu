// libpspmm_baselines: cuSPARSE comparators, kept out of libpspmm so the product library has no
// cuSPARSE dependency.  These reproduce the call sequences the reference times its kernels
// against (SpMM/Baseline_kernel.cu:24-599: cusparseSpMM on CSR with ALG_DEFAULT and CSR_ALG2,
// COO, CSC; SDDMM/sddmm_baseline_kernel.cu:24-164: cusparseSDDMM), with the handle,
// descriptors and workspace created once per plan instead of once per call.
#include <cuda_runtime.h>
#include <cusparse.h>
#include <stdint.h>
#include <stdio.h>

#define PB_API extern "C" __attribute__((visibility("default")))

static thread_local char g_err[256] = "";
PB_API const char *pspmm_baselines_last_error(void) { return g_err; }

#define PB_CUSPARSE(expr)                                                                  \
    do {                                                                                   \
        cusparseStatus_t s__ = (expr);                                                     \
        if (s__ != CUSPARSE_STATUS_SUCCESS) {                                              \
            snprintf(g_err, sizeof(g_err), "cuSPARSE: %s (%s)", cusparseGetErrorString(s__), #expr); \
            return -1;                                                                     \
        }                                                                                  \
    } while (0)
#define PB_CUDA(expr)                                                                      \
    do {                                                                                   \
        cudaError_t e__ = (expr);                                                          \
        if (e__ != cudaSuccess) {                                                          \
            snprintf(g_err, sizeof(g_err), "CUDA: %s (%s)", cudaGetErrorString(e__), #expr); \
            return -1;                                                                     \
        }                                                                                  \
    } while (0)

struct Plan {
    cusparseHandle_t handle = nullptr;
    cusparseSpMatDescr_t A = nullptr;
    cusparseDnMatDescr_t X = nullptr, Y = nullptr;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    int kind = 0;  // 0 SpMM, 1 SDDMM
    cusparseSpMMAlg_t alg = CUSPARSE_SPMM_ALG_DEFAULT;
    cusparseOperation_t opB = CUSPARSE_OPERATION_NON_TRANSPOSE;
};

static void plan_free(Plan *p)
{
    if (!p)
        return;
    if (p->X) cusparseDestroyDnMat(p->X);
    if (p->Y) cusparseDestroyDnMat(p->Y);
    if (p->A) cusparseDestroySpMat(p->A);
    if (p->workspace) cudaFree(p->workspace);
    if (p->handle) cusparseDestroy(p->handle);
    delete p;
}

PB_API int pspmm_baselines_plan_destroy(void *plan)
{
    plan_free((Plan *)plan);
    return 0;
}

// fmt: 0 CSR + ALG_DEFAULT, 1 CSR + CSR_ALG2, 2 COO + ALG_DEFAULT, 3 CSC + ALG_DEFAULT.
// idx0/idx1: (rowPtr, colIdx) for CSR, (row, col) for COO, (colPtr, rowIdx) for CSC.
PB_API int pspmm_baselines_spmm_plan(void **out, int fmt, const int32_t *idx0, const int32_t *idx1,
                                     const float *val, const float *B, float *C, int64_t n_rows,
                                     int64_t n_cols, int64_t nnz, int32_t dim, int64_t ldB,
                                     int64_t ldC)
{
    if (!out || fmt < 0 || fmt > 3)
        return -1;
    Plan *p = new Plan();
    struct Guard { Plan *&p; ~Guard() { if (p) plan_free(p); } } guard{p};
    PB_CUSPARSE(cusparseCreate(&p->handle));
    void *i0 = (void *)idx0, *i1 = (void *)idx1, *v = (void *)val;
    if (fmt == 0 || fmt == 1)
        PB_CUSPARSE(cusparseCreateCsr(&p->A, n_rows, n_cols, nnz, i0, i1, v, CUSPARSE_INDEX_32I,
                                      CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    else if (fmt == 2)
        PB_CUSPARSE(cusparseCreateCoo(&p->A, n_rows, n_cols, nnz, i0, i1, v, CUSPARSE_INDEX_32I,
                                      CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    else
        PB_CUSPARSE(cusparseCreateCsc(&p->A, n_rows, n_cols, nnz, i0, i1, v, CUSPARSE_INDEX_32I,
                                      CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    PB_CUSPARSE(cusparseCreateDnMat(&p->X, n_cols, dim, ldB, (void *)B, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    PB_CUSPARSE(cusparseCreateDnMat(&p->Y, n_rows, dim, ldC, (void *)C, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    p->alg = fmt == 1 ? CUSPARSE_SPMM_CSR_ALG2 : CUSPARSE_SPMM_ALG_DEFAULT;
    const float alpha = 1.f, beta = 0.f;
    PB_CUSPARSE(cusparseSpMM_bufferSize(p->handle, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                        CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, p->A, p->X, &beta,
                                        p->Y, CUDA_R_32F, p->alg, &p->workspace_bytes));
    if (p->workspace_bytes)
        PB_CUDA(cudaMalloc(&p->workspace, p->workspace_bytes));
    *out = p;
    p = nullptr;  // released to the caller
    return 0;
}

// Sampled product on the CSR pattern: val[k] = <A[row(k)], B[colIdx[k]]> (B given row-major
// [n_cols, dim] and used transposed, as the reference does).
PB_API int pspmm_baselines_sddmm_plan(void **out, const int32_t *rowPtr, const int32_t *colIdx,
                                      float *val, const float *A, const float *B, int64_t n_rows,
                                      int64_t n_cols, int64_t nnz, int32_t dim, int64_t ldA,
                                      int64_t ldB)
{
    if (!out)
        return -1;
    Plan *p = new Plan();
    struct Guard { Plan *&p; ~Guard() { if (p) plan_free(p); } } guard{p};
    p->kind = 1;
    PB_CUSPARSE(cusparseCreate(&p->handle));
    PB_CUSPARSE(cusparseCreateCsr(&p->A, n_rows, n_cols, nnz, (void *)rowPtr, (void *)colIdx, val,
                                  CUSPARSE_INDEX_32I, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO,
                                  CUDA_R_32F));
    PB_CUSPARSE(cusparseCreateDnMat(&p->X, n_rows, dim, ldA, (void *)A, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    // B^T as a column-major [dim, n_cols] matrix with leading dimension ldB is the row-major B.
    PB_CUSPARSE(cusparseCreateDnMat(&p->Y, dim, n_cols, ldB, (void *)B, CUDA_R_32F, CUSPARSE_ORDER_COL));
    const float alpha = 1.f, beta = 0.f;
    PB_CUSPARSE(cusparseSDDMM_bufferSize(p->handle, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                         CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, p->X, p->Y, &beta,
                                         p->A, CUDA_R_32F, CUSPARSE_SDDMM_ALG_DEFAULT,
                                         &p->workspace_bytes));
    if (p->workspace_bytes)
        PB_CUDA(cudaMalloc(&p->workspace, p->workspace_bytes));
    PB_CUSPARSE(cusparseSDDMM_preprocess(p->handle, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                         CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, p->X, p->Y, &beta,
                                         p->A, CUDA_R_32F, CUSPARSE_SDDMM_ALG_DEFAULT, p->workspace));
    *out = p;
    p = nullptr;
    return 0;
}

PB_API int pspmm_baselines_run(void *plan, void *stream)
{
    Plan *p = (Plan *)plan;
    if (!p)
        return -1;
    const float alpha = 1.f, beta = 0.f;
    PB_CUSPARSE(cusparseSetStream(p->handle, (cudaStream_t)stream));
    if (p->kind == 0)
        PB_CUSPARSE(cusparseSpMM(p->handle, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                 CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, p->A, p->X, &beta, p->Y,
                                 CUDA_R_32F, p->alg, p->workspace));
    else
        PB_CUSPARSE(cusparseSDDMM(p->handle, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                  CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, p->X, p->Y, &beta, p->A,
                                  CUDA_R_32F, CUSPARSE_SDDMM_ALG_DEFAULT, p->workspace));
    return 0;
}

// ----------------------------------------------------------------------------- GE-SpMM comparator
// A restatement, in this library's own code, of the algorithm published as GE-SpMM (Huang et al.,
// SC 2020), which the reference times its kernels against (its vendored copy is
// SpMM/Baseline_kernel.cu:601-857): one warp per row and per tile of 32*CF dense columns;
// "coalesced row caching" = the warp loads 32 (column, value) pairs of the row into shared memory
// with one coalesced access and every lane then walks them; "coarse-grained warp merging" = each
// lane produces CF output columns (stride 32) so the cached pairs are reused CF times.
// It is a comparator only: nothing in libpspmm uses it.
template <int CF>
__global__ void __launch_bounds__(256) gespmm_like_kernel(const int32_t *__restrict__ rowPtr,
                                                          const int32_t *__restrict__ colIdx,
                                                          const float *__restrict__ val,
                                                          const float *__restrict__ B, float *__restrict__ C,
                                                          int64_t n_rows, int dim, int64_t ldB, int64_t ldC)
{
    __shared__ int s_col[8][32];
    __shared__ float s_val[8][32];
    const int lane = threadIdx.x, w = threadIdx.y;
    const int64_t row = (int64_t)blockIdx.x * blockDim.y + w;
    if (row >= n_rows)
        return;  // whole warps leave: row is warp-uniform
    const int col0 = blockIdx.y * 32 * CF + lane;
    const int lb = rowPtr[row], hb = rowPtr[row + 1];
    float acc[CF];
#pragma unroll
    for (int j = 0; j < CF; ++j)
        acc[j] = 0.f;
    for (int ptr = lb; ptr < hb; ptr += 32) {
        if (ptr + lane < hb) {
            s_col[w][lane] = colIdx[ptr + lane];
            s_val[w][lane] = val[ptr + lane];
        }
        __syncwarp();
        const int n = hb - ptr < 32 ? hb - ptr : 32;
        for (int k = 0; k < n; ++k) {
            const float *brow = B + (int64_t)s_col[w][k] * ldB;
            const float v = s_val[w][k];
#pragma unroll
            for (int j = 0; j < CF; ++j)
                if (col0 + 32 * j < dim)
                    acc[j] = fmaf(v, brow[col0 + 32 * j], acc[j]);
        }
        __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < CF; ++j)
        if (col0 + 32 * j < dim)
            C[row * ldC + col0 + 32 * j] = acc[j];
}

PB_API int pspmm_baselines_gespmm(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                                  const float *B, float *C, int64_t n_rows, int32_t dim, int64_t ldB,
                                  int64_t ldC, void *stream)
{
    if (!rowPtr || !B || !C || n_rows < 0 || dim <= 0)
        return -1;
    if (n_rows == 0)
        return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 block(32, 8);
    const unsigned gx = (unsigned)((n_rows + 7) / 8);
    // Coarsening as the reference's wrapper picks it (SpMM/Baseline_kernel.cu:763): 1 below 128
    // dense columns, 2 from 128, 4 from 512.
    if (dim < 128)
        gespmm_like_kernel<1><<<dim3(gx, (dim + 31) / 32), block, 0, st>>>(rowPtr, colIdx, val, B, C, n_rows, dim, ldB, ldC);
    else if (dim < 512)
        gespmm_like_kernel<2><<<dim3(gx, (dim + 63) / 64), block, 0, st>>>(rowPtr, colIdx, val, B, C, n_rows, dim, ldB, ldC);
    else
        gespmm_like_kernel<4><<<dim3(gx, (dim + 127) / 128), block, 0, st>>>(rowPtr, colIdx, val, B, C, n_rows, dim, ldB, ldC);
    PB_CUDA(cudaGetLastError());
    return 0;
}

// ----------------------------------------------------------------------------- gather ceiling
// How fast can ANY kernel on this GPU fetch the rows B[colIdx[k]] for the whole column stream of
// a matrix?  This measures it: lane groups of dim/4 lanes (one 16-byte slice of a row per lane)
// walk contiguous runs of the stream with 8 independent row loads in flight per lane and fold
// what they load into one float4 per lane, written once at the end so that the loads cannot be
// dropped.  No values, no row pointers, no output rows: the time of this kernel is a lower bound
// for a row-major-gather SpMM over the same stream and the same dense operand, and
// 4 * dim * nnz / time is the gather rate the memory system delivers for it (L2 hits included).
// It is a measuring stick: nothing in libpspmm uses it.
template <int LPR>
__global__ void __launch_bounds__(256) gather_ceiling_kernel(const int32_t *__restrict__ colIdx, int64_t nnz,
                                                             const float *__restrict__ B, int64_t ldB,
                                                             int run, int active, float4 *__restrict__ sink)
{
    const int gl = threadIdx.x % LPR;
    const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const int64_t k0 = group * run;
    if (gl >= active || k0 >= nnz)
        return;  // lanes beyond the last 16-byte slice of a row, groups beyond the stream
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float *base = B + gl * 4;
    int64_t k = k0;
    const int64_t kend = k0 + run < nnz ? k0 + run : nnz;
    for (; k + 8 <= kend; k += 8) {
        // one 32-byte sector of column ids per 8 entries, read by every lane of the group (broadcast)
        const int4 c0 = __ldg(reinterpret_cast<const int4 *>(colIdx + k));
        const int4 c1 = __ldg(reinterpret_cast<const int4 *>(colIdx + k + 4));
        const int c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float4 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            x[u] = __ldg(reinterpret_cast<const float4 *>(base + (int64_t)c[u] * ldB));
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            acc.x += x[u].x; acc.y += x[u].y; acc.z += x[u].z; acc.w += x[u].w;
        }
    }
    for (; k < kend; ++k) {
        const float4 x = __ldg(reinterpret_cast<const float4 *>(base + (int64_t)__ldg(colIdx + k) * ldB));
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    sink[(int64_t)blockIdx.x * blockDim.x + threadIdx.x] = acc;
}

// dim: a multiple of 4.  Rows wider than 128 floats are fetched in passes of 32 lanes over
// successive 512-byte parts (the time of all passes counts).  run: entries per lane group (a
// multiple of 8, e.g. 64).  sink: device buffer of pspmm_baselines_gather_sink_bytes(nnz, dim, run)
// bytes.  colIdx must be 16-byte aligned.
static int gather_lanes(int32_t dim)
{
    const int nvec = dim / 4;
    int lpr = 4;
    while (lpr < nvec && lpr < 32)
        lpr <<= 1;
    return lpr;
}

PB_API int64_t pspmm_baselines_gather_sink_bytes(int64_t nnz, int32_t dim, int32_t run)
{
    const int lpr = gather_lanes(dim);
    const int64_t groups = (nnz + run - 1) / run;
    const int64_t threads = (groups * lpr + 255) / 256 * 256;
    return threads * 16;
}

PB_API int pspmm_baselines_gather_ceiling(const int32_t *colIdx, int64_t nnz, const float *B, int32_t dim,
                                          int64_t ldB, int32_t run, void *sink, void *stream)
{
    if (!colIdx || !B || !sink || nnz <= 0 || dim <= 0 || dim % 4 != 0 || run <= 0 || run % 8 != 0 ||
        ((uintptr_t)colIdx) % 16 != 0 || ((uintptr_t)B) % 16 != 0 || ldB % 4 != 0)
        return -1;
    const int nvec = dim / 4;
    cudaStream_t st = (cudaStream_t)stream;
    const int lpr = gather_lanes(dim);
    const int64_t groups = (nnz + run - 1) / run;
    const unsigned grid = (unsigned)((groups * lpr + 255) / 256);
    for (int v0 = 0; v0 < nvec; v0 += lpr) {
        const float *b = B + (int64_t)v0 * 4;
        const int active = nvec - v0 < lpr ? nvec - v0 : lpr;
        if (lpr == 4)
            gather_ceiling_kernel<4><<<grid, 256, 0, st>>>(colIdx, nnz, b, ldB, run, active, (float4 *)sink);
        else if (lpr == 8)
            gather_ceiling_kernel<8><<<grid, 256, 0, st>>>(colIdx, nnz, b, ldB, run, active, (float4 *)sink);
        else if (lpr == 16)
            gather_ceiling_kernel<16><<<grid, 256, 0, st>>>(colIdx, nnz, b, ldB, run, active, (float4 *)sink);
        else
            gather_ceiling_kernel<32><<<grid, 256, 0, st>>>(colIdx, nnz, b, ldB, run, active, (float4 *)sink);
    }
    PB_CUDA(cudaGetLastError());
    return 0;
}
