// C ABI of libpspmm: argument checks, launch-shape resolution and kernel launches.
#include <stdio.h>
#include <string.h>

#include "pspmm_common.cuh"
#include "vec_ops.cuh"

// ----------------------------------------------------------------------------- errors
static thread_local char g_cuda_err[256] = "";

int pspmm_note_cuda_error(cudaError_t e)
{
    const char *name = cudaGetErrorName(e);
    const char *text = cudaGetErrorString(e);
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", name ? name : "?", text ? text : "?");
    return PSPMM_E_CUDA;
}

extern "C" const char *pspmm_last_cuda_error(void) { return g_cuda_err; }

extern "C" int pspmm_version(void) { return 100; }

extern "C" const char *pspmm_strerror(int code)
{
    switch (code) {
    case PSPMM_OK: return "ok";
    case PSPMM_E_ARG: return "invalid argument (null pointer, negative size or leading dimension smaller than dim)";
    case PSPMM_E_CONFIG: return "invalid configuration (CF must be 1..8 (1..4 for SDDMM), blkWarpNum 4 or 8, lanes_per_row a power of two <= 32, vec_width 1/2/4, cta_threads 32/64/128/256, rows_per_group 1..16)";
    case PSPMM_E_CUDA: return "CUDA error (see pspmm_last_cuda_error)";
    case PSPMM_E_UNSUPPORTED: return "unsupported combination";
    case PSPMM_E_RANGE: return "size exceeds the int32 index range (or, for pspmm_split_csr_device_static, the 16,777,216 rows its built-in scratch covers)";
    case PSPMM_E_IO: return "file cannot be opened, mapped, written or renamed";
    case PSPMM_E_FORMAT: return "file contents contradict the header or the checksum";
    case PSPMM_E_NOMEM: return "out of host memory";
    default: return "unknown error code";
    }
}

// ----------------------------------------------------------------------------- configuration
static bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

int pspmm_validate_cfg(const pspmm_cfg *cfg, bool sddmm)
{
    if (!cfg)
        return PSPMM_OK;
    // The legacy pair keeps the reference's domain (SpMM/SpMM.cpp:110,139; SDDMM/sddmm.cpp:31-43).
    if (cfg->hint_CF != 0 && (cfg->hint_CF < 1 || cfg->hint_CF > (sddmm ? 4 : 8)))
        return PSPMM_E_CONFIG;
    if (cfg->hint_blkWarpNum != 0 && cfg->hint_blkWarpNum != 4 && cfg->hint_blkWarpNum != 8)
        return PSPMM_E_CONFIG;
    if (cfg->lanes_per_row != 0 && (!is_pow2(cfg->lanes_per_row) || cfg->lanes_per_row > 32))
        return PSPMM_E_CONFIG;
    if (cfg->vec_width != 0 && cfg->vec_width != 1 && cfg->vec_width != 2 && cfg->vec_width != 4)
        return PSPMM_E_CONFIG;
    if (cfg->cta_threads != 0 && cfg->cta_threads != 32 && cfg->cta_threads != 64 && cfg->cta_threads != 128 &&
        cfg->cta_threads != 256)
        return PSPMM_E_CONFIG;
    if (cfg->rows_per_group < 0 || cfg->rows_per_group > PSPMM_RPG_MAX)
        return PSPMM_E_CONFIG;
    if (cfg->accumulate != 0 && (cfg->accumulate != 1 || sddmm))
        return PSPMM_E_CONFIG;
    if (cfg->gather_batch != 0 && cfg->gather_batch != 2 && cfg->gather_batch != 4 &&
        cfg->gather_batch != 8 && cfg->gather_batch != 16)
        return PSPMM_E_CONFIG;
    if (cfg->col_tile < 0 || cfg->col_tile % 4 != 0)
        return PSPMM_E_CONFIG;
    if (cfg->bucketed != 0 && (cfg->bucketed != 1 || sddmm))
        return PSPMM_E_CONFIG;
    return PSPMM_OK;
}

// Widest vector width the operands allow: every row start must be aligned to it.
int pspmm_vw_max(int32_t dim, int64_t ld0, int64_t ld1, const void *p0, const void *p1)
{
    const uintptr_t a0 = (uintptr_t)p0, a1 = (uintptr_t)p1;
    if (dim % 4 == 0 && ld0 % 4 == 0 && ld1 % 4 == 0 && a0 % 16 == 0 && a1 % 16 == 0)
        return 4;
    if (dim % 2 == 0 && ld0 % 2 == 0 && ld1 % 2 == 0 && a0 % 8 == 0 && a1 % 8 == 0)
        return 2;
    return 1;
}

// Which (lanes per row, coarsening) pairs exist per vector width and block height; must
// mirror the instantiation lists in spmm_vw*.cu / sddmm_vw*.cu.
static int lpr_min_for(int vw, int V)
{
    if (vw == 4)
        return V == 1 ? 2 : (V == 2 ? 4 : 16);
    return V == 1 ? 8 : (V == 2 ? 16 : 32);
}
static int cf_max_for(int vw, int V)
{
    if (vw == 4)
        return V == 1 ? 8 : (V == 2 ? 4 : 2);
    if (vw == 2)
        return V == 3 ? 4 : 8;
    return 8;
}

int pspmm_resolve_shape(const pspmm_cfg *cfg, int32_t dim, int vw_max, int V, LaunchShape *out)
{
    LaunchShape s;
    s.vw = vw_max;
    if (cfg && cfg->vec_width != 0 && cfg->vec_width < vw_max)
        s.vw = cfg->vec_width;
    const int nvec = dim / s.vw;
    const int lmin = lpr_min_for(s.vw, V), cmax = cf_max_for(s.vw, V);
    int lpr;
    if (cfg && cfg->lanes_per_row != 0) {
        lpr = cfg->lanes_per_row;
    } else {
        lpr = 1;
        while (lpr < nvec && lpr < 32)
            lpr <<= 1;
    }
    if (lpr < lmin)
        lpr = lmin;
    int need = (nvec + lpr - 1) / lpr;
    // A narrow group would need more accumulators than are instantiated: widen it first.
    while (need > cmax && lpr < 32) {
        lpr <<= 1;
        need = (nvec + lpr - 1) / lpr;
    }
    s.lpr = lpr;
    if (need > cmax) {
        s.cf = cmax;
        s.tiles = (nvec + lpr * cmax - 1) / (lpr * cmax);
    } else {
        s.cf = pspmm_round_cf(need);
        s.tiles = 1;
    }
    s.threads = (cfg && cfg->cta_threads) ? cfg->cta_threads : 256;
    s.rpg = (cfg && cfg->rows_per_group) ? cfg->rows_per_group : 4;
    s.mlp = (cfg && cfg->gather_batch) ? cfg->gather_batch : 8;
    *out = s;
    return PSPMM_OK;
}

extern "C" int pspmm_resolve_cfg(pspmm_cfg *cfg, int32_t dim, int64_t ldB, int64_t ldC, int32_t V,
                                 const void *B, const void *C)
{
    if (!cfg || dim <= 0 || V < 1 || V > 3)
        return PSPMM_E_ARG;
    int rc = pspmm_validate_cfg(cfg, false);
    if (rc)
        return rc;
    LaunchShape s;
    pspmm_resolve_shape(cfg, dim, pspmm_vw_max(dim, ldB, ldC, B, C), V, &s);
    cfg->lanes_per_row = s.lpr;
    cfg->vec_width = s.vw;
    cfg->cta_threads = s.threads;
    cfg->rows_per_group = s.rpg;
    cfg->gather_batch = s.mlp;
    return PSPMM_OK;
}

// ----------------------------------------------------------------------------- zero pre-pass
// For a split layout, before the SpMM kernel runs.  Lane groups of the SpMM kernel own `rpg`
// consecutive segments each, so group boundaries sit at segment indices that are multiples of
// rpg; a row whose segments straddle such a boundary is accumulated with REDs and must start
// from zero.  This kernel zeroes those rows (once, from the first boundary they straddle) and
// every run of more than PSPMM_GAP_MAX rows that no segment covers (the SpMM kernel zeroes
// shorter runs itself).  Thread s looks at segment s.  Straddled rows are zeroed by the
// finding warp; long runs are queued in shared memory and zeroed by the whole CTA, one row per
// warp per step.  target_row must be non-decreasing.
__global__ void __launch_bounds__(256)
zero_shared_rows_kernel(const int32_t *__restrict__ target_row, int64_t n_seg, int64_t n_out, int rpg,
                        int V, float *C, int64_t ldC, int dim, int vecok)
{
    __shared__ int q_lo[512], q_hi[512];
    __shared__ int q_n;
    if (threadIdx.x == 0)
        q_n = 0;
    __syncthreads();
    const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const bool in = s < n_seg;
    // Own, previous and next target row: one coalesced load, neighbours by shuffle, warp edges by
    // a second load.
    const int me = in ? __ldg(target_row + s) : (int)n_out;
    int prev = __shfl_up_sync(PSPMM_FULL_MASK, me, 1);
    int next = __shfl_down_sync(PSPMM_FULL_MASK, me, 1);
    if (lane == 0)
        prev = (in && s > 0) ? __ldg(target_row + s - 1) : -1;
    if (lane == 31)
        next = (s + 1 < n_seg) ? __ldg(target_row + s + 1) : (int)n_out;
    int one = -1;  // a straddled row to zero, or -1
    if (in) {
        if (s > 0 && s % rpg == 0 && prev == me) {
            const int64_t before = s - rpg - 1;  // last segment ahead of the previous boundary
            if (before < 0 || __ldg(target_row + before) != me)
                one = me;
        }
        if (next - me - 1 > PSPMM_GAP_MAX) {
            const int i = atomicAdd(&q_n, 1);
            q_lo[i] = me + 1;
            q_hi[i] = next;
        }
        if (s == 0 && me > PSPMM_GAP_MAX) {
            const int i = atomicAdd(&q_n, 1);
            q_lo[i] = 0;
            q_hi[i] = me;
        }
    }
    // Straddled rows: the finding warp zeroes them, 32 / lanes_per_row rows per step.
    const int lpr_z = vecok ? ((dim + 3) / 4 < 32 ? (dim + 3) / 4 : 32) : 32;  // lanes that cover one row
    int lanes_row = 1;
    while (lanes_row < lpr_z)
        lanes_row <<= 1;
    const int rows_step = 32 / lanes_row;
    const int sub = lane / lanes_row, sl = lane % lanes_row;
    auto zero_part = [&](int64_t r, int l, int nl) {  // lanes l of nl zero row r
        float *row = C + r * ldC;
        if (vecok) {
            for (int j = l * 4; j < dim; j += nl * 4)
                *reinterpret_cast<float4 *>(row + j) = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int j = l; j < dim; j += nl)
                row[j] = 0.f;
        }
    };
    unsigned todo = __ballot_sync(PSPMM_FULL_MASK, one >= 0);
    while (todo) {
        // pick the sub-th pending lane for this sub-group
        unsigned t = todo;
        int src = -1;
        for (int k = 0; k <= sub && t; ++k) {
            src = __ffs(t) - 1;
            t &= t - 1;
        }
        const bool have = __popc(todo) > sub;
        const int r = __shfl_sync(PSPMM_FULL_MASK, one, have ? src : 0);
        if (have)
            for (int w = 0; w < V; ++w)
                zero_part((int64_t)r * V + w, sl, lanes_row);
        for (int k = 0; k < rows_step && todo; ++k)
            todo &= todo - 1;
    }
    if (__syncthreads_or(q_n > 0) == 0)
        return;
    // Long uncovered runs: the whole CTA zeroes them, rows_step * warps rows per step.
    const int warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int i = 0; i < q_n; ++i)
        for (int64_t r = (int64_t)q_lo[i] * V + warp * rows_step + sub; r < (int64_t)q_hi[i] * V; r += nwarp * rows_step)
            zero_part(r, sl, lanes_row);
}

// Pre-pass of a length-bucketed plan: rows that are cut into several segments receive REDs from all
// of them and must start from zero; the segment flagged as the first one of its row zeroes it.
// (Rows with a single segment, empty ones included, are stored by the SpMM kernel itself.)
// One warp looks at 32 segments and zeroes the flagged rows one after the other, all lanes on a row.
__global__ void __launch_bounds__(256)
zero_first_pieces_kernel(const int32_t *__restrict__ target_row, int64_t n_seg, int V, float *C, int64_t ldC,
                         int dim, int vecok)
{
    const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    const unsigned t = s < n_seg ? (unsigned)__ldg(target_row + s) : 0u;
    unsigned todo = __ballot_sync(PSPMM_FULL_MASK, (t & PSPMM_SEG_FIRST) != 0);
    while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const int64_t r = (int64_t)(__shfl_sync(PSPMM_FULL_MASK, t, src) & PSPMM_SEG_ROW_MASK);
        for (int w = 0; w < V; ++w) {
            float *row = C + (r * V + w) * ldC;
            if (vecok) {
                for (int j = lane * 4; j < dim; j += 128)
                    *reinterpret_cast<float4 *>(row + j) = make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                for (int j = lane; j < dim; j += 32)
                    row[j] = 0.f;
            }
        }
    }
}

// ----------------------------------------------------------------------------- SpMM
static int check_sizes(int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t dim)
{
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || dim <= 0)
        return PSPMM_E_ARG;
    if (n_rows >= INT32_MAX || n_cols > INT32_MAX || nnz > INT32_MAX)
        return PSPMM_E_RANGE;
    return PSPMM_OK;
}

// Fraction of the gathered operand to pin in L2: all of it when it fits in about three quarters
// of the cache, otherwise the share that does.
static float l2_keep_fraction(double operand_bytes)
{
    static thread_local int cached_dev = -1;
    static thread_local double l2_bytes = 0.0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess)
        return 1.0f;
    if (dev != cached_dev) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) != cudaSuccess || v <= 0)
            v = 64 << 20;
        l2_bytes = (double)v;
        cached_dev = dev;
    }
    const double budget = 0.75 * l2_bytes;
    if (operand_bytes <= budget)
        return 1.0f;
    const double f = budget / operand_bytes;
    return (float)(f < 0.02 ? 0.02 : f);
}

static int spmm_launch(const int32_t *segPtr, const int32_t *target_row, int64_t n_seg,
                       const int32_t *colIdx, const float *val, int V, const float *B, float *C,
                       int64_t n_out_blk_rows, int64_t n_cols, int32_t dim, int64_t ldB, int64_t ldC,
                       const pspmm_cfg *cfg, cudaStream_t st)
{
    int rc = pspmm_validate_cfg(cfg, false);
    if (rc)
        return rc;
    if (n_out_blk_rows == 0)
        return PSPMM_OK;
    const bool accumulate = cfg && cfg->accumulate;
    if (n_seg == 0 && accumulate)
        return PSPMM_OK;  // nothing stored: nothing to add
    if (n_seg == 0) {  // nothing stored: the product is zero
        PSPMM_CUDA_TRY(cudaMemset2DAsync(C, (size_t)ldC * 4, 0, (size_t)dim * 4,
                                         (size_t)(n_out_blk_rows * V), st));
        return PSPMM_OK;
    }
    if (cfg && cfg->col_tile > 0 && cfg->col_tile < dim) {
        // Column ranges as separate launches: a 128-wide launch keeps one 16-byte slice per lane,
        // and a narrow remainder gets a narrow lane group instead of idle lanes in a wide one.
        for (int32_t off = 0; off < dim; off += cfg->col_tile) {
            const int32_t w = dim - off < cfg->col_tile ? dim - off : cfg->col_tile;
            pspmm_cfg sub = *cfg;
            sub.col_tile = 0;
            if (sub.lanes_per_row * (sub.vec_width ? sub.vec_width : 4) > w)
                sub.lanes_per_row = 0;  // let the launch pick the group width for the narrow range
            rc = spmm_launch(segPtr, target_row, n_seg, colIdx, val, V, B + off, C + off, n_out_blk_rows, n_cols, w,
                             ldB, ldC, &sub, st);
            if (rc)
                return rc;
        }
        return PSPMM_OK;
    }
    LaunchShape s;
    pspmm_resolve_shape(cfg, dim, pspmm_vw_max(dim, ldB, ldC, B, C), V, &s);
    if (accumulate) {
        // built for 128-bit loads on CSR / split CSR with at least four lanes per row
        if (s.vw != 4 || V != 1)
            return PSPMM_E_UNSUPPORTED;
        if (s.lpr < 4) {
            LaunchShape t = s;
            pspmm_cfg wide = *cfg;
            wide.lanes_per_row = 4;
            pspmm_resolve_shape(&wide, dim, 4, V, &t);
            s = t;
        }
    }

    const bool bucketed = target_row && cfg && cfg->bucketed;
    if (target_row && !accumulate) {
        const int vecok = (dim % 4 == 0 && ldC % 4 == 0 && ((uintptr_t)C) % 16 == 0) ? 1 : 0;
        if (bucketed)
            zero_first_pieces_kernel<<<(unsigned)((n_seg + 255) / 256), 256, 0, st>>>(target_row, n_seg, V, C, ldC,
                                                                                      dim, vecok);
        else
            zero_shared_rows_kernel<<<(unsigned)((n_seg + 255) / 256), 256, 0, st>>>(
                target_row, n_seg, n_out_blk_rows, s.rpg, V, C, ldC, dim, vecok);
    }

    SpmmArgs a;
    a.segPtr = segPtr;
    a.target_row = target_row;
    a.colIdx = colIdx;
    a.val = val;
    a.B = B;
    a.C = C;
    a.n_seg = n_seg;
    a.n_out = n_out_blk_rows;
    a.ldB = ldB;
    a.ldC = ldC;
    a.nvec = dim / s.vw;
    a.rows_per_group = s.rpg;
    a.bucketed = bucketed ? 1 : 0;
    a.keep_fraction = l2_keep_fraction((double)n_cols * (double)ldB * 4.0);
    const int64_t per_cta = (int64_t)(s.threads / s.lpr) * s.rpg;
    const int64_t gx = (n_seg + per_cta - 1) / per_cta;
    if (gx > INT32_MAX || s.tiles > 65535)
        return PSPMM_E_RANGE;
    dim3 grid((unsigned)gx, (unsigned)s.tiles, 1);
    bool ok = false;
    if (accumulate)
        ok = pspmm_launch_spmm_vw4_acc(s, a, grid, st);
    else if (s.vw == 4)
        ok = pspmm_launch_spmm_vw4(s, V, a, grid, st);
    else if (s.vw == 2)
        ok = pspmm_launch_spmm_vw2(s, V, a, grid, st);
    else
        ok = pspmm_launch_spmm_vw1(s, V, a, grid, st);
    if (!ok)
        return PSPMM_E_UNSUPPORTED;
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

extern "C" int pspmm_spmm_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                              const float *B, float *C, int64_t n_rows, int64_t n_cols,
                              int64_t nnz, int32_t dim, int64_t ldB, int64_t ldC,
                              const pspmm_cfg *cfg, const int32_t *rowPtr_split,
                              const int32_t *target_row, int64_t n_seg, void *stream)
{
    int rc = check_sizes(n_rows, n_cols, nnz, dim);
    if (rc)
        return rc;
    const bool split = target_row != nullptr || rowPtr_split != nullptr;
    if (split && (!rowPtr_split || n_seg < 0 || (n_seg > 0 && !target_row)))
        return PSPMM_E_ARG;
    if (!split && !rowPtr)
        return PSPMM_E_ARG;
    if (!B || !C || ldB < dim || ldC < dim)
        return PSPMM_E_ARG;
    if (nnz > 0 && !colIdx)
        return PSPMM_E_ARG;  // (val may be NULL: the pattern with unit values)
    if (split && n_seg >= INT32_MAX)
        return PSPMM_E_RANGE;
    return spmm_launch(split ? rowPtr_split : rowPtr, target_row, split ? n_seg : n_rows, colIdx,
                       val, 1, B, C, n_rows, n_cols, dim, ldB, ldC, cfg, (cudaStream_t)stream);
}

extern "C" int pspmm_spmm_bcsr(const int32_t *rowPtr_b, const int32_t *colIdx, const float *val,
                               int32_t V, const float *B, float *C, int64_t n_blk_rows,
                               int64_t n_cols, int64_t nblk, int32_t dim, int64_t ldB,
                               int64_t ldC, const pspmm_cfg *cfg, const int32_t *rowPtr_b_split,
                               const int32_t *target_row, int64_t n_seg, void *stream)
{
    if (V != 2 && V != 3)
        return PSPMM_E_UNSUPPORTED;
    int rc = check_sizes(n_blk_rows * V, n_cols, nblk * V, dim);
    if (rc)
        return rc;
    const bool split = target_row != nullptr || rowPtr_b_split != nullptr;
    if (split && (!rowPtr_b_split || n_seg < 0 || (n_seg > 0 && !target_row)))
        return PSPMM_E_ARG;
    if (!split && !rowPtr_b)
        return PSPMM_E_ARG;
    if (!B || !C || ldB < dim || ldC < dim)
        return PSPMM_E_ARG;
    if (nblk > 0 && (!colIdx || !val))
        return PSPMM_E_ARG;
    return spmm_launch(split ? rowPtr_b_split : rowPtr_b, target_row, split ? n_seg : n_blk_rows,
                       colIdx, val, V, B, C, n_blk_rows, n_cols, dim, ldB, ldC, cfg, (cudaStream_t)stream);
}

// ----------------------------------------------------------------------------- SDDMM
static int sddmm_launch(const int32_t *segPtr, const int32_t *target_row, int64_t n_seg,
                        const int32_t *colIdx, const float *val, int V, const float *A,
                        const float *B, float *out, int64_t n_rows_A, int32_t dim, int64_t ldA, int64_t ldB,
                        const pspmm_cfg *cfg, cudaStream_t st)
{
    int rc = pspmm_validate_cfg(cfg, true);
    if (rc)
        return rc;
    if (n_seg == 0)
        return PSPMM_OK;
    LaunchShape s;
    pspmm_resolve_shape(cfg, dim, pspmm_vw_max(dim, ldA, ldB, A, B), V, &s);
    if (!cfg || cfg->cta_threads == 0)
        s.threads = 128;  // measured: 128-thread CTAs are 7 % faster than 256 for this kernel
    SddmmArgs a;
    a.segPtr = segPtr;
    a.target_row = target_row;
    a.colIdx = colIdx;
    a.val = val;
    a.A = A;
    a.B = B;
    a.out = out;
    a.n_seg = n_seg;
    a.n_rows_A = n_rows_A;
    a.ldA = ldA;
    a.ldB = ldB;
    a.nvec = dim / s.vw;
    a.rows_per_group = s.rpg;
    a.keep_fraction = 1.0f;  // the row count of B is not part of the call: no partial pinning
    const int64_t per_cta = (int64_t)(s.threads / s.lpr) * s.rpg;
    const int64_t gx = (n_seg + per_cta - 1) / per_cta;
    if (gx > INT32_MAX)
        return PSPMM_E_RANGE;
    dim3 grid((unsigned)gx, 1, 1);
    bool ok = false;
    if (s.vw == 4)
        ok = pspmm_launch_sddmm_vw4(s, V, a, grid, st);
    else if (s.vw == 2)
        ok = pspmm_launch_sddmm_vw2(s, V, a, grid, st);
    else
        ok = pspmm_launch_sddmm_vw1(s, V, a, grid, st);
    if (!ok)
        return PSPMM_E_UNSUPPORTED;
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

extern "C" int pspmm_sddmm_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *A,
                               const float *B, float *out, int64_t n_rows, int64_t nnz,
                               int32_t dim, int64_t ldA, int64_t ldB, const pspmm_cfg *cfg,
                               const int32_t *rowPtr_split, const int32_t *target_row,
                               int64_t n_seg, void *stream)
{
    int rc = check_sizes(n_rows, 0, nnz, dim);
    if (rc)
        return rc;
    const bool split = target_row != nullptr || rowPtr_split != nullptr;
    if (split && (!rowPtr_split || n_seg < 0 || (n_seg > 0 && !target_row)))
        return PSPMM_E_ARG;
    if (!split && !rowPtr)
        return PSPMM_E_ARG;
    if (!A || !B || ldA < dim || ldB < dim)
        return PSPMM_E_ARG;
    if (nnz == 0)
        return PSPMM_OK;
    if (!colIdx || !out)
        return PSPMM_E_ARG;
    return sddmm_launch(split ? rowPtr_split : rowPtr, target_row, split ? n_seg : n_rows, colIdx,
                        nullptr, 1, A, B, out, n_rows, dim, ldA, ldB, cfg, (cudaStream_t)stream);
}

extern "C" int pspmm_sddmm_bcsr(const int32_t *rowPtr_b, const int32_t *colIdx, const float *val,
                                int32_t V, const float *A, const float *B, float *out,
                                int64_t n_blk_rows, int64_t n_rows_A, int64_t nblk, int32_t dim, int64_t ldA,
                                int64_t ldB, const pspmm_cfg *cfg, const int32_t *rowPtr_b_split,
                                const int32_t *target_row, int64_t n_seg, void *stream)
{
    if (V != 2 && V != 3)
        return PSPMM_E_UNSUPPORTED;
    int rc = check_sizes(n_blk_rows * V, 0, nblk * V, dim);
    if (rc)
        return rc;
    // A may stop inside the last block-row (a row count that is not a multiple of V), not before it.
    if (n_rows_A < 0 || (n_blk_rows > 0 && n_rows_A <= (n_blk_rows - 1) * V))
        return PSPMM_E_ARG;
    const bool split = target_row != nullptr || rowPtr_b_split != nullptr;
    if (split && (!rowPtr_b_split || n_seg < 0 || (n_seg > 0 && !target_row)))
        return PSPMM_E_ARG;
    if (!split && !rowPtr_b)
        return PSPMM_E_ARG;
    if (!A || !B || ldA < dim || ldB < dim)
        return PSPMM_E_ARG;
    if (nblk == 0)
        return PSPMM_OK;
    if (!colIdx || !val || !out)
        return PSPMM_E_ARG;
    return sddmm_launch(split ? rowPtr_b_split : rowPtr_b, target_row,
                        split ? n_seg : n_blk_rows, colIdx, val, V, A, B, out, n_rows_A, dim, ldA, ldB, cfg,
                        (cudaStream_t)stream);
}

// ----------------------------------------------------------------------------- genmask
// One warp per block-row.  Lanes take 32 blocks at a time; the position of every non-zero
// lane value inside its CSR row is the running count of earlier non-zeros in the same
// block-row column, obtained from a ballot and a prefix population count.
__global__ void genmask_kernel(const int32_t *__restrict__ rowPtr_b, const int32_t *__restrict__ rowPtr,
                               const float *__restrict__ val_b, int64_t n_blk_rows, int64_t n_rows,
                               int32_t *__restrict__ mask)
{
    const int64_t br = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (br >= n_blk_rows)
        return;  // whole warps leave together: br is warp-uniform
    const int lo = rowPtr_b[br], hi = rowPtr_b[br + 1];
    if (lo == hi)
        return;
    int cur0 = rowPtr[2 * br];
    int cur1 = (2 * br + 1 <= n_rows) ? rowPtr[2 * br + 1] : 0;
    const unsigned below = (1u << lane) - 1u;
    for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        const bool in = i < hi;
        const bool nz0 = in && val_b[2 * (int64_t)i] != 0.f;
        const bool nz1 = in && val_b[2 * (int64_t)i + 1] != 0.f;
        const unsigned b0 = __ballot_sync(PSPMM_FULL_MASK, nz0);
        const unsigned b1 = __ballot_sync(PSPMM_FULL_MASK, nz1);
        if (nz0)
            mask[cur0 + __popc(b0 & below)] = 2 * i;
        if (nz1)
            mask[cur1 + __popc(b1 & below)] = 2 * i + 1;
        cur0 += __popc(b0);
        cur1 += __popc(b1);
    }
}

extern "C" int pspmm_genmask(const int32_t *rowPtr_b, const int32_t *rowPtr, const float *val_b,
                             int64_t n_blk_rows, int64_t n_rows, int64_t nnz, int32_t *mask,
                             void *stream)
{
    if (n_blk_rows < 0 || n_rows < 0 || nnz < 0)
        return PSPMM_E_ARG;
    if (n_blk_rows * 2 < n_rows || n_blk_rows * 2 > n_rows + 1)
        return PSPMM_E_ARG;
    if (nnz > INT32_MAX || n_rows >= INT32_MAX)
        return PSPMM_E_RANGE;
    if (n_blk_rows == 0 || nnz == 0)
        return PSPMM_OK;
    if (!rowPtr_b || !rowPtr || !val_b || !mask)
        return PSPMM_E_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // The reference returns a zero-filled array with the mapped positions written into it.
    PSPMM_CUDA_TRY(cudaMemsetAsync(mask, 0, (size_t)nnz * 4, st));
    const int64_t threads = n_blk_rows * 32;
    genmask_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(rowPtr_b, rowPtr, val_b,
                                                                      n_blk_rows, n_rows, mask);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

// ----------------------------------------------------------------------------- timing loops
template <typename F>
static int time_loop(F &&launch, int warmup, int iters, float *ms, cudaStream_t st)
{
    if (warmup < 0 || iters <= 0 || !ms)
        return PSPMM_E_ARG;
    for (int i = 0; i < warmup; ++i) {
        int rc = launch();
        if (rc)
            return rc;
    }
    cudaEvent_t e0, e1;
    PSPMM_CUDA_TRY(cudaEventCreate(&e0));
    if (cudaEventCreate(&e1) != cudaSuccess) {
        cudaEventDestroy(e0);
        return pspmm_note_cuda_error(cudaGetLastError());
    }
    int rc = PSPMM_OK;
    cudaError_t ce = cudaEventRecord(e0, st);
    for (int i = 0; i < iters && rc == PSPMM_OK && ce == cudaSuccess; ++i)
        rc = launch();
    if (ce == cudaSuccess)
        ce = cudaEventRecord(e1, st);
    if (ce == cudaSuccess)
        ce = cudaEventSynchronize(e1);
    float total = 0.f;
    if (ce == cudaSuccess)
        ce = cudaEventElapsedTime(&total, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc)
        return rc;
    if (ce != cudaSuccess)
        return pspmm_note_cuda_error(ce);
    *ms = total / (float)iters;
    return PSPMM_OK;
}

extern "C" int pspmm_profile_spmm(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                                  int32_t V, const float *B, float *C, int64_t n_rows,
                                  int64_t n_cols, int64_t nnz, int32_t dim, int64_t ldB,
                                  int64_t ldC, const pspmm_cfg *cfg, const int32_t *rowPtr_split,
                                  const int32_t *target_row, int64_t n_seg, int32_t warmup,
                                  int32_t iters, float *ms_per_iter, void *stream)
{
    auto launch = [&]() -> int {
        if (V == 1)
            return pspmm_spmm_csr(rowPtr, colIdx, val, B, C, n_rows, n_cols, nnz, dim, ldB, ldC,
                                  cfg, rowPtr_split, target_row, n_seg, stream);
        return pspmm_spmm_bcsr(rowPtr, colIdx, val, V, B, C, n_rows, n_cols, nnz, dim, ldB, ldC,
                               cfg, rowPtr_split, target_row, n_seg, stream);
    };
    return time_loop(launch, warmup, iters, ms_per_iter, (cudaStream_t)stream);
}

extern "C" int pspmm_profile_sddmm(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                                   int32_t V, const float *A, const float *B, float *out,
                                   int64_t n_rows, int64_t n_rows_A, int64_t nnz, int32_t dim, int64_t ldA,
                                   int64_t ldB, const pspmm_cfg *cfg, const int32_t *rowPtr_split,
                                   const int32_t *target_row, int64_t n_seg, int32_t warmup,
                                   int32_t iters, float *ms_per_iter, void *stream)
{
    auto launch = [&]() -> int {
        if (V == 1)
            return pspmm_sddmm_csr(rowPtr, colIdx, A, B, out, n_rows, nnz, dim, ldA, ldB, cfg,
                                   rowPtr_split, target_row, n_seg, stream);
        return pspmm_sddmm_bcsr(rowPtr, colIdx, val, V, A, B, out, n_rows, n_rows_A, nnz, dim, ldA, ldB, cfg,
                                rowPtr_split, target_row, n_seg, stream);
    };
    return time_loop(launch, warmup, iters, ms_per_iter, (cudaStream_t)stream);
}
