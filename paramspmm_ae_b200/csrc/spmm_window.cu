// Window SpMM kernel for sm_100a: C = A B for CSR matrices whose rows reference NEARBY rows of B
// (banded and locality-ordered matrices).
//
// The segment kernel (spmm_kernel.cuh) fetches a row of B from global memory for every entry.  When
// the rows of a block of A reference a narrow range of columns, every row of B in that range is
// fetched many times by the same SM and the L1 data path becomes the limit.  Here a CTA that owns
// `cta_rows` consecutive rows of A first copies the rows [lo, lo + window_rows) of B, restricted to
// its tile of 4*LPR dense columns, into shared memory with asynchronous 16-byte copies (cp.async,
// no register staging), where lo is the smallest column any of its rows starts with; entries then
// read their row of B from shared memory with one conflict-free 128-bit load per lane.  An entry
// whose column falls outside the window is fetched from global memory as before, so the result is
// right for every matrix; the path only pays off when nearly all entries hit (the decider checks).
//
// Work split: lane groups of LPR lanes (16 or 32) own one row at a time; lane gl holds the dense
// columns [(tile*LPR + gl)*4, +4).  The (column, value) pairs of a row are staged LPR at a time in
// a small per-warp area (lane j loads entry j: coalesced) and read back two at a time with one
// broadcast 128-bit load.  Several CTAs are resident per SM (64 KB windows), so the window copy of
// one overlaps the arithmetic of the others.
#include <limits.h>

#include "pspmm_common.cuh"
#include "vec_ops.cuh"

namespace {

struct WindowArgs {
    const int32_t *rowPtr;
    const int32_t *colIdx;
    const float *val;
    const float *B;
    float *C;
    int64_t n_rows, n_cols, ldB, ldC;
    int32_t nvec;         // dim / 4
    int32_t cta_rows;     // rows of A per CTA
    int32_t window_rows;  // rows of B staged per CTA
};

__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem)
{
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}

template <int LPR>
__global__ void __launch_bounds__(256) spmm_window_kernel(const WindowArgs a)
{
    constexpr int G = 32 / LPR;  // rows a warp works on at a time
    extern __shared__ __align__(16) float4 smem4[];
    float4 *win = smem4;                                                        // [window_rows][LPR]
    int2 *stage_all = reinterpret_cast<int2 *>(win + (size_t)a.window_rows * LPR);  // [warps][32]
    __shared__ int s_lo;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int g = lane / LPR, gl = lane % LPR;
    const int64_t row0 = (int64_t)blockIdx.x * a.cta_rows;
    const int nrows = (a.n_rows - row0 < a.cta_rows) ? (int)(a.n_rows - row0) : a.cta_rows;

    // ---- where the window starts: the smallest first column of the CTA's rows (columns ascend in a row)
    if (tid == 0)
        s_lo = INT_MAX;
    __syncthreads();
    int mn = INT_MAX;
    for (int i = tid; i < nrows; i += blockDim.x) {
        const int b = __ldg(a.rowPtr + row0 + i), e = __ldg(a.rowPtr + row0 + i + 1);
        if (e > b)
            mn = min(mn, __ldg(a.colIdx + b));
    }
    mn = __reduce_min_sync(PSPMM_FULL_MASK, mn);
    if (lane == 0 && mn != INT_MAX)
        atomicMin(&s_lo, mn);
    __syncthreads();
    const int lo = (s_lo == INT_MAX) ? 0 : s_lo;
    const int64_t left = a.n_cols - lo;
    const int wr = left < a.window_rows ? (int)(left < 0 ? 0 : left) : a.window_rows;

    // ---- copy the window: rows [lo, lo + wr) of B, this CTA's tile of dense columns
    const int v0 = blockIdx.y * LPR;
    {
        const float *src = a.B + (int64_t)lo * a.ldB + (int64_t)v0 * 4;
        for (int i = tid; i < wr * LPR; i += blockDim.x) {
            const int r = i / LPR, v = i % LPR;
            if (v0 + v < a.nvec)
                cp_async_16(win + i, src + (int64_t)r * a.ldB + v * 4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();

    const bool act = v0 + gl < a.nvec;
    const float *bcol = a.B + (act ? (int64_t)(v0 + gl) * 4 : 0);
    int2 *stage = stage_all + warp * 32 + g * LPR;
    const unsigned long long stream = l2_policy_stream();

    for (int base = warp * G; base < nrows; base += nwarp * G) {  // warp-uniform trip count
        const int rr = base + g;
        const bool live = rr < nrows;
        int rb = 0, re = 0;
        if (live) {
            rb = __ldg(a.rowPtr + row0 + rr);
            re = __ldg(a.rowPtr + row0 + rr + 1);
        }
        const int len = re - rb;
        const int maxlen = (G == 1) ? len : __reduce_max_sync(PSPMM_FULL_MASK, len);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int off = 0; off < maxlen; off += LPR) {
            const int cnt = (len - off < LPR) ? (len - off) : LPR;  // entries of this group's row in the chunk (may be <= 0)
            {
                const int k = rb + off + gl;
                int2 cv = make_int2(lo, 0);  // slots past the row's end: an in-window column, never used in the sum
                if (gl < cnt)
                    cv = make_int2(ldg_stream_b32(a.colIdx + k, stream), ldg_stream_b32(a.val + k, stream));
                stage[gl] = cv;
            }
            __syncwarp();
#pragma unroll 1
            for (int j = 0; j < cnt; j += 4) {
                const int4 p0 = *reinterpret_cast<const int4 *>(stage + j);
                const int4 p1 = *reinterpret_cast<const int4 *>(stage + j + 2);
                const int c[4] = {p0.x, p0.z, p1.x, p1.z};
                const float v[4] = {__int_as_float(p0.y), __int_as_float(p0.w), __int_as_float(p1.y),
                                    __int_as_float(p1.w)};
                float4 x[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const unsigned rel = (unsigned)(c[u] - lo);
                    if (rel < (unsigned)wr)
                        x[u] = win[rel * LPR + gl];
                    else if (act)  // outside the staged range: from global memory, as the segment kernel does
                        x[u] = __ldg(reinterpret_cast<const float4 *>(bcol + (int64_t)c[u] * a.ldB));
                    else
                        x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (j + u < cnt) {  // a predicate, not a zero factor: 0 * inf must not reach the sum
                        acc[0] = fmaf(v[u], x[u].x, acc[0]);
                        acc[1] = fmaf(v[u], x[u].y, acc[1]);
                        acc[2] = fmaf(v[u], x[u].z, acc[2]);
                        acc[3] = fmaf(v[u], x[u].w, acc[3]);
                    }
                }
            }
            __syncwarp();  // everyone has read the staged pairs before they are overwritten
        }
        if (live && act)
            st_vec_hint<4>(a.C + (row0 + rr) * a.ldC + (int64_t)(v0 + gl) * 4, acc, stream);
    }
}

template <int LPR>
int launch(const WindowArgs &a, cudaStream_t st)
{
    const int threads = 256;
    const size_t smem = (size_t)a.window_rows * LPR * 16 + (threads / 32) * 32 * sizeof(int2);
    auto kern = spmm_window_kernel<LPR>;
    if (smem > 48 * 1024)
        PSPMM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t gx = (a.n_rows + a.cta_rows - 1) / a.cta_rows;
    const int64_t gy = (a.nvec + LPR - 1) / LPR;
    if (gx > INT32_MAX || gy > 65535)
        return PSPMM_E_RANGE;
    kern<<<dim3((unsigned)gx, (unsigned)gy, 1), threads, smem, st>>>(a);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

}  // namespace

// Called by pspmm_spmm_csr when pspmm_cfg.window_rows > 0 and the call is a plain CSR product with
// 128-bit accessible operands; returns PSPMM_E_UNSUPPORTED for anything else, and the caller then
// takes the segment kernel.
int pspmm_launch_spmm_window(const int32_t *rowPtr, const int32_t *colIdx, const float *val, const float *B,
                             float *C, int64_t n_rows, int64_t n_cols, int32_t dim, int64_t ldB, int64_t ldC,
                             int32_t window_rows, int32_t cta_rows, int32_t lanes_per_row, cudaStream_t st)
{
    if (dim % 4 != 0 || ldB % 4 != 0 || ldC % 4 != 0 || ((uintptr_t)B) % 16 != 0 || ((uintptr_t)C) % 16 != 0)
        return PSPMM_E_UNSUPPORTED;
    WindowArgs a;
    a.rowPtr = rowPtr;
    a.colIdx = colIdx;
    a.val = val;
    a.B = B;
    a.C = C;
    a.n_rows = n_rows;
    a.n_cols = n_cols;
    a.ldB = ldB;
    a.ldC = ldC;
    a.nvec = dim / 4;
    int lpr = lanes_per_row;
    if (lpr != 16 && lpr != 32)
        lpr = a.nvec > 16 ? 32 : 16;
    // the window and the staging area must fit the 227 KB a CTA can have
    const int64_t cap_rows = (227 * 1024 - 8 * 32 * 8 - 64) / (lpr * 16);
    a.window_rows = window_rows > cap_rows ? (int32_t)cap_rows : window_rows;
    a.cta_rows = cta_rows > 0 ? cta_rows : (a.window_rows >= 2 ? a.window_rows / 2 : 1);
    return lpr == 32 ? launch<32>(a, st) : launch<16>(a, st);
}
