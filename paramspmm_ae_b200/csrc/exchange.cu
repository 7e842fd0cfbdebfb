// Row pull for the multi-GPU exchange step of the row-sharded SpMM: every rank copies the rows of
// the dense operand that its shard of A references out of the owners' blocks into one compact
// local buffer.  The owners' blocks are plain device pointers: this GPU's own memory or peer
// memory mapped into this process (NVLink), read with ordinary 16-byte loads, no TMA, no
// multicast, no spin-wait on anything a peer writes.  Ordering against the producers and the
// other readers is the caller's business (a barrier before and after, see shard.py).
//
// One warp moves U rows at a time: U independent 16-byte loads in flight per lane, issued before
// the stores, so a few dozen CTAs keep enough bytes in flight to fill the links while the rest of
// the GPU runs the SpMM of the previous chunk.
#include "pspmm_common.cuh"

namespace {

struct PullArgs {
    const float *base[PSPMM_MAX_ROW_SOURCES];
    int64_t first[PSPMM_MAX_ROW_SOURCES + 1];
    const int32_t *rows;
    float *dst;
    int64_t n, rotate, ld_src, ld_dst;
    int32_t nvec, n_src;
};

template <int U>
__global__ void __launch_bounds__(256) pull_rows_kernel(const PullArgs a)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t blk = warp * U; blk < a.n; blk += nwarps * U) {
        const float4 *src[U];
        float4 *dst[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            ok[u] = blk + u < a.n;
            // the list is walked from `rotate` on, wrapping round, so that the ranks of a node do
            // not all read from the same owner at the same moment
            int64_t j = ok[u] ? blk + u + a.rotate : 0;
            if (j >= a.n)
                j -= a.n;
            int s = 0;
            while (s + 1 < a.n_src && j >= a.first[s + 1])
                ++s;
            const int32_t r = __ldg(a.rows + j);
            src[u] = reinterpret_cast<const float4 *>(a.base[s] + (int64_t)r * a.ld_src);
            dst[u] = reinterpret_cast<float4 *>(a.dst + j * a.ld_dst);
        }
        for (int v = lane; v < a.nvec; v += 32) {
            float4 x[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (ok[u])
                    x[u] = __ldcs(src[u] + v);  // read once: streaming
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (ok[u])
                    dst[u][v] = x[u];  // plain store: the SpMM gathers these rows next
        }
    }
}

// The same copy through the bulk asynchronous copy unit: a row travels global (this GPU's or a
// peer's memory) -> shared memory -> global as two cp.async.bulk transfers, completion of the first
// counted on an mbarrier.  One warp per thread block, lane l owning slot l of every stage of a ring
// in shared memory: no registers hold data and the warp only issues copies, so the block takes one
// warp slot and its shared memory from the SM while tens of kilobytes are in flight per block.  That
// is what a fetch that runs beside the SpMM wants: the SpMM is latency-bound and slows down in
// proportion to the warps and registers the copy takes from it.  No multicast, no tensor map: plain
// untiled bulk copies of 16-byte aligned rows.  Every wait is bounded; a wait that runs out sets
// the status word and the block stops issuing work.
constexpr int BULK_ROWS = 16;  // rows per stage

__device__ int g_pull_status = 0;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t now_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for the phase with this parity for at most `limit_ns`; false when the time ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns)
{
    const uint64_t t0 = now_ns();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok)
            return true;
        if (now_ns() - t0 > limit_ns)
            return false;
    }
}

template <int S>
__global__ void __launch_bounds__(32) pull_rows_bulk_kernel(const PullArgs a, const uint32_t row_bytes)
{
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ __align__(8) uint64_t full[S];
    const int lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < S; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&full[s])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    const int64_t nb = (a.n + BULK_ROWS - 1) / BULK_ROWS;
    const int64_t mine = blockIdx.x < nb ? (nb - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    constexpr int AHEAD = S - 2;  // stages of loads in flight before the oldest is stored
    const uint32_t slot = lane * row_bytes;
    bool alive = true;
    for (int64_t i = 0; i < mine + AHEAD && alive; ++i) {
        if (i < mine) {
            const int s = (int)(i % S);
            // the stores that last read this stage were committed two steps ago
            if (i >= S)
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            const int64_t blk = (blockIdx.x + i * (int64_t)gridDim.x) * BULK_ROWS;
            const int64_t left = a.n - blk;
            const int valid = left < BULK_ROWS ? (int)left : BULK_ROWS;
            const uint32_t bar = smem_addr(&full[s]);
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(valid * row_bytes) : "memory");
            __syncwarp();
            if (lane < valid) {
                int64_t j = blk + lane + a.rotate;
                if (j >= a.n)
                    j -= a.n;
                int src = 0;
                while (src + 1 < a.n_src && j >= a.first[src + 1])
                    ++src;
                const float *from = a.base[src] + (int64_t)__ldg(a.rows + j) * a.ld_src;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_addr(ring) + s * (BULK_ROWS * row_bytes) + slot),
                               "l"(__cvta_generic_to_global(from)), "r"(row_bytes), "r"(bar) : "memory");
            }
        }
        const int64_t c = i - AHEAD;
        if (c >= 0) {
            const int s = (int)(c % S);
            // (the verdict is taken by the whole warp, so that all lanes leave the loop together)
            if (!__all_sync(PSPMM_FULL_MASK, mbar_wait(smem_addr(&full[s]), (uint32_t)((c / S) & 1), 500000000ull))) {
                atomicExch(&g_pull_status, 1);  // a load did not arrive within half a second
                alive = false;
                break;
            }
            const int64_t blk = (blockIdx.x + c * (int64_t)gridDim.x) * BULK_ROWS;
            if (blk + lane < a.n && lane < BULK_ROWS) {
                int64_t j = blk + lane + a.rotate;
                if (j >= a.n)
                    j -= a.n;
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(__cvta_generic_to_global(a.dst + j * a.ld_dst)),
                               "r"(smem_addr(ring) + s * (BULK_ROWS * row_bytes) + slot), "r"(row_bytes) : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
    if (!alive) {
        // loads still in flight write into this block's shared memory: give each stage one more
        // bounded wait before the block returns
        for (int s = 0; s < S; ++s)
            if (!mbar_wait(smem_addr(&full[s]), 0, 20000000ull))
                mbar_wait(smem_addr(&full[s]), 1, 20000000ull);
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

template <int S>
int launch_bulk(const PullArgs &a, uint32_t row_bytes, unsigned grid, cudaStream_t st)
{
    const size_t bytes = (size_t)S * BULK_ROWS * row_bytes;
    PSPMM_CUDA_TRY(cudaFuncSetAttribute(pull_rows_bulk_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    pull_rows_bulk_kernel<S><<<grid, 32, bytes, st>>>(a, row_bytes);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

int pull_rows_impl(const pspmm_row_sources *sources, const int32_t *rows, int64_t n, float *dst, int32_t dim,
                   int64_t ld_src, int64_t ld_dst, int64_t rotate, int32_t ctas, void *stream, bool bulk);

}  // namespace

extern "C" int pspmm_pull_rows(const pspmm_row_sources *sources, const int32_t *rows, int64_t n,
                               float *dst, int32_t dim, int64_t ld_src, int64_t ld_dst, int64_t rotate,
                               int32_t ctas, void *stream)
{
    return pull_rows_impl(sources, rows, n, dst, dim, ld_src, ld_dst, rotate, ctas, stream, false);
}

extern "C" int pspmm_pull_rows_bulk(const pspmm_row_sources *sources, const int32_t *rows, int64_t n,
                                    float *dst, int32_t dim, int64_t ld_src, int64_t ld_dst, int64_t rotate,
                                    int32_t ctas, void *stream)
{
    return pull_rows_impl(sources, rows, n, dst, dim, ld_src, ld_dst, rotate, ctas, stream, true);
}

extern "C" int pspmm_pull_rows_status(int32_t *status)
{
    if (!status)
        return PSPMM_E_ARG;
    int v = 0;
    PSPMM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_pull_status, sizeof(int)));
    *status = v;
    return PSPMM_OK;
}

namespace {

int pull_rows_impl(const pspmm_row_sources *sources, const int32_t *rows, int64_t n, float *dst, int32_t dim,
                   int64_t ld_src, int64_t ld_dst, int64_t rotate, int32_t ctas, void *stream, bool bulk)
{
    if (!sources || n < 0 || dim <= 0 || ld_src < dim || ld_dst < dim || ctas < 0)
        return PSPMM_E_ARG;
    if (sources->n_src < 1 || sources->n_src > PSPMM_MAX_ROW_SOURCES || rotate < 0 || (n > 0 && rotate >= n))
        return PSPMM_E_ARG;
    if (n == 0)
        return PSPMM_OK;
    if (!rows || !dst)
        return PSPMM_E_ARG;
    if (dim % 4 != 0 || ld_src % 4 != 0 || ld_dst % 4 != 0 || ((uintptr_t)dst) % 16 != 0)
        return PSPMM_E_UNSUPPORTED;
    PullArgs a;
    a.n_src = sources->n_src;
    if (sources->first[0] != 0 || sources->first[a.n_src] != n)
        return PSPMM_E_ARG;
    for (int s = 0; s < PSPMM_MAX_ROW_SOURCES; ++s) {
        const bool used = s < a.n_src;
        a.base[s] = used ? sources->base[s] : nullptr;
        a.first[s + 1] = used ? sources->first[s + 1] : n;
        if (used && sources->first[s + 1] < sources->first[s])
            return PSPMM_E_ARG;
        if (used && sources->first[s + 1] > sources->first[s] &&
            (!sources->base[s] || ((uintptr_t)sources->base[s]) % 16 != 0))
            return PSPMM_E_ARG;
    }
    a.first[0] = 0;
    a.rows = rows;
    a.dst = dst;
    a.n = n;
    a.rotate = rotate;
    a.ld_src = ld_src;
    a.ld_dst = ld_dst;
    a.nvec = dim / 4;
    int64_t grid = ctas > 0 ? ctas : 64;
    if (bulk) {
        // ring of S stages of 16 rows in at most 96 KB of shared memory; rows too long for four
        // stages go through the load/store kernel
        const uint32_t row_bytes = (uint32_t)dim * 4u;
        const int64_t stages = (96 * 1024) / ((int64_t)BULK_ROWS * row_bytes);
        const int64_t batches = (n + BULK_ROWS - 1) / BULK_ROWS;
        if (grid > batches)
            grid = batches;
        if (stages >= 8)
            return launch_bulk<8>(a, row_bytes, (unsigned)grid, (cudaStream_t)stream);
        if (stages >= 6)
            return launch_bulk<6>(a, row_bytes, (unsigned)grid, (cudaStream_t)stream);
        if (stages >= 4)
            return launch_bulk<4>(a, row_bytes, (unsigned)grid, (cudaStream_t)stream);
    }
    constexpr int U = 4;
    const int64_t want = (n + 8 * U - 1) / (8 * U);  // CTAs that would each do one step
    if (grid > want)
        grid = want;
    pull_rows_kernel<U><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(a);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

}  // namespace
