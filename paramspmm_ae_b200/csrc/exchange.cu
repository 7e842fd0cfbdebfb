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

}  // namespace

extern "C" int pspmm_pull_rows(const pspmm_row_sources *sources, const int32_t *rows, int64_t n,
                               float *dst, int32_t dim, int64_t ld_src, int64_t ld_dst, int64_t rotate,
                               int32_t ctas, void *stream)
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
    constexpr int U = 4;
    const int64_t want = (n + 8 * U - 1) / (8 * U);  // CTAs that would each do one step
    int64_t grid = ctas > 0 ? ctas : 64;
    if (grid > want)
        grid = want;
    pull_rows_kernel<U><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(a);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}
