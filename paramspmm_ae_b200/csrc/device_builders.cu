// Device-side PCSR partition: the same arrays as pspmm_split_csr (host_builders.cpp), built on the
// GPU from a device-resident rowPtr so that shards generated or received on the device never
// travel to the host.  Integer work, bit-exact with the host builder.
//
// Three kernels over tiles of TILE rows:
//   1. tile_piece_counts : pieces of every tile (sum over its rows of ceil(len / gran)) -> scratch
//   2. scan_tile_counts  : exclusive prefix sum of the tile counts, one CTA          -> scratch
//   3. fill_split        : every tile re-derives its rows' piece counts, scans them in shared
//                          memory, adds the tile offset and writes rowPtr_split / target_row
// Scratch (global memory beyond inputs and outputs): (tiles + 1) int64 values, caller-provided.
#include "pspmm_common.cuh"

namespace {

constexpr int TILE = 1024;  // rows per tile = threads per CTA

__device__ __forceinline__ int pieces_of(const int32_t *rowPtr, int64_t r, int64_t n_rows, int gran)
{
    if (r >= n_rows)
        return 0;
    const int len = rowPtr[r + 1] - rowPtr[r];
    // 64-bit: len + gran overflows int32 for a granularity near INT32_MAX
    return len > 0 ? (int)(((int64_t)len + gran - 1) / gran) : 0;
}

// CTA-wide inclusive scan of one int per thread (blockDim.x == TILE); returns the inclusive sum.
__device__ int block_inclusive_scan(int v, int *warp_sums)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(PSPMM_FULL_MASK, v, d);
        if (lane >= d)
            v += t;
    }
    if (lane == 31)
        warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];  // TILE / 32 == 32 warps
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(PSPMM_FULL_MASK, w, d);
            if (lane >= d)
                w += t;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    if (warp > 0)
        v += warp_sums[warp - 1];
    return v;
}

__global__ void __launch_bounds__(TILE) tile_piece_counts(const int32_t *__restrict__ rowPtr, int64_t n_rows,
                                                         int gran, long long *__restrict__ tile_off)
{
    __shared__ int warp_sums[32];
    const int64_t r = (int64_t)blockIdx.x * TILE + threadIdx.x;
    const int total = block_inclusive_scan(pieces_of(rowPtr, r, n_rows, gran), warp_sums);
    if (threadIdx.x == TILE - 1)
        tile_off[blockIdx.x] = total;
}

// In-place exclusive scan of tile_off[0 .. n_tiles); tile_off[n_tiles] receives the grand total.
__global__ void __launch_bounds__(1024) scan_tile_counts(long long *tile_off, int64_t n_tiles)
{
    __shared__ long long carry;
    __shared__ long long warp_sums[32];
    if (threadIdx.x == 0)
        carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t base = 0; base < n_tiles; base += 1024) {
        const int64_t i = base + threadIdx.x;
        const long long mine = i < n_tiles ? tile_off[i] : 0;
        long long v = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long t = __shfl_up_sync(PSPMM_FULL_MASK, v, d);
            if (lane >= d)
                v += t;
        }
        if (lane == 31)
            warp_sums[warp] = v;
        __syncthreads();
        if (warp == 0) {
            long long w = warp_sums[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const long long t = __shfl_up_sync(PSPMM_FULL_MASK, w, d);
                if (lane >= d)
                    w += t;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        if (warp > 0)
            v += warp_sums[warp - 1];
        const long long before = carry;
        if (i < n_tiles)
            tile_off[i] = before + v - mine;
        __syncthreads();
        if (threadIdx.x == 1023)
            carry = before + v;
        __syncthreads();
    }
    if (threadIdx.x == 0)
        tile_off[n_tiles] = carry;
}

__global__ void __launch_bounds__(TILE) fill_split(const int32_t *__restrict__ rowPtr, int64_t n_rows, int gran,
                                                  const long long *__restrict__ tile_off,
                                                  int32_t *__restrict__ rowPtr_split,
                                                  int32_t *__restrict__ target_row, int64_t n_seg)
{
    __shared__ int warp_sums[32];
    const int64_t r = (int64_t)blockIdx.x * TILE + threadIdx.x;
    const int mine = pieces_of(rowPtr, r, n_rows, gran);
    const int incl = block_inclusive_scan(mine, warp_sums);
    int64_t s = tile_off[blockIdx.x] + (incl - mine);
    if (r == 0)  // 0, or -1 when the caller's n_seg is not this partition's piece count
        rowPtr_split[0] = (tile_off[gridDim.x] == n_seg) ? 0 : -1;
    if (mine > 0) {
        const int64_t end = rowPtr[r + 1];
        for (int64_t at = rowPtr[r]; at < end; at += gran, ++s) {
            if (s < n_seg) {  // a wrong n_seg from the caller must not write out of bounds
                target_row[s] = (int32_t)r;
                rowPtr_split[s + 1] = (int32_t)(at + gran < end ? at + gran : end);
            }
        }
    }
}

int launch_counts(const int32_t *rowPtr, int64_t n_rows, int gran, long long *tile_off, cudaStream_t st)
{
    const int64_t n_tiles = (n_rows + TILE - 1) / TILE;
    tile_piece_counts<<<(unsigned)n_tiles, TILE, 0, st>>>(rowPtr, n_rows, gran, tile_off);
    scan_tile_counts<<<1, 1024, 0, st>>>(tile_off, n_tiles);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

int check_args(const int32_t *rowPtr, int64_t n_rows, int32_t gran, const void *scratch, size_t scratch_bytes)
{
    if (!rowPtr || n_rows < 0 || gran <= 0)
        return PSPMM_E_ARG;
    if (n_rows >= INT32_MAX)
        return PSPMM_E_RANGE;
    const size_t need = ((size_t)((n_rows + TILE - 1) / TILE) + 1) * sizeof(long long);
    if (!scratch || scratch_bytes < need || ((uintptr_t)scratch) % 8 != 0)
        return PSPMM_E_ARG;
    return PSPMM_OK;
}

}  // namespace

extern "C" int pspmm_split_device_scratch_bytes(int64_t n_rows, size_t *bytes)
{
    if (n_rows < 0 || !bytes)
        return PSPMM_E_ARG;
    *bytes = ((size_t)((n_rows + TILE - 1) / TILE) + 1) * sizeof(long long);
    return PSPMM_OK;
}

extern "C" int pspmm_split_count_device(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                        void *scratch, size_t scratch_bytes, int64_t *n_seg, void *stream)
{
    int rc = check_args(rowPtr, n_rows, granularity, scratch, scratch_bytes);
    if (rc)
        return rc;
    if (!n_seg)
        return PSPMM_E_ARG;
    if (n_rows == 0) {
        *n_seg = 0;
        return PSPMM_OK;
    }
    cudaStream_t st = (cudaStream_t)stream;
    long long *tile_off = (long long *)scratch;
    rc = launch_counts(rowPtr, n_rows, granularity, tile_off, st);
    if (rc)
        return rc;
    const int64_t n_tiles = (n_rows + TILE - 1) / TILE;
    long long total = 0;
    PSPMM_CUDA_TRY(cudaMemcpyAsync(&total, tile_off + n_tiles, sizeof(total), cudaMemcpyDeviceToHost, st));
    PSPMM_CUDA_TRY(cudaStreamSynchronize(st));
    *n_seg = (int64_t)total;
    return PSPMM_OK;
}

extern "C" int pspmm_split_csr_device(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                      int32_t *rowPtr_split, int32_t *target_row, int64_t n_seg,
                                      void *scratch, size_t scratch_bytes, void *stream)
{
    int rc = check_args(rowPtr, n_rows, granularity, scratch, scratch_bytes);
    if (rc)
        return rc;
    if (!rowPtr_split || n_seg < 0 || (n_seg > 0 && !target_row))
        return PSPMM_E_ARG;
    if (n_seg >= INT32_MAX)
        return PSPMM_E_RANGE;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_rows == 0) {
        PSPMM_CUDA_TRY(cudaMemsetAsync(rowPtr_split, 0, sizeof(int32_t), st));
        return PSPMM_OK;
    }
    long long *tile_off = (long long *)scratch;
    rc = launch_counts(rowPtr, n_rows, granularity, tile_off, st);
    if (rc)
        return rc;
    const int64_t n_tiles = (n_rows + TILE - 1) / TILE;
    fill_split<<<(unsigned)n_tiles, TILE, 0, st>>>(rowPtr, n_rows, granularity, tile_off, rowPtr_split,
                                                  target_row, n_seg);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}

// ----------------------------------------------------------------------------- no-allocation variant
// Some hosts of this library are not allowed to create device memory at the moment they need a
// partition: a serving process whose device memory was carved up completely at start-up, code
// that runs under another framework's memory pool and must not step outside it, or a plug-in
// called at a point where the embedding application forbids CUDA allocation calls.  Such a
// caller cannot obtain the few kilobytes of tile offsets that pspmm_split_csr_device asks for.
// For them the offsets live in the array below, which is part of the library image: every GPU
// that loads the library holds these bytes until the process exits.
//
// The array bounds the problem: PSPMM_STATIC_SPLIT_MAX_TILES tiles of 1024 rows, i.e. at most
// 16,777,216 rows.  All calls on a device share the one array, so two calls whose kernels may
// overlap on the GPU (different streams, or different host threads) corrupt each other's
// offsets; issue them on one stream or order them yourself.  Nothing in the array has to be
// zero when a call starts: the first kernel of each call overwrites every element the later
// kernels read, so contents left behind by the previous call are harmless.
#define PSPMM_STATIC_SPLIT_MAX_TILES 16384
static __device__ __align__(256) long long g_static_tile_off[PSPMM_STATIC_SPLIT_MAX_TILES + 1];

namespace {
constexpr int MAX_DEVICES = 64;
long long *g_static_ptr[MAX_DEVICES] = {};  // device address of the array, per device ordinal

// The array's name is only a host-side handle; kernels need its address in the current
// device's address space, which the runtime reports per device.
int static_scratch_for_current_device(long long **out)
{
    int dev = -1;
    PSPMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES)
        return PSPMM_E_UNSUPPORTED;
    long long *p = __atomic_load_n(&g_static_ptr[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        void *addr = nullptr;
        PSPMM_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_tile_off));
        p = static_cast<long long *>(addr);
        __atomic_store_n(&g_static_ptr[dev], p, __ATOMIC_RELEASE);  // same value from any thread
    }
    *out = p;
    return PSPMM_OK;
}
}  // namespace

extern "C" int pspmm_split_csr_device_static(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                             int32_t *rowPtr_split, int32_t *target_row, int64_t n_seg,
                                             void *stream)
{
    if (!rowPtr || n_rows < 0 || granularity <= 0)
        return PSPMM_E_ARG;
    if (!rowPtr_split || n_seg < 0 || (n_seg > 0 && !target_row))
        return PSPMM_E_ARG;
    const int64_t n_tiles = (n_rows + TILE - 1) / TILE;
    if (n_tiles > PSPMM_STATIC_SPLIT_MAX_TILES || n_seg >= INT32_MAX)
        return PSPMM_E_RANGE;  // more rows than the built-in scratch covers: use pspmm_split_csr_device
    cudaStream_t st = (cudaStream_t)stream;
    if (n_rows == 0) {
        PSPMM_CUDA_TRY(cudaMemsetAsync(rowPtr_split, 0, sizeof(int32_t), st));
        return PSPMM_OK;
    }
    long long *tile_off = nullptr;
    int rc = static_scratch_for_current_device(&tile_off);
    if (rc)
        return rc;
    rc = launch_counts(rowPtr, n_rows, granularity, tile_off, st);
    if (rc)
        return rc;
    fill_split<<<(unsigned)n_tiles, TILE, 0, st>>>(rowPtr, n_rows, granularity, tile_off, rowPtr_split,
                                                  target_row, n_seg);
    PSPMM_CUDA_TRY(cudaGetLastError());
    return PSPMM_OK;
}
