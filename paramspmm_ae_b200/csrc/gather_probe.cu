// Stand-alone microbenchmark (not part of libpspmm): gather throughput of 256-byte rows by three
// mechanisms on sm_100a.  It answers which data path the SpMM / SDDMM kernels should gather with.
// Build and run:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -lineinfo \
//          paramspmm_ae_b200/csrc/gather_probe.cu -o gather_probe && ./gather_probe
// Every wait on an mbarrier is bounded; a wait that runs out sets the error flag that is printed.
//   ldg   : group of 16 lanes, LDG.128 per lane, U rows in flight per group (registers)
//   cpa   : group of 16 lanes, cp.async 16 B per lane into a shared-memory ring, NST stages of EPS rows
//   bulk  : each lane issues one cp.async.bulk of 256 B (row) into a shared-memory ring + mbarrier
// Rows are picked from an index stream; the sum of everything read is written out so nothing is elided.
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <cuda_runtime.h>

#define ROWB 256
#define CHECK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1); } } while (0)

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

template <int U>
__global__ void __launch_bounds__(256) k_ldg(const float *B, const int *idx, long n_idx, float *out)
{
    const int gl = threadIdx.x & 15;
    const long g = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const long ng = ((long)gridDim.x * blockDim.x) >> 4;
    const long per = n_idx / ng;
    const int *my = idx + g * per;
    float4 acc = make_float4(0, 0, 0, 0);
    for (long e = 0; e + U <= per; e += U) {
        int c[U];
        float4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) c[u] = __ldg(my + e + u);
#pragma unroll
        for (int u = 0; u < U; ++u) x[u] = __ldg(reinterpret_cast<const float4 *>(B + (size_t)c[u] * (ROWB / 4)) + gl);
#pragma unroll
        for (int u = 0; u < U; ++u) { acc.x += x[u].x; acc.y += x[u].y; acc.z += x[u].z; acc.w += x[u].w; }
    }
    if (acc.x + acc.y + acc.z + acc.w == 123.456f) out[0] = acc.x;
}

// cp.async ring: each lane copies and later reads back its own 16 bytes of every row.
template <int EPS, int NST>
__global__ void __launch_bounds__(256) k_cpa(const float *B, const int *idx, long n_idx, float *out)
{
    extern __shared__ __align__(16) char smem[];
    const int gl = threadIdx.x & 15;
    const int gin = threadIdx.x >> 4;
    const long g = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const long ng = ((long)gridDim.x * blockDim.x) >> 4;
    const long per = n_idx / ng;
    const int *my = idx + g * per;
    char *ring = smem + (size_t)gin * NST * EPS * ROWB;
    const long nst = per / EPS;
    float4 acc = make_float4(0, 0, 0, 0);
    auto issue = [&](long t) {
        char *dst = ring + (t % NST) * EPS * ROWB + gl * 16;
#pragma unroll
        for (int u = 0; u < EPS; ++u) {
            const int c = __ldg(my + t * EPS + u);
            const char *src = reinterpret_cast<const char *>(B) + (size_t)c * ROWB + gl * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + u * ROWB)), "l"(src));
        }
        asm volatile("cp.async.commit_group;");
    };
    for (int s = 0; s < NST - 1; ++s) {
        if (s < nst) issue(s); else asm volatile("cp.async.commit_group;");
    }
    for (long t = 0; t < nst; ++t) {
        if (t + NST - 1 < nst) issue(t + NST - 1); else asm volatile("cp.async.commit_group;");
        asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1));
        const char *srcs = ring + (t % NST) * EPS * ROWB + gl * 16;
#pragma unroll
        for (int u = 0; u < EPS; ++u) {
            const float4 x = *reinterpret_cast<const float4 *>(srcs + u * ROWB);
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
    }
    if (acc.x + acc.y + acc.z + acc.w == 123.456f) out[0] = acc.x;
}

// bulk ring: lane u of a 16-lane group issues the 256-byte copy of row u of the stage.
template <int NST>
__global__ void __launch_bounds__(256) k_bulk(const float *B, const int *idx, long n_idx, float *out, int *err)
{
    constexpr int EPS = 16;
    extern __shared__ __align__(16) char smem[];
    const int gl = threadIdx.x & 15;
    const int gin = threadIdx.x >> 4;
    const int ngrp = blockDim.x >> 4;
    const unsigned gmask = 0xffffu << ((threadIdx.x & 16));
    const long g = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const long ng = ((long)gridDim.x * blockDim.x) >> 4;
    const long per = n_idx / ng;
    const int *my = idx + g * per;
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(smem) + gin * NST;
    char *ring = smem + ((ngrp * NST * 8 + 127) / 128 * 128) + (size_t)gin * NST * EPS * ROWB;
    if (gl == 0) {
        for (int s = 0; s < NST; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bars + s)));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    const long nst = per / EPS;
    float4 acc = make_float4(0, 0, 0, 0);
    auto issue = [&](long t) {
        const int s = (int)(t % NST);
        const int c = __ldg(my + t * EPS + gl);
        if (gl == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bars + s)), "r"(EPS * ROWB) : "memory");
        __syncwarp(gmask);
        const char *src = reinterpret_cast<const char *>(B) + (size_t)c * ROWB;
        asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(ring + (s * EPS + gl) * ROWB)), "l"(src), "r"(ROWB), "r"(smem_u32(bars + s)) : "memory");
    };
    for (int s = 0; s < NST; ++s)
        if (s < nst) issue(s);
    bool dead = false;
    for (long t = 0; t < nst && !dead; ++t) {
        const int s = (int)(t % NST);
        const unsigned parity = (unsigned)((t / NST) & 1);
        unsigned done = 0;
        for (int spin = 0; spin < (1 << 20); ++spin) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(smem_u32(bars + s)), "r"(parity) : "memory");
            if (done) break;
        }
        if (!done) { *err = 1; dead = true; break; }
        const char *srcs = ring + (s * EPS) * ROWB + gl * 16;
#pragma unroll
        for (int u = 0; u < EPS; ++u) {
            const float4 x = *reinterpret_cast<const float4 *>(srcs + u * ROWB);
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        __syncwarp(gmask);
        if (t + NST < nst) issue(t + NST);
    }
    if (acc.x + acc.y + acc.z + acc.w == 123.456f) out[0] = acc.x;
}

template <class F> float time_ms(F f, int iters) {
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    f(); CHECK(cudaDeviceSynchronize());
    cudaEventRecord(a); for (int i = 0; i < iters; ++i) f(); cudaEventRecord(b);
    CHECK(cudaEventSynchronize(b)); float ms; cudaEventElapsedTime(&ms, a, b); return ms / iters;
}

int main() {
    const long n_idx = 16L << 20;  // 16 Mi gathers = 4 GiB of rows
    int *d_idx; float *d_B, *d_out; int *d_err;
    CHECK(cudaMalloc(&d_idx, n_idx * 4)); CHECK(cudaMalloc(&d_out, 64)); CHECK(cudaMalloc(&d_err, 4)); CHECK(cudaMemset(d_err, 0, 4));
    for (long rows : {65536L, 1L << 20}) {
        CHECK(cudaMalloc(&d_B, rows * ROWB)); CHECK(cudaMemset(d_B, 0, rows * ROWB));
        std::vector<int> h(n_idx); unsigned long long s = 88172645463325252ull;
        for (long i = 0; i < n_idx; ++i) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; h[i] = (int)(s % (unsigned long long)rows); }
        CHECK(cudaMemcpy(d_idx, h.data(), n_idx * 4, cudaMemcpyHostToDevice));
        const double gb = (double)n_idx * ROWB / 1e9;
        printf("rows %ld (B = %.0f MB)\n", rows, rows * ROWB / 1e6);
        for (int ctas : {148 * 2, 148 * 3, 148 * 5, 148 * 8}) {
            float ms;
            ms = time_ms([&] { k_ldg<4><<<ctas, 256>>>(d_B, d_idx, n_idx, d_out); }, 5); printf("  ldg U=4  ctas %4d: %.3f ms %.0f GB/s\n", ctas, ms, gb / ms * 1e3);
            ms = time_ms([&] { k_ldg<8><<<ctas, 256>>>(d_B, d_idx, n_idx, d_out); }, 5); printf("  ldg U=8  ctas %4d: %.3f ms %.0f GB/s\n", ctas, ms, gb / ms * 1e3);
        }
        {
            auto run_cpa = [&](auto kern, int eps, int nst, const char *name) {
                const int smem = 16 * nst * eps * ROWB;
                CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                const int per_sm = (220 * 1024) / smem;
                float ms = time_ms([&] { kern<<<148 * per_sm, 256, smem>>>(d_B, d_idx, n_idx, d_out); }, 5);
                printf("  %s smem %d KB x %d CTA/SM: %.3f ms %.0f GB/s\n", name, smem / 1024, per_sm, ms, gb / ms * 1e3);
            };
            run_cpa(k_cpa<4, 2>, 4, 2, "cpa EPS4 NST2");
            run_cpa(k_cpa<4, 3>, 4, 3, "cpa EPS4 NST3");
            run_cpa(k_cpa<8, 2>, 8, 2, "cpa EPS8 NST2");
            run_cpa(k_cpa<8, 3>, 8, 3, "cpa EPS8 NST3");
            run_cpa(k_cpa<16, 3>, 16, 3, "cpa EPS16 NST3");
        }
        {
            auto run_bulk = [&](auto kern, int nst, const char *name) {
                const int smem = 1024 + 16 * nst * 16 * ROWB;
                CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                const int per_sm = (224 * 1024) / smem;
                float ms = time_ms([&] { kern<<<148 * per_sm, 256, smem>>>(d_B, d_idx, n_idx, d_out, d_err); }, 5);
                int herr = 0; cudaMemcpy(&herr, d_err, 4, cudaMemcpyDeviceToHost);
                printf("  %s smem %d KB x %d CTA/SM: %.3f ms %.0f GB/s err %d\n", name, smem / 1024, per_sm, ms, gb / ms * 1e3, herr);
            };
            run_bulk(k_bulk<1>, 1, "bulk NST1");
            run_bulk(k_bulk<2>, 2, "bulk NST2");
            run_bulk(k_bulk<3>, 3, "bulk NST3");
        }
        CHECK(cudaFree(d_B));
    }
    return 0;
}
