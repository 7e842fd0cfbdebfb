// Segment SpMM kernel for sm_100a.
//
// Work unit: a "segment" = one CSR row, one PCSR row piece, or the V x 1 block-row forms of
// either.  A group of LPR lanes (LPR = 1..32, a power of two, so 32/LPR segments are in
// flight per warp) owns one segment at a time.  Lane gl of the group covers the dense
// columns [(cf*LPR + gl)*VW, +VW) for cf = 0..CF-1, so one group-wide load instruction
// reads LPR*VW*4 contiguous bytes of a row of B (128-bit loads for VW = 4).
//
// Entries of the segment are fetched CHUNK at a time with one coalesced load per lane
// (column index + V values), then handed round the group with width-LPR shuffles; the
// gathers of B for U consecutive entries are issued before their FMAs so that U*CF
// independent 16-byte loads are in flight per lane.
//
// Output: a segment that is the only piece of its row stores its result (rows without
// entries store zeros, so the output needs no prior memset); a segment that shares its
// row with neighbours adds its partial sum with one vector RED per lane.  Rows that
// receive REDs, and rows that no segment covers, are zeroed beforehand by
// zero_uncovered_rows_kernel (see spmm_api.cu).
#pragma once

#include "pspmm_common.cuh"
#include "vec_ops.cuh"

template <int LPR, int VW, int CF, int V>
__global__ void __launch_bounds__(512) spmm_seg_kernel(const SpmmArgs a)
{
    constexpr int ENT = (LPR >= 16) ? 1 : (16 / LPR);  // entries each lane fetches per chunk
    constexpr int CHUNK = LPR * ENT;                   // 16 or 32 entries per group per chunk
    constexpr int U0 = 8 / (CF * (V > 1 ? 2 : 1));
    constexpr int U = U0 < 1 ? 1 : U0;                 // entries whose gathers are batched

    const int gpc = blockDim.x / LPR;
    const int g = threadIdx.x / LPR;
    const int gl = threadIdx.x % LPR;
    const int vec0 = blockIdx.y * (LPR * CF);

    int voff[CF];
    bool act[CF];
#pragma unroll
    for (int cf = 0; cf < CF; ++cf) {
        int v = vec0 + cf * LPR + gl;
        act[cf] = v < a.nvec;
        voff[cf] = v * VW;
    }

    const int64_t seg0 = (int64_t)blockIdx.x * gpc * a.rows_per_group;
    for (int it = 0; it < a.rows_per_group; ++it) {
        const int64_t seg = seg0 + (int64_t)it * gpc + g;
        const bool live = seg < a.n_seg;
        int lb = 0, hb = 0;
        if (live) {
            lb = __ldg(a.segPtr + seg);
            hb = __ldg(a.segPtr + seg + 1);
        }
        const int len = hb - lb;
        int maxlen = len;
        if constexpr (LPR < 32)
            maxlen = __reduce_max_sync(PSPMM_FULL_MASK, len);

        float acc[V][CF][VW];
#pragma unroll
        for (int w = 0; w < V; ++w)
#pragma unroll
            for (int cf = 0; cf < CF; ++cf)
#pragma unroll
                for (int i = 0; i < VW; ++i)
                    acc[w][cf][i] = 0.f;

        for (int off = 0; off < maxlen; off += CHUNK) {
            int ccol[ENT];
            float cval[ENT][V];
#pragma unroll
            for (int t = 0; t < ENT; ++t) {
                const int k = lb + off + t * LPR + gl;
                const bool ok = k < hb;
                ccol[t] = ok ? __ldg(a.colIdx + k) : 0;
#pragma unroll
                for (int w = 0; w < V; ++w)
                    cval[t][w] = ok ? __ldg(a.val + (int64_t)k * V + w) : 0.f;
            }
            const int cnt = len - off;      // entries this group still owns (may be <= 0)
            const int wcnt = maxlen - off;  // same, maximum over the warp (warp-uniform)
#pragma unroll
            for (int e0 = 0; e0 < CHUNK; e0 += U) {
                if (e0 >= wcnt)
                    break;
                FVec<VW> x[U][CF];
                float v[U][V];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = e0 + u;
                    const int c = __shfl_sync(PSPMM_FULL_MASK, ccol[e / LPR], e % LPR, LPR);
#pragma unroll
                    for (int w = 0; w < V; ++w)
                        v[u][w] = __shfl_sync(PSPMM_FULL_MASK, cval[e / LPR][w], e % LPR, LPR);
                    const float *brow = a.B + (int64_t)c * a.ldB;
                    const bool p = e < cnt;
#pragma unroll
                    for (int cf = 0; cf < CF; ++cf)
                        x[u][cf] = ldg_vec_if<VW>(brow + voff[cf], p && act[cf]);
                }
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int w = 0; w < V; ++w) {
                        // Block layouts carry explicit zeros for absent lanes; they are skipped,
                        // as the reference does, so a non-finite B entry cannot leak through them.
                        if (V > 1 && v[u][w] == 0.f)
                            continue;
#pragma unroll
                        for (int cf = 0; cf < CF; ++cf)
#pragma unroll
                            for (int i = 0; i < VW; ++i)
                                acc[w][cf][i] = fmaf(v[u][w], x[u][cf].v[i], acc[w][cf][i]);
                    }
            }
        }

        if (live) {
            int64_t orow = seg;
            bool shared = false;
            if (a.target_row) {
                const int me = __ldg(a.target_row + seg);
                orow = me;
                const int prev = seg > 0 ? __ldg(a.target_row + seg - 1) : -1;
                const int next = seg + 1 < a.n_seg ? __ldg(a.target_row + seg + 1) : -1;
                shared = (prev == me) || (next == me);
            }
#pragma unroll
            for (int w = 0; w < V; ++w) {
                float *crow = a.C + (orow * V + w) * a.ldC;
#pragma unroll
                for (int cf = 0; cf < CF; ++cf) {
                    if (!act[cf])
                        continue;
                    if (shared)
                        red_add_vec<VW>(crow + voff[cf], acc[w][cf]);
                    else
                        st_stream_vec<VW>(crow + voff[cf], acc[w][cf]);
                }
            }
        }
    }
}

template <int LPR, int VW, int CF, int V>
static inline void spmm_launch_one(const SpmmArgs &a, dim3 grid, int threads, cudaStream_t st)
{
    spmm_seg_kernel<LPR, VW, CF, V><<<grid, threads, 0, st>>>(a);
}

// Expands to the dispatch over the instantiated (LPR, CF) pairs of one (VW, V).
#define PSPMM_SPMM_CASE(LPR_, CF_, VW_, V_)                              \
    if (s.lpr == LPR_ && s.cf == CF_) {                                  \
        spmm_launch_one<LPR_, VW_, CF_, V_>(a, grid, s.threads, st);     \
        return true;                                                     \
    }
