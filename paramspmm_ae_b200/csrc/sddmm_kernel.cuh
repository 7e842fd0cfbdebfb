// Segment SDDMM kernel for sm_100a: out[k] = <A[row(k)], B[colIdx[k]]> on a sparsity pattern.
//
// Same work decomposition as the SpMM kernel: a group of LPR lanes owns one segment (CSR
// row, PCSR row piece, or a V x 1 block-row form), lane gl holds the slice
// [(cf*LPR + gl)*VW, +VW), cf < CF, of the segment's A row(s) in registers and multiplies it
// with the same slice of every gathered B row (128-bit loads for VW = 4).
//
// The per-entry lane partials are not reduced one entry at a time.  LPR entries are
// processed together and reduced with a recursive-halving exchange: at stride s each lane
// keeps the half of the entries selected by its own lane bit and ships the other half to
// lane ^ s.  After log2(LPR) rounds lane gl owns the complete dot product of entry gl of
// the batch, at a cost of LPR-1 shuffles per LPR entries (about one per entry instead of
// log2(LPR)), and the results leave as one coalesced store per group.
#pragma once

#include "pspmm_common.cuh"
#include "vec_ops.cuh"

// p[0..N) per lane -> returns, on lane gl of each LPR-wide group, the sum over the group of p[gl].
template <int N>
__device__ __forceinline__ float transpose_reduce(float (&p)[N], int gl)
{
    if constexpr (N == 1) {
        return p[0];
    } else {
        constexpr int H = N / 2;
        float q[H];
        const bool upper = (gl & H) != 0;
#pragma unroll
        for (int i = 0; i < H; ++i) {
            const float keep = upper ? p[i + H] : p[i];
            const float send = upper ? p[i] : p[i + H];
            q[i] = keep + __shfl_xor_sync(PSPMM_FULL_MASK, send, H);
        }
        return transpose_reduce<H>(q, gl);
    }
}

template <int LPR, int VW, int CF, int V>
__global__ void __launch_bounds__(512) sddmm_seg_kernel(const SddmmArgs a)
{
    constexpr int ENT = (LPR >= 16) ? 1 : (16 / LPR);
    constexpr int CHUNK = LPR * ENT;
    constexpr int U0 = 8 / CF;
    constexpr int U1 = U0 < 1 ? 1 : U0;
    constexpr int U = U1 > LPR ? LPR : U1;  // entries whose gathers are batched (divides LPR)

    const int gpc = blockDim.x / LPR;
    const int g = threadIdx.x / LPR;
    const int gl = threadIdx.x % LPR;
    const int tiles = (a.nvec + LPR * CF - 1) / (LPR * CF);

    const int64_t seg0 = (int64_t)blockIdx.x * gpc * a.rows_per_group;
    for (int it = 0; it < a.rows_per_group; ++it) {
        const int64_t seg = seg0 + (int64_t)it * gpc + g;
        const bool live = seg < a.n_seg;
        int lb = 0, hb = 0;
        int64_t arow = 0;
        if (live) {
            lb = __ldg(a.segPtr + seg);
            hb = __ldg(a.segPtr + seg + 1);
            arow = a.target_row ? (int64_t)__ldg(a.target_row + seg) : seg;
        }
        const int len = hb - lb;
        int maxlen = len;
        if constexpr (LPR < 32)
            maxlen = __reduce_max_sync(PSPMM_FULL_MASK, len);

        for (int off = 0; off < maxlen; off += CHUNK) {
            int ccol[ENT];
            float cval[ENT][V];
            float res[ENT][V];
#pragma unroll
            for (int t = 0; t < ENT; ++t) {
                const int k = lb + off + t * LPR + gl;
                const bool ok = k < hb;
                ccol[t] = ok ? __ldg(a.colIdx + k) : 0;
#pragma unroll
                for (int w = 0; w < V; ++w) {
                    cval[t][w] = (V > 1 && ok) ? __ldg(a.val + (int64_t)k * V + w) : 1.f;
                    res[t][w] = 0.f;
                }
            }
            const int cnt = len - off;
            const int wcnt = maxlen - off;

            for (int tile = 0; tile < tiles; ++tile) {
                // Slice of the A row(s) this lane is responsible for in this tile.
                FVec<VW> av[V][CF];
                int voff[CF];
                bool act[CF];
#pragma unroll
                for (int cf = 0; cf < CF; ++cf) {
                    const int vi = (tile * CF + cf) * LPR + gl;
                    act[cf] = vi < a.nvec;
                    voff[cf] = vi * VW;
#pragma unroll
                    for (int w = 0; w < V; ++w)
                        // (the last block-row of an odd row count has lanes without a row of A)
                        av[w][cf] = (live && act[cf] && arow * V + w < a.n_rows_A)
                                        ? ldg_vec<VW>(a.A + (arow * V + w) * a.ldA + voff[cf])
                                        : zero_vec<VW>();
                }
#pragma unroll
                for (int t = 0; t < ENT; ++t) {
                    if (t * LPR >= wcnt)
                        break;
                    float part[V][LPR];
#pragma unroll
                    for (int j0 = 0; j0 < LPR; j0 += U) {
                        FVec<VW> x[U][CF];
                        const bool batch_on = (t * LPR + j0) < wcnt;  // warp-uniform
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const int e = t * LPR + j0 + u;
                            const int c = __shfl_sync(PSPMM_FULL_MASK, ccol[t], j0 + u, LPR);
                            const float *brow = a.B + (int64_t)c * a.ldB;
                            const bool p = batch_on && (e < cnt);
#pragma unroll
                            for (int cf = 0; cf < CF; ++cf)
                                x[u][cf] = ldg_vec_if<VW>(brow + voff[cf], p && act[cf]);
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u)
#pragma unroll
                            for (int w = 0; w < V; ++w) {
                                float s = 0.f;
#pragma unroll
                                for (int cf = 0; cf < CF; ++cf)
#pragma unroll
                                    for (int i = 0; i < VW; ++i)
                                        s = fmaf(av[w][cf].v[i], x[u][cf].v[i], s);
                                part[w][j0 + u] = s;
                            }
                    }
#pragma unroll
                    for (int w = 0; w < V; ++w)
                        res[t][w] += transpose_reduce<LPR>(part[w], gl);
                }
            }
#pragma unroll
            for (int t = 0; t < ENT; ++t) {
                const int k = lb + off + t * LPR + gl;
                if (k < hb) {
#pragma unroll
                    for (int w = 0; w < V; ++w) {
                        // Block layouts: positions whose stored value is zero are not part of
                        // the pattern and receive zero.
                        const float r = (V > 1 && cval[t][w] == 0.f) ? 0.f : res[t][w];
                        __stcs(a.out + (int64_t)k * V + w, r);
                    }
                }
            }
        }
    }
}

template <int LPR, int VW, int CF, int V>
static inline void sddmm_launch_one(const SddmmArgs &a, dim3 grid, int threads, cudaStream_t st)
{
    sddmm_seg_kernel<LPR, VW, CF, V><<<grid, threads, 0, st>>>(a);
}

#define PSPMM_SDDMM_CASE(LPR_, CF_, VW_, V_)                             \
    if (s.lpr == LPR_ && s.cf == CF_) {                                  \
        sddmm_launch_one<LPR_, VW_, CF_, V_>(a, grid, s.threads, st);    \
        return true;                                                     \
    }
