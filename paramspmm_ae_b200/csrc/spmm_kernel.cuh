// Segment SpMM kernel for sm_100a.
//
// Work unit: a "segment" = one CSR row, one PCSR row piece, or the V x 1 block-row forms of
// either.  A group of LPR lanes (LPR = 2..32, a power of two, so 32/LPR groups share a warp)
// owns `rows_per_group` CONSECUTIVE segments, whose entries are therefore one contiguous
// range of colIdx / val.  Lane gl of the group covers the dense columns
// [(cf*LPR + gl)*VW, +VW) for cf = 0..CF-1, so one group-wide load reads LPR*VW*4 contiguous
// bytes of a row of B (128-bit loads for VW = 4).
//
// Staging: the group first copies its segment pointers (and, for split layouts, the target
// rows of its segments and of the two neighbouring ones) into shared memory, then streams its
// entry range through a small shared-memory window (CAP entries, column index and value
// interleaved).  All lanes of a group need the same (column, value) pair for an entry; they
// get it with one broadcast LDS.64 instead of two register shuffles, which halves the
// load/store-unit wavefronts spent on distributing A, and the pointer -> entries -> gather
// dependency is paid once per group of rows instead of once per row.  Groups synchronise only
// among their own lanes, so groups of one warp walk rows of different lengths independently.
//
// Inner loop per entry and lane: LDS.64, one IMAD.WIDE, CF x LDG.128, 4*CF FFMA.  The gathers
// of U consecutive entries are issued before their FMAs (U*CF independent 16-byte loads in
// flight per lane); row tails fall through batches of U/2, U/4, ... 1 entries.  Lanes beyond
// the last dense column (dim not a multiple of LPR*VW) read column 0 of the same row instead
// of being predicated, and simply do not store.
//
// Output: consecutive segments of one group that target the same row are summed in
// registers.  A row whose segments all lie inside one group is stored with streaming stores
// (rows without entries store zeros, so the output needs no prior memset).  A row that
// straddles groups receives one vector RED per lane from each of them; such rows are zeroed
// beforehand by zero_shared_rows_kernel (pspmm_api.cu).  In a split layout rows that no
// segment covers lie between the target rows of consecutive segments: every group zeroes the
// short gap that follows each of its rows (up to PSPMM_GAP_MAX rows); longer gaps are left to
// the pre-pass.
#pragma once

#include "pspmm_common.cuh"
#include "vec_ops.cuh"

template <int LPR, int V>
struct SpmmTile {
    static constexpr int CAP = (LPR * 4 < 16) ? 16 : ((LPR * 4 > 64) ? 64 : LPR * 4);
    // Per-group shared memory: pointers [RPG_MAX+1], target rows [RPG_MAX+2] (padded to a
    // multiple of 8 bytes), then CAP entries of (1 + V) words.
    static constexpr int HEAD_WORDS = ((PSPMM_RPG_MAX + 1) + (PSPMM_RPG_MAX + 2) + 1) / 2 * 2;
    static constexpr int GROUP_WORDS = HEAD_WORDS + CAP * (1 + V);
};

// One batch of UU entries starting at shared-memory index e: gathers first, FMAs after.
template <int UU, int LPR, int VW, int CF, int V>
__device__ __forceinline__ void spmm_batch(const int *ent, int e, const char *const (&bcol)[CF],
                                           unsigned ldB_bytes, unsigned long long keep,
                                           float (&acc)[V][CF][VW])
{
    int c[UU];
    float v[UU][V];
#pragma unroll
    for (int u = 0; u < UU; ++u) {
        if constexpr (V == 1) {
            const int2 cv = *reinterpret_cast<const int2 *>(ent + 2 * (e + u));
            c[u] = cv.x;
            v[u][0] = __int_as_float(cv.y);
        } else {
            c[u] = ent[(1 + V) * (e + u)];
#pragma unroll
            for (int w = 0; w < V; ++w)
                v[u][w] = __int_as_float(ent[(1 + V) * (e + u) + 1 + w]);
        }
    }
    FVec<VW> x[UU][CF];
#pragma unroll
    for (int u = 0; u < UU; ++u)
#pragma unroll
        for (int cf = 0; cf < CF; ++cf)
            x[u][cf] = ldg_vec_hint<VW>(row_slice(bcol[cf], c[u], ldB_bytes), keep);
#pragma unroll
    for (int u = 0; u < UU; ++u)
#pragma unroll
        for (int w = 0; w < V; ++w) {
            // Block layouts carry explicit zeros for absent lanes; they are skipped, as the
            // reference does, so a non-finite B entry cannot leak through them.
            if (V > 1 && v[u][w] == 0.f)
                continue;
#pragma unroll
            for (int cf = 0; cf < CF; ++cf)
#pragma unroll
                for (int i = 0; i < VW; ++i)
                    acc[w][cf][i] = fmaf(v[u][w], x[u][cf].v[i], acc[w][cf][i]);
        }
}

// MLP = 16-byte gathers a lane keeps in flight per batch (2, 4, 8 or 16).  It trades registers
// (and so resident warps per SM) against memory-level parallelism inside one warp; the
// launch bound asks for the matching number of resident 256-thread CTAs.
template <int MLP>
struct SpmmOcc {
    static constexpr int MIN_CTAS = MLP >= 16 ? 2 : (MLP >= 8 ? 3 : (MLP >= 4 ? 5 : 8));
};

// ACC = true adds the product to C instead of overwriting it: every contribution is a RED, rows
// without entries add nothing, and nothing is zeroed (no pre-pass either).
template <int LPR, int VW, int CF, int V, int MLP, bool ACC = false>
__global__ void __launch_bounds__(256, SpmmOcc<MLP>::MIN_CTAS) spmm_seg_kernel(const SpmmArgs a)
{
    using Tile = SpmmTile<LPR, V>;
    constexpr int CAP = Tile::CAP;
    constexpr int U0 = MLP / (CF * (V > 1 ? 2 : 1));
    // entries per full gather batch: a power of two (the row tail falls through U/2, U/4, ...)
    constexpr int U = U0 >= 16 ? 16 : (U0 >= 8 ? 8 : (U0 >= 4 ? 4 : (U0 >= 2 ? 2 : 1)));

    extern __shared__ __align__(16) int smem_words[];
    const int gpc = blockDim.x / LPR;
    const int g = threadIdx.x / LPR;
    const int gl = threadIdx.x % LPR;
    const unsigned gmask =
        (LPR == 32) ? PSPMM_FULL_MASK : (((1u << LPR) - 1u) << (((threadIdx.x & 31) / LPR) * LPR));
    int *sp = smem_words + g * Tile::GROUP_WORDS;            // segment pointers
    int *st = sp + (PSPMM_RPG_MAX + 1);                     // target rows: [0] previous, [1..] own, then next
    int *ent = sp + Tile::HEAD_WORDS;                       // staged entries

    const int rpg = a.rows_per_group;
    const int64_t first = ((int64_t)blockIdx.x * gpc + g) * rpg;
    if (first >= a.n_seg)
        return;  // the whole group leaves; groups only ever synchronise among themselves
    const int nrow = (a.n_seg - first < rpg) ? (int)(a.n_seg - first) : rpg;
    const bool split = a.target_row != nullptr;

    for (int i = gl; i <= nrow; i += LPR)
        sp[i] = __ldg(a.segPtr + first + i);
    if (split) {
        for (int i = gl; i < nrow + 2; i += LPR) {
            const int64_t s = first - 1 + i;
            st[i] = (s < 0) ? -1 : (s >= a.n_seg ? (int)a.n_out : __ldg(a.target_row + s));
        }
    }

    // Per-lane column slices; lanes past the last column read slice 0 and never store.
    const int vec0 = blockIdx.y * (LPR * CF);
    bool act[CF];
    int voff[CF];
    const char *bcol[CF];
#pragma unroll
    for (int cf = 0; cf < CF; ++cf) {
        const int v = vec0 + cf * LPR + gl;
        act[cf] = v < a.nvec;
        voff[cf] = act[cf] ? v * VW : 0;
        bcol[cf] = reinterpret_cast<const char *>(a.B + voff[cf]);
    }
    const unsigned ldB_bytes = (unsigned)(a.ldB * 4);
    // B is gathered many times: keep a stable fraction of it in L2.  A is read once and C is
    // written once: both are marked evict-first so they do not push B out.
    const unsigned long long keep = l2_policy_keep(a.keep_fraction);
    const unsigned long long stream = l2_policy_stream();

    float acc[V][CF][VW];
#pragma unroll
    for (int w = 0; w < V; ++w)
#pragma unroll
        for (int cf = 0; cf < CF; ++cf)
#pragma unroll
            for (int i = 0; i < VW; ++i)
                acc[w][cf][i] = 0.f;

    __syncwarp(gmask);
    int cur = sp[0];
    const int end = sp[nrow];
    int row = 0;
    int run_start = 0;  // first of the group's segments accumulated into the current row
    bool head_pending = (first == 0);  // the rows ahead of the very first segment are still to be zeroed
    while (true) {
        const int fill = (end - cur < CAP) ? (end - cur) : CAP;
        for (int i = gl; i < fill; i += LPR) {
            const int k = cur + i;
            if constexpr (V == 1) {
                // (no value array: the pattern itself, every stored entry counts as 1)
                *reinterpret_cast<int2 *>(ent + 2 * i) =
                    make_int2(ldg_stream_b32(a.colIdx + k, stream),
                              a.val ? ldg_stream_b32(a.val + k, stream) : __float_as_int(1.f));
            } else {
                ent[(1 + V) * i] = ldg_stream_b32(a.colIdx + k, stream);
#pragma unroll
                for (int w = 0; w < V; ++w)
                    ent[(1 + V) * i + 1 + w] = ldg_stream_b32(a.val + (int64_t)k * V + w, stream);
            }
        }
        __syncwarp(gmask);
        const int lim = cur + fill;
        while (row < nrow) {
            const int rb = sp[row], re = sp[row + 1];
            int e = (rb > cur ? rb : cur) - cur;
            const int eh = (re < lim ? re : lim) - cur;
            for (; e + U <= eh; e += U)
                spmm_batch<U, LPR, VW, CF, V>(ent, e, bcol, ldB_bytes, keep, acc);
            if constexpr (U >= 16) {
                if (e + 8 <= eh) {
                    spmm_batch<8, LPR, VW, CF, V>(ent, e, bcol, ldB_bytes, keep, acc);
                    e += 8;
                }
            }
            if constexpr (U >= 8) {
                if (e + 4 <= eh) {
                    spmm_batch<4, LPR, VW, CF, V>(ent, e, bcol, ldB_bytes, keep, acc);
                    e += 4;
                }
            }
            if constexpr (U >= 4) {
                if (e + 2 <= eh) {
                    spmm_batch<2, LPR, VW, CF, V>(ent, e, bcol, ldB_bytes, keep, acc);
                    e += 2;
                }
            }
            if constexpr (U >= 2) {
                if (e < eh)
                    spmm_batch<1, LPR, VW, CF, V>(ent, e, bcol, ldB_bytes, keep, acc);
            }
            if (re > lim)
                break;  // the row continues in the next window

            // ---- the segment is complete
            int64_t orow = first + row;
            bool shared = false;
            int next = 0;
            if (split && a.bucketed) {
                // Length-bucketed plan: segments in any order, flags in the high bits of the target.
                const unsigned me = (unsigned)st[row + 1];
                const unsigned nx = (unsigned)st[row + 2];
                if (row + 1 < nrow && ((nx ^ me) & PSPMM_SEG_ROW_MASK) == 0) {
                    ++row;  // the group's next segment is another piece of the same row
                    continue;
                }
                orow = me & PSPMM_SEG_ROW_MASK;
                shared = (me & PSPMM_SEG_MULTI) != 0;
            } else if (split) {
                const int me = st[row + 1];
                next = st[row + 2];
                if (next == me && row + 1 < nrow) {
                    ++row;  // the group's next segment continues the same row: keep accumulating
                    continue;
                }
                orow = me;
                // Pieces of this row held by other groups add into it as well.
                shared = (run_start == 0 && st[0] == me) || (next == me);
                run_start = row + 1;
            }
            // (pieces of a split layout are never empty)
            const bool emit = !ACC || split || re > rb;
#pragma unroll
            for (int w = 0; w < V; ++w) {
                float *crow = a.C + (orow * V + w) * a.ldC;
#pragma unroll
                for (int cf = 0; cf < CF; ++cf) {
                    if (act[cf] && emit) {
                        if (ACC || shared)
                            red_add_vec<VW>(crow + voff[cf], acc[w][cf]);
                        else
                            st_vec_hint<VW>(crow + voff[cf], acc[w][cf], stream);
                    }
#pragma unroll
                    for (int i = 0; i < VW; ++i)
                        acc[w][cf][i] = 0.f;
                }
            }
            if (!ACC && split && !a.bucketed) {
                // Rows strictly between this segment's row and the next segment's row (and, for
                // the very first segment, the rows before it) have no entries: zero short runs
                // here; runs longer than PSPMM_GAP_MAX are left to the pre-pass.
                const float zero[VW] = {};
                auto zero_rows = [&](int64_t r0, int64_t r1) {
                    for (int64_t r = r0 * V; r < r1 * V; ++r) {
                        float *crow = a.C + r * a.ldC;
#pragma unroll
                        for (int cf = 0; cf < CF; ++cf)
                            if (act[cf])
                                st_vec_hint<VW>(crow + voff[cf], zero, stream);
                    }
                };
                const int64_t after = (int64_t)next - orow - 1;
                if (after > 0 && after <= PSPMM_GAP_MAX)
                    zero_rows(orow + 1, next);
                if (head_pending && orow > 0 && orow <= PSPMM_GAP_MAX)
                    zero_rows(0, orow);
                head_pending = false;
            }
            ++row;
        }
        if (row >= nrow)
            break;
        cur = lim;
        __syncwarp(gmask);  // everyone is done reading the window before it is refilled
    }
}

template <int LPR, int VW, int CF, int V, int MLP, bool ACC = false>
static inline void spmm_launch_one(const SpmmArgs &a, dim3 grid, int threads, cudaStream_t st)
{
    const int smem = (threads / LPR) * SpmmTile<LPR, V>::GROUP_WORDS * 4;
    auto kern = spmm_seg_kernel<LPR, VW, CF, V, MLP, ACC>;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    kern<<<grid, threads, smem, st>>>(a);
}

// Expands to the dispatch over the instantiated (LPR, CF) pairs of one (VW, V).
#define PSPMM_SPMM_CASE(LPR_, CF_, VW_, V_)                                  \
    if (s.lpr == LPR_ && s.cf == CF_) {                                      \
        spmm_launch_one<LPR_, VW_, CF_, V_, 8>(a, grid, s.threads, st);      \
        return true;                                                         \
    }
// Same, with every gather-batch depth instantiated (used for the 128-bit CSR family).
#define PSPMM_SPMM_CASE_MLP(LPR_, CF_, VW_, V_)                              \
    if (s.lpr == LPR_ && s.cf == CF_) {                                      \
        if (s.mlp == 2)                                                      \
            spmm_launch_one<LPR_, VW_, CF_, V_, 2>(a, grid, s.threads, st);  \
        else if (s.mlp == 4)                                                 \
            spmm_launch_one<LPR_, VW_, CF_, V_, 4>(a, grid, s.threads, st);  \
        else if (s.mlp == 16)                                                \
            spmm_launch_one<LPR_, VW_, CF_, V_, 16>(a, grid, s.threads, st); \
        else                                                                 \
            spmm_launch_one<LPR_, VW_, CF_, V_, 8>(a, grid, s.threads, st);  \
        return true;                                                         \
    }
// The accumulating form is built for the 128-bit CSR family at one gather-batch depth.
#define PSPMM_SPMM_CASE_ACC(LPR_, CF_)                                       \
    if (s.lpr == LPR_ && s.cf == CF_) {                                      \
        spmm_launch_one<LPR_, 4, CF_, 1, 8, true>(a, grid, s.threads, st);   \
        return true;                                                         \
    }
