// Fused attention aggregation over a sparsity pattern (sm_100a):
//
//     s_ij  = beta * <A_i, B_j>                 for every stored (i, j)          (the SDDMM)
//     a_ij  = softmax_j(s_ij)  or  s_ij                                           (edge softmax, optional)
//     out_i = sum_j a_ij * V_j        (V = B in the forward pass)                 (the SpMM)
//
// in ONE pass over the pattern: every gathered row B_j is used for its score and for the
// aggregation while it sits in registers, the per-edge values never reach memory, and the
// softmax is the running-maximum ("online") form, so a row needs no second sweep.  This is the
// AGNN propagation (A = B = the projected node features) without the two edge-array round trips
// and with half the gathers of SDDMM followed by SpMM.  With a separate aggregation operand V
// (template flag SEP: a second gather per entry) the same pass gives the layer's backward products
// from recomputed scores: sum_j a_ij G_j for an upstream gradient G, again without an edge array.
//
// Work unit = segment (CSR row or PCSR row piece); a group of LPR lanes owns one segment, lane gl
// holds the slice [(cf*LPR + gl)*4, +4) of A_i and of the accumulator.  Entries are taken BS at a
// time: BS gathers (128-bit loads), BS lane-partial dot products, a recursive-halving exchange
// after which lane e holds the complete score of entry e (about one shuffle per entry), one
// max / exp / sum step for the batch, then BS broadcasts of the weights and the FMAs.
//
// A row that is a single segment is normalised and stored directly.  Pieces of a split row leave
// (running max, running sum, unnormalised accumulator) in caller-provided scratch and are merged
// by agnn_combine_kernel.  Rows that no segment covers are zeroed by a memset of the output
// (split layouts only; in plain CSR every row is a segment and stores its own zeros).
#include <math_constants.h>

#include "pspmm_common.cuh"
#include "vec_ops.cuh"

namespace {

struct AgnnArgs {
    const int32_t *segPtr;
    const int32_t *target_row;  // nullptr: row == segment
    const int32_t *colIdx;
    const float *A;
    const float *B;
    const float *Vm;  // aggregated rows (SEP kernels); row stride ldV, 0 = one row shared by all columns
    float *out;
    float *scratch;  // [n_seg][4 + dim_pad] partials of split rows: max, sum, 2 unused, accumulator
    int64_t n_seg;
    int64_t ldA, ldB, ldV, ldOut;
    int32_t dim, dim_pad;
    float beta;
    int32_t softmax;
};

// Sum over the LPR lanes of a group of p[e], delivered to lane (gl % BS) == e.
template <int LPR, int BS>
__device__ __forceinline__ float group_transpose_reduce(float (&p)[BS], int gl)
{
    // fold the lane bits above BS first (plain butterflies on all BS values) ...
#pragma unroll
    for (int d = LPR / 2; d >= BS; d >>= 1)
#pragma unroll
        for (int e = 0; e < BS; ++e)
            p[e] += __shfl_xor_sync(PSPMM_FULL_MASK, p[e], d);
    // ... then halve the value set at every remaining step
    float q[BS];
#pragma unroll
    for (int e = 0; e < BS; ++e)
        q[e] = p[e];
    // recursive halving, written out iteratively
    int n = BS;
#pragma unroll
    for (int h = BS / 2; h >= 1; h >>= 1) {
        const bool upper = (gl & h) != 0;
#pragma unroll
        for (int i = 0; i < BS / 2; ++i) {
            if (i < h) {
                const float keep = upper ? q[i + h] : q[i];
                const float send = upper ? q[i] : q[i + h];
                q[i] = keep + __shfl_xor_sync(PSPMM_FULL_MASK, send, h);
            }
        }
        n = h;
    }
    (void)n;
    return q[0];
}

template <int LPR, int CF, int BS, int VW, bool SEP = false>
__global__ void __launch_bounds__(256) agnn_fused_kernel(const AgnnArgs a)
{
    static_assert(BS <= LPR, "a batch cannot be wider than the lane group");
    const int gpc = blockDim.x / LPR;
    const int g = threadIdx.x / LPR;
    const int gl = threadIdx.x % LPR;
    const int64_t seg = (int64_t)blockIdx.x * gpc + g;
    // Lanes of dead groups run along with empty ranges: the shuffles below are full-warp.
    const bool live = seg < a.n_seg;
    int lb = 0, hb = 0;
    int64_t row = 0;
    bool single = true;
    if (live) {
        lb = __ldg(a.segPtr + seg);
        hb = __ldg(a.segPtr + seg + 1);
        row = seg;
        if (a.target_row) {
            const int me = __ldg(a.target_row + seg);
            const int prev = seg > 0 ? __ldg(a.target_row + seg - 1) : -1;
            const int next = seg + 1 < a.n_seg ? __ldg(a.target_row + seg + 1) : -1;
            row = me;
            single = (prev != me) && (next != me);
        }
    }
    const int nvec = a.dim / VW;
    bool act[CF];
    int voff[CF];
    FVec<VW> av[CF];
    float acc[CF][VW];
#pragma unroll
    for (int cf = 0; cf < CF; ++cf) {
        const int v = cf * LPR + gl;
        act[cf] = v < nvec;
        voff[cf] = act[cf] ? v * VW : 0;
        av[cf] = (live && act[cf]) ? ldg_vec<VW>(a.A + row * a.ldA + voff[cf]) : zero_vec<VW>();
#pragma unroll
        for (int i = 0; i < VW; ++i)
            acc[cf][i] = 0.f;
    }
    float m = -CUDART_INF_F, l = 0.f;
    const int len = hb - lb;
    int maxlen = len;
    if constexpr (LPR < 32)
        maxlen = __reduce_max_sync(PSPMM_FULL_MASK, len);
    const int sub = gl % BS;  // position inside the batch this lane answers for

    // Column indices are read LPR at a time (lane gl <-> entry gl of the chunk, one coalesced
    // load) and one chunk ahead, so that their latency is not part of the per-batch chain.
    int c_next = (lb + gl < hb) ? __ldg(a.colIdx + lb + gl) : 0;
    for (int off0 = 0; off0 < maxlen; off0 += LPR) {
        const int c_chunk = c_next;
        {
            const int kn = lb + off0 + LPR + gl;
            c_next = (kn < hb) ? __ldg(a.colIdx + kn) : 0;
        }
#pragma unroll
        for (int b = 0; b < LPR / BS; ++b) {
            const int off = off0 + b * BS;
            if (off >= maxlen)
                break;  // warp-uniform
            const bool mine = (lb + off + sub) < hb;
            const bool full = (off + BS <= len);
            FVec<VW> x[BS][CF];
            FVec<VW> y[SEP ? BS : 1][SEP ? CF : 1];  // the rows that are aggregated, when they are not B's
            float part[BS];
            int ce[BS];
#pragma unroll
            for (int e = 0; e < BS; ++e)
                ce[e] = __shfl_sync(PSPMM_FULL_MASK, c_chunk, b * BS + e, LPR);
#pragma unroll
            for (int e = 0; e < BS; ++e) {
                const float *brow = a.B + (int64_t)ce[e] * a.ldB;
                if (full) {
#pragma unroll
                    for (int cf = 0; cf < CF; ++cf)
                        x[e][cf] = ldg_vec<VW>(brow + voff[cf]);
                } else {
                    const bool on = (off + e) < len;
#pragma unroll
                    for (int cf = 0; cf < CF; ++cf)
                        x[e][cf] = ldg_vec_if<VW>(brow + voff[cf], on);
                }
                if constexpr (SEP) {
                    const float *vrow = a.Vm + (int64_t)ce[e] * a.ldV;
                    const bool on = (off + e) < len;
#pragma unroll
                    for (int cf = 0; cf < CF; ++cf)
                        y[e][cf] = ldg_vec_if<VW>(vrow + voff[cf], on);
                }
            }
#pragma unroll
            for (int e = 0; e < BS; ++e) {
                float s = 0.f;
#pragma unroll
                for (int cf = 0; cf < CF; ++cf)
                    if (act[cf]) {
#pragma unroll
                        for (int i = 0; i < VW; ++i)
                            s = fmaf(av[cf].v[i], x[e][cf].v[i], s);
                    }
                part[e] = s;
            }
            const float score = a.beta * group_transpose_reduce<LPR, BS>(part, gl);  // entry `sub`
            float p;
            if (a.softmax) {
                float bm = mine ? score : -CUDART_INF_F;
#pragma unroll
                for (int d = BS / 2; d >= 1; d >>= 1)
                    bm = fmaxf(bm, __shfl_xor_sync(PSPMM_FULL_MASK, bm, d));
                const float m_new = fmaxf(m, bm);
                // a group past the end of its segment sees only -inf: keep its state untouched
                const bool any = m_new > -CUDART_INF_F;
                const float sc = any ? expf(m - m_new) : 1.f;
                p = (mine && any) ? expf(score - m_new) : 0.f;
                float ls = p;
#pragma unroll
                for (int d = BS / 2; d >= 1; d >>= 1)
                    ls += __shfl_xor_sync(PSPMM_FULL_MASK, ls, d);
                l = l * sc + ls;
                m = m_new;
#pragma unroll
                for (int cf = 0; cf < CF; ++cf)
#pragma unroll
                    for (int i = 0; i < VW; ++i)
                        acc[cf][i] *= sc;
            } else {
                p = mine ? score : 0.f;
            }
#pragma unroll
            for (int e = 0; e < BS; ++e) {
                const float pe = __shfl_sync(PSPMM_FULL_MASK, p, e, BS);
#pragma unroll
                for (int cf = 0; cf < CF; ++cf)
#pragma unroll
                    for (int i = 0; i < VW; ++i) {
                        if constexpr (SEP)
                            acc[cf][i] = fmaf(pe, y[e][cf].v[i], acc[cf][i]);
                        else
                            acc[cf][i] = fmaf(pe, x[e][cf].v[i], acc[cf][i]);
                    }
            }
        }
    }
    if (!live)
        return;
    if (single) {
        const float inv = a.softmax ? (l > 0.f ? 1.f / l : 0.f) : 1.f;
        float *orow = a.out + row * a.ldOut;
#pragma unroll
        for (int cf = 0; cf < CF; ++cf)
            if (act[cf]) {
                float v[VW];
#pragma unroll
                for (int i = 0; i < VW; ++i)
                    v[i] = acc[cf][i] * inv;
                st_stream_vec<VW>(orow + voff[cf], v);
            }
    } else {
        float *ps = a.scratch + seg * (int64_t)(4 + a.dim_pad);
        if (gl == 0) {
            ps[0] = m;
            ps[1] = l;
        }
#pragma unroll
        for (int cf = 0; cf < CF; ++cf)
            if (act[cf])
                st_vec<VW>(ps + 4 + voff[cf], acc[cf]);
    }
}

// One warp per segment; the warp of the first piece of a split row merges all its pieces.
__global__ void __launch_bounds__(256) agnn_combine_kernel(const AgnnArgs a)
{
    const int64_t seg = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (seg >= a.n_seg)
        return;
    const int me = __ldg(a.target_row + seg);
    const int prev = seg > 0 ? __ldg(a.target_row + seg - 1) : -1;
    const int next = seg + 1 < a.n_seg ? __ldg(a.target_row + seg + 1) : -1;
    if (prev == me || next != me)
        return;  // not the first piece of a row that has several
    const int64_t stride = 4 + a.dim_pad;
    int64_t last = seg;
    float M = -CUDART_INF_F;
    while (last < a.n_seg && __ldg(a.target_row + last) == me) {
        M = fmaxf(M, a.scratch[last * stride]);
        ++last;
    }
    float L = 0.f;
    if (a.softmax) {
        for (int64_t t = seg; t < last; ++t) {
            const float mt = a.scratch[t * stride];
            if (mt > -CUDART_INF_F)
                L += expf(mt - M) * a.scratch[t * stride + 1];
        }
    }
    const float inv = a.softmax ? (L > 0.f ? 1.f / L : 0.f) : 1.f;
    float *orow = a.out + (int64_t)me * a.ldOut;
    for (int j = lane; j < a.dim; j += 32) {
        float s = 0.f;
        for (int64_t t = seg; t < last; ++t) {
            float w = 1.f;
            if (a.softmax) {
                const float mt = a.scratch[t * stride];
                w = mt > -CUDART_INF_F ? expf(mt - M) : 0.f;
            }
            s = fmaf(w, a.scratch[t * stride + 4 + j], s);
        }
        orow[j] = s * inv;
    }
}

template <int LPR, int CF, int BS, int VW, bool SEP = false>
void launch_fused(const AgnnArgs &a, cudaStream_t st)
{
    const int gpc = 256 / LPR;
    const int64_t gx = (a.n_seg + gpc - 1) / gpc;
    agnn_fused_kernel<LPR, CF, BS, VW, SEP><<<(unsigned)gx, 256, 0, st>>>(a);
}

}  // namespace

extern "C" int pspmm_agnn_scratch_bytes(int64_t n_seg, int32_t dim, size_t *bytes)
{
    if (n_seg < 0 || dim <= 0 || !bytes)
        return PSPMM_E_ARG;
    const int64_t dim_pad = (dim + 3) / 4 * 4;
    *bytes = (size_t)n_seg * (size_t)(4 + dim_pad) * sizeof(float);
    return PSPMM_OK;
}

extern "C" int pspmm_agnn_fused_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *A,
                                    const float *B, float *out, int64_t n_rows, int64_t nnz, int32_t dim,
                                    int64_t ldA, int64_t ldB, int64_t ldOut, float beta, int32_t softmax,
                                    int32_t vec_width, int32_t lanes_per_row, int32_t batch,
                                    const int32_t *rowPtr_split, const int32_t *target_row,
                                    int64_t n_seg, void *scratch, size_t scratch_bytes, void *stream)
{
    return pspmm_agnn_fused_apply_csr(rowPtr, colIdx, A, B, B, out, n_rows, nnz, dim, ldA, ldB, ldB, ldOut, beta,
                                      softmax, vec_width, lanes_per_row, batch, rowPtr_split, target_row, n_seg,
                                      scratch, scratch_bytes, stream);
}

extern "C" int pspmm_agnn_fused_apply_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *A,
                                          const float *B, const float *V, float *out, int64_t n_rows, int64_t nnz,
                                          int32_t dim, int64_t ldA, int64_t ldB, int64_t ldV, int64_t ldOut,
                                          float beta, int32_t softmax, int32_t vec_width, int32_t lanes_per_row,
                                          int32_t batch, const int32_t *rowPtr_split, const int32_t *target_row,
                                          int64_t n_seg, void *scratch, size_t scratch_bytes, void *stream)
{
    if (n_rows < 0 || nnz < 0 || dim <= 0)
        return PSPMM_E_ARG;
    if (!V || (ldV != 0 && ldV < dim))
        return PSPMM_E_ARG;
    const bool sep = (V != B) || (ldV != ldB);
    if (sep && (ldV % 4 != 0 || ((uintptr_t)V) % 16 != 0))
        return PSPMM_E_UNSUPPORTED;
    if (n_rows >= INT32_MAX || nnz > INT32_MAX)
        return PSPMM_E_RANGE;
    const bool split = target_row != nullptr || rowPtr_split != nullptr;
    if (split && (!rowPtr_split || !target_row || n_seg < 0 || n_seg >= INT32_MAX))
        return PSPMM_E_ARG;
    if (!split && !rowPtr)
        return PSPMM_E_ARG;
    if (!A || !B || !out || ldA < dim || ldB < dim || ldOut < dim)
        return PSPMM_E_ARG;
    if (nnz > 0 && !colIdx)
        return PSPMM_E_ARG;
    if (batch != 0 && batch != 4 && batch != 8 && batch != 16)
        return PSPMM_E_CONFIG;
    if (lanes_per_row != 0 && lanes_per_row != 4 && lanes_per_row != 8 && lanes_per_row != 16 && lanes_per_row != 32)
        return PSPMM_E_CONFIG;
    // 128-bit accesses throughout: dim a multiple of 4 (at most 256) and 16-byte aligned rows.
    if (dim % 4 != 0 || dim > 256 || ldA % 4 != 0 || ldB % 4 != 0 || ldOut % 4 != 0 ||
        ((uintptr_t)A) % 16 != 0 || ((uintptr_t)B) % 16 != 0 || ((uintptr_t)out) % 16 != 0)
        return PSPMM_E_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_rows == 0)
        return PSPMM_OK;
    AgnnArgs a;
    a.segPtr = split ? rowPtr_split : rowPtr;
    a.target_row = split ? target_row : nullptr;
    a.colIdx = colIdx;
    a.A = A;
    a.B = B;
    a.Vm = V;
    a.ldV = ldV;
    a.out = out;
    a.scratch = (float *)scratch;
    a.n_seg = split ? n_seg : n_rows;
    a.ldA = ldA;
    a.ldB = ldB;
    a.ldOut = ldOut;
    a.dim = dim;
    a.dim_pad = (dim + 3) / 4 * 4;
    a.beta = beta;
    a.softmax = softmax ? 1 : 0;
    if (split) {
        const size_t need = (size_t)n_seg * (size_t)(4 + a.dim_pad) * sizeof(float);
        if (n_seg > 0 && (!scratch || scratch_bytes < need || ((uintptr_t)scratch) % 16 != 0))
            return PSPMM_E_ARG;
        // rows without any segment stay zero
        PSPMM_CUDA_TRY(cudaMemset2DAsync(out, (size_t)ldOut * 4, 0, (size_t)dim * 4, (size_t)n_rows, st));
        if (n_seg == 0)
            return PSPMM_OK;
    }
    // Launch shape: floats per lane per load (VW: 8 = 256-bit loads when the rows are 32-byte
    // aligned, else 4), lanes per row (LPR), slices per lane (CF = ceil(dim / VW / LPR)) and
    // entries per batch (BS).  Few lanes per row put more entries into every warp instruction (the
    // 128-bit form at 16 lanes is bound by instruction issue); wide loads keep the L1 wavefronts
    // full (the 128-bit form at 4 lanes is bound by the L1 data pipe).  Defaults = measured best.
    // (a separate aggregation operand doubles the gathered registers: batches of 4, and with 256-bit
    // loads one slice per lane)
    const bool can8 = dim % 8 == 0 && dim >= 32 && ldA % 8 == 0 && ldB % 8 == 0 && ((uintptr_t)A) % 32 == 0 &&
                      ((uintptr_t)B) % 32 == 0 && (!sep || (ldV % 8 == 0 && ((uintptr_t)V) % 32 == 0));
    if (sep)
        batch = 4;
    if (vec_width != 0 && vec_width != 4 && vec_width != 8)
        return PSPMM_E_CONFIG;
    const int vw = (vec_width == 8 && !can8) ? 4 : (vec_width ? vec_width : (can8 ? 8 : 4));
    const int nvec = dim / vw;
    int lpr = lanes_per_row;
    if (lpr == 0)
        lpr = vw == 8 ? (nvec <= 8 ? 4 : (nvec <= 16 ? 8 : 16)) : (nvec <= 16 ? 4 : (nvec <= 32 ? 8 : 16));
    const int cf_max = vw == 8 ? 2 : 4;
    int cf = (nvec + lpr - 1) / lpr;
    while (cf > cf_max && lpr < 32) {
        lpr *= 2;
        cf = (nvec + lpr - 1) / lpr;
    }
    if (sep && lanes_per_row == 0) {  // two gathered rows per entry: at most two slices per lane (one of 32 bytes) keeps them in registers
        while (cf > (vw == 8 ? 1 : 2) && lpr < 32) {
            lpr *= 2;
            cf = (nvec + lpr - 1) / lpr;
        }
    }
    if (cf > cf_max)
        return PSPMM_E_UNSUPPORTED;
    if (cf == 3)
        cf = 4;
    int bs = batch ? batch : 4;
    if (bs > lpr)
        bs = lpr;
    if (cf * vw >= 16 && bs > 4)
        bs = 4;
    if (cf * vw >= 8 && bs > 8)
        bs = 8;
    bool ok = false;
#define AGNN_CASE_SEP(LPR_, CF_, VW_)                                 \
    if (!ok && sep && vw == VW_ && lpr == LPR_ && cf == CF_ && bs == 4) { \
        launch_fused<LPR_, CF_, 4, VW_, true>(a, st);                 \
        ok = true;                                                    \
    }
    AGNN_CASE_SEP(4, 1, 4) AGNN_CASE_SEP(4, 2, 4) AGNN_CASE_SEP(4, 4, 4) AGNN_CASE_SEP(8, 1, 4) AGNN_CASE_SEP(8, 2, 4)
    AGNN_CASE_SEP(8, 4, 4) AGNN_CASE_SEP(16, 1, 4) AGNN_CASE_SEP(16, 2, 4) AGNN_CASE_SEP(16, 4, 4)
    AGNN_CASE_SEP(32, 1, 4) AGNN_CASE_SEP(32, 2, 4)
    AGNN_CASE_SEP(4, 1, 8) AGNN_CASE_SEP(8, 1, 8) AGNN_CASE_SEP(16, 1, 8) AGNN_CASE_SEP(32, 1, 8)
    AGNN_CASE_SEP(4, 2, 8) AGNN_CASE_SEP(8, 2, 8) AGNN_CASE_SEP(16, 2, 8)
#undef AGNN_CASE_SEP
    if (sep && !ok)
        return PSPMM_E_UNSUPPORTED;
#define AGNN_CASE(LPR_, CF_, BS_, VW_)                             \
    if (!ok && vw == VW_ && lpr == LPR_ && cf == CF_ && bs == BS_) { \
        launch_fused<LPR_, CF_, BS_, VW_>(a, st);                  \
        ok = true;                                                 \
    }
    AGNN_CASE(4, 1, 4, 4) AGNN_CASE(4, 2, 4, 4) AGNN_CASE(4, 4, 4, 4)
    AGNN_CASE(8, 1, 4, 4) AGNN_CASE(8, 1, 8, 4) AGNN_CASE(8, 2, 4, 4) AGNN_CASE(8, 2, 8, 4) AGNN_CASE(8, 4, 4, 4)
    AGNN_CASE(16, 1, 4, 4) AGNN_CASE(16, 1, 8, 4) AGNN_CASE(16, 1, 16, 4) AGNN_CASE(16, 2, 4, 4) AGNN_CASE(16, 2, 8, 4)
    AGNN_CASE(16, 4, 4, 4)
    AGNN_CASE(32, 1, 4, 4) AGNN_CASE(32, 1, 8, 4) AGNN_CASE(32, 1, 16, 4) AGNN_CASE(32, 2, 4, 4) AGNN_CASE(32, 2, 8, 4)
    AGNN_CASE(4, 1, 4, 8) AGNN_CASE(4, 2, 4, 8)
    AGNN_CASE(8, 1, 4, 8) AGNN_CASE(8, 1, 8, 8) AGNN_CASE(8, 2, 4, 8)
    AGNN_CASE(16, 1, 4, 8) AGNN_CASE(16, 1, 8, 8) AGNN_CASE(16, 2, 4, 8)
    AGNN_CASE(32, 1, 4, 8) AGNN_CASE(32, 1, 8, 8)
#undef AGNN_CASE
    if (!ok)
        return PSPMM_E_UNSUPPORTED;
    PSPMM_CUDA_TRY(cudaGetLastError());
    if (split) {
        const int64_t threads = a.n_seg * 32;
        agnn_combine_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(a);
        PSPMM_CUDA_TRY(cudaGetLastError());
    }
    return PSPMM_OK;
}
