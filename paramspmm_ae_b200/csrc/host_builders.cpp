// Host-side PCSR index builders of libpspmm: row splitting and CSR -> V x 1 block CSR.
// Integer work, bit-exact with the reference's builders; parallel over rows with OpenMP.
#include <stdint.h>

#include <algorithm>
#include <new>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#include "pspmm.h"

namespace {

int max_threads()
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Exclusive prefix sum of per-row counts, computed blockwise in parallel with 64-bit sums.
// counts(r) must be cheap and pure.  off has n + 1 entries on return.
template <typename F>
void prefix_counts(int64_t n, std::vector<int64_t> &off, F &&counts)
{
    off.assign((size_t)n + 1, 0);
    const int T = (int)std::max<int64_t>(1, std::min<int64_t>(max_threads(), (n + 4095) / 4096));
    std::vector<int64_t> part((size_t)T + 1, 0);
#pragma omp parallel num_threads(T)
    {
#ifdef _OPENMP
        const int t = omp_get_thread_num();
#else
        const int t = 0;
#endif
        const int64_t lo = n * t / T, hi = n * (t + 1) / T;
        int64_t run = 0;
        for (int64_t r = lo; r < hi; ++r) {
            off[(size_t)r] = run;
            run += counts(r);
        }
        part[(size_t)t + 1] = run;
#pragma omp barrier
#pragma omp single
        {
            for (int i = 0; i < T; ++i)
                part[(size_t)i + 1] += part[(size_t)i];
        }
        const int64_t base = part[(size_t)t];
        for (int64_t r = lo; r < hi; ++r)
            off[(size_t)r] += base;
    }
    off[(size_t)n] = part[(size_t)T];
}

}  // namespace

extern "C" int pspmm_split_count(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                 int64_t *n_seg)
{
    if (!rowPtr || !n_seg || n_rows < 0 || granularity <= 0)
        return PSPMM_E_ARG;
    int64_t total = 0;
#pragma omp parallel for reduction(+ : total) schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        const int64_t len = (int64_t)rowPtr[r + 1] - rowPtr[r];
        if (len > 0)
            total += (len + granularity - 1) / granularity;
    }
    *n_seg = total;
    return PSPMM_OK;
}

extern "C" int pspmm_split_csr(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                               int32_t *rowPtr_split, int32_t *target_row, int64_t n_seg)
{
    if (!rowPtr || !rowPtr_split || n_rows < 0 || granularity <= 0 || n_seg < 0)
        return PSPMM_E_ARG;
    if (n_seg > 0 && !target_row)
        return PSPMM_E_ARG;
    if (n_seg >= INT32_MAX || n_rows >= INT32_MAX)
        return PSPMM_E_RANGE;
    const int64_t gran = granularity;
    std::vector<int64_t> off;
    try {
        prefix_counts(n_rows, off, [&](int64_t r) {
            const int64_t len = (int64_t)rowPtr[r + 1] - rowPtr[r];
            return len > 0 ? (len + gran - 1) / gran : (int64_t)0;
        });
    } catch (const std::bad_alloc &) {
        return PSPMM_E_NOMEM;
    }
    if (off[(size_t)n_rows] != n_seg)
        return PSPMM_E_ARG;  // caller's piece count does not match this rowPtr / granularity
    rowPtr_split[0] = 0;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        const int64_t end = rowPtr[r + 1];
        int64_t s = off[(size_t)r];
        for (int64_t at = rowPtr[r]; at < end; at += gran, ++s) {
            target_row[s] = (int32_t)r;
            rowPtr_split[s + 1] = (int32_t)std::min(at + gran, end);
        }
    }
    return PSPMM_OK;
}

// Blocks of one block-row in first-encounter order.  `slot` is a per-thread array of n_cols
// entries, all -1 on entry and restored to -1 on exit.  With cols/vals null it only counts.
// `room` bounds the blocks that may be written (the caller's rowPtr_b says how many the
// block-row has); the return value is the number of blocks met, which exceeds `room` when the
// inputs disagree, or -1 when a column id lies outside [0, n_cols).
static int64_t walk_block_row(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                              int64_t n_rows, int64_t n_cols, int32_t V, int64_t br, int32_t *slot,
                              int32_t *cols, float *vals, int64_t room)
{
    int64_t made = 0;
    bool bad_col = false;
    for (int32_t v = 0; v < V && !bad_col; ++v) {
        const int64_t r = br * V + v;
        if (r >= n_rows)
            break;
        for (int32_t k = rowPtr[r]; k < rowPtr[r + 1]; ++k) {
            const int32_t c = colIdx[k];
            if (c < 0 || c >= n_cols) {
                bad_col = true;
                break;
            }
            if (slot[c] < 0) {
                slot[c] = (int32_t)made;
                if (cols && made < room) {
                    cols[made] = c;
                    for (int32_t u = 0; u < V; ++u)
                        vals[made * V + u] = 0.0f;
                }
                ++made;
            }
            if (cols && slot[c] < room)
                vals[(int64_t)slot[c] * V + v] += val[k];
        }
    }
    for (int32_t v = 0; v < V; ++v) {
        const int64_t r = br * V + v;
        if (r >= n_rows)
            break;
        for (int32_t k = rowPtr[r]; k < rowPtr[r + 1]; ++k) {
            const int32_t c = colIdx[k];
            if (c >= 0 && c < n_cols)
                slot[c] = -1;
        }
    }
    return bad_col ? -1 : made;
}

// One column -> slot array per worker thread, allocated before the parallel region so that an
// allocation failure surfaces as an exception in the calling thread.
static std::vector<std::vector<int32_t>> make_slots(int64_t n_cols)
{
    std::vector<std::vector<int32_t>> slots((size_t)max_threads());
    for (auto &s : slots)
        s.assign((size_t)std::max<int64_t>(n_cols, 1), -1);
    return slots;
}

static int this_thread()
{
#ifdef _OPENMP
    return omp_get_thread_num();
#else
    return 0;
#endif
}

extern "C" int pspmm_bcsr_count(const int32_t *rowPtr, const int32_t *colIdx, int64_t n_rows,
                                int64_t n_cols, int32_t V, int32_t *rowPtr_b, int64_t *nblk)
{
    if (!rowPtr || !rowPtr_b || !nblk || n_rows < 0 || n_cols < 0 || V < 1)
        return PSPMM_E_ARG;
    if (n_rows > 0 && rowPtr[n_rows] > 0 && !colIdx)
        return PSPMM_E_ARG;
    try {
        const int64_t nbr = (n_rows + V - 1) / V;
        std::vector<int64_t> cnt((size_t)nbr, 0);
        auto slots = make_slots(n_cols);
        const int T = (int)slots.size();
#pragma omp parallel for schedule(dynamic, 1024) num_threads(T)
        for (int64_t br = 0; br < nbr; ++br)
            cnt[(size_t)br] = walk_block_row(rowPtr, colIdx, nullptr, n_rows, n_cols, V, br,
                                             slots[(size_t)this_thread()].data(), nullptr, nullptr, 0);
        int64_t run = 0;
        rowPtr_b[0] = 0;
        for (int64_t br = 0; br < nbr; ++br) {
            if (cnt[(size_t)br] < 0)
                return PSPMM_E_ARG;  // a column id outside [0, n_cols)
            run += cnt[(size_t)br];
            if (run > INT32_MAX)
                return PSPMM_E_RANGE;
            rowPtr_b[br + 1] = (int32_t)run;
        }
        *nblk = run;
    } catch (const std::bad_alloc &) {
        return PSPMM_E_NOMEM;
    }
    return PSPMM_OK;
}

extern "C" int pspmm_bcsr_fill(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                               int64_t n_rows, int64_t n_cols, int32_t V, const int32_t *rowPtr_b,
                               int32_t *colIdx_b, float *val_b)
{
    if (!rowPtr || !rowPtr_b || n_rows < 0 || n_cols < 0 || V < 1)
        return PSPMM_E_ARG;
    const int64_t nbr = (n_rows + V - 1) / V;
    if (nbr > 0 && rowPtr_b[nbr] > 0 && (!colIdx || !val || !colIdx_b || !val_b))
        return PSPMM_E_ARG;
    int bad = 0;
    try {
        auto slots = make_slots(n_cols);
        const int T = (int)slots.size();
#pragma omp parallel for schedule(dynamic, 1024) num_threads(T)
        for (int64_t br = 0; br < nbr; ++br) {
            const int64_t at = rowPtr_b[br];
            const int64_t room = (int64_t)rowPtr_b[br + 1] - at;
            // never more than `room` blocks are written, whatever the row pointers claim
            const int64_t made = walk_block_row(rowPtr, colIdx, val, n_rows, n_cols, V, br,
                                                slots[(size_t)this_thread()].data(), colIdx_b + at,
                                                val_b + at * V, room < 0 ? 0 : room);
            if (made != room) {
#pragma omp atomic write
                bad = 1;
            }
        }
    } catch (const std::bad_alloc &) {
        return PSPMM_E_NOMEM;
    }
    return bad ? PSPMM_E_ARG : PSPMM_OK;
}
