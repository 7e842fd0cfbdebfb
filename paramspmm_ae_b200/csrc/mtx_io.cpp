// On-disk side of libpspmm: a parallel MatrixMarket reader that produces canonical CSR
// (sorted columns, duplicates summed) and a binary CSR container for re-loading without
// parsing.  The reference parses the text file with scipy on every run and converts with
// coo -> csr (graph_input.py:226-232); the arrays produced here are the ones that path yields.
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <charconv>
#include <memory>
#include <new>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#include "pspmm.h"

namespace {

int io_threads()
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// A read-only mapping of a whole file; empty files map to a null pointer of size 0.
struct Mapped {
    const char *p = nullptr;
    size_t size = 0;
    int fd = -1;
    int open_file(const char *path)
    {
        fd = ::open(path, O_RDONLY);
        if (fd < 0)
            return PSPMM_E_IO;
        struct stat st;
        if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode))
            return PSPMM_E_IO;
        size = (size_t)st.st_size;
        if (size == 0)
            return PSPMM_OK;
        void *m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (m == MAP_FAILED)
            return PSPMM_E_IO;
        p = (const char *)m;
        madvise(m, size, MADV_SEQUENTIAL);
        return PSPMM_OK;
    }
    ~Mapped()
    {
        if (p)
            munmap((void *)p, size);
        if (fd >= 0)
            ::close(fd);
    }
};

inline bool is_blank(char c) { return c == ' ' || c == '\t' || c == '\r'; }

std::string lower_token(const char *&s, const char *end)
{
    while (s < end && is_blank(*s))
        ++s;
    std::string t;
    while (s < end && !is_blank(*s) && *s != '\n')
        t.push_back((char)((*s >= 'A' && *s <= 'Z') ? *s + 32 : *s)), ++s;
    return t;
}

inline const char *line_end(const char *s, const char *end)
{
    const void *nl = memchr(s, '\n', (size_t)(end - s));
    return nl ? (const char *)nl : end;
}

inline bool parse_i64(const char *&s, const char *end, int64_t *out)
{
    while (s < end && is_blank(*s))
        ++s;
    bool neg = false;
    if (s < end && (*s == '+' || *s == '-'))
        neg = *s == '-', ++s;
    if (s >= end || *s < '0' || *s > '9')
        return false;
    int64_t v = 0;
    int digits = 0;
    while (s < end && *s >= '0' && *s <= '9') {
        if (++digits > 18)
            return false;
        v = v * 10 + (*s - '0');
        ++s;
    }
    *out = neg ? -v : v;
    return true;
}

inline bool parse_f64(const char *&s, const char *end, double *out)
{
    while (s < end && is_blank(*s))
        ++s;
    if (s < end && *s == '+')
        ++s;
    auto r = std::from_chars(s, end, *out);
    if (r.ec != std::errc())
        return false;
    s = r.ptr;
    return true;
}

// Banner + size line.  On success *data points at the first byte after the size line.
int parse_header(const Mapped &f, pspmm_mtx_info *info, const char **data)
{
    const char *s = f.p, *end = f.p + f.size;
    if (f.size < 15 || lower_token(s, end) != "%%matrixmarket")
        return PSPMM_E_FORMAT;
    const std::string object = lower_token(s, end), format = lower_token(s, end), field = lower_token(s, end),
                      symmetry = lower_token(s, end);
    if (object != "matrix")
        return PSPMM_E_FORMAT;
    if (format != "coordinate")
        return PSPMM_E_UNSUPPORTED;  // dense "array" files are not sparse input
    if (field == "pattern")
        info->field = 0;
    else if (field == "real" || field == "double")
        info->field = 1;
    else if (field == "integer")
        info->field = 2;
    else if (field == "complex")
        return PSPMM_E_UNSUPPORTED;
    else
        return PSPMM_E_FORMAT;
    if (symmetry == "general")
        info->symmetric = 0;
    else if (symmetry == "symmetric")
        info->symmetric = 1;
    else if (symmetry == "skew-symmetric")
        info->symmetric = 2;
    else if (symmetry == "hermitian")
        return PSPMM_E_UNSUPPORTED;
    else
        return PSPMM_E_FORMAT;
    s = line_end(s, end);
    // comment and blank lines, then "rows cols entries"
    for (;;) {
        if (s >= end)
            return PSPMM_E_FORMAT;
        ++s;  // past the newline
        const char *t = s;
        while (t < end && is_blank(*t))
            ++t;
        if (t < end && (*t == '%' || *t == '\n')) {
            s = line_end(t, end);
            continue;
        }
        s = t;
        break;
    }
    int64_t r, c, e;
    if (!parse_i64(s, end, &r) || !parse_i64(s, end, &c) || !parse_i64(s, end, &e) || r < 0 || c < 0 || e < 0)
        return PSPMM_E_FORMAT;
    if (info->symmetric && r != c)
        return PSPMM_E_FORMAT;
    info->n_rows = r;
    info->n_cols = c;
    info->stored = e;
    info->nnz_max = info->symmetric ? 2 * e : e;
    s = line_end(s, end);
    *data = s < end ? s + 1 : end;
    return PSPMM_OK;
}

struct Entry {
    int32_t row, col;
    double val;
};

// Parses the coordinate lines in [s, end); every line is complete inside the range.
int parse_chunk(const char *s, const char *end, const pspmm_mtx_info &info, bool ones, std::vector<Entry> &out)
{
    while (s < end) {
        while (s < end && (is_blank(*s) || *s == '\n'))
            ++s;
        if (s >= end)
            break;
        if (*s == '%') {
            s = line_end(s, end);
            continue;
        }
        const char *le = line_end(s, end);
        int64_t i, j;
        double v = 1.0;
        if (!parse_i64(s, le, &i) || !parse_i64(s, le, &j))
            return PSPMM_E_FORMAT;
        if (info.field != 0) {
            if (!parse_f64(s, le, &v))
                return PSPMM_E_FORMAT;
            if (ones)
                v = 1.0;
        }
        if (i < 1 || j < 1 || i > info.n_rows || j > info.n_cols)
            return PSPMM_E_FORMAT;
        out.push_back(Entry{(int32_t)(i - 1), (int32_t)(j - 1), v});
        s = le;
    }
    return PSPMM_OK;
}

}  // namespace

extern "C" int pspmm_mtx_info_read(const char *path, pspmm_mtx_info *info)
{
    if (!path || !info)
        return PSPMM_E_ARG;
    Mapped f;
    int rc = f.open_file(path);
    if (rc)
        return rc;
    const char *data;
    return parse_header(f, info, &data);
}

extern "C" int pspmm_mtx_read_csr(const char *path, int32_t force_ones, int32_t *rowPtr, int32_t *colIdx,
                                  float *val, int64_t capacity, int64_t *nnz)
{
    if (!path || !rowPtr || !nnz || capacity < 0 || (capacity > 0 && (!colIdx || !val)))
        return PSPMM_E_ARG;
    Mapped f;
    int rc = f.open_file(path);
    if (rc)
        return rc;
    pspmm_mtx_info info;
    const char *data;
    rc = parse_header(f, &info, &data);
    if (rc)
        return rc;
    if (info.n_rows >= INT32_MAX || info.n_cols >= INT32_MAX || info.nnz_max > INT32_MAX)
        return PSPMM_E_RANGE;
    const char *end = f.p + f.size;
    const int64_t n = info.n_rows;

    // 1. parse: the data region is cut at line ends into one range per thread
    const size_t bytes = (size_t)(end - data);
    const int T = (int)std::max<size_t>(1, std::min<size_t>((size_t)io_threads(), bytes >> 16));
    std::vector<const char *> cut((size_t)T + 1);
    cut[0] = data;
    cut[(size_t)T] = end;
    for (int t = 1; t < T; ++t) {
        const char *c = data + bytes * (size_t)t / (size_t)T;
        c = line_end(c, end);
        cut[(size_t)t] = c < end ? c + 1 : end;
    }
    std::vector<std::vector<Entry>> parts((size_t)T);
    std::vector<int> prc((size_t)T, PSPMM_OK);
#pragma omp parallel for num_threads(T) schedule(static, 1)
    for (int t = 0; t < T; ++t) {
        if (cut[(size_t)t] >= cut[(size_t)t + 1])
            continue;
        try {
            parts[(size_t)t].reserve((size_t)(info.stored / T + 1024));
            prc[(size_t)t] = parse_chunk(cut[(size_t)t], cut[(size_t)t + 1], info, force_ones != 0, parts[(size_t)t]);
        } catch (const std::bad_alloc &) {
            prc[(size_t)t] = PSPMM_E_NOMEM;
        }
    }
    int64_t stored = 0;
    for (int t = 0; t < T; ++t) {
        if (prc[(size_t)t])
            return prc[(size_t)t];
        stored += (int64_t)parts[(size_t)t].size();
    }
    if (stored != info.stored)
        return PSPMM_E_FORMAT;

    // 2. partition by row bucket.  A direct scatter by row is 16-byte stores at random places of
    //    the whole array; buckets of consecutive rows whose entries fit the cache are filled with
    //    sequential streams instead (per thread and bucket, in file order: the layout does not
    //    depend on timing), and the scatter by row happens inside one bucket at a time.
    try {
    const bool mirror = info.symmetric != 0;
    // the reference overwrites the values after the expansion, so forced ones stay +1
    const double sign = (info.symmetric == 2 && !force_ones) ? -1.0 : 1.0;
    int shift = 0;  // rows per bucket = 1 << shift: about 16 K entries (256 KiB) per bucket
    {
        const int64_t want_buckets = std::max<int64_t>(1, std::min<int64_t>(4096, info.nnz_max / 16384));
        while (((n + ((int64_t)1 << shift) - 1) >> shift) > want_buckets)
            ++shift;
    }
    const int64_t NB = std::max<int64_t>(1, (n + ((int64_t)1 << shift) - 1) >> shift);
    std::vector<int64_t> hist((size_t)T * (size_t)NB, 0);  // [thread][bucket], then start offsets
#pragma omp parallel for num_threads(T) schedule(static, 1)
    for (int t = 0; t < T; ++t) {
        int64_t *h = hist.data() + (size_t)t * (size_t)NB;
        for (const Entry &e : parts[(size_t)t]) {
            ++h[e.row >> shift];
            if (mirror && e.row != e.col)
                ++h[e.col >> shift];
        }
    }
    std::vector<int64_t> bstart((size_t)NB + 1, 0);
    {
        int64_t run = 0;
        for (int64_t bk = 0; bk < NB; ++bk) {
            bstart[(size_t)bk] = run;
            for (int t = 0; t < T; ++t) {
                int64_t &h = hist[(size_t)t * (size_t)NB + (size_t)bk];
                const int64_t c = h;
                h = run;
                run += c;
            }
        }
        bstart[(size_t)NB] = run;
    }
    const int64_t expanded = bstart[(size_t)NB];
    // (left uninitialised: every slot is written below)
    std::unique_ptr<Entry[]> byrow(new Entry[(size_t)expanded + 1]);
#pragma omp parallel for num_threads(T) schedule(static, 1)
    for (int t = 0; t < T; ++t) {
        int64_t *cur = hist.data() + (size_t)t * (size_t)NB;
        for (const Entry &e : parts[(size_t)t]) {
            byrow[(size_t)cur[e.row >> shift]++] = e;
            if (mirror && e.row != e.col)
                byrow[(size_t)cur[e.col >> shift]++] = Entry{e.col, e.row, sign * e.val};
        }
        std::vector<Entry>().swap(parts[(size_t)t]);
    }

    // 3. inside every bucket: count per row, then place the entries row by row (through a copy of
    //    the bucket, which is cache-sized)
    std::vector<int64_t> off((size_t)n + 1, 0);
    int fail = 0;
#pragma omp parallel
    {
        std::vector<Entry> tmp;
        std::vector<int64_t> cnt;
#pragma omp for schedule(dynamic, 1)
        for (int64_t bk = 0; bk < NB; ++bk) {
            const int64_t r0 = bk << shift, r1 = std::min<int64_t>(n, (bk + 1) << shift);
            const int64_t lo = bstart[(size_t)bk], hi = bstart[(size_t)bk + 1];
            try {
                tmp.assign(byrow.get() + lo, byrow.get() + hi);
                cnt.assign((size_t)(r1 - r0) + 1, 0);
            } catch (const std::bad_alloc &) {
                __atomic_store_n(&fail, 1, __ATOMIC_RELAXED);
                continue;
            }
            for (const Entry &e : tmp)
                ++cnt[(size_t)(e.row - r0) + 1];
            int64_t run = lo;
            for (int64_t r = r0; r < r1; ++r) {
                const int64_t c = cnt[(size_t)(r - r0) + 1];
                off[(size_t)r] = run;
                cnt[(size_t)(r - r0)] = run;  // becomes the write cursor of row r
                run += c;
            }
            for (const Entry &e : tmp)
                byrow[(size_t)cnt[(size_t)(e.row - r0)]++] = e;
        }
    }
    if (fail)
        return PSPMM_E_NOMEM;
    off[(size_t)n] = expanded;

    // 4. canonical rows: columns ascending, equal coordinates summed (in double, as scipy does)
    std::vector<int64_t> uniq((size_t)n + 1, 0);
#pragma omp parallel for schedule(dynamic, 1024)
    for (int64_t r = 0; r < n; ++r) {
        Entry *b = byrow.get() + off[(size_t)r], *e = byrow.get() + off[(size_t)r + 1];
        std::sort(b, e, [](const Entry &x, const Entry &y) {
            if (x.col != y.col)
                return x.col < y.col;
            uint64_t xb, yb;
            memcpy(&xb, &x.val, 8);
            memcpy(&yb, &y.val, 8);
            return xb < yb;
        });
        int64_t u = 0;
        for (Entry *p = b; p < e; ++p)
            u += (p == b || p->col != (p - 1)->col);
        uniq[(size_t)r + 1] = u;
    }
    for (int64_t r = 0; r < n; ++r)
        uniq[(size_t)r + 1] += uniq[(size_t)r];
    const int64_t total = uniq[(size_t)n];
    *nnz = total;
    if (total > capacity)
        return PSPMM_E_ARG;
#pragma omp parallel for schedule(dynamic, 1024)
    for (int64_t r = 0; r < n; ++r) {
        const Entry *b = byrow.get() + off[(size_t)r], *e = byrow.get() + off[(size_t)r + 1];
        int64_t o = uniq[(size_t)r];
        rowPtr[r] = (int32_t)o;
        for (const Entry *p = b; p < e;) {
            double s = p->val;
            const Entry *q = p + 1;
            for (; q < e && q->col == p->col; ++q)
                s += q->val;
            colIdx[o] = p->col;
            val[o] = (float)s;
            ++o;
            p = q;
        }
    }
    rowPtr[n] = (int32_t)total;
    } catch (const std::bad_alloc &) {
        return PSPMM_E_NOMEM;
    }
    return PSPMM_OK;
}

// ------------------------------------------------------------------- binary CSR container
//
//   bytes 0..63   header (little endian):
//       char  magic[8] = "PSPMMCSR";  uint32 version = 1;  uint32 reserved = 0;
//       int64 n_rows, n_cols, nnz;  int64 source_size, source_mtime_ns;  uint64 checksum
//   then rowPtr[n_rows + 1] (int32), colIdx[nnz] (int32), val[nnz] (float32), each section
//   starting on a 64-byte boundary (zero padding in between).
//   checksum covers the three arrays; source_size / source_mtime_ns describe the text file the
//   arrays were parsed from, so a reader can tell a stale container from a current one.

namespace {

const char CSR_MAGIC[8] = {'P', 'S', 'P', 'M', 'M', 'C', 'S', 'R'};
const uint32_t CSR_VERSION = 1;

struct CsrHeader {
    char magic[8];
    uint32_t version, reserved;
    int64_t n_rows, n_cols, nnz;
    int64_t source_size, source_mtime_ns;
    uint64_t checksum;
};
static_assert(sizeof(CsrHeader) == 64, "the container header is 64 bytes");

inline size_t pad64(size_t x) { return (x + 63) & ~(size_t)63; }

// FNV-1a over 32-bit words, block by block (blocks in parallel), block digests chained in order.
uint64_t digest_words(const void *p, size_t words, uint64_t seed)
{
    const uint32_t *w = (const uint32_t *)p;
    const size_t BLOCK = (size_t)1 << 18;
    const size_t nb = (words + BLOCK - 1) / BLOCK;
    std::vector<uint64_t> d(nb);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < (int64_t)nb; ++b) {
        uint64_t h = 1469598103934665603ull;
        const size_t lo = (size_t)b * BLOCK, hi = std::min(words, lo + BLOCK);
        for (size_t i = lo; i < hi; ++i)
            h = (h ^ w[i]) * 1099511628211ull;
        d[(size_t)b] = h;
    }
    uint64_t h = seed;
    for (size_t b = 0; b < nb; ++b)
        h = (h ^ d[b]) * 1099511628211ull + words;
    return h;
}

uint64_t digest_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *val, int64_t n_rows, int64_t nnz)
{
    uint64_t h = digest_words(rowPtr, (size_t)n_rows + 1, 0x9e3779b97f4a7c15ull);
    h = digest_words(colIdx, (size_t)nnz, h);
    return digest_words(val, (size_t)nnz, h);
}

int header_of(const Mapped &f, CsrHeader *h, size_t *o_rp, size_t *o_ci, size_t *o_v)
{
    if (f.size < sizeof(CsrHeader))
        return PSPMM_E_FORMAT;
    memcpy(h, f.p, sizeof(CsrHeader));
    if (memcmp(h->magic, CSR_MAGIC, 8) != 0 || h->version != CSR_VERSION)
        return PSPMM_E_FORMAT;
    if (h->n_rows < 0 || h->n_cols < 0 || h->nnz < 0 || h->n_rows >= INT32_MAX || h->nnz > INT32_MAX)
        return PSPMM_E_FORMAT;
    *o_rp = sizeof(CsrHeader);
    *o_ci = *o_rp + pad64(((size_t)h->n_rows + 1) * 4);
    *o_v = *o_ci + pad64((size_t)h->nnz * 4);
    if (f.size != *o_v + (size_t)h->nnz * 4)
        return PSPMM_E_FORMAT;
    return PSPMM_OK;
}

bool write_all(int fd, const void *p, size_t n)
{
    const char *c = (const char *)p;
    while (n) {
        ssize_t w = ::write(fd, c, std::min<size_t>(n, (size_t)1 << 30));
        if (w < 0) {
            if (errno == EINTR)
                continue;
            return false;
        }
        c += w;
        n -= (size_t)w;
    }
    return true;
}

void copy_parallel(void *dst, const void *src, size_t bytes)
{
    const size_t BLOCK = (size_t)4 << 20;
    const int64_t nb = (int64_t)((bytes + BLOCK - 1) / BLOCK);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const size_t lo = (size_t)b * BLOCK;
        memcpy((char *)dst + lo, (const char *)src + lo, std::min(BLOCK, bytes - lo));
    }
}

}  // namespace

extern "C" int pspmm_csr_file_write(const char *path, int64_t n_rows, int64_t n_cols, int64_t nnz,
                                    const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                                    int64_t source_size, int64_t source_mtime_ns)
{
    if (!path || !rowPtr || n_rows < 0 || n_cols < 0 || nnz < 0 || (nnz > 0 && (!colIdx || !val)))
        return PSPMM_E_ARG;
    if (n_rows >= INT32_MAX || nnz > INT32_MAX)
        return PSPMM_E_RANGE;
    if (rowPtr[0] != 0 || rowPtr[n_rows] != nnz)
        return PSPMM_E_ARG;
    CsrHeader h;
    memset(&h, 0, sizeof h);
    memcpy(h.magic, CSR_MAGIC, 8);
    h.version = CSR_VERSION;
    h.n_rows = n_rows, h.n_cols = n_cols, h.nnz = nnz;
    h.source_size = source_size, h.source_mtime_ns = source_mtime_ns;
    h.checksum = digest_csr(rowPtr, colIdx, val, n_rows, nnz);
    // written next to the target and renamed, so a reader never sees a partial file
    std::string tmp = std::string(path) + ".tmp." + std::to_string((long long)getpid());
    int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0)
        return PSPMM_E_IO;
    static const char zeros[64] = {0};
    const size_t b_rp = ((size_t)n_rows + 1) * 4, b_e = (size_t)nnz * 4;
    bool ok = write_all(fd, &h, sizeof h) && write_all(fd, rowPtr, b_rp) && write_all(fd, zeros, pad64(b_rp) - b_rp) &&
              write_all(fd, colIdx, b_e) && write_all(fd, zeros, pad64(b_e) - b_e) && write_all(fd, val, b_e);
    ok = (::close(fd) == 0) && ok;
    if (!ok || ::rename(tmp.c_str(), path) != 0) {
        ::unlink(tmp.c_str());
        return PSPMM_E_IO;
    }
    return PSPMM_OK;
}

extern "C" int pspmm_csr_file_info(const char *path, pspmm_csr_file_info_t *info)
{
    if (!path || !info)
        return PSPMM_E_ARG;
    Mapped f;
    int rc = f.open_file(path);
    if (rc)
        return rc;
    CsrHeader h;
    size_t a, b, c;
    rc = header_of(f, &h, &a, &b, &c);
    if (rc)
        return rc;
    info->n_rows = h.n_rows, info->n_cols = h.n_cols, info->nnz = h.nnz;
    info->source_size = h.source_size, info->source_mtime_ns = h.source_mtime_ns;
    return PSPMM_OK;
}

extern "C" int pspmm_csr_file_read(const char *path, int32_t *rowPtr, int32_t *colIdx, float *val,
                                   int64_t n_rows, int64_t nnz, int32_t verify)
{
    if (!path || !rowPtr || n_rows < 0 || nnz < 0 || (nnz > 0 && (!colIdx || !val)))
        return PSPMM_E_ARG;
    Mapped f;
    int rc = f.open_file(path);
    if (rc)
        return rc;
    CsrHeader h;
    size_t o_rp, o_ci, o_v;
    rc = header_of(f, &h, &o_rp, &o_ci, &o_v);
    if (rc)
        return rc;
    if (h.n_rows != n_rows || h.nnz != nnz)
        return PSPMM_E_ARG;  // the caller sized its arrays for another file
    copy_parallel(rowPtr, f.p + o_rp, ((size_t)n_rows + 1) * 4);
    copy_parallel(colIdx, f.p + o_ci, (size_t)nnz * 4);
    copy_parallel(val, f.p + o_v, (size_t)nnz * 4);
    if (rowPtr[0] != 0 || rowPtr[n_rows] != nnz)
        return PSPMM_E_FORMAT;
    if (verify && digest_csr(rowPtr, colIdx, val, n_rows, nnz) != h.checksum)
        return PSPMM_E_FORMAT;
    return PSPMM_OK;
}
