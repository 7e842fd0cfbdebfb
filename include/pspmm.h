/*
 * libpspmm — C ABI of the B200 (sm_100a) sparse hot path: CSR/PCSR x dense SpMM, the
 * pattern-masked SDDMM, and the PCSR index builders.
 *
 * This is the drop-in boundary.  Each entry point states which function of the
 * ParamSpMM_AE project (path inside that project : lines) it stands in for.  All device
 * pointers are plain CUDA device addresses on the current device; all "host" pointers are
 * ordinary process memory.  Index arrays are int32, values and dense operands fp32,
 * dense matrices row-major with an explicit leading dimension counted in floats.
 *
 * Conventions
 *   - Every function returns 0 (PSPMM_OK) or a negative PSPMM_E_* code; nothing here ever
 *     calls exit() or prints.  pspmm_strerror() names a code; pspmm_last_cuda_error()
 *     returns the CUDA runtime error text behind the most recent PSPMM_E_CUDA on this thread.
 *   - Device functions enqueue work on `stream` (a cudaStream_t passed as void*; NULL is the
 *     legacy default stream) and return without synchronising, except the pspmm_profile_*
 *     family, which synchronises on its own events.
 *   - Device functions allocate nothing: outputs are caller-allocated.  Unless stated
 *     otherwise an output is fully overwritten, so it does not have to be zeroed first.
 *   - Inputs are never modified.
 */
#ifndef PSPMM_H
#define PSPMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Marks the exported entry points (the library is built with hidden default visibility). */
#if defined(__GNUC__)
#define PSPMM_API __attribute__((visibility("default")))
#else
#define PSPMM_API
#endif

#define PSPMM_OK 0
#define PSPMM_E_ARG (-1)      /* null pointer, negative size, misaligned leading dimension ... */
#define PSPMM_E_CONFIG (-2)   /* a pspmm_cfg field or CF / blkWarpNum hint outside its domain */
#define PSPMM_E_CUDA (-3)     /* a CUDA runtime call or kernel launch failed */
#define PSPMM_E_UNSUPPORTED (-4)
#define PSPMM_E_RANGE (-5)    /* a size exceeds what int32 indices (or a fixed built-in buffer) can address */
#define PSPMM_E_IO (-6)       /* a file cannot be opened, mapped, written or renamed */
#define PSPMM_E_FORMAT (-7)   /* a file's contents contradict its header (or its checksum) */
#define PSPMM_E_NOMEM (-8)    /* host memory for temporary arrays could not be obtained */

/*
 * Kernel parameters.  Zero in any field means "let the library choose".  These replace the
 * reference's template tuple <CF, blkWarpNum> (SpMM/SpMM.cpp:77-141): the legacy pair is
 * still accepted as hint_CF / hint_blkWarpNum and validated against the reference's domain
 * (CF 1..8, blkWarpNum 4 or 8; CF 1..4 for SDDMM), but it does not constrain the launch.
 */
typedef struct pspmm_cfg {
    int32_t lanes_per_row;   /* lanes that share one (split-)row: 1,2,4,8,16,32; rows per warp = 32 / this */
    int32_t vec_width;       /* floats per lane per load of a dense row: 1, 2 or 4 (128-bit) */
    int32_t cta_threads;     /* 32, 64, 128 or 256 */
    int32_t rows_per_group;  /* consecutive (split-)rows one lane group owns: 1..16 */
    int32_t gather_batch;    /* 16-byte gathers a lane keeps in flight: 2, 4, 8 or 16 (registers vs occupancy) */
    int32_t col_tile;        /* SpMM only: dense columns per launch (a multiple of 4, e.g. 128); wider products run as
                                several launches over column ranges.  0 = one launch */
    int32_t hint_CF;         /* legacy coarsening factor, validated only */
    int32_t hint_blkWarpNum; /* legacy warps per block, validated only */
    int32_t bucketed;        /* SpMM on a split layout only: 1 = the split arrays are a length-bucketed plan (see
                                pspmm_spmm_csr): segments in any order, flags in the two high bits of target_row */
    int32_t accumulate;      /* SpMM only: 0 = C is overwritten (every row is written, empty rows with zeros);
                                1 = the product is added to what C holds (reduction instructions; the order in
                                which contributions reach a row is not fixed).  Lets a caller sum products over
                                column blocks of A, e.g. as blocks of B arrive from other GPUs */
} pspmm_cfg;

PSPMM_API int pspmm_version(void);
PSPMM_API const char *pspmm_strerror(int code);
PSPMM_API const char *pspmm_last_cuda_error(void);

/* Resolve a configuration exactly as the SpMM entry points would (fills the zero fields of
 * *cfg for the given dim / leading dimensions / alignment) without launching anything. */
PSPMM_API int pspmm_resolve_cfg(pspmm_cfg *cfg, int32_t dim, int64_t ldB, int64_t ldC, int32_t V,
                      const void *B, const void *C);

/*
 * C[n_rows, dim] = A[n_rows, n_cols] * B[n_cols, dim], A in CSR or in PCSR (row-split CSR).
 *
 * Stands in for csr_spmm (SpMM/SpMM.cpp:77-141 -> SpMM_kernel.cu:129-197, 1157-1243) when
 * rowPtr_split/target_row are NULL, and for csr_split_spmm (SpMM.cpp:143-207 ->
 * SpMM_kernel.cu:199-272, 1245-1360) when they are given; in the split form `rowPtr` may be
 * NULL.  val may be NULL: every stored entry then counts as 1 (the product with the pattern itself).  target_row must be non-decreasing (what split_csr produces).  Unlike the reference
 * the output may have a different row count from B (row shards) and C needs no prior zeroing:
 * rows without entries are written as zeros.  Rows cut into several pieces are accumulated
 * with vector atomics, so their summation order is not fixed.
 *
 * Length-bucketed plan (cfg->bucketed = 1; an internal layout of this library, not one of the
 * reference's): the segments may come in any order, typically sorted by length so that the lane
 * groups of a warp walk equally long pieces, with colIdx / val permuted to match (segment s owns
 * entries rowPtr_split[s] .. rowPtr_split[s+1]).  target_row[s] then holds the row in its low 30
 * bits, bit 31 set when the row has more than one segment (all of them add with atomics) and
 * bit 30 set on exactly one segment of such a row (the pre-pass zeroes the row there).  Every row
 * must appear: rows without entries as empty segments.  n_rows must be below 2^30.
 */
PSPMM_API int pspmm_spmm_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                   const float *B, float *C, int64_t n_rows, int64_t n_cols, int64_t nnz,
                   int32_t dim, int64_t ldB, int64_t ldC, const pspmm_cfg *cfg,
                   const int32_t *rowPtr_split, const int32_t *target_row, int64_t n_seg,
                   void *stream);

/*
 * Same product with V x 1 blocks: block k of block-row r has column colIdx[k] and V values
 * val[k*V .. k*V+V) that multiply B[colIdx[k]] into output rows V*r .. V*r+V-1.
 * V = 2 stands in for bcsr_spmm / bcsr_split_spmm (SpMM/SpMM.cpp:209-337 ->
 * SpMM_kernel.cu:274-417, 1362-1651), V = 3 for vec_spmm / vec_split_spmm
 * (SpMM.cpp:339-480 -> SpMM_kernel.cu:419-562, 1653-1972).  C must have V * n_blk_rows rows.
 * n_seg / target_row describe a split of the block-rows as above (NULL, 0 for none).
 */
PSPMM_API int pspmm_spmm_bcsr(const int32_t *rowPtr_b, const int32_t *colIdx, const float *val, int32_t V,
                    const float *B, float *C, int64_t n_blk_rows, int64_t n_cols, int64_t nblk,
                    int32_t dim, int64_t ldB, int64_t ldC, const pspmm_cfg *cfg,
                    const int32_t *rowPtr_b_split, const int32_t *target_row, int64_t n_seg,
                    void *stream);

/*
 * out[k] = <A[row(k), :], B[colIdx[k], :]> for every stored position k of a CSR pattern.
 * Stands in for csr_sddmm / csr_split_sddmm (SDDMM/sddmm.cpp:15-117 ->
 * sddmm_kernel.cu:143-246, 917-1057).  Stored values are not read.  Any dim is accepted
 * (the reference stops at 128).
 */
PSPMM_API int pspmm_sddmm_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *A, const float *B,
                    float *out, int64_t n_rows, int64_t nnz, int32_t dim, int64_t ldA,
                    int64_t ldB, const pspmm_cfg *cfg, const int32_t *rowPtr_split,
                    const int32_t *target_row, int64_t n_seg, void *stream);

/*
 * Block form: out[k*V+u] = <A[V*row(k)+u, :], B[colIdx[k], :]> where val[k*V+u] != 0, and 0
 * elsewhere (the stored values act as the mask).  Stands in for bcsr_sddmm /
 * bcsr_split_sddmm (SDDMM/sddmm.cpp:119-219 -> sddmm_kernel.cu:248-351, 1059-1287) with
 * V = 2 and vec_sddmm / vec_split_sddmm (sddmm.cpp:221-336) with V = 3.  n_rows_A is the
 * number of rows A really has, at least V*(n_blk_rows-1)+1 (PSPMM_E_ARG below that): when the row
 * count of the matrix is not a multiple of V the last block-row has lanes without a row of A,
 * their (masked) results are zero and nothing is read past row n_rows_A-1.  (The reference's
 * kernels read those rows; its own callers pad A, PCSR.py:322-325.)
 */
PSPMM_API int pspmm_sddmm_bcsr(const int32_t *rowPtr_b, const int32_t *colIdx, const float *val, int32_t V,
                     const float *A, const float *B, float *out, int64_t n_blk_rows, int64_t n_rows_A,
                     int64_t nblk, int32_t dim, int64_t ldA, int64_t ldB, const pspmm_cfg *cfg,
                     const int32_t *rowPtr_b_split, const int32_t *target_row, int64_t n_seg,
                     void *stream);

/*
 * mask[nnz]: position of every CSR entry inside the flattened [nblk, 2] value array of the
 * 2 x 1 block layout.  Stands in for genmask (SDDMM/sddmm.cpp:663-673 ->
 * sddmm_kernel.cu:78-141); bit-exact, device arrays, prints nothing.
 */
PSPMM_API int pspmm_genmask(const int32_t *rowPtr_b, const int32_t *rowPtr, const float *val_b,
                  int64_t n_blk_rows, int64_t n_rows, int64_t nnz, int32_t *mask, void *stream);

/*
 * Host-side PCSR partition.  Stands in for split_csr / split_csr_par (SpMM/SpMM.cpp:15-75;
 * duplicated at SpCONV/SpCONV.cpp:14-74): every row is cut into ceil(len / granularity)
 * pieces.  pspmm_split_count returns the piece count S through *n_seg (int64 prefix sums, so
 * it stays exact where the reference's fp32 cumulative sum does not); pspmm_split_csr fills
 * rowPtr_split[S+1] and target_row[S].  Host arrays; bit-exact with the reference.
 */
PSPMM_API int pspmm_split_count(const int32_t *rowPtr, int64_t n_rows, int32_t granularity, int64_t *n_seg);
PSPMM_API int pspmm_split_csr(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                    int32_t *rowPtr_split, int32_t *target_row, int64_t n_seg);

/*
 * The same partition built on the GPU from a device-resident rowPtr (device arrays in, device
 * arrays out; bit-exact with pspmm_split_csr, hence with SpMM/SpMM.cpp:15-75).  The kernels
 * need scratch memory for per-tile offsets: pspmm_split_device_scratch_bytes() tells how much
 * for a row count, the caller provides it (8-byte aligned device memory).
 * pspmm_split_count_device copies the piece count back and therefore synchronises `stream`;
 * pspmm_split_csr_device only enqueues work, so it cannot return an error for an n_seg that is
 * not the piece count of this rowPtr and granularity: in that case nothing is written outside
 * the arrays and rowPtr_split[0] becomes -1 instead of 0, which the caller can test once the
 * stream has drained (the _static variant below behaves the same).
 */
PSPMM_API int pspmm_split_device_scratch_bytes(int64_t n_rows, size_t *bytes);
PSPMM_API int pspmm_split_count_device(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                       void *scratch, size_t scratch_bytes, int64_t *n_seg, void *stream);
PSPMM_API int pspmm_split_csr_device(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                     int32_t *rowPtr_split, int32_t *target_row, int64_t n_seg,
                                     void *scratch, size_t scratch_bytes, void *stream);

/*
 * pspmm_split_csr_device without any scratch argument and without a single allocation (it has
 * no counterpart in the reference).  Meant for callers that are barred from creating device
 * memory when they need the partition: processes whose GPU memory is fully handed out at
 * start-up, code confined to someone else's memory pool, plug-ins invoked where allocation
 * calls are off limits.  The tile offsets live in a fixed array inside the library (about
 * 128 KiB on every GPU that loads it), which limits the input to 16,777,216 rows; larger
 * inputs get PSPMM_E_RANGE and should use pspmm_split_csr_device.  n_seg comes from
 * pspmm_split_count (host) as usual.  The first call on each device looks up the array's device
 * address; make that first call outside any stream capture.  All calls on a device share the
 * array: calls that can overlap on the GPU race with each other, so keep them on one stream.
 * Leftovers of an earlier call need no clearing, each call rewrites what it reads.
 */
PSPMM_API int pspmm_split_csr_device_static(const int32_t *rowPtr, int64_t n_rows, int32_t granularity,
                                            int32_t *rowPtr_split, int32_t *target_row, int64_t n_seg,
                                            void *stream);

/*
 * Fused attention aggregation over a sparsity pattern: for every stored (i, j)
 *     s_ij = beta * <A_i, B_j>,   a_ij = softmax over the entries of row i of s_ij (softmax != 0)
 *     or a_ij = s_ij (softmax == 0),   out_i = sum_j a_ij * B_j.
 * With softmax == 0 and A == B this is exactly the AGNN propagation the reference composes from
 * ParamSDDMM, a multiplication by the attention weight and ParamSpMM (gnn_conv.py:130-151:
 * AGNN_sddmm, `* attention_w`, AGNN_spmm), computed in one pass without the per-edge array; with
 * softmax != 0 the per-row edge softmax sits between the two.  Stored values are ignored (the
 * pattern is a mask, as in pspmm_sddmm_csr).  Rows without entries give zero rows.
 * dim must be a multiple of 4 and at most 256, A, B and out 16-byte aligned with leading
 * dimensions that are multiples of 4 (PSPMM_E_UNSUPPORTED otherwise).  `vec_width` = floats per lane
 * per load: 0 (library's choice), 4, or 8 (256-bit loads; needs dim a multiple of 8 and 32-byte
 * aligned rows, else 4 is used).  `lanes_per_row` (0 = library's
 * choice, 4, 8, 16 or 32) lanes share one row; `batch` (0, 4, 8 or 16) entries are gathered together
 * per lane group; combinations that are not built are rounded to the nearest built one.
 * Split layouts (rowPtr_split/target_row/n_seg as in pspmm_spmm_csr) need scratch of
 * pspmm_agnn_scratch_bytes(n_seg, dim) bytes, 16-byte aligned, for the partial results of the
 * pieces of split rows; plain CSR needs none (NULL, 0).
 *
 * pspmm_agnn_fused_apply_csr is the same pass with a separate aggregation operand:
 *     out_i = sum_j a_ij * V_j,   a_ij from A and B as above.
 * With A = B = the projected features and V = the upstream gradient G it yields the layer's backward
 * product sum_j a_ij G_j (what gnn_conv.py:157 computes from the saved edge array, AGNN_spmm) from
 * recomputed scores, so training keeps no per-edge array either.  ldV = 0 makes every column use the
 * one row V[0, :] (a row of ones turns the pass into per-row sums of the scores).  V and ldV follow
 * the alignment rules of B; this form runs with 128-bit loads and batches of 4.
 */
PSPMM_API int pspmm_agnn_scratch_bytes(int64_t n_seg, int32_t dim, size_t *bytes);
PSPMM_API int pspmm_agnn_fused_apply_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *A,
                                         const float *B, const float *V, float *out, int64_t n_rows, int64_t nnz,
                                         int32_t dim, int64_t ldA, int64_t ldB, int64_t ldV, int64_t ldOut,
                                         float beta, int32_t softmax, int32_t vec_width, int32_t lanes_per_row,
                                         int32_t batch, const int32_t *rowPtr_split, const int32_t *target_row,
                                         int64_t n_seg, void *scratch, size_t scratch_bytes, void *stream);
PSPMM_API int pspmm_agnn_fused_csr(const int32_t *rowPtr, const int32_t *colIdx, const float *A,
                                   const float *B, float *out, int64_t n_rows, int64_t nnz, int32_t dim,
                                   int64_t ldA, int64_t ldB, int64_t ldOut, float beta, int32_t softmax,
                                   int32_t vec_width, int32_t lanes_per_row, int32_t batch,
                                   const int32_t *rowPtr_split, const int32_t *target_row, int64_t n_seg,
                                   void *scratch, size_t scratch_bytes, void *stream);

/*
 * Exchange step of a row-sharded SpMM across GPUs (it has no counterpart in the reference, which
 * runs on one GPU): copy n rows of a dense operand that is spread over several blocks of memory
 * into the compact buffer dst[n, dim].  Row j of dst is row rows[j] of block s, where s is the
 * source with first[s] <= j < first[s+1] (the list is grouped by source; first[0] = 0,
 * first[n_src] = n).  The blocks are device pointers valid in this process: memory of the current
 * GPU, or another GPU's memory mapped here (peer access over NVLink), read with plain 16-byte
 * loads.  The kernel waits on nothing: the caller orders it after the producers of the blocks and
 * keeps the blocks unchanged until it has finished (one barrier across the ranks on each side).
 * `rotate` (0 <= rotate < n) is the list position the copy starts from, wrapping round: give every
 * rank a different owner's first[] so that the ranks do not read one owner all at once.  `ctas`
 * bounds the thread blocks used (0 = 64), so the copy can run beside a compute kernel.
 * dim, ld_src and ld_dst must be multiples of 4, every base and dst 16-byte aligned.
 */
#define PSPMM_MAX_ROW_SOURCES 16
typedef struct pspmm_row_sources {
    const float *base[PSPMM_MAX_ROW_SOURCES];
    int64_t first[PSPMM_MAX_ROW_SOURCES + 1];
    int32_t n_src;
} pspmm_row_sources;
PSPMM_API int pspmm_pull_rows(const pspmm_row_sources *sources, const int32_t *rows, int64_t n, float *dst,
                              int32_t dim, int64_t ld_src, int64_t ld_dst, int64_t rotate, int32_t ctas,
                              void *stream);
/*
 * The same copy through the bulk asynchronous copy unit (cp.async.bulk global -> shared -> global,
 * completion on an mbarrier; plain untiled copies, no tensor map, no multicast): one warp and a
 * ring of at most 96 KB of shared memory per thread block, no data in registers, so a fetch that
 * runs beside a compute kernel takes far fewer warp slots and registers from it.  Same arguments;
 * `ctas` thread blocks of one warp each.  Rows longer than 1536 bytes go through pspmm_pull_rows.
 * Every wait inside the kernel is bounded (half a second); pspmm_pull_rows_status returns 1 once a
 * wait has run out on this GPU since the library was loaded (it synchronises with the device).
 */
PSPMM_API int pspmm_pull_rows_bulk(const pspmm_row_sources *sources, const int32_t *rows, int64_t n, float *dst,
                              int32_t dim, int64_t ld_src, int64_t ld_dst, int64_t rotate, int32_t ctas,
                              void *stream);
PSPMM_API int pspmm_pull_rows_status(int32_t *status);

/*
 * Host-side CSR -> V x 1 block CSR, laid out exactly as scipy's tobsr((V,1)) (which the
 * reference calls at graph_input.py:245-266): blocks of a block-row appear in order of first
 * encounter while walking its V rows top to bottom.  pspmm_bcsr_count fills rowPtr_b
 * [ceil(n_rows/V)+1] and returns the block count through *nblk; pspmm_bcsr_fill writes
 * colIdx_b[nblk] and val_b[nblk*V] (zeros where a lane has no entry).
 */
PSPMM_API int pspmm_bcsr_count(const int32_t *rowPtr, const int32_t *colIdx, int64_t n_rows, int64_t n_cols,
                     int32_t V, int32_t *rowPtr_b, int64_t *nblk);
PSPMM_API int pspmm_bcsr_fill(const int32_t *rowPtr, const int32_t *colIdx, const float *val, int64_t n_rows,
                    int64_t n_cols, int32_t V, const int32_t *rowPtr_b, int32_t *colIdx_b,
                    float *val_b);

/*
 * MatrixMarket coordinate file -> canonical CSR on the host (columns ascending inside a row,
 * entries with equal coordinates summed in double precision), parsed in parallel from a memory
 * mapping.  Stands in for scipy's mmread followed by tocsr() in the reference's loader
 * (graph_input.py:226-232) and yields the same arrays: symmetric and skew-symmetric files are
 * expanded by mirroring their off-diagonal entries, indices become 0-based.  force_ones != 0
 * replaces every stored value by 1 before the summation, as the reference does
 * (`mtx.data = np.ones_like(mtx.data)`, graph_input.py:227).  pattern / real / integer fields
 * are read; complex or hermitian files and the dense "array" format give PSPMM_E_UNSUPPORTED.
 *
 * pspmm_mtx_info_read parses only the banner and the size line; nnz_max (2 x stored entries for a
 * symmetric file) bounds the CSR entry count, so the caller can size colIdx / val before
 * pspmm_mtx_read_csr, which fills rowPtr[n_rows + 1], colIdx and val (at most `capacity` entries)
 * and returns the entry count through *nnz.  If `capacity` is too small the call returns
 * PSPMM_E_ARG with *nnz set to the count that is needed and colIdx / val untouched.
 */
typedef struct pspmm_mtx_info {
    int64_t n_rows, n_cols;
    int64_t stored;    /* coordinate lines in the file */
    int64_t nnz_max;   /* upper bound of the CSR entry count after expansion */
    int32_t symmetric; /* 0 general, 1 symmetric, 2 skew-symmetric */
    int32_t field;     /* 0 pattern, 1 real, 2 integer */
} pspmm_mtx_info;
PSPMM_API int pspmm_mtx_info_read(const char *path, pspmm_mtx_info *info);
PSPMM_API int pspmm_mtx_read_csr(const char *path, int32_t force_ones, int32_t *rowPtr, int32_t *colIdx,
                                 float *val, int64_t capacity, int64_t *nnz);

/*
 * Binary CSR container, so that a matrix is parsed once and re-loaded at memory-copy speed (the
 * reference re-parses the text file on every run).  Little endian: a 64-byte header (magic
 * "PSPMMCSR", version, n_rows, n_cols, nnz, size and modification time in ns of the text file the
 * arrays came from, checksum of the arrays), then rowPtr, colIdx, val, each section starting on a
 * 64-byte boundary.  pspmm_csr_file_write writes to a temporary name beside `path` and renames;
 * pspmm_csr_file_info reads the header (a caller compares source_size / source_mtime_ns with the
 * text file to detect a stale container); pspmm_csr_file_read copies the arrays into host arrays
 * sized from the header and, with verify != 0, recomputes the checksum (PSPMM_E_FORMAT if it
 * differs, if the header is not a container's, or if the file length disagrees with the header).
 */
typedef struct pspmm_csr_file_info_t {
    int64_t n_rows, n_cols, nnz;
    int64_t source_size, source_mtime_ns;
} pspmm_csr_file_info_t;
PSPMM_API int pspmm_csr_file_write(const char *path, int64_t n_rows, int64_t n_cols, int64_t nnz,
                                   const int32_t *rowPtr, const int32_t *colIdx, const float *val,
                                   int64_t source_size, int64_t source_mtime_ns);
PSPMM_API int pspmm_csr_file_info(const char *path, pspmm_csr_file_info_t *info);
PSPMM_API int pspmm_csr_file_read(const char *path, int32_t *rowPtr, int32_t *colIdx, float *val,
                                  int64_t n_rows, int64_t nnz, int32_t verify);

/*
 * Timing loops.  Stand in for the *_spmm_profile / *_sddmm_profile functions
 * (SpMM/SpMM.cpp:482-889 -> SpMM_kernel.cu:564-1155; SDDMM/sddmm.cpp:338-661): `warmup`
 * untimed launches, then `iters` back-to-back launches between two CUDA events on `stream`;
 * *ms_per_iter receives the mean.  V = 1 selects the CSR kernels, V = 2 / 3 the block ones
 * (n_rows then counts block-rows; n_rows_A of pspmm_profile_sddmm is the row count of A as in
 * pspmm_sddmm_bcsr and is ignored for V = 1).
 */
PSPMM_API int pspmm_profile_spmm(const int32_t *rowPtr, const int32_t *colIdx, const float *val, int32_t V,
                       const float *B, float *C, int64_t n_rows, int64_t n_cols, int64_t nnz,
                       int32_t dim, int64_t ldB, int64_t ldC, const pspmm_cfg *cfg,
                       const int32_t *rowPtr_split, const int32_t *target_row, int64_t n_seg,
                       int32_t warmup, int32_t iters, float *ms_per_iter, void *stream);
PSPMM_API int pspmm_profile_sddmm(const int32_t *rowPtr, const int32_t *colIdx, const float *val, int32_t V,
                        const float *A, const float *B, float *out, int64_t n_rows, int64_t n_rows_A,
                        int64_t nnz, int32_t dim, int64_t ldA, int64_t ldB, const pspmm_cfg *cfg,
                        const int32_t *rowPtr_split, const int32_t *target_row, int64_t n_seg,
                        int32_t warmup, int32_t iters, float *ms_per_iter, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PSPMM_H */
