/*
 * b200_spmm.h - C ABI of the B200 (sm_100a) condensed row-window SpMM.
 *
 * The library replaces the host-side operator path of Ritt2020/hopper_spmm
 *
 *     CSR_MTX --CSR2BTCFNOBITMAP--> BTCF_MTX_NO_BITMAP --fp16_spmm / tf32--> dense C
 *
 * behind plain C entry points: pointers, sizes, integer status codes.  Nothing here
 * exits the process or prints; every call returns B200SPMM_OK (0) or a negative code
 * that b200spmm_status_string() explains.  Each declaration cites the reference
 * interface it stands in for (paths are inside the reference project).
 *
 * Threading: handles are immutable once created and may be shared between threads.
 * One launch per plan may be in flight at a time (the plan owns one status word and
 * one persistent-schedule table on the device).
 */
#ifndef B200_SPMM_H_
#define B200_SPMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status codes */
/* The reference reports errors by printing and exit(1) (src/utils/utils.h:9-21). */
enum {
    B200SPMM_OK = 0,
    B200SPMM_ERR_INVALID_ARG = -1,   /* null pointer, bad enum, negative size            */
    B200SPMM_ERR_BAD_CSR = -2,       /* row_ptr not monotone / ends != nnz / col >= cols */
    B200SPMM_ERR_UNSUPPORTED = -3,   /* shape or alignment the kernels do not handle     */
    B200SPMM_ERR_NO_MEMORY = -4,     /* host allocation failed                           */
    B200SPMM_ERR_CUDA = -5,          /* a CUDA runtime / driver call failed              */
    B200SPMM_ERR_NO_DEVICE = -6,     /* no sm_100 device, or the driver is missing       */
    B200SPMM_ERR_DEVICE_TIMEOUT = -7 /* a bounded wait inside a kernel ran out           */
};

/* Element type of A's values and of B.  Mirrors -DUSE_FP16 / -DUSE_TF32 (src/common.h:14-43). */
enum { B200SPMM_F16 = 0, B200SPMM_TF32 = 1 };
/* Element type C is stored in.  The reference's DENSE_MTX is MAT_VAL_TYPE (src/utils/class.h:44-48). */
enum { B200SPMM_C_F32 = 0, B200SPMM_C_F16 = 1 };

const char *b200spmm_status_string(int status);
/* Text of the last CUDA error seen by the calling thread ("" if none). */
const char *b200spmm_last_cuda_error(void);
int b200spmm_version(void);

/* ------------------------------------------------------------------ format (host) */

/* Opaque host-side BTCF_MTX_NO_BITMAP (src/utils/class.h:74-85). */
typedef struct b200spmm_btcf b200spmm_btcf_t;

/* Scalar fields of BTCF_MTX_NO_BITMAP plus the window shape, which the reference fixes at
 * compile time (ROW_WINDOW / COL_WINDOW, src/common.h:17-18,40-41). */
typedef struct {
    uint64_t rows, cols, nnzs;
    uint64_t total_row_windows; /* ceil(rows / row_window)             */
    uint64_t eff_row_windows;   /* windows holding at least one entry  */
    uint64_t total_tiles;       /* rowOffset[eff_row_windows]          */
    int32_t row_window, col_window;
    int32_t dtype;    /* B200SPMM_F16 / B200SPMM_TF32 */
    int32_t elt_size; /* bytes per value in `data`    */
} b200spmm_btcf_info_t;

/*
 * Replaces  void CSR2BTCFNOBITMAP(const CSR_MTX&, BTCF_MTX_NO_BITMAP&)   src/utils/convert.h:146-225
 * with CSR_MTX (src/utils/class.h:30-37) passed as its fields.  Output is bit-identical to
 * the reference algorithm for the same window shape: per non-empty row window the sorted
 * distinct columns padded with 0xFFFFFFFF to a multiple of col_window, zero-filled
 * row-major row_window x col_window tiles, rowOffset in tiles, rowIdx = first row.
 *   dtype       B200SPMM_F16 (values are IEEE binary16) or B200SPMM_TF32 (values are fp32)
 *   row_window  8 or 16 (the reference uses 8; the sm_100a kernels consume 16)
 *   col_window  0 = the reference's choice for dtype (16 for f16, 8 for tf32), or 4/8/16
 *   n_threads   host threads for the conversion, 0 = all
 * Validates the CSR (the reference does not) and fails with B200SPMM_ERR_BAD_CSR.
 */
int b200spmm_csr2btcf_nobitmap(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr,
                               const uint32_t *col_idx, const void *values, int dtype, int row_window,
                               int col_window, int n_threads, b200spmm_btcf_t **out);

/* Field access of BTCF_MTX_NO_BITMAP (src/utils/class.h:74-85). Pointers stay valid until destroy. */
int b200spmm_btcf_info(const b200spmm_btcf_t *f, b200spmm_btcf_info_t *info);
const uint32_t *b200spmm_btcf_rowOffset(const b200spmm_btcf_t *f); /* [eff_row_windows + 1]              */
const uint32_t *b200spmm_btcf_tcA2B(const b200spmm_btcf_t *f);     /* [total_tiles * col_window]         */
const void *b200spmm_btcf_data(const b200spmm_btcf_t *f);          /* [total_tiles * row_window * col_window] */
const uint32_t *b200spmm_btcf_rowIdx(const b200spmm_btcf_t *f);    /* [eff_row_windows]                  */
/*
 * Re-windows a BTCF_MTX_NO_BITMAP given as its host arrays (src/utils/class.h:74-85; `info`
 * carries rows, cols, nnzs, eff_row_windows, total_tiles, row_window, col_window, dtype): the
 * result has windows of `row_window` rows (8, 16, 32, 64 or 128, a multiple of info->row_window) and
 * is bit-identical to converting the same matrix directly at that height.  The reference's converter is fixed at
 * 8-row windows (ROW_WINDOW, src/common.h:17) while the sm_100a kernels consume 16: this is how a
 * format built by the reference's own CSR2BTCFNOBITMAP (src/utils/convert.h:146-225) reaches
 * b200spmm_plan_create, in place of handing it to fp16_spmm (src/fp16.cu:221).  The input is
 * validated (ascending aligned windows, ascending columns below cols, padding only at the end of
 * a window's last tile); anything else fails with B200SPMM_ERR_INVALID_ARG.
 */
int b200spmm_btcf_rewindow(const b200spmm_btcf_info_t *info, const uint32_t *rowOffset, const uint32_t *tcA2B,
                           const void *data, const uint32_t *rowIdx, int row_window, int n_threads,
                           b200spmm_btcf_t **out);

/*
 * The reference's SPARSE_A_TRANSPOSE build stores every tile column by column (src/utils/convert.h:207-213:
 * offset = local_col * ROW_WINDOW + local_row).  b200spmm_btcf_transpose_tiles rewrites the tiles of `f` in
 * place from row-major to column-major or back; b200spmm_btcf_tiles_col_major says which it holds (1 / 0).
 * Everything else in the format is the same in both builds.  The kernels read row-major tiles, so
 * b200spmm_plan_create refuses a column-major format with B200SPMM_ERR_UNSUPPORTED (the reference's own
 * kernel never reads the transposed tiles either: its tensor map is the row-major one, src/fp16.cu:177-219).
 */
int b200spmm_btcf_transpose_tiles(b200spmm_btcf_t *f);
int b200spmm_btcf_tiles_col_major(const b200spmm_btcf_t *f);

/* The reference's structs are freed by going out of scope (std::vector members). */
void b200spmm_btcf_destroy(b200spmm_btcf_t *f);

/*
 * The same conversion on the GPU, for CSR arrays that already live on `device`; output arrays
 * stay on the device (hand them to b200spmm_plan_create_device).  Bit-identical to
 * b200spmm_csr2btcf_nobitmap - and so to src/utils/convert.h:146-225 - for rows whose columns are
 * ascending and distinct, which is what the reference's loader produces (src/utils/load.h:137-145);
 * anything else is refused with B200SPMM_ERR_BAD_CSR.  Synchronous with respect to `stream`.
 */
typedef struct b200spmm_dbtcf b200spmm_dbtcf_t;
int b200spmm_csr2btcf_nobitmap_device(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *d_row_ptr,
                                      const uint32_t *d_col_idx, const void *d_values, int dtype, int row_window,
                                      int col_window, int device, void *stream, b200spmm_dbtcf_t **out);
int b200spmm_dbtcf_info(const b200spmm_dbtcf_t *f, b200spmm_btcf_info_t *info);
const uint32_t *b200spmm_dbtcf_rowOffset(const b200spmm_dbtcf_t *f); /* device pointers, valid until destroy */
const uint32_t *b200spmm_dbtcf_tcA2B(const b200spmm_dbtcf_t *f);
const void *b200spmm_dbtcf_data(const b200spmm_dbtcf_t *f);
const uint32_t *b200spmm_dbtcf_rowIdx(const b200spmm_dbtcf_t *f);
/* Copies the four arrays into host buffers sized from b200spmm_dbtcf_info. */
int b200spmm_dbtcf_copy_to_host(const b200spmm_dbtcf_t *f, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                                uint32_t *rowIdx);
void b200spmm_dbtcf_destroy(b200spmm_dbtcf_t *f);

/* ------------------------------------------------------------------ row-window sharding */

/*
 * nnz-balanced contiguous row ranges for `parts` GPUs, cut on row-window boundaries
 * (the reference has no multi-GPU path; its only decomposition is row windows over CTAs,
 * src/fp16.cu:86,138).  row_begin[parts+1] receives the cuts: part p owns rows
 * [row_begin[p], row_begin[p+1]); every cut is a multiple of row_window or equals rows.
 */
int b200spmm_shard_rows(uint64_t rows, const uint32_t *row_ptr, int row_window, int parts, uint64_t *row_begin);
/*
 * Same cuts on the cost  nnz + row_charge * rows.  Every row costs a GPU time whatever it holds
 * (its share of a window's accumulator hand-over and of C's bytes), so on power-law matrices a
 * charge of about 6 entries per row evens out the ranks' times where pure nnz balance leaves the
 * rank with the long sparse tail slower.  row_charge = 0 is b200spmm_shard_rows.
 */
int b200spmm_shard_rows_weighted(uint64_t rows, const uint32_t *row_ptr, int row_window, int parts,
                                 uint64_t row_charge, uint64_t *row_begin);

/*
 * The sharded operator: the same blocking host call as fp16_spmm (src/fp16.cu:221-281), over several
 * GPUs of this process.  b200spmm_sharded_create cuts the rows with b200spmm_shard_rows_weighted
 * (row_charge: 6 balances the GPUs' times on power-law graphs, 0 is plain nnz balance), gives every
 * device its rows of the CSR, converts them there and plans them.  devices[] lists distinct CUDA device
 * ordinals; shard p lives on devices[p] and owns rows [row_begin[p], row_begin[p+1]).
 *   b200spmm_spmm_sharded       every shard's product on its own device and stream: d_B[p] is B
 *                               (replicated: a device pointer on devices[p]), d_C[p] receives the
 *                               shard's rows of C.  Asynchronous; b200spmm_sharded_sync waits for all
 *                               shards and returns the first kernel status that is not OK.
 *   b200spmm_spmm_sharded_host  B [cols, n] and C [rows, n] in host memory (pinned for full speed):
 *                               every device copies 1/N of B in and the parts are exchanged GPU to GPU
 *                               (NCCL all-gather over NVLink), so B crosses the host link once, not N
 *                               times; then the products; then every shard's rows of C go back to
 *                               their place in h_C.  Blocking.
 *   b200spmm_allgather_c        the optional collective: d_C_full[p] is a [rows, n] array on
 *                               devices[p] that already holds shard p's rows in place (let
 *                               b200spmm_spmm_sharded write them there: d_C[p] = d_C_full[p] +
 *                               row_begin[p] * ldc); on return, in stream order, every device holds
 *                               all rows.  The ranges may differ in length: bytes outside their holder's
 *                               even share first move to the device whose even share they fall into (one
 *                               grouped send/receive), then NCCL's in-place all-gather of the even shares
 *                               loads all links alike; where that saves the busiest device less than 15 %
 *                               of its sends, every range goes to everybody directly.
 *                               b200spmm_allgather_plan (below) gives the plan for given ranges.
 *   b200spmm_sharded_stream     the cudaStream_t shard p's work is queued on (a non-blocking stream of the
 *                               handle's own: whatever produces d_B / d_C on other streams has to be
 *                               complete, or ordered before this stream, when the calls above are made).
 * NCCL (libnccl.so.2) is loaded when the first collective is needed; without it the two collective
 * calls fail with B200SPMM_ERR_UNSUPPORTED on more than one device and everything else works.  Every
 * buffer a kernel or NCCL sees is memory of the device it runs on.  One call at a time per handle.
 */
typedef struct b200spmm_sharded b200spmm_sharded_t;
int b200spmm_sharded_create(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx,
                            const void *values, int dtype, const int *devices, int n_devices, uint64_t row_charge,
                            b200spmm_sharded_t **out);
int b200spmm_sharded_info(const b200spmm_sharded_t *s, int *n_devices, uint64_t *row_begin /* [n_devices + 1] */);
void *b200spmm_sharded_stream(const b200spmm_sharded_t *s, int shard);
int b200spmm_spmm_sharded(b200spmm_sharded_t *s, const void *const *d_B, int64_t ldb, int64_t n, void *const *d_C,
                          int64_t ldc, int c_dtype);
int b200spmm_sharded_sync(b200spmm_sharded_t *s);
int b200spmm_spmm_sharded_host(b200spmm_sharded_t *s, const void *h_B, int64_t n, void *h_C, int c_dtype);
int b200spmm_allgather_c(b200spmm_sharded_t *s, void *const *d_C_full, int64_t n, int c_dtype);
/*
 * The plan b200spmm_allgather_c follows for byte ranges [cut[p], cut[p+1]), p < n_parts (host arithmetic only;
 * for callers who run the exchange over a transport of their own, and for tests).  *even_part: bytes of an even
 * share when the exchange runs in two steps, the common length when all ranges are equal (the all-gather
 * alone), 0 when every range goes to everybody.  pieces[(p * (n_parts - 1) + step - 1) * 10 ..]: for device p and
 * step = 1 .. n_parts - 1 the ten numbers {to, from, send lo, send hi, send-tail lo, send-tail hi, receive lo,
 * receive hi, receive-tail lo, receive-tail hi}: p sends to `to` what it holds of to's even share and of the tail
 * past n_parts whole shares, and receives the same from `from`; a pair lo >= hi is empty.  After these, the
 * all-gather of [q * even_part, (q + 1) * even_part) from every q completes the job.
 */
int b200spmm_allgather_plan(const uint64_t *cut, int n_parts, uint64_t *even_part, uint64_t *pieces);
void b200spmm_sharded_destroy(b200spmm_sharded_t *s);

/*
 * Persistent schedule: cta_window[n_ctas+1] receives the cuts of the effective row windows
 * over n_ctas persistent CTAs; CTA c streams windows [cta_window[c], cta_window[c+1]).  Cuts
 * follow the running tile count (rowOffset), so every CTA gets about the same number of tiles
 * however skewed the rows are.  Stands in for the reference's static `row += gridDim.x`
 * round-robin (src/fp16.cu:86,138) and its unused Scheduler singleton (src/scheduler.h:5-42).
 */
int b200spmm_build_schedule(const uint32_t *rowOffset, uint64_t eff_row_windows, int n_ctas, uint32_t *cta_window);
/*
 * The schedule the plan-based SpMM runs: the tile stream cut into n_parts chunks of about equal
 * cost.  Cutting on TILES lets a window heavier than one chunk (a hub row window of a power-law
 * graph) be shared out.  Chunk c holds tiles [cta_tile[c], cta_tile[c+1]), which lie in windows
 * cta_wfirst[c] .. cta_wlast[c]; the plan cuts several chunks per CTA and CTA b runs chunks b,
 * b + n_ctas, ..., so every CTA works in all regions of the matrix.  A window cut at a chunk
 * boundary is computed in pieces: each piece goes to an fp32 slot and a second small kernel sums
 * a window's pieces in tile order, so results do not depend on timing.  slot_window[2*n_parts]
 * receives, for chunk c, at [2c] the window whose piece sits at the head of the chunk (it began
 * in an earlier chunk) and at [2c+1] the window cut at the chunk's end, or 0xFFFFFFFF where the
 * chunk's first / last window is whole; a piece cut on both sides counts as a head piece.  Cuts
 * snap to a window boundary when one is near, so most windows stay whole.  No counterpart in the
 * reference (one CTA per window, src/fp16.cu:86,138).
 */
int b200spmm_build_tile_schedule(const uint32_t *rowOffset, uint64_t eff_row_windows, int n_parts, uint32_t *cta_tile,
                                 uint32_t *cta_wfirst, uint32_t *cta_wlast, uint32_t *slot_window);

/*
 * Bands of that schedule, as the host-buffer SpMM uses them on large matrices: at most max_bands
 * runs of consecutive chunks, cut only where a chunk starts on a window boundary, so a band's rows
 * of C are complete when its chunks are done and can be copied out while the next band is
 * computed.  band_chunk[n_bands+1] and band_row[n_bands+1] (arrays of max_bands+1 elements)
 * receive the chunk and row cuts; band k covers chunks [band_chunk[k], band_chunk[k+1]) and rows
 * [band_row[k], band_row[k+1]).  No counterpart in the reference.
 */
int b200spmm_build_row_bands(const uint32_t *rowOffset, const uint32_t *rowIdx, uint64_t eff_row_windows, uint64_t rows,
                             int n_parts, int max_bands, uint32_t *band_chunk, uint64_t *band_row, int *n_bands);

/* ------------------------------------------------------------------ the reference's other formats */

/*
 * Bitmap-compressed condensed format: BTCF_MTX (src/utils/class.h:55-67) built by CSR2BTCF
 * (src/utils/convert.h:22-139).  Windows, column lists and tile order are those of the
 * uncompressed format; a tile keeps one bit per slot (bit lr*col_window + lc, row-major) in
 * row_window*col_window/64 consecutive 64-bit words, its stored values in bit order, and
 * nnzOffset[tiles+1] gives the first stored value of each tile.  The reference's fp16 build
 * indexes the second bitmap word of a tile by tile number (convert.h:98-100), so its words
 * overlap; here word j of tile t is tcBit[t*words + j].  With 8-row windows every other array
 * equals the reference's bit for bit, and tcBit too in the tf32 build.  Rows must hold strictly
 * ascending columns (B200SPMM_ERR_BAD_CSR otherwise).  col_window 0 selects 16 (fp16) / 8 (tf32).
 */
typedef struct b200spmm_btcfb b200spmm_btcfb_t;
int b200spmm_csr2btcf(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx,
                      const void *values, int dtype, int row_window, int col_window, int n_threads,
                      b200spmm_btcfb_t **out);
int b200spmm_btcfb_info(const b200spmm_btcfb_t *f, b200spmm_btcf_info_t *info, int *bitmap_words);
const uint32_t *b200spmm_btcfb_rowOffset(const b200spmm_btcfb_t *f); /* [eff+1] */
const uint32_t *b200spmm_btcfb_nnzOffset(const b200spmm_btcfb_t *f); /* [tiles+1] */
const uint32_t *b200spmm_btcfb_tcA2B(const b200spmm_btcfb_t *f);     /* [tiles*col_window] */
const uint64_t *b200spmm_btcfb_tcBit(const b200spmm_btcfb_t *f);     /* [tiles*bitmap_words] */
const void *b200spmm_btcfb_data(const b200spmm_btcfb_t *f);          /* [nnz] stored values */
const uint32_t *b200spmm_btcfb_rowIdx(const b200spmm_btcfb_t *f);    /* [eff] */
void b200spmm_btcfb_destroy(b200spmm_btcfb_t *f);
/* The same matrix in the uncompressed format (dense tiles), e.g. to build an SpMM plan from it. */
int b200spmm_btcfb_expand(const b200spmm_btcfb_t *f, b200spmm_btcf_t **out);

/*
 * Group-split work list: GBTCF_MTX (src/utils/class.h:93-108) built by BTCF2GBTCF
 * (src/utils/convert.h:232-276).  The group length is max(floor(mean tiles per window), 32); a
 * window of T tiles becomes ceil(T/length) groups of ceil(T/groups) tiles; groupOffset[groups+1]
 * holds each group's first tile, rowIdx[groups] the first row of its window, atomic[groups] is 1
 * for the groups of a window that has several (their results must be added).  The tile arrays
 * (nnzOffset, tcA2B, tcBit, data) are those of the format the offsets came from, unchanged.
 */
typedef struct b200spmm_gbtcf b200spmm_gbtcf_t;
int b200spmm_btcf2gbtcf(const uint32_t *rowOffset, const uint32_t *rowIdx, uint64_t eff_row_windows, b200spmm_gbtcf_t **out);
int b200spmm_gbtcf_info(const b200spmm_gbtcf_t *g, uint64_t *total_groups, uint32_t *group_len);
const uint32_t *b200spmm_gbtcf_groupOffset(const b200spmm_gbtcf_t *g);
const uint32_t *b200spmm_gbtcf_rowIdx(const b200spmm_gbtcf_t *g);
const uint8_t *b200spmm_gbtcf_atomic(const b200spmm_gbtcf_t *g);
void b200spmm_gbtcf_destroy(b200spmm_gbtcf_t *g);
/*
 * Checks a group list against the windows it was cut from: groups tile every window in order,
 * carry its first row, none is empty, and atomic marks exactly the windows with several groups.
 * Stands in for validateBTCF2GBTCFConversion (src/utils/convert.h:283-402), which assumes a group
 * length of 4 and reads past empty windows.  first_bad_group receives 0, or the 1-based number of
 * the first offending group; the return value is B200SPMM_ERR_BAD_CSR in that case.
 */
int b200spmm_gbtcf_validate(const uint32_t *rowOffset, const uint32_t *rowIdx, uint64_t eff_row_windows,
                            const uint32_t *groupOffset, const uint32_t *group_rowIdx, const uint8_t *atomic,
                            uint64_t total_groups, uint64_t *first_bad_group);

/*
 * MatrixMarket coordinate text -> CSR: load_matrix (src/utils/load.h:152-322).  Leading '%' lines
 * are skipped, the size line is "rows cols entries", every later line that reads as
 * "row col value" (1-based) is an entry and other lines are ignored, reading stops after the
 * promised number of entries and a short file simply has fewer.  The banner is not interpreted
 * (no mirroring of symmetric files; pattern files give no entries).  Entries are ordered by
 * (row, column), repeated pairs in file order.  Values are rounded to fp16 (round to nearest
 * even, load.h:225) or kept as fp32.  Indices outside the matrix give B200SPMM_ERR_BAD_CSR, a
 * file that cannot be opened B200SPMM_ERR_INVALID_ARG.
 */
typedef struct b200spmm_csr b200spmm_csr_t;
int b200spmm_load_matrix(const char *path, int dtype, b200spmm_csr_t **out);
int b200spmm_csr_info(const b200spmm_csr_t *m, uint64_t *rows, uint64_t *cols, uint64_t *nnz, uint64_t *declared_nnz);
const uint32_t *b200spmm_csr_row_ptr(const b200spmm_csr_t *m);
const uint32_t *b200spmm_csr_col_idx(const b200spmm_csr_t *m);
const void *b200spmm_csr_values(const b200spmm_csr_t *m);
void b200spmm_csr_destroy(b200spmm_csr_t *m); /* free_csr_matrix, src/utils/load.h:338 */

/* ------------------------------------------------------------------ device plan */

/* Device-resident format + persistent schedule. Replaces the cudaMalloc/cudaMemcpy block and
 * create_tma_desc_A of fp16_spmm (src/fp16.cu:236-252, 177-219) and the unused Scheduler
 * (src/scheduler.h:5-42). */
typedef struct b200spmm_plan b200spmm_plan_t;

/*
 * Uploads a converted matrix to `device` and builds the schedule: contiguous runs of row
 * windows per persistent CTA, balanced on tile count.  row_window must be 16.
 * n_ctas = 0 selects two CTAs per SM (the kernels are sized for two resident CTAs; B wider than
 * 128 columns is multiplied in passes of 128 features).
 */
int b200spmm_plan_create(const b200spmm_btcf_t *f, int device, int n_ctas, b200spmm_plan_t **out);

/*
 * Same, from format arrays that already live on `device` (for a GPU-side converter or a
 * caller that keeps the format resident).  The plan borrows the four arrays; they must
 * outlive it.  rowOffset is read back once to build the schedule.
 */
int b200spmm_plan_create_device(const b200spmm_btcf_info_t *info, const uint32_t *d_rowOffset,
                                const uint32_t *d_tcA2B, const void *d_data, const uint32_t *d_rowIdx,
                                int device, int n_ctas, b200spmm_plan_t **out);
void b200spmm_plan_destroy(b200spmm_plan_t *p);
int b200spmm_plan_info(const b200spmm_plan_t *p, b200spmm_btcf_info_t *info);

/*
 * C[rows, n] = A * B[cols, n] on the plan's device; B and C are device pointers, row-major
 * with leading dimensions ldb / ldc in elements.  Asynchronous on `stream` (a cudaStream_t).
 * Replaces the launch of fp16_spmm_kernel inside fp16_spmm (src/fp16.cu:36-175, 255-264)
 * for both element types (the reference's tf32.cu has no kernel).
 * Rows of windows with no entries are written as zeros, so C needs no prior clearing.
 *   B, C 16-byte aligned; ldb*sizeof(b) and ldc*sizeof(c) multiples of 16; n a multiple of 8.
 */
int b200spmm_spmm(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc,
                  int c_dtype, void *stream);
/* Named like the reference's operators (src/fp16.cu:221, src/tf32.cu); check the plan's dtype. */
int b200spmm_fp16_spmm(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc,
                       int c_dtype, void *stream);
int b200spmm_tf32_spmm(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc,
                       int c_dtype, void *stream);

/*
 * Blocks until `stream` is idle, then returns the kernel-side status of the plan's last
 * launch (B200SPMM_ERR_DEVICE_TIMEOUT if a bounded wait gave up).
 */
int b200spmm_plan_sync(b200spmm_plan_t *p, void *stream);

/*
 * Host-buffer form of  PERF_RESULT fp16_spmm(BTCF_MTX_NO_BITMAP&, DENSE_MTX& B, DENSE_MTX& C)
 * (src/fp16.cu:221-281): B [cols, n] and C [rows, n] are host arrays (dense, ld = n).  Copies B
 * to the device, runs the product and - unlike the reference, which never reads C back -
 * copies C to the host.  Device buffers for B and C are kept in the plan between calls.
 * Synchronous.
 */
int b200spmm_spmm_host(b200spmm_plan_t *p, const void *h_B, int64_t n, void *h_C, int c_dtype);

/*
 * The reference's timing protocol (WARMUP_RUNS = 3, RUNS = 5, src/common.h:48-49; cudaEvent
 * bracket, src/fp16.cu:255-268): `warmup` untimed launches, then `runs` back-to-back launches
 * between two events on `stream`.  *total_ms receives the bracket time (PERF_RESULT.time).
 */
int b200spmm_bench(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc,
                   int c_dtype, int warmup, int runs, void *stream, float *total_ms);

/*
 * Allocation-free SpMM.  No counterpart in the reference, whose operator allocates and frees
 * all device memory on every call (src/fp16.cu:236-279).
 *
 * For callers that must not, or cannot, allocate device memory at the moment they need the
 * product: a serving loop that has handed every free byte of HBM to its own pool allocator, a
 * host thread inside a latency budget where cudaMalloc's implicit device synchronisation is not
 * acceptable, or a component that is simply not allowed to grow the process's footprint after
 * start-up.  b200spmm_plan_create allocates (the device copy of the matrix, the schedule table,
 * a status word); this entry point allocates no device memory and calls no allocating library
 * routine (on the host it allocates nothing either unless a CUDA call fails, when the runtime's
 * message is composed into a string for b200spmm_last_cuda_error()).  The caller passes the converted matrix as four arrays
 * that already live on `device` (for example carved out of its own pool), B and C.
 *
 * The kernel still needs working memory: the schedule table (one cut per CTA) and its status
 * word.  Both live in a 16 KiB array that is part of the library image on every GPU that loads
 * the library.  Consequences:
 *   - n_ctas may be at most 1024 (0 = two CTAs per SM); more is refused with
 *     B200SPMM_ERR_UNSUPPORTED and a message in b200spmm_last_cuda_error().
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
 *     outside any stream capture.
 *   - Every call rewrites the table and clears the status word on `stream` before the SpMM
 *     kernel reads them, so nothing is carried over from the previous call - but all calls on
 *     a device share the one array: two calls whose kernels can overlap on the GPU (different
 *     streams, no dependency) race on it.  Serialise them.
 *   - The call is asynchronous and does not read the kernel's status word back;
 *     b200spmm_spmm_noalloc_status(device, stream) waits for `stream` and returns
 *     B200SPMM_ERR_DEVICE_TIMEOUT if a bounded wait inside the last allocation-free launch on that
 *     device gave up (it allocates nothing either).
 * Same requirements on shapes and alignment as b200spmm_spmm; d_tcA2B and d_data 16-byte aligned.
 * Asynchronous on `stream`.
 */
int b200spmm_spmm_noalloc(const b200spmm_btcf_info_t *info, const uint32_t *d_rowOffset, const uint32_t *d_tcA2B,
                          const void *d_data, const uint32_t *d_rowIdx, const void *d_B, int64_t ldb, int64_t n,
                          void *d_C, int64_t ldc, int c_dtype, int device, int n_ctas, void *stream);
int b200spmm_spmm_noalloc_status(int device, void *stream);

/*
 * Super-windows.  When the 16-row windows of a matrix already touch most of its columns (a pruned
 * weight matrix: at 10 % unstructured density a 16-row window holds 81 % of all columns) the plan
 * also keeps the matrix in windows of 128 rows - eight windows merged, column lists united, the
 * converter's algorithm (src/utils/convert.h:146-225) at ROW_WINDOW = 128 - and multiplies it with a
 * kernel whose MMA is 128 window rows x 128/256 features instead of 128 features x 16 rows.  The choice
 * is made when the plan is created (the merge must leave fewer than ~0.7 of the tiles, estimated on a
 * sample of windows; B200SPMM_WINDOW=16 or =128 in the environment overrides it) and per launch (B at
 * least 128 bytes wide, enough windows x feature slabs to occupy every SM).  The format handed to
 * callers is unchanged.  b200spmm_plan_tall_info reports the merged format (row_window 128, or 0 when
 * the plan has none); b200spmm_plan_tall_copy_to_host copies its four arrays out (buffers sized from
 * that info) so that it can be compared with a conversion at 128 rows.  No counterpart in the
 * reference, which fixes ROW_WINDOW at 8 (src/common.h:17).
 */
int b200spmm_plan_tall_info(const b200spmm_plan_t *p, b200spmm_btcf_info_t *info);
int b200spmm_plan_tall_copy_to_host(const b200spmm_plan_t *p, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                                    uint32_t *rowIdx);
/*
 * Such a plan may keep the matrix a third time, in windows of 256 rows, for launches wider than 128
 * features: a pair of CTAs on neighbouring SMs (a cluster of two) then shares one MMA of 256 window rows x
 * 256 features, each CTA holding half of either operand, which halves what an SM fetches of B per tile.
 * Kept when the 256-row windows have at most 0.55 of the 128-row tiles (B200SPMM_WINDOW=256 forces it,
 * =128 keeps it out).  The two calls below are the counterparts of the two above for that copy
 * (row_window 256, or 0 when the plan has none).
 */
int b200spmm_plan_pair_info(const b200spmm_plan_t *p, b200spmm_btcf_info_t *info);
int b200spmm_plan_pair_copy_to_host(const b200spmm_plan_t *p, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                                    uint32_t *rowIdx);

/* Per-launch facts of the most recent b200spmm_spmm on this plan. */
typedef struct {
    int32_t n_ctas, threads, stages;
    int32_t feature_slab; /* features one CTA pass covers */
    int32_t n_slabs;
    int64_t smem_bytes;
    int64_t kernel_launches; /* launches issued by that call */
    int32_t tma_gather;      /* 1: rows of B fetched by TMA tile::gather4, 0: by cp.async copies */
    int32_t bitmap_tiles;    /* 0: dense tiles; 1: tiles streamed as bitmap + stored values and expanded in the kernel;
                                2: tiles streamed as records of 32 (position, value) words (B200SPMM_TILES=entries) */
    int32_t row_window;      /* rows per window the launched kernel consumed: 16, or 128 (super-windows) */
} b200spmm_launch_info_t;
int b200spmm_plan_launch_info(const b200spmm_plan_t *p, b200spmm_launch_info_t *info);

#ifdef __cplusplus
}
#endif
#endif /* B200_SPMM_H_ */
