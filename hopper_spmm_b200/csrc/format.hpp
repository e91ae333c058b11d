// Host-side condensed row-window format (the reference's BTCF_MTX_NO_BITMAP,
// src/utils/class.h:74-85) and its converter (src/utils/convert.h:146-225), with the
// window shape as a run-time parameter and 64-bit element offsets.
#pragma once

#include <cstdint>
#include <vector>

namespace b200spmm {

constexpr uint32_t kIdxMax = 0xFFFFFFFFu;  // IDX_MAX, src/common.h:47

// Schedule cost model.  Starting and draining an accumulator costs the MMA issuer and the epilogue
// warps about as much time as a dozen tiles, so a window is charged its tiles plus this constant;
// matrices with many short windows (the tail of a power-law graph) are then split by time, not by
// tile count alone.
constexpr uint64_t kWindowCharge = 12;

struct Btcf {
    uint64_t rows = 0, cols = 0, nnzs = 0;
    uint64_t total_row_windows = 0, eff_row_windows = 0, total_tiles = 0;
    int row_window = 16, col_window = 16;
    int dtype = 0;     // B200SPMM_F16 / B200SPMM_TF32
    int elt_size = 2;  // bytes per value
    std::vector<uint32_t> rowOffset;  // [eff+1], in tiles
    std::vector<uint32_t> tcA2B;      // [tiles*CW], padded with kIdxMax
    std::vector<uint8_t> data;        // [tiles*RW*CW*elt_size]
    std::vector<uint32_t> rowIdx;     // [eff], first row of each non-empty window
    bool col_major_tiles = false;     // tiles stored column by column (the reference's SPARSE_A_TRANSPOSE build)
};

// Rewrites every tile from row-major to column-major storage or back (src/utils/convert.h:207-213:
// offset = local_col * ROW_WINDOW + local_row under SPARSE_A_TRANSPOSE) and flips the flag.
void transpose_tiles(Btcf *f);

// Returns a B200SPMM_* status.
int validate_csr(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx);

int convert_csr_to_btcf(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr,
                        const uint32_t *col_idx, const void *values, int dtype, int row_window, int col_window,
                        int n_threads, Btcf *out);

// Re-windows a condensed format: `in_*` describe a format with row windows of rw_in rows (the
// reference builds 8, src/common.h:17); the result has windows of rw_out rows (a multiple of
// rw_in) and is, bit for bit, what convert_csr_to_btcf gives at rw_out for the same matrix: the
// column list of an output window is the union of the lists of the input windows it covers, and
// every stored tile entry moves to its row and column slot there.  Lets a format produced by the
// reference's own CSR2BTCFNOBITMAP feed the 16-row kernels without going back to the CSR.
int rewindow_btcf(uint64_t rows, uint64_t cols, uint64_t nnz, int dtype, int rw_in, int col_window,
                  uint64_t eff_row_windows, const uint32_t *in_rowOffset, const uint32_t *in_tcA2B,
                  const void *in_data, const uint32_t *in_rowIdx, int rw_out, int n_threads, Btcf *out);

int shard_rows(uint64_t rows, const uint32_t *row_ptr, int row_window, int parts, uint64_t row_charge,
               uint64_t *row_begin);

// Persistent schedule: CTA c owns effective windows [cta_window[c], cta_window[c+1]); the cuts
// follow the running tile count so every CTA streams about total_tiles / n_ctas tiles.
void build_cta_schedule(const uint32_t *rowOffset, uint64_t eff_row_windows, int n_ctas,
                        std::vector<uint32_t> *cta_window);

// Tile-granular schedule: the tile stream is cut into `n_parts` chunks of about equal cost
// (tiles + kWindowCharge per window); chunk c holds tiles [tile[c], tile[c+1]), which lie in
// windows wfirst[c] .. wlast[c].  Cutting on tiles lets a window heavier than one chunk be shared
// out.  A window whose tiles end up in more than one chunk is a "split": each chunk writes its
// piece to a partial-result slot (head_slot[c] for the chunk's first window when it began in an
// earlier chunk, tail_slot[c] for a window cut at the chunk's end, kNoSlot otherwise; a piece cut
// on both sides uses the head slot) and the pieces are summed afterwards in tile order.  Cuts
// closer than a small tolerance to a window boundary snap to it.  With allow_split == false every
// cut is a window boundary.
constexpr uint32_t kNoSlot = 0xFFFFFFFFu;
struct TileSchedule {
    std::vector<uint32_t> tile, wfirst, wlast;  // [n_parts + 1], [n_parts], [n_parts]
    std::vector<uint32_t> head_slot, tail_slot;  // [n_parts]
    uint32_t n_slots = 0;
    struct Split { uint32_t window, piece_begin, piece_end; };
    std::vector<Split> splits;
    std::vector<uint32_t> piece_slots;  // slots of every split window's pieces, in tile order
};
void build_tile_schedule(const uint32_t *rowOffset, uint64_t eff_row_windows, int n_parts, bool allow_split,
                         TileSchedule *out);

// Bands of a schedule: up to `want` runs of consecutive chunks with about the same number of
// chunks each, cut only where a chunk starts on a window boundary, so that no window is shared
// between two bands.  Band k covers chunks [chunk[k], chunk[k+1]), rows [row[k], row[k+1]) of C
// (the rows of its windows and of the empty windows after them; band 0 also the rows before the
// first window) and the split windows [split[k], split[k+1]) of the schedule.
struct RowBands {
    std::vector<uint32_t> chunk, split;
    std::vector<uint64_t> row;
};
void build_row_bands(const TileSchedule &sc, const uint32_t *rowIdx, uint64_t rows, uint32_t want, RowBands *out);

// The all-gather of N byte ranges [cut[d], cut[d+1]) of unequal length (see exchange_ranges in sharded.cu).
// exchange_even_part: bytes of an even part when the exchange runs in two steps (misplaced bytes to the holder of
// their even part, then an all-gather of the even parts), the common length when all ranges are equal (the
// all-gather alone), or 0: every range goes to everybody directly.
uint64_t exchange_even_part(const uint64_t *cut, int n);
// Step 1 of device d with its step-th peer pair: it sends to `to` what it holds of to's even part (out[0..1]) and
// of the tail past n whole parts (out[2..3]), and receives from `from` what that one holds of d's even part
// (out[4..5]) and of the tail (out[6..7]); a pair lo >= hi is empty.
void exchange_pieces(const uint64_t *cut, int n, uint64_t part, int d, int step, int *to, int *from, uint64_t out[8]);

}  // namespace b200spmm
