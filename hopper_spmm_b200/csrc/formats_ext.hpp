// The reference's other host-side formats and its file loader, rebuilt:
//   BtcfBitmap  - BTCF_MTX, the bitmap-compressed condensed format (src/utils/class.h:55-67) and
//                 its converter CSR2BTCF (src/utils/convert.h:22-139);
//   Gbtcf       - GBTCF_MTX, windows split into groups of tiles (src/utils/class.h:93-108) and
//                 BTCF2GBTCF (src/utils/convert.h:232-276) with a working validator;
//   CsrHost     - load_matrix (src/utils/load.h:152-322): MatrixMarket coordinate text -> CSR.
#pragma once

#include <cstdint>
#include <vector>

#include "format.hpp"

namespace b200spmm {

// Same windows, column lists and tile order as Btcf; instead of dense tiles it keeps, per tile,
// one bit per slot (row-major: bit lr*CW + lc) and the stored values in that order.
struct BtcfBitmap {
    uint64_t rows = 0, cols = 0, nnzs = 0;
    uint64_t total_row_windows = 0, eff_row_windows = 0, total_tiles = 0;
    int row_window = 8, col_window = 16;
    int dtype = 0, elt_size = 2;
    int bitmap_words = 2;                 // 64-bit words per tile = RW*CW/64
    std::vector<uint32_t> rowOffset;      // [eff+1] tiles
    std::vector<uint32_t> nnzOffset;      // [tiles+1] first stored value of each tile
    std::vector<uint32_t> tcA2B;          // [tiles*CW]
    std::vector<uint64_t> tcBit;          // [tiles*bitmap_words], word j of tile t at t*bitmap_words + j
    std::vector<uint8_t> data;            // [nnzs*elt_size]
    std::vector<uint32_t> rowIdx;         // [eff]
};

// Rows must hold strictly ascending columns (the stored values follow the CSR order while the
// bits follow the columns, so anything else makes the two disagree): B200SPMM_ERR_BAD_CSR otherwise.
int convert_csr_to_btcf_bitmap(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr,
                               const uint32_t *col_idx, const void *values, int dtype, int row_window,
                               int col_window, int n_threads, BtcfBitmap *out);

// Bitmap format -> uncompressed format (dense tiles), e.g. to build an SpMM plan from it.
int expand_bitmap(const BtcfBitmap &in, Btcf *out);

struct Gbtcf {
    uint64_t total_groups = 0;
    uint32_t group_len = 0;               // the reference's tgl: max(floor(mean tiles per window), 32)
    std::vector<uint32_t> groupOffset;    // [groups+1] first tile of each group
    std::vector<uint32_t> rowIdx;         // [groups] first row of the group's window
    std::vector<uint8_t> atomic;          // [groups] 1 when the window has several groups (results must be added)
};

void btcf_to_gbtcf(const std::vector<uint32_t> &rowOffset, const std::vector<uint32_t> &rowIdx, Gbtcf *out);
// 0 when the groups tile every window in order, carry its first row and flag shared windows; else
// the 1-based number of the first group that breaks one of these rules.
uint64_t validate_gbtcf(const std::vector<uint32_t> &rowOffset, const std::vector<uint32_t> &rowIdx, const Gbtcf &g);

struct CsrHost {
    uint64_t rows = 0, cols = 0, nnzs = 0;
    int dtype = 0, elt_size = 2;
    uint64_t declared_nnz = 0;            // what the size line promised
    std::vector<uint32_t> row_ptr, col_idx;
    std::vector<uint8_t> values;
};

int load_matrix_market(const char *path, int dtype, CsrHost *out);

}  // namespace b200spmm
