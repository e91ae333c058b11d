// 128-row super-windows built on the device from a 16-row condensed format (tall_gpu.cu).
// Plan-internal: callers only ever see the reference's format (src/utils/class.h:74-85).
#pragma once

#include <cstdint>

#include "../../include/b200_spmm.h"

namespace b200spmm {

struct TallFormat {
    uint32_t rows = 128;          // rows of a super-window: 128, or 256 for the CTA-pair kernel
    uint64_t eff = 0, tiles = 0;  // super-windows holding entries, their tiles (rows x CW each)
    uint32_t *d_rowOffset = nullptr, *d_tcA2B = nullptr, *d_rowIdx = nullptr;
    void *d_data = nullptr;  // tiles in the kernel's shared-memory image, 128 rows each: row r of an image has its
                             // two 16-byte halves swapped when (r / 4) is odd.  rows == 256: per window the
                             // images of rows 0-127 of all its tiles, then those of rows 128-255
};

// How many tiles the matrix would have with 128-row windows, as a fraction of its 16-row tiles,
// estimated from up to `max_samples` super-windows spread over the matrix (their column lists are
// copied from the device and merged on the host).  1/8 means every merged window kept the column
// list of its fullest part (executed work unchanged); 1 means nothing was shared (work x 8).
// h_rowOffset / h_rowIdx are host copies of the 16-row arrays.  Returns a B200SPMM status.
int estimate_tall_tile_ratio(const b200spmm_btcf_info_t &info, const uint32_t *h_rowOffset, const uint32_t *h_rowIdx,
                             const uint32_t *d_tcA2B, uint32_t tall_rows, int max_samples, double *ratio,
                             uint64_t *n_super_windows);

// Merges the 16-row windows that share a 128-row window: the column list of a super-window is the
// sorted union of theirs (padded with 0xFFFFFFFF to whole tiles), and every stored tile entry moves
// to its row and column slot in tiles of 128 rows - bit for bit what the converter gives at a window
// height of 128 (src/utils/convert.h:146-225 with ROW_WINDOW = 128).  All arrays in device memory of
// the current device; synchronous.  Only the order of the two halves of a tile row differs from that
// conversion (see TallFormat::d_data).
int build_tall_device(const b200spmm_btcf_info_t &info, const uint32_t *h_rowOffset, const uint32_t *h_rowIdx,
                      const uint32_t *d_rowOffset, const uint32_t *d_tcA2B, const void *d_data, const uint32_t *d_rowIdx,
                      uint32_t tall_rows, TallFormat *out);
void free_tall(TallFormat *t);

}  // namespace b200spmm
