// Bitmap-compressed and group-split formats and the MatrixMarket loader (see formats_ext.hpp).
// Compiled by nvcc only for the host-side half conversion of cuda_fp16.h; no device code.
#include "formats_ext.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <numeric>

#include <cuda_fp16.h>

#include "../../include/b200_spmm.h"

namespace b200spmm {

// ------------------------------------------------------------------ CSR -> bitmap format
//
// Follows CSR2BTCF (src/utils/convert.h:22-139): per non-empty window the sorted distinct columns
// padded to a multiple of CW; per tile the number of entries, a bitmap with bit lr*CW + lc set for
// an entry at local row lr and local column lc, and the entries' values in row-major order.
// nnzOffset becomes the running sum with a leading zero (convert.h:136-137).  The bitmap of a
// tile takes RW*CW/64 words, word j at tile*words + j; the reference's fp16 build reserves two
// words per tile but indexes them by tile number (convert.h:98-100), which this does not repeat.
int convert_csr_to_btcf_bitmap(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr,
                               const uint32_t *col_idx, const void *values, int dtype, int row_window,
                               int col_window, int n_threads, BtcfBitmap *out) {
    (void)n_threads;
    if (!out || (nnz && !values)) return B200SPMM_ERR_INVALID_ARG;
    if (dtype != B200SPMM_F16 && dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    if (row_window != 8 && row_window != 16) return B200SPMM_ERR_INVALID_ARG;
    if (col_window == 0) col_window = dtype == B200SPMM_F16 ? 16 : 8;
    if (col_window != 8 && col_window != 16) return B200SPMM_ERR_INVALID_ARG;  // a tile fills whole 64-bit words
    int st = validate_csr(rows, cols, nnz, row_ptr, col_idx);
    if (st != B200SPMM_OK) return st;
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t p = row_ptr[r] + 1; p < row_ptr[r + 1]; ++p)
            if (col_idx[p] <= col_idx[p - 1]) return B200SPMM_ERR_BAD_CSR;

    const uint64_t RW = (uint64_t)row_window, CW = (uint64_t)col_window;
    const int esz = dtype == B200SPMM_F16 ? 2 : 4;
    const int words = (int)(RW * CW / 64);
    BtcfBitmap &f = *out;
    f = BtcfBitmap();
    f.rows = rows;
    f.cols = cols;
    f.nnzs = nnz;
    f.row_window = row_window;
    f.col_window = col_window;
    f.dtype = dtype;
    f.elt_size = esz;
    f.bitmap_words = words;
    f.total_row_windows = (rows + RW - 1) / RW;
    f.rowOffset.push_back(0);
    f.nnzOffset.push_back(0);
    try {
        f.data.resize(nnz * esz);
        const uint8_t *vals = static_cast<const uint8_t *>(values);
        std::vector<uint32_t> cols_w, count, fill;
        uint64_t written = 0;  // values placed so far = first value of the current window
        for (uint64_t first = 0; first < rows; first += RW) {
            const uint64_t last = std::min(rows, first + RW);
            if (row_ptr[first] == row_ptr[last]) continue;
            cols_w.assign(col_idx + row_ptr[first], col_idx + row_ptr[last]);
            std::sort(cols_w.begin(), cols_w.end());
            cols_w.erase(std::unique(cols_w.begin(), cols_w.end()), cols_w.end());
            const uint64_t n_tiles = (cols_w.size() + CW - 1) / CW;
            const uint64_t t0 = f.rowOffset.back();
            if (t0 + n_tiles > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;
            f.tcA2B.insert(f.tcA2B.end(), cols_w.begin(), cols_w.end());
            f.tcA2B.resize((t0 + n_tiles) * CW, kIdxMax);
            f.rowOffset.push_back((uint32_t)(t0 + n_tiles));
            f.rowIdx.push_back((uint32_t)first);
            f.tcBit.resize((t0 + n_tiles) * words, 0);
            // entries per tile, then where each tile's values start
            count.assign(n_tiles, 0);
            for (uint64_t p = row_ptr[first]; p < row_ptr[last]; ++p) {
                const uint64_t slot = std::lower_bound(cols_w.begin(), cols_w.end(), col_idx[p]) - cols_w.begin();
                ++count[slot / CW];
            }
            fill.assign(n_tiles, 0);
            uint64_t run = written;
            for (uint64_t t = 0; t < n_tiles; ++t) {
                fill[t] = (uint32_t)run;
                run += count[t];
                f.nnzOffset.push_back((uint32_t)run);
            }
            // rows in order, entries of a row in order: row-major inside every tile
            for (uint64_t r = first; r < last; ++r) {
                const uint64_t lr = r % RW;
                for (uint64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                    const uint64_t slot = std::lower_bound(cols_w.begin(), cols_w.end(), col_idx[p]) - cols_w.begin();
                    const uint64_t t = slot / CW, bit = lr * CW + slot % CW;
                    f.tcBit[(t0 + t) * words + bit / 64] |= 1ull << (bit % 64);
                    std::memcpy(&f.data[(uint64_t)fill[t]++ * esz], vals + p * esz, esz);
                }
            }
            written = run;
        }
    } catch (const std::bad_alloc &) {
        return B200SPMM_ERR_NO_MEMORY;
    }
    f.eff_row_windows = f.rowIdx.size();
    f.total_tiles = f.rowOffset.back();
    return B200SPMM_OK;
}

int expand_bitmap(const BtcfBitmap &in, Btcf *out) {
    if (!out) return B200SPMM_ERR_INVALID_ARG;
    Btcf &f = *out;
    f = Btcf();
    f.rows = in.rows;
    f.cols = in.cols;
    f.nnzs = in.nnzs;
    f.total_row_windows = in.total_row_windows;
    f.eff_row_windows = in.eff_row_windows;
    f.total_tiles = in.total_tiles;
    f.row_window = in.row_window;
    f.col_window = in.col_window;
    f.dtype = in.dtype;
    f.elt_size = in.elt_size;
    const uint64_t slots = (uint64_t)in.row_window * in.col_window, esz = (uint64_t)in.elt_size;
    try {
        f.rowOffset = in.rowOffset;
        f.tcA2B = in.tcA2B;
        f.rowIdx = in.rowIdx;
        f.data.assign(in.total_tiles * slots * esz, 0);
    } catch (const std::bad_alloc &) {
        return B200SPMM_ERR_NO_MEMORY;
    }
    for (uint64_t t = 0; t < in.total_tiles; ++t) {
        uint64_t v = in.nnzOffset[t];
        for (uint64_t bit = 0; bit < slots; ++bit) {
            if (in.tcBit[t * in.bitmap_words + bit / 64] >> (bit % 64) & 1ull) {
                std::memcpy(&f.data[(t * slots + bit) * esz], &in.data[v * esz], esz);
                ++v;
            }
        }
        if (v != in.nnzOffset[t + 1]) return B200SPMM_ERR_INVALID_ARG;  // bits and offsets disagree
    }
    return B200SPMM_OK;
}

// ------------------------------------------------------------------ windows -> groups of tiles
//
// BTCF2GBTCF (src/utils/convert.h:232-276): the group length is the mean number of tiles per
// window, rounded down, but at least 32; a window of T tiles is cut into ceil(T / length) groups
// of ceil(T / groups) tiles (the last one shorter); groups of a shared window carry atomic = 1
// because their results have to be added.
void btcf_to_gbtcf(const std::vector<uint32_t> &rowOffset, const std::vector<uint32_t> &rowIdx, Gbtcf *out) {
    Gbtcf &g = *out;
    g = Gbtcf();
    const uint64_t eff = rowIdx.size();
    const uint64_t tiles = eff ? rowOffset[eff] : 0;
    const double mean = eff ? (double)tiles / (double)eff : 0.0;
    g.group_len = std::max<uint32_t>((uint32_t)mean, 32u);
    for (uint64_t w = 0; w < eff; ++w) {
        const uint32_t T = rowOffset[w + 1] - rowOffset[w];
        const uint32_t n_groups = (T + g.group_len - 1) / g.group_len;
        const uint32_t per_group = n_groups ? (T + n_groups - 1) / n_groups : 0;
        for (uint32_t j = 0; j < n_groups; ++j) {
            g.groupOffset.push_back(rowOffset[w] + per_group * j);
            g.rowIdx.push_back(rowIdx[w]);
            g.atomic.push_back(n_groups == 1 ? 0 : 1);
        }
    }
    g.groupOffset.push_back((uint32_t)tiles);
    g.total_groups = g.groupOffset.size() - 1;
}

// What validateBTCF2GBTCFConversion (src/utils/convert.h:283-402) set out to check, without its
// fixed group length of 4 and its reads past empty windows.
uint64_t validate_gbtcf(const std::vector<uint32_t> &rowOffset, const std::vector<uint32_t> &rowIdx, const Gbtcf &g) {
    const uint64_t eff = rowIdx.size();
    if (g.groupOffset.size() != g.total_groups + 1 || g.rowIdx.size() != g.total_groups || g.atomic.size() != g.total_groups)
        return 1;
    uint64_t k = 0;
    for (uint64_t w = 0; w < eff; ++w) {
        uint32_t at = rowOffset[w];
        uint64_t first = k;
        while (k < g.total_groups && at < rowOffset[w + 1]) {
            if (g.groupOffset[k] != at || g.rowIdx[k] != rowIdx[w]) return k + 1;
            const uint32_t end = g.groupOffset[k + 1];
            if (end <= at || end > rowOffset[w + 1]) return k + 1;  // empty group, or one that leaves its window
            at = end;
            ++k;
        }
        if (at != rowOffset[w + 1]) return k + 1;
        for (uint64_t j = first; j < k; ++j)
            if (g.atomic[j] != (k - first > 1 ? 1 : 0)) return j + 1;
    }
    return k == g.total_groups ? 0 : k + 1;
}

// ------------------------------------------------------------------ MatrixMarket coordinate text -> CSR
//
// load_matrix (src/utils/load.h:152-322): lines that start with '%' before the size line are
// skipped; the size line is "rows cols entries"; every further line that reads as "row col value"
// is an entry with 1-based indices, any other line is ignored; reading stops after the promised
// number of entries, and a file with fewer just has fewer (load.h:232-236).  Nothing in the
// banner is interpreted - a "symmetric" file is not mirrored, a "pattern" file (no values) yields
// no entries.  Entries are ordered by (row, column).  The reference orders them with qsort, which
// leaves the order of repeated (row, column) pairs open; here they keep their file order.
// Indices outside the matrix, which the reference stores unchecked, are refused.
int load_matrix_market(const char *path, int dtype, CsrHost *out) {
    if (!path || !out) return B200SPMM_ERR_INVALID_ARG;
    if (dtype != B200SPMM_F16 && dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    FILE *file = std::fopen(path, "r");
    if (!file) return B200SPMM_ERR_INVALID_ARG;
    char line[1024];
    bool have_size = false;
    while (std::fgets(line, sizeof(line), file)) {
        if (line[0] != '%') {
            have_size = true;
            break;
        }
    }
    unsigned rows = 0, cols = 0, declared = 0;
    if (!have_size || std::sscanf(line, "%u %u %u", &rows, &cols, &declared) != 3) {
        std::fclose(file);
        return B200SPMM_ERR_BAD_CSR;
    }
    CsrHost &m = *out;
    m = CsrHost();
    m.rows = rows;
    m.cols = cols;
    m.declared_nnz = declared;
    m.dtype = dtype;
    m.elt_size = dtype == B200SPMM_F16 ? 2 : 4;
    std::vector<uint32_t> r_idx, c_idx;
    std::vector<float> vals;
    bool out_of_range = false, file_open = true;
    try {
        while (r_idx.size() < declared && std::fgets(line, sizeof(line), file)) {
            unsigned r = 0, c = 0;
            float v = 0.f;
            if (std::sscanf(line, "%u %u %f", &r, &c, &v) != 3) continue;
            if (r < 1 || r > rows || c < 1 || c > cols) {
                out_of_range = true;
                break;
            }
            r_idx.push_back(r - 1);
            c_idx.push_back(c - 1);
            vals.push_back(v);
        }
        std::fclose(file);
        file_open = false;
        if (out_of_range) return B200SPMM_ERR_BAD_CSR;
        const uint64_t nnz = r_idx.size();
        std::vector<uint32_t> order(nnz);
        std::iota(order.begin(), order.end(), 0u);
        std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
            return r_idx[a] != r_idx[b] ? r_idx[a] < r_idx[b] : c_idx[a] < c_idx[b];
        });
        m.nnzs = nnz;
        m.row_ptr.assign((uint64_t)rows + 1, 0);
        m.col_idx.resize(nnz);
        m.values.resize(nnz * m.elt_size);
        for (uint64_t i = 0; i < nnz; ++i) {
            const uint32_t e = order[i];
            ++m.row_ptr[r_idx[e] + 1];
            m.col_idx[i] = c_idx[e];
            if (dtype == B200SPMM_F16) {
                const __half h = __float2half_rn(vals[e]);  // load.h:225
                std::memcpy(&m.values[i * 2], &h, 2);
            } else {
                std::memcpy(&m.values[i * 4], &vals[e], 4);
            }
        }
        for (uint64_t r = 0; r < rows; ++r) m.row_ptr[r + 1] += m.row_ptr[r];
    } catch (const std::bad_alloc &) {
        if (file_open) std::fclose(file);
        return B200SPMM_ERR_NO_MEMORY;
    }
    return B200SPMM_OK;
}

}  // namespace b200spmm
