// C ABI of the bitmap-compressed format, the group-split format and the MatrixMarket loader.
#include <cstring>
#include <new>

#include "../../include/b200_spmm.h"
#include "handles.hpp"

using namespace b200spmm;

extern "C" {

int b200spmm_csr2btcf(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx,
                      const void *values, int dtype, int row_window, int col_window, int n_threads,
                      b200spmm_btcfb_t **out) {
    if (!out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    b200spmm_btcfb *h = new (std::nothrow) b200spmm_btcfb();
    if (!h) return B200SPMM_ERR_NO_MEMORY;
    int st = convert_csr_to_btcf_bitmap(rows, cols, nnz, row_ptr, col_idx, values, dtype, row_window, col_window,
                                        n_threads, &h->f);
    if (st != B200SPMM_OK) {
        delete h;
        return st;
    }
    *out = h;
    return B200SPMM_OK;
}

int b200spmm_btcfb_info(const b200spmm_btcfb_t *h, b200spmm_btcf_info_t *info, int *bitmap_words) {
    if (!h || !info) return B200SPMM_ERR_INVALID_ARG;
    const BtcfBitmap &f = h->f;
    info->rows = f.rows;
    info->cols = f.cols;
    info->nnzs = f.nnzs;
    info->total_row_windows = f.total_row_windows;
    info->eff_row_windows = f.eff_row_windows;
    info->total_tiles = f.total_tiles;
    info->row_window = f.row_window;
    info->col_window = f.col_window;
    info->dtype = f.dtype;
    info->elt_size = f.elt_size;
    if (bitmap_words) *bitmap_words = f.bitmap_words;
    return B200SPMM_OK;
}

const uint32_t *b200spmm_btcfb_rowOffset(const b200spmm_btcfb_t *h) { return h ? h->f.rowOffset.data() : nullptr; }
const uint32_t *b200spmm_btcfb_nnzOffset(const b200spmm_btcfb_t *h) { return h ? h->f.nnzOffset.data() : nullptr; }
const uint32_t *b200spmm_btcfb_tcA2B(const b200spmm_btcfb_t *h) { return h ? h->f.tcA2B.data() : nullptr; }
const uint64_t *b200spmm_btcfb_tcBit(const b200spmm_btcfb_t *h) { return h ? h->f.tcBit.data() : nullptr; }
const void *b200spmm_btcfb_data(const b200spmm_btcfb_t *h) { return h ? h->f.data.data() : nullptr; }
const uint32_t *b200spmm_btcfb_rowIdx(const b200spmm_btcfb_t *h) { return h ? h->f.rowIdx.data() : nullptr; }
void b200spmm_btcfb_destroy(b200spmm_btcfb_t *h) { delete h; }

int b200spmm_btcfb_expand(const b200spmm_btcfb_t *in, b200spmm_btcf_t **out) {
    if (!in || !out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    b200spmm_btcf *h = new (std::nothrow) b200spmm_btcf();
    if (!h) return B200SPMM_ERR_NO_MEMORY;
    int st = expand_bitmap(in->f, &h->f);
    if (st != B200SPMM_OK) {
        delete h;
        return st;
    }
    *out = h;
    return B200SPMM_OK;
}

int b200spmm_btcf2gbtcf(const uint32_t *rowOffset, const uint32_t *rowIdx, uint64_t eff_row_windows, b200spmm_gbtcf_t **out) {
    if (!out || !rowOffset || (eff_row_windows && !rowIdx)) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    b200spmm_gbtcf *h = new (std::nothrow) b200spmm_gbtcf();
    if (!h) return B200SPMM_ERR_NO_MEMORY;
    try {
        std::vector<uint32_t> ro(rowOffset, rowOffset + eff_row_windows + 1), ri(rowIdx, rowIdx + eff_row_windows);
        btcf_to_gbtcf(ro, ri, &h->g);
    } catch (const std::bad_alloc &) {
        delete h;
        return B200SPMM_ERR_NO_MEMORY;
    }
    *out = h;
    return B200SPMM_OK;
}

int b200spmm_gbtcf_info(const b200spmm_gbtcf_t *h, uint64_t *total_groups, uint32_t *group_len) {
    if (!h) return B200SPMM_ERR_INVALID_ARG;
    if (total_groups) *total_groups = h->g.total_groups;
    if (group_len) *group_len = h->g.group_len;
    return B200SPMM_OK;
}
const uint32_t *b200spmm_gbtcf_groupOffset(const b200spmm_gbtcf_t *h) { return h ? h->g.groupOffset.data() : nullptr; }
const uint32_t *b200spmm_gbtcf_rowIdx(const b200spmm_gbtcf_t *h) { return h ? h->g.rowIdx.data() : nullptr; }
const uint8_t *b200spmm_gbtcf_atomic(const b200spmm_gbtcf_t *h) { return h ? h->g.atomic.data() : nullptr; }
void b200spmm_gbtcf_destroy(b200spmm_gbtcf_t *h) { delete h; }

int b200spmm_gbtcf_validate(const uint32_t *rowOffset, const uint32_t *rowIdx, uint64_t eff_row_windows,
                            const uint32_t *groupOffset, const uint32_t *group_rowIdx, const uint8_t *atomic,
                            uint64_t total_groups, uint64_t *first_bad_group) {
    if (!rowOffset || !groupOffset || (eff_row_windows && !rowIdx) || (total_groups && (!group_rowIdx || !atomic)))
        return B200SPMM_ERR_INVALID_ARG;
    try {
        std::vector<uint32_t> ro(rowOffset, rowOffset + eff_row_windows + 1), ri(rowIdx, rowIdx + eff_row_windows);
        Gbtcf g;
        g.total_groups = total_groups;
        g.groupOffset.assign(groupOffset, groupOffset + total_groups + 1);
        g.rowIdx.assign(group_rowIdx, group_rowIdx + total_groups);
        g.atomic.assign(atomic, atomic + total_groups);
        const uint64_t bad = validate_gbtcf(ro, ri, g);
        if (first_bad_group) *first_bad_group = bad;
        return bad ? B200SPMM_ERR_BAD_CSR : B200SPMM_OK;
    } catch (const std::bad_alloc &) {
        return B200SPMM_ERR_NO_MEMORY;
    }
}

int b200spmm_load_matrix(const char *path, int dtype, b200spmm_csr_t **out) {
    if (!out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    b200spmm_csr *h = new (std::nothrow) b200spmm_csr();
    if (!h) return B200SPMM_ERR_NO_MEMORY;
    int st = load_matrix_market(path, dtype, &h->m);
    if (st != B200SPMM_OK) {
        delete h;
        return st;
    }
    *out = h;
    return B200SPMM_OK;
}

int b200spmm_csr_info(const b200spmm_csr_t *h, uint64_t *rows, uint64_t *cols, uint64_t *nnz, uint64_t *declared_nnz) {
    if (!h) return B200SPMM_ERR_INVALID_ARG;
    if (rows) *rows = h->m.rows;
    if (cols) *cols = h->m.cols;
    if (nnz) *nnz = h->m.nnzs;
    if (declared_nnz) *declared_nnz = h->m.declared_nnz;
    return B200SPMM_OK;
}
const uint32_t *b200spmm_csr_row_ptr(const b200spmm_csr_t *h) { return h ? h->m.row_ptr.data() : nullptr; }
const uint32_t *b200spmm_csr_col_idx(const b200spmm_csr_t *h) { return h ? h->m.col_idx.data() : nullptr; }
const void *b200spmm_csr_values(const b200spmm_csr_t *h) { return h ? h->m.values.data() : nullptr; }
void b200spmm_csr_destroy(b200spmm_csr_t *h) { delete h; }

}  // extern "C"
