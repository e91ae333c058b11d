/*
 * Harness around the reference project's OWN host-side converter.  TEST INFRASTRUCTURE ONLY.
 *
 * This file contains no reference code: it includes the reference's headers from the
 * place they are mounted at build time (see oracle/Makefile, REF=...) and exposes
 * CSR2BTCFNOBITMAP (src/utils/convert.h:146-225), CSR2BTCF (:22-139), BTCF2GBTCF (:232-276)
 * and load_matrix (src/utils/load.h:152-322) through a flat C interface so the restated oracle
 * and the shipped code can be compared with them bit for bit.
 *
 * The reference fixes its window shape at compile time (src/common.h:14-42): 8x16 with
 * -DUSE_FP16, 8x8 with -DUSE_TF32.  One shared object is built per flavour.
 * The reference keeps running element offsets in 32 bits (convert.h:191-192), so this
 * harness is only meaningful while tiles*ROW_WINDOW*COL_WINDOW < 2^32.
 */
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "utils/utils.h"
#include "utils/class.h"
#include "utils/convert.h"
#include "utils/load.h"

namespace {
BTCF_MTX_NO_BITMAP *g_last = nullptr;
}

namespace {
BTCF_MTX *g_bitmap = nullptr;
GBTCF_MTX *g_groups = nullptr;
CSR_MTX g_loaded = {0, 0, 0, nullptr, nullptr, nullptr};

template <class Fn>
void quietly(Fn fn) {  /* the reference prints progress lines */
    FILE *saved = stdout;
    FILE *sink = fopen("/dev/null", "w");
    if (sink) stdout = sink;
    fn();
    if (sink) { fflush(sink); stdout = saved; fclose(sink); }
}
}  // namespace


extern "C" {

int ref_row_window() { return ROW_WINDOW; }
int ref_col_window() { return COL_WINDOW; }
int ref_elt_size() { return (int)sizeof(MAT_VAL_TYPE); }

/* Runs the reference converter; keeps the result until the next call or ref_release(). */
int ref_convert(uint32_t rows, uint32_t cols, uint32_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx,
                const void *values, uint64_t *sizes /* eff, tiles, total_windows, len_tcA2B, len_data */) {
    delete g_last;
    g_last = new BTCF_MTX_NO_BITMAP();
    CSR_MTX csr;
    csr.rows = rows;
    csr.cols = cols;
    csr.nnzs = nnz;
    csr.row_ptr = const_cast<uint32_t *>(row_ptr);
    csr.col_idx = const_cast<uint32_t *>(col_idx);
    csr.values = reinterpret_cast<MAT_VAL_TYPE *>(const_cast<void *>(values));
    /* the reference prints progress lines; keep test output clean */
    FILE *saved = stdout;
    FILE *sink = fopen("/dev/null", "w");
    if (sink) stdout = sink;
    CSR2BTCFNOBITMAP(csr, *g_last);
    if (sink) { fflush(sink); stdout = saved; fclose(sink); }
    sizes[0] = g_last->eff_row_windows;
    sizes[1] = g_last->total_tiles;
    sizes[2] = g_last->total_row_windows;
    sizes[3] = g_last->tcA2B.size();
    sizes[4] = g_last->data.size();
    return 0;
}

int ref_fetch(uint32_t *rowOffset, uint32_t *tcA2B, void *data, uint32_t *rowIdx) {
    if (!g_last) return -1;
    memcpy(rowOffset, g_last->rowOffset.data(), g_last->rowOffset.size() * sizeof(uint32_t));
    memcpy(tcA2B, g_last->tcA2B.data(), g_last->tcA2B.size() * sizeof(uint32_t));
    memcpy(data, g_last->data.data(), g_last->data.size() * sizeof(MAT_VAL_TYPE));
    memcpy(rowIdx, g_last->rowIdx.data(), g_last->rowIdx.size() * sizeof(uint32_t));
    return 0;
}

void ref_release() {
    delete g_last;
    g_last = nullptr;
}

/* ---- the bitmap-compressed format (CSR2BTCF, convert.h:22-139) and its group split (BTCF2GBTCF, :232-276) */

int ref_map_word_size() { return (int)sizeof(MAT_MAP_TYPE); }

int ref_convert_bitmap(uint32_t rows, uint32_t cols, uint32_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx,
                       const void *values, uint64_t *sizes /* eff, len_nnzOffset, len_tcA2B, len_tcBit, len_data */) {
    delete g_bitmap;
    g_bitmap = new BTCF_MTX();
    CSR_MTX csr;
    csr.rows = rows;
    csr.cols = cols;
    csr.nnzs = nnz;
    csr.row_ptr = const_cast<uint32_t *>(row_ptr);
    csr.col_idx = const_cast<uint32_t *>(col_idx);
    csr.values = reinterpret_cast<MAT_VAL_TYPE *>(const_cast<void *>(values));
    quietly([&] { CSR2BTCF(csr, *g_bitmap); });
    sizes[0] = g_bitmap->eff_row_windows;
    sizes[1] = g_bitmap->nnzOffset.size();
    sizes[2] = g_bitmap->tcA2B.size();
    sizes[3] = g_bitmap->tcBit.size();
    sizes[4] = g_bitmap->data.size();
    return 0;
}

int ref_fetch_bitmap(uint32_t *rowOffset, uint32_t *nnzOffset, uint32_t *tcA2B, void *tcBit, void *data, uint32_t *rowIdx) {
    if (!g_bitmap) return -1;
    memcpy(rowOffset, g_bitmap->rowOffset.data(), g_bitmap->rowOffset.size() * sizeof(uint32_t));
    memcpy(nnzOffset, g_bitmap->nnzOffset.data(), g_bitmap->nnzOffset.size() * sizeof(uint32_t));
    memcpy(tcA2B, g_bitmap->tcA2B.data(), g_bitmap->tcA2B.size() * sizeof(uint32_t));
    memcpy(tcBit, g_bitmap->tcBit.data(), g_bitmap->tcBit.size() * sizeof(MAT_MAP_TYPE));
    memcpy(data, g_bitmap->data.data(), g_bitmap->data.size() * sizeof(MAT_VAL_TYPE));
    memcpy(rowIdx, g_bitmap->rowIdx.data(), g_bitmap->rowIdx.size() * sizeof(uint32_t));
    return 0;
}

/* Group split of the matrix last given to ref_convert_bitmap. */
int ref_group(uint64_t *total_groups) {
    if (!g_bitmap) return -1;
    delete g_groups;
    g_groups = new GBTCF_MTX();
    quietly([&] { BTCF2GBTCF(*g_bitmap, *g_groups); });
    *total_groups = g_groups->total_groups;
    return 0;
}

int ref_fetch_groups(uint32_t *groupOffset, uint32_t *rowIdx, uint8_t *atomic) {
    if (!g_groups) return -1;
    memcpy(groupOffset, g_groups->groupOffset.data(), g_groups->groupOffset.size() * sizeof(uint32_t));
    memcpy(rowIdx, g_groups->rowIdx.data(), g_groups->rowIdx.size() * sizeof(uint32_t));
    memcpy(atomic, g_groups->atomic.data(), g_groups->atomic.size() * sizeof(uint8_t));
    return 0;
}

/* ---- the file loader (load_matrix, load.h:152-322) */

int ref_load(const char *path, uint32_t *dims /* rows, cols, nnz */) {
    quietly([&] { g_loaded = load_matrix(path, 0); });
    dims[0] = g_loaded.rows;
    dims[1] = g_loaded.cols;
    dims[2] = g_loaded.nnzs;
    return g_loaded.row_ptr ? 0 : -1;
}

int ref_fetch_loaded(uint32_t *row_ptr, uint32_t *col_idx, void *values) {
    if (!g_loaded.row_ptr) return -1;
    memcpy(row_ptr, g_loaded.row_ptr, ((size_t)g_loaded.rows + 1) * sizeof(uint32_t));
    memcpy(col_idx, g_loaded.col_idx, (size_t)g_loaded.nnzs * sizeof(uint32_t));
    memcpy(values, g_loaded.values, (size_t)g_loaded.nnzs * sizeof(MAT_VAL_TYPE));
    free_csr_matrix(&g_loaded);
    g_loaded.row_ptr = nullptr;
    return 0;
}

}  // extern "C"
