/*
 * Harness around the reference project's OWN host-side converter.  TEST INFRASTRUCTURE ONLY.
 *
 * This file contains no reference code: it includes the reference's headers from the
 * place they are mounted at build time (see oracle/Makefile, REF=...) and exposes
 * CSR2BTCFNOBITMAP (src/utils/convert.h:146-225) through a flat C interface so the
 * restated oracle and the shipped converter can be compared with it bit for bit.
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

namespace {
BTCF_MTX_NO_BITMAP *g_last = nullptr;
}

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

}  // extern "C"
