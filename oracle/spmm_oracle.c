/*
 * CPU oracle for the condensed row-window SpMM path.  TEST INFRASTRUCTURE ONLY:
 * nothing that ships may call into this file; it is the checker for the CUDA path
 * and the timed CPU baseline of the benchmark.
 *
 * It restates, in plain C, the algorithms of the reference project
 * (Ritt2020/hopper_spmm):
 *
 *   - format conversion   src/utils/convert.h:146-225   (CSR2BTCFNOBITMAP)
 *   - tile-accumulate     src/tf32.cu:20-28, test/03.warp_specialized/utils.h:35-43
 *                         (verify_result: tiles outer, k inner, fp32 accumulator)
 *   - single-tile product src/test_fp16.cu:284-298      (test_result_cpu, fp16 widened
 *                         to fp32 before the multiply)
 *   - pass/fail rule      src/tf32.cu:38-71             (relative above 1e-6, else
 *                         absolute 1e-5)
 *   - dense comparer      src/utils/verify.h:18-42      (absolute threshold)
 *
 * Differences from the reference that are deliberate and documented:
 *   - ROW_WINDOW / COL_WINDOW are run-time parameters (the reference fixes 8x16 / 8x8
 *     in src/common.h:17-18,40-41); element offsets are 64-bit (the reference keeps
 *     them in uint32_t, src/utils/convert.h:191-192).
 *   - The reference has no CSR-level SpMM.  spmm_csr_* below is the same arithmetic
 *     (inputs widened to fp32, fp32 accumulate, sequential order) applied to CSR rows;
 *     spmm_btcf_* is the loop nest of verify_result applied to the converted format.
 *
 * Parity pin: the converter is checked bit-for-bit against the reference's own
 * CSR2BTCFNOBITMAP compiled from its sources (oracle/_ref, built by oracle/Makefile),
 * and the tile arithmetic against the closed-form answers of the reference's
 * single-tile tests (src/test_fp16.cu:407-415, test/02.tma_and_wgmma/tma_wgmma.cu:340-348).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__F16C__) && defined(__AVX__)
#include <immintrin.h>
#define ORACLE_HAVE_F16C 1
#endif

#define ORACLE_IDX_MAX 0xFFFFFFFFu /* src/common.h:47 */

/* ---------------------------------------------------------------- fp16 <-> fp32 */

/* IEEE binary16 -> binary32, exact (what __half2float does, src/test_fp16.cu:295). */
static inline float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else { /* subnormal: normalise */
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            out = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (what __float2half does, src/utils/load.h:226). */
static inline uint16_t float_to_half_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* below half of the smallest subnormal */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return (uint16_t)(sign | (base + q)); /* a mantissa carry bumps the exponent correctly */
}

void oracle_half_to_float(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = half_bits_to_float(src[i]);
}

void oracle_float_to_half(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = float_to_half_bits(src[i]);
}

/* tf32 view of an fp32 value.  mode 0: unchanged; 1: low 13 mantissa bits dropped
 * (what the tensor core sees when it is handed raw fp32 bits; the reference's
 * cvt.rna helper is a no-op, src/ptx/ptx_utils.h:32-36); 2: round to nearest, ties away. */
static inline float tf32_view(float f, int mode) {
    if (mode == 0) return f;
    uint32_t x;
    memcpy(&x, &f, 4);
    if (mode == 2 && (x & 0x7F800000u) != 0x7F800000u) x += 0x1000u;
    x &= 0xFFFFE000u;
    memcpy(&f, &x, 4);
    return f;
}

/* ---------------------------------------------------------------- format converter */

static int cmp_u32(const void *a, const void *b) {
    uint32_t x = *(const uint32_t *)a, y = *(const uint32_t *)b;
    return (x > y) - (x < y);
}

/* Sorted distinct columns of one row window into `scratch`; returns how many. */
static int64_t window_unique_cols(const uint32_t *col_idx, int64_t lo, int64_t hi, uint32_t *scratch) {
    int64_t n = hi - lo;
    memcpy(scratch, col_idx + lo, (size_t)n * sizeof(uint32_t));
    qsort(scratch, (size_t)n, sizeof(uint32_t), cmp_u32);
    int64_t u = 0;
    for (int64_t i = 0; i < n; ++i)
        if (i == 0 || scratch[i] != scratch[i - 1]) scratch[u++] = scratch[i];
    return u;
}

/* Pass 1 (convert.h:151-187 without the data): number of non-empty windows and tiles. */
int oracle_btcf_count(int64_t rows, const uint32_t *row_ptr, const uint32_t *col_idx, int row_window,
                      int col_window, int64_t *eff_row_windows, int64_t *total_tiles) {
    int64_t eff = 0, tiles = 0, cap = 0;
    uint32_t *scratch = NULL;
    for (int64_t first = 0; first < rows; first += row_window) {
        int64_t last = first + row_window < rows ? first + row_window : rows;
        int64_t lo = row_ptr[first], hi = row_ptr[last];
        if (hi == lo) continue; /* empty windows leave no trace (convert.h:162) */
        if (hi - lo > cap) {
            cap = (hi - lo) * 2;
            free(scratch);
            scratch = (uint32_t *)malloc((size_t)cap * sizeof(uint32_t));
            if (!scratch) return -1;
        }
        int64_t u = window_unique_cols(col_idx, lo, hi, scratch);
        tiles += (u + col_window - 1) / col_window;
        ++eff;
    }
    free(scratch);
    *eff_row_windows = eff;
    *total_tiles = tiles;
    return 0;
}

/*
 * Pass 2: fill caller-allocated arrays sized from oracle_btcf_count.
 *   rowOffset[eff+1], tcA2B[tiles*CW], data[tiles*RW*CW*elt_size bytes], rowIdx[eff].
 * col_major_tiles != 0 stores each tile column-major (SPARSE_A_TRANSPOSE, convert.h:207-209).
 */
int oracle_csr2btcf_nobitmap(int64_t rows, const uint32_t *row_ptr, const uint32_t *col_idx,
                             const void *values, int elt_size, int row_window, int col_window,
                             int col_major_tiles, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                             uint32_t *rowIdx) {
    const int64_t tile_elems = (int64_t)row_window * col_window;
    int64_t eff = 0, tiles = 0, cap = 0;
    uint32_t *uniq = NULL;
    rowOffset[0] = 0;
    for (int64_t first = 0; first < rows; first += row_window) {
        int64_t last = first + row_window < rows ? first + row_window : rows;
        int64_t lo = row_ptr[first], hi = row_ptr[last];
        if (hi == lo) continue;
        if (hi - lo > cap) {
            cap = (hi - lo) * 2;
            free(uniq);
            uniq = (uint32_t *)malloc((size_t)cap * sizeof(uint32_t));
            if (!uniq) return -1;
        }
        int64_t u = window_unique_cols(col_idx, lo, hi, uniq);
        int64_t wtiles = (u + col_window - 1) / col_window;

        /* column list, padded at the end with IDX_MAX (convert.h:178-184) */
        uint32_t *list = tcA2B + tiles * col_window;
        memcpy(list, uniq, (size_t)u * sizeof(uint32_t));
        for (int64_t i = u; i < wtiles * col_window; ++i) list[i] = ORACLE_IDX_MAX;

        rowOffset[eff + 1] = (uint32_t)(tiles + wtiles);
        rowIdx[eff] = (uint32_t)first;

        /* zero-filled tiles, then scatter every stored entry (convert.h:191-216) */
        char *wdata = (char *)data + tiles * tile_elems * elt_size;
        memset(wdata, 0, (size_t)(wtiles * tile_elems * elt_size));
        for (int64_t r = first; r < last; ++r) {
            for (int64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                uint32_t key = col_idx[p];
                const uint32_t *hit = (const uint32_t *)bsearch(&key, uniq, (size_t)u, sizeof(uint32_t), cmp_u32);
                int64_t slot = hit - uniq;
                int64_t t = slot / col_window, lc = slot % col_window, lr = r % row_window;
                int64_t in_tile = col_major_tiles ? lc * row_window + lr : lr * col_window + lc;
                memcpy(wdata + (t * tile_elems + in_tile) * elt_size, (const char *)values + p * elt_size,
                       (size_t)elt_size); /* a repeated (r,c) keeps the last value, as the reference does */
            }
        }
        tiles += wtiles;
        ++eff;
    }
    free(uniq);
    return 0;
}

/*
 * Bitmap-compressed format, restating CSR2BTCF (convert.h:22-139).  Caller-allocated arrays sized
 * from oracle_btcf_count: rowOffset[eff+1], nnzOffset[tiles+1], tcA2B[tiles*CW],
 * tcBit[tiles*words] with words = RW*CW/64, data[nnz*elt_size bytes], rowIdx[eff].
 * Per entry: nnzOffset[tile]++ (made a running sum with a leading zero at the end, :136-137),
 * bit (r % RW)*CW + (slot % CW) of the tile set (:88-96), value appended to the tile's list in
 * CSR order (:115), lists concatenated tile after tile (:127-130).
 * legacy_word_index != 0 repeats the reference's fp16 indexing, which addresses the bitmap word of
 * bit b of tile t as tcBit[t + b/64] (:98-102) although it reserves two words per tile (:62-66):
 * that is what the reference binary produces, kept here only to pin this restatement against it.
 * Otherwise word j of tile t is tcBit[t*words + j].
 */
int oracle_csr2btcf_bitmap(int64_t rows, const uint32_t *row_ptr, const uint32_t *col_idx, const void *values,
                           int elt_size, int row_window, int col_window, int legacy_word_index,
                           uint32_t *rowOffset, uint32_t *nnzOffset, uint32_t *tcA2B, uint64_t *tcBit,
                           void *data, uint32_t *rowIdx) {
    const int words = row_window * col_window / 64;
    int64_t eff = 0, tiles = 0, cap = 0, total_tiles = 0, placed = 0;
    uint32_t *uniq = NULL;
    int64_t *cursor = NULL, cursor_cap = 0;
    /* total tiles first: nnzOffset and tcBit are cleared up front like the reference's resize(…, 0) */
    {
        int64_t e = 0;
        if (oracle_btcf_count(rows, row_ptr, col_idx, row_window, col_window, &e, &total_tiles)) return -1;
    }
    memset(nnzOffset, 0, (size_t)(total_tiles + 1) * sizeof(uint32_t));
    memset(tcBit, 0, (size_t)(total_tiles * words) * sizeof(uint64_t));
    rowOffset[0] = 0;
    for (int64_t first = 0; first < rows; first += row_window) {
        int64_t last = first + row_window < rows ? first + row_window : rows;
        int64_t lo = row_ptr[first], hi = row_ptr[last];
        if (hi == lo) continue;
        if (hi - lo > cap) {
            cap = (hi - lo) * 2;
            free(uniq);
            uniq = (uint32_t *)malloc((size_t)cap * sizeof(uint32_t));
            if (!uniq) return -1;
        }
        int64_t u = window_unique_cols(col_idx, lo, hi, uniq);
        int64_t wtiles = (u + col_window - 1) / col_window;
        uint32_t *list = tcA2B + tiles * col_window;
        memcpy(list, uniq, (size_t)u * sizeof(uint32_t));
        for (int64_t i = u; i < wtiles * col_window; ++i) list[i] = ORACLE_IDX_MAX;
        rowOffset[eff + 1] = (uint32_t)(tiles + wtiles);
        rowIdx[eff] = (uint32_t)first;
        if (wtiles > cursor_cap) {
            cursor_cap = wtiles * 2;
            free(cursor);
            cursor = (int64_t *)malloc((size_t)cursor_cap * sizeof(int64_t));
            if (!cursor) return -1;
        }
        /* count per tile (kept in nnzOffset[tile+1] until the final running sum), set bits */
        for (int64_t r = first; r < last; ++r) {
            for (int64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                uint32_t key = col_idx[p];
                const uint32_t *hit = (const uint32_t *)bsearch(&key, uniq, (size_t)u, sizeof(uint32_t), cmp_u32);
                int64_t slot = hit - uniq, t = tiles + slot / col_window;
                int64_t bit = (r % row_window) * col_window + slot % col_window;
                nnzOffset[t + 1]++;
                if (legacy_word_index) {
                    if (t + bit / 64 < total_tiles * words) tcBit[t + bit / 64] |= 1ull << (bit % 64);
                } else {
                    tcBit[t * words + bit / 64] |= 1ull << (bit % 64);
                }
            }
        }
        /* values: tile after tile, inside a tile in CSR order */
        int64_t run = placed;
        for (int64_t t = 0; t < wtiles; ++t) {
            cursor[t] = run;
            run += nnzOffset[tiles + t + 1];
        }
        for (int64_t r = first; r < last; ++r) {
            for (int64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                uint32_t key = col_idx[p];
                const uint32_t *hit = (const uint32_t *)bsearch(&key, uniq, (size_t)u, sizeof(uint32_t), cmp_u32);
                int64_t t = (hit - uniq) / col_window;
                memcpy((char *)data + cursor[t]++ * elt_size, (const char *)values + p * elt_size, (size_t)elt_size);
            }
        }
        placed = run;
        tiles += wtiles;
        ++eff;
    }
    for (int64_t t = 0; t < total_tiles; ++t) nnzOffset[t + 1] += nnzOffset[t];
    free(uniq);
    free(cursor);
    return 0;
}

/*
 * Group split, restating BTCF2GBTCF (convert.h:232-276).  With groupOffset == NULL only counts
 * (total_groups, group_len).  group_len = max((uint32)mean tiles per window, 32) (:244-245); a
 * window of T tiles gets ceil(T/len) groups starting at rowOffset + ceil(T/groups)*j (:250-253),
 * each carrying the window's first row and atomic = (groups != 1) (:255-259); one closing offset
 * (:262).
 */
int oracle_btcf2gbtcf(const uint32_t *rowOffset, const uint32_t *rowIdx, int64_t eff, uint32_t *groupOffset,
                      uint32_t *group_rowIdx, uint8_t *atomic, int64_t *total_groups, uint32_t *group_len) {
    double sum = 0.0;
    for (int64_t i = 0; i < eff; ++i) sum += (double)(rowOffset[i + 1] - rowOffset[i]);
    uint32_t len = eff ? (uint32_t)(sum / (double)eff) : 0;
    if (len < 32) len = 32;
    int64_t g = 0;
    for (int64_t i = 0; i < eff; ++i) {
        uint32_t T = rowOffset[i + 1] - rowOffset[i];
        uint32_t n = (T + len - 1) / len;
        for (uint32_t j = 0; j < n; ++j, ++g) {
            if (!groupOffset) continue;
            groupOffset[g] = rowOffset[i] + (T + n - 1) / n * j;
            group_rowIdx[g] = rowIdx[i];
            atomic[g] = n == 1 ? 0 : 1;
        }
    }
    if (groupOffset) groupOffset[g] = eff ? rowOffset[eff] : 0;
    *total_groups = g;
    *group_len = len;
    return 0;
}

/* ---------------------------------------------------------------- SpMM, CSR form (O1) */

/* C[r,:] = sum_p A[p] * B[col[p],:], fp16 inputs widened to fp32, fp32 accumulate, CSR order. */
void oracle_spmm_csr_f16(int64_t rows, const uint32_t *row_ptr, const uint32_t *col_idx,
                         const uint16_t *values, const uint16_t *B, int64_t ldb, int64_t n, float *C,
                         int64_t ldc, int64_t row_begin, int64_t row_end, int n_threads) {
    (void)rows;
#ifdef _OPENMP
    if (n_threads < 1) n_threads = omp_get_max_threads();
#else
    (void)n_threads;
#endif
#pragma omp parallel for schedule(dynamic, 64) num_threads(n_threads)
    for (int64_t r = row_begin; r < row_end; ++r) {
        float *c = C + r * ldc;
        for (int64_t j = 0; j < n; ++j) c[j] = 0.0f;
        for (int64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
            float a = half_bits_to_float(values[p]);
            const uint16_t *b = B + (int64_t)col_idx[p] * ldb;
            int64_t j = 0;
#ifdef ORACLE_HAVE_F16C
            /* same widening and the same per-element multiply-then-add, eight lanes at a time */
            __m256 va = _mm256_set1_ps(a);
            for (; j + 8 <= n; j += 8) {
                __m256 vb = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(b + j)));
                __m256 vc = _mm256_loadu_ps(c + j);
                _mm256_storeu_ps(c + j, _mm256_add_ps(vc, _mm256_mul_ps(va, vb)));
            }
#endif
            for (; j < n; ++j) c[j] += a * half_bits_to_float(b[j]);
        }
    }
}

/* Same for fp32 inputs; tf32_mode selects how inputs are viewed (see tf32_view). */
void oracle_spmm_csr_f32(int64_t rows, const uint32_t *row_ptr, const uint32_t *col_idx,
                         const float *values, const float *B, int64_t ldb, int64_t n, float *C, int64_t ldc,
                         int64_t row_begin, int64_t row_end, int tf32_mode, int n_threads) {
    (void)rows;
#ifdef _OPENMP
    if (n_threads < 1) n_threads = omp_get_max_threads();
#else
    (void)n_threads;
#endif
#pragma omp parallel for schedule(dynamic, 64) num_threads(n_threads)
    for (int64_t r = row_begin; r < row_end; ++r) {
        float *c = C + r * ldc;
        for (int64_t j = 0; j < n; ++j) c[j] = 0.0f;
        for (int64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
            float a = tf32_view(values[p], tf32_mode);
            const float *b = B + (int64_t)col_idx[p] * ldb;
            if (tf32_mode == 0) {
                for (int64_t j = 0; j < n; ++j) c[j] += a * b[j];
            } else {
                for (int64_t j = 0; j < n; ++j) c[j] += a * tf32_view(b[j], tf32_mode);
            }
        }
    }
}

/* ---------------------------------------------------------------- SpMM, tile form (O2) */

/*
 * Loop nest of verify_result (tf32.cu:20-28) over the converted format: for every
 * effective window, tiles outer, then window row, feature, k inner.  Padded column slots
 * (IDX_MAX) are skipped: their tile entries are zero by construction.  C must hold
 * `rows` rows; rows of windows that do not exist in the format are zeroed.
 */
void oracle_spmm_btcf(int64_t rows, int64_t eff_row_windows, const uint32_t *rowOffset,
                      const uint32_t *tcA2B, const void *data, const uint32_t *rowIdx, int is_half,
                      int row_window, int col_window, const void *B, int64_t ldb, int64_t n, float *C,
                      int64_t ldc, int tf32_mode, int n_threads) {
#ifdef _OPENMP
    if (n_threads < 1) n_threads = omp_get_max_threads();
#else
    (void)n_threads;
#endif
    for (int64_t r = 0; r < rows; ++r) memset(C + r * ldc, 0, (size_t)n * sizeof(float));
    const int64_t tile_elems = (int64_t)row_window * col_window;
#pragma omp parallel for schedule(dynamic, 16) num_threads(n_threads)
    for (int64_t w = 0; w < eff_row_windows; ++w) {
        int64_t first = rowIdx[w];
        for (int64_t t = rowOffset[w]; t < rowOffset[w + 1]; ++t) {
            const uint32_t *cols = tcA2B + t * col_window;
            for (int lr = 0; lr < row_window; ++lr) {
                int64_t r = first + lr;
                if (r >= rows) break;
                float *c = C + r * ldc;
                for (int64_t j = 0; j < n; ++j) {
                    float acc = c[j];
                    for (int k = 0; k < col_window; ++k) {
                        if (cols[k] == ORACLE_IDX_MAX) continue;
                        int64_t e = t * tile_elems + (int64_t)lr * col_window + k;
                        float a, b;
                        if (is_half) {
                            a = half_bits_to_float(((const uint16_t *)data)[e]);
                            b = half_bits_to_float(((const uint16_t *)B)[(int64_t)cols[k] * ldb + j]);
                        } else {
                            a = tf32_view(((const float *)data)[e], tf32_mode);
                            b = tf32_view(((const float *)B)[(int64_t)cols[k] * ldb + j], tf32_mode);
                        }
                        acc += a * b;
                    }
                    c[j] = acc;
                }
            }
        }
    }
}

/* ---------------------------------------------------------------- tile-accumulate KAT math */

/*
 * verify_result's reference product: A is [tile_m][tile_k*tile_num], B is
 * [tile_n][tile_k*tile_num], both K-major; C[r][c] accumulates tile after tile.
 */
void oracle_tile_accumulate(const float *A, const float *B, float *C, int tile_m, int tile_n, int tile_k,
                            int tile_num) {
    for (int i = 0; i < tile_m * tile_n; ++i) C[i] = 0.0f;
    for (int t = 0; t < tile_num; ++t)
        for (int r = 0; r < tile_m; ++r)
            for (int c = 0; c < tile_n; ++c)
                for (int k = 0; k < tile_k; ++k)
                    C[r * tile_n + c] += A[(int64_t)r * tile_k * tile_num + k + t * tile_k] *
                                         B[(int64_t)c * tile_k * tile_num + k + t * tile_k];
}

/* glibc rand()/RAND_MAX stream used by the reference's pipeline test after srand(seed)
 * (test/03.warp_specialized/main.cu:235-241). */
void oracle_rand_fill(unsigned seed, float *dst, int64_t n) {
    srand(seed);
    for (int64_t i = 0; i < n; ++i) dst[i] = (float)rand() / (float)RAND_MAX;
}

/* ---------------------------------------------------------------- comparers */

/*
 * verify_result's rule (tf32.cu:38-71): relative error against |ref| when |ref| > 1e-6,
 * otherwise absolute error against 1e-5.  Returns the number of failing elements and
 * reports the largest relative and absolute errors seen.
 */
int64_t oracle_compare(const float *got, const float *ref, int64_t rows, int64_t n, int64_t ld_got,
                       int64_t ld_ref, double rel_tol, double *max_rel, double *max_abs) {
    int64_t bad = 0;
    double mr = 0.0, ma = 0.0;
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t j = 0; j < n; ++j) {
            double g = got[r * ld_got + j], f = ref[r * ld_ref + j];
            double err = fabs(g - f), af = fabs(f);
            if (!(err == err)) { ++bad; continue; } /* NaN never passes */
            if (err > ma) ma = err;
            if (af > 1e-6) {
                double rel = err / af;
                if (rel > mr) mr = rel;
                if (rel > rel_tol) ++bad;
            } else if (err > 1e-5) {
                ++bad;
            }
        }
    }
    if (max_rel) *max_rel = mr;
    if (max_abs) *max_abs = ma;
    return bad;
}

/* verify_dense_matrix's rule (verify.h:18-42): an element fails when |a-b| exceeds abs_tol
 * (the reference hard-codes 1). */
int64_t oracle_compare_abs(const float *a, const float *b, int64_t count, double abs_tol) {
    int64_t bad = 0;
    for (int64_t i = 0; i < count; ++i)
        if (!(fabs((double)a[i] - (double)b[i]) <= abs_tol)) ++bad;
    return bad;
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
