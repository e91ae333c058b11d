// CSR -> condensed row-window tiles, multi-threaded.  Same output, bit for bit, as the
// reference's single-threaded CSR2BTCFNOBITMAP (src/utils/convert.h:146-225) at the same
// window shape; row windows are independent, so each is converted by one thread.
#include "format.hpp"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <thread>

#include "../../include/b200_spmm.h"

namespace b200spmm {

namespace {

template <class Fn>
void parallel_chunks(uint64_t n_items, uint64_t chunk, int n_threads, Fn fn) {
    if (n_threads <= 0) n_threads = (int)std::thread::hardware_concurrency();
    if (n_threads <= 0) n_threads = 1;
    uint64_t n_chunks = (n_items + chunk - 1) / chunk;
    if ((uint64_t)n_threads > n_chunks) n_threads = (int)std::max<uint64_t>(1, n_chunks);
    std::atomic<uint64_t> next{0};
    auto worker = [&]() {
        for (;;) {
            uint64_t c = next.fetch_add(1);
            if (c >= n_chunks) break;
            fn(c * chunk, std::min(n_items, (c + 1) * chunk));
        }
    };
    if (n_threads == 1) {
        worker();
        return;
    }
    std::vector<std::thread> pool;
    pool.reserve(n_threads);
    for (int t = 0; t < n_threads; ++t) pool.emplace_back(worker);
    for (auto &t : pool) t.join();
}

// Sorted distinct columns of rows [first, last).
void window_columns(const uint32_t *row_ptr, const uint32_t *col_idx, uint64_t first, uint64_t last,
                    std::vector<uint32_t> *cols) {
    cols->assign(col_idx + row_ptr[first], col_idx + row_ptr[last]);
    std::sort(cols->begin(), cols->end());
    cols->erase(std::unique(cols->begin(), cols->end()), cols->end());
}

}  // namespace

int validate_csr(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr, const uint32_t *col_idx) {
    if (!row_ptr || (nnz && !col_idx)) return B200SPMM_ERR_INVALID_ARG;
    if (rows >= 0xFFFFFFFFull || cols > 0xFFFFFFFFull || nnz > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;
    if (row_ptr[0] != 0 || row_ptr[rows] != nnz) return B200SPMM_ERR_BAD_CSR;
    std::atomic<int> bad{0};
    parallel_chunks(rows, 1 << 16, 0, [&](uint64_t lo, uint64_t hi) {
        for (uint64_t r = lo; r < hi; ++r) {
            if (row_ptr[r + 1] < row_ptr[r] || row_ptr[r + 1] > nnz) {
                bad = 1;
                return;
            }
            for (uint64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p)
                if (col_idx[p] >= cols) {
                    bad = 1;
                    return;
                }
        }
    });
    return bad ? B200SPMM_ERR_BAD_CSR : B200SPMM_OK;
}

int convert_csr_to_btcf(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr,
                        const uint32_t *col_idx, const void *values, int dtype, int row_window, int col_window,
                        int n_threads, Btcf *out) {
    if (!out || (nnz && !values)) return B200SPMM_ERR_INVALID_ARG;
    if (dtype != B200SPMM_F16 && dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    if (row_window != 8 && row_window != 16) return B200SPMM_ERR_INVALID_ARG;
    if (col_window == 0) col_window = dtype == B200SPMM_F16 ? 16 : 8;  // src/common.h:18,41
    if (col_window != 4 && col_window != 8 && col_window != 16) return B200SPMM_ERR_INVALID_ARG;
    int st = validate_csr(rows, cols, nnz, row_ptr, col_idx);
    if (st != B200SPMM_OK) return st;

    const uint64_t RW = (uint64_t)row_window, CW = (uint64_t)col_window;
    const int esz = dtype == B200SPMM_F16 ? 2 : 4;
    const uint64_t n_windows = (rows + RW - 1) / RW;

    // Pass 1: tiles per window (0 marks an empty window, which the format omits, convert.h:162).
    std::vector<uint32_t> window_tiles(n_windows);
    parallel_chunks(n_windows, 256, n_threads, [&](uint64_t lo, uint64_t hi) {
        std::vector<uint32_t> cols_w;
        for (uint64_t w = lo; w < hi; ++w) {
            uint64_t first = w * RW, last = std::min(rows, first + RW);
            if (row_ptr[first] == row_ptr[last]) {
                window_tiles[w] = 0;
                continue;
            }
            window_columns(row_ptr, col_idx, first, last, &cols_w);
            window_tiles[w] = (uint32_t)((cols_w.size() + CW - 1) / CW);
        }
    });

    // Running sums over the non-empty windows.
    std::vector<uint64_t> tile_base(n_windows + 1), eff_base(n_windows + 1);
    uint64_t tiles = 0, eff = 0;
    for (uint64_t w = 0; w < n_windows; ++w) {
        tile_base[w] = tiles;
        eff_base[w] = eff;
        tiles += window_tiles[w];
        eff += window_tiles[w] ? 1 : 0;
    }
    tile_base[n_windows] = tiles;
    eff_base[n_windows] = eff;
    if (tiles > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;  // rowOffset is 32-bit (src/common.h:11)

    Btcf &f = *out;
    f = Btcf();
    f.rows = rows;
    f.cols = cols;
    f.nnzs = nnz;
    f.row_window = row_window;
    f.col_window = col_window;
    f.dtype = dtype;
    f.elt_size = esz;
    f.total_row_windows = n_windows;
    f.eff_row_windows = eff;
    f.total_tiles = tiles;
    try {
        f.rowOffset.assign(eff + 1, 0);
        f.rowIdx.assign(eff, 0);
        f.tcA2B.assign(tiles * CW, kIdxMax);
        f.data.assign(tiles * RW * CW * esz, 0);
    } catch (const std::bad_alloc &) {
        return B200SPMM_ERR_NO_MEMORY;
    }

    // Pass 2: column lists and tile values.
    const uint8_t *vals = static_cast<const uint8_t *>(values);
    parallel_chunks(n_windows, 256, n_threads, [&](uint64_t lo, uint64_t hi) {
        std::vector<uint32_t> cols_w;
        for (uint64_t w = lo; w < hi; ++w) {
            if (!window_tiles[w]) continue;
            uint64_t first = w * RW, last = std::min(rows, first + RW);
            window_columns(row_ptr, col_idx, first, last, &cols_w);
            uint64_t e = eff_base[w], t0 = tile_base[w];
            f.rowOffset[e + 1] = (uint32_t)(t0 + window_tiles[w]);
            f.rowIdx[e] = (uint32_t)first;
            std::memcpy(&f.tcA2B[t0 * CW], cols_w.data(), cols_w.size() * sizeof(uint32_t));
            uint8_t *wdata = f.data.data() + t0 * RW * CW * esz;
            for (uint64_t r = first; r < last; ++r) {
                const uint64_t lr = r % RW;
                for (uint64_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
                    uint64_t slot = std::lower_bound(cols_w.begin(), cols_w.end(), col_idx[p]) - cols_w.begin();
                    uint64_t off = (slot / CW) * RW * CW + lr * CW + slot % CW;  // row-major tile
                    std::memcpy(wdata + off * esz, vals + p * esz, esz);  // repeated (r,c): last one stays
                }
            }
        }
    });
    return B200SPMM_OK;
}

int rewindow_btcf(uint64_t rows, uint64_t cols, uint64_t nnz, int dtype, int rw_in, int col_window,
                  uint64_t eff_row_windows, const uint32_t *in_rowOffset, const uint32_t *in_tcA2B,
                  const void *in_data, const uint32_t *in_rowIdx, int rw_out, int n_threads, Btcf *out) {
    if (!out || !in_rowOffset) return B200SPMM_ERR_INVALID_ARG;
    if (dtype != B200SPMM_F16 && dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    if (rw_in < 1 || rw_out < rw_in || rw_out % rw_in) return B200SPMM_ERR_INVALID_ARG;
    if (rw_out != 8 && rw_out != 16 && rw_out != 32 && rw_out != 64 && rw_out != 128) return B200SPMM_ERR_INVALID_ARG;
    if (col_window != 4 && col_window != 8 && col_window != 16) return B200SPMM_ERR_INVALID_ARG;
    if (rows >= 0xFFFFFFFFull || cols > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;
    const uint64_t eff_in = eff_row_windows, RWI = (uint64_t)rw_in, RWO = (uint64_t)rw_out, CW = (uint64_t)col_window;
    const uint64_t tiles_in = in_rowOffset[eff_in];
    if (in_rowOffset[0] != 0 || (eff_in && (!in_rowIdx || !in_tcA2B || !in_data))) return B200SPMM_ERR_INVALID_ARG;
    const int esz = dtype == B200SPMM_F16 ? 2 : 4;

    // Input windows are listed by ascending first row; a run of them that falls into one output
    // window is a group.  group_first[g] = first input window of group g.
    std::vector<uint64_t> group_first;
    for (uint64_t i = 0; i < eff_in; ++i) {
        const uint64_t r = in_rowIdx[i];
        if (r >= rows || r % RWI || in_rowOffset[i + 1] <= in_rowOffset[i] || in_rowOffset[i + 1] > tiles_in)
            return B200SPMM_ERR_INVALID_ARG;
        if (i && r <= in_rowIdx[i - 1]) return B200SPMM_ERR_INVALID_ARG;
        if (i == 0 || r / RWO != in_rowIdx[i - 1] / RWO) group_first.push_back(i);
    }
    const uint64_t eff = group_first.size();
    group_first.push_back(eff_in);

    // Sorted union of a group's column lists (each list ascending, padded with kIdxMax at its end).
    std::atomic<int> bad{0};
    auto group_columns = [&](uint64_t g, std::vector<uint32_t> *u) {
        u->clear();
        for (uint64_t i = group_first[g]; i < group_first[g + 1]; ++i) {
            const uint32_t *lo = in_tcA2B + (uint64_t)in_rowOffset[i] * CW, *hi = in_tcA2B + (uint64_t)in_rowOffset[i + 1] * CW;
            const uint32_t *end = hi;
            while (end > lo && end[-1] == kIdxMax) --end;
            if ((uint64_t)(hi - end) >= CW || end == lo) bad = 1;  // padding fills the last tile only
            for (const uint32_t *p = lo; p < end; ++p)
                if (*p >= cols || (p > lo && *p <= p[-1])) bad = 1;
            const size_t mid = u->size();
            u->insert(u->end(), lo, end);
            std::inplace_merge(u->begin(), u->begin() + mid, u->end());
        }
        u->erase(std::unique(u->begin(), u->end()), u->end());
    };

    std::vector<uint32_t> group_tiles(eff);
    parallel_chunks(eff, 256, n_threads, [&](uint64_t lo, uint64_t hi) {
        std::vector<uint32_t> u;
        for (uint64_t g = lo; g < hi; ++g) {
            group_columns(g, &u);
            group_tiles[g] = (uint32_t)((u.size() + CW - 1) / CW);
        }
    });
    if (bad) return B200SPMM_ERR_INVALID_ARG;
    uint64_t tiles = 0;
    for (uint64_t g = 0; g < eff; ++g) tiles += group_tiles[g];
    if (tiles > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;

    Btcf &f = *out;
    f = Btcf();
    f.rows = rows;
    f.cols = cols;
    f.nnzs = nnz;
    f.row_window = rw_out;
    f.col_window = col_window;
    f.dtype = dtype;
    f.elt_size = esz;
    f.total_row_windows = (rows + RWO - 1) / RWO;
    f.eff_row_windows = eff;
    f.total_tiles = tiles;
    try {
        f.rowOffset.assign(eff + 1, 0);
        f.rowIdx.assign(eff, 0);
        f.tcA2B.assign(tiles * CW, kIdxMax);
        f.data.assign(tiles * RWO * CW * esz, 0);
    } catch (const std::bad_alloc &) {
        return B200SPMM_ERR_NO_MEMORY;
    }
    for (uint64_t g = 0; g < eff; ++g) {
        f.rowOffset[g + 1] = f.rowOffset[g] + group_tiles[g];
        f.rowIdx[g] = (uint32_t)(in_rowIdx[group_first[g]] / RWO * RWO);
    }
    const uint8_t *src = static_cast<const uint8_t *>(in_data);
    parallel_chunks(eff, 256, n_threads, [&](uint64_t lo, uint64_t hi) {
        std::vector<uint32_t> u;
        for (uint64_t g = lo; g < hi; ++g) {
            group_columns(g, &u);
            const uint64_t tile0 = f.rowOffset[g];
            std::copy(u.begin(), u.end(), f.tcA2B.begin() + tile0 * CW);
            for (uint64_t i = group_first[g]; i < group_first[g + 1]; ++i) {
                const uint64_t row_shift = in_rowIdx[i] - f.rowIdx[g];  // rows of this input window inside the group
                size_t s = 0;  // position in u; the input list is ascending, so s only moves forward
                for (uint64_t t = in_rowOffset[i]; t < in_rowOffset[i + 1]; ++t)
                    for (uint64_t lc = 0; lc < CW; ++lc) {
                        const uint32_t c = in_tcA2B[t * CW + lc];
                        if (c == kIdxMax) break;
                        while (u[s] != c) ++s;
                        const uint64_t ot = tile0 + s / CW, olc = s % CW;
                        for (uint64_t lr = 0; lr < RWI; ++lr)
                            std::memcpy(&f.data[((ot * RWO + row_shift + lr) * CW + olc) * esz],
                                        src + ((t * RWI + lr) * CW + lc) * esz, esz);
                    }
            }
        }
    });
    return B200SPMM_OK;
}

int shard_rows(uint64_t rows, const uint32_t *row_ptr, int row_window, int parts, uint64_t row_charge,
               uint64_t *row_begin) {
    if (!row_ptr || !row_begin || parts < 1 || row_window < 1) return B200SPMM_ERR_INVALID_ARG;
    const uint64_t RW = (uint64_t)row_window;
    const uint64_t n_windows = (rows + RW - 1) / RW;
    // cost of rows [0, r): their entries plus a fixed charge per row (0 = balance on nnz alone)
    auto cost = [&](uint64_t r) { return (uint64_t)row_ptr[r] + row_charge * r; };
    const uint64_t total = cost(rows);
    row_begin[0] = 0;
    uint64_t w = 0;
    for (int p = 1; p < parts; ++p) {
        // first window whose starting cost reaches p/parts of the total
        const uint64_t target = (total * (uint64_t)p + parts - 1) / parts;
        uint64_t lo = w, hi = n_windows;
        while (lo < hi) {
            uint64_t mid = (lo + hi) / 2;
            if (cost(std::min(rows, mid * RW)) < target) lo = mid + 1; else hi = mid;
        }
        w = lo;
        row_begin[p] = std::min(rows, w * RW);
    }
    row_begin[parts] = rows;
    return B200SPMM_OK;
}

void build_cta_schedule(const uint32_t *rowOffset, uint64_t eff, int n_ctas, std::vector<uint32_t> *cta_window) {
    cta_window->assign((size_t)n_ctas + 1, (uint32_t)eff);
    (*cta_window)[0] = 0;
    // Cost of windows [0, w): their tiles plus a fixed charge per window.
    auto cost = [&](uint64_t w) { return (uint64_t)rowOffset[w] + kWindowCharge * w; };
    const uint64_t total = eff ? cost(eff) : 0;
    uint64_t w = 0;
    for (int c = 1; c < n_ctas; ++c) {
        const uint64_t target = (total * (uint64_t)c) / (uint64_t)n_ctas;
        uint64_t lo = w, hi = eff;
        while (lo < hi) {
            uint64_t mid = (lo + hi) / 2;
            if (cost(mid) < target) lo = mid + 1; else hi = mid;
        }
        w = lo;
        (*cta_window)[c] = (uint32_t)w;
    }
    (*cta_window)[n_ctas] = (uint32_t)eff;
}

void transpose_tiles(Btcf *f) {
    const size_t rw = (size_t)f->row_window, cw = (size_t)f->col_window, esz = (size_t)f->elt_size;
    const size_t tile_bytes = rw * cw * esz;
    // rows x row_len elements in, row_len x rows out: row-major (rw x cw) <-> column-major (cw x rw)
    const size_t in_rows = f->col_major_tiles ? cw : rw, in_len = f->col_major_tiles ? rw : cw;
    std::vector<uint8_t> tmp(tile_bytes);
    for (uint64_t t = 0; t < f->total_tiles; ++t) {
        uint8_t *tile = f->data.data() + t * tile_bytes;
        std::memcpy(tmp.data(), tile, tile_bytes);
        for (size_t r = 0; r < in_rows; ++r)
            for (size_t c = 0; c < in_len; ++c) std::memcpy(tile + (c * in_rows + r) * esz, tmp.data() + (r * in_len + c) * esz, esz);
    }
    f->col_major_tiles = !f->col_major_tiles;
}

void build_tile_schedule(const uint32_t *rowOffset, uint64_t eff, int n_ctas, bool allow_split, TileSchedule *out) {
    TileSchedule &sc = *out;
    const uint64_t tiles = eff ? rowOffset[eff] : 0;
    sc.tile.assign((size_t)n_ctas + 1, (uint32_t)tiles);
    sc.wfirst.assign((size_t)n_ctas, 0);
    sc.wlast.assign((size_t)n_ctas, 0);
    sc.splits.clear();
    sc.piece_slots.clear();
    sc.head_slot.assign((size_t)n_ctas, kNoSlot);
    sc.tail_slot.assign((size_t)n_ctas, kNoSlot);
    sc.n_slots = 0;
    sc.tile[0] = 0;
    if (!eff) return;
    auto cost_start = [&](uint64_t w) { return (uint64_t)rowOffset[w] + kWindowCharge * w; };  // cost before window w
    const uint64_t total = cost_start(eff);
    const uint64_t tol = std::max<uint64_t>(32, tiles / (uint64_t)n_ctas / 16);
    uint64_t prev = 0;
    for (int c = 1; c < n_ctas; ++c) {
        const uint64_t target = total * (uint64_t)c / (uint64_t)n_ctas;
        // last window whose starting cost does not exceed the target
        uint64_t lo = 0, hi = eff;
        while (hi - lo > 1) {
            const uint64_t mid = (lo + hi) / 2;
            if (cost_start(mid) <= target) lo = mid; else hi = mid;
        }
        const uint64_t w = lo, w_tiles = (uint64_t)rowOffset[w + 1] - rowOffset[w];
        uint64_t inside = target - cost_start(w);
        inside = inside > kWindowCharge ? inside - kWindowCharge : 0;  // the window's fixed charge comes first
        inside = std::min(inside, w_tiles);
        if (!allow_split) inside = inside * 2 < w_tiles ? 0 : w_tiles;  // nearest window boundary
        else if (inside <= tol) inside = 0;
        else if (w_tiles - inside <= tol) inside = w_tiles;
        uint64_t cut = (uint64_t)rowOffset[w] + inside;
        cut = std::max(cut, prev);
        sc.tile[c] = (uint32_t)cut;
        prev = cut;
    }
    auto window_of_tile = [&](uint64_t t) {  // window holding tile t < tiles
        return (uint32_t)(std::upper_bound(rowOffset, rowOffset + eff + 1, (uint32_t)t) - rowOffset - 1);
    };
    for (int c = 0; c < n_ctas; ++c) {
        if (sc.tile[c + 1] > sc.tile[c]) {
            sc.wfirst[c] = window_of_tile(sc.tile[c]);
            sc.wlast[c] = window_of_tile(sc.tile[c + 1] - 1);
        } else {
            sc.wfirst[c] = sc.wlast[c] = c ? sc.wlast[c - 1] : 0;
        }
    }
    // split windows: a chunk whose last window is cut at its end opens one; following chunks that
    // begin inside the same window add their piece
    for (int c = 0; c < n_ctas; ++c) {
        if (sc.tile[c + 1] == sc.tile[c]) continue;
        const uint32_t w = sc.wlast[c];
        if (rowOffset[w + 1] <= sc.tile[c + 1]) continue;          // window ends inside this chunk
        if (rowOffset[w] < sc.tile[c]) continue;                     // not the first piece: it began in an earlier chunk
        TileSchedule::Split sp{w, (uint32_t)sc.piece_slots.size(), 0};
        sc.tail_slot[c] = sc.n_slots++;
        sc.piece_slots.push_back(sc.tail_slot[c]);
        for (int d = c + 1; d < n_ctas; ++d) {
            if (sc.tile[d + 1] == sc.tile[d]) continue;
            if (sc.wfirst[d] != w || rowOffset[w] >= sc.tile[d]) break;
            sc.head_slot[d] = sc.n_slots++;
            sc.piece_slots.push_back(sc.head_slot[d]);
            if (rowOffset[w + 1] <= sc.tile[d + 1]) break;          // the window's last piece
        }
        sp.piece_end = (uint32_t)sc.piece_slots.size();
        sc.splits.push_back(sp);
    }
}

void build_row_bands(const TileSchedule &sc, const uint32_t *rowIdx, uint64_t rows, uint32_t want, RowBands *out) {
    RowBands &b = *out;
    const uint32_t n_chunks = (uint32_t)sc.wfirst.size();
    b.chunk.assign(1, 0);
    for (uint32_t k = 1; k < want; ++k) {
        uint32_t c = (uint32_t)((uint64_t)n_chunks * k / want);
        // a band starts with a chunk that holds tiles and begins its first window
        while (c < n_chunks && (sc.head_slot[c] != kNoSlot || sc.tile[c + 1] == sc.tile[c])) ++c;
        if (c < n_chunks && c > b.chunk.back()) b.chunk.push_back(c);
    }
    b.chunk.push_back(n_chunks);
    b.row.clear();
    b.split.clear();
    uint32_t first_split = 0;  // the splits are ordered by window
    for (size_t k = 0; k + 1 < b.chunk.size(); ++k) {
        const uint32_t c = b.chunk[k];
        b.row.push_back(k == 0 ? 0 : rowIdx[sc.wfirst[c]]);
        while (k != 0 && first_split < sc.splits.size() && sc.splits[first_split].window < sc.wfirst[c]) ++first_split;
        b.split.push_back(first_split);
    }
    b.row.push_back(rows);
    b.split.push_back((uint32_t)sc.splits.size());
}

uint64_t exchange_even_part(const uint64_t *cut, int n) {
    const uint64_t total = cut[n];
    bool equal = true;
    for (int d = 0; d < n; ++d) equal = equal && (cut[d + 1] - cut[d] == cut[1] - cut[0]);
    if (equal) return cut[1] - cut[0];
    const uint64_t part = total / (uint64_t)n / 512u * 512u;
    if (!part) return 0;
    // does the two-step exchange save the busiest device at least 15 % of its sends?
    uint64_t longest = 0, outside = 0;
    for (int d = 0; d < n; ++d) {
        const uint64_t len = cut[d + 1] - cut[d];
        const uint64_t lo = std::max(cut[d], part * (uint64_t)d), hi = std::min(cut[d + 1], part * (uint64_t)(d + 1));
        longest = std::max(longest, len);
        outside = std::max(outside, len - (hi > lo ? hi - lo : 0));
    }
    if ((double)(outside + part * (uint64_t)(n - 1)) * 1.15 >= (double)longest * (double)(n - 1)) return 0;
    return part;
}

void exchange_pieces(const uint64_t *cut, int n, uint64_t part, int d, int step, int *to_out, int *from_out, uint64_t out[8]) {
    const int to = (d + step) % n, from = (d - step + n) % n;  // a different peer for every device at every step
    const uint64_t whole = part * (uint64_t)n;                 // bytes the all-gather covers; [whole, total) is the tail
    *to_out = to;
    *from_out = from;
    out[0] = std::max(cut[d], part * (uint64_t)to);
    out[1] = std::min(cut[d + 1], part * (uint64_t)(to + 1));
    out[2] = std::max(cut[d], whole);
    out[3] = cut[d + 1];
    out[4] = std::max(cut[from], part * (uint64_t)d);
    out[5] = std::min(cut[from + 1], part * (uint64_t)(d + 1));
    out[6] = std::max(cut[from], whole);
    out[7] = cut[from + 1];
}

}  // namespace b200spmm
