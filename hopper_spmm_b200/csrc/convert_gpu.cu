// CSR -> condensed row-window tiles on the GPU.  Same output, bit for bit, as the host converter
// (format.cpp) and therefore as the reference's CSR2BTCFNOBITMAP (src/utils/convert.h:146-225),
// for CSR whose rows hold ascending, distinct columns (what the reference's loader produces,
// src/utils/load.h:137-145,256).  The reference converts on one host thread; the largest
// benchmark matrix (5.2e8 entries) takes ten seconds on sixteen host cores and well under one on
// the device.
//
// Steps (all integer work, bound by HBM traffic):
//   1. one key (window << 32 | column) per entry, the entry's row found by binary search in row_ptr
//   2. radix sort of the keys, then unique -> the sorted distinct columns of every window
//      (CUB device primitives: sort, select-unique, run-length encode, scans)
//   3. run lengths per window -> tiles per window -> rowOffset, rowIdx; column lists scattered into
//      tcA2B (pre-filled with 0xFFFFFFFF padding)
//   4. every entry finds its slot by binary search in its window's column list and is written into
//      the zero-filled tile array
#include <cstdint>
#include <cub/cub.cuh>
#include <thrust/iterator/transform_iterator.h>
#include <new>

#include "../../include/b200_spmm.h"
#include "common.hpp"
#include "format.hpp"

struct b200spmm_dbtcf {
    b200spmm_btcf_info_t info{};
    int device = 0;
    uint32_t *d_rowOffset = nullptr, *d_tcA2B = nullptr, *d_rowIdx = nullptr;
    void *d_data = nullptr;
};

namespace b200spmm {
namespace gpuconv {

constexpr int kBlock = 256;

__device__ __forceinline__ uint32_t row_of_entry(const uint32_t *__restrict__ row_ptr, uint32_t rows, uint32_t p) {
    // last row r with row_ptr[r] <= p
    uint32_t lo = 0, hi = rows;
    while (hi - lo > 1) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (row_ptr[mid] <= p) lo = mid; else hi = mid;
    }
    return lo;
}

// keys[p] = window(p) << 32 | col[p]; row_of[p]; flags a column out of range or a row whose
// columns are not strictly ascending.
__global__ void make_keys_kernel(const uint32_t *__restrict__ row_ptr, const uint32_t *__restrict__ col_idx,
                                 uint32_t rows, uint32_t cols, uint64_t nnz, uint32_t row_window,
                                 uint64_t *__restrict__ keys, uint32_t *__restrict__ row_of, uint32_t *__restrict__ bad) {
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = row_of_entry(row_ptr, rows, (uint32_t)p);
        const uint32_t c = col_idx[p];
        if (c >= cols || (p > row_ptr[r] && col_idx[p - 1] >= c)) atomicOr(bad, 1u);
        keys[p] = ((uint64_t)(r / row_window) << 32) | c;
        row_of[p] = r;
    }
}

struct WindowOfKey {
    __host__ __device__ uint32_t operator()(uint64_t k) const { return (uint32_t)(k >> 32); }
};

// per effective window e: tiles, first row; dense map window -> e
__global__ void window_tables_kernel(const uint32_t *__restrict__ win_ids, const uint32_t *__restrict__ counts,
                                     uint32_t eff, uint32_t row_window, uint32_t col_window,
                                     uint32_t *__restrict__ tiles, uint32_t *__restrict__ rowIdx,
                                     uint32_t *__restrict__ win2eff) {
    const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= eff) return;
    tiles[e] = (counts[e] + col_window - 1) / col_window;
    rowIdx[e] = win_ids[e] * row_window;
    win2eff[win_ids[e]] = e;
}

// distinct column j (sorted by window, column) -> its place in the window's padded column list
__global__ void scatter_columns_kernel(const uint64_t *__restrict__ ukeys, uint64_t n_unique,
                                       const uint32_t *__restrict__ win2eff, const uint32_t *__restrict__ ubase,
                                       const uint32_t *__restrict__ rowOffset, uint32_t col_window,
                                       uint32_t *__restrict__ tcA2B) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_unique; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t k = ukeys[j];
        const uint32_t e = win2eff[(uint32_t)(k >> 32)];
        const uint64_t pos = j - ubase[e];
        tcA2B[(uint64_t)rowOffset[e] * col_window + pos] = (uint32_t)k;
    }
}

// entry p -> data[(rowOffset[e] + slot / CW) * RW * CW + (r % RW) * CW + slot % CW]
template <typename T>
__global__ void scatter_values_kernel(const uint32_t *__restrict__ col_idx, const T *__restrict__ values,
                                      const uint32_t *__restrict__ row_of, uint64_t nnz,
                                      const uint32_t *__restrict__ win2eff, const uint32_t *__restrict__ rowOffset,
                                      const uint32_t *__restrict__ counts, const uint32_t *__restrict__ tcA2B,
                                      uint32_t row_window, uint32_t col_window, T *__restrict__ data) {
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = row_of[p], c = col_idx[p];
        const uint32_t e = win2eff[r / row_window];
        const uint32_t *list = tcA2B + (uint64_t)rowOffset[e] * col_window;
        uint32_t lo = 0, hi = counts[e];  // the window's real columns are ascending; padding follows them
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2;
            if (list[mid] < c) lo = mid + 1; else hi = mid;
        }
        const uint64_t tile = (uint64_t)rowOffset[e] + lo / col_window;
        data[tile * row_window * col_window + (uint64_t)(r % row_window) * col_window + lo % col_window] = values[p];
    }
}

struct Scratch {  // device buffers released on every exit path
    void *ptrs[16] = {};
    int n = 0;
    template <typename T>
    cudaError_t alloc(T **out, size_t count) {
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, std::max<size_t>(count * sizeof(T), 16));
        if (e == cudaSuccess) ptrs[n++] = p;
        *out = static_cast<T *>(p);
        return e;
    }
    ~Scratch() { for (int i = 0; i < n; ++i) cudaFree(ptrs[i]); }
};

inline int grid_for(uint64_t n) { return (int)std::min<uint64_t>((n + kBlock - 1) / kBlock, 148 * 32); }

}  // namespace gpuconv
}  // namespace b200spmm

using namespace b200spmm;
using namespace b200spmm::gpuconv;

extern "C" {

void b200spmm_dbtcf_destroy(b200spmm_dbtcf_t *f) {
    if (!f) return;
    cudaSetDevice(f->device);
    cudaFree(f->d_rowOffset);
    cudaFree(f->d_tcA2B);
    cudaFree(f->d_rowIdx);
    cudaFree(f->d_data);
    delete f;
}

int b200spmm_dbtcf_info(const b200spmm_dbtcf_t *f, b200spmm_btcf_info_t *info) {
    if (!f || !info) return B200SPMM_ERR_INVALID_ARG;
    *info = f->info;
    return B200SPMM_OK;
}
const uint32_t *b200spmm_dbtcf_rowOffset(const b200spmm_dbtcf_t *f) { return f ? f->d_rowOffset : nullptr; }
const uint32_t *b200spmm_dbtcf_tcA2B(const b200spmm_dbtcf_t *f) { return f ? f->d_tcA2B : nullptr; }
const void *b200spmm_dbtcf_data(const b200spmm_dbtcf_t *f) { return f ? f->d_data : nullptr; }
const uint32_t *b200spmm_dbtcf_rowIdx(const b200spmm_dbtcf_t *f) { return f ? f->d_rowIdx : nullptr; }

int b200spmm_dbtcf_copy_to_host(const b200spmm_dbtcf_t *f, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                                uint32_t *rowIdx) {
    if (!f || !rowOffset || !tcA2B || !data || !rowIdx) return B200SPMM_ERR_INVALID_ARG;
    B200_CUDA_TRY(cudaSetDevice(f->device));
    const auto &i = f->info;
    const uint64_t tile_elems = (uint64_t)i.row_window * i.col_window;
    B200_CUDA_TRY(cudaMemcpy(rowOffset, f->d_rowOffset, (i.eff_row_windows + 1) * 4, cudaMemcpyDeviceToHost));
    if (i.total_tiles) {
        B200_CUDA_TRY(cudaMemcpy(tcA2B, f->d_tcA2B, i.total_tiles * i.col_window * 4, cudaMemcpyDeviceToHost));
        B200_CUDA_TRY(cudaMemcpy(data, f->d_data, i.total_tiles * tile_elems * i.elt_size, cudaMemcpyDeviceToHost));
        B200_CUDA_TRY(cudaMemcpy(rowIdx, f->d_rowIdx, i.eff_row_windows * 4, cudaMemcpyDeviceToHost));
    }
    return B200SPMM_OK;
}

int b200spmm_csr2btcf_nobitmap_device(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *d_row_ptr,
                                      const uint32_t *d_col_idx, const void *d_values, int dtype, int row_window,
                                      int col_window, int device, void *stream_v, b200spmm_dbtcf_t **out) {
    if (!out || !d_row_ptr || (nnz && (!d_col_idx || !d_values))) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    if (dtype != B200SPMM_F16 && dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    if (row_window != 8 && row_window != 16) return B200SPMM_ERR_INVALID_ARG;
    if (col_window == 0) col_window = dtype == B200SPMM_F16 ? 16 : 8;
    if (col_window != 4 && col_window != 8 && col_window != 16) return B200SPMM_ERR_INVALID_ARG;
    if (rows >= 0xFFFFFFFFull || cols > 0xFFFFFFFFull || nnz > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    B200_CUDA_TRY(cudaSetDevice(device));
    const uint32_t RW = (uint32_t)row_window, CW = (uint32_t)col_window;
    const int esz = dtype == B200SPMM_F16 ? 2 : 4;
    const uint64_t n_windows = (rows + RW - 1) / RW;

    b200spmm_dbtcf *f = new (std::nothrow) b200spmm_dbtcf();
    if (!f) return B200SPMM_ERR_NO_MEMORY;
    f->device = device;
    f->info.rows = rows;
    f->info.cols = cols;
    f->info.nnzs = nnz;
    f->info.total_row_windows = n_windows;
    f->info.row_window = row_window;
    f->info.col_window = col_window;
    f->info.dtype = dtype;
    f->info.elt_size = esz;
    struct Guard {  // frees the half-built result unless released
        b200spmm_dbtcf *f;
        ~Guard() { if (f) b200spmm_dbtcf_destroy(f); }
    } guard{f};

    uint32_t head[2] = {0, 0};
    {   // row_ptr must start at 0 and end at nnz
        B200_CUDA_TRY(cudaMemcpyAsync(&head[0], d_row_ptr, 4, cudaMemcpyDeviceToHost, stream));
        B200_CUDA_TRY(cudaMemcpyAsync(&head[1], d_row_ptr + rows, 4, cudaMemcpyDeviceToHost, stream));
        B200_CUDA_TRY(cudaStreamSynchronize(stream));
        if (head[0] != 0 || head[1] != nnz) return B200SPMM_ERR_BAD_CSR;
    }
    if (nnz == 0) {
        B200_CUDA_TRY(cudaMalloc(&f->d_rowOffset, 16));
        B200_CUDA_TRY(cudaMemsetAsync(f->d_rowOffset, 0, 16, stream));
        B200_CUDA_TRY(cudaStreamSynchronize(stream));
        guard.f = nullptr;
        *out = f;
        return B200SPMM_OK;
    }

    Scratch tmp;
    uint64_t *keys = nullptr, *keys_sorted = nullptr, *ukeys = nullptr, *n_sel = nullptr;
    uint32_t *row_of = nullptr, *bad = nullptr, *win_ids = nullptr, *counts = nullptr, *n_runs = nullptr;
    uint32_t *tiles = nullptr, *ubase = nullptr, *win2eff = nullptr;
    B200_CUDA_TRY(tmp.alloc(&keys, nnz));
    B200_CUDA_TRY(tmp.alloc(&keys_sorted, nnz));
    B200_CUDA_TRY(tmp.alloc(&row_of, nnz));
    B200_CUDA_TRY(tmp.alloc(&bad, 1));
    B200_CUDA_TRY(tmp.alloc(&n_sel, 1));
    B200_CUDA_TRY(tmp.alloc(&n_runs, 1));
    B200_CUDA_TRY(cudaMemsetAsync(bad, 0, 4, stream));

    // 1. keys
    make_keys_kernel<<<grid_for(nnz), kBlock, 0, stream>>>(d_row_ptr, d_col_idx, (uint32_t)rows, (uint32_t)cols, nnz, RW,
                                                           keys, row_of, bad);
    B200_CUDA_TRY(cudaGetLastError());

    // 2. sort, unique
    int win_bits = 1;
    while ((1ull << win_bits) < n_windows) ++win_bits;
    size_t sort_bytes = 0, sel_bytes = 0, rle_bytes = 0, scan_bytes = 0;
    B200_CUDA_TRY(cub::DeviceRadixSort::SortKeys(nullptr, sort_bytes, keys, keys_sorted, (int64_t)nnz, 0, 32 + win_bits, stream));
    ukeys = keys;  // the unsorted keys are dead once sorted: reuse their buffer for the distinct keys
    B200_CUDA_TRY(cub::DeviceSelect::Unique(nullptr, sel_bytes, keys_sorted, ukeys, n_sel, (int64_t)nnz, stream));
    uint8_t *cub_tmp = nullptr;
    B200_CUDA_TRY(tmp.alloc(&cub_tmp, std::max(sort_bytes, sel_bytes)));
    B200_CUDA_TRY(cub::DeviceRadixSort::SortKeys(cub_tmp, sort_bytes, keys, keys_sorted, (int64_t)nnz, 0, 32 + win_bits, stream));
    B200_CUDA_TRY(cub::DeviceSelect::Unique(cub_tmp, sel_bytes, keys_sorted, ukeys, n_sel, (int64_t)nnz, stream));
    uint64_t n_unique = 0;
    uint32_t bad_h = 0;
    B200_CUDA_TRY(cudaMemcpyAsync(&n_unique, n_sel, 8, cudaMemcpyDeviceToHost, stream));
    B200_CUDA_TRY(cudaMemcpyAsync(&bad_h, bad, 4, cudaMemcpyDeviceToHost, stream));
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    if (bad_h) return B200SPMM_ERR_BAD_CSR;

    // 3. windows: run lengths of the window id over the distinct keys
    B200_CUDA_TRY(tmp.alloc(&win_ids, std::min<uint64_t>(n_windows, n_unique)));
    B200_CUDA_TRY(tmp.alloc(&counts, std::min<uint64_t>(n_windows, n_unique) + 1));
    auto win_of = thrust::make_transform_iterator(static_cast<const uint64_t *>(ukeys), WindowOfKey());
    B200_CUDA_TRY(cub::DeviceRunLengthEncode::Encode(nullptr, rle_bytes, win_of, win_ids, counts, n_runs, (int64_t)n_unique, stream));
    uint8_t *rle_tmp = nullptr;
    B200_CUDA_TRY(tmp.alloc(&rle_tmp, rle_bytes));
    B200_CUDA_TRY(cub::DeviceRunLengthEncode::Encode(rle_tmp, rle_bytes, win_of, win_ids, counts, n_runs, (int64_t)n_unique, stream));
    uint32_t eff = 0;
    B200_CUDA_TRY(cudaMemcpyAsync(&eff, n_runs, 4, cudaMemcpyDeviceToHost, stream));
    B200_CUDA_TRY(cudaStreamSynchronize(stream));

    B200_CUDA_TRY(tmp.alloc(&tiles, (uint64_t)eff + 1));
    B200_CUDA_TRY(tmp.alloc(&ubase, (uint64_t)eff + 1));
    B200_CUDA_TRY(tmp.alloc(&win2eff, n_windows));
    B200_CUDA_TRY(cudaMalloc(&f->d_rowOffset, ((uint64_t)eff + 1) * 4));
    B200_CUDA_TRY(cudaMalloc(&f->d_rowIdx, std::max<uint64_t>((uint64_t)eff * 4, 16)));
    B200_CUDA_TRY(cudaMemsetAsync(tiles + eff, 0, 4, stream));
    B200_CUDA_TRY(cudaMemsetAsync(counts + eff, 0, 4, stream));
    window_tables_kernel<<<(eff + kBlock - 1) / kBlock, kBlock, 0, stream>>>(win_ids, counts, eff, RW, CW, tiles,
                                                                             f->d_rowIdx, win2eff);
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, tiles, f->d_rowOffset, (int)(eff + 1), stream));
    uint8_t *scan_tmp = nullptr;
    B200_CUDA_TRY(tmp.alloc(&scan_tmp, scan_bytes));
    B200_CUDA_TRY(cub::DeviceScan::ExclusiveSum(scan_tmp, scan_bytes, tiles, f->d_rowOffset, (int)(eff + 1), stream));
    B200_CUDA_TRY(cub::DeviceScan::ExclusiveSum(scan_tmp, scan_bytes, counts, ubase, (int)(eff + 1), stream));
    uint32_t total_tiles = 0;
    B200_CUDA_TRY(cudaMemcpyAsync(&total_tiles, f->d_rowOffset + eff, 4, cudaMemcpyDeviceToHost, stream));
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    // (a tile count beyond 32 bits would have wrapped in the scan: bound it by the entry count instead)
    if ((uint64_t)n_unique / CW + eff > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;

    f->info.eff_row_windows = eff;
    f->info.total_tiles = total_tiles;
    const uint64_t list_len = (uint64_t)total_tiles * CW, data_len = (uint64_t)total_tiles * RW * CW;
    B200_CUDA_TRY(cudaMalloc(&f->d_tcA2B, std::max<uint64_t>(list_len * 4, 16)));
    B200_CUDA_TRY(cudaMalloc(&f->d_data, std::max<uint64_t>(data_len * esz, 16)));
    B200_CUDA_TRY(cudaMemsetAsync(f->d_tcA2B, 0xFF, list_len * 4, stream));  // kIdxMax padding
    B200_CUDA_TRY(cudaMemsetAsync(f->d_data, 0, data_len * esz, stream));
    scatter_columns_kernel<<<grid_for(n_unique), kBlock, 0, stream>>>(ukeys, n_unique, win2eff, ubase, f->d_rowOffset, CW,
                                                                      f->d_tcA2B);
    B200_CUDA_TRY(cudaGetLastError());

    // 4. values
    if (esz == 2)
        scatter_values_kernel<uint16_t><<<grid_for(nnz), kBlock, 0, stream>>>(
            d_col_idx, static_cast<const uint16_t *>(d_values), row_of, nnz, win2eff, f->d_rowOffset, counts, f->d_tcA2B,
            RW, CW, static_cast<uint16_t *>(f->d_data));
    else
        scatter_values_kernel<uint32_t><<<grid_for(nnz), kBlock, 0, stream>>>(
            d_col_idx, static_cast<const uint32_t *>(d_values), row_of, nnz, win2eff, f->d_rowOffset, counts, f->d_tcA2B,
            RW, CW, static_cast<uint32_t *>(f->d_data));
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    guard.f = nullptr;
    *out = f;
    return B200SPMM_OK;
}

}  // extern "C"
