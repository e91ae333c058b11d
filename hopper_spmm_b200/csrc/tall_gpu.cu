// 16-row condensed format -> super-windows of 128 or 256 rows, on the device.  Same result as converting the
// matrix at that window height with the reference's algorithm (src/utils/convert.h:146-225):
// sorted distinct columns per window, padded to whole tiles; entries at (row % 128, column slot).
//
// Steps (integer work, bound by HBM traffic):
//   1. one key (super-window << 32 | column) per column-list entry of the 16-row format
//   2. radix sort + unique (CUB): the sorted distinct columns of every super-window
//   3. per super-window: first distinct key and count (binary search) -> tiles -> rowOffset
//   4. column lists scattered into tcA2B (pre-filled with 0xFFFFFFFF)
//   5. every (16-row tile, column slot) finds its slot in the super-window's list and its sixteen
//      values move into the zero-filled 128-row tiles, which are stored as the kernel's shared-memory
//      image (the two 16-byte halves of a tile row swapped when row / 4 is odd: the 32-byte swizzle)
#include <algorithm>
#include <cub/cub.cuh>
#include <vector>

#include "common.hpp"
#include "format.hpp"
#include "tall_gpu.hpp"

namespace b200spmm {
namespace {

constexpr int kBlock = 256;
constexpr uint32_t kShort = 16;

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

inline int grid_for(uint64_t n) { return (int)std::max<uint64_t>(1, std::min<uint64_t>((n + kBlock - 1) / kBlock, 148 * 32)); }

// window holding tile t: last i with rowOffset[i] <= t
__device__ __forceinline__ uint32_t window_of_tile(const uint32_t *__restrict__ rowOffset, uint32_t eff, uint32_t t) {
    uint32_t lo = 0, hi = eff;
    while (hi - lo > 1) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (rowOffset[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// keys[e] = group(window of entry e) << 32 | column; padding entries get the key of a group past the end
__global__ void tall_keys_kernel(const uint32_t *__restrict__ rowOffset, const uint32_t *__restrict__ tcA2B,
                                 const uint32_t *__restrict__ win_group, uint32_t eff, uint32_t n_groups, uint32_t cw,
                                 uint64_t n_entries, uint64_t *__restrict__ keys) {
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_entries; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t c = tcA2B[e];
        if (c == kIdxMax) {
            keys[e] = ((uint64_t)n_groups << 32) | kIdxMax;
        } else {
            const uint32_t i = window_of_tile(rowOffset, eff, (uint32_t)(e / cw));
            keys[e] = ((uint64_t)win_group[i] << 32) | c;
        }
    }
}

// ubase[g] = index of the first distinct key of group g (g = n_groups: the end of the real keys)
__global__ void tall_group_base_kernel(const uint64_t *__restrict__ ukeys, uint64_t n_unique, uint32_t n_groups,
                                       uint32_t *__restrict__ ubase) {
    const uint32_t g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g > n_groups) return;
    const uint64_t want = (uint64_t)g << 32;
    uint64_t lo = 0, hi = n_unique;
    while (lo < hi) {
        const uint64_t mid = lo + (hi - lo) / 2;
        if (ukeys[mid] < want) lo = mid + 1; else hi = mid;
    }
    ubase[g] = (uint32_t)lo;
}

__global__ void tall_scatter_columns_kernel(const uint64_t *__restrict__ ukeys, uint64_t n_real,
                                            const uint32_t *__restrict__ ubase, const uint32_t *__restrict__ t_rowOffset,
                                            uint32_t cw, uint32_t *__restrict__ t_tcA2B) {
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_real; j += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t k = ukeys[j];
        const uint32_t g = (uint32_t)(k >> 32);
        t_tcA2B[(uint64_t)t_rowOffset[g] * cw + (j - ubase[g])] = (uint32_t)k;
    }
}

// one thread per (16-row tile, column slot): its sixteen values go to the super-window's tile
template <typename T>
__global__ void tall_scatter_values_kernel(const uint32_t *__restrict__ rowOffset, const uint32_t *__restrict__ tcA2B,
                                           const T *__restrict__ data, const uint32_t *__restrict__ rowIdx,
                                           const uint32_t *__restrict__ win_group, uint32_t eff, uint32_t cw,
                                           uint64_t n_entries, const uint32_t *__restrict__ ubase,
                                           const uint32_t *__restrict__ t_rowOffset, const uint32_t *__restrict__ t_tcA2B,
                                           const uint32_t *__restrict__ t_rowIdx, uint32_t tall_rows, T *__restrict__ t_data) {
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_entries; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t c = tcA2B[e];
        if (c == kIdxMax) continue;
        const uint32_t t = (uint32_t)(e / cw), lc = (uint32_t)(e % cw);
        const uint32_t i = window_of_tile(rowOffset, eff, t);
        const uint32_t g = win_group[i];
        const uint32_t *list = t_tcA2B + (uint64_t)t_rowOffset[g] * cw;
        uint32_t lo = 0, hi = ubase[g + 1] - ubase[g];  // the group's real columns, ascending
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2;
            if (list[mid] < c) lo = mid + 1; else hi = mid;
        }
        // A tile image is 128 rows.  Windows of 256 rows keep, per window, the images of rows 0-127 of all
        // its tiles and then those of rows 128-255 (each CTA of a pair reads its own run).
        const uint32_t olc = lo % cw, shift = rowIdx[i] - t_rowIdx[g], part = shift / 128u, row_shift = shift % 128u;
        const uint64_t g_first = t_rowOffset[g], g_tiles = t_rowOffset[g + 1] - g_first;
        const uint64_t ot = g_first * (tall_rows / 128u) + part * g_tiles + lo / cw;
        const T *src = data + ((uint64_t)t * kShort) * cw + lc;
        T *dst = t_data + (ot * 128u + row_shift) * cw;
        const uint32_t half = cw / 2;  // elements per 16-byte half of a tile row
#pragma unroll 4
        for (uint32_t lr = 0; lr < kShort; ++lr) {
            const uint32_t flip = ((row_shift + lr) >> 2) & 1u;  // the 32-byte swizzle of the shared-memory image
            dst[(uint64_t)lr * cw + (((olc / half) ^ flip) * half + olc % half)] = src[(uint64_t)lr * cw];
        }
    }
}

// Runs of 16-row windows that fall into the same 128-row window.
void group_windows(const uint32_t *h_rowIdx, uint64_t eff, uint32_t kTall, std::vector<uint32_t> *win_group,
                   std::vector<uint64_t> *group_first) {
    win_group->resize(eff);
    group_first->clear();
    for (uint64_t i = 0; i < eff; ++i) {
        if (i == 0 || h_rowIdx[i] / kTall != h_rowIdx[i - 1] / kTall) group_first->push_back(i);
        (*win_group)[i] = (uint32_t)(group_first->size() - 1);
    }
    group_first->push_back(eff);
}

}  // namespace

int estimate_tall_tile_ratio(const b200spmm_btcf_info_t &info, const uint32_t *h_rowOffset, const uint32_t *h_rowIdx,
                             const uint32_t *d_tcA2B, uint32_t tall_rows, int max_samples, double *ratio,
                             uint64_t *n_super_windows) {
    const uint64_t eff = info.eff_row_windows, cw = (uint64_t)info.col_window;
    std::vector<uint32_t> win_group;
    std::vector<uint64_t> group_first;
    group_windows(h_rowIdx, eff, tall_rows, &win_group, &group_first);
    const uint64_t n_groups = group_first.size() - 1;
    *n_super_windows = n_groups;
    *ratio = 1.0;
    if (!n_groups || max_samples < 1) return B200SPMM_OK;
    const uint64_t step = std::max<uint64_t>(1, n_groups / (uint64_t)max_samples);
    uint64_t short_tiles = 0, tall_tiles = 0, copied = 0;
    std::vector<uint32_t> list;
    for (uint64_t g = step / 2; g < n_groups; g += step) {
        const uint64_t t0 = h_rowOffset[group_first[g]], t1 = h_rowOffset[group_first[g + 1]];
        if ((t1 - t0) * cw * 4 > (64u << 20) || copied > (256u << 20)) continue;  // keep the probe small
        list.resize((t1 - t0) * cw);
        B200_CUDA_TRY(cudaMemcpy(list.data(), d_tcA2B + t0 * cw, list.size() * 4, cudaMemcpyDeviceToHost));
        copied += list.size() * 4;
        std::sort(list.begin(), list.end());
        list.erase(std::unique(list.begin(), list.end()), list.end());
        while (!list.empty() && list.back() == kIdxMax) list.pop_back();
        short_tiles += t1 - t0;
        tall_tiles += (list.size() + cw - 1) / cw;
    }
    if (short_tiles) *ratio = (double)tall_tiles / (double)short_tiles;
    return B200SPMM_OK;
}

void free_tall(TallFormat *t) {
    cudaFree(t->d_rowOffset);
    cudaFree(t->d_tcA2B);
    cudaFree(t->d_rowIdx);
    cudaFree(t->d_data);
    *t = TallFormat();
}

int build_tall_device(const b200spmm_btcf_info_t &info, const uint32_t *h_rowOffset, const uint32_t *h_rowIdx,
                      const uint32_t *d_rowOffset, const uint32_t *d_tcA2B, const void *d_data, const uint32_t *d_rowIdx,
                      uint32_t tall_rows, TallFormat *out) {
    *out = TallFormat();
    if (info.row_window != (int)kShort || (tall_rows != 128 && tall_rows != 256)) return B200SPMM_ERR_UNSUPPORTED;
    const uint32_t kTall = tall_rows;
    const uint64_t eff = info.eff_row_windows, cw = (uint64_t)info.col_window, tiles = info.total_tiles;
    if (!eff || !tiles) return B200SPMM_OK;
    const uint64_t n_entries = tiles * cw;
    std::vector<uint32_t> win_group;
    std::vector<uint64_t> group_first;
    group_windows(h_rowIdx, eff, tall_rows, &win_group, &group_first);
    const uint64_t n_groups = group_first.size() - 1;
    std::vector<uint32_t> h_t_rowIdx(n_groups);
    for (uint64_t g = 0; g < n_groups; ++g) h_t_rowIdx[g] = h_rowIdx[group_first[g]] / kTall * kTall;

    Scratch tmp;
    uint32_t *d_group = nullptr, *d_ubase = nullptr;
    uint64_t *keys = nullptr, *keys_sorted = nullptr, *n_sel = nullptr;
    B200_CUDA_TRY(tmp.alloc(&d_group, eff));
    B200_CUDA_TRY(tmp.alloc(&d_ubase, n_groups + 2));
    B200_CUDA_TRY(tmp.alloc(&keys, n_entries));
    B200_CUDA_TRY(tmp.alloc(&keys_sorted, n_entries));
    B200_CUDA_TRY(tmp.alloc(&n_sel, 1));
    B200_CUDA_TRY(cudaMemcpy(d_group, win_group.data(), eff * 4, cudaMemcpyHostToDevice));
    tall_keys_kernel<<<grid_for(n_entries), kBlock>>>(d_rowOffset, d_tcA2B, d_group, (uint32_t)eff, (uint32_t)n_groups,
                                                      (uint32_t)cw, n_entries, keys);
    B200_CUDA_TRY(cudaGetLastError());
    int group_bits = 1;
    while ((1ull << group_bits) < n_groups + 1) ++group_bits;
    size_t sort_bytes = 0, sel_bytes = 0;
    B200_CUDA_TRY(cub::DeviceRadixSort::SortKeys(nullptr, sort_bytes, keys, keys_sorted, (int64_t)n_entries, 0, 32 + group_bits));
    uint64_t *ukeys = keys;  // the unsorted keys are dead once sorted
    B200_CUDA_TRY(cub::DeviceSelect::Unique(nullptr, sel_bytes, keys_sorted, ukeys, n_sel, (int64_t)n_entries));
    uint8_t *cub_tmp = nullptr;
    B200_CUDA_TRY(tmp.alloc(&cub_tmp, std::max(sort_bytes, sel_bytes)));
    B200_CUDA_TRY(cub::DeviceRadixSort::SortKeys(cub_tmp, sort_bytes, keys, keys_sorted, (int64_t)n_entries, 0, 32 + group_bits));
    B200_CUDA_TRY(cub::DeviceSelect::Unique(cub_tmp, sel_bytes, keys_sorted, ukeys, n_sel, (int64_t)n_entries));
    uint64_t n_unique = 0;
    B200_CUDA_TRY(cudaMemcpy(&n_unique, n_sel, 8, cudaMemcpyDeviceToHost));
    tall_group_base_kernel<<<(unsigned)((n_groups + 1 + kBlock - 1) / kBlock), kBlock>>>(ukeys, n_unique, (uint32_t)n_groups, d_ubase);
    B200_CUDA_TRY(cudaGetLastError());
    std::vector<uint32_t> ubase(n_groups + 1), t_rowOffset(n_groups + 1, 0);
    B200_CUDA_TRY(cudaMemcpy(ubase.data(), d_ubase, (n_groups + 1) * 4, cudaMemcpyDeviceToHost));
    uint64_t t_tiles = 0;
    for (uint64_t g = 0; g < n_groups; ++g) {
        t_tiles += ((uint64_t)(ubase[g + 1] - ubase[g]) + cw - 1) / cw;
        t_rowOffset[g + 1] = (uint32_t)t_tiles;
    }
    if (t_tiles > 0xFFFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;  // rowOffset is 32-bit

    TallFormat t;
    t.rows = kTall;
    t.eff = n_groups;
    t.tiles = t_tiles;
    struct Guard {
        TallFormat *t;
        ~Guard() { if (t) free_tall(t); }
    } guard{&t};
    const uint64_t list_len = t_tiles * cw, data_len = t_tiles * kTall * cw;
    B200_CUDA_TRY(cudaMalloc(&t.d_rowOffset, (n_groups + 1) * 4));
    B200_CUDA_TRY(cudaMalloc(&t.d_rowIdx, n_groups * 4));
    B200_CUDA_TRY(cudaMalloc(&t.d_tcA2B, list_len * 4));
    B200_CUDA_TRY(cudaMalloc(&t.d_data, data_len * info.elt_size));
    B200_CUDA_TRY(cudaMemcpy(t.d_rowOffset, t_rowOffset.data(), (n_groups + 1) * 4, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMemcpy(t.d_rowIdx, h_t_rowIdx.data(), n_groups * 4, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMemset(t.d_tcA2B, 0xFF, list_len * 4));
    B200_CUDA_TRY(cudaMemset(t.d_data, 0, data_len * info.elt_size));
    const uint64_t n_real = ubase[n_groups];
    tall_scatter_columns_kernel<<<grid_for(n_real), kBlock>>>(ukeys, n_real, d_ubase, t.d_rowOffset, (uint32_t)cw, t.d_tcA2B);
    B200_CUDA_TRY(cudaGetLastError());
    if (info.elt_size == 2)
        tall_scatter_values_kernel<uint16_t><<<grid_for(n_entries), kBlock>>>(
            d_rowOffset, d_tcA2B, static_cast<const uint16_t *>(d_data), d_rowIdx, d_group, (uint32_t)eff, (uint32_t)cw,
            n_entries, d_ubase, t.d_rowOffset, t.d_tcA2B, t.d_rowIdx, kTall, static_cast<uint16_t *>(t.d_data));
    else
        tall_scatter_values_kernel<uint32_t><<<grid_for(n_entries), kBlock>>>(
            d_rowOffset, d_tcA2B, static_cast<const uint32_t *>(d_data), d_rowIdx, d_group, (uint32_t)eff, (uint32_t)cw,
            n_entries, d_ubase, t.d_rowOffset, t.d_tcA2B, t.d_rowIdx, kTall, static_cast<uint32_t *>(t.d_data));
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaDeviceSynchronize());
    *out = t;
    guard.t = nullptr;
    return B200SPMM_OK;
}

}  // namespace b200spmm
