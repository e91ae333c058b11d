// C ABI of the library (include/b200_spmm.h): format handles, device plans, launches.
// Replaces the host side of the reference's operator, fp16_spmm (src/fp16.cu:221-281).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/b200_spmm.h"
#include "common.hpp"
#include "compress_gpu.hpp"
#include "format.hpp"
#include "handles.hpp"
#include "spmm_kernel.cuh"
#include "spmm_pair_kernel.cuh"
#include "spmm_tall_kernel.cuh"
#include "tall_gpu.hpp"
#include "tensormap.hpp"

namespace b200spmm {

namespace {
// The last error of the calling thread: either a composed text (CUDA failures: the failing call
// and the runtime's message) or a pointer to a fixed message, which needs no allocation.
thread_local std::string g_last_cuda_error;
thread_local const char *g_last_static_error = nullptr;
}

void record_cuda_error(cudaError_t e, const char *what) {
    g_last_static_error = nullptr;
    g_last_cuda_error = std::string(what) + ": " + cudaGetErrorString(e);
    cudaGetLastError();  // clear the sticky-free error so later calls start clean
}

void set_last_error_static(const char *message) { g_last_static_error = message; }

}  // namespace b200spmm

using namespace b200spmm;


struct b200spmm_plan {
    b200spmm_btcf_info_t info{};
    int device = 0;
    bool owns_format = false;
    uint32_t *d_rowOffset = nullptr, *d_tcA2B = nullptr, *d_rowIdx = nullptr;
    void *d_data = nullptr;
    // The schedule: the tile stream cut into chunks (tile cuts, first / last window and the
    // partial-result slots of each chunk), which the CTAs claim at run time, plus the split
    // windows and their slots for the fix-up kernel.
    struct Sched {
        int n_ctas = 0;
        uint32_t n_chunks = 0;
        uint32_t *d_tile = nullptr, *d_wfirst = nullptr, *d_wlast = nullptr, *d_head_slot = nullptr, *d_tail_slot = nullptr;
        SplitWindow *d_splits = nullptr;
        uint32_t *d_piece_slots = nullptr;
        uint32_t n_splits = 0, n_slots = 0;
        // Bands: the chunk table cut into a few runs of whole windows, so that a caller can launch
        // band after band and start copying a band's rows of C out while the next one is computed.
        // Band k covers chunks [band_chunk[k], band_chunk[k+1]), rows [band_row[k], band_row[k+1])
        // and the split windows [band_split[k], band_split[k+1]).
        std::vector<uint32_t> band_chunk, band_split;
        std::vector<uint64_t> band_row;
    } sched;
    cudaStream_t copy_stream = nullptr;       // host-buffer call: C goes out on this one
    cudaStream_t upload_stream = nullptr;     // ... and the second half of B's features comes in on this one
    cudaEvent_t half_up[2] = {nullptr, nullptr};
    bool host_split = true;                   // B200SPMM_HOST_SPLIT=0 (read when the plan is made) turns the halves off
    std::vector<cudaEvent_t> band_done;
    const Sched *launch_sched = nullptr;  // the one the next launch uses
    CompressedTiles comp;                 // the tiles as bitmap + stored values (empty: dense tiles only)
    // fp16 tiles as records of 32 (position, value) words (SpmmParams::tile_entries), or null: B200SPMM_TILES=entries
    uint32_t *d_tile_entries = nullptr;
    uint64_t entry_dense_tiles = 0;       // tiles with more than 32 entries, which stay dense
    // The same matrix in 128-row super-windows, built when merging eight windows shortens the tile
    // stream enough for the wide-MMA kernel (spmm_tall_kernel.cuh) to win; empty otherwise.
    TallFormat tall;
    bool tall_forced = false;  // B200SPMM_WINDOW=128 or 256: use it whatever the launch's size
    // ... and in 256-row super-windows for the CTA-pair kernel (spmm_pair_kernel.cuh), which takes the
    // launches wider than 128 features when doubling the window height again halves the tile count.
    TallFormat pair;
    int pair_clusters = 0;     // two-CTA clusters of that kernel the GPU runs at the same time
    // Most tiles of the super-window format name one aligned group of CW consecutive rows of B: then B
    // is re-laid as shared-memory images at every launch (scratch of the plan, as large as B) and such a
    // tile's operand arrives by one bulk copy.
    bool tall_pack_b = false;
    void *d_b_packed = nullptr;
    size_t b_packed_bytes = 0;
    int n_sms = 0;
    // The tiles as the kernel's shared-memory image (spmm_kernel.cuh, SpmmParams::tiles_image): the plan's own
    // array swizzled in place when it owns the format, a swizzled copy when the arrays are the caller's.
    void *d_tiles_image = nullptr;
    bool image_is_copy = false;
    float *d_partial = nullptr;  // [n_slots][16][n] fp32, grown to the largest need seen
    size_t partial_floats = 0;
    uint32_t *d_status = nullptr;
    CUtensorMap tmap_a{};
    // Tensor map over B, kept between launches: B's address, pitch and width rarely change from call
    // to call, and encoding a map costs the host several microseconds of a 10-microsecond launch.
    CUtensorMap tmap_b{};   // box: 128 bytes of one row (the unit of tile::gather4)
    CUtensorMap tmap_bt{};  // box: 128 bytes of CW consecutive rows (tiles whose columns are neighbours)
    const void *tmap_b_ptr = nullptr;
    int64_t tmap_b_ldb = 0;
    uint32_t tmap_b_n = 0;
    bool gather_cpasync = false;  // B200SPMM_GATHER=cpasync, read when the plan is made
    unsigned long long wait_limit_ns = kDeviceWaitLimitNs;  // how long a wait inside the kernel may last
    bool starve_gathers = false;  // b200spmm_kat_spmm_starved only: B's tensor map delivers half the bytes
    // buffers of the host-pointer entry point, grown on demand
    void *d_B = nullptr, *d_C = nullptr;
    size_t d_B_bytes = 0, d_C_bytes = 0;
    b200spmm_launch_info_t last{};
};

namespace tileimage {
// dst row r (32 bytes) = src row r with its 16-byte halves swapped when (r / 4) is odd; dst may be src.
__global__ void swizzle_tiles_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, uint64_t n_rows) {
    for (uint64_t r = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += (uint64_t)gridDim.x * blockDim.x) {
        const uint4 lo = src[2 * r], hi = src[2 * r + 1];
        const bool flip = (r >> 2) & 1u;
        dst[2 * r] = flip ? hi : lo;
        dst[2 * r + 1] = flip ? lo : hi;
    }
}

// One warp per fp16 tile of the reference's layout (16 rows x 16 columns, row-major): the tile's record of 32
// words.  Lane l looks at row l / 2, columns 8 (l % 2) .. +7; a stored entry is any value whose bits are not
// zero; its word is (byte offset in the tile's shared-memory image << 16) | bits, where the image swaps the
// two 16-byte halves of a row when row / 4 is odd (the 32-byte swizzle).
__global__ void __launch_bounds__(256)
tile_entries_kernel(const uint16_t *__restrict__ data, uint64_t tiles, uint32_t *__restrict__ records,
                    unsigned long long *__restrict__ n_dense) {
    const uint32_t lane = threadIdx.x & 31u;
    for (uint64_t t = (uint64_t)blockIdx.x * 8u + (threadIdx.x >> 5); t < tiles; t += (uint64_t)gridDim.x * 8u) {
        const uint4 v = *reinterpret_cast<const uint4 *>(data + t * 256u + lane * 8u);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t mask = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) mask |= (((w[k >> 1] >> ((k & 1) * 16)) & 0xFFFFu) != 0u) ? (1u << k) : 0u;
        const uint32_t mine = (uint32_t)__popc(mask);
        uint32_t before = mine;  // inclusive warp scan
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, before, d);
            if ((int)lane >= d) before += up;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, before, 31);
        before -= mine;
        uint32_t *rec = records + (t << 5);
        if (total > 32u) {
            rec[lane] = b200spmm::kDenseTile;
            if (lane == 0) atomicAdd(n_dense, 1ull);
            continue;
        }
        rec[lane] = b200spmm::kNoEntry;
        __syncwarp();
        const uint32_t row = lane >> 1, half = lane & 1u;
        const uint32_t base = row * 32u + ((half ^ ((row >> 2) & 1u)) << 4);
        uint32_t k_out = before;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (mask & (1u << k)) {
                const uint32_t bits = (w[k >> 1] >> ((k & 1) * 16)) & 0xFFFFu;
                rec[k_out++] = ((base + (uint32_t)k * 2u) << 16) | bits;
            }
        }
    }
}

}  // namespace tileimage

namespace {

template <bool kTf32, int kNs, bool kTma, int kTiles>
int launch_one(b200spmm_plan *p, const SpmmParams &prm, const CUtensorMap &tmap_b, cudaStream_t stream) {
    using Cfg = SpmmCfg<kTf32, kNs, kTma, kTiles>;
    auto kernel = spmm_sm100_kernel<kTf32, kNs, kTma, kTiles>;
    static thread_local int configured_device = -1;
    if (configured_device != p->device) {
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes));
        // all of the SM's shared-memory/L1 array as shared memory: two CTAs of the narrow slabs fit only then
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        configured_device = p->device;
    }
    kernel<<<p->launch_sched->n_ctas, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p->tmap_a, tmap_b, prm);
    B200_CUDA_TRY(cudaGetLastError());
    p->last.n_ctas = p->launch_sched->n_ctas;
    p->last.threads = Cfg::kThreads;
    p->last.stages = Cfg::kStages;
    p->last.feature_slab = kNs;
    p->last.n_slabs = (int)prm.n_slabs;
    p->last.smem_bytes = (int64_t)Cfg::kSmemBytes;
    p->last.kernel_launches = 1;
    p->last.tma_gather = kTma ? 1 : 0;
    p->last.bitmap_tiles = kTiles;
    p->last.row_window = kRowWindow;
    return B200SPMM_OK;
}

// Feature slab a launch uses for B of width n, and how many CTAs of that kernel share an SM.
constexpr uint64_t kMaxChunksPerCta = 16;
constexpr uint32_t kRowBands = 8;  // bands of the host-buffer call (large matrices only)
// Up to 128 features per pass: a CTA of that width leaves room for a second one on the SM, and two
// MMA-issuing threads per SM outweigh streaming the tiles once more per extra pass (n = 2048:
// 4.27 ms in sixteen passes of 128 against 4.65 ms in eight of 256).
inline uint32_t slab_for(uint32_t n) { return std::min(128u, (n + 63u) / 64u * 64u); }
constexpr int kCtasPerSm = 2;  // every kernel variant in use is sized for two resident CTAs per SM

template <bool kTf32, bool kTma, int kTiles>
int launch_slab(b200spmm_plan *p, SpmmParams &prm, const CUtensorMap &tmap_b, cudaStream_t stream) {
    const uint32_t ns = slab_for(prm.n);
    prm.n_slabs = (prm.n + ns - 1) / ns;
    switch (ns) {
        case 64: return launch_one<kTf32, 64, kTma, kTiles>(p, prm, tmap_b, stream);
        default: return launch_one<kTf32, 128, kTma, kTiles>(p, prm, tmap_b, stream);
    }
}

// The environment is consulted when a plan is made (and once per process for the plan-less
// allocation-free call), never on a launch.
bool env_is(const char *name, const char *value) {
    const char *v = std::getenv(name);
    return v && std::strcmp(v, value) == 0;
}

// Tensor map over B seen as [cols][n] with its real row pitch; a box is 128 bytes of one row.
// Rows or features past the end read as zeros.  Re-encoded only when B's address, pitch or width
// differ from the previous launch of this plan.
int b_tensor_map(b200spmm_plan *p, const void *B, int64_t ldb, uint32_t n, uint32_t cols, bool tf32) {
    if (p->tmap_b_ptr == B && p->tmap_b_ldb == ldb && p->tmap_b_n == n) return B200SPMM_OK;
    const uint32_t esz = tf32 ? 4 : 2, box = (p->starve_gathers ? 64 : 128) / esz;
    p->tmap_b_ptr = nullptr;
    if (!encode_2d(&p->tmap_b, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, B, n,
                   cols, (uint64_t)ldb * esz, box, 1,
                   tf32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) {
        set_last_error_static("cuTensorMapEncodeTiled failed for B");
        return B200SPMM_ERR_CUDA;
    }
    if (p->tall.tiles &&
        !encode_2d(&p->tmap_bt, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, B, n, cols,
                   (uint64_t)ldb * esz, 128 / esz, std::min<uint32_t>((uint32_t)p->info.col_window, cols),
                   tf32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) {
        set_last_error_static("cuTensorMapEncodeTiled failed for B (row boxes)");
        return B200SPMM_ERR_CUDA;
    }
    p->tmap_b_ptr = B;
    p->tmap_b_ldb = ldb;
    p->tmap_b_n = n;
    return B200SPMM_OK;
}

// How the rows of B are gathered: TMA tile::gather4 unless the plan was made with
// B200SPMM_GATHER=cpasync or B is narrower than one 128-byte TMA box.
template <bool kTf32>
int launch_dtype(b200spmm_plan *p, SpmmParams &prm, cudaStream_t stream) {
    constexpr uint32_t esz = kTf32 ? 4 : 2, box = 128 / esz;
    if (p->gather_cpasync || prm.n < box) return launch_slab<kTf32, false, 0>(p, prm, p->tmap_b, stream);
    {
        int st = b_tensor_map(p, prm.B, prm.ldb, prm.n, prm.cols, kTf32);
        if (st != B200SPMM_OK) return st;
    }
    const CUtensorMap &tmap_b = p->tmap_b;
    if (p->comp.tcBit) {  // stream the compressed tiles
        prm.tcBit = p->comp.tcBit;
        prm.nnzOffset = p->comp.nnzOffset;
        prm.values = p->comp.values;
        return launch_slab<kTf32, true, 1>(p, prm, tmap_b, stream);
    }
    if constexpr (!kTf32) {
        if (p->d_tile_entries && prm.tiles_image) {  // stream the entry lists; tiles with many entries come from the image
            prm.tile_entries = p->d_tile_entries;
            return launch_slab<false, true, 2>(p, prm, tmap_b, stream);
        }
    }
    return launch_slab<kTf32, true, 0>(p, prm, tmap_b, stream);
}

// Tensor map over `data` seen as rows of 32 bytes: one tile is 16 consecutive rows, one box is
// the eight consecutive tiles of a ring stage.
int encode_tile_map(b200spmm_plan *p) {
    const auto &info = p->info;
    if (!info.total_tiles) return B200SPMM_OK;
    const bool f16 = info.dtype == B200SPMM_F16;
    if (!encode_2d(&p->tmap_a, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p->d_data,
                   f16 ? 16 : 8, info.total_tiles * kRowWindow, 32, f16 ? 16 : 8, kRowWindow * kTilesPerStage,
                   CU_TENSOR_MAP_SWIZZLE_32B)) {
        set_last_error_static("cuTensorMapEncodeTiled failed for the tile array");
        return B200SPMM_ERR_CUDA;
    }
    return B200SPMM_OK;
}

#ifdef B200SPMM_PROFILE
unsigned long long *g_prof = nullptr;
#endif

// ---- 128-row super-windows
template <bool kTf32, int kNs>
int launch_tall_one(b200spmm_plan *p, TallParams &prm, cudaStream_t stream) {
    using Cfg = TallCfg<kTf32, kNs>;
    auto kernel = spmm_tall_kernel<kTf32, kNs>;
    static thread_local int configured_device = -1;
    if (configured_device != p->device) {
        B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes));
        configured_device = p->device;
    }
    prm.n_slabs = (prm.n + kNs - 1) / kNs;
    prm.n_items = prm.eff_row_windows * prm.n_slabs;
    const int n_ctas = (int)std::min<uint32_t>(prm.n_items, (uint32_t)p->n_sms);
    kernel<<<n_ctas, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p->tmap_b, p->tmap_bt, prm);
    B200_CUDA_TRY(cudaGetLastError());
    p->last.n_ctas = n_ctas;
    p->last.threads = Cfg::kThreads;
    p->last.stages = Cfg::kStages;
    p->last.feature_slab = kNs;
    p->last.n_slabs = (int)prm.n_slabs;
    p->last.smem_bytes = (int64_t)Cfg::kSmemBytes;
    p->last.kernel_launches = prm.b_packed ? 2 : 1;
    p->last.tma_gather = 1;
    p->last.bitmap_tiles = 0;
    p->last.row_window = kTallRows;
    return B200SPMM_OK;
}

template <bool kTf32>
int launch_pair_one(b200spmm_plan *p, TallParams &prm, cudaStream_t stream) {
    using Cfg = PairCfg<kTf32>;
    auto kernel = spmm_pair_kernel<kTf32>;
    prm.n_slabs = (prm.n + Cfg::kNs - 1) / Cfg::kNs;
    prm.n_items = prm.eff_row_windows * prm.n_slabs;
    const int n_pairs = (int)std::min<uint32_t>(prm.n_items, (uint32_t)p->pair_clusters);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * n_pairs);
    cfg.blockDim = dim3(Cfg::kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p->tmap_b, p->tmap_bt, prm));
    p->last.n_ctas = 2 * n_pairs;
    p->last.threads = Cfg::kThreads;
    p->last.stages = Cfg::kStages;
    p->last.feature_slab = Cfg::kNs;
    p->last.n_slabs = (int)prm.n_slabs;
    p->last.smem_bytes = (int64_t)Cfg::kSmemBytes;
    p->last.kernel_launches = prm.b_packed ? 2 : 1;
    p->last.tma_gather = 1;
    p->last.bitmap_tiles = 0;
    p->last.row_window = kPairRows;
    return B200SPMM_OK;
}

// How many two-CTA clusters of the pair kernel the device runs at once (0: it cannot run it).
template <bool kTf32>
int pair_max_clusters(int *out) {
    using Cfg = PairCfg<kTf32>;
    auto kernel = spmm_pair_kernel<kTf32>;
    B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * 148);
    cfg.blockDim = dim3(Cfg::kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    B200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    *out = n;
    return B200SPMM_OK;
}

bool use_pair(const b200spmm_plan *p, int64_t n) {
    if (!p->pair.tiles || p->pair_clusters < 1 || n <= 128) return false;
    if (p->tall_forced) return true;
    return (int64_t)p->pair.eff * ((n + 255) / 256) >= p->pair_clusters;
}

// Does this launch go to the super-window kernel?  Only with the TMA gathers (B at least one
// 128-byte box wide), and - unless forced - only when there are enough (window, slab) items to
// occupy every SM.
bool use_tall(const b200spmm_plan *p, int64_t n) {
    if (!p->tall.tiles || p->gather_cpasync) return false;
    if (n * p->info.elt_size < 128) return false;
    if (p->tall_forced) return true;
    const int64_t slab = n <= 128 ? 128 : 256;
    return (int64_t)p->tall.eff * ((n + slab - 1) / slab) >= p->n_sms;
}

int launch_tall(b200spmm_plan *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc, int c_dtype,
                cudaStream_t stream) {
    const bool tf32 = p->info.dtype == B200SPMM_TF32;
    int st = b_tensor_map(p, d_B, ldb, (uint32_t)n, (uint32_t)p->info.cols, tf32);
    if (st != B200SPMM_OK) return st;
    const bool pair = use_pair(p, n);
    const TallFormat &fmt = pair ? p->pair : p->tall;
    TallParams prm{};
    prm.rowOffset = fmt.d_rowOffset;
    prm.tcA2B = fmt.d_tcA2B;
    prm.rowIdx = fmt.d_rowIdx;
    prm.data = static_cast<const uint8_t *>(fmt.d_data);
    if (p->tall_pack_b) {
        const uint32_t cw = (uint32_t)p->info.col_window, esz = (uint32_t)p->info.elt_size;
        // the pair kernel's CTAs fetch 128-feature halves of a 256-feature slab: both halves of the last slab must
        // exist in the packed copy (as zeros past n), so an even number of 128-feature blocks
        const uint32_t slab = (n <= 128 || pair) ? 128u : 256u;
        const uint32_t n_slabs = pair ? 2u * (uint32_t)((n + 255) / 256) : (uint32_t)((n + slab - 1) / slab);
        const uint32_t groups = (uint32_t)((p->info.cols + cw - 1) / cw);
        const size_t need = (size_t)n_slabs * groups * 32u * slab;
        if (need > p->b_packed_bytes) {
            cudaFree(p->d_b_packed);
            p->d_b_packed = nullptr;
            p->b_packed_bytes = 0;
            B200_CUDA_TRY(cudaMalloc(&p->d_b_packed, need));
            p->b_packed_bytes = need;
        }
        const int grid = (int)std::min<size_t>((need / 16 + 255) / 256, (size_t)p->n_sms * 16);
        if (tf32)
            pack_b_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint8_t *>(d_B), ldb * esz, (uint32_t)p->info.cols,
                                                          (uint32_t)n, slab, n_slabs, groups, static_cast<uint8_t *>(p->d_b_packed));
        else
            pack_b_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint8_t *>(d_B), ldb * esz, (uint32_t)p->info.cols,
                                                           (uint32_t)n, slab, n_slabs, groups, static_cast<uint8_t *>(p->d_b_packed));
        B200_CUDA_TRY(cudaGetLastError());
        prm.b_packed = static_cast<const uint8_t *>(p->d_b_packed);
        prm.b_groups = groups;
    }
    prm.sched_counter = p->d_status + 1;
    prm.C = d_C;
    prm.ldc = ldc;
    prm.rows = (uint32_t)p->info.rows;
    prm.cols = (uint32_t)p->info.cols;
    prm.n = (uint32_t)n;
    prm.eff_row_windows = (uint32_t)fmt.eff;
    prm.c_is_half = c_dtype == B200SPMM_C_F16;
    prm.status = p->d_status;
    prm.wait_limit_ns = p->wait_limit_ns;
    prm.starve_bytes = p->starve_gathers ? 16u : 0u;
#ifdef B200SPMM_PROFILE
    if (const char *dbg = std::getenv("B200SPMM_DEBUG")) prm.debug = (uint32_t)std::atoi(dbg);  // results invalid
    if (!g_prof) cudaMalloc(&g_prof, 1024 * 32 * 8);
    cudaMemsetAsync(g_prof, 0, 1024 * 32 * 8, stream);
    prm.prof = g_prof;
#endif
    if (pair) return tf32 ? launch_pair_one<true>(p, prm, stream) : launch_pair_one<false>(p, prm, stream);
    if (n <= 128) return tf32 ? launch_tall_one<true, 128>(p, prm, stream) : launch_tall_one<false, 128>(p, prm, stream);
    return tf32 ? launch_tall_one<true, 256>(p, prm, stream) : launch_tall_one<false, 256>(p, prm, stream);
}

// Builds the super-window copy of the matrix when it pays.  The 16-row kernel spends about 100 SM
// clocks per tile and 128 features whatever the tile holds; the super-window kernel about 70 per
// 128-row tile and 128 features.  So the merge pays when it leaves fewer than ~0.7 of the tiles -
// i.e. when the parts of a super-window share most of their columns (a pruned weight matrix: 0.15;
// a power-law graph: ~0.9, stays with 16 rows).  B200SPMM_WINDOW=16 / 128 overrides the choice.
int plan_build_tall(b200spmm_plan *p, const uint32_t *h_rowOffset, const uint32_t *h_rowIdx) {
    const auto &info = p->info;
    if (!info.total_tiles || env_is("B200SPMM_WINDOW", "16")) return B200SPMM_OK;
    const bool want_pair = env_is("B200SPMM_WINDOW", "256");
    p->tall_forced = env_is("B200SPMM_WINDOW", "128") || want_pair;
    if (!p->tall_forced) {
        double ratio = 1.0;
        uint64_t n_super = 0;
        int st = estimate_tall_tile_ratio(info, h_rowOffset, h_rowIdx, p->d_tcA2B, kTallRows, 48, &ratio, &n_super);
        if (st != B200SPMM_OK) return st;
        // fewer super-windows than SMs / 16 can never fill the GPU, however wide B is
        if (ratio > 0.7 || n_super * 16 < (uint64_t)p->n_sms) return B200SPMM_OK;
    }
    int st = build_tall_device(info, h_rowOffset, h_rowIdx, p->d_rowOffset, p->d_tcA2B, p->d_data, p->d_rowIdx, kTallRows, &p->tall);
    if (st == B200SPMM_ERR_UNSUPPORTED) return B200SPMM_OK;  // too many tiles for 32-bit offsets: 16-row kernel
    if (st != B200SPMM_OK || !p->tall.tiles) return st;
    // The pair kernel does twice the work per tile: it pays when a 256-row window has (about) the column
    // list of its halves, i.e. half the tiles.  B200SPMM_WINDOW=256 forces it, =128 keeps it out.
    if (!env_is("B200SPMM_WINDOW", "128")) {
        st = info.dtype == B200SPMM_TF32 ? pair_max_clusters<true>(&p->pair_clusters) : pair_max_clusters<false>(&p->pair_clusters);
        if (st != B200SPMM_OK) return st;
        if (p->pair_clusters > 0) {
            st = build_tall_device(info, h_rowOffset, h_rowIdx, p->d_rowOffset, p->d_tcA2B, p->d_data, p->d_rowIdx, kPairRows, &p->pair);
            if (st != B200SPMM_OK && st != B200SPMM_ERR_UNSUPPORTED) return st;
            if (!want_pair && (double)p->pair.tiles > 0.55 * (double)p->tall.tiles) free_tall(&p->pair);
        }
    }
    // how many tiles name one aligned row group of B (sampled on the host: every 16th tile's list ends)
    {
        const uint64_t cw = (uint64_t)info.col_window, step = 16, n_probe = (p->tall.tiles + step - 1) / step;
        std::vector<uint32_t> probe(n_probe * 2);
        // first and last entry of every 16th tile's column list: two strided copies
        B200_CUDA_TRY(cudaMemcpy2D(probe.data(), 8, p->tall.d_tcA2B, step * cw * 4, 4, n_probe, cudaMemcpyDeviceToHost));
        B200_CUDA_TRY(cudaMemcpy2D(probe.data() + 1, 8, p->tall.d_tcA2B + (cw - 1), step * cw * 4, 4, n_probe, cudaMemcpyDeviceToHost));
        uint64_t aligned = 0;
        for (uint64_t i = 0; i < n_probe; ++i)
            aligned += (probe[2 * i] % cw == 0 && probe[2 * i + 1] - probe[2 * i] == cw - 1) ? 1 : 0;
        p->tall_pack_b = aligned * 2 >= n_probe && !env_is("B200SPMM_PACK_B", "0");
    }
    return B200SPMM_OK;
}

// Gives the plan its tile image.  Called last in plan_finish: everything that reads the tiles in the
// reference's layout (compression, the super-window merge) has run by then.
int plan_build_tile_image(b200spmm_plan *p) {
    const uint64_t n_rows = p->info.total_tiles * (uint64_t)kRowWindow;
    if (!n_rows || p->comp.tcBit) return B200SPMM_OK;  // compressed tiles are expanded in the kernel
    void *dst = p->d_data;
    if (!p->owns_format) {
        if (cudaMalloc(&dst, n_rows * 32) != cudaSuccess) {  // no room for a copy: the tiled loads still work
            cudaGetLastError();
            return B200SPMM_OK;
        }
        p->image_is_copy = true;
    }
    const int grid = (int)std::min<uint64_t>((n_rows + 255) / 256, 148 * 16);
    tileimage::swizzle_tiles_kernel<<<grid, 256>>>(static_cast<const uint4 *>(p->d_data), static_cast<uint4 *>(dst), n_rows);
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaDeviceSynchronize());
    p->d_tiles_image = dst;
    return B200SPMM_OK;
}

int plan_finish(b200spmm_plan *p, const uint32_t *h_rowOffset, const uint32_t *h_rowIdx, int n_ctas) {
    const auto &info = p->info;
    if (info.row_window != kRowWindow) return B200SPMM_ERR_UNSUPPORTED;
    const int cw = info.dtype == B200SPMM_F16 ? 16 : 8;
    if (info.col_window != cw) return B200SPMM_ERR_UNSUPPORTED;
    if (info.total_tiles * (uint64_t)kRowWindow >= 0x7FFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;  // TMA row coordinate
    cudaDeviceProp prop;
    B200_CUDA_TRY(cudaGetDeviceProperties(&prop, p->device));
    if (prop.major != 10) return B200SPMM_ERR_NO_DEVICE;
    p->n_sms = prop.multiProcessorCount;
    auto upload = [](auto **dst, const auto &v) -> int {
        using T = typename std::remove_reference<decltype(v)>::type::value_type;
        B200_CUDA_TRY(cudaMalloc(dst, std::max<size_t>(v.size() * sizeof(T), 16)));
        if (!v.empty()) B200_CUDA_TRY(cudaMemcpy(*dst, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
        return B200SPMM_OK;
    };
    {
        b200spmm_plan::Sched &ps = p->sched;
        ps.n_ctas = n_ctas > 0 ? n_ctas : prop.multiProcessorCount * kCtasPerSm;
        // Several chunks per CTA, taken from all over the matrix, even out regions whose tiles
        // cost more than the schedule's model says; a chunk stays long enough (512 tiles or
        // more) for the hand-over at its start not to matter.
        const uint64_t per_cta = info.total_tiles / (uint64_t)ps.n_ctas;
        const int chunks_per_cta = (int)std::min<uint64_t>(kMaxChunksPerCta, std::max<uint64_t>(1, per_cta / 512));
        ps.n_chunks = (uint32_t)(ps.n_ctas * chunks_per_cta);
        TileSchedule sc;
        build_tile_schedule(h_rowOffset, info.eff_row_windows, (int)ps.n_chunks, /*allow_split=*/true, &sc);
        std::vector<SplitWindow> splits;
        for (const auto &sp : sc.splits) splits.push_back(SplitWindow{sp.window, sp.piece_begin, sp.piece_end});
        int st_up = upload(&ps.d_tile, sc.tile);
        if (st_up == B200SPMM_OK) st_up = upload(&ps.d_wfirst, sc.wfirst);
        if (st_up == B200SPMM_OK) st_up = upload(&ps.d_wlast, sc.wlast);
        if (st_up == B200SPMM_OK) st_up = upload(&ps.d_head_slot, sc.head_slot);
        if (st_up == B200SPMM_OK) st_up = upload(&ps.d_tail_slot, sc.tail_slot);
        if (st_up == B200SPMM_OK) st_up = upload(&ps.d_splits, splits);
        if (st_up == B200SPMM_OK) st_up = upload(&ps.d_piece_slots, sc.piece_slots);
        if (st_up != B200SPMM_OK) return st_up;
        ps.n_splits = (uint32_t)splits.size();
        ps.n_slots = sc.n_slots;
        RowBands bands;  // only schedules with many chunks are worth launching in bands
        build_row_bands(sc, h_rowIdx, info.rows, ps.n_chunks >= (uint32_t)ps.n_ctas * 8u ? kRowBands : 1u, &bands);
        ps.band_chunk = bands.chunk;
        ps.band_row = bands.row;
        ps.band_split = bands.split;
    }
    // status word, then the two counters of the chunk hand-out (the kernel leaves them at zero)
    B200_CUDA_TRY(cudaMalloc(&p->d_status, 4 * sizeof(uint32_t)));
    B200_CUDA_TRY(cudaMemset(p->d_status, 0, 4 * sizeof(uint32_t)));
    {
        int st = encode_tile_map(p);
        if (st != B200SPMM_OK) return st;
    }
    // On request (B200SPMM_TILES=bitmap) the kernels stream the tiles in compressed form - bitmap +
    // stored values, expanded by the producer warps - instead of the dense 512-byte tiles; both
    // give the same C bit for bit.  The compressed form moves an eighth of the tile bytes at a
    // few per cent fill but costs the producer warps more instructions per tile than they can
    // spare today, so dense tiles are the default.
    p->gather_cpasync = env_is("B200SPMM_GATHER", "cpasync");
    p->host_split = !env_is("B200SPMM_HOST_SPLIT", "0");
    if (info.total_tiles && env_is("B200SPMM_TILES", "bitmap")) {
        int st = compress_tiles_device(p->d_data, info.total_tiles, info.dtype, &p->comp);
        if (st != B200SPMM_OK) return st;
    }
    // B200SPMM_TILES=entries (fp16): the kernels stream the tiles as records of 32 (position, value) words - a
    // quarter of the dense bytes - which a producer warp expands with two stores per lane; tiles with more than
    // 32 entries still come from the dense image.  Same C bit for bit.
    if (info.total_tiles && info.dtype == B200SPMM_F16 && env_is("B200SPMM_TILES", "entries")) {
        B200_CUDA_TRY(cudaMalloc(&p->d_tile_entries, info.total_tiles * 128));
        unsigned long long *d_count = nullptr;
        B200_CUDA_TRY(cudaMalloc(&d_count, 8));
        B200_CUDA_TRY(cudaMemset(d_count, 0, 8));
        const int grid = (int)std::min<uint64_t>((info.total_tiles + 7) / 8, (uint64_t)p->n_sms * 32);
        tileimage::tile_entries_kernel<<<grid, 256>>>(static_cast<const uint16_t *>(p->d_data), info.total_tiles, p->d_tile_entries, d_count);
        cudaError_t e = cudaGetLastError();
        unsigned long long n_dense = 0;
        if (e == cudaSuccess) e = cudaMemcpy(&n_dense, d_count, 8, cudaMemcpyDeviceToHost);
        cudaFree(d_count);
        B200_CUDA_TRY(e);
        p->entry_dense_tiles = n_dense;
    }
    if (n_ctas <= 0 && !p->comp.tcBit) {  // an explicit CTA count or compressed tiles ask for the 16-row kernel
        int st = plan_build_tall(p, h_rowOffset, h_rowIdx);
        if (st != B200SPMM_OK) return st;
    }
    return plan_build_tile_image(p);
}

}  // namespace

// ------------------------------------------------------------------ allocation-free launch path
namespace noalloc {
//
// Working memory of b200spmm_spmm_noalloc: the schedule tables (tile cuts, first and last window
// per CTA) and the kernel status word.  It is part of the library image, so every GPU that loads
// the library holds these 16 KiB until the process exits and no call ever has to allocate them.
constexpr int kNoAllocMaxCtas = 1024;
constexpr int kNoAllocTile = 0;                                  // [kNoAllocMaxCtas + 1]
constexpr int kNoAllocWfirst = kNoAllocTile + kNoAllocMaxCtas + 1;  // [kNoAllocMaxCtas]
constexpr int kNoAllocWlast = kNoAllocWfirst + kNoAllocMaxCtas;     // [kNoAllocMaxCtas]
constexpr int kNoAllocStatusWord = kNoAllocWlast + kNoAllocMaxCtas;
static __device__ __align__(256) uint32_t g_noalloc_scratch[4096];

// Cuts of the effective row windows over n_ctas CTAs by the same cost model as the host
// scheduler, always on window boundaries (no window is shared between CTAs, so no partial-result
// slots are needed).  One block; also clears the status word.
__global__ void noalloc_schedule_kernel(const uint32_t *__restrict__ rowOffset, uint32_t eff, int n_ctas,
                                        uint32_t *__restrict__ scratch) {
    __shared__ uint32_t cut[kNoAllocMaxCtas + 1];
    if (threadIdx.x == 0) scratch[kNoAllocStatusWord] = 0;
    auto cost = [&](uint64_t w) { return (uint64_t)rowOffset[w] + kWindowCharge * w; };
    const uint64_t total = eff ? cost(eff) : 0;
    for (int c = (int)threadIdx.x; c <= n_ctas; c += (int)blockDim.x) {
        uint64_t lo = 0, hi = eff;
        if (c == n_ctas) {
            lo = eff;
        } else if (c > 0) {
            const uint64_t target = total * (uint64_t)c / (uint64_t)n_ctas;
            while (lo < hi) {
                const uint64_t mid = (lo + hi) / 2;
                if (cost(mid) < target) lo = mid + 1; else hi = mid;
            }
        }
        cut[c] = (uint32_t)lo;
        scratch[kNoAllocTile + c] = rowOffset[lo];
    }
    __syncthreads();
    for (int c = (int)threadIdx.x; c < n_ctas; c += (int)blockDim.x) {
        scratch[kNoAllocWfirst + c] = cut[c];
        scratch[kNoAllocWlast + c] = cut[c + 1] > cut[c] ? cut[c + 1] - 1 : cut[c];
    }
}

// Device address of g_noalloc_scratch on `device`, looked up on first use.  The name of a
// __device__ array is only a host-side handle; kernels must be given this address.
int noalloc_scratch_address(int device, uint32_t **out) {
    constexpr int kMaxDevices = 64;
    static uint32_t *cache[kMaxDevices] = {};
    static std::mutex lock;
    if (device < 0 || device >= kMaxDevices) return B200SPMM_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> guard(lock);
    if (!cache[device]) {
        void *ptr = nullptr;
        B200_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));  // `device` is current (set by the caller)
        cache[device] = static_cast<uint32_t *>(ptr);
    }
    *out = cache[device];
    return B200SPMM_OK;
}

}  // namespace noalloc
using namespace noalloc;

#ifdef B200SPMM_PROFILE
extern "C" int b200spmm_debug_read_profile(unsigned long long *out, int n_ctas) {
    return cudaMemcpy(out, g_prof, (size_t)n_ctas * 32 * 8, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -5;
}
#endif

extern "C" {

const char *b200spmm_status_string(int status) {
    switch (status) {
        case B200SPMM_OK: return "ok";
        case B200SPMM_ERR_INVALID_ARG: return "invalid argument";
        case B200SPMM_ERR_BAD_CSR: return "malformed CSR (row_ptr not monotone, wrong nnz, or column out of range)";
        case B200SPMM_ERR_UNSUPPORTED: return "shape, size or alignment not supported";
        case B200SPMM_ERR_NO_MEMORY: return "host allocation failed";
        case B200SPMM_ERR_CUDA: return "CUDA call failed (see b200spmm_last_cuda_error)";
        case B200SPMM_ERR_NO_DEVICE: return "no sm_100 device available";
        case B200SPMM_ERR_DEVICE_TIMEOUT: return "a bounded wait inside the kernel ran out";
        default: return "unknown status";
    }
}

const char *b200spmm_last_cuda_error(void) { return g_last_static_error ? g_last_static_error : g_last_cuda_error.c_str(); }

int b200spmm_version(void) { return 100; }

int b200spmm_csr2btcf_nobitmap(uint64_t rows, uint64_t cols, uint64_t nnz, const uint32_t *row_ptr,
                               const uint32_t *col_idx, const void *values, int dtype, int row_window,
                               int col_window, int n_threads, b200spmm_btcf_t **out) {
    if (!out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    b200spmm_btcf *h = new (std::nothrow) b200spmm_btcf();
    if (!h) return B200SPMM_ERR_NO_MEMORY;
    int st = convert_csr_to_btcf(rows, cols, nnz, row_ptr, col_idx, values, dtype, row_window, col_window, n_threads, &h->f);
    if (st != B200SPMM_OK) {
        delete h;
        return st;
    }
    *out = h;
    return B200SPMM_OK;
}

int b200spmm_btcf_transpose_tiles(b200spmm_btcf_t *f) {
    if (!f) return B200SPMM_ERR_INVALID_ARG;
    transpose_tiles(&f->f);
    return B200SPMM_OK;
}

int b200spmm_btcf_tiles_col_major(const b200spmm_btcf_t *f) { return f && f->f.col_major_tiles ? 1 : 0; }

int b200spmm_btcf_rewindow(const b200spmm_btcf_info_t *info, const uint32_t *rowOffset, const uint32_t *tcA2B,
                           const void *data, const uint32_t *rowIdx, int row_window, int n_threads,
                           b200spmm_btcf_t **out) {
    if (!out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    if (!info || !rowOffset) return B200SPMM_ERR_INVALID_ARG;
    if (rowOffset[info->eff_row_windows] != info->total_tiles) return B200SPMM_ERR_INVALID_ARG;
    b200spmm_btcf *h = new (std::nothrow) b200spmm_btcf();
    if (!h) return B200SPMM_ERR_NO_MEMORY;
    int st = rewindow_btcf(info->rows, info->cols, info->nnzs, info->dtype, info->row_window, info->col_window,
                           info->eff_row_windows, rowOffset, tcA2B, data, rowIdx, row_window, n_threads, &h->f);
    if (st != B200SPMM_OK) {
        delete h;
        return st;
    }
    *out = h;
    return B200SPMM_OK;
}

int b200spmm_btcf_info(const b200spmm_btcf_t *h, b200spmm_btcf_info_t *info) {
    if (!h || !info) return B200SPMM_ERR_INVALID_ARG;
    const Btcf &f = h->f;
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
    return B200SPMM_OK;
}

const uint32_t *b200spmm_btcf_rowOffset(const b200spmm_btcf_t *h) { return h ? h->f.rowOffset.data() : nullptr; }
const uint32_t *b200spmm_btcf_tcA2B(const b200spmm_btcf_t *h) { return h ? h->f.tcA2B.data() : nullptr; }
const void *b200spmm_btcf_data(const b200spmm_btcf_t *h) { return h ? h->f.data.data() : nullptr; }
const uint32_t *b200spmm_btcf_rowIdx(const b200spmm_btcf_t *h) { return h ? h->f.rowIdx.data() : nullptr; }
void b200spmm_btcf_destroy(b200spmm_btcf_t *h) { delete h; }

int b200spmm_shard_rows(uint64_t rows, const uint32_t *row_ptr, int row_window, int parts, uint64_t *row_begin) {
    return shard_rows(rows, row_ptr, row_window, parts, 0, row_begin);
}

int b200spmm_shard_rows_weighted(uint64_t rows, const uint32_t *row_ptr, int row_window, int parts,
                                 uint64_t row_charge, uint64_t *row_begin) {
    return shard_rows(rows, row_ptr, row_window, parts, row_charge, row_begin);
}

int b200spmm_allgather_plan(const uint64_t *cut, int n_parts, uint64_t *even_part, uint64_t *pieces) {
    if (!cut || !even_part || n_parts < 1 || (n_parts > 1 && !pieces)) return B200SPMM_ERR_INVALID_ARG;
    for (int d = 0; d < n_parts; ++d)
        if (cut[d + 1] < cut[d]) return B200SPMM_ERR_INVALID_ARG;
    *even_part = exchange_even_part(cut, n_parts);
    for (int d = 0; d < n_parts; ++d)
        for (int step = 1; step < n_parts; ++step) {
            uint64_t *out = pieces + ((size_t)d * (size_t)(n_parts - 1) + (size_t)(step - 1)) * 10;
            int to = 0, from = 0;
            exchange_pieces(cut, n_parts, *even_part, d, step, &to, &from, out + 2);
            out[0] = (uint64_t)to;
            out[1] = (uint64_t)from;
        }
    return B200SPMM_OK;
}

int b200spmm_build_schedule(const uint32_t *rowOffset, uint64_t eff_row_windows, int n_ctas, uint32_t *cta_window) {
    if (!rowOffset || !cta_window || n_ctas < 1) return B200SPMM_ERR_INVALID_ARG;
    std::vector<uint32_t> cuts;
    build_cta_schedule(rowOffset, eff_row_windows, n_ctas, &cuts);
    std::memcpy(cta_window, cuts.data(), cuts.size() * sizeof(uint32_t));
    return B200SPMM_OK;
}

int b200spmm_build_tile_schedule(const uint32_t *rowOffset, uint64_t eff_row_windows, int n_ctas, uint32_t *cta_tile,
                                 uint32_t *cta_wfirst, uint32_t *cta_wlast, uint32_t *slot_window) {
    if (!rowOffset || !cta_tile || !cta_wfirst || !cta_wlast || !slot_window || n_ctas < 1) return B200SPMM_ERR_INVALID_ARG;
    TileSchedule sc;
    build_tile_schedule(rowOffset, eff_row_windows, n_ctas, /*allow_split=*/true, &sc);
    std::memcpy(cta_tile, sc.tile.data(), sc.tile.size() * sizeof(uint32_t));
    std::memcpy(cta_wfirst, sc.wfirst.data(), sc.wfirst.size() * sizeof(uint32_t));
    std::memcpy(cta_wlast, sc.wlast.data(), sc.wlast.size() * sizeof(uint32_t));
    for (int c = 0; c < n_ctas; ++c) {
        slot_window[2 * c] = sc.head_slot[c] != kNoSlot ? sc.wfirst[c] : 0xFFFFFFFFu;
        slot_window[2 * c + 1] = sc.tail_slot[c] != kNoSlot ? sc.wlast[c] : 0xFFFFFFFFu;
    }
    return B200SPMM_OK;
}

int b200spmm_build_row_bands(const uint32_t *rowOffset, const uint32_t *rowIdx, uint64_t eff_row_windows, uint64_t rows,
                             int n_parts, int max_bands, uint32_t *band_chunk, uint64_t *band_row, int *n_bands) {
    if (!rowOffset || !band_chunk || !band_row || !n_bands || n_parts < 1 || max_bands < 1 || (eff_row_windows && !rowIdx))
        return B200SPMM_ERR_INVALID_ARG;
    TileSchedule sc;
    build_tile_schedule(rowOffset, eff_row_windows, n_parts, /*allow_split=*/true, &sc);
    RowBands bands;
    build_row_bands(sc, rowIdx, rows, (uint32_t)max_bands, &bands);
    *n_bands = (int)bands.chunk.size() - 1;
    std::memcpy(band_chunk, bands.chunk.data(), bands.chunk.size() * sizeof(uint32_t));
    std::memcpy(band_row, bands.row.data(), bands.row.size() * sizeof(uint64_t));
    return B200SPMM_OK;
}

void b200spmm_plan_destroy(b200spmm_plan_t *p) {
    if (!p) return;
    cudaSetDevice(p->device);
    if (p->owns_format) {
        cudaFree(p->d_rowOffset);
        cudaFree(p->d_tcA2B);
        cudaFree(p->d_rowIdx);
        cudaFree(p->d_data);
    }
    {
        auto &ps = p->sched;
        cudaFree(ps.d_tile);
        cudaFree(ps.d_wfirst);
        cudaFree(ps.d_wlast);
        cudaFree(ps.d_head_slot);
        cudaFree(ps.d_tail_slot);
        cudaFree(ps.d_splits);
        cudaFree(ps.d_piece_slots);
    }
    free_compressed_tiles(&p->comp);
    cudaFree(p->d_tile_entries);
    free_tall(&p->tall);
    free_tall(&p->pair);
    cudaFree(p->d_b_packed);
    if (p->image_is_copy) cudaFree(p->d_tiles_image);
    for (cudaEvent_t e : p->band_done) cudaEventDestroy(e);
    if (p->copy_stream) cudaStreamDestroy(p->copy_stream);
    if (p->upload_stream) cudaStreamDestroy(p->upload_stream);
    for (cudaEvent_t e : p->half_up)
        if (e) cudaEventDestroy(e);
    cudaFree(p->d_partial);
    cudaFree(p->d_status);
    cudaFree(p->d_B);
    cudaFree(p->d_C);
    delete p;
}

int b200spmm_plan_create(const b200spmm_btcf_t *h, int device, int n_ctas, b200spmm_plan_t **out) {
    if (!h || !out) return B200SPMM_ERR_INVALID_ARG;
    *out = nullptr;
    if (h->f.col_major_tiles) {  // the kernels read row-major tiles (the reference's default build)
        set_last_error_static("tiles are stored column-major: b200spmm_btcf_transpose_tiles brings them back");
        return B200SPMM_ERR_UNSUPPORTED;
    }
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev) {
        cudaGetLastError();
        return B200SPMM_ERR_NO_DEVICE;
    }
    B200_CUDA_TRY(cudaSetDevice(device));
    b200spmm_plan *p = new (std::nothrow) b200spmm_plan();
    if (!p) return B200SPMM_ERR_NO_MEMORY;
    p->device = device;
    p->owns_format = true;
    b200spmm_btcf_info(h, &p->info);
    const Btcf &f = h->f;
    auto upload = [&](void **dst, const void *src, size_t bytes) -> int {
        B200_CUDA_TRY(cudaMalloc(dst, std::max<size_t>(bytes, 16)));
        if (bytes) B200_CUDA_TRY(cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice));
        return B200SPMM_OK;
    };
    int st = upload((void **)&p->d_rowOffset, f.rowOffset.data(), f.rowOffset.size() * 4);
    if (st == B200SPMM_OK) st = upload((void **)&p->d_tcA2B, f.tcA2B.data(), f.tcA2B.size() * 4);
    if (st == B200SPMM_OK) st = upload((void **)&p->d_rowIdx, f.rowIdx.data(), f.rowIdx.size() * 4);
    if (st == B200SPMM_OK) st = upload(&p->d_data, f.data.data(), f.data.size());
    if (st == B200SPMM_OK) st = plan_finish(p, f.rowOffset.data(), f.rowIdx.data(), n_ctas);
    if (st != B200SPMM_OK) {
        b200spmm_plan_destroy(p);
        return st;
    }
    *out = p;
    return B200SPMM_OK;
}

int b200spmm_plan_create_device(const b200spmm_btcf_info_t *info, const uint32_t *d_rowOffset, const uint32_t *d_tcA2B,
                                const void *d_data, const uint32_t *d_rowIdx, int device, int n_ctas,
                                b200spmm_plan_t **out) {
    if (!info || !out || !d_rowOffset) return B200SPMM_ERR_INVALID_ARG;
    if (info->total_tiles && (!d_tcA2B || !d_data || !d_rowIdx)) return B200SPMM_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(d_data) & 15u) != 0) return B200SPMM_ERR_UNSUPPORTED;
    *out = nullptr;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev) {
        cudaGetLastError();
        return B200SPMM_ERR_NO_DEVICE;
    }
    B200_CUDA_TRY(cudaSetDevice(device));
    b200spmm_plan *p = new (std::nothrow) b200spmm_plan();
    if (!p) return B200SPMM_ERR_NO_MEMORY;
    p->device = device;
    p->owns_format = false;
    p->info = *info;
    p->d_rowOffset = const_cast<uint32_t *>(d_rowOffset);
    p->d_tcA2B = const_cast<uint32_t *>(d_tcA2B);
    p->d_rowIdx = const_cast<uint32_t *>(d_rowIdx);
    p->d_data = const_cast<void *>(d_data);
    std::vector<uint32_t> h_rowOffset(info->eff_row_windows + 1);
    int st = B200SPMM_OK;
    if (cudaMemcpy(h_rowOffset.data(), d_rowOffset, h_rowOffset.size() * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
        record_cuda_error(cudaGetLastError(), "cudaMemcpy(rowOffset)");
        st = B200SPMM_ERR_CUDA;
    }
    if (st == B200SPMM_OK && h_rowOffset[info->eff_row_windows] != info->total_tiles) st = B200SPMM_ERR_INVALID_ARG;
    std::vector<uint32_t> h_rowIdx(info->eff_row_windows);
    if (st == B200SPMM_OK && info->eff_row_windows &&
        cudaMemcpy(h_rowIdx.data(), d_rowIdx, h_rowIdx.size() * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
        record_cuda_error(cudaGetLastError(), "cudaMemcpy(rowIdx)");
        st = B200SPMM_ERR_CUDA;
    }
    if (st == B200SPMM_OK) st = plan_finish(p, h_rowOffset.data(), h_rowIdx.data(), n_ctas);
    if (st != B200SPMM_OK) {
        b200spmm_plan_destroy(p);
        return st;
    }
    *out = p;
    return B200SPMM_OK;
}

int b200spmm_plan_info(const b200spmm_plan_t *p, b200spmm_btcf_info_t *info) {
    if (!p || !info) return B200SPMM_ERR_INVALID_ARG;
    *info = p->info;
    return B200SPMM_OK;
}

static int super_window_info(const b200spmm_plan_t *p, const TallFormat &f, int rows, b200spmm_btcf_info_t *info) {
    if (!p || !info) return B200SPMM_ERR_INVALID_ARG;
    *info = p->info;
    info->row_window = f.tiles ? rows : 0;
    info->total_row_windows = (p->info.rows + rows - 1) / rows;
    info->eff_row_windows = f.eff;
    info->total_tiles = f.tiles;
    return B200SPMM_OK;
}

static int super_window_copy_to_host(const b200spmm_plan_t *p, const TallFormat &f, uint32_t *rowOffset, uint32_t *tcA2B,
                                     void *data, uint32_t *rowIdx) {
    if (!p || !rowOffset || !tcA2B || !data || !rowIdx) return B200SPMM_ERR_INVALID_ARG;
    if (!f.tiles) return B200SPMM_ERR_UNSUPPORTED;
    B200_CUDA_TRY(cudaSetDevice(p->device));
    const uint64_t cw = (uint64_t)p->info.col_window, parts = f.rows / 128u;
    B200_CUDA_TRY(cudaMemcpy(rowOffset, f.d_rowOffset, (f.eff + 1) * 4, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(rowIdx, f.d_rowIdx, f.eff * 4, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(tcA2B, f.d_tcA2B, f.tiles * cw * 4, cudaMemcpyDeviceToHost));
    // The device copy holds 128-row images as they lie in shared memory (the halves of a row swapped when
    // row / 4 is odd), for 256-row windows per window first rows 0-127 of all its tiles, then rows 128-255:
    // put the halves back and the images where the converter would have them.
    std::vector<uint8_t> img(f.tiles * parts * 4096);
    B200_CUDA_TRY(cudaMemcpy(img.data(), f.d_data, img.size(), cudaMemcpyDeviceToHost));
    uint8_t *bytes = static_cast<uint8_t *>(data);
    for (uint64_t g = 0; g < f.eff; ++g) {
        const uint64_t first = rowOffset[g], n_tiles = rowOffset[g + 1] - first;
        for (uint64_t part = 0; part < parts; ++part)
            for (uint64_t t = 0; t < n_tiles; ++t) {
                const uint8_t *src = img.data() + (first * parts + part * n_tiles + t) * 4096;
                uint8_t *dst = bytes + ((first + t) * parts + part) * 4096;
                for (uint32_t r = 0; r < 128; ++r) {
                    const uint32_t flip = (r >> 2) & 1u;
                    std::memcpy(dst + r * 32, src + r * 32 + (flip ? 16 : 0), 16);
                    std::memcpy(dst + r * 32 + 16, src + r * 32 + (flip ? 0 : 16), 16);
                }
            }
    }
    return B200SPMM_OK;
}

int b200spmm_plan_tall_info(const b200spmm_plan_t *p, b200spmm_btcf_info_t *info) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    return super_window_info(p, p->tall, kTallRows, info);
}
int b200spmm_plan_tall_copy_to_host(const b200spmm_plan_t *p, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                                    uint32_t *rowIdx) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    return super_window_copy_to_host(p, p->tall, rowOffset, tcA2B, data, rowIdx);
}
int b200spmm_plan_pair_info(const b200spmm_plan_t *p, b200spmm_btcf_info_t *info) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    return super_window_info(p, p->pair, kPairRows, info);
}
int b200spmm_plan_pair_copy_to_host(const b200spmm_plan_t *p, uint32_t *rowOffset, uint32_t *tcA2B, void *data,
                                    uint32_t *rowIdx) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    return super_window_copy_to_host(p, p->pair, rowOffset, tcA2B, data, rowIdx);
}

int b200spmm_plan_launch_info(const b200spmm_plan_t *p, b200spmm_launch_info_t *info) {
    if (!p || !info) return B200SPMM_ERR_INVALID_ARG;
    *info = p->last;
    return B200SPMM_OK;
}

}  // extern "C"

namespace {

// The product, or one band of it (band < 0: every chunk; otherwise the chunks, rows and split
// windows of that band of the schedule the launch selects - see b200spmm_plan::Sched).
int spmm_launch(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc, int c_dtype,
                void *stream_v, int band) {
    if (!p || !d_B || !d_C || n <= 0 || ldb < n || ldc < n) return B200SPMM_ERR_INVALID_ARG;
    if (c_dtype != B200SPMM_C_F32 && c_dtype != B200SPMM_C_F16) return B200SPMM_ERR_INVALID_ARG;
    const int esz = p->info.elt_size, csz = c_dtype == B200SPMM_C_F32 ? 4 : 2;
    if (n % 8 || n > 0x7FFFFFFF || p->info.cols > 0x7FFFFFFFull) return B200SPMM_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(d_B) & 15u) || (reinterpret_cast<uintptr_t>(d_C) & 15u)) return B200SPMM_ERR_UNSUPPORTED;
    if ((ldb * esz) % 16 || (ldc * csz) % 16) return B200SPMM_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    B200_CUDA_TRY(cudaSetDevice(p->device));
    p->last = b200spmm_launch_info_t{};
    if (p->info.eff_row_windows == 0) {  // nothing stored: C is all zeros
        B200_CUDA_TRY(cudaMemset2DAsync(d_C, (size_t)ldc * csz, 0, (size_t)n * csz, p->info.rows, stream));
        return B200SPMM_OK;
    }
    if (band < 0 && use_tall(p, n)) return launch_tall(p, d_B, ldb, n, d_C, ldc, c_dtype, stream);
    SpmmParams prm{};
    prm.rowOffset = p->d_rowOffset;
    prm.tcA2B = p->d_tcA2B;
    prm.rowIdx = p->d_rowIdx;
    const b200spmm_plan::Sched &sc = p->sched;
    p->launch_sched = &sc;
    prm.chunk_tile = sc.d_tile;
    prm.chunk_wfirst = sc.d_wfirst;
    prm.chunk_wlast = sc.d_wlast;
    prm.chunk_head_slot = sc.d_head_slot;
    prm.chunk_tail_slot = sc.d_tail_slot;
    if (band >= 0 && (size_t)band + 1 >= sc.band_chunk.size()) return B200SPMM_ERR_INVALID_ARG;
    prm.chunk_begin = band < 0 ? 0u : sc.band_chunk[band];
    prm.chunk_end = band < 0 ? sc.n_chunks : sc.band_chunk[band + 1];
    const uint32_t split_begin = band < 0 ? 0u : sc.band_split[band];
    const uint32_t split_end = band < 0 ? sc.n_splits : sc.band_split[band + 1];
    prm.sched_counter = sc.n_chunks > (uint32_t)sc.n_ctas ? p->d_status + 1 : nullptr;
    if (sc.n_slots) {  // slots for the pieces of windows that span chunks
        const size_t need = (size_t)sc.n_slots * kRowWindow * (size_t)n;
        if (need > p->partial_floats) {
            cudaFree(p->d_partial);
            p->d_partial = nullptr;
            p->partial_floats = 0;
            B200_CUDA_TRY(cudaMalloc(&p->d_partial, need * sizeof(float)));
            p->partial_floats = need;
        }
    }
    prm.partial = p->d_partial;
    prm.tiles_image = static_cast<const uint8_t *>(p->d_tiles_image);
    prm.total_tiles = (uint32_t)p->info.total_tiles;
    prm.B = d_B;
    prm.C = d_C;
    prm.ldb = ldb;
    prm.ldc = ldc;
    prm.rows = (uint32_t)p->info.rows;
    prm.cols = (uint32_t)p->info.cols;
    prm.n = (uint32_t)n;
    prm.eff_row_windows = (uint32_t)p->info.eff_row_windows;
    prm.c_is_half = c_dtype == B200SPMM_C_F16;
    prm.status = p->d_status;
    prm.wait_limit_ns = p->wait_limit_ns;
#ifdef B200SPMM_PROFILE
    if (!g_prof) cudaMalloc(&g_prof, 1024 * 32 * 8);
    cudaMemsetAsync(g_prof, 0, 1024 * 32 * 8, stream);
    prm.prof = g_prof;
    if (const char *dbg = std::getenv("B200SPMM_DEBUG")) prm.debug = (uint32_t)std::atoi(dbg);  // results invalid
#endif
    int st = p->info.dtype == B200SPMM_F16 ? launch_dtype<false>(p, prm, stream) : launch_dtype<true>(p, prm, stream);
    if (st != B200SPMM_OK || split_end == split_begin) return st;
    // windows shared out over several CTAs: sum their pieces
    spmm_fixup_kernel<<<split_end - split_begin, 256, 0, stream>>>(sc.d_splits + split_begin, sc.d_piece_slots, p->d_partial,
                                                                   p->d_rowIdx, d_C, ldc, prm.rows, prm.n, prm.c_is_half);
    B200_CUDA_TRY(cudaGetLastError());
    p->last.kernel_launches = 2;
    return B200SPMM_OK;
}

}  // namespace

extern "C" {

int b200spmm_spmm(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc, int c_dtype,
                  void *stream_v) {
    return spmm_launch(p, d_B, ldb, n, d_C, ldc, c_dtype, stream_v, -1);
}

int b200spmm_fp16_spmm(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc, int c_dtype,
                       void *stream) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    if (p->info.dtype != B200SPMM_F16) return B200SPMM_ERR_INVALID_ARG;
    return b200spmm_spmm(p, d_B, ldb, n, d_C, ldc, c_dtype, stream);
}

int b200spmm_tf32_spmm(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc, int c_dtype,
                       void *stream) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    if (p->info.dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    return b200spmm_spmm(p, d_B, ldb, n, d_C, ldc, c_dtype, stream);
}

int b200spmm_plan_sync(b200spmm_plan_t *p, void *stream_v) {
    if (!p) return B200SPMM_ERR_INVALID_ARG;
    B200_CUDA_TRY(cudaSetDevice(p->device));
    B200_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_v)));
    uint32_t status = 0;
    B200_CUDA_TRY(cudaMemcpy(&status, p->d_status, sizeof(status), cudaMemcpyDeviceToHost));
    if (status) {
        B200_CUDA_TRY(cudaMemset(p->d_status, 0, 4 * sizeof(uint32_t)));  // status and the hand-out counters
        return B200SPMM_ERR_DEVICE_TIMEOUT;
    }
    return B200SPMM_OK;
}

int b200spmm_spmm_host(b200spmm_plan_t *p, const void *h_B, int64_t n, void *h_C, int c_dtype) {
    if (!p || !h_B || !h_C || n <= 0) return B200SPMM_ERR_INVALID_ARG;
    if (c_dtype != B200SPMM_C_F32 && c_dtype != B200SPMM_C_F16) return B200SPMM_ERR_INVALID_ARG;
    B200_CUDA_TRY(cudaSetDevice(p->device));
    const size_t b_bytes = (size_t)p->info.cols * n * p->info.elt_size;
    const size_t c_bytes = (size_t)p->info.rows * n * (c_dtype == B200SPMM_C_F32 ? 4 : 2);
    if (b_bytes > p->d_B_bytes) {
        cudaFree(p->d_B);
        p->d_B = nullptr;
        p->d_B_bytes = 0;
        B200_CUDA_TRY(cudaMalloc(&p->d_B, b_bytes));
        p->d_B_bytes = b_bytes;
    }
    if (c_bytes > p->d_C_bytes) {
        cudaFree(p->d_C);
        p->d_C = nullptr;
        p->d_C_bytes = 0;
        B200_CUDA_TRY(cudaMalloc(&p->d_C, c_bytes));
        p->d_C_bytes = c_bytes;
    }
    const b200spmm_plan::Sched &sc = p->sched;
    const size_t bands = sc.band_chunk.size() > 1 && !use_tall(p, n) ? sc.band_chunk.size() - 1 : 1;
    if (bands == 1 || p->info.eff_row_windows == 0) {
        B200_CUDA_TRY(cudaMemcpyAsync(p->d_B, h_B, b_bytes, cudaMemcpyHostToDevice, nullptr));
        int st = b200spmm_spmm(p, p->d_B, n, n, p->d_C, n, c_dtype, nullptr);
        if (st != B200SPMM_OK) return st;
        B200_CUDA_TRY(cudaMemcpyAsync(h_C, p->d_C, c_bytes, cudaMemcpyDeviceToHost, nullptr));
        return b200spmm_plan_sync(p, nullptr);
    }
    // Large matrix: band after band on the compute stream; as soon as a band is done its rows of C
    // leave on a second stream while the next band is computed.
    //
    // Every row of C needs all rows of B, so the two copies of a step cannot overlap - except by
    // features: with the features cut in two halves, the first half of C goes out while the second
    // half of B comes in, and the host link carries both directions at once for the middle third of
    // the step.  Each half is a product of its own (B and C as views with the full leading dimension).
    const size_t esz = (size_t)p->info.elt_size, csz = c_dtype == B200SPMM_C_F32 ? 4 : 2;
    const int64_t n_first = n / 2;
    const bool halves = p->host_split && n % 16 == 0 && (size_t)n_first * esz >= 128;
    const int n_parts = halves ? 2 : 1;
    if (!p->copy_stream) B200_CUDA_TRY(cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking));
    if (halves && !p->upload_stream) {
        B200_CUDA_TRY(cudaStreamCreateWithFlags(&p->upload_stream, cudaStreamNonBlocking));
        for (cudaEvent_t &e : p->half_up) B200_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    while (p->band_done.size() < bands * (size_t)n_parts) {
        cudaEvent_t e;
        B200_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->band_done.push_back(e);
    }
    const size_t b_pitch = (size_t)n * esz, c_pitch = (size_t)n * csz;
    if (!halves) {
        B200_CUDA_TRY(cudaMemcpyAsync(p->d_B, h_B, b_bytes, cudaMemcpyHostToDevice, nullptr));
    } else {  // first half on the compute stream, the second one behind it on a stream of its own
        B200_CUDA_TRY(cudaMemcpy2DAsync(p->d_B, b_pitch, h_B, b_pitch, (size_t)n_first * esz, (size_t)p->info.cols,
                                        cudaMemcpyHostToDevice, nullptr));
        B200_CUDA_TRY(cudaEventRecord(p->half_up[0], nullptr));
        B200_CUDA_TRY(cudaStreamWaitEvent(p->upload_stream, p->half_up[0], 0));
        B200_CUDA_TRY(cudaMemcpy2DAsync(static_cast<char *>(p->d_B) + (size_t)n_first * esz, b_pitch,
                                        static_cast<const char *>(h_B) + (size_t)n_first * esz, b_pitch,
                                        (size_t)(n - n_first) * esz, (size_t)p->info.cols, cudaMemcpyHostToDevice, p->upload_stream));
        B200_CUDA_TRY(cudaEventRecord(p->half_up[1], p->upload_stream));
    }
    int64_t launches = 0;
    for (int part = 0; part < n_parts; ++part) {
        const int64_t f0 = part == 0 ? 0 : n_first, nf = halves ? (part == 0 ? n_first : n - n_first) : n;
        if (part == 1) B200_CUDA_TRY(cudaStreamWaitEvent(nullptr, p->half_up[1], 0));
        const char *b_part = static_cast<const char *>(p->d_B) + (size_t)f0 * esz;
        char *c_part = static_cast<char *>(p->d_C) + (size_t)f0 * csz;
        for (size_t k = 0; k < bands; ++k) {
            int st = spmm_launch(p, b_part, n, nf, c_part, n, c_dtype, nullptr, (int)k);
            if (st != B200SPMM_OK) return st;
            launches += p->last.kernel_launches;
            cudaEvent_t done = p->band_done[(size_t)part * bands + k];
            B200_CUDA_TRY(cudaEventRecord(done, nullptr));
            B200_CUDA_TRY(cudaStreamWaitEvent(p->copy_stream, done, 0));
            const uint64_t r0 = sc.band_row[k], r1 = sc.band_row[k + 1];
            if (r1 == r0) continue;
            B200_CUDA_TRY(cudaMemcpy2DAsync(static_cast<char *>(h_C) + r0 * c_pitch + (size_t)f0 * csz, c_pitch, c_part + r0 * c_pitch,
                                            c_pitch, (size_t)nf * csz, r1 - r0, cudaMemcpyDeviceToHost, p->copy_stream));
        }
    }
    p->last.kernel_launches = launches;
    B200_CUDA_TRY(cudaStreamSynchronize(p->copy_stream));
    return b200spmm_plan_sync(p, nullptr);
}

int b200spmm_bench(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc, int c_dtype,
                   int warmup, int runs, void *stream_v, float *total_ms) {
    if (!p || !total_ms || warmup < 0 || runs < 1) return B200SPMM_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    B200_CUDA_TRY(cudaSetDevice(p->device));
    for (int i = 0; i < warmup; ++i) {
        int st = b200spmm_spmm(p, d_B, ldb, n, d_C, ldc, c_dtype, stream_v);
        if (st != B200SPMM_OK) return st;
    }
    cudaEvent_t e0, e1;
    B200_CUDA_TRY(cudaEventCreate(&e0));
    B200_CUDA_TRY(cudaEventCreate(&e1));
    int st = B200SPMM_OK;
    cudaEventRecord(e0, stream);
    for (int i = 0; i < runs && st == B200SPMM_OK; ++i) st = b200spmm_spmm(p, d_B, ldb, n, d_C, ldc, c_dtype, stream_v);
    cudaEventRecord(e1, stream);
    if (st == B200SPMM_OK) st = b200spmm_plan_sync(p, stream_v);
    if (st == B200SPMM_OK && cudaEventElapsedTime(total_ms, e0, e1) != cudaSuccess) {
        record_cuda_error(cudaGetLastError(), "cudaEventElapsedTime");
        st = B200SPMM_ERR_CUDA;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return st;
}

/* Declared in b200_spmm_kat.h: the product launched so that its stage barriers can never complete. */
int b200spmm_kat_spmm_starved(b200spmm_plan_t *p, const void *d_B, int64_t ldb, int64_t n, void *d_C, int64_t ldc,
                              unsigned long long limit_ns, void *stream) {
    if (!p || limit_ns == 0 || limit_ns > kDeviceWaitLimitNs) return B200SPMM_ERR_INVALID_ARG;
    if (p->gather_cpasync || n * p->info.elt_size < 128) return B200SPMM_ERR_UNSUPPORTED;  // needs the TMA gathers
    p->starve_gathers = true;
    p->wait_limit_ns = limit_ns;
    p->tmap_b_ptr = nullptr;  // a map encoded for a normal launch must not be reused, nor this one later
    const int st = spmm_launch(p, d_B, ldb, n, d_C, ldc, B200SPMM_C_F32, stream, -1);
    p->starve_gathers = false;
    p->wait_limit_ns = kDeviceWaitLimitNs;
    p->tmap_b_ptr = nullptr;
    return st;
}

int b200spmm_spmm_noalloc_status(int device, void *stream_v) {
    B200_CUDA_TRY(cudaSetDevice(device));
    uint32_t *scratch = nullptr;
    int st = noalloc_scratch_address(device, &scratch);
    if (st != B200SPMM_OK) return st;
    B200_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_v)));
    uint32_t status = 0;  // a copy into a stack word: nothing is allocated
    B200_CUDA_TRY(cudaMemcpy(&status, scratch + kNoAllocStatusWord, sizeof(status), cudaMemcpyDeviceToHost));
    return (status & kDevStatusTimeout) ? B200SPMM_ERR_DEVICE_TIMEOUT : B200SPMM_OK;
}

int b200spmm_spmm_noalloc(const b200spmm_btcf_info_t *info, const uint32_t *d_rowOffset, const uint32_t *d_tcA2B,
                          const void *d_data, const uint32_t *d_rowIdx, const void *d_B, int64_t ldb, int64_t n,
                          void *d_C, int64_t ldc, int c_dtype, int device, int n_ctas, void *stream_v) {
    if (!info || !d_rowOffset || !d_B || !d_C || n <= 0 || ldb < n || ldc < n) return B200SPMM_ERR_INVALID_ARG;
    if (info->total_tiles && (!d_tcA2B || !d_data || !d_rowIdx)) return B200SPMM_ERR_INVALID_ARG;
    if (c_dtype != B200SPMM_C_F32 && c_dtype != B200SPMM_C_F16) return B200SPMM_ERR_INVALID_ARG;
    if (info->dtype != B200SPMM_F16 && info->dtype != B200SPMM_TF32) return B200SPMM_ERR_INVALID_ARG;
    if (info->row_window != kRowWindow || info->col_window != (info->dtype == B200SPMM_F16 ? 16 : 8))
        return B200SPMM_ERR_UNSUPPORTED;
    if (n_ctas > kNoAllocMaxCtas) {
        set_last_error_static("b200spmm_spmm_noalloc: n_ctas exceeds the 1024 CTAs the built-in schedule table holds");
        return B200SPMM_ERR_UNSUPPORTED;
    }
    if (info->total_tiles * (uint64_t)kRowWindow >= 0x7FFFFFFFull || info->cols > 0x7FFFFFFFull || n > 0x7FFFFFFF || n % 8)
        return B200SPMM_ERR_UNSUPPORTED;
    const int esz = info->dtype == B200SPMM_F16 ? 2 : 4, csz = c_dtype == B200SPMM_C_F32 ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(d_B) & 15u) || (reinterpret_cast<uintptr_t>(d_C) & 15u) ||
        (reinterpret_cast<uintptr_t>(d_data) & 15u) || (reinterpret_cast<uintptr_t>(d_tcA2B) & 15u) ||
        (ldb * esz) % 16 || (ldc * csz) % 16)
        return B200SPMM_ERR_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    B200_CUDA_TRY(cudaSetDevice(device));
    if (n_ctas <= 0) {
        B200_CUDA_TRY(cudaDeviceGetAttribute(&n_ctas, cudaDevAttrMultiProcessorCount, device));
        n_ctas *= kCtasPerSm;
        if (n_ctas > kNoAllocMaxCtas) n_ctas = kNoAllocMaxCtas;
    }
    if (info->eff_row_windows == 0) {  // nothing stored: C is all zeros
        B200_CUDA_TRY(cudaMemset2DAsync(d_C, (size_t)ldc * csz, 0, (size_t)n * csz, info->rows, stream));
        return B200SPMM_OK;
    }
    uint32_t *scratch = nullptr;
    int st = noalloc_scratch_address(device, &scratch);
    if (st != B200SPMM_OK) return st;

    b200spmm_plan tmp;  // lives on the stack; owns nothing
    static const bool cpasync = env_is("B200SPMM_GATHER", "cpasync");  // read once per process
    tmp.gather_cpasync = cpasync;
    tmp.info = *info;
    tmp.device = device;
    tmp.sched.n_ctas = n_ctas;  // the tables themselves are in the built-in array
    tmp.launch_sched = &tmp.sched;
    tmp.d_rowOffset = const_cast<uint32_t *>(d_rowOffset);
    tmp.d_tcA2B = const_cast<uint32_t *>(d_tcA2B);
    tmp.d_rowIdx = const_cast<uint32_t *>(d_rowIdx);
    tmp.d_data = const_cast<void *>(d_data);
    st = encode_tile_map(&tmp);
    if (st != B200SPMM_OK) return st;

    // The table and the status word keep the previous call's contents: both are rewritten here,
    // on the same stream, before the SpMM kernel reads them.
    noalloc_schedule_kernel<<<1, 256, 0, stream>>>(
        d_rowOffset, (uint32_t)info->eff_row_windows, n_ctas, scratch);
    B200_CUDA_TRY(cudaGetLastError());

    SpmmParams prm{};
    prm.rowOffset = d_rowOffset;
    prm.tcA2B = d_tcA2B;
    prm.rowIdx = d_rowIdx;
    prm.chunk_tile = scratch + kNoAllocTile;  // one chunk per CTA
    prm.chunk_wfirst = scratch + kNoAllocWfirst;
    prm.chunk_wlast = scratch + kNoAllocWlast;
    prm.chunk_head_slot = prm.chunk_tail_slot = nullptr;  // cuts lie on window boundaries: no shared windows
    prm.chunk_begin = 0;
    prm.chunk_end = (uint32_t)n_ctas;
    prm.sched_counter = nullptr;
    prm.partial = nullptr;
    prm.tiles_image = nullptr;  // the caller's tiles, as they are, through the tensor map
    prm.total_tiles = (uint32_t)info->total_tiles;
    prm.B = d_B;
    prm.C = d_C;
    prm.ldb = ldb;
    prm.ldc = ldc;
    prm.rows = (uint32_t)info->rows;
    prm.cols = (uint32_t)info->cols;
    prm.n = (uint32_t)n;
    prm.eff_row_windows = (uint32_t)info->eff_row_windows;
    prm.c_is_half = c_dtype == B200SPMM_C_F16;
    prm.status = scratch + kNoAllocStatusWord;
    prm.wait_limit_ns = kDeviceWaitLimitNs;
    return info->dtype == B200SPMM_F16 ? launch_dtype<false>(&tmp, prm, stream) : launch_dtype<true>(&tmp, prm, stream);
}

}  // extern "C"
