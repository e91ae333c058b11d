// SpMM kernel for 128-row super-windows: the variant for matrices whose 16-row windows already touch
// most columns (a pruned weight matrix: 10 % unstructured density puts 81 % of all columns into every
// 16-row window), where the condensed tile stream is as long as a dense one.
//
// The 16-row kernel (spmm_kernel.cuh) keeps the reference's transposition (src/fp16.cu:147): the
// gathered rows of B are the wide operand and the window's 16 rows are the MMA's N.  An N = 16 MMA
// holds the tensor pipe for the ~40 clocks it takes to read its 4 KB operand from shared memory and
// does 8 clocks of arithmetic.  Here eight windows are merged (plan-internal, the format handed to
// callers stays the reference's) and the transposition is undone:
//     D[128 window rows x kNs features] += Atile[128 x CW] * Bgather[CW x kNs]
// The sparse tile is the UMMA A operand (M = 128, K-major, 32-byte swizzle: 128 rows of 32 bytes; the
// plan stores the merged tiles already in that shared-memory image, so a tile arrives by one plain
// 4 KB bulk copy instead of a tiled load of 128 narrow rows), the gathered rows of B are the UMMA B
// operand (N = kNs = 128 or 256 features, MN-major, 128-byte swizzle: as TMA tile::gather4 lays B's
// rows down).  One MMA per tile does
// 128 x kNs x CW multiply-adds at the pipe's full rate, and the accumulator's lane is the window row,
// so an epilogue thread holds consecutive features of one row and stores them as 16-byte vectors.
//
// A work item is (super-window, feature slab); items are numbered window-major, so the CTAs that
// run at the same time work on the slabs of the same few windows and share their tiles in L2.  CTA b
// starts with item b and claims further items from a global counter.
//
// Roles in a CTA of 416 threads, one CTA per SM:
//   warps 0-7   epilogue: warp w drains TMEM lanes 32 (w % 4) .. +31 (32 window rows), columns half
//               w / 4 of the accumulator; tcgen05.ld 32x32b.x32 gives a thread 32 consecutive features
//               of its row
//   warp  8     lane 0 issues tcgen05.mma / tcgen05.commit; the warp owns the TMEM allocation
//               (two accumulators of kNs columns)
//   warps 9-12  producers: warp g fills every fourth stage of the tile stream; a stage is four consecutive
//               tiles: their 4 x 4 KB of A by one bulk copy, their rows of B by tiled TMA boxes where a
//               tile's columns are neighbours (CW rows x 128 bytes per instruction) and by tile::gather4
//               elsewhere (four rows per instruction)
// Every wait is bounded, as in the 16-row kernel.
#pragma once

#include "spmm_kernel.cuh"

namespace b200spmm {

constexpr int kTallRows = 128;                  // rows of a super-window
constexpr int kTallTileBytes = kTallRows * 32;  // one tile of it: 128 rows x 32 bytes

struct TallParams {
    const uint32_t *rowOffset;  // [eff+1] tiles
    const uint32_t *tcA2B;      // [tiles*CW]
    const uint32_t *rowIdx;     // [eff] first row of each super-window (a multiple of 128)
    const uint8_t *data;        // [tiles][4 KB] tiles as they lie in shared memory: row r of a tile at r * 32 bytes,
                                // its two 16-byte halves swapped when (r / 4) is odd (the 32-byte swizzle)
    // B re-laid per launch as shared-memory images (pack_b_kernel), or null: block (slab, row group) holds
    // the CW rows [group * CW, group * CW + CW) x the slab's kNs features exactly as the MMA's B operand
    // lies in shared memory, so a tile whose columns are that row group arrives by one bulk copy.
    const uint8_t *b_packed;
    uint32_t b_groups;          // row groups of B: ceil(cols / CW)
    uint32_t *sched_counter;    // [2] items handed out beyond the first gridDim.x, CTAs finished; zero at launch and at exit
    void *C;                    // [rows, n] row-major
    int64_t ldc;                // elements
    uint32_t rows, cols, n;
    uint32_t eff_row_windows;
    uint32_t n_slabs;           // ceil(n / kNs)
    uint32_t n_items;           // eff_row_windows * n_slabs
    uint32_t c_is_half;
    uint32_t *status;
    unsigned long long wait_limit_ns;
    uint32_t starve_bytes;      // known-answer launches only: bytes every stage expects on top of what its loads deliver,
                                // so that no stage ever fills and the bounded waits run out (0 in a product)
#ifdef B200SPMM_PROFILE
    uint32_t debug;  // measurement builds only: bit 0 skips the B gathers, bit 1 the MMAs, bit 2 the A tiles
    unsigned long long *prof;  // [gridDim.x][32] cycle counters
#endif
};

// A thread's 32 consecutive features (fp32 bits, feat0 ..) of row `row` -> C, as 16-byte vectors: 8 features per
// store for fp16 C, 4 for fp32 C (n is a multiple of 8).  Rows past the end and features past n are dropped.
B200_DEVICE void tall_store_row32(const TallParams &p, uint32_t row, uint32_t feat0, const uint32_t (&r)[32]) {
    if (row >= p.rows || feat0 >= p.n) return;
    if (p.c_is_half) {
        __half *dst = static_cast<__half *>(p.C) + (int64_t)row * p.ldc + feat0;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (feat0 + v * 8 < p.n) {
                uint4 pk;
                __half2 h0 = __floats2half2_rn(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                __half2 h1 = __floats2half2_rn(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                __half2 h2 = __floats2half2_rn(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                __half2 h3 = __floats2half2_rn(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                pk.x = *reinterpret_cast<uint32_t *>(&h0);
                pk.y = *reinterpret_cast<uint32_t *>(&h1);
                pk.z = *reinterpret_cast<uint32_t *>(&h2);
                pk.w = *reinterpret_cast<uint32_t *>(&h3);
                *reinterpret_cast<uint4 *>(dst + v * 8) = pk;
            }
        }
    } else {
        float *dst = static_cast<float *>(p.C) + (int64_t)row * p.ldc + feat0;
#pragma unroll
        for (int v = 0; v < 8; ++v)
            if (feat0 + v * 4 < p.n)
                *reinterpret_cast<uint4 *>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
    }
}

// Zeros into rows [lo, hi) of C, features [f0, f0 + feats): warp `who` of `of` takes every of-th row.
B200_DEVICE void tall_clear_rows(const TallParams &p, uint32_t lo, uint32_t hi, uint32_t who, uint32_t of, uint32_t f0,
                                 uint32_t feats, int lane) {
    const uint32_t vec_per_row = feats / 4;
    for (uint32_t rr = lo + who; rr < hi; rr += of) {
        for (uint32_t v4 = lane; v4 < vec_per_row; v4 += 32) {
            const uint32_t feat = f0 + v4 * 4;
            if (p.c_is_half)
                *reinterpret_cast<uint2 *>(static_cast<__half *>(p.C) + (int64_t)rr * p.ldc + feat) = make_uint2(0, 0);
            else
                *reinterpret_cast<float4 *>(static_cast<float *>(p.C) + (int64_t)rr * p.ldc + feat) = make_float4(0, 0, 0, 0);
        }
    }
}

template <bool kTf32, int kNs>
struct TallCfg {
    static_assert(kNs == 128 || kNs == 256, "feature slab");
    static constexpr int kCW = kTf32 ? 8 : 16;
    static constexpr int kEsz = kTf32 ? 4 : 2;
    // Four tiles per ring stage: the MMA-issuing thread pays its wait, its commit and its ring
    // bookkeeping (about 330 SM clocks, measured) once per stage, and four MMAs keep the tensor pipe
    // busy for 512 clocks.  With two tiles per stage that thread, not the pipe, set the pace.
    static constexpr int kTps = 4;                          // tiles per ring stage
    static constexpr int kGatherBytes = 32 * kNs;           // CW rows x kNs features
    static constexpr int kStageBytes = kTps * (kGatherBytes + kTallTileBytes);
    static constexpr int kProducerWarps = 4;
    static constexpr int kStages = kNs == 256 ? 4 : 6;      // 192 KB of operands in flight
    static constexpr int kEpilogueWarps = 8;
    static constexpr int kMmaWarp = 8;
    static constexpr int kFirstProducerWarp = 9;
    static constexpr int kThreads = 32 * (kFirstProducerWarp + kProducerWarps);  // 416
    static constexpr int kBoxFeatures = 128 / kEsz;         // features in one 128-byte TMA box
    static constexpr int kRowQuads = kCW / 4;
    static constexpr int kBoxes = kNs / kBoxFeatures;       // 128-byte column blocks of a slab
    static constexpr int kGatherOps = kRowQuads * kBoxes;   // gather4 instructions per tile: 16 or 8
    static constexpr int kBoxBytes = kCW * 128;             // CW consecutive rows of B, one column block
    static_assert(kGatherOps <= 16 && kTps % 2 == 0, "16 lanes serve one tile, a warp two tiles at a time");
    static constexpr int kIdxSlots = 4;                     // per producer warp: column lists of its next stages
    static constexpr int kIdxAhead = kIdxSlots - 1;
    static constexpr int kSlotBytes = kTps * kCW * 4;
    static constexpr int kIdxBytes = kProducerWarps * kIdxSlots * kSlotBytes;
    static constexpr int kBarriers = 2 * kStages + 5;       // full, empty, 2 x acc_full, 2 x acc_empty, drain
    static constexpr int kItemSlots = 64;                   // circular list of the items this CTA runs
    static constexpr uint32_t kTmemCols = 2 * kNs;          // two accumulators
    static constexpr size_t kSmemBytes =
        1024 + (size_t)kStages * kStageBytes + kIdxBytes + kBarriers * 8 + 16 + kItemSlots * 4 + 8;
};

template <bool kTf32, int kNs>
__global__ void __launch_bounds__((TallCfg<kTf32, kNs>::kThreads), 1)
spmm_tall_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_bt,
                 const TallParams p) {
    using Cfg = TallCfg<kTf32, kNs>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kTps = Cfg::kTps;
    extern __shared__ uint8_t smem_raw[];

    // ---- shared memory carve-up (1024-byte aligned: swizzle patterns follow address bits)
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *base = smem_raw + pad;
    const uint32_t gather_addr = raw_addr + pad;                                      // kStages x 2 x kGatherBytes
    const uint32_t atile_addr = gather_addr + kStages * kTps * Cfg::kGatherBytes;      // kStages x 2 x 4 KB
    uint32_t *idx_ring = reinterpret_cast<uint32_t *>(base + kStages * Cfg::kStageBytes);
    const uint32_t idx_ring_addr = atile_addr + kStages * kTps * kTallTileBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + kStages * Cfg::kStageBytes + Cfg::kIdxBytes);
    const uint32_t bars_addr = idx_ring_addr + Cfg::kIdxBytes;
    auto full_bar = [&](uint32_t s) { return bars_addr + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bars_addr + 8u * ((uint32_t)kStages + s); };
    auto acc_full_bar = [&](uint32_t a) { return bars_addr + 8u * (uint32_t)(2 * kStages + a); };
    auto acc_empty_bar = [&](uint32_t a) { return bars_addr + 8u * (uint32_t)(2 * kStages + 2 + a); };
    const uint32_t drain_bar = bars_addr + 8u * (uint32_t)(2 * kStages + 4);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bars + Cfg::kBarriers);
    uint32_t *tmem_slot = const_cast<uint32_t *>(abort_flag) + 1;
    volatile uint32_t *mma_done = abort_flag + 2;
    volatile uint32_t *item_list = abort_flag + 4;                 // items this CTA runs, in order (circular)
    volatile uint32_t *item_avail = item_list + Cfg::kItemSlots;   // entries written so far

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t limit = p.wait_limit_ns;

    // ---- this CTA's items.  Every role follows the list at its own pace; the roles are never further
    // apart than the ring and the two accumulators allow (far fewer than kItemSlots items), so a slot
    // is not rewritten while a slower role still has to read it.
    constexpr uint32_t kNoItem = 0xFFFFFFFFu;
    auto item_id = [&](uint32_t k) -> uint32_t {
        if (*item_avail <= k) {
            const uint64_t t0 = ptx::global_timer_ns();
            while (*item_avail <= k) {
                __nanosleep(100);
                if (*abort_flag) return kNoItem;
                if (ptx::global_timer_ns() - t0 > limit) {
                    *abort_flag = 1;
                    return kNoItem;
                }
            }
        }
        __threadfence_block();
        return item_list[k % Cfg::kItemSlots];
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {
            ptx::mbar_init(full_bar(s), 1);   // lane 0 of the stage's producer warp (+ the bytes of its loads)
            ptx::mbar_init(empty_bar(s), 1);  // tcgen05.commit of the MMA issuer
        }
        for (uint32_t a = 0; a < 2; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), Cfg::kEpilogueWarps);
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        *mma_done = 0;
        item_list[0] = blockIdx.x < p.n_items ? blockIdx.x : kNoItem;
        *item_avail = 1;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_bt);
    }
    if (warp == Cfg::kMmaWarp) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), Cfg::kTmemCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < Cfg::kEpilogueWarps) {
        // =========================================================== epilogue warps
        const uint32_t q = (uint32_t)warp & 3u;      // TMEM lane quarter: window rows 32q .. 32q + 31
        const uint32_t hsel = (uint32_t)warp >> 2;   // which half of the accumulator's columns
        constexpr uint32_t kHalf = kNs / 2;
        bool epi_alive = true;
        for (uint32_t round = 0; epi_alive; ++round) {
            const uint32_t item = item_id(round);
            if (item == kNoItem) break;
            const uint32_t w = item / p.n_slabs, slab = item - w * p.n_slabs;
            const uint32_t row0 = p.rowIdx[w];
            const uint32_t gap_hi = w + 1 < p.eff_row_windows ? p.rowIdx[w + 1] : p.rows;
            const uint32_t a = round & 1u;
            uint32_t ok = 1;
            if (lane == 0) ok = ptx::mbar_wait(acc_full_bar(a), (round >> 1) & 1u, abort_flag, limit) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { epi_alive = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t row = row0 + q * 32u + (uint32_t)lane;
            const uint32_t f_slab = slab * kNs;
#pragma unroll 1
            for (uint32_t c = 0; c < kHalf / 32u; ++c) {
                const uint32_t col0 = hsel * kHalf + c * 32u;
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + ((q * 32u) << 16) + a * kNs + col0, r);
                ptx::tmem_ld_wait();
                if (c + 1 == kHalf / 32u) {  // the last read of this buffer: it may be overwritten from here on
                    ptx::tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_empty_bar(a));
                }
                const uint32_t feat0 = f_slab + col0;  // this thread: features feat0 .. feat0 + 31 of its row
                tall_store_row32(p, row, feat0, r);
            }
            // Rows of super-windows without entries are absent from the format: clear the gap after this
            // window (and the rows before the very first one), this slab's features.  Warp w takes every
            // eighth row.
            const bool lead = w == 0 && row0 > 0;
            if (gap_hi > row0 + kTallRows || lead) {
                const uint32_t slab_feats = min((uint32_t)kNs, p.n - f_slab);
                tall_clear_rows(p, row0 + kTallRows, min(gap_hi, p.rows), (uint32_t)warp, Cfg::kEpilogueWarps, f_slab, slab_feats, lane);
                if (lead) tall_clear_rows(p, 0u, row0, (uint32_t)warp, Cfg::kEpilogueWarps, f_slab, slab_feats, lane);
            }
        }
    } else if (warp >= Cfg::kFirstProducerWarp) {
        // =========================================================== producer warps
        const uint32_t pid = (uint32_t)(warp - Cfg::kFirstProducerWarp);  // fills stages pid, pid + 4, ...
        const uint32_t half = (uint32_t)lane >> 4, hl = (uint32_t)lane & 15u;  // lanes 16j .. serve tile j of the stage
        constexpr uint32_t kSlotWords = Cfg::kSlotBytes / 4;
        uint32_t *my_idx = idx_ring + pid * Cfg::kIdxSlots * kSlotWords;
        const uint32_t my_idx_addr = idx_ring_addr + pid * Cfg::kIdxSlots * Cfg::kSlotBytes;
        constexpr int kIdxLanes = Cfg::kCW * 4 / 16;  // lanes that copy one column list (16 bytes each)
        // lane o of a half issues gather instruction o of its tile: row quad g = o % kRowQuads of
        // 128-byte column block h = o / kRowQuads
        const uint32_t g = hl % Cfg::kRowQuads, h = hl / Cfg::kRowQuads;
        const uint32_t op_quad = g, op_x = h * Cfg::kBoxFeatures;
        // fp16: block (h, rows 8j..8j+7) is 1 KiB, a quad is half of it; tf32: block (h, quad) is 512 B
        const uint32_t op_dst = kTf32 ? (h * 2 + g) * 512u : (h * 2 + (g >> 1)) * 1024u + (g & 1u) * 512u;

        struct Cursor {
            uint32_t round, sp, tile_begin, n_tiles, stages, slab, done;
        };
        uint32_t grabbed = 1;  // first producer warp: entries of the CTA's item list written so far
        auto open_item = [&](Cursor &c) {
            if (pid == 0 && c.round == grabbed) {  // nobody has asked for this one yet: claim the next item
                if (lane == 0) {
                    uint32_t next = gridDim.x + atomicAdd(p.sched_counter, 1u);
                    if (next >= p.n_items) next = kNoItem;
                    item_list[c.round % Cfg::kItemSlots] = next;
                    __threadfence_block();
                    *item_avail = c.round + 1;
                }
                ++grabbed;
                __syncwarp();
            }
            const uint32_t item = item_id(c.round);
            if (item == kNoItem) {
                c.done = 1;
                return;
            }
            const uint32_t w = item / p.n_slabs;
            c.slab = item - w * p.n_slabs;
            c.tile_begin = p.rowOffset[w];
            c.n_tiles = p.rowOffset[w + 1] - c.tile_begin;
            c.stages = (c.n_tiles + kTps - 1) / kTps;
        };
        auto normalise = [&](Cursor &c) {  // stage cursor past the end of an item: next item
            while (!c.done && c.sp >= c.stages) {
                c.sp -= c.stages;
                ++c.round;
                open_item(c);
            }
        };
        Cursor cur{0, pid, 0, 0, 0, 0, 0};
        open_item(cur);
        normalise(cur);
        Cursor fc = cur;
        uint32_t it = 0, it_f = 0;
        auto fetch_list = [&]() {  // column lists of the fetch cursor's stage -> its ring slot; then advance
            if (!fc.done) {
                const uint32_t tpos0 = fc.sp * kTps;
                const uint32_t here = min((uint32_t)kTps, fc.n_tiles - tpos0);
                const uint32_t slot_addr = my_idx_addr + (it_f % Cfg::kIdxSlots) * Cfg::kSlotBytes;
                const uint64_t t = (uint64_t)fc.tile_begin + tpos0;
                if ((uint32_t)lane < kIdxLanes * kTps && (uint32_t)lane / kIdxLanes < here)
                    ptx::cp_async_16(slot_addr + lane * 16, p.tcA2B + t * Cfg::kCW + lane * 4, 16u);
                fc.sp += Cfg::kProducerWarps;
                normalise(fc);
            }
            ++it_f;
        };
        for (int i = 0; i < Cfg::kIdxAhead; ++i) fetch_list();
        ptx::cp_async_commit();
        ptx::cp_async_wait_group<0>();
        __syncwarp();

        uint32_t s = pid, use = 0;
        B200_PROF_DECL(prof_wait_empty);
        B200_PROF_DECL(prof_issue);
#ifdef B200SPMM_PROFILE
        const long long prof_start = clock64();
#endif
        while (!cur.done) {
            const uint32_t tpos0 = cur.sp * kTps;
            const uint32_t here = min((uint32_t)kTps, cur.n_tiles - tpos0);
            const uint32_t *slot_words = my_idx + (it % Cfg::kIdxSlots) * kSlotWords;
            uint32_t ok = 1;
            if (lane == 0) {
                {
                    B200_PROF_T0();
                    ok = ptx::mbar_wait(empty_bar(s), (use & 1u) ^ 1u, abort_flag, limit) ? 1u : 0u;
                    B200_PROF_ADD(prof_wait_empty);
                }
                if (ok) {
                    const uint32_t gather_bytes = (B200_DEBUG_BITS(p) & 1u) ? 0u : (uint32_t)Cfg::kGatherBytes;
                    const uint32_t tile_bytes = (B200_DEBUG_BITS(p) & 4u) ? 0u : (uint32_t)kTallTileBytes;
                    ptx::mbar_arrive_expect_tx(full_bar(s), here * (gather_bytes + tile_bytes) + p.starve_bytes);
                    // the stage's tiles of A are neighbours in memory and in the ring: one copy
                    if (tile_bytes)
                        ptx::bulk_load(atile_addr + s * kTps * kTallTileBytes,
                                       p.data + (uint64_t)(cur.tile_begin + tpos0) * kTallTileBytes, here * kTallTileBytes, full_bar(s));
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            B200_PROF_T0();
            // The whole stage at once: when its tiles name consecutive aligned row groups of B (the column
            // list of a window that holds every column), their images are neighbours in the packed copy of B
            // and in the ring, and one bulk copy brings them all.  A bulk copy holds the issuing warp for a
            // couple of hundred clocks whatever its size, so fewer and larger ones keep the producers ahead.
            bool stage_run = false;
            if (p.b_packed) {
                bool good = true;
                if ((uint32_t)lane < here) {
                    const uint32_t *l = slot_words + lane * Cfg::kCW;
                    const uint32_t f = l[0];
                    good = l[Cfg::kCW - 1] - f == (uint32_t)Cfg::kCW - 1u && f % (uint32_t)Cfg::kCW == 0u &&
                           f == slot_words[0] + (uint32_t)lane * Cfg::kCW;
                }
                stage_run = __all_sync(0xffffffffu, good);
            }
            if (stage_run) {
                if (lane == 0 && !(B200_DEBUG_BITS(p) & 1u))
                    ptx::bulk_load(gather_addr + s * kTps * Cfg::kGatherBytes,
                                   p.b_packed + ((uint64_t)cur.slab * p.b_groups + slot_words[0] / (uint32_t)Cfg::kCW) * Cfg::kGatherBytes,
                                   here * (uint32_t)Cfg::kGatherBytes, full_bar(s));
            } else
#pragma unroll
            for (uint32_t r = 0; r < (uint32_t)kTps / 2; ++r) {  // two tiles at a time, 16 lanes each
                const uint32_t j = 2 * r + half;
                if (j < here && !(B200_DEBUG_BITS(p) & 1u)) {
                    const uint32_t *list = slot_words + j * Cfg::kCW;
                    const uint32_t dst = gather_addr + (s * kTps + j) * Cfg::kGatherBytes;
                    const uint32_t first = list[0];
                    // A list is ascending and distinct (padding 0xFFFFFFFF at its end): when its last entry
                    // is CW - 1 past its first, the tile's rows of B are neighbours and arrive as tiled
                    // boxes of CW rows - the TMA unit moves those several times faster than four-row
                    // gathers (about 39 bytes per clock and SM, measured).  In a matrix that takes this
                    // kernel nearly every tile is of that kind.
                    if (list[Cfg::kCW - 1] - first == (uint32_t)Cfg::kCW - 1u) {
                        // ... and when they are one aligned row group and B was packed for this launch, as
                        // one bulk copy of the group's image: one request to the TMA unit instead of one per
                        // row and column block (that unit's request rate, ~3 clocks per row, bounds this kernel)
                        if (p.b_packed && first % (uint32_t)Cfg::kCW == 0u) {
                            if (hl == 0)
                                ptx::bulk_load(dst, p.b_packed + ((uint64_t)cur.slab * p.b_groups + first / (uint32_t)Cfg::kCW) * Cfg::kGatherBytes,
                                               (uint32_t)Cfg::kGatherBytes, full_bar(s));
                        } else if (hl < (uint32_t)Cfg::kBoxes)
                            ptx::tma_load_2d(dst + hl * Cfg::kBoxBytes, &tmap_bt, (int32_t)(cur.slab * kNs + hl * Cfg::kBoxFeatures),
                                             (int32_t)first, full_bar(s));
                    } else if (hl < (uint32_t)Cfg::kGatherOps) {
                        const uint4 rows4 = *reinterpret_cast<const uint4 *>(list + op_quad * 4);
                        // padded slots hold 0xFFFFFFFF: clamp to the first row past the end, which reads zeros
                        ptx::tma_gather4_2d(dst + op_dst, &tmap_b, (int32_t)(cur.slab * kNs + op_x),
                                            (int32_t)min(rows4.x, p.cols), (int32_t)min(rows4.y, p.cols),
                                            (int32_t)min(rows4.z, p.cols), (int32_t)min(rows4.w, p.cols), full_bar(s));
                    }
                }
            }
            fetch_list();
            ptx::cp_async_commit();
            // the list needed next iteration was fetched kIdxAhead groups ago
            ptx::cp_async_wait_group<Cfg::kIdxAhead - 1>();
            __syncwarp();
            B200_PROF_ADD(prof_issue);
            ++it;
            cur.sp += Cfg::kProducerWarps;
            normalise(cur);
            s += Cfg::kProducerWarps;
            while (s >= (uint32_t)kStages) { s -= kStages; ++use; }
        }
        ptx::cp_async_wait_group<0>();
        __syncwarp();
#ifdef B200SPMM_PROFILE
        if (lane == 0 && pid == 1) {
            B200_PROF_STORE(0, clock64() - prof_start);
            B200_PROF_STORE(1, prof_wait_empty);
            B200_PROF_STORE(3, it);
            B200_PROF_STORE(11, prof_issue);
        }
#endif
    } else if (warp == Cfg::kMmaWarp && lane == 0) {
        // =========================================================== MMA issuer (warp 8, lane 0)
        constexpr uint32_t fmt = kTf32 ? ptx::kFmtTF32 : ptx::kFmtF16;
        // A = the sparse tile, K-major; B = the gathered rows, MN-major
        constexpr uint32_t idesc = ptx::make_instr_desc(fmt, kTallRows, kNs, false, true);
        // sparse tile: K-major rows of 32 bytes, 32-byte swizzle, 8-row groups 256 bytes apart
        const uint64_t a_desc0 = ptx::make_smem_desc(atile_addr, 16, 256, ptx::kSwizzle32B);
        // gathered rows: MN-major, 128-byte swizzle.  fp16: 64-feature blocks 2 KiB apart, 8-row groups
        // 1 KiB apart; tf32: 32-feature blocks 1 KiB apart, 4-row groups 512 B apart
        constexpr uint32_t b_lbo = kTf32 ? 1024u : 2048u, b_sbo = kTf32 ? 512u : 1024u;
        const uint64_t b_desc0 =
            ptx::make_smem_desc(gather_addr, b_lbo, b_sbo, kTf32 ? ptx::kSwizzle128BBase32B : ptx::kSwizzle128B);
        const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
        const uint32_t a_lo0 = (uint32_t)a_desc0, b_lo0 = (uint32_t)b_desc0;
        constexpr uint32_t kATile16 = kTallTileBytes >> 4, kGather16 = Cfg::kGatherBytes >> 4;
        uint32_t s = 0, phase = 0;
        uint32_t alo = a_lo0, blo = b_lo0;  // low descriptor words of the first tile of stage s
        bool alive = true;
        const uint32_t do_mma = (B200_DEBUG_BITS(p) & 2u) ? 0u : 1u;
        B200_PROF_DECL(prof_wait_full);
        B200_PROF_DECL(prof_wait_acc);
#ifdef B200SPMM_PROFILE
        const long long prof_start = clock64();
        long long prof_stages = 0;
#endif
        for (uint32_t round = 0; alive; ++round) {
            const uint32_t item = item_id(round);
            if (item == kNoItem) break;
            const uint32_t w = item / p.n_slabs;
            uint32_t nt = p.rowOffset[w + 1] - p.rowOffset[w];
            const uint32_t a = round & 1u;
            {
                B200_PROF_T0();
                alive = ptx::mbar_wait(acc_empty_bar(a), ((round >> 1) & 1u) ^ 1u, abort_flag, limit);
                B200_PROF_ADD(prof_wait_acc);
            }
            ptx::tcgen05_fence_after_sync();
            const uint32_t d = tmem_base + a * kNs;
            uint32_t accumulate = 0;
            while (nt != 0 && alive) {
                {
                    B200_PROF_T0();
                    alive = ptx::mbar_wait(full_bar(s), phase, abort_flag, limit);
                    B200_PROF_ADD(prof_wait_full);
                }
#ifdef B200SPMM_PROFILE
                ++prof_stages;
#endif
                ptx::tcgen05_fence_after_sync();
                if (!alive) break;
                const uint32_t here = min(nt, (uint32_t)kTps);
#pragma unroll
                for (uint32_t q = 0; q < (uint32_t)kTps; ++q) {  // predicated, no branches: the last stage of an item may be short
                    const uint32_t on = q < here ? do_mma : 0u;
                    const uint32_t acc = q == 0 ? accumulate : 1u;
                    if (kTf32) ptx::umma_tf32_ss_lohi_if(on, d, alo + q * kATile16, a_hi, blo + q * kGather16, b_hi, idesc, acc);
                    else ptx::umma_f16_ss_lohi_if(on, d, alo + q * kATile16, a_hi, blo + q * kGather16, b_hi, idesc, acc);
                }
                accumulate = 1;
                nt -= here;
                ptx::umma_commit(empty_bar(s));
                const bool wrap = s + 1 == (uint32_t)kStages;  // selects, no branch
                s = wrap ? 0u : s + 1;
                phase ^= wrap ? 1u : 0u;
                alo = wrap ? a_lo0 : alo + kTps * kATile16;
                blo = wrap ? b_lo0 : blo + kTps * kGather16;
            }
            if (alive) ptx::umma_commit(acc_full_bar(a));
        }
#ifdef B200SPMM_PROFILE
        B200_PROF_STORE(4, clock64() - prof_start);
        B200_PROF_STORE(5, prof_wait_full);
        B200_PROF_STORE(6, prof_wait_acc);
        B200_PROF_STORE(7, prof_stages);
#endif
        if (!alive || *abort_flag) {  // MMAs may be in flight that no awaited commit covers: see the 16-row kernel
            ptx::umma_commit(drain_bar);
            ptx::mbar_wait_bounded(drain_bar, 0, limit);
            ptx::tcgen05_fence_after_sync();
        }
    }

    if (warp == Cfg::kMmaWarp) {  // the idle lanes of the MMA warp sleep until lane 0 is done
        if (lane == 0) {
            *mma_done = 1;
        } else {
            while (*mma_done == 0) __nanosleep(2000);
        }
        __syncwarp();
    }
    // ---- teardown: every role ends up here, on success and on timeout alike
    if (*abort_flag) {  // loads may still be on their way into shared memory: see the 16-row kernel
        const uint64_t t0 = ptx::global_timer_ns();
        while (ptx::global_timer_ns() - t0 < kAbortLingerNs) __nanosleep(1000);
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == Cfg::kMmaWarp) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
    if (tid == 0 && *abort_flag) atomicOr(p.status, kDevStatusTimeout);
    if (tid == 0) {  // the last CTA to finish leaves both counters at zero for the next launch
        __threadfence();
        if (atomicAdd(p.sched_counter + 1, 1u) == gridDim.x - 1u) {
            p.sched_counter[0] = 0;
            p.sched_counter[1] = 0;
        }
    }
}

// B [cols x n, leading dimension ldb] -> images of the MMA's B operand: block (slab, row group) of
// 32 * kNs bytes holds rows [group * CW, +CW) x features [slab * kNs, +kNs) in the layout TMA lays a
// gathered tile down - fp16: 64-feature column blocks of 2 KB (16 rows x 128 B, the 16-byte pieces of a
// row XORed with row % 8 inside each 8-row half); tf32: 32-feature column blocks of 1 KB (8 rows x 128 B,
// the 32-byte units XORed with row % 4 inside each 4-row half).  Rows past `cols` and features past n are
// zeros.  One thread per 16-byte piece.
template <bool kTf32>
__global__ void __launch_bounds__(256)
pack_b_kernel(const uint8_t *__restrict__ B, int64_t ldb_bytes, uint32_t cols, uint32_t n, uint32_t kNs, uint32_t n_slabs,
              uint32_t n_groups, uint8_t *__restrict__ packed) {
    constexpr uint32_t kCW = kTf32 ? 8 : 16, kEsz = kTf32 ? 4 : 2;
    const uint32_t row_pieces = kNs * kEsz / 16;                       // 16-byte pieces of one row of a slab
    const uint64_t total = (uint64_t)n_slabs * n_groups * kCW * row_pieces;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t piece = (uint32_t)(i % row_pieces);             // consecutive threads: consecutive pieces of a row
        uint64_t rest = i / row_pieces;
        const uint32_t k = (uint32_t)(rest % kCW);                     // row inside the group
        rest /= kCW;
        const uint32_t group = (uint32_t)(rest % n_groups), slab = (uint32_t)(rest / n_groups);
        const uint32_t row = group * kCW + k;
        const uint32_t feat_byte = (slab * kNs * kEsz) + piece * 16;   // byte offset inside the row of B
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < cols && feat_byte < n * kEsz) v = *reinterpret_cast<const uint4 *>(B + (uint64_t)row * ldb_bytes + feat_byte);
        const uint32_t h = piece >> 3, cc = piece & 7u;                // 128-byte column block, piece inside it
        uint32_t off;
        if (kTf32) {
            const uint32_t kr = k & 3u;
            off = (h * 2 + (k >> 2)) * 512u + kr * 128u + ((((cc >> 1) ^ kr) << 5) | ((cc & 1u) << 4));
        } else {
            const uint32_t kr = k & 7u;
            off = (h * 2 + (k >> 3)) * 1024u + kr * 128u + ((cc ^ kr) << 4);
        }
        *reinterpret_cast<uint4 *>(packed + ((uint64_t)slab * n_groups + group) * (32u * kNs) + off) = v;
    }
}

}  // namespace b200spmm
