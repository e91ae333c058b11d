// SpMM kernel for 256-row super-windows run by PAIRS of CTAs on neighbouring SMs (a cluster of two,
// tcgen05.mma.cta_group::2): the 128-row kernel (spmm_tall_kernel.cuh) with the MMA widened to
//     D[256 window rows x 256 features] += Atile[256 x CW] * Bgather[CW x 256]
// CTA r of the pair holds rows 128 r .. of the tile and of the accumulator, and columns 128 r .. of the
// gathered rows of B, in its own shared and tensor memory; the even CTA issues the MMA for both.  A tile
// step then costs each SM 4 KB of A and 4 KB of B from L2 where the 128-row kernel fetches 4 + 8 KB for the
// same 128 tensor-pipe clocks - and that path (about 51 bytes per clock and SM, measured) is what bounds the
// 128-row kernel on a pruned weight matrix.  The reference's kernel keeps a window inside one SM
// (src/fp16.cu:147); it has no counterpart of this pairing.
//
// A work item is (256-row super-window, 256-feature slab); pair k starts with item k, the even CTA
// claims further items from a global counter and writes them into both CTAs' item lists.
//
// Roles in a CTA of 416 threads, one CTA per SM:
//   warps 0-7   epilogue: warp w drains TMEM lanes 32 (w % 4) .. +31 of its own CTA (window rows
//               128 r + 32 (w % 4) ..), columns half w / 4; an emptied accumulator is reported to the even
//               CTA's barrier (a remote arrive from the odd CTA)
//   warp  8     even CTA: lane 0 issues tcgen05.mma / tcgen05.commit (the commit arrives on both CTAs'
//               barriers); odd CTA: lane 0 forwards "my part of stage s has landed" to the even CTA's
//               full barrier.  The warp owns the TMEM allocation (made by both CTAs together).
//   warps 9-12  producers, as in the 128-row kernel, for this CTA's half of A and of B
// Every wait is bounded; both CTAs meet at a cluster barrier before either lets go of its shared or
// tensor memory.
#pragma once

#include "spmm_tall_kernel.cuh"

namespace b200spmm {

constexpr int kPairRows = 256;  // rows of a super-window of the pair kernel

// TallParams as for the 128-row kernel, with: rowIdx a multiple of 256; data = per window the tiles of
// the even CTA (rows 0-127, 4 KB images) followed by the tiles of the odd CTA (rows 128-255); b_packed
// packed for 128-feature slabs (slab 2 S + r is CTA r's half of item slab S); n_slabs = ceil(n / 256).
template <bool kTf32>
struct PairCfg {
    static constexpr int kNs = 256;                         // features of an item
    static constexpr int kNc = 128;                         // ... of which one CTA fetches
    static constexpr int kCW = kTf32 ? 8 : 16;
    static constexpr int kEsz = kTf32 ? 4 : 2;
    static constexpr int kTps = 4;                          // tiles per ring stage (6 and 8 were slower: 711 / 729 us against 678)
    static constexpr int kGatherBytes = 32 * kNc;           // CW rows x 128 features
    static constexpr int kStageBytes = kTps * (kGatherBytes + kTallTileBytes);
    static constexpr int kStages = 24 / kTps;               // 192 KB of operands in flight per CTA
    static constexpr int kProducerWarps = kStages < 4 ? kStages : 4;
    static constexpr int kEpilogueWarps = 8;
    static constexpr int kMmaWarp = 8;
    static constexpr int kFirstProducerWarp = 9;
    static constexpr int kThreads = 32 * (kFirstProducerWarp + kProducerWarps);  // 416
    static constexpr int kBoxFeatures = 128 / kEsz;
    static constexpr int kRowQuads = kCW / 4;
    static constexpr int kBoxes = kNc / kBoxFeatures;       // 128-byte column blocks of a CTA's half slab
    static constexpr int kGatherOps = kRowQuads * kBoxes;   // gather4 instructions per tile: 8
    static constexpr int kBoxBytes = kCW * 128;
    static_assert(kGatherOps <= 16 && kTps % 2 == 0 && kProducerWarps <= kStages, "see the 128-row kernel");
    static constexpr int kIdxSlots = 4;
    static constexpr int kIdxAhead = kIdxSlots - 1;
    static constexpr int kSlotBytes = kTps * kCW * 4;
    static constexpr int kIdxBytes = kProducerWarps * kIdxSlots * kSlotBytes;
    static constexpr int kBarriers = 2 * kStages + 5;       // full, empty, 2 x acc_full, 2 x acc_empty, drain
    static constexpr int kItemSlots = 64;
    static constexpr uint32_t kTmemCols = 2 * kNs;          // two accumulators of 256 columns in each CTA
    static constexpr size_t kSmemBytes =
        1024 + (size_t)kStages * kStageBytes + kIdxBytes + kBarriers * 8 + 16 + kItemSlots * 4 + 8;
};

template <bool kTf32>
__global__ void __launch_bounds__((PairCfg<kTf32>::kThreads), 1)
spmm_pair_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_bt,
                 const TallParams p) {
    using Cfg = PairCfg<kTf32>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kTps = Cfg::kTps;
    constexpr int kNs = Cfg::kNs;
    extern __shared__ uint8_t smem_raw[];

    // ---- shared memory carve-up: the same offsets in both CTAs (the dynamic area starts at the same
    // address in every CTA of a launch), which the MMA's descriptors and the multicast commits rely on
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *base = smem_raw + pad;
    const uint32_t gather_addr = raw_addr + pad;
    const uint32_t atile_addr = gather_addr + kStages * kTps * Cfg::kGatherBytes;
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
    volatile uint32_t *item_list = abort_flag + 4;
    volatile uint32_t *item_avail = item_list + Cfg::kItemSlots;
    const uint32_t item_list_addr = bars_addr + Cfg::kBarriers * 8 + 16;
    const uint32_t item_avail_addr = item_list_addr + Cfg::kItemSlots * 4;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t limit = p.wait_limit_ns;
    const uint32_t rank = ptx::cluster_cta_rank();  // 0: issues the MMAs and claims the items
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

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
        __threadfence();  // the entry may have been written by the other CTA of the pair
        return item_list[k % Cfg::kItemSlots];
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {
            // even CTA: its own producer (+ the bytes of its loads) and the odd CTA's forwarder
            ptx::mbar_init(full_bar(s), rank == 0 ? 2 : 1);
            ptx::mbar_init(empty_bar(s), 1);  // the even CTA's tcgen05.commit, multicast to both
        }
        for (uint32_t a = 0; a < 2; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), 2 * Cfg::kEpilogueWarps);  // both CTAs' epilogue warps (used in the even CTA)
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        *mma_done = 0;
        item_list[0] = pair < p.n_items ? pair : kNoItem;
        *item_avail = 1;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_bt);
    }
    if (warp == Cfg::kMmaWarp) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), Cfg::kTmemCols);
        ptx::tmem_relinquish_alloc_permit_pair();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();  // the other CTA's barriers exist before anything arrives on them
    ptx::cluster_wait();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < Cfg::kEpilogueWarps) {
        // =========================================================== epilogue warps
        const uint32_t q = (uint32_t)warp & 3u;
        const uint32_t hsel = (uint32_t)warp >> 2;
        constexpr uint32_t kHalf = kNs / 2;
        const uint32_t leader_acc_empty0 = ptx::map_to_cta(acc_empty_bar(0), 0), leader_acc_empty1 = ptx::map_to_cta(acc_empty_bar(1), 0);
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
            const uint32_t row = row0 + rank * kTallRows + q * 32u + (uint32_t)lane;
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
                    if (lane == 0) ptx::mbar_arrive_cluster(a ? leader_acc_empty1 : leader_acc_empty0);
                }
                const uint32_t feat0 = f_slab + col0;
                tall_store_row32(p, row, feat0, r);
            }
            // Rows of super-windows without entries are absent from the format: clear the gap after this
            // window (and the rows before the very first one), this slab's features.  The sixteen epilogue
            // warps of the pair take every sixteenth row each.
            const bool lead = w == 0 && row0 > 0;
            if (gap_hi > row0 + kPairRows || lead) {
                const uint32_t slab_feats = min((uint32_t)kNs, p.n - f_slab);
                const uint32_t who = rank * Cfg::kEpilogueWarps + (uint32_t)warp, of = 2 * Cfg::kEpilogueWarps;
                tall_clear_rows(p, row0 + kPairRows, min(gap_hi, p.rows), who, of, f_slab, slab_feats, lane);
                if (lead) tall_clear_rows(p, 0u, row0, who, of, f_slab, slab_feats, lane);
            }
        }
    } else if (warp >= Cfg::kFirstProducerWarp) {
        // =========================================================== producer warps
        const uint32_t pid = (uint32_t)(warp - Cfg::kFirstProducerWarp);
        const uint32_t half = (uint32_t)lane >> 4, hl = (uint32_t)lane & 15u;
        constexpr uint32_t kSlotWords = Cfg::kSlotBytes / 4;
        uint32_t *my_idx = idx_ring + pid * Cfg::kIdxSlots * kSlotWords;
        const uint32_t my_idx_addr = idx_ring_addr + pid * Cfg::kIdxSlots * Cfg::kSlotBytes;
        constexpr int kIdxLanes = Cfg::kCW * 4 / 16;
        const uint32_t g = hl % Cfg::kRowQuads, h = hl / Cfg::kRowQuads;
        const uint32_t op_quad = g, op_x = h * Cfg::kBoxFeatures;
        const uint32_t op_dst = kTf32 ? (h * 2 + g) * 512u : (h * 2 + (g >> 1)) * 1024u + (g & 1u) * 512u;
        const uint32_t peer_list_addr = ptx::map_to_cta(item_list_addr, 1), peer_avail_addr = ptx::map_to_cta(item_avail_addr, 1);

        struct Cursor {
            uint32_t round, sp, tile_begin, n_tiles, stages, slab, done;
        };
        uint32_t grabbed = 1;
        auto open_item = [&](Cursor &c) {
            if (rank == 0 && pid == 0 && c.round == grabbed) {  // nobody has asked for this one yet: claim the next item
                if (lane == 0) {
                    uint32_t next = n_pairs + atomicAdd(p.sched_counter, 1u);
                    if (next >= p.n_items) next = kNoItem;
                    item_list[c.round % Cfg::kItemSlots] = next;
                    ptx::st_cluster_u32(peer_list_addr + (c.round % Cfg::kItemSlots) * 4u, next);
                    __threadfence();
                    *item_avail = c.round + 1;
                    ptx::st_cluster_u32(peer_avail_addr, c.round + 1);
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
            const uint32_t t0 = p.rowOffset[w];
            c.n_tiles = p.rowOffset[w + 1] - t0;
            c.tile_begin = t0;
            c.stages = (c.n_tiles + kTps - 1) / kTps;
        };
        auto normalise = [&](Cursor &c) {
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
        auto fetch_list = [&]() {
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
        B200_PROF_DECL(prof_a_issue);
        B200_PROF_DECL(prof_b_issue);
        B200_PROF_DECL(prof_fetch);
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
                    B200_PROF_T0();
                    ptx::mbar_arrive_expect_tx(full_bar(s), here * (gather_bytes + tile_bytes) + p.starve_bytes);
                    // this CTA's halves of the stage's tiles are neighbours in memory and in the ring: one copy
                    if (tile_bytes)
                        ptx::bulk_load(atile_addr + s * kTps * kTallTileBytes,
                                       p.data + ((uint64_t)cur.tile_begin * 2u + (uint64_t)rank * cur.n_tiles + tpos0) * kTallTileBytes,
                                       here * kTallTileBytes, full_bar(s));
                    B200_PROF_ADD(prof_a_issue);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            B200_PROF_T0();
            const uint32_t my_slab = cur.slab * 2u + rank;  // 128-feature half slab of this CTA
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
                                   p.b_packed + ((uint64_t)my_slab * p.b_groups + slot_words[0] / (uint32_t)Cfg::kCW) * Cfg::kGatherBytes,
                                   here * (uint32_t)Cfg::kGatherBytes, full_bar(s));
            } else
#pragma unroll
            for (uint32_t r = 0; r < (uint32_t)kTps / 2; ++r) {
                const uint32_t j = 2 * r + half;
                if (j < here && !(B200_DEBUG_BITS(p) & 1u)) {
                    const uint32_t *list = slot_words + j * Cfg::kCW;
                    const uint32_t dst = gather_addr + (s * kTps + j) * Cfg::kGatherBytes;
                    const uint32_t first = list[0];
                    if (list[Cfg::kCW - 1] - first == (uint32_t)Cfg::kCW - 1u) {  // neighbouring rows of B: see the 128-row kernel
                        if (p.b_packed && first % (uint32_t)Cfg::kCW == 0u) {
                            if (hl == 0)
                                ptx::bulk_load(dst, p.b_packed + ((uint64_t)my_slab * p.b_groups + first / (uint32_t)Cfg::kCW) * Cfg::kGatherBytes,
                                               (uint32_t)Cfg::kGatherBytes, full_bar(s));
                        } else if (hl < (uint32_t)Cfg::kBoxes)
                            ptx::tma_load_2d(dst + hl * Cfg::kBoxBytes, &tmap_bt, (int32_t)(my_slab * Cfg::kNc + hl * Cfg::kBoxFeatures),
                                             (int32_t)first, full_bar(s));
                    } else if (hl < (uint32_t)Cfg::kGatherOps) {
                        const uint4 rows4 = *reinterpret_cast<const uint4 *>(list + op_quad * 4);
                        ptx::tma_gather4_2d(dst + op_dst, &tmap_b, (int32_t)(my_slab * Cfg::kNc + op_x),
                                            (int32_t)min(rows4.x, p.cols), (int32_t)min(rows4.y, p.cols),
                                            (int32_t)min(rows4.z, p.cols), (int32_t)min(rows4.w, p.cols), full_bar(s));
                    }
                }
            }
#ifdef B200SPMM_PROFILE
            __syncwarp();
            prof_b_issue += clock64() - prof_t0__;
            const long long prof_t1 = clock64();
#endif
            fetch_list();
#ifdef B200SPMM_PROFILE
            prof_fetch += clock64() - prof_t1;
#endif
            ptx::cp_async_commit();
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
            B200_PROF_STORE(12, prof_a_issue);
            B200_PROF_STORE(13, prof_b_issue);
            B200_PROF_STORE(14, prof_fetch);
        }
#endif
    } else if (warp == Cfg::kMmaWarp && lane == 0 && rank == 0) {
        // =========================================================== MMA issuer (even CTA, warp 8, lane 0)
        constexpr uint32_t fmt = kTf32 ? ptx::kFmtTF32 : ptx::kFmtF16;
        constexpr uint32_t idesc = ptx::make_instr_desc(fmt, kPairRows, kNs, false, true);
        const uint64_t a_desc0 = ptx::make_smem_desc(atile_addr, 16, 256, ptx::kSwizzle32B);
        constexpr uint32_t b_lbo = kTf32 ? 1024u : 2048u, b_sbo = kTf32 ? 512u : 1024u;
        const uint64_t b_desc0 =
            ptx::make_smem_desc(gather_addr, b_lbo, b_sbo, kTf32 ? ptx::kSwizzle128BBase32B : ptx::kSwizzle128B);
        const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
        const uint32_t a_lo0 = (uint32_t)a_desc0, b_lo0 = (uint32_t)b_desc0;
        constexpr uint32_t kATile16 = kTallTileBytes >> 4, kGather16 = Cfg::kGatherBytes >> 4;
        uint32_t s = 0, phase = 0;
        uint32_t alo = a_lo0, blo = b_lo0;
        bool alive = true;
        const uint32_t do_mma = (B200_DEBUG_BITS(p) & 2u) ? 0u : 1u;
        B200_PROF_DECL(prof_wait_full);
        B200_PROF_DECL(prof_wait_acc);
        B200_PROF_DECL(prof_mma);
        B200_PROF_DECL(prof_commit);
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
                alive = ptx::mbar_wait_cluster(acc_empty_bar(a), ((round >> 1) & 1u) ^ 1u, abort_flag, limit);
                B200_PROF_ADD(prof_wait_acc);
            }
            ptx::tcgen05_fence_after_sync();
            const uint32_t d = tmem_base + a * kNs;
            uint32_t accumulate = 0;
            while (nt != 0 && alive) {
                {
                    B200_PROF_T0();
                    alive = ptx::mbar_wait_cluster(full_bar(s), phase, abort_flag, limit);
                    B200_PROF_ADD(prof_wait_full);
                }
#ifdef B200SPMM_PROFILE
                ++prof_stages;
#endif
                ptx::tcgen05_fence_after_sync();
                if (!alive) break;
                const uint32_t here = min(nt, (uint32_t)kTps);
#ifdef B200SPMM_PROFILE
                const long long prof_m0 = clock64();
#endif
#pragma unroll
                for (uint32_t q = 0; q < (uint32_t)kTps; ++q) {
                    const uint32_t on = q < here ? do_mma : 0u;
                    const uint32_t acc = q == 0 ? accumulate : 1u;
                    ptx::umma_pair_ss_lohi_if(kTf32, on, d, alo + q * kATile16, a_hi, blo + q * kGather16, b_hi, idesc, acc);
                }
                accumulate = 1;
                nt -= here;
#ifdef B200SPMM_PROFILE
                const long long prof_m1 = clock64();
                prof_mma += prof_m1 - prof_m0;
#endif
                ptx::umma_commit_pair(empty_bar(s));  // the stage is free in both CTAs
#ifdef B200SPMM_PROFILE
                prof_commit += clock64() - prof_m1;
#endif
                const bool wrap = s + 1 == (uint32_t)kStages;
                s = wrap ? 0u : s + 1;
                phase ^= wrap ? 1u : 0u;
                alo = wrap ? a_lo0 : alo + kTps * kATile16;
                blo = wrap ? b_lo0 : blo + kTps * kGather16;
            }
            if (alive) ptx::umma_commit_pair(acc_full_bar(a));  // both CTAs' epilogues
        }
#ifdef B200SPMM_PROFILE
        B200_PROF_STORE(4, clock64() - prof_start);
        B200_PROF_STORE(5, prof_wait_full);
        B200_PROF_STORE(6, prof_wait_acc);
        B200_PROF_STORE(7, prof_stages);
        B200_PROF_STORE(15, prof_mma);
        B200_PROF_STORE(16, prof_commit);
#endif
        if (!alive || *abort_flag) {  // MMAs may be in flight that no awaited commit covers
            ptx::umma_commit_pair_local(drain_bar);
            ptx::mbar_wait_bounded(drain_bar, 0, limit);
            ptx::tcgen05_fence_after_sync();
        }
    } else if (warp == Cfg::kMmaWarp && lane == 0) {
        // =========================================================== forwarder (odd CTA, warp 8, lane 0)
        // The even CTA's MMA reads this CTA's shared memory too: tell its full barrier when this CTA's
        // part of a stage has landed.
        uint32_t leader_full[kStages];
#pragma unroll
        for (int i = 0; i < kStages; ++i) leader_full[i] = ptx::map_to_cta(full_bar((uint32_t)i), 0);
        uint32_t s = 0, phase = 0;
        bool alive = true;
        B200_PROF_DECL(prof_wait_full);
        B200_PROF_DECL(prof_arrive);
#ifdef B200SPMM_PROFILE
        const long long prof_start = clock64();
#endif
        for (uint32_t round = 0; alive; ++round) {
            const uint32_t item = item_id(round);
            if (item == kNoItem) break;
            const uint32_t w = item / p.n_slabs;
            const uint32_t nt = p.rowOffset[w + 1] - p.rowOffset[w];
            for (uint32_t st = 0; st < (nt + kTps - 1) / kTps && alive; ++st) {
                {
                    B200_PROF_T0();
                    alive = ptx::mbar_wait(full_bar(s), phase, abort_flag, limit);
                    B200_PROF_ADD(prof_wait_full);
                }
                if (!alive) break;
                uint32_t remote = leader_full[0];
#pragma unroll
                for (int i = 1; i < kStages; ++i) remote = s == (uint32_t)i ? leader_full[i] : remote;
                {
                    // Relaxed: this thread has seen its CTA's barrier complete, and the operands were written
                    // by the async proxy and are read by this SM's tensor core once the even CTA has issued the
                    // MMA - after its wait on the barrier this arrive completes.  A releasing arrive at cluster
                    // scope holds the thread for ~1,400 clocks while loads are in flight (measured), which made
                    // this thread the pace of the whole pair.
                    B200_PROF_T0();
                    ptx::mbar_arrive_cluster_relaxed(remote);
                    B200_PROF_ADD(prof_arrive);
                }
                const bool wrap = s + 1 == (uint32_t)kStages;
                s = wrap ? 0u : s + 1;
                phase ^= wrap ? 1u : 0u;
            }
        }
#ifdef B200SPMM_PROFILE
        B200_PROF_STORE(4, clock64() - prof_start);
        B200_PROF_STORE(5, prof_wait_full);
        B200_PROF_STORE(6, prof_arrive);
#endif
    }

    if (warp == Cfg::kMmaWarp) {  // the idle lanes of warp 8 sleep until lane 0 is done
        if (lane == 0) {
            *mma_done = 1;
        } else {
            while (*mma_done == 0) __nanosleep(2000);
        }
        __syncwarp();
    }
    // ---- teardown: every role ends up here, on success and on timeout alike
    if (*abort_flag) {  // loads may still be on their way into shared memory
        const uint64_t t0 = ptx::global_timer_ns();
        while (ptx::global_timer_ns() - t0 < kAbortLingerNs) __nanosleep(1000);
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    // neither CTA lets go of shared or tensor memory that the other's MMAs, commits or arrives may still reach
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == Cfg::kMmaWarp) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
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

}  // namespace b200spmm
