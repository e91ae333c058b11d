// Warp-specialised persistent SpMM kernel for sm_100a over the condensed row-window format.
//
// Takes the place of the reference's fp16_spmm_kernel (src/fp16.cu:36-175), which is an
// sm_90a wgmma kernel with a two-stage ring, and supplies the tf32 kernel the reference
// never wrote (src/tf32.cu holds only a CPU check).
//
// Mapping (same transposition the reference uses, src/fp16.cu:147): for a 16-row window and a
// tile of CW condensed columns,
//     Dt[features x 16 rows] += Bgather[features x CW] * Atile^T[CW x 16]
// so the gathered rows of B are the UMMA "A" operand (M = 128 or 64 features, MN-major,
// 128-byte swizzle - 16-byte units for fp16, 32-byte units for tf32: how B's rows lie in memory) and the 16 x CW tile of the sparse
// matrix is the UMMA "B" operand (N = 16, K-major, 32-byte swizzle: exactly how the tile lies
// in `data`).  K per tile is 32 bytes for both element types (16 fp16 / 8 tf32), one
// tcgen05.mma per tile and 128-feature chunk.  The accumulator lives in TMEM (16 columns per
// chunk), double-buffered so a window's epilogue overlaps the next window's MMAs.
//
// A single GPU thread retires roughly one dependent instruction every ten cycles, so the kernel
// is organised around instruction counts on each role's critical path, not only around bytes.
//
// Roles in a CTA of 544 threads (a pass covers at most 128 features, so that two CTAs share an SM
// and give it two MMA-issuing threads; wider B is multiplied in several passes):
//   warps 0-7  epilogue, two sets of four warps; set e drains accumulator buffer e, i.e. every
//              other window.  Warp q of a set owns TMEM lanes 32q..32q+31 (32 features): after
//              tcgen05.ld lane l holds one feature of the 16 window rows and stores them straight
//              to C, 32 lanes covering one 128-byte line of a row per instruction; no barrier
//              between warps.  Also zero-fills rows that belong to windows without entries
//   warp  8    lane 0 issues tcgen05.mma / tcgen05.commit; the warp owns the TMEM allocation
//   warps 9-16 producers, two groups of four warps.  A ring stage holds eight consecutive tiles;
//              group g fills stages g, g+2, g+4, ... - two tiles per warp, 16 lanes each.  The first
//              warp of the group brings the stage's eight 512-byte A tiles with one TMA load; every
//              half-warp fetches the CW rows of B its tile selects with TMA tile::gather4 (four rows
//              per instruction, one instruction per lane, landing in the swizzled operand layout;
//              a cp.async variant exists for comparison and for very narrow B).  Column lists are
//              fetched a few iterations ahead into a per-warp ring.  Two tiles per warp and
//              iteration halve the producers' instructions per tile; eight tiles per stage halve
//              the barrier round trips of the MMA issuer.
//
// The schedule cuts the tile stream, not the window list, so a window heavier than a CTA's share
// is computed in pieces by several CTAs; pieces go to fp32 slots and spmm_fixup_kernel adds them.
//
// Every wait is bounded; on a timeout the roles drain and the kernel raises a status bit.
#pragma once

#include <cstdint>
#include <type_traits>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.hpp"
#include "format.hpp"
#include "ptx_sm100.cuh"

// Optional cycle accounting of the roles' waits, compiled in only with -DB200SPMM_PROFILE.
#ifdef B200SPMM_PROFILE
#define B200_PROF_DECL(name) long long name = 0
#define B200_PROF_T0() const long long prof_t0__ = clock64()
#define B200_PROF_ADD(name) name += clock64() - prof_t0__
#define B200_PROF_STORE(slot, value) p.prof[(size_t)blockIdx.x * 32 + (slot)] = (unsigned long long)(value)
#define B200_DEBUG_BITS(p) ((p).debug)
#else
#define B200_PROF_DECL(name)
#define B200_PROF_T0()
#define B200_PROF_ADD(name)
#define B200_PROF_STORE(slot, value)
#define B200_DEBUG_BITS(p) 0u
#endif

namespace b200spmm {

constexpr int kRowWindow = 16;       // rows per window the kernels consume
constexpr int kProducerWarps = 4;    // warps per producer group
constexpr int kTilesPerWarp = 2;     // tiles a producer warp brings per iteration (16 lanes each)
constexpr int kTilesPerStage = kProducerWarps * kTilesPerWarp;  // a ring stage: eight consecutive tiles
constexpr int kEpilogueWarps = 8;    // two sets of four: set e drains accumulator buffer e
constexpr int kMmaWarp = 8;
constexpr int kFirstProducerWarp = 9;
constexpr int kATileBytes = 512;     // 16 rows x 32 bytes
constexpr uint32_t kAccCols = 32;    // TMEM columns per accumulator buffer (2 chunks x 16)
constexpr uint32_t kTmemCols = 64;   // two accumulator buffers
constexpr uint64_t kAbortLingerNs = 200000;  // failure path: how long a CTA lingers before it exits

struct SpmmParams {
    const uint32_t *rowOffset;   // [eff+1] tiles
    const uint32_t *tcA2B;       // [tiles*CW]
    const uint32_t *rowIdx;      // [eff]
    // The tiles as they lie in shared memory (the two 16-byte halves of a tile row swapped when row / 4 is
    // odd: the 32-byte swizzle), or null.  With it a ring stage's eight tiles arrive by ONE plain 4 KB bulk
    // copy; the tiled load of the caller's array costs the TMA unit a request per 32-byte row - 128 per
    // stage, as many as half of the stage's gathers - and that unit's request rate is what bounds the
    // kernel on matrices whose B fits L2.
    const uint8_t *tiles_image;
    uint32_t total_tiles;
    // schedule: chunk c holds tiles [chunk_tile[c], chunk_tile[c+1]); CTA b starts with chunk chunk_begin + b and
    // takes further chunks, from chunk_begin + gridDim.x on, in the order in which the CTAs ask for them
    const uint32_t *chunk_tile;       // [n_chunks+1]
    const uint32_t *chunk_wfirst;     // [n_chunks] window holding the chunk's first tile
    const uint32_t *chunk_wlast;      // [n_chunks] window holding the chunk's last tile
    const uint32_t *chunk_head_slot;  // [n_chunks] slot for the piece at the chunk's head, or kNoSlot (null: no pieces)
    const uint32_t *chunk_tail_slot;  // [n_chunks] slot for the piece at the chunk's tail, or kNoSlot
    uint32_t chunk_begin, chunk_end;  // the chunks this launch covers (the whole table, or one band of rows)
    uint32_t *sched_counter;     // [2] chunks handed out beyond the first gridDim.x, CTAs finished; both zero
                                 // at launch and again at exit (null: every CTA runs its first chunk only)
    float *partial;              // [slots][16][n] fp32 pieces of windows cut at a chunk boundary (may be null)
    // bitmap kernels only: the tiles in compressed form instead of the dense `data` behind the tile tensor map
    const uint64_t *tcBit;       // [tiles * 16*CW/64] one bit per tile slot, row-major, low bit first
    const uint32_t *nnzOffset;   // [tiles+1] first stored value of each tile
    const void *values;          // stored values, tile after tile, row-major inside a tile
    // entry-list kernels only (fp16): per tile a record of 32 words, one per lane of a producer warp -
    // (byte offset inside the tile's shared-memory image << 16) | value bits for a stored entry, kNoEntry for an
    // unused word, kDenseTile in all 32 words of a tile with more than 32 entries (that tile comes from
    // tiles_image by a bulk copy).  The expansion is a zero fill and one 2-byte store per lane.
    const uint32_t *tile_entries;
    const void *B;               // [cols, n] row-major
    void *C;                     // [rows, n] row-major
    int64_t ldb, ldc;            // elements
    uint32_t rows, cols, n;
    uint32_t eff_row_windows;
    uint32_t n_slabs;            // ceil(n / kNs)
    uint32_t c_is_half;          // 0: fp32 C, 1: fp16 C
    uint32_t *status;            // device status word
    unsigned long long wait_limit_ns;
#ifdef B200SPMM_PROFILE
    // measurement builds only: bit 0 skips the B gathers, bit 1 the MMAs, bit 2 the A tiles, bit 3 the
    // loads of a compressed tile's stored values (results are then invalid)
    uint32_t debug;
    unsigned long long *prof;    // [gridDim.x][32] cycle counters
#endif
};

// kTma selects how the rows of B reach shared memory: true = TMA tile::gather4 (four rows per
// instruction, issued by a few lanes, completion counted in bytes on the stage's mbarrier);
// false = 16-byte cp.async copies by all lanes of the producer warps.
// kTiles: 0 = dense tiles (512 bytes each, by TMA / bulk copy); 1 = the tiles come compressed as bitmap +
// stored values (the reference's bitmap format) and the producer warps expand them into the ring; 2 = the
// tiles come as records of 32 (position, value) words (SpmmParams::tile_entries), a quarter of the dense
// bytes, which a producer warp expands with two stores per lane.
constexpr uint32_t kNoEntry = 0xFFFF0000u, kDenseTile = 0xFFFFFFFEu;
template <bool kTf32, int kNs, bool kTma = true, int kTiles = 0>
struct SpmmCfg {
    static constexpr bool kBitmap = kTiles == 1, kEntries = kTiles == 2;
    static_assert(kTma || kTiles == 0, "compressed tiles go with the TMA gather");
    static_assert(!kEntries || !kTf32, "entry lists hold 16-bit values");
    static_assert(kNs == 64 || kNs == 128 || kNs == 192 || kNs == 256, "feature slab");  // in use: 64 and 128
    // One thread issues a CTA's MMAs, and with 16-row windows every MMA is small: the issuing
    // thread, not the tensor core, sets the pace.  Up to 128 features a CTA is small enough for
    // two to share an SM, which gives the SM two issuing threads and two rings to keep full.
    static constexpr int kCtasPerSm = kNs <= 128 ? 2 : 1;
    static constexpr int kProducerGroups = 2;
    static constexpr int kThreads = 32 * (kFirstProducerWarp + kProducerWarps * kProducerGroups);  // 544
    static constexpr int kCW = kTf32 ? 8 : 16;           // condensed columns per tile
    static constexpr int kEsz = kTf32 ? 4 : 2;           // bytes per element of A and B
    static constexpr int kGatherBytes = 32 * kNs;        // CW rows x kNs features, one tile
    static constexpr int kTilesPerStage = b200spmm::kTilesPerStage;
    static constexpr int kStageBytes = kTilesPerStage * (kGatherBytes + kATileBytes);
    static constexpr int kFullChunks = kNs / 128;        // M = 128 MMAs per tile
    static constexpr bool kHalfChunk = (kNs % 128) != 0; // plus one M = 64 MMA
    static constexpr int kChunks = kFullChunks + (kHalfChunk ? 1 : 0);
    // Ring depth: 24-40 tiles (about 110 KB for two CTAs per SM, 210 KB for one) are in flight per
    // CTA.  One barrier pair serves eight tiles, which keeps the per-tile cost of waits, fences and
    // commits low.  (With compressed tiles the wider list slots leave room for two stages only.)
    static constexpr int kStages = kNs == 64 ? 5 : kNs == 128 ? (kBitmap ? 2 : 3) : kNs == 192 ? 4 : 3;
    // cp.async variant only: groups a warp keeps in flight before it reports the oldest as landed
    static constexpr int kLag = kStages / kProducerGroups >= 3 ? kStages / kProducerGroups - 2 : 0;
    static_assert(kTma ? kStages >= kProducerGroups : kStages > kProducerGroups * (kLag + 1), "ring too shallow");
    static constexpr int kChunksPerRow = kNs * kEsz / 16;           // 16-byte pieces per gathered row
    static constexpr int kCopiesPerLane = kCW * kChunksPerRow / 32;  // == kNs / 16
    // TMA gather: a box is 128 bytes of a row (64 fp16 / 32 tf32 features); one instruction moves
    // that box for four of the tile's rows.
    static constexpr int kBoxFeatures = 128 / kEsz;
    static constexpr int kRowQuads = kCW / 4;
    static constexpr int kGatherOps = kRowQuads * (kNs / kBoxFeatures);  // per tile, at most 16
    static constexpr int kWinAhead = 16;   // windows whose tile counts the MMA issuer prefetches
    static constexpr int kWinSlots = 32;
    // Each producer warp keeps the column lists of its next kIdxAhead tiles in a private ring of
    // kIdxSlots entries, fetched in the same cp.async groups as the rows of the current tile.
    // With compressed tiles a slot also holds the tile's bitmap and its two value offsets.
    static constexpr int kIdxSlots = kBitmap ? 4 : (kCtasPerSm == 2 ? 3 : 8);
    static constexpr int kIdxAhead = kIdxSlots - 1;
    // Compressed tiles: the slot of the tile after the current one has to be in shared memory
    // when the current one is expanded, because the loads of its stored values start right then.
    static constexpr int kSlotLead = kBitmap ? 2 : 1;
    static_assert((kTma || kIdxAhead > kLag) && kIdxAhead < kIdxSlots, "column lists must land before they are needed");
    static constexpr int kBitWords = kRowWindow * kCW / 64;  // 64-bit bitmap words per tile
    static constexpr int kSlotBytes =
        kBitmap ? (kTilesPerWarp * (kCW * 4 + kBitWords * 8) + (kTilesPerWarp + 1) * 4 + 15) / 16 * 16 : kTilesPerWarp * kCW * 4;
    static_assert(kTilesPerWarp == 2 && kGatherOps <= 16, "a producer warp splits into two halves of 16 lanes, one per tile");
    static constexpr int kIdxBytes = kProducerWarps * kProducerGroups * kIdxSlots * kSlotBytes;
    static constexpr int kBarrierBytes = (2 * kStages + 5) * 8 + 16;
    static constexpr int kWinBytes = kWinSlots * 4;
    static constexpr int kChunkSlots = 32;  // chunks one CTA may take; the last entry always ends the list
    static constexpr int kChunkBytes = kChunkSlots * 4 + 8;
    static constexpr size_t kSmemBytes =
        1024 + (size_t)kStages * kStageBytes + kIdxBytes + kBarrierBytes + kWinBytes + kChunkBytes;
};

template <bool kTf32, int kNs, bool kTma, int kTiles>
__global__ void __launch_bounds__((SpmmCfg<kTf32, kNs, kTma, kTiles>::kThreads), (SpmmCfg<kTf32, kNs, kTma, kTiles>::kCtasPerSm))
spmm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const SpmmParams p) {
    using Cfg = SpmmCfg<kTf32, kNs, kTma, kTiles>;
    constexpr bool kBitmap = Cfg::kBitmap, kEntries = Cfg::kEntries;
    constexpr int kStages = Cfg::kStages;
    constexpr int kTps = Cfg::kTilesPerStage;
    constexpr int kProducerGroups = Cfg::kProducerGroups;
    extern __shared__ uint8_t smem_raw[];

    // ---- shared memory carve-up (1024-byte aligned: swizzle patterns follow address bits)
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *base = smem_raw + pad;
    const uint32_t gather_addr = raw_addr + pad;                                    // kStages x 8 x kGatherBytes
    const uint32_t atile_addr = gather_addr + kStages * kTps * Cfg::kGatherBytes;    // kStages x 8 x 512
    uint32_t *idx_ring = reinterpret_cast<uint32_t *>(base + kStages * Cfg::kStageBytes);
    const uint32_t idx_ring_addr = atile_addr + kStages * kTps * kATileBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + kStages * Cfg::kStageBytes + Cfg::kIdxBytes);
    const uint32_t bars_addr = idx_ring_addr + Cfg::kIdxBytes;
    auto full_bar = [&](uint32_t s) { return bars_addr + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bars_addr + 8u * ((uint32_t)kStages + s); };
    auto acc_full_bar = [&](uint32_t a) { return bars_addr + 8u * (uint32_t)(2 * kStages + a); };
    auto acc_empty_bar = [&](uint32_t a) { return bars_addr + 8u * (uint32_t)(2 * kStages + 2 + a); };
    const uint32_t drain_bar = bars_addr + 8u * (uint32_t)(2 * kStages + 4);  // failure path only, see the MMA issuer
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bars + 2 * kStages + 5);
    uint32_t *tmem_slot = const_cast<uint32_t *>(abort_flag) + 1;
    volatile uint32_t *mma_done = abort_flag + 2;
    volatile uint32_t *win_ends = reinterpret_cast<volatile uint32_t *>(bars + 2 * kStages + 5 + 2);
    const uint32_t win_ends_addr = bars_addr + 8u * (uint32_t)(2 * kStages + 5 + 2);
    volatile uint32_t *chunk_list = win_ends + Cfg::kWinSlots;          // chunks this CTA runs, in order
    volatile uint32_t *chunk_avail = chunk_list + Cfg::kChunkSlots;     // entries of chunk_list written so far

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef B200SPMM_PROFILE
    const unsigned long long prof_cta_t0 = ptx::global_timer_ns();
#endif
    const uint64_t limit = p.wait_limit_ns;

    // ---- this CTA's share of the schedule.  The tile stream is cut into many more chunks than
    // there are CTAs.  CTA b starts with chunk b; whenever its producers get near the end of a
    // chunk, the first producer warp takes the next unclaimed one from a global counter and
    // appends it to a list in shared memory, which all roles follow at their own pace.  So a CTA
    // that gets through its tiles faster (warmer columns of B, or simply the better share of the
    // SM it lives on) ends up with more chunks, and all CTAs finish together.  Which CTA ran a
    // chunk has no influence on the result.
    // A chunk's tiles are streamed once per feature slab; a pass is cut into stages of eight
    // consecutive tiles (the last stage of a pass may be short).  Ring stages, barrier phases and
    // accumulator buffers simply carry on from one pass and chunk to the next.
    // The schedule may cut inside a window: then the chunk computes a piece of it, which goes to
    // a partial-result slot instead of C and is summed by spmm_fixup_kernel.
    constexpr uint32_t kNoChunk = 0xFFFFFFFFu;
    // k-th chunk of this CTA, or kNoChunk after the last (also when the wait for the entry gives up)
    auto chunk_id = [&](uint32_t k) -> uint32_t {
        if (*chunk_avail <= k) {
            const uint64_t t0 = ptx::global_timer_ns();
            while (*chunk_avail <= k) {
                __nanosleep(100);
                if (*abort_flag) return kNoChunk;
                if (ptx::global_timer_ns() - t0 > limit) {
                    *abort_flag = 1;
                    return kNoChunk;
                }
            }
        }
        __threadfence_block();
        return chunk_list[k];
    };
    struct Chunk {
        uint32_t tile_begin, tile_end, w_begin, n_win, head_slot, tail_slot;
    };
    auto load_chunk = [&](uint32_t c) {
        Chunk ch;
        ch.tile_begin = p.chunk_tile[c];
        ch.tile_end = p.chunk_tile[c + 1];
        ch.w_begin = p.chunk_wfirst[c];
        ch.n_win = ch.tile_end > ch.tile_begin ? p.chunk_wlast[c] + 1 - ch.w_begin : 0u;
        ch.head_slot = p.chunk_head_slot ? p.chunk_head_slot[c] : kNoSlot;
        ch.tail_slot = p.chunk_tail_slot ? p.chunk_tail_slot[c] : kNoSlot;
        return ch;
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {
            ptx::mbar_init(full_bar(s), kProducerWarps);  // lane 0 of each producer warp (+ the A tiles' bytes)
            ptx::mbar_init(empty_bar(s), 1);              // tcgen05.commit of the MMA issuer
        }
        for (uint32_t a = 0; a < 2; ++a) {
            ptx::mbar_init(acc_full_bar(a), 1);
            ptx::mbar_init(acc_empty_bar(a), 4);
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        *mma_done = 0;
        chunk_list[0] = p.chunk_begin + blockIdx.x < p.chunk_end ? p.chunk_begin + blockIdx.x : kNoChunk;
        *chunk_avail = 1;
        ptx::fence_mbar_init();
        if (kTiles == 0) ptx::prefetch_tensormap(&tmap_a);
        if (kTma) ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == kMmaWarp) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kEpilogueWarps) {
        // =========================================================== epilogue warps
        const uint32_t e = (uint32_t)warp >> 2;  // accumulator buffer this set drains
        const uint32_t q = (uint32_t)warp & 3u;  // TMEM lane quarter = which 32 features of a 128-chunk
        uint32_t g0 = 0;  // accumulators this CTA has produced before the current chunk
        bool epi_alive = true;
        B200_PROF_DECL(prof_wait_accfull);
#ifdef B200SPMM_PROFILE
        const long long prof_start = clock64();
        uint32_t prof_windows = 0;
#endif
        // First row of a window and of the window after it (or the row count), fetched two of
        // this set's windows ahead so the loads are never waited for.
        for (uint32_t round = 0; epi_alive; ++round) {
            const uint32_t chunk = chunk_id(round);
            if (chunk == kNoChunk) break;
            const Chunk ch = load_chunk(chunk);
            const uint32_t n_win = ch.n_win, w_begin = ch.w_begin;
            if (n_win == 0) continue;
            const uint32_t total = p.n_slabs * n_win;  // accumulators this chunk produces, in order
            const uint32_t first = (e ^ g0) & 1u;      // this set drains the accumulators whose running number is e mod 2
            // accumulator `it` belongs to window (it mod n_win) of the chunk; the position is carried
            // along (pf) instead of divided out
            auto meta = [&](uint32_t it, uint32_t wi, uint32_t &row0, uint32_t &after) {
                if (it < total) {
                    const uint32_t w = w_begin + wi;
                    row0 = p.rowIdx[w];
                    after = w + 1 < p.eff_row_windows ? p.rowIdx[w + 1] : p.rows;
                }
            };
            auto wrap = [&](uint32_t x) {
                while (x >= n_win) x -= n_win;
                return x;
            };
            uint32_t row0_a = 0, after_a = 0, row0_b = 0, after_b = 0;
            uint32_t pf = wrap(first);
            meta(first, pf, row0_a, after_a);
            pf = wrap(pf + 2);
            meta(first + 2, pf, row0_b, after_b);
            pf = wrap(pf + 2);
            uint32_t slab = 0, i = first;  // position of accumulator `it`: window i of slab `slab`
            while (i >= n_win) { i -= n_win; ++slab; }
            for (uint32_t it = first; it < total; it += 2) {
                const uint32_t row0 = row0_a, gap_hi = after_a;
                row0_a = row0_b;
                after_a = after_b;
                meta(it + 4, pf, row0_b, after_b);
                pf = wrap(pf + 2);
                const uint32_t f0 = slab * kNs;  // first feature of the slab
                // a piece of a window shared with a neighbouring CTA goes to a partial-result slot
                const bool is_head_piece = i == 0 && ch.head_slot != kNoSlot;
                const bool is_tail_piece = i + 1 == n_win && ch.tail_slot != kNoSlot;
                const bool piece = is_head_piece || is_tail_piece;
                float *slot_rows = piece ? p.partial + (size_t)(is_head_piece ? ch.head_slot : ch.tail_slot) * kRowWindow * p.n : nullptr;
                uint32_t ok = 1;
                if (lane == 0) {  // one lane polls; every mbarrier operation costs a shared-memory slot per thread
                    B200_PROF_T0();
                    ok = ptx::mbar_wait(acc_full_bar(e), ((g0 + it) >> 1) & 1u, abort_flag, limit) ? 1u : 0u;
                    B200_PROF_ADD(prof_wait_accfull);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { epi_alive = false; break; }
                ptx::tcgen05_fence_after_sync();
                uint32_t r[Cfg::kChunks][16];
#pragma unroll
                for (int c = 0; c < Cfg::kChunks; ++c)
                    ptx::tmem_ld_32x32b_x16(tmem_base + ((q * 32u) << 16) + e * kAccCols + c * 16, r[c]);
                ptx::tmem_ld_wait();
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(acc_empty_bar(e));  // the buffer may be overwritten from here on
                // Lane l of this warp holds one feature of the 16 window rows (M = 128: feature 32q + l
                // of the chunk; M = 64: lanes 0-15 hold feature 16q + l), so a row of C receives 32
                // consecutive values from the warp: one full 128-byte line per store instruction.
#pragma unroll
                for (int c = 0; c < Cfg::kChunks; ++c) {
                    const bool half_chunk = Cfg::kHalfChunk && c == Cfg::kFullChunks;
                    const uint32_t width = half_chunk ? 16 : 32;  // features this warp owns in the chunk
                    const uint32_t feat = f0 + c * 128 + q * width + lane;
                    if (lane < width && feat < p.n) {
                        // The address of row j is walked with one 64-bit add per store and the row check is
                        // made once per window: the SM is short of issue slots, and sixteen multiplies and
                        // sixteen comparisons per window and warp cost a fifth of the time on short windows.
                        if (piece) {
                            float *dst = slot_rows + feat;
#pragma unroll
                            for (int j = 0; j < kRowWindow; ++j) {
                                *dst = __uint_as_float(r[c][j]);
                                dst += p.n;
                            }
                        } else if (p.c_is_half) {
                            __half *dst = static_cast<__half *>(p.C) + (int64_t)row0 * p.ldc + feat;
                            if (row0 + kRowWindow <= p.rows) {
#pragma unroll
                                for (int j = 0; j < kRowWindow; ++j) {
                                    *dst = __float2half_rn(__uint_as_float(r[c][j]));
                                    dst += p.ldc;
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < kRowWindow; ++j)
                                    if (row0 + j < p.rows) dst[(int64_t)j * p.ldc] = __float2half_rn(__uint_as_float(r[c][j]));
                            }
                        } else {
                            float *dst = static_cast<float *>(p.C) + (int64_t)row0 * p.ldc + feat;
                            if (row0 + kRowWindow <= p.rows) {
#pragma unroll
                                for (int j = 0; j < kRowWindow; ++j) {
                                    *dst = __uint_as_float(r[c][j]);
                                    dst += p.ldc;
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < kRowWindow; ++j)
                                    if (row0 + j < p.rows) dst[(int64_t)j * p.ldc] = __uint_as_float(r[c][j]);
                            }
                        }
                    }
                }
                // Rows of windows that hold no entries are absent from the format: clear the gap that
                // follows this window (and the one before the very first window).  Warp q of the set
                // takes every fourth row.
                // (the CTA that finishes a window clears the gap after it; the one that starts window 0 the lead)
                const bool lead = (w_begin + i == 0) && row0 > 0 && !is_head_piece;
                if ((gap_hi > row0 + kRowWindow && !is_tail_piece) || lead) {
                    const uint32_t slab_feats = min((uint32_t)kNs, p.n - f0);
                    const uint32_t vec_per_row = slab_feats / 4;
                    for (int pass = 0; pass < 2; ++pass) {
                        const uint32_t lo = pass == 0 ? row0 + kRowWindow : 0u;
                        const uint32_t hi = pass == 0 ? (is_tail_piece ? 0u : min(gap_hi, p.rows)) : (lead ? row0 : 0u);
                        for (uint32_t row = lo + q; row < hi; row += 4) {
                            for (uint32_t v4 = lane; v4 < vec_per_row; v4 += 32) {
                                const uint32_t feat = f0 + v4 * 4;
                                if (p.c_is_half)
                                    *reinterpret_cast<uint2 *>(static_cast<__half *>(p.C) + (int64_t)row * p.ldc + feat) = make_uint2(0, 0);
                                else
                                    *reinterpret_cast<float4 *>(static_cast<float *>(p.C) + (int64_t)row * p.ldc + feat) = make_float4(0, 0, 0, 0);
                            }
                        }
                    }
                }
                i += 2;
                while (i >= n_win) { i -= n_win; ++slab; }
#ifdef B200SPMM_PROFILE
                ++prof_windows;
#endif
            }
            g0 += total;
        }  // chunks
#ifdef B200SPMM_PROFILE
        if (tid == 0) {
            B200_PROF_STORE(8, clock64() - prof_start);
            B200_PROF_STORE(9, prof_wait_accfull);
            B200_PROF_STORE(10, prof_windows);
        }
#endif
    } else if (warp >= kFirstProducerWarp) {
        // =========================================================== producer warps
        const uint32_t pid = (uint32_t)(warp - kFirstProducerWarp);
        const uint32_t grp = pid / kProducerWarps;  // fills stages grp, grp + 2, grp + 4, ...
        const uint32_t pw = pid % kProducerWarps;   // with tile slots 2*pw and 2*pw + 1 of each of them
        constexpr uint32_t kTpw = kTilesPerWarp;
        const uint32_t half = (uint32_t)lane >> 4, hl = (uint32_t)lane & 15u;  // TMA gathers: lanes 16*j.. serve tile j of the warp
        // This warp's ring of column lists: slot (iteration % kIdxSlots) holds the CW indices of its
        // two tiles.  With compressed tiles the slot continues with the two bitmaps and three value offsets.
        constexpr uint32_t kSlotWords = Cfg::kSlotBytes / 4, kBitOff = kTpw * Cfg::kCW * 4, kNnzOff = kBitOff + kTpw * Cfg::kBitWords * 8;
        uint32_t *my_idx = idx_ring + pid * Cfg::kIdxSlots * kSlotWords;
        const uint32_t my_idx_addr = idx_ring_addr + pid * Cfg::kIdxSlots * Cfg::kSlotBytes;
        constexpr int kIdxLanes = Cfg::kCW * 4 / 16;  // lanes that copy one column list (16 bytes each)
        constexpr int kBitLanes = Cfg::kBitWords / 2;  // lanes that copy one bitmap

        // ---- per-lane constants of the gather
        // TMA: lane o issues gather instruction o of the tile: row quad g = o % kRowQuads of
        // 128-byte column block h = o / kRowQuads.
        uint32_t op_dst = 0, op_x = 0, op_quad = 0;
        if (kTma) {
            const uint32_t g = hl % Cfg::kRowQuads, h = hl / Cfg::kRowQuads;
            op_quad = g;
            op_x = h * Cfg::kBoxFeatures;
            // fp16: block (h, rows 8j..8j+7) is 1 KiB, a quad is half of it; tf32: block (h, quad) is 512 B
            op_dst = kTf32 ? (h * 2 + g) * 512u : (h * 2 + (g >> 1)) * 1024u + (g & 1u) * 512u;
        }
        // cp.async: copy i of a lane moves 16-byte piece (i*32 + lane) of the tile.
        const uint8_t *Bbytes = static_cast<const uint8_t *>(p.B);
        const uint64_t row_pitch = (uint64_t)p.ldb * Cfg::kEsz;
        constexpr int kCopies = kTma ? 1 : Cfg::kCopiesPerLane;
        uint32_t dst_off[kCopies];   // byte offset inside the tile's operand area, swizzled
        uint32_t src_off[kCopies];   // byte offset inside the slab's part of a B row
        uint32_t k_of[kCopies];      // which of the tile's CW rows
        if (!kTma) {
#pragma unroll
            for (int i = 0; i < kCopies; ++i) {
                const uint32_t q = i * 32 + lane;
                const uint32_t k = q / Cfg::kChunksPerRow, piece = q % Cfg::kChunksPerRow;
                const uint32_t h = piece >> 3, cc = piece & 7u;  // 128-byte column block, piece inside it
                if (kTf32) {
                    // 32-feature blocks of 4 k-rows x 128 B; 32-byte units are XORed with the row number
                    const uint32_t kr = k & 3u;
                    dst_off[i] = (h * 2 + (k >> 2)) * 512u + kr * 128u + ((((cc >> 1) ^ kr) << 5) | ((cc & 1u) << 4));
                } else {
                    // 64-feature blocks of 8 k-rows x 128 B; 16-byte units are XORed with the row number
                    const uint32_t kr = k & 7u;
                    dst_off[i] = (h * 2 + (k >> 3)) * 1024u + kr * 128u + ((cc ^ kr) << 4);
                }
                src_off[i] = piece * 16u;
                k_of[i] = k;
            }
        }

        bool failed = false;
        B200_PROF_DECL(prof_wait_empty);
        B200_PROF_DECL(prof_wait_group);
        B200_PROF_DECL(prof_issue);
        B200_PROF_DECL(prof_arrive);
#ifdef B200SPMM_PROFILE
        const long long prof_start = clock64();
#endif
        // Stage cursor of the main loop - (chunk, slab, stage inside the pass) with the chunk's
        // tile range - plus ring slot and use count, and a second cursor kIdxAhead iterations
        // further on for the column-list fetch.
        struct Cursor {
            uint32_t round, slab, sp, tile_begin, n_tiles, stages, done;
        };
        uint32_t grabbed = 1;  // first producer warp: entries of the CTA's chunk list written so far
        auto open_chunk = [&](Cursor &c) {  // the cursor enters its c.round-th chunk
            if (pid == 0 && c.round == grabbed) {  // nobody has asked for this one yet: claim the next chunk
                if (lane == 0) {
                    uint32_t next = kNoChunk;
                    if (p.sched_counter && c.round + 1 < (uint32_t)Cfg::kChunkSlots) {
                        next = p.chunk_begin + gridDim.x + atomicAdd(p.sched_counter, 1u);
                        if (next >= p.chunk_end) next = kNoChunk;
                    }
                    chunk_list[c.round] = next;
                    __threadfence_block();
                    *chunk_avail = c.round + 1;
                }
                ++grabbed;
                __syncwarp();
            }
            const uint32_t chunk = chunk_id(c.round);
            if (chunk == kNoChunk) {
                c.done = 1;
                return;
            }
            c.tile_begin = p.chunk_tile[chunk];
            c.n_tiles = p.chunk_tile[chunk + 1] - c.tile_begin;
            c.stages = (c.n_tiles + kTps - 1) / kTps;
        };
        auto normalise = [&](Cursor &c) {  // stage cursor past the end of a pass: next slab, then next chunk
            while (!c.done && c.sp >= c.stages) {
                c.sp -= c.stages;
                if (++c.slab == p.n_slabs || c.stages == 0) {
                    c.slab = 0;
                    ++c.round;
                    open_chunk(c);
                }
            }
        };
        Cursor cur{0, 0, grp, 0, 0, 0, 0};
        open_chunk(cur);
        normalise(cur);
        Cursor fc = cur;
        uint32_t s = grp, use = 0, s_arrive = grp;
        uint32_t it = 0, it_f = 0;  // iterations issued / fetched (only their low bits are used)
        auto fetch_list = [&]() {  // column list of the fetch cursor's tile -> its ring slot; then advance
            if (!fc.done) {
                const uint32_t tpos0 = fc.sp * kTps + pw * kTpw;
                if (tpos0 < fc.n_tiles) {
                    const uint32_t here = min(kTpw, fc.n_tiles - tpos0);  // the warp's tiles in this stage
                    const uint32_t slot_addr = my_idx_addr + (it_f % Cfg::kIdxSlots) * Cfg::kSlotBytes;
                    const uint64_t t = fc.tile_begin + tpos0;
                    constexpr uint32_t kL0 = kIdxLanes * kTpw, kL1 = kL0 + kBitLanes * kTpw;
                    if ((uint32_t)lane < kL0) {  // the tiles are neighbours: so are their lists, bitmaps and offsets
                        if ((uint32_t)lane / kIdxLanes < here)
                            ptx::cp_async_16(slot_addr + lane * 16, p.tcA2B + t * Cfg::kCW + lane * 4, 16u);
                    } else if (kBitmap && (uint32_t)lane < kL1) {
                        const uint32_t j = (uint32_t)lane - kL0;
                        if (j / kBitLanes < here)
                            ptx::cp_async_16(slot_addr + kBitOff + j * 16, p.tcBit + t * Cfg::kBitWords + j * 2, 16u);
                    } else if (kBitmap && (uint32_t)lane <= kL1 + here) {
                        const uint32_t j = (uint32_t)lane - kL1;
                        ptx::cp_async_4(slot_addr + kNnzOff + j * 4, p.nnzOffset + t + j);
                    }
                }
                fc.sp += kProducerGroups;
                normalise(fc);
            }
            ++it_f;
        };
        for (int i = 0; i < Cfg::kIdxAhead; ++i) fetch_list();
        ptx::cp_async_commit();
        ptx::cp_async_wait_group<0>();
        __syncwarp();

        // Compressed tiles.  Lane l owns the 16-byte piece of the tile that holds row l/2, columns
        // (l%2) * CW/2 ... of it: kPer slots, whose bits are consecutive in the bitmap.  The stored
        // values of a tile follow the bit order, so the lane's first value sits at the tile's
        // offset plus the number of bits set before its own.  The loads of the NEXT tile's values
        // are issued right after the current tile has been expanded and fenced - a proxy fence
        // waits for the thread's loads in flight, so none may be pending when it executes - and
        // have one whole iteration to land.
        constexpr int kPer = Cfg::kCW / 2;
        uint32_t my_vals[kTpw][kPer] = {};  // stored values (fp16 in the low half), zero where the bit is clear
        Cursor vc = cur;                    // the stage whose values are loaded next
        uint32_t it_v = 0;
        auto prefetch_values = [&]() {  // loads the value cursor's two tiles into my_vals, then advances the cursor
            if (!kBitmap) return;
            const uint32_t *slot_words = my_idx + (it_v % Cfg::kIdxSlots) * kSlotWords;
            const uint32_t tpos0 = vc.sp * kTps + pw * kTpw;
            const uint32_t here = (!vc.done && tpos0 < vc.n_tiles && !(B200_DEBUG_BITS(p) & 8u)) ? min(kTpw, vc.n_tiles - tpos0) : 0u;
#pragma unroll
            for (uint32_t j = 0; j < kTpw; ++j) {
#pragma unroll
                for (int b = 0; b < kPer; ++b) my_vals[j][b] = 0;
                if (j < here) {
                    const uint64_t *bits = reinterpret_cast<const uint64_t *>(slot_words + kBitOff / 4) + j * Cfg::kBitWords;
                    const uint32_t first_bit = (uint32_t)lane * kPer, w = first_bit >> 6, sh = first_bit & 63u;
                    uint32_t before = 0;
#pragma unroll
                    for (int k = 0; k < Cfg::kBitWords; ++k) before += (uint32_t)k < w ? (uint32_t)__popcll(bits[k]) : 0u;
                    const uint64_t word = bits[w];
                    before += (uint32_t)__popcll(word & ((1ull << sh) - 1ull));
                    const uint32_t mine = (uint32_t)(word >> sh) & ((1u << kPer) - 1u);
                    uint32_t idx = slot_words[kNnzOff / 4 + j] + before;
#pragma unroll
                    for (int b = 0; b < kPer; ++b) {
                        if (mine & (1u << b)) {
                            if (kTf32) my_vals[j][b] = __ldg(static_cast<const uint32_t *>(p.values) + idx);
                            else my_vals[j][b] = __ldg(static_cast<const uint16_t *>(p.values) + idx);
                            ++idx;
                        }
                    }
                }
            }
            if (!vc.done) {
                vc.sp += kProducerGroups;
                normalise(vc);
            }
            ++it_v;
        };
        // where the lane's piece goes: K-major rows of 32 bytes, 16-byte halves swapped in rows 4-7 and 12-15
        const uint32_t piece_off = ((uint32_t)lane >> 1) * 32u + ((((uint32_t)lane & 1u) ^ (((uint32_t)lane >> 3) & 1u)) << 4);
        prefetch_values();
        // Entry lists: lane l holds word l of the record of each of the warp's two tiles of the NEXT iteration
        // (loaded right after the current tiles were expanded and fenced, like the stored values above).
        uint32_t my_ent[kTpw] = {};
        Cursor ec = cur;
        auto prefetch_entries = [&]() {
            if (!kEntries) return;
            const uint32_t tpos0 = ec.sp * kTps + pw * kTpw;
            const uint32_t here = (!ec.done && tpos0 < ec.n_tiles) ? min(kTpw, ec.n_tiles - tpos0) : 0u;
#pragma unroll
            for (uint32_t j = 0; j < kTpw; ++j)
                my_ent[j] = (j < here && !(B200_DEBUG_BITS(p) & 8u)) ? __ldg(p.tile_entries + ((uint64_t)(ec.tile_begin + tpos0 + j) << 5) + lane) : kNoEntry;
            if (!ec.done) {
                ec.sp += kProducerGroups;
                normalise(ec);
            }
        };
        prefetch_entries();

        const uint32_t n_bytes = p.n * Cfg::kEsz;
        uint32_t issued = 0;  // cp.async path: stages whose copies were issued and not yet reported
        while (!cur.done) {
            const uint32_t slab = cur.slab, sp = cur.sp, tile_begin = cur.tile_begin;
            const uint32_t tpos0 = sp * kTps + pw * kTpw;
            // the warp's tiles in this stage (the last stage of a pass may be short), and those it gathers rows for
            const uint32_t here = tpos0 < cur.n_tiles ? min(kTpw, cur.n_tiles - tpos0) : 0u;
            const uint32_t gather_here = (B200_DEBUG_BITS(p) & 1u) ? 0u : here;
            const uint32_t *slot_words = my_idx + (it % Cfg::kIdxSlots) * kSlotWords;
            const uint32_t first_slot = s * kTps + pw * kTpw;  // the warp's first tile slot of the ring

            // One lane polls (every mbarrier operation costs a shared-memory pipeline slot per
            // thread); the shuffle hands the verdict to the warp and lines the lanes up again.
            uint32_t ok = 1;
            if (lane == 0) {
                {
                    B200_PROF_T0();
                    ok = ptx::mbar_wait(empty_bar(s), (use & 1u) ^ 1u, abort_flag, limit) ? 1u : 0u;
                    B200_PROF_ADD(prof_wait_empty);
                }
                if (ok && kTiles == 0) {
                    const bool a_tiles = pw == 0 && !(B200_DEBUG_BITS(p) & 4u);
                    // the stage's eight A tiles (tiles past the chunk's end are fetched too, as long as the
                    // array holds them: they are never multiplied)
                    const uint32_t first_tile = tile_begin + sp * kTps;
                    const uint32_t a_bytes = p.tiles_image ? min((uint32_t)kTps, p.total_tiles - first_tile) * kATileBytes
                                                           : (uint32_t)kTps * kATileBytes;
                    if (kTma) {
                        // this warp's arrival, announcing the bytes its TMA loads will deliver
                        const uint32_t bytes = gather_here * Cfg::kGatherBytes + (a_tiles ? a_bytes : 0u);
                        ptx::mbar_arrive_expect_tx(full_bar(s), bytes);
                    } else if (a_tiles) {
                        ptx::mbar_expect_tx(full_bar(s), a_bytes);
                    }
                    if (a_tiles) {
                        if (p.tiles_image)  // one bulk copy from the shared-memory image
                            ptx::bulk_load(atile_addr + s * kTps * kATileBytes, p.tiles_image + (uint64_t)first_tile * kATileBytes,
                                           a_bytes, full_bar(s));
                        else  // the caller's array as it is: 128 rows of 32 bytes through the swizzling tensor map
                            ptx::tma_load_2d(atile_addr + s * kTps * kATileBytes, &tmap_a, 0,
                                             (int32_t)(first_tile * kRowWindow), full_bar(s));
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { failed = true; break; }
            if (kBitmap) {
                // expand this warp's tiles into their 512 bytes of the stage, then announce the gathers' bytes
                if (here && !(B200_DEBUG_BITS(p) & 4u)) {
#pragma unroll
                    for (uint32_t j = 0; j < kTpw; ++j) {
                        if (j < here) {
                            uint4 piece;
                            const uint32_t *v = my_vals[j];
                            if constexpr (kTf32) {
                                piece = make_uint4(v[0], v[1], v[2], v[3]);
                            } else {
                                piece = make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
                            }
                            ptx::st_shared_v4(atile_addr + (first_slot + j) * kATileBytes + piece_off, piece);
                        }
                    }
                    ptx::fence_proxy_async_smem();
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_expect_tx(full_bar(s), gather_here * Cfg::kGatherBytes);
                prefetch_values();  // the next iteration's, whose slot landed an iteration ago (see the wait below)
            }
            if (kTma) {
                B200_PROF_T0();
                if (half < gather_here && hl < (uint32_t)Cfg::kGatherOps) {
                    const uint4 rows4 = *reinterpret_cast<const uint4 *>(slot_words + half * Cfg::kCW + op_quad * 4);
                    // padded slots hold 0xFFFFFFFF: clamp to the first row past the end, which reads zeros
                    ptx::tma_gather4_2d(gather_addr + (first_slot + half) * Cfg::kGatherBytes + op_dst, &tmap_b,
                                        (int32_t)(slab * kNs + op_x),
                                        (int32_t)min(rows4.x, p.cols), (int32_t)min(rows4.y, p.cols),
                                        (int32_t)min(rows4.z, p.cols), (int32_t)min(rows4.w, p.cols), full_bar(s));
                }
                if (kEntries) {  // after the gathers were issued: the expansion runs while they are in flight (their bytes may
                                 // be counted before this warp announces them: the phase cannot end before its arrival)
                    // expand this warp's tiles: zeros, then every lane drops its entry at its place; a tile with more
                    // than 32 entries comes whole from the tile image instead (async proxy: no zero fill for it)
                    uint32_t n_dense = 0;
                    if (here && !(B200_DEBUG_BITS(p) & 4u)) {
#pragma unroll
                        for (uint32_t j = 0; j < kTpw; ++j)
                            if (j < here && my_ent[j] != kDenseTile)
                                ptx::st_shared_v4(atile_addr + (first_slot + j) * kATileBytes + (uint32_t)lane * 16u, make_uint4(0, 0, 0, 0));
                        __syncwarp();
#pragma unroll
                        for (uint32_t j = 0; j < kTpw; ++j) {
                            if (j < here) {
                                const uint32_t e = my_ent[j];
                                if (e == kDenseTile) ++n_dense;
                                else if ((e >> 16) != 0xFFFFu)
                                    ptx::st_shared_u16(atile_addr + (first_slot + j) * kATileBytes + (e >> 16), (uint16_t)e);
                            }
                        }
                        ptx::fence_proxy_async_smem();
                    }
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive_expect_tx(full_bar(s), gather_here * Cfg::kGatherBytes + n_dense * kATileBytes);
#pragma unroll
                        for (uint32_t j = 0; j < kTpw; ++j)
                            if (j < here && my_ent[j] == kDenseTile && !(B200_DEBUG_BITS(p) & 4u))
                                ptx::bulk_load(atile_addr + (first_slot + j) * kATileBytes,
                                               p.tiles_image + (uint64_t)(tile_begin + tpos0 + j) * kATileBytes, kATileBytes, full_bar(s));
                    }
                    prefetch_entries();
                }
                fetch_list();
                ptx::cp_async_commit();
                // The list needed next iteration was fetched kIdxAhead groups ago: this only blocks
                // when that many groups are still pending, and makes the guarantee explicit.
                ptx::cp_async_wait_group<Cfg::kIdxAhead - Cfg::kSlotLead>();
                __syncwarp();
                B200_PROF_ADD(prof_issue);
            } else {
                {
                    B200_PROF_T0();
                    const uint32_t slab_byte0 = slab * kNs * Cfg::kEsz;
#pragma unroll
                    for (uint32_t j = 0; j < kTpw; ++j) {
                        if (j < gather_here) {
                            const uint32_t *list = slot_words + j * Cfg::kCW;
                            const uint32_t tile_area = gather_addr + (first_slot + j) * Cfg::kGatherBytes;
#pragma unroll
                            for (int i = 0; i < kCopies; ++i) {
                                const uint32_t col = list[k_of[i]];
                                const uint32_t in_row = slab_byte0 + src_off[i];
                                const bool live = col < p.cols && in_row < n_bytes;  // padded slots hold 0xFFFFFFFF
                                const uint8_t *src = live ? Bbytes + (uint64_t)col * row_pitch + in_row : Bbytes;
                                ptx::cp_async_16(tile_area + dst_off[i], src, live ? 16u : 0u);
                            }
                        }
                    }
                    fetch_list();  // rides in the same group as this tile's rows
                    ptx::cp_async_commit();
                    B200_PROF_ADD(prof_issue);
                }
                ++issued;
                if (issued > (uint32_t)Cfg::kLag) {  // the copies issued kLag stages ago have landed
                    {
                        B200_PROF_T0();
                        ptx::cp_async_wait_group<Cfg::kLag>();
                        B200_PROF_ADD(prof_wait_group);
                    }
                    B200_PROF_T0();
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(full_bar(s_arrive));
                    s_arrive += kProducerGroups;
                    if (s_arrive >= (uint32_t)kStages) s_arrive -= kStages;
                    --issued;
                    B200_PROF_ADD(prof_arrive);
                }
            }
            ++it;
            cur.sp += kProducerGroups;
            normalise(cur);
            s += kProducerGroups;
            if (s >= (uint32_t)kStages) { s -= kStages; ++use; }
        }
#ifdef B200SPMM_PROFILE
        if (lane == 0 && pid == 1) {
            B200_PROF_STORE(0, clock64() - prof_start);
            B200_PROF_STORE(1, prof_wait_empty);

            B200_PROF_STORE(3, it);
            B200_PROF_STORE(11, prof_issue);
            B200_PROF_STORE(12, prof_arrive);
        }
#endif
        // drain: everything this warp issued has to land before the CTA may exit
        ptx::cp_async_wait_group<0>();
        __syncwarp();
        if (!kTma) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (!failed && lane == 0) {
                for (; issued > 0; --issued) {
                    ptx::mbar_arrive(full_bar(s_arrive));
                    s_arrive += kProducerGroups;
                    if (s_arrive >= (uint32_t)kStages) s_arrive -= kStages;
                }
            }
        }
        (void)failed; (void)n_bytes; (void)Bbytes; (void)row_pitch; (void)op_dst; (void)op_x; (void)op_quad; (void)s_arrive;
    } else if (warp == kMmaWarp && lane == 0) {
        // =========================================================== MMA issuer (warp 8, lane 0)
        // A single thread: every instruction it executes per tile is on the critical path, so the
        // loop is kept to a wait per eight tiles, one or two MMAs per tile and a commit per eight
        // tiles.  The tile counts of the next kWinAhead windows are prefetched into shared memory
        // with 4-byte cp.async copies, one group per window.
        constexpr uint32_t fmt = kTf32 ? ptx::kFmtTF32 : ptx::kFmtF16;
        constexpr uint32_t idesc_full = ptx::make_instr_desc(fmt, 128, kRowWindow, true, false);
        constexpr uint32_t idesc_half = ptx::make_instr_desc(fmt, 64, kRowWindow, true, false);
        // gathered-B operand: MN-major, 128-byte swizzle.  fp16: 64-feature blocks 2 KiB apart,
        // 8-row groups 1 KiB apart, 16-byte swizzle units.  tf32: the only MN-major layout for
        // 32-bit operands swizzles 32-byte units over groups of 4 rows: 32-feature blocks
        // 1 KiB apart, 4-row groups 512 B apart.
        constexpr uint32_t a_lbo = kTf32 ? 1024u : 2048u, a_sbo = kTf32 ? 512u : 1024u;
        // Descriptors are handled as 32-bit halves: the high word is constant, the low word is
        // (leading byte offset << 16) | (address >> 4), so moving to another tile is one add.
        const uint64_t a_desc0 =
            ptx::make_smem_desc(gather_addr, a_lbo, a_sbo, kTf32 ? ptx::kSwizzle128BBase32B : ptx::kSwizzle128B);
        // A-tile operand: K-major, 32-byte swizzle, 8-row groups 256 bytes apart.
        const uint64_t b_desc0 = ptx::make_smem_desc(atile_addr, 16, 256, ptx::kSwizzle32B);
        const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
        const uint32_t a_lo0 = (uint32_t)a_desc0, b_lo0 = (uint32_t)b_desc0;  // stage 0, tile slot 0
        constexpr uint32_t kATile16 = kATileBytes >> 4, kGather16 = Cfg::kGatherBytes >> 4;
        uint32_t s = 0, phase = 0;   // ring stage in use and the parity of its current use
        uint32_t slot = 0;           // next tile slot inside the stage; 0 = the stage still has to be awaited
        uint32_t ad_lo = a_lo0, bd_lo = b_lo0;  // low descriptor words of tile (s, slot)
        uint32_t acc_it = 0;
        bool alive = true;
        const bool do_mma = !(B200_DEBUG_BITS(p) & 2u);
        B200_PROF_DECL(prof_wait_full);
        B200_PROF_DECL(prof_wait_acc);
        B200_PROF_DECL(prof_mma);
        B200_PROF_DECL(prof_commit);
        B200_PROF_DECL(prof_head);
        B200_PROF_DECL(prof_tail);
#ifdef B200SPMM_PROFILE
        long long prof_tiles = 0;
        const long long prof_start = clock64();
#endif
        auto release_stage = [&]() {  // the stage's operands are free once the MMAs issued so far are done
            B200_PROF_T0();
            ptx::umma_commit(empty_bar(s));
            slot = 0;
            if (++s == (uint32_t)kStages) {
                s = 0;
                phase ^= 1u;
                ad_lo = a_lo0;
                bd_lo = b_lo0;
            }
            B200_PROF_ADD(prof_commit);
        };
        auto issue = [&](uint32_t d, uint32_t alo, uint32_t blo, uint32_t idesc, uint32_t acc) {
            if (kTf32) ptx::umma_tf32_ss_lohi(d, alo, a_hi, blo, b_hi, idesc, acc);
            else ptx::umma_f16_ss_lohi(d, alo, a_hi, blo, b_hi, idesc, acc);
        };
        for (uint32_t round = 0; alive; ++round) {
            const uint32_t chunk = chunk_id(round);
            if (chunk == kNoChunk) break;
            const Chunk ch = load_chunk(chunk);
            const uint32_t n_win = ch.n_win, w_begin = ch.w_begin, tile_begin = ch.tile_begin, tile_end = ch.tile_end;
            for (uint32_t slab = 0; slab < p.n_slabs && alive; ++slab) {
                // window i's last tile + 1 goes to slot i % kWinSlots, one cp.async group per window
                for (uint32_t i = 0; i < (uint32_t)Cfg::kWinAhead; ++i) {
                    if (i < n_win) ptx::cp_async_4(win_ends_addr + (i % Cfg::kWinSlots) * 4, p.rowOffset + w_begin + i + 1);
                    ptx::cp_async_commit();
                }
                uint32_t off_lo = tile_begin;
                for (uint32_t i = 0; i < n_win && alive; ++i, ++acc_it) {
#ifdef B200SPMM_PROFILE
                    const long long prof_h0 = clock64();
#endif
                    const uint32_t ahead = i + Cfg::kWinAhead;
                    if (ahead < n_win) ptx::cp_async_4(win_ends_addr + (ahead % Cfg::kWinSlots) * 4, p.rowOffset + w_begin + ahead + 1);
                    ptx::cp_async_commit();
                    ptx::cp_async_wait_group<Cfg::kWinAhead>();  // window i's group has landed
                    const uint32_t off_hi = min(win_ends[i % Cfg::kWinSlots], tile_end);  // the last window may be cut
#ifdef B200SPMM_PROFILE
                    prof_head += clock64() - prof_h0;
                    prof_tiles += off_hi - off_lo;
#endif
                    uint32_t nt = off_hi - off_lo;
                    off_lo = off_hi;
                    const uint32_t a = acc_it & 1u;
                    {
                        B200_PROF_T0();
                        alive = ptx::mbar_wait(acc_empty_bar(a), ((acc_it >> 1) & 1u) ^ 1u, abort_flag, limit);
                        ptx::tcgen05_fence_after_sync();
                        B200_PROF_ADD(prof_wait_acc);
                    }
                    const uint32_t d = tmem_base + a * kAccCols;
                    uint32_t accumulate = 0;
                    // A segment is the run of tiles that share a ring stage and a window: at most eight.
                    // Branches are what a lone thread can least afford, so the window is walked as
                    //   head - the rest of a stage the previous window left partly used,
                    //   body - whole stages: wait, eight MMAs, commit; ring bookkeeping by selects,
                    //   tail - the first tiles of a stage the next window will finish.
                    // `count` MMAs (a compile-time number) for the tiles q0 .. of the current segment
                    auto burst = [&](auto count_tag, uint32_t q0) {
                        constexpr int kCount = decltype(count_tag)::value;
                        const uint32_t alo0 = ad_lo + q0 * kGather16, blo0 = bd_lo + q0 * kATile16;
#pragma unroll
                        for (int q = 0; q < kCount; ++q) {
#pragma unroll
                            for (int c = 0; c < Cfg::kChunks; ++c) {
                                const bool half_chunk = Cfg::kHalfChunk && c == Cfg::kFullChunks;
                                issue(d + c * 16, alo0 + q * kGather16 + c * 256u, blo0 + q * kATile16,
                                      half_chunk ? idesc_half : idesc_full, q == 0 ? accumulate : 1u);
                            }
                        }
                        accumulate = 1;
                    };
                    // k tiles starting at (s, slot), 0 < k < 8: bursts of four, two and one.  (Eight predicated
                    // MMAs, of which the dead ones still cost the thread 30-40 clocks each, were slower: on a
                    // graph with 15 tiles per window 24 slots were walked for 15 MMAs.)
                    auto partial = [&](uint32_t k) {
                        B200_PROF_T0();
                        if (do_mma) {
                            uint32_t q0 = 0;
                            if (k & 4u) { burst(std::integral_constant<int, 4>{}, q0); q0 = 4; }
                            if (k & 2u) { burst(std::integral_constant<int, 2>{}, q0); q0 += 2; }
                            if (k & 1u) burst(std::integral_constant<int, 1>{}, q0);
                        }
                        accumulate = 1;
                        nt -= k;
                        slot += k;
                        ad_lo += k * kGather16;
                        bd_lo += k * kATile16;
                        B200_PROF_ADD(prof_mma);
                    };
                    auto await_stage = [&]() {  // the operands of stage s must have landed
                        B200_PROF_T0();
                        alive = ptx::mbar_wait(full_bar(s), phase, abort_flag, limit);
                        ptx::tcgen05_fence_after_sync();
                        B200_PROF_ADD(prof_wait_full);
                    };
                    if (slot != 0 && alive) {  // head
                        partial(min(nt, (uint32_t)kTps - slot));
                        if (slot == (uint32_t)kTps) release_stage();
                    }
                    while (nt >= (uint32_t)kTps && alive) {  // body: slot == 0 here
                        await_stage();
                        if (!alive) break;
                        {
                            B200_PROF_T0();
                            if (do_mma) {
#pragma unroll
                                for (int q = 0; q < kTps; ++q) {
#pragma unroll
                                    for (int c = 0; c < Cfg::kChunks; ++c) {
                                        const bool half_chunk = Cfg::kHalfChunk && c == Cfg::kFullChunks;
                                        issue(d + c * 16, ad_lo + q * kGather16 + c * 256u, bd_lo + q * kATile16,
                                              half_chunk ? idesc_half : idesc_full, q == 0 ? accumulate : 1u);
                                    }
                                }
                            }
                            B200_PROF_ADD(prof_mma);
                        }
                        accumulate = 1;
                        nt -= kTps;
                        {
                            B200_PROF_T0();
                            ptx::umma_commit(empty_bar(s));
                            const bool wrap = s + 1 == (uint32_t)kStages;  // selects, no branch
                            s = wrap ? 0u : s + 1;
                            phase ^= wrap ? 1u : 0u;
                            ad_lo = wrap ? a_lo0 : ad_lo + kTps * kGather16;
                            bd_lo = wrap ? b_lo0 : bd_lo + kTps * kATile16;
                            B200_PROF_ADD(prof_commit);
                        }
                    }
                    if (nt != 0 && alive) {  // tail: slot == 0, 0 < nt < 8
                        await_stage();
                        if (alive) partial(nt);
                    }
                    {
                        B200_PROF_T0();
                        if (alive) ptx::umma_commit(acc_full_bar(a));
                        B200_PROF_ADD(prof_tail);
                    }
                }
                // a pass ends on a stage boundary: give back a partly used last stage
                if (slot != 0 && alive) {
                    ad_lo += ((uint32_t)kTps - slot) * kGather16;
                    bd_lo += ((uint32_t)kTps - slot) * kATile16;
                    release_stage();
                }
            }
        }  // chunks
        ptx::cp_async_wait_group<0>();
        if (!alive || *abort_flag) {
            // Gave up, possibly in the middle of a window: MMAs may have been issued that no commit covers yet.
            // They read shared memory and write TMEM, so they must be finished before the CTA frees
            // either: one more commit, and a wait (bounded like every other) for its arrival.
            ptx::umma_commit(drain_bar);
            ptx::mbar_wait_bounded(drain_bar, 0, limit);
            ptx::tcgen05_fence_after_sync();
        }
#ifdef B200SPMM_PROFILE
        B200_PROF_STORE(4, clock64() - prof_start);
        B200_PROF_STORE(5, prof_wait_full);
        B200_PROF_STORE(6, prof_wait_acc);
        B200_PROF_STORE(7, prof_tiles);
        B200_PROF_STORE(13, prof_mma);
        B200_PROF_STORE(14, prof_commit);
        B200_PROF_STORE(15, prof_head);
        B200_PROF_STORE(2, prof_tail);
#endif
    }

    // The idle lanes of the MMA warp sleep until lane 0 is done instead of waiting at the CTA
    // barrier below while their warp-mate is still issuing.
    if (warp == kMmaWarp) {
        if (lane == 0) {
            *mma_done = 1;
        } else {
            while (*mma_done == 0) __nanosleep(2000);
        }
        __syncwarp();
    }
    // ---- teardown: every role ends up here, on success and on timeout alike
    if (*abort_flag) {
        // After a failure TMA loads may still be on their way into this CTA's shared memory: the
        // producers stop at their next wait, which can be right after an issue, and a load whose
        // barrier phase never completes offers nothing to wait on.  The thread that gave up has
        // already waited the full limit; everybody else stays this long after its last instruction,
        // many times the latency of a load, before the CTA lets go of its shared memory.
        const uint64_t t0 = ptx::global_timer_ns();
        while (ptx::global_timer_ns() - t0 < kAbortLingerNs) __nanosleep(1000);
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
    if (tid == 0 && *abort_flag) atomicOr(p.status, kDevStatusTimeout);
    if (tid == 0 && p.sched_counter) {  // the last CTA to finish leaves both counters at zero for the next launch
        __threadfence();
        if (atomicAdd(p.sched_counter + 1, 1u) == gridDim.x - 1u) {
            p.sched_counter[0] = 0;
            p.sched_counter[1] = 0;
        }
    }
#ifdef B200SPMM_PROFILE
    if (tid == 0) {  // where and when this CTA ran
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        B200_PROF_STORE(16, smid);
        B200_PROF_STORE(17, prof_cta_t0);
        B200_PROF_STORE(18, ptx::global_timer_ns());
    }
#endif
}

// A window whose tiles were shared out over several CTAs: pieces piece_begin .. piece_end-1 of
// piece_slots name the partial-result slots that hold its pieces, in tile order.
struct SplitWindow {
    uint32_t window, piece_begin, piece_end;
};

// Sums the pieces of every split window in a fixed order and writes the window's rows of C.
// One CTA per split window; thread t handles four consecutive features of one row at a time.
__global__ void __launch_bounds__(256)
spmm_fixup_kernel(const SplitWindow *__restrict__ splits, const uint32_t *__restrict__ piece_slots,
                  const float *__restrict__ partial, const uint32_t *__restrict__ rowIdx, void *__restrict__ C,
                  int64_t ldc, uint32_t rows, uint32_t n, uint32_t c_is_half) {
    const SplitWindow sp = splits[blockIdx.x];
    const uint32_t row0 = rowIdx[sp.window];
    const uint32_t vec_per_row = n / 4;
    for (uint32_t idx = threadIdx.x; idx < kRowWindow * vec_per_row; idx += blockDim.x) {
        const uint32_t r = idx / vec_per_row, c4 = idx % vec_per_row;
        if (row0 + r >= rows) continue;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t k = sp.piece_begin; k < sp.piece_end; ++k) {
            const float4 v = *reinterpret_cast<const float4 *>(partial + ((size_t)piece_slots[k] * kRowWindow + r) * n + c4 * 4);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (c_is_half) {
            __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t *>(&lo);
            packed.y = *reinterpret_cast<uint32_t *>(&hi);
            *reinterpret_cast<uint2 *>(static_cast<__half *>(C) + (int64_t)(row0 + r) * ldc + c4 * 4) = packed;
        } else {
            *reinterpret_cast<float4 *>(static_cast<float *>(C) + (int64_t)(row0 + r) * ldc + c4 * 4) = acc;
        }
    }
}

}  // namespace b200spmm
