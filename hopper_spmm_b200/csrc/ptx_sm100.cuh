// Inline-PTX layer for sm_100a: mbarrier (bounded waits), TMA tiled / gather4 loads,
// cp.async row gathers, tcgen05 (TMEM allocation, MMA, commit, load) and the shared-memory /
// instruction descriptors they consume.  Takes the place of the reference's sm_90a wrappers
// (src/ptx/barrier.h, src/ptx/tma.h, src/ptx/wgmma.h, src/ptx/ptx_utils.h).
//
// Unlike the reference's mbarrier_wait (src/ptx/barrier.h:29-41), every wait here gives up
// after a time limit and reports it, so a broken pipeline ends the kernel instead of hanging
// the device.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200spmm {
namespace ptx {

#define B200_DEVICE __device__ __forceinline__

B200_DEVICE uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

B200_DEVICE uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

B200_DEVICE bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------ mbarrier

B200_DEVICE void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

B200_DEVICE void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

B200_DEVICE void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Adds `bytes` to the transaction count the current phase waits for, without arriving.
B200_DEVICE void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

B200_DEVICE void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

B200_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Wait for the phase with the given parity to complete.  Returns false when `*abort_flag`
// (shared memory) is raised by another role or when `limit_ns` elapses, in which case this
// thread raises the flag itself.  The caller must then leave its loop.
B200_DEVICE bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// The same wait without an abort flag: for the teardown after a failure, where the flag is already
// up and the waiter only wants its own outstanding work to finish (or the time to run out).
B200_DEVICE bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0 && global_timer_ns() - t0 > limit_ns) return false;
    }
}

// ------------------------------------------------------------------ proxies and fences

// Orders this thread's generic-proxy shared-memory accesses with async-proxy accesses
// (TMA, tcgen05.mma operand reads).
B200_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

B200_DEVICE void tcgen05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
B200_DEVICE void tcgen05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

B200_DEVICE void named_barrier_sync(uint32_t id, uint32_t n_threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

// ------------------------------------------------------------------ TMA loads (own HBM only)

B200_DEVICE void prefetch_tensormap(const void *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// 2-D tiled load: box at (x, y) -> smem, completion as bytes on `bar`.
// x * element size must be a multiple of 16 bytes.
B200_DEVICE void tma_load_2d(uint32_t dst, const void *tmap, int32_t x, int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Plain bulk copy global -> shared of `bytes` contiguous bytes (a multiple of 16, both addresses
// 16-byte aligned), completion counted in bytes on `bar`.  One request whatever the size, where a
// tiled load of narrow rows costs the TMA unit one request per row.
B200_DEVICE void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Gather of four rows y0..y3 of a 2-D tensor, box width taken from the tensor map, starting at
// column x.  The four rows land one after another in shared memory.
B200_DEVICE void tma_gather4_2d(uint32_t dst, const void *tmap, int32_t x, int32_t y0, int32_t y1, int32_t y2,
                                int32_t y3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
        "%4, %5, %6}], [%7];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(bar)
        : "memory");
}

B200_DEVICE void st_shared_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
B200_DEVICE void st_shared_u16(uint32_t addr, uint16_t v) {
    asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}

// ------------------------------------------------------------------ cp.async (16-byte gathers)

// Copies 16 bytes global -> shared, bypassing L1; src_bytes < 16 zero-fills the rest
// (src_bytes == 0 reads nothing and writes 16 zero bytes).
B200_DEVICE void cp_async_16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Copies 4 bytes global -> shared (cached in L1: neighbouring words are fetched next).
B200_DEVICE void cp_async_4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
B200_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Makes `bar` receive one arrival (counted among the expected ones) once every cp.async this
// thread has issued so far has completed.
B200_DEVICE void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
template <int N>
B200_DEVICE void cp_async_wait_group() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------ tensor memory

// Whole-warp calls.  `n_cols` is a power of two in [32, 512]; the base address is written to
// shared memory at `dst_smem`.
B200_DEVICE void tmem_alloc(uint32_t dst_smem, uint32_t n_cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(n_cols)
                 : "memory");
}
B200_DEVICE void tmem_relinquish_alloc_permit() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
B200_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t n_cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(n_cols) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp receives lane
// (taddr.lane + i), columns taddr.col .. +15.  A warp may only touch the 32 lanes of its own
// quarter: lanes 32*(warp_id % 4) .. +31.
B200_DEVICE void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i receives lane (taddr.lane + i), columns
// taddr.col .. +31, i.e. 128 contiguous bytes of one accumulator row.
B200_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
B200_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ CTA pairs (cta_group::2)
// A cluster of two CTAs on neighbouring SMs can run ONE tcgen05.mma of M = 256: CTA r holds rows
// 128 r .. of A and of the accumulator and columns (N / 2) r .. of B in its own shared / tensor memory, at
// the same offsets in both CTAs; the even CTA (rank 0) issues.  Every byte of B is then fetched from L2
// by one of the two SMs only.

B200_DEVICE uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
B200_DEVICE void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
B200_DEVICE void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// The address of `local_smem_addr` in the shared memory of CTA `rank` of this cluster.
B200_DEVICE uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
// One arrival on a barrier that may live in the other CTA of the cluster (address from map_to_cta).
B200_DEVICE void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// The same without ordering of this thread's earlier memory operations (for data that another proxy wrote
// and whose completion this thread has already observed).
B200_DEVICE void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
B200_DEVICE void tmem_alloc_pair(uint32_t dst_smem, uint32_t n_cols) {  // whole warp, the same warp in both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(n_cols) : "memory");
}
B200_DEVICE void tmem_relinquish_alloc_permit_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
B200_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t n_cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(n_cols) : "memory");
}
// D (+)= A * B over the pair; issued by ONE thread of the even CTA.  `on` == 0 skips it.
B200_DEVICE void umma_pair_ss_lohi_if(bool tf32, uint32_t on, uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                      uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    if (tf32)
        asm volatile(
            "{\n.reg .pred p, q;\n.reg .b64 da, db;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
            "setp.ne.b32 p, %6, 0;\nsetp.ne.b32 q, %7, 0;\n"
            "@q tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %5, p;\n}\n"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(on) : "memory");
    else
        asm volatile(
            "{\n.reg .pred p, q;\n.reg .b64 da, db;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
            "setp.ne.b32 p, %6, 0;\nsetp.ne.b32 q, %7, 0;\n"
            "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n}\n"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(on) : "memory");
}
// One arrival on the barrier at offset `bar` in BOTH CTAs of the pair (mask 0b11) when every MMA this
// thread issued so far has finished.
B200_DEVICE void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// The same, arriving on the issuing CTA's barrier only.
B200_DEVICE void umma_commit_pair_local(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
B200_DEVICE void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// mbar_wait for a barrier on which the other CTA of the cluster arrives: acquire at cluster scope.
B200_DEVICE bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
B200_DEVICE bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint64_t limit_ns) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------ tcgen05.mma

// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4          [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4     [46,48) version = 1
//   [49,52) base offset = 0             [61,64) swizzle: 0 none, 1 128B over 32-byte units,
//                                               2 128B, 4 64B, 6 32B (16-byte units)
enum : uint32_t { kSwizzleNone = 0, kSwizzle128BBase32B = 1, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6 };

B200_DEVICE uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(swizzle & 7u) << 61;
    return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation:
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format  (0 f16, 1 bf16, 2 tf32)
//   [15] A is MN-major   [16] B is MN-major   [17,23) N >> 3   [24,29) M >> 4
enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };

__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t fmt, uint32_t m, uint32_t n, bool a_mn_major,
                                                       bool b_mn_major) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  accumulate == 0 overwrites D.
B200_DEVICE void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
B200_DEVICE void umma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Descriptors given as 32-bit halves (the high words are loop constants, the low words change by
// one add per tile).
B200_DEVICE void umma_f16_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "setp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same, issued only when `on` is non-zero (predicated, no branch).
B200_DEVICE void umma_f16_ss_lohi_if(uint32_t on, uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                    uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "setp.ne.b32 p, %6, 0;\n"
        "setp.ne.b32 q, %7, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(on)
        : "memory");
}
// Descriptors given as 32-bit halves (the high words are loop constants, the low words change by
// one add per tile).
B200_DEVICE void umma_tf32_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "setp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same, issued only when `on` is non-zero (predicated, no branch).
B200_DEVICE void umma_tf32_ss_lohi_if(uint32_t on, uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                    uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "setp.ne.b32 p, %6, 0;\n"
        "setp.ne.b32 q, %7, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(on)
        : "memory");
}

// Makes `bar` receive one arrival when every tcgen05.mma this thread issued so far has
// finished (implies tcgen05.fence::before_thread_sync).
B200_DEVICE void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace ptx
}  // namespace b200spmm
