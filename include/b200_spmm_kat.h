/*
 * b200_spmm_kat.h - single-tile known-answer entry points for the sm_100a primitives the
 * SpMM kernels are built from.  They take the place of the reference's stand-alone bring-up
 * programs: src/test_fp16.cu (one fp16 MMA tile), test/02.tma_and_wgmma/tma_wgmma.cu (one tf32
 * MMA tile), test/01.tma_copy_matrix/copy.cu (a TMA box landing in shared memory) and
 * test/03.warp_specialized/main.cu (tiles accumulated through a ring).
 *
 * Each call runs one CTA on `device`, is synchronous, takes HOST pointers and returns a
 * B200SPMM_* status (b200_spmm.h).  Waits inside the kernels are bounded: a pipeline that never
 * completes yields B200SPMM_ERR_DEVICE_TIMEOUT, not a hang.
 */
#ifndef B200_SPMM_KAT_H_
#define B200_SPMM_KAT_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One tcgen05.mma: operands described relative to the start of the shared-memory image. */
typedef struct {
    uint32_t a_off, a_lbo, a_sbo, a_swizzle; /* byte offset / leading / stride / swizzle code (0,2,4,6) */
    uint32_t b_off, b_lbo, b_sbo, b_swizzle;
    uint32_t idesc;      /* instruction descriptor                         */
    uint32_t d_col;      /* first TMEM column of the accumulator           */
    uint32_t accumulate; /* 0 = overwrite D, 1 = add to D                  */
    uint32_t kind;       /* 0 = kind::f16, 1 = kind::tf32                  */
} b200spmm_kat_mma_t;

/*
 * Copies `image` (image_bytes <= 96 KiB) into 1024-byte-aligned shared memory, issues the listed
 * MMAs in order from one thread, then dumps TMEM lanes 0..127 x columns 0..n_cols-1 as fp32 into
 * out[128 * n_cols].  n_cols is a multiple of 16, at most 256.
 * Replaces tma_wgmma_kernel + test_result_cpu (src/test_fp16.cu:238-315).
 */
int b200spmm_kat_umma(const void *image, uint32_t image_bytes, const b200spmm_kat_mma_t *mmas, int n_mmas,
                      int n_cols, float *out, int device);

/*
 * The same for the MMA of a CTA pair (tcgen05.mma.cta_group::2, M = 256): `images` holds two images of
 * image_bytes each, one per CTA of a two-CTA cluster (CTA r: rows 128 r .. of operand A and columns
 * (N / 2) r .. of operand B, at the same offsets in both images); the even CTA issues the listed MMAs;
 * out[2][128][n_cols] receives each CTA's 128 lanes of tensor memory (rows 128 r .. of D).  The reference
 * has no counterpart (its wgmma tiles live in one SM: src/fp16.cu:147).
 */
int b200spmm_kat_umma_pair(const void *images, uint32_t image_bytes, const b200spmm_kat_mma_t *mmas, int n_mmas,
                           int n_cols, float *out, int device);

/*
 * Sets how long a wait inside the known-answer kernels may last, in nanoseconds (0 restores the
 * default of two seconds), and returns the previous value.  A test shortens it, hands
 * b200spmm_kat_tma an expect_bytes larger than its loads deliver and must get
 * B200SPMM_ERR_DEVICE_TIMEOUT back - the bounded wait that replaces the reference's endless
 * mbarrier spin (src/ptx/barrier.h:29-41) - with the device still usable afterwards.
 */
unsigned long long b200spmm_kat_wait_limit(unsigned long long limit_ns);

/*
 * The whole SpMM kernel with a failure made on the host: the product of `plan` (b200_spmm.h) is
 * launched with a tensor map over B whose box is half as wide as the kernel counts on, so every ring
 * stage receives fewer bytes than its barrier expects and no stage ever completes.  Every load that
 * is issued still lands, inside its own slot.  With waits limited to limit_ns (at most two seconds)
 * the kernel must unwind by itself - all warp roles leave their loops, pending MMAs are waited for,
 * tensor memory is released - and b200spmm_plan_sync must then report B200SPMM_ERR_DEVICE_TIMEOUT
 * and leave the plan ready for a normal launch.  C receives nothing meaningful.  This is the bounded
 * replacement of the reference's endless waits (src/ptx/barrier.h:29-41, 72-86) under test; fp32 C,
 * n at least one 128-byte box wide.  A plan that would run one of its super-window kernels for this n runs that
 * one, every stage expecting sixteen bytes more than its loads deliver, and must unwind the same way (both
 * CTAs of a pair included).  The plan type is declared in b200_spmm.h.
 */
struct b200spmm_plan;
int b200spmm_kat_spmm_starved(struct b200spmm_plan *plan, const void *d_B, int64_t ldb, int64_t n, void *d_C,
                              int64_t ldc, unsigned long long limit_ns, void *stream);

/* Builds an instruction descriptor: fmt 0 = f16, 1 = bf16, 2 = tf32; fp32 accumulate. */
uint32_t b200spmm_kat_instr_desc(int fmt, int m, int n, int a_mn_major, int b_mn_major);

/*
 * Uploads a 2-D row-major tensor (rows x inner_elems, pitch_bytes between rows), encodes a tiled
 * tensor map over it (box_inner x box_rows elements, swizzle 0 none / 1 32B / 2 64B / 3 128B / 4 128B over 32-byte units),
 * issues `n_loads` TMA loads and dumps dump_bytes of shared memory (from its 1024-byte-aligned
 * start) to `dump`.  loads[i] = {mode, smem_off, x, y0, y1, y2, y3}: mode 0 is a tiled load of the
 * box at (x, y0); mode 1 is a four-row gather (tile::gather4) of rows y0..y3 starting at column x.
 * expect_bytes is the total byte count the loads must deliver.
 * Replaces copy_and_verify_kernel (test/01.tma_copy_matrix/copy.cu:77-171).
 */
int b200spmm_kat_tma(const void *tensor, uint64_t inner_elems, uint64_t rows, uint64_t pitch_bytes, int elt_size,
                     uint32_t box_inner, uint32_t box_rows, int swizzle, const int32_t *loads, int n_loads,
                     uint32_t expect_bytes, void *dump, uint32_t dump_bytes, int device);

/*
 * Issue-rate probe for the SpMM's MMA shape.  `issuers` (1 or 2) threads of one CTA each issue
 * `count` tcgen05.mma of M = m (64 or 128), N = n (16..256, multiple of 16), K = 32 bytes back to
 * back into their own TMEM accumulator, with the operand layouts of the SpMM kernel (operand A
 * MN-major, 128-byte swizzle; operand B K-major, 32-byte swizzle; zero-filled).
 * cycles_per_mma[0] = SM clocks per MMA the first issuer spent in its issue loop,
 * cycles_per_mma[1] = the same including the wait for the last MMA to retire.
 * It measures what one condensed tile costs the tensor pipe whatever its fill.  The reference
 * times its MMA chain only as part of a whole kernel (the consumer loop of
 * test/03.warp_specialized/main.cu:87-100 inside the event window of its main).
 */
int b200spmm_kat_umma_rate(int tf32, int m, int n, int count, int issuers, double *cycles_per_mma, int device);

#ifdef __cplusplus
}
#endif
#endif /* B200_SPMM_KAT_H_ */
