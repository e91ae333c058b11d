// Single-CTA known-answer kernels for the sm_100a primitives (tcgen05.mma with arbitrary
// descriptors, TMA tiled / gather4 loads).  They replace the reference's bring-up programs
// (src/test_fp16.cu, test/01.tma_copy_matrix/copy.cu, test/02.tma_and_wgmma/tma_wgmma.cu): the
// host prepares a shared-memory image or a tensor, the kernel runs the primitive once and
// returns the raw TMEM / shared-memory contents for the test to judge.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../include/b200_spmm_kat.h"
#include "common.hpp"
#include "ptx_sm100.cuh"
#include "tensormap.hpp"

namespace b200spmm {
namespace {

constexpr uint32_t kKatTmemCols = 256;

// Wait limit of the known-answer kernels; a test shortens it to see a bounded wait run out.
unsigned long long g_kat_wait_limit_ns = kDeviceWaitLimitNs;

__global__ void __launch_bounds__(128, 1)
kat_umma_kernel(const uint8_t *__restrict__ image, uint32_t image_bytes, const b200spmm_kat_mma_t *__restrict__ mmas,
                int n_mmas, int n_cols, float *__restrict__ out, uint32_t *__restrict__ status,
                unsigned long long limit_ns) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t abort_flag;

    // 1024-byte aligned operand area (the swizzle patterns are functions of the address bits).
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *area = smem_raw + pad;
    const uint32_t area_addr = raw_addr + pad;

    const int tid = threadIdx.x, warp = tid >> 5;
    for (uint32_t i = tid * 16u; i < image_bytes; i += blockDim.x * 16u)
        *reinterpret_cast<uint4 *>(area + i) = *reinterpret_cast<const uint4 *>(image + i);
    if (tid == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&done_bar), 1);
        ptx::fence_mbar_init();
    }
    ptx::fence_proxy_async_smem();  // operand bytes were written through the generic proxy
    if (warp == 0) {
        ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), kKatTmemCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (tid == 0) {
        for (int i = 0; i < n_mmas; ++i) {
            const b200spmm_kat_mma_t m = mmas[i];
            const uint64_t ad = ptx::make_smem_desc(area_addr + m.a_off, m.a_lbo, m.a_sbo, m.a_swizzle);
            const uint64_t bd = ptx::make_smem_desc(area_addr + m.b_off, m.b_lbo, m.b_sbo, m.b_swizzle);
            if (m.kind == 0)
                ptx::umma_f16_ss(tmem_base + m.d_col, ad, bd, m.idesc, m.accumulate);
            else
                ptx::umma_tf32_ss(tmem_base + m.d_col, ad, bd, m.idesc, m.accumulate);
        }
        ptx::umma_commit(ptx::smem_u32(&done_bar));
    }
    __syncwarp();
    const bool ok = ptx::mbar_wait(ptx::smem_u32(&done_bar), 0, &abort_flag, limit_ns);
    ptx::tcgen05_fence_after_sync();
    if (!ok && tid == 0) atomicOr(status, kDevStatusTimeout);

    // Every warp dumps its own 32 lanes.
    for (int c0 = 0; c0 < n_cols; c0 += 16) {
        uint32_t r[16];
        ptx::tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) out[(size_t)tid * n_cols + c0 + j] = __uint_as_float(r[j]);
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem_base, kKatTmemCols);
}

__global__ void __launch_bounds__(32, 1)
kat_tma_kernel(const __grid_constant__ CUtensorMap tmap, const int32_t *__restrict__ loads, int n_loads,
               uint32_t expect_bytes, uint8_t *__restrict__ dump, uint32_t dump_bytes, uint32_t *__restrict__ status,
               unsigned long long limit_ns) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_flag;
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *area = smem_raw + pad;
    const uint32_t area_addr = raw_addr + pad;
    const int tid = threadIdx.x;

    // Poison so untouched bytes are recognisable.
    for (uint32_t i = tid * 4u; i < dump_bytes; i += 32u * 4u) *reinterpret_cast<uint32_t *>(area + i) = 0xDEADBEEFu;
    if (tid == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        ptx::fence_mbar_init();
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (tid == 0) {
        ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bar), expect_bytes);
        for (int i = 0; i < n_loads; ++i) {
            const int32_t *l = loads + i * 7;
            if (l[0] == 0)
                ptx::tma_load_2d(area_addr + (uint32_t)l[1], &tmap, l[2], l[3], ptx::smem_u32(&bar));
            else
                ptx::tma_gather4_2d(area_addr + (uint32_t)l[1], &tmap, l[2], l[3], l[4], l[5], l[6], ptx::smem_u32(&bar));
        }
    }
    __syncwarp();
    // Every load that was issued is given its bytes' worth of waiting even when the barrier expects
    // more than the loads deliver: nothing is still writing shared memory when the dump is read.
    const bool ok = ptx::mbar_wait(ptx::smem_u32(&bar), 0, &abort_flag, limit_ns);
    if (!ok && tid == 0) atomicOr(status, kDevStatusTimeout);
    __syncwarp();
    for (uint32_t i = tid * 4u; i < dump_bytes; i += 32u * 4u)
        *reinterpret_cast<uint32_t *>(dump + i) = *reinterpret_cast<const uint32_t *>(area + i);
}

// Issue-rate probe: `issuers` threads (lane 0 of warps 1 and 2) each issue `count` MMAs of
// M = m, N = n, K = 32 bytes back to back into their own accumulator, operands rotating over
// eight positions of a zero-filled image laid out as the SpMM kernel lays them out (operand A
// MN-major under the 128-byte swizzle, operand B K-major under the 32-byte swizzle).
// cycles[0] = clocks the first issuer spent issuing, cycles[1] = issuing plus draining.
__global__ void __launch_bounds__(128, 1)
kat_umma_rate_kernel(int tf32, uint32_t idesc, int count, int issuers, long long *__restrict__ cycles,
                     uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t done_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t abort_flag;
    constexpr uint32_t kImageBytes = 64u * 1024u, kBOff = 32u * 1024u, kCols = 512;
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *area = smem_raw + pad;
    const uint32_t area_addr = raw_addr + pad;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (uint32_t i = tid * 16u; i < kImageBytes; i += blockDim.x * 16u) *reinterpret_cast<uint4 *>(area + i) = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&done_bar[0]), 1);
        ptx::mbar_init(ptx::smem_u32(&done_bar[1]), 1);
        ptx::fence_mbar_init();
    }
    ptx::fence_proxy_async_smem();
    if (warp == 0) {
        ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), kCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    if (warp >= 1 && warp <= issuers && lane == 0) {
        const int w = warp - 1;
        const uint64_t a0 = tf32 ? ptx::make_smem_desc(area_addr, 1024, 512, ptx::kSwizzle128BBase32B)
                                 : ptx::make_smem_desc(area_addr, 2048, 1024, ptx::kSwizzle128B);
        const uint64_t b0 = ptx::make_smem_desc(area_addr + kBOff, 16, 256, ptx::kSwizzle32B);
        const uint32_t a_hi = (uint32_t)(a0 >> 32), b_hi = (uint32_t)(b0 >> 32), a_lo = (uint32_t)a0, b_lo = (uint32_t)b0;
        const uint32_t acc = tmem_base + (uint32_t)w * 256u;
        const long long t0 = clock64();
        for (int i = 0; i < count; ++i) {
            // operand A advances by 4 KB (one gathered tile), operand B by 512 bytes (one sparse tile)
            if (tf32)
                ptx::umma_tf32_ss_lohi(acc, a_lo + (uint32_t)(i & 7) * 256u, a_hi, b_lo + (uint32_t)(i & 7) * 32u, b_hi, idesc, i > 0);
            else
                ptx::umma_f16_ss_lohi(acc, a_lo + (uint32_t)(i & 7) * 256u, a_hi, b_lo + (uint32_t)(i & 7) * 32u, b_hi, idesc, i > 0);
        }
        const long long t1 = clock64();
        ptx::umma_commit(ptx::smem_u32(&done_bar[w]));
        const bool ok = ptx::mbar_wait(ptx::smem_u32(&done_bar[w]), 0, &abort_flag, kDeviceWaitLimitNs);
        const long long t2 = clock64();
        if (!ok) atomicOr(status, kDevStatusTimeout);
        if (w == 0) {
            cycles[0] = t1 - t0;
            cycles[1] = t2 - t0;
        }
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    if (warp == 0) ptx::tmem_dealloc(tmem_base, kCols);
}

// Known answer for the MMA of a CTA pair (cta_group::2): two CTAs of one cluster each copy their own
// image into shared memory, the even CTA issues the listed MMAs for both, each CTA dumps its 128 lanes of
// tensor memory.  out[cta][128][n_cols].
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
kat_umma_pair_kernel(const uint8_t *__restrict__ images, uint32_t image_bytes, const b200spmm_kat_mma_t *__restrict__ mmas,
                     int n_mmas, int n_cols, float *__restrict__ out, uint32_t *__restrict__ status, unsigned long long limit_ns) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t abort_flag;
    const uint32_t rank = ptx::cluster_cta_rank();
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *area = smem_raw + pad;
    const uint32_t area_addr = raw_addr + pad;
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint8_t *image = images + (size_t)rank * image_bytes;
    for (uint32_t i = tid * 16u; i < image_bytes; i += blockDim.x * 16u)
        *reinterpret_cast<uint4 *>(area + i) = *reinterpret_cast<const uint4 *>(image + i);
    if (tid == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&done_bar), 1);
        ptx::fence_mbar_init();
    }
    ptx::fence_proxy_async_smem();
    if (warp == 0) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_slot), kKatTmemCols);
        ptx::tmem_relinquish_alloc_permit_pair();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();  // both images are in place and both barriers initialised before anything is issued
    ptx::cluster_wait();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    if (rank == 0 && tid == 0) {
        for (int i = 0; i < n_mmas; ++i) {
            const b200spmm_kat_mma_t m = mmas[i];
            const uint64_t ad = ptx::make_smem_desc(area_addr + m.a_off, m.a_lbo, m.a_sbo, m.a_swizzle);
            const uint64_t bd = ptx::make_smem_desc(area_addr + m.b_off, m.b_lbo, m.b_sbo, m.b_swizzle);
            ptx::umma_pair_ss_lohi_if(m.kind != 0, 1u, tmem_base + m.d_col, (uint32_t)ad, (uint32_t)(ad >> 32), (uint32_t)bd,
                                      (uint32_t)(bd >> 32), m.idesc, m.accumulate);
        }
        ptx::umma_commit_pair(ptx::smem_u32(&done_bar));
    }
    __syncwarp();
    const bool ok = ptx::mbar_wait(ptx::smem_u32(&done_bar), 0, &abort_flag, limit_ns);
    ptx::tcgen05_fence_after_sync();
    if (!ok && tid == 0) atomicOr(status, kDevStatusTimeout);
    for (int c0 = 0; c0 < n_cols; c0 += 16) {  // every warp dumps its own 32 lanes
        uint32_t r[16];
        ptx::tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) out[((size_t)rank * 128 + tid) * n_cols + c0 + j] = __uint_as_float(r[j]);
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();  // neither CTA lets go of its shared or tensor memory while the other may still use it
    ptx::cluster_wait();
    if (warp == 0) ptx::tmem_dealloc_pair(tmem_base, kKatTmemCols);
}

struct DevBuf {
    void *p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
};

int check_device(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) {
        cudaGetLastError();
        return B200SPMM_ERR_NO_DEVICE;
    }
    cudaDeviceProp prop;
    B200_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return B200SPMM_ERR_NO_DEVICE;
    B200_CUDA_TRY(cudaSetDevice(device));
    return B200SPMM_OK;
}

}  // namespace
}  // namespace b200spmm

using namespace b200spmm;

extern "C" unsigned long long b200spmm_kat_wait_limit(unsigned long long limit_ns) {
    const unsigned long long before = g_kat_wait_limit_ns;
    g_kat_wait_limit_ns = limit_ns ? limit_ns : kDeviceWaitLimitNs;
    return before;
}

extern "C" uint32_t b200spmm_kat_instr_desc(int fmt, int m, int n, int a_mn_major, int b_mn_major) {
    return ptx::make_instr_desc((uint32_t)fmt, (uint32_t)m, (uint32_t)n, a_mn_major != 0, b_mn_major != 0);
}

extern "C" int b200spmm_kat_umma(const void *image, uint32_t image_bytes, const b200spmm_kat_mma_t *mmas, int n_mmas,
                                 int n_cols, float *out, int device) {
    if (!image || !mmas || !out || n_mmas < 1 || n_cols < 16 || n_cols > (int)kKatTmemCols || n_cols % 16) return B200SPMM_ERR_INVALID_ARG;
    if (image_bytes > 96u * 1024u) return B200SPMM_ERR_INVALID_ARG;
    int st = check_device(device);
    if (st != B200SPMM_OK) return st;
    const uint32_t padded = (image_bytes + 15u) & ~15u;
    // Every operand read must stay inside the image.
    DevBuf d_img, d_mma, d_out, d_status;
    B200_CUDA_TRY(cudaMalloc(&d_img.p, padded));
    B200_CUDA_TRY(cudaMemset(d_img.p, 0, padded));
    B200_CUDA_TRY(cudaMemcpy(d_img.p, image, image_bytes, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMalloc(&d_mma.p, sizeof(b200spmm_kat_mma_t) * n_mmas));
    B200_CUDA_TRY(cudaMemcpy(d_mma.p, mmas, sizeof(b200spmm_kat_mma_t) * n_mmas, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMalloc(&d_out.p, sizeof(float) * 128 * n_cols));
    B200_CUDA_TRY(cudaMemset(d_out.p, 0, sizeof(float) * 128 * n_cols));
    B200_CUDA_TRY(cudaMalloc(&d_status.p, 4));
    B200_CUDA_TRY(cudaMemset(d_status.p, 0, 4));
    const size_t smem = (size_t)padded + 1024 + 4096;  // slack so descriptor strides never leave the allocation
    B200_CUDA_TRY(cudaFuncSetAttribute(kat_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kat_umma_kernel<<<1, 128, smem>>>((const uint8_t *)d_img.p, padded, (const b200spmm_kat_mma_t *)d_mma.p, n_mmas,
                                      n_cols, (float *)d_out.p, (uint32_t *)d_status.p, g_kat_wait_limit_ns);
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaDeviceSynchronize());
    uint32_t status = 0;
    B200_CUDA_TRY(cudaMemcpy(&status, d_status.p, 4, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(out, d_out.p, sizeof(float) * 128 * n_cols, cudaMemcpyDeviceToHost));
    return (status & kDevStatusTimeout) ? B200SPMM_ERR_DEVICE_TIMEOUT : B200SPMM_OK;
}

extern "C" int b200spmm_kat_umma_pair(const void *images, uint32_t image_bytes, const b200spmm_kat_mma_t *mmas, int n_mmas,
                                      int n_cols, float *out, int device) {
    if (!images || !mmas || !out || n_mmas < 1 || n_cols < 16 || n_cols > (int)kKatTmemCols || n_cols % 16) return B200SPMM_ERR_INVALID_ARG;
    if (image_bytes > 96u * 1024u || image_bytes % 16) return B200SPMM_ERR_INVALID_ARG;
    int st = check_device(device);
    if (st != B200SPMM_OK) return st;
    DevBuf d_img, d_mma, d_out, d_status;
    B200_CUDA_TRY(cudaMalloc(&d_img.p, 2 * (size_t)image_bytes));
    B200_CUDA_TRY(cudaMemcpy(d_img.p, images, 2 * (size_t)image_bytes, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMalloc(&d_mma.p, sizeof(b200spmm_kat_mma_t) * n_mmas));
    B200_CUDA_TRY(cudaMemcpy(d_mma.p, mmas, sizeof(b200spmm_kat_mma_t) * n_mmas, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMalloc(&d_out.p, sizeof(float) * 256 * n_cols));
    B200_CUDA_TRY(cudaMemset(d_out.p, 0, sizeof(float) * 256 * n_cols));
    B200_CUDA_TRY(cudaMalloc(&d_status.p, 4));
    B200_CUDA_TRY(cudaMemset(d_status.p, 0, 4));
    const size_t smem = (size_t)image_bytes + 1024 + 4096;
    B200_CUDA_TRY(cudaFuncSetAttribute(kat_umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kat_umma_pair_kernel<<<2, 128, smem>>>((const uint8_t *)d_img.p, image_bytes, (const b200spmm_kat_mma_t *)d_mma.p, n_mmas,
                                           n_cols, (float *)d_out.p, (uint32_t *)d_status.p, g_kat_wait_limit_ns);
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaDeviceSynchronize());
    uint32_t status = 0;
    B200_CUDA_TRY(cudaMemcpy(&status, d_status.p, 4, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(out, d_out.p, sizeof(float) * 256 * n_cols, cudaMemcpyDeviceToHost));
    return (status & kDevStatusTimeout) ? B200SPMM_ERR_DEVICE_TIMEOUT : B200SPMM_OK;
}

extern "C" int b200spmm_kat_tma(const void *tensor, uint64_t inner_elems, uint64_t rows, uint64_t pitch_bytes,
                                int elt_size, uint32_t box_inner, uint32_t box_rows, int swizzle, const int32_t *loads,
                                int n_loads, uint32_t expect_bytes, void *dump, uint32_t dump_bytes, int device) {
    if (!tensor || !loads || !dump || n_loads < 1 || dump_bytes % 4 || dump_bytes > 96u * 1024u) return B200SPMM_ERR_INVALID_ARG;
    if (elt_size != 1 && elt_size != 2 && elt_size != 4) return B200SPMM_ERR_INVALID_ARG;
    if (pitch_bytes % 16 || swizzle < 0 || swizzle > 4) return B200SPMM_ERR_INVALID_ARG;
    for (int i = 0; i < n_loads; ++i) {
        const int32_t *l = loads + i * 7;
        if ((l[0] != 0 && l[0] != 1) || l[1] < 0 || (l[1] % 128) || ((int64_t)l[2] * elt_size) % 16) return B200SPMM_ERR_INVALID_ARG;
    }
    int st = check_device(device);
    if (st != B200SPMM_OK) return st;
    DevBuf d_t, d_loads, d_dump, d_status;
    const size_t bytes = (size_t)rows * pitch_bytes;
    B200_CUDA_TRY(cudaMalloc(&d_t.p, bytes));
    B200_CUDA_TRY(cudaMemcpy(d_t.p, tensor, bytes, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMalloc(&d_loads.p, sizeof(int32_t) * 7 * n_loads));
    B200_CUDA_TRY(cudaMemcpy(d_loads.p, loads, sizeof(int32_t) * 7 * n_loads, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMalloc(&d_dump.p, dump_bytes));
    B200_CUDA_TRY(cudaMalloc(&d_status.p, 4));
    B200_CUDA_TRY(cudaMemset(d_status.p, 0, 4));
    CUtensorMap map;
    const CUtensorMapDataType type = elt_size == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : elt_size == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    const CUtensorMapSwizzle sw = swizzle == 0 ? CU_TENSOR_MAP_SWIZZLE_NONE : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    if (!encode_2d(&map, type, d_t.p, inner_elems, rows, pitch_bytes, box_inner, box_rows, sw)) return B200SPMM_ERR_CUDA;
    const size_t smem = (size_t)dump_bytes + 1024;
    B200_CUDA_TRY(cudaFuncSetAttribute(kat_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kat_tma_kernel<<<1, 32, smem>>>(map, (const int32_t *)d_loads.p, n_loads, expect_bytes, (uint8_t *)d_dump.p,
                                    dump_bytes, (uint32_t *)d_status.p, g_kat_wait_limit_ns);
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaDeviceSynchronize());
    uint32_t status = 0;
    B200_CUDA_TRY(cudaMemcpy(&status, d_status.p, 4, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(dump, d_dump.p, dump_bytes, cudaMemcpyDeviceToHost));
    return (status & kDevStatusTimeout) ? B200SPMM_ERR_DEVICE_TIMEOUT : B200SPMM_OK;
}

extern "C" int b200spmm_kat_umma_rate(int tf32, int m, int n, int count, int issuers, double *cycles_per_mma, int device) {
    if (!cycles_per_mma || (m != 64 && m != 128) || n < 16 || n > 256 || n % 16 || count < 1 || count > (1 << 20) ||
        issuers < 1 || issuers > 2)
        return B200SPMM_ERR_INVALID_ARG;
    int st = check_device(device);
    if (st != B200SPMM_OK) return st;
    DevBuf d_cycles, d_status;
    B200_CUDA_TRY(cudaMalloc(&d_cycles.p, 2 * sizeof(long long)));
    B200_CUDA_TRY(cudaMemset(d_cycles.p, 0, 2 * sizeof(long long)));
    B200_CUDA_TRY(cudaMalloc(&d_status.p, 4));
    B200_CUDA_TRY(cudaMemset(d_status.p, 0, 4));
    const uint32_t idesc = ptx::make_instr_desc(tf32 ? ptx::kFmtTF32 : ptx::kFmtF16, (uint32_t)m, (uint32_t)n, true, false);
    const size_t smem = 64 * 1024 + 1024 + 4096;
    B200_CUDA_TRY(cudaFuncSetAttribute(kat_umma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kat_umma_rate_kernel<<<1, 128, smem>>>(tf32 ? 1 : 0, idesc, count, issuers, (long long *)d_cycles.p, (uint32_t *)d_status.p);
    B200_CUDA_TRY(cudaGetLastError());
    B200_CUDA_TRY(cudaDeviceSynchronize());
    uint32_t status = 0;
    long long cycles[2] = {0, 0};
    B200_CUDA_TRY(cudaMemcpy(&status, d_status.p, 4, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(cycles, d_cycles.p, sizeof(cycles), cudaMemcpyDeviceToHost));
    cycles_per_mma[0] = (double)cycles[0] / count;
    cycles_per_mma[1] = (double)cycles[1] / count;
    return (status & kDevStatusTimeout) ? B200SPMM_ERR_DEVICE_TIMEOUT : B200SPMM_OK;
}
