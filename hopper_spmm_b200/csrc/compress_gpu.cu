// Dense 16-row tiles -> bitmap + stored values, on the device.
//
// The SpMM kernels read the sparse matrix's tiles either as the dense 512-byte blocks of the
// uncompressed format (src/utils/class.h:74-85) or in the shape of the reference's
// bitmap-compressed format (src/utils/class.h:55-67, built by CSR2BTCF, src/utils/convert.h:22-139):
// one bit per tile slot in row-major order, the stored values of a tile one after another in the
// same order, and a running offset of the first stored value of every tile.  At a few per cent
// fill that is an eighth of the bytes.  This file derives the compressed arrays from dense tiles
// so that a plan built from the uncompressed format can stream the smaller form; a slot counts
// as stored when any bit of it is set, so expanding the result gives back the dense tile bit for
// bit (an explicit +0.0 of the CSR input is the one thing that is not kept as a stored value).
//
// The bitmap of a tile is kept as 16*CW/64 consecutive 64-bit words, bit b of the tile in word
// b/64 - the layout the reference's fp16 build intended (its converter indexes the second word of
// a tile by tile number instead of word number, src/utils/convert.h:98-100, so its own fp16 words
// overlap).
#include <cstdint>
#include <cub/device/device_scan.cuh>
#include <cuda_runtime.h>

#include "common.hpp"
#include "compress_gpu.hpp"

namespace b200spmm {

namespace {

constexpr int kTileBytes = 512;  // 16 rows x 32 bytes, both element types

// One warp per tile; lane l holds the 16-byte piece with row l/2, half l%2 of the row-major tile,
// i.e. slots [l*kPer, (l+1)*kPer) of it.  Returns the lane's bits (bit b = slot l*kPer + b stored).
template <bool kTf32>
__device__ uint32_t piece_bits(const uint4 &v) {
    if constexpr (kTf32) {
        return (v.x ? 1u : 0u) | (v.y ? 2u : 0u) | (v.z ? 4u : 0u) | (v.w ? 8u : 0u);
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t bits = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) bits |= ((w[k] & 0xFFFFu) ? 1u : 0u) << (2 * k) | ((w[k] >> 16) ? 1u : 0u) << (2 * k + 1);
        return bits;
    }
}

template <bool kTf32>
__global__ void __launch_bounds__(256)
tile_bitmaps_kernel(const uint4 *__restrict__ data, uint64_t tiles, uint8_t *__restrict__ bit_bytes, uint32_t *__restrict__ counts) {
    const uint64_t t = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (t >= tiles) return;
    const uint32_t bits = piece_bits<kTf32>(data[t * (kTileBytes / 16) + lane]);
    if constexpr (kTf32) {  // four bits per lane: two lanes share a byte
        const uint32_t other = __shfl_xor_sync(0xffffffffu, bits, 1);
        if (!(lane & 1u)) bit_bytes[t * 16 + (lane >> 1)] = (uint8_t)(bits | (other << 4));
    } else {                // eight bits per lane: byte l of the tile's four little-endian words
        bit_bytes[t * 32 + lane] = (uint8_t)bits;
    }
    uint32_t n = (uint32_t)__popc(bits);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) n += __shfl_xor_sync(0xffffffffu, n, d);
    if (lane == 0) counts[t] = n;
}

template <bool kTf32>
__global__ void __launch_bounds__(256)
tile_values_kernel(const uint4 *__restrict__ data, uint64_t tiles, const uint32_t *__restrict__ nnzOffset, void *__restrict__ values) {
    const uint64_t t = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (t >= tiles) return;
    const uint4 v = data[t * (kTileBytes / 16) + lane];
    const uint32_t bits = piece_bits<kTf32>(v);
    uint32_t before = (uint32_t)__popc(bits);  // inclusive scan over the lanes, then made exclusive
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, before, d);
        if (lane >= (uint32_t)d) before += up;
    }
    uint32_t idx = nnzOffset[t] + before - (uint32_t)__popc(bits);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if constexpr (kTf32) {
        uint32_t *out = static_cast<uint32_t *>(values);
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (w[k]) out[idx++] = w[k];
    } else {
        uint16_t *out = static_cast<uint16_t *>(values);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (w[k] & 0xFFFFu) out[idx++] = (uint16_t)(w[k] & 0xFFFFu);
            if (w[k] >> 16) out[idx++] = (uint16_t)(w[k] >> 16);
        }
    }
}

}  // namespace

void free_compressed_tiles(CompressedTiles *c) {
    cudaFree(c->tcBit);
    cudaFree(c->nnzOffset);
    cudaFree(c->values);
    *c = CompressedTiles{};
}

int compress_tiles_device(const void *d_data, uint64_t tiles, int dtype, CompressedTiles *out) {
    *out = CompressedTiles{};
    if (!tiles) return B200SPMM_OK;
    const bool tf32 = dtype == B200SPMM_TF32;
    const int cw = tf32 ? 8 : 16, words = 16 * cw / 64;
    uint32_t *counts = nullptr;
    void *scan_tmp = nullptr;
    size_t scan_bytes = 0;
    auto fail = [&](int code) {
        cudaFree(counts);
        cudaFree(scan_tmp);
        free_compressed_tiles(out);
        return code;
    };
#define B200_TRY_OR_FAIL(expr)                       \
    do {                                             \
        cudaError_t e__ = (expr);                    \
        if (e__ != cudaSuccess) {                    \
            record_cuda_error(e__, #expr);           \
            return fail(B200SPMM_ERR_CUDA);          \
        }                                            \
    } while (0)
    B200_TRY_OR_FAIL(cudaMalloc(&out->tcBit, tiles * words * sizeof(uint64_t)));
    B200_TRY_OR_FAIL(cudaMalloc(&out->nnzOffset, (tiles + 1) * sizeof(uint32_t)));
    B200_TRY_OR_FAIL(cudaMalloc(&counts, (tiles + 1) * sizeof(uint32_t)));
    B200_TRY_OR_FAIL(cudaMemset(counts + tiles, 0, sizeof(uint32_t)));
    const unsigned blocks = (unsigned)((tiles * 32 + 255) / 256);
    const uint4 *data = static_cast<const uint4 *>(d_data);
    if (tf32) tile_bitmaps_kernel<true><<<blocks, 256>>>(data, tiles, reinterpret_cast<uint8_t *>(out->tcBit), counts);
    else tile_bitmaps_kernel<false><<<blocks, 256>>>(data, tiles, reinterpret_cast<uint8_t *>(out->tcBit), counts);
    B200_TRY_OR_FAIL(cudaGetLastError());
    // nnzOffset[t] = stored values before tile t; the extra last element gives the total
    B200_TRY_OR_FAIL(cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, counts, out->nnzOffset, tiles + 1));
    B200_TRY_OR_FAIL(cudaMalloc(&scan_tmp, scan_bytes));
    B200_TRY_OR_FAIL(cub::DeviceScan::ExclusiveSum(scan_tmp, scan_bytes, counts, out->nnzOffset, tiles + 1));
    uint32_t total = 0;
    B200_TRY_OR_FAIL(cudaMemcpy(&total, out->nnzOffset + tiles, sizeof(total), cudaMemcpyDeviceToHost));
    out->stored = total;
    // 16 spare bytes: the kernel's loads never pass the end, and an empty array still has an address
    B200_TRY_OR_FAIL(cudaMalloc(&out->values, (size_t)total * (tf32 ? 4 : 2) + 16));
    if (tf32) tile_values_kernel<true><<<blocks, 256>>>(data, tiles, out->nnzOffset, out->values);
    else tile_values_kernel<false><<<blocks, 256>>>(data, tiles, out->nnzOffset, out->values);
    B200_TRY_OR_FAIL(cudaGetLastError());
    B200_TRY_OR_FAIL(cudaDeviceSynchronize());
#undef B200_TRY_OR_FAIL
    cudaFree(counts);
    cudaFree(scan_tmp);
    return B200SPMM_OK;
}

}  // namespace b200spmm
