// Device-side compression of dense 16-row tiles into bitmap + stored values (compress_gpu.cu).
#pragma once

#include <cstdint>

namespace b200spmm {

struct CompressedTiles {
    uint64_t *tcBit = nullptr;      // [tiles * 16*CW/64]
    uint32_t *nnzOffset = nullptr;  // [tiles + 1]
    void *values = nullptr;         // [stored] elements of the matrix's type
    uint64_t stored = 0;
};

// Builds the three arrays in device memory of the current device from `tiles` dense tiles at
// d_data (dtype B200SPMM_F16 or B200SPMM_TF32).  Synchronous.  Returns a B200SPMM status.
int compress_tiles_device(const void *d_data, uint64_t tiles, int dtype, CompressedTiles *out);
void free_compressed_tiles(CompressedTiles *c);

}  // namespace b200spmm
