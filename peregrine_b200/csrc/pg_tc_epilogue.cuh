// Epilogue store shared by the tcgen05 GEMM kernels.
//
// tcgen05.ld (32x32b) hands each lane one accumulator ROW (32 consecutive columns).  Writing that
// straight to global memory makes every warp store touch 32 different rows, 16 bytes each, which
// held the whole GEMM to the speed of its output stores.  Here the warp first exchanges the 32 x 32
// block through a small shared-memory tile (row stride 36 words: conflict-free for the 128-bit
// writes by row and the 128-bit reads by column group), so that every store instruction writes four
// complete 128-byte row segments.
#pragma once

#include <stdint.h>

constexpr int PG_EPI_STRIDE = 36;                         // words per staged row (32 + 4 pad)
constexpr int PG_EPI_WARP_BYTES = 32 * PG_EPI_STRIDE * 4;  // 4608 B per epilogue warp

// vals[j] = word for (row = lane, column j) of the block.  dst points at element (row0, col0) of a
// row-major matrix with leading dimension ld (elements of 4 bytes); rows_left / cols_left say how much
// of the 32 x 32 block lies inside the matrix (cols_left is a multiple of 4 on this path).
__device__ __forceinline__ void pg_store_block_32x32(uint32_t *dst, int64_t ld, int rows_left, int cols_left, uint32_t stage,
                                                     int lane, const uint32_t (&vals)[32])
{
    const uint32_t mine = stage + (uint32_t)lane * (PG_EPI_STRIDE * 4);
#pragma unroll
    for (int j = 0; j < 32; j += 4)
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(mine + j * 4), "r"(vals[j]), "r"(vals[j + 1]), "r"(vals[j + 2]),
                     "r"(vals[j + 3])
                     : "memory");
    __syncwarp();
    const int c4 = (lane & 7) * 4, r4 = lane >> 3;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = i * 4 + r4;
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(stage + (uint32_t)(r * PG_EPI_STRIDE + c4) * 4));
        if (r < rows_left && c4 < cols_left) *reinterpret_cast<uint4 *>(dst + (int64_t)r * ld + c4) = v;
    }
    __syncwarp();
}

