// Helpers shared by the fused attention kernels (forward and backward).
#pragma once

#include <stdint.h>

namespace brk {

constexpr int AT_BQ = 128;      // query rows per tile
constexpr int AT_BKV = 128;     // keys per tile
constexpr int AT_THREADS = 192; // producer warp, MMA warp, four row-owner warps

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// byte offset of element (row, col) inside a [128 x 64*atoms] fp16 operand tile stored as
// 64-column atoms of 16 KB with 128-byte swizzle (the layout TMA writes and tcgen05 reads)
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
    const int atom = col >> 6, c = col & 63;
    return (uint32_t)(atom * 16384 + row * 128 + ((((c >> 3) ^ (row & 7)) << 4) | ((c & 7) << 1)));
}

}  // namespace brk
