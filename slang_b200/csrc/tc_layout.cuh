// Shared-memory operand geometry used by the tensor-core kernels: a [rows][D] 16-bit matrix is cut
// into panels of min(64, D) elements per row, stored with the swizzle whose span equals the panel row
// (32, 64 or 128 bytes).  This is what a TMA tile load with that swizzle produces and what the UMMA
// shared-memory descriptors of the matching layout type expect.
#pragma once

#include <stdint.h>

namespace mlpb200 {
namespace layout {

// Panel geometry of a [rows][D] 16-bit operand.
__host__ __device__ constexpr int panel_w(int d) { return d < 64 ? d : 64; }              // elements per panel row
__host__ __device__ constexpr int row_bytes(int d) { return panel_w(d) * 2; }             // 32, 64 or 128
__host__ __device__ constexpr int swz_shift(int d) { return d >= 64 ? 0 : d == 32 ? 1 : 2; }
__host__ __device__ constexpr int swz_mask(int d) { return d >= 64 ? 7 : d == 32 ? 3 : 1; }
__host__ __device__ constexpr uint32_t layout_type(int d) { return d >= 64 ? 2u : d == 32 ? 4u : 6u; }  // SW128 / SW64 / SW32
__host__ __device__ constexpr int imax(int a, int b) { return a > b ? a : b; }
__host__ __device__ constexpr uint32_t pow2_at_least_32(uint32_t n) { uint32_t p = 32; while (p < n) p <<= 1; return p; }

// Byte offset of the 16-byte chunk j (8 elements) of row r in a [rows][D] operand buffer.
template <int D>
__device__ __forceinline__ uint32_t chunk_offset(int rows, int r, int j)
{
    constexpr int cpp = panel_w(D) / 8;  // chunks per panel row
    const int panel = j / cpp, cj = j % cpp;
    return (uint32_t)panel * (uint32_t)(rows * row_bytes(D)) + (uint32_t)r * row_bytes(D) +
           (uint32_t)((cj ^ ((r >> swz_shift(D)) & swz_mask(D))) << 4);
}

}  // namespace layout
}  // namespace mlpb200
