// Pieces shared by the W8A8 GEMM kernels.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace b200 {

constexpr int TILE_N = 128;     // rows of the operand that fills the MMA M dimension
constexpr int BLOCK_K = 128;    // int8 elements (= bytes) per k-block: one 128-byte swizzle row
constexpr int UMMA_K = 32;      // int8 elements per tcgen05.mma
constexpr int GEMM_THREADS = 192;
constexpr int SWAP_MAX_M = 64;  // up to this many tokens the weights fill the MMA M dimension

// 2-D row-major byte matrix [rows][cols] with row pitch `pitch` bytes; box = 128 bytes x box_rows, 128-byte swizzle.
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_rows);

}  // namespace b200
