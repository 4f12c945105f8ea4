// Block-128 Hadamard rotation and per-token int8 quantisation, shared by every kernel that produces the int8 operand
// of a W8A8 linear (the stand-alone activation prologue, the attention epilogue, the GEMM-side producers).
//
// Layout convention: one warp owns one 128-block, lane l holds the four consecutive elements 4l..4l+3.  The seven
// butterfly stages are two in-register stages plus five warp-shuffle stages; the result is scaled by 1/sqrt(128).
// The quantise helpers spell their rounding out with IEEE intrinsics, so a file compiled with fast-math produces the
// same bits as one compiled without.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void fwht128_lane4(float (&v)[4], int lane) {
  // stages on index bits 0 and 1 (inside the lane)
  float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]), a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
  v[0] = __fadd_rn(a0, a2); v[1] = __fadd_rn(a1, a3); v[2] = __fsub_rn(a0, a2); v[3] = __fsub_rn(a1, a3);
  // stages on index bits 2..6 (lane bits 0..4)
#pragma unroll
  for (int b = 0; b < 5; ++b) {
    const int mask = 1 << b;
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], mask);
      v[i] = upper ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
    }
  }
  const float s = 0.08838834764831845f;  // 1/sqrt(128)
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(v[i], s);
}

// per-token scale from the row's largest rotated magnitude (a row of zeros quantises with scale 1)
__device__ __forceinline__ float quant_scale_from_amax(float amax) {
  return (amax > 0.f) ? __fdiv_rn(amax, 127.f) : 1.f;
}
__device__ __forceinline__ float quant_inv_scale(float scale) { return __fdiv_rn(1.0f, scale); }

// four rotated values -> four int8 packed little-endian into one 32-bit word
__device__ __forceinline__ uint32_t quant_pack4(const float (&v)[4], float inv_scale) {
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int qi = __float2int_rn(__fmul_rn(v[j], inv_scale));
    qi = max(-127, min(127, qi));
    packed |= (static_cast<uint32_t>(qi) & 0xffu) << (8 * j);
  }
  return packed;
}

}  // namespace b200
