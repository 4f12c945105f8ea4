// Activation prologue for every W8A8 linear: (residual add) -> (RMSNorm) | (SwiGLU) -> block-Hadamard
// rotation (block 128, Sylvester order, scaled 1/sqrt(128)) -> per-token symmetric int8 quantisation.
//
//   one CTA per token row, 8 warps; warp w owns 128-blocks w, w+8, ...; inside a block lane l holds the four
//   consecutive elements 4l..4l+3, so the seven butterfly stages are two in-register stages plus five
//   warp-shuffle stages.  Rotated values stay in registers between the abs-max pass and the quantise pass,
//   so the row is read from HBM exactly once and written once (int8 + one fp32 scale).
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include "hadamard.cuh"

namespace b200 {

constexpr int AQ_THREADS = 256;
constexpr int AQ_WARPS = AQ_THREADS / 32;

enum ActQuantMode : int { AQ_PLAIN = 0, AQ_NORM = 1, AQ_ADD_NORM = 2, AQ_SWIGLU = 3 };

__device__ __forceinline__ void load4_bf16(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
__device__ __forceinline__ void store4_bf16(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
  __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&lo);
  raw.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <int MAXB, int MODE>
__global__ void __launch_bounds__(AQ_THREADS)
act_quant_kernel(const __nv_bfloat16* x, long long ldx, __nv_bfloat16* residual,
                 long long ldr, const __nv_bfloat16* gamma, float eps, int8_t* q,
                 long long ldq, float* scale, __nv_bfloat16* xn_out, long long ldn,
                 int K) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  B200_TRACE_INIT();
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, TP_START);
  pdl_wait();                // everything before this kernel in the stream has completed
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, TP_DEPS);

  __shared__ float red[AQ_WARPS];
  __shared__ float bcast;
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblocks = K >> 7;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;

  float v[MAXB][4];
  float ss = 0.f;
  // All global loads of the row are issued first, with no arithmetic in between, so their latencies overlap;
  // the element-wise math (which contains slow-path divisions / exponentials) runs afterwards.
  uint2 raw_a[MAXB], raw_b[MAXB];
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = warp + i * AQ_WARPS;
    raw_a[i] = make_uint2(0u, 0u);
    raw_b[i] = make_uint2(0u, 0u);
    if (b < nblocks) {
      const int k = b * 128 + lane * 4;
      raw_a[i] = *reinterpret_cast<const uint2*>(xr + k);
      if constexpr (MODE == AQ_SWIGLU) raw_b[i] = *reinterpret_cast<const uint2*>(xr + K + k);
      if constexpr (MODE == AQ_ADD_NORM) raw_b[i] = *reinterpret_cast<const uint2*>(residual + static_cast<size_t>(row) * ldr + k);
    }
  }
  auto unpack4 = [](const uint2& r, float (&o)[4]) {
    o[0] = __uint_as_float(r.x << 16); o[1] = __uint_as_float(r.x & 0xffff0000u);
    o[2] = __uint_as_float(r.y << 16); o[3] = __uint_as_float(r.y & 0xffff0000u);
  };
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = warp + i * AQ_WARPS;
    if (b < nblocks) {
      const int k = b * 128 + lane * 4;
      if constexpr (MODE == AQ_SWIGLU) {
        float g[4], u[4];
        unpack4(raw_a[i], g);
        unpack4(raw_b[i], u);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i][j] = __fdividef(g[j], 1.f + __expf(-g[j])) * u[j];
      } else {
        unpack4(raw_a[i], v[i]);
        if constexpr (MODE == AQ_ADD_NORM) {
          float r[4];
          unpack4(raw_b[i], r);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // the residual stream is kept in bf16: round the sum once, and normalise what was stored
            v[i][j] = __bfloat162float(__float2bfloat16(v[i][j] + r[j]));
          }
          store4_bf16(residual + static_cast<size_t>(row) * ldr + k, v[i]);
        }
        if constexpr (MODE == AQ_NORM || MODE == AQ_ADD_NORM) {
#pragma unroll
          for (int j = 0; j < 4; ++j) ss += v[i][j] * v[i][j];
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[i][j] = 0.f;
    }
  }

  uint2 raw_g[MAXB];
  if constexpr (MODE == AQ_NORM || MODE == AQ_ADD_NORM) {
#pragma unroll
    for (int i = 0; i < MAXB; ++i) {
      const int b = warp + i * AQ_WARPS;
      raw_g[i] = make_uint2(0u, 0u);
      if (b < nblocks) raw_g[i] = __ldg(reinterpret_cast<const uint2*>(gamma + b * 128 + lane * 4));
    }
  }
  if constexpr (MODE == AQ_NORM || MODE == AQ_ADD_NORM) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < AQ_WARPS; ++w) t += red[w];
      bcast = rsqrtf(t / static_cast<float>(K) + eps);
    }
    __syncthreads();
    const float rstd = bcast;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MAXB; ++i) {
      const int b = warp + i * AQ_WARPS;
      if (b < nblocks) {
        const int k = b * 128 + lane * 4;
        float g[4];
        unpack4(raw_g[i], g);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i][j] = v[i][j] * rstd * g[j];
        if (xn_out) store4_bf16(xn_out + static_cast<size_t>(row) * ldn + k, v[i]);
      }
    }
  }

  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = warp + i * AQ_WARPS;
    if (b < nblocks) {
      fwht128_lane4(v[i], lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    }
  }
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, 2);
  amax = warp_max(amax);
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < AQ_WARPS; ++w) t = fmaxf(t, red[w]);
    const float s = quant_scale_from_amax(t);
    bcast = s;
    scale[row] = s;
  }
  __syncthreads();
  const float s = bcast;
  const float inv_s = quant_inv_scale(s);
  int8_t* qr = q + static_cast<size_t>(row) * ldq;
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = warp + i * AQ_WARPS;
    if (b < nblocks) {
      *reinterpret_cast<uint32_t*>(qr + b * 128 + lane * 4) = quant_pack4(v[i], inv_s);
    }
  }
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, TP_EXIT);
  B200_TRACE_FLUSH(TK_ACT_QUANT);
}

template <int MAXB>
static void launch_aq(int mode, const __nv_bfloat16* x, long long ldx, __nv_bfloat16* residual, long long ldr,
                      const __nv_bfloat16* gamma, float eps, int8_t* q, long long ldq, float* scale,
                      __nv_bfloat16* xn, long long ldn, int M, int K, cudaStream_t st) {
  switch (mode) {
    case AQ_PLAIN: launch_ex(act_quant_kernel<MAXB, AQ_PLAIN>, dim3(M), dim3(AQ_THREADS), 0, st, 0, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, xn, ldn, K); break;
    case AQ_NORM: launch_ex(act_quant_kernel<MAXB, AQ_NORM>, dim3(M), dim3(AQ_THREADS), 0, st, 0, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, xn, ldn, K); break;
    case AQ_ADD_NORM: launch_ex(act_quant_kernel<MAXB, AQ_ADD_NORM>, dim3(M), dim3(AQ_THREADS), 0, st, 0, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, xn, ldn, K); break;
    default: launch_ex(act_quant_kernel<MAXB, AQ_SWIGLU>, dim3(M), dim3(AQ_THREADS), 0, st, 0, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, xn, ldn, K); break;
  }
}

}  // namespace b200

using namespace b200;

// mode: 0 plain, 1 rmsnorm, 2 residual-add + rmsnorm (residual updated in place), 3 swiglu (x is [M, 2K]: gate | up)
extern "C" int b200_act_quant(const void* x, long long ldx, void* residual, long long ldr, const void* gamma, float eps,
                              void* q, long long ldq, float* scale, void* xn_out, long long ldn, int M, int K, int mode,
                              cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K <= 0 || (K % 128) != 0 || K > 128 * AQ_WARPS * 16) return -1;
  if (mode < 0 || mode > 3) return -1;
  if ((mode == AQ_NORM || mode == AQ_ADD_NORM) && !gamma) return -1;
  if (mode == AQ_ADD_NORM && !residual) return -1;
  if ((ldx % 4) || (ldq % 4) || (reinterpret_cast<uintptr_t>(x) & 7) || (reinterpret_cast<uintptr_t>(q) & 3)) return -2;
  const int nb = K / 128;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<__nv_bfloat16*>(residual);
  auto G = static_cast<const __nv_bfloat16*>(gamma);
  auto Q = static_cast<int8_t*>(q);
  auto XN = static_cast<__nv_bfloat16*>(xn_out);
  if (nb <= 4 * AQ_WARPS) launch_aq<4>(mode, X, ldx, R, ldr, G, eps, Q, ldq, scale, XN, ldn, M, K, stream);
  else launch_aq<16>(mode, X, ldx, R, ldr, G, eps, Q, ldq, scale, XN, ldn, M, K, stream);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
