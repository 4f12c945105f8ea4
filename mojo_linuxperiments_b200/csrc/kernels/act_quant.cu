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
#include <cstdlib>

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

// A few token rows (decode): one CTA per row leaves most SMs idle and makes each warp walk several 128-blocks one
// after the other, and every step of that walk is exposed latency.  Here a row belongs to a thread-block cluster of C
// CTAs: CTA c takes the c-th run of blocks, the row statistics cross the cluster once through distributed shared
// memory.  One exchange is enough because the rotation is linear: the values are rotated before the norm's scalar
// 1/rms is known (sum of squares and maximum travel together), and 1/rms is folded into the quantisation step.
template <int MAXB, int MODE>
__global__ void __launch_bounds__(AQ_THREADS)
act_quant_cluster_kernel(const __nv_bfloat16* x, long long ldx, __nv_bfloat16* residual, long long ldr,
                         const __nv_bfloat16* gamma, float eps, int8_t* q, long long ldq, float* scale, int K, int C) {
  pdl_launch_dependents();
  B200_TRACE_INIT();
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, TP_START);
  __shared__ float red[2 * AQ_WARPS];
  __shared__ __align__(16) float rx[8 * 4];                  // [sender CTA][sum of squares, maximum, -, -]
  cluster_arrive_relaxed();                                  // "this CTA runs": waited for before the remote stores
  pdl_wait();
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, TP_DEPS);

  const int row = blockIdx.y, c = static_cast<int>(cluster_ctarank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblocks = K >> 7, per = (nblocks + C - 1) / C;
  const int b_lo = c * per, b_hi = min(nblocks, b_lo + per);
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  constexpr bool NORM = MODE == AQ_NORM || MODE == AQ_ADD_NORM;

  uint2 raw_a[MAXB], raw_b[MAXB], raw_g[MAXB];
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = b_lo + warp + i * AQ_WARPS;
    raw_a[i] = make_uint2(0u, 0u); raw_b[i] = make_uint2(0u, 0u); raw_g[i] = make_uint2(0u, 0u);
    if (b < b_hi) {
      const int k = b * 128 + lane * 4;
      raw_a[i] = *reinterpret_cast<const uint2*>(xr + k);
      if constexpr (MODE == AQ_SWIGLU) raw_b[i] = *reinterpret_cast<const uint2*>(xr + K + k);
      if constexpr (MODE == AQ_ADD_NORM) raw_b[i] = *reinterpret_cast<const uint2*>(residual + static_cast<size_t>(row) * ldr + k);
      if constexpr (NORM) raw_g[i] = __ldg(reinterpret_cast<const uint2*>(gamma + k));
    }
  }
  auto unpack4 = [](const uint2& r, float (&o)[4]) {
    o[0] = __uint_as_float(r.x << 16); o[1] = __uint_as_float(r.x & 0xffff0000u);
    o[2] = __uint_as_float(r.y << 16); o[3] = __uint_as_float(r.y & 0xffff0000u);
  };
  float v[MAXB][4];
  float ss = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = b_lo + warp + i * AQ_WARPS;
    if (b < b_hi) {
      unpack4(raw_a[i], v[i]);
      if constexpr (MODE == AQ_SWIGLU) {
        float u[4];
        unpack4(raw_b[i], u);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i][j] = __fdividef(v[i][j], 1.f + __expf(-v[i][j])) * u[j];
      }
      if constexpr (MODE == AQ_ADD_NORM) {
        float r[4];
        unpack4(raw_b[i], r);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j] + r[j]));
        store4_bf16(residual + static_cast<size_t>(row) * ldr + b * 128 + lane * 4, v[i]);
      }
      if constexpr (NORM) {
        float g[4];
        unpack4(raw_g[i], g);
#pragma unroll
        for (int j = 0; j < 4; ++j) { ss += v[i][j] * v[i][j]; v[i][j] *= g[j]; }
      }
      fwht128_lane4(v[i], lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[i][j] = 0.f;
    }
  }
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, 2);
  // the two statistics walk the butterflies together
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  }
  if (lane == 0) { red[warp] = ss; red[AQ_WARPS + warp] = amax; }
  __syncthreads();
  cluster_wait_acquire();                                    // every CTA of the cluster runs
  if (threadIdx.x < C) {                                     // thread d tells CTA d what this CTA saw
    float s_cta = 0.f, a_cta = 0.f;
#pragma unroll
    for (int w = 0; w < AQ_WARPS; ++w) { s_cta += red[w]; a_cta = fmaxf(a_cta, red[AQ_WARPS + w]); }
    st_shared_cluster_v4(mapa_shared(smem_u32(rx + 4 * c), threadIdx.x), __float_as_uint(s_cta), __float_as_uint(a_cta), 0u, 0u);
  }
  cluster_arrive_release();
  cluster_wait_acquire();
  float tss = 0.f, tam = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r)
    if (r < C) { tss += rx[4 * r]; tam = fmaxf(tam, rx[4 * r + 1]); }
  const float rstd = NORM ? rsqrtf(tss / static_cast<float>(K) + eps) : 1.f;
  const float s = quant_scale_from_amax(tam * rstd);
  const float inv = rstd * quant_inv_scale(s);
  if (c == 0 && threadIdx.x == 0) scale[row] = s;
  int8_t* qr = q + static_cast<size_t>(row) * ldq;
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = b_lo + warp + i * AQ_WARPS;
    if (b < b_hi) *reinterpret_cast<uint32_t*>(qr + b * 128 + lane * 4) = quant_pack4(v[i], inv);
  }
  if (threadIdx.x == 0) B200_TRACE(TK_ACT_QUANT, TP_EXIT);
  B200_TRACE_FLUSH(TK_ACT_QUANT);
}

template <int MAXB>
static void launch_aq_cluster(int mode, const __nv_bfloat16* x, long long ldx, __nv_bfloat16* residual, long long ldr,
                              const __nv_bfloat16* gamma, float eps, int8_t* q, long long ldq, float* scale,
                              int M, int K, int C, cudaStream_t st) {
  const dim3 grid(C, M), block(AQ_THREADS), cl(C, 1, 1);
  switch (mode) {
    case AQ_PLAIN: launch_ex_cluster(act_quant_cluster_kernel<MAXB, AQ_PLAIN>, grid, block, 0, st, cl, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, K, C); break;
    case AQ_NORM: launch_ex_cluster(act_quant_cluster_kernel<MAXB, AQ_NORM>, grid, block, 0, st, cl, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, K, C); break;
    case AQ_ADD_NORM: launch_ex_cluster(act_quant_cluster_kernel<MAXB, AQ_ADD_NORM>, grid, block, 0, st, cl, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, K, C); break;
    default: launch_ex_cluster(act_quant_cluster_kernel<MAXB, AQ_SWIGLU>, grid, block, 0, st, cl, x, ldx, residual, ldr, gamma, eps, q, ldq, scale, K, C); break;
  }
}

// Cluster size for a decode-sized call: about one block per warp, at most 8 CTAs per row, and only while the grid
// stays within one wave (B200RT_AQ_CLUSTER=0 turns the form off).
static int aq_cluster_size(int M, int K, bool want_normed) {
  static int env = -1;
  if (env < 0) { const char* e = std::getenv("B200RT_AQ_CLUSTER"); env = (e && e[0] == '0') ? 0 : 1; }
  if (!env || want_normed || M > 64) return 1;
  const int nb = K / 128;
  int c = 1;
  while (c < 8 && nb / (2 * c) >= AQ_WARPS && M * 2 * c <= 296) c *= 2;
  if ((nb + c - 1) / c > 2 * AQ_WARPS) return 1;             // more than two blocks per warp: the one-CTA form holds them
  return c;
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
  const int C = aq_cluster_size(M, K, xn_out != nullptr);
  if (C > 1) {
    const int per = (nb + C - 1) / C;
    if (per <= AQ_WARPS) launch_aq_cluster<1>(mode, X, ldx, R, ldr, G, eps, Q, ldq, scale, M, K, C, stream);
    else launch_aq_cluster<2>(mode, X, ldx, R, ldr, G, eps, Q, ldq, scale, M, K, C, stream);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
  }
  if (nb <= 4 * AQ_WARPS) launch_aq<4>(mode, X, ldx, R, ldr, G, eps, Q, ldq, scale, XN, ldn, M, K, stream);
  else launch_aq<16>(mode, X, ldx, R, ldr, G, eps, Q, ldq, scale, XN, ldn, M, K, stream);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
