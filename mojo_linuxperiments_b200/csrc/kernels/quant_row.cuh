// One activation row through the prologue of a W8A8 linear, by one whole CTA, with the row parked in shared memory:
//   (residual add) -> (RMSNorm) | (SwiGLU) -> block-128 Hadamard rotation -> per-token int8.
// This is the body of the stand-alone activation kernel (act_quant.cu) restated so that a CTA of any warp count can
// run it with few registers (the row lives in shared memory between the passes instead of in registers), which is
// what lets the decode GEMM carry its own quantiser CTAs: the CTAs with the lowest block indices of a GEMM launch turn
// the bf16 rows into the int8 operand, publish a flag per row, and the GEMM CTAs of the same launch wait for the flags
// instead of for a previous kernel.  No counterpart in the reference (it has no quantisation).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hadamard.cuh"

namespace b200 {

enum QuantRowMode : int { QR_NONE = 0, QR_PLAIN = 1, QR_NORM = 2, QR_ADD_NORM = 3, QR_SWIGLU = 4 };

struct QuantProlog {
  int mode;                        // QuantRowMode; QR_NONE: the GEMM reads int8 rows an earlier kernel made
  const __nv_bfloat16* x;          // [M][K] (QR_SWIGLU: [M][2K] = gate | up), row pitch ldx elements
  long long ldx;
  __nv_bfloat16* residual;         // QR_ADD_NORM: [M][K], updated in place to bf16(residual + x)
  long long ldr;
  const __nv_bfloat16* gamma;      // QR_NORM / QR_ADD_NORM: [K]
  float eps;
  int8_t* q;                       // [M][K] int8 out (row pitch K): the operand the GEMM CTAs load by TMA
  float* scale;                    // [M] per-token scales out
  uint32_t* flags;                 // [M] one word per row: holds `ticket` once the row is complete
  const uint32_t* step;            // device word that changes between replays of a captured launch
  uint32_t launch_id;              // differs between the launches of one step
  int rows;                        // grid rows (blockIdx.y values) taken by quantiser CTAs; 0 with a mode set: the inline
                                   // form (a few tokens) - every GEMM CTA quantises its own K slice of the rows straight
                                   // into its operand stages, the cluster exchanges the row statistics
  __nv_bfloat16* residual_out;     // QR_ADD_NORM: where bf16(residual + x) goes (may equal residual with quantiser CTAs;
  long long ldro;                  // must differ for the inline form, where every cluster reads the old residual)
  int allow_inline;                // host only: the caller accepts the inline form
};

__device__ __forceinline__ uint32_t quant_ticket(const QuantProlog& q) {
  return ((*reinterpret_cast<const volatile uint32_t*>(q.step) & 0xffffu) << 16) | (q.launch_id & 0xffffu) | 0x80000000u;
}

__device__ __forceinline__ void unpack4_bf16(const uint2& r, float (&o)[4]) {
  o[0] = __uint_as_float(r.x << 16); o[1] = __uint_as_float(r.x & 0xffff0000u);
  o[2] = __uint_as_float(r.y << 16); o[3] = __uint_as_float(r.y & 0xffff0000u);
}

// buf: K floats of shared memory; red: 2 * NW + 2 floats of shared memory.  Every thread of the CTA calls this.
template <int NW>
__device__ void quant_row_cta(const QuantProlog& p, int row, int K, float* buf, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = K >> 7;
  const __nv_bfloat16* xr = p.x + static_cast<size_t>(row) * p.ldx;
  const bool norm = p.mode == QR_NORM || p.mode == QR_ADD_NORM;
  float ss = 0.f, amax = 0.f;
  // With one or two warps per scheduler every global round trip is exposed, so the loads of up to QR_CH blocks are
  // issued back to back before any of them is used (as the stand-alone kernel does with the whole row).
  constexpr int QR_CH = 8;
  // pass A: load, element-wise part; rotate right away unless a row statistic (the norm) is needed first
  for (int b0 = warp; b0 < nb; b0 += NW * QR_CH) {
    uint2 ra[QR_CH], rb[QR_CH];
#pragma unroll
    for (int c = 0; c < QR_CH; ++c) {
      const int b = b0 + c * NW;
      ra[c] = make_uint2(0u, 0u); rb[c] = make_uint2(0u, 0u);
      if (b < nb) {
        const int k = b * 128 + lane * 4;
        ra[c] = *reinterpret_cast<const uint2*>(xr + k);
        if (p.mode == QR_SWIGLU) rb[c] = *reinterpret_cast<const uint2*>(xr + K + k);
        if (p.mode == QR_ADD_NORM) rb[c] = *reinterpret_cast<const uint2*>(p.residual + static_cast<size_t>(row) * p.ldr + k);
      }
    }
#pragma unroll
    for (int c = 0; c < QR_CH; ++c) {
      const int b = b0 + c * NW;
      if (b >= nb) continue;
      const int k = b * 128 + lane * 4;
      float v[4];
      unpack4_bf16(ra[c], v);
      if (p.mode == QR_SWIGLU) {
        float u[4];
        unpack4_bf16(rb[c], u);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __fdividef(v[j], 1.f + __expf(-v[j])) * u[j];
      } else if (p.mode == QR_ADD_NORM) {
        float r[4];
        unpack4_bf16(rb[c], r);
        // the residual stream is kept in bf16: round the sum once, and normalise what was stored
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(__float2bfloat16(__fadd_rn(v[j], r[j])));
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&lo);
        raw.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.residual_out + static_cast<size_t>(row) * p.ldro + k) = raw;
      }
      if (norm) {
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += v[j] * v[j];
      } else {
        fwht128_lane4(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[j]));
      }
      *reinterpret_cast<float4*>(buf + k) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
  if (norm) {
    // the norm weights of this warp's first blocks are requested before the reduction is waited for
    uint2 rg[QR_CH];
#pragma unroll
    for (int c = 0; c < QR_CH; ++c) {
      const int b = warp + c * NW;
      rg[c] = make_uint2(0u, 0u);
      if (b < nb) rg[c] = __ldg(reinterpret_cast<const uint2*>(p.gamma + b * 128 + lane * 4));
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) t += red[w];
    const float rstd = rsqrtf(t / static_cast<float>(K) + p.eps);
    // pass B: normalise, rotate
    for (int b0 = warp; b0 < nb; b0 += NW * QR_CH) {
      if (b0 != warp) {
#pragma unroll
        for (int c = 0; c < QR_CH; ++c) {
          const int b = b0 + c * NW;
          if (b < nb) rg[c] = __ldg(reinterpret_cast<const uint2*>(p.gamma + b * 128 + lane * 4));
        }
      }
#pragma unroll
      for (int c = 0; c < QR_CH; ++c) {
        const int b = b0 + c * NW;
        if (b >= nb) continue;
        const int k = b * 128 + lane * 4;
        const float4 x4 = *reinterpret_cast<const float4*>(buf + k);
        float g[4];
        unpack4_bf16(rg[c], g);
        float v[4] = {x4.x * rstd * g[0], x4.y * rstd * g[1], x4.z * rstd * g[2], x4.w * rstd * g[3]};
        fwht128_lane4(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(v[j]));
        *reinterpret_cast<float4*>(buf + k) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
  }
  amax = warp_max(amax);
  if (lane == 0) red[NW + warp] = amax;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < NW; ++w) t = fmaxf(t, red[NW + w]);
  const float s = quant_scale_from_amax(t), inv_s = quant_inv_scale(s);
  // pass C: quantise (every warp re-reads only what it wrote itself)
  int8_t* qr = p.q + static_cast<size_t>(row) * K;
  for (int b = warp; b < nb; b += NW) {
    const int k = b * 128 + lane * 4;
    const float4 x4 = *reinterpret_cast<const float4*>(buf + k);
    const float v[4] = {x4.x, x4.y, x4.z, x4.w};
    *reinterpret_cast<uint32_t*>(qr + k) = quant_pack4(v, inv_s);
  }
  if (threadIdx.x == 0) p.scale[row] = s;
}

}  // namespace b200
