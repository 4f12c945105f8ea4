// Mixture-of-experts glue kernels (expert parallelism with replicated tokens: after the attention all-reduce every
// rank holds every token, routes identically, runs only its own experts and the partial outputs are summed across
// ranks like any row-parallel layer).
//
//   router_topk    fp32 router logits [M, E] -> softmax -> top-k ids + (optionally renormalised) weights
//   moe_align      build this rank's work list: per local expert a contiguous run of slots; slot -> token, and for
//                  every (token, k) its slot (or -1 when the expert lives on another rank); plus the table of
//                  128-row tiles the grouped prefill GEMM walks
//   moe_gather     copy the int8 activations (and scales) of the listed tokens into slot order
//   moe_combine    out[token] = sum_k weight[token,k] * expert_out[slot(token,k)]  (local experts only)
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"

namespace b200 {

// one warp per token; E <= 256 (each lane holds E/32 logits)
template <int EPL>
__global__ void __launch_bounds__(128) router_topk_kernel(const float* logits, long long ld, int M, int E, int k,
                                                          int renorm, int* ids, float* wts) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * 4 + warp;
  if (tok >= M) return;
  const float* x = logits + static_cast<size_t>(tok) * ld;
  float v[EPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? x[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) { v[i] = (lane + 32 * i < E) ? __expf(v[i] - mx) : -1.f; sum += fmaxf(v[i], 0.f); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    // arg-max over the remaining probabilities; the lowest expert id wins ties
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best || (v[i] == best && e < bi)) { best = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) if (lane + 32 * i == bi) v[i] = -1.f;      // remove the winner
    picked_sum += best * inv;
    if (lane == j) { my_w = best * inv; my_id = bi; }
  }
  if (lane < k) {
    ids[static_cast<size_t>(tok) * k + lane] = my_id;
    wts[static_cast<size_t>(tok) * k + lane] = renorm ? my_w / picked_sum : my_w;
  }
}

// Single CTA.  counts/offsets: [n_local], [n_local + 1]; slot_token: [M*k] (first offsets[n_local] valid);
// inv: [M*k] slot of each (token, k) or -1; tiles: int4 {expert, first_row, rows, 0} per 128-row tile; meta: [0] total
// slots, [1] number of tiles.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* ids, int M, int k, int e0, int n_local,
                                                         int* counts, int* offsets,
                                                         int* slot_token, int* inv,
                                                         int4* tiles, int* meta) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  extern __shared__ int sm[];
  int* cnt = sm;                  // [n_local]
  int* off = sm + n_local;        // [n_local + 1]
  int* cur = off + n_local + 1;   // [n_local]
  const int pairs = M * k;
  for (int i = threadIdx.x; i < n_local; i += blockDim.x) { cnt[i] = 0; cur[i] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i] - e0;
    if (e >= 0 && e < n_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, nt = 0;
    for (int e = 0; e < n_local; ++e) {
      off[e] = run;
      for (int r = 0; r < cnt[e]; r += 128) { tiles[nt] = make_int4(e, run + r, min(128, cnt[e] - r), 0); ++nt; }
      run += cnt[e];
    }
    off[n_local] = run;
    meta[0] = run;
    meta[1] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_local; i += blockDim.x) { counts[i] = cnt[i]; offsets[i] = off[i]; }
  if (threadIdx.x == 0) offsets[n_local] = off[n_local];
  // Slot assignment.  Tokens are visited in index order by consecutive threads, so slots inside an expert are only
  // approximately token-ordered; every row is processed independently, so values do not depend on the order.
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i] - e0;
    if (e >= 0 && e < n_local) {
      const int s = off[e] + atomicAdd(&cur[e], 1);
      slot_token[s] = i / k;
      inv[i] = s;
    } else {
      inv[i] = -1;
    }
  }
}

// grid = max slots; rows beyond meta[0] exit.  xq int8 [M][d] -> xq_perm [slots][d]
__global__ void __launch_bounds__(128) moe_gather_kernel(const int8_t* xq, const float* sx, int d,
                                                         const int* slot_token, const int* meta,
                                                         int8_t* xq_perm, float* sx_perm) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  const int s = blockIdx.x;
  if (s >= meta[0]) return;
  const int t = slot_token[s];
  const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<size_t>(t) * d);
  uint4* dst = reinterpret_cast<uint4*>(xq_perm + static_cast<size_t>(s) * d);
  for (int i = threadIdx.x; i < d / 16; i += blockDim.x) dst[i] = src[i];
  if (threadIdx.x == 0) sx_perm[s] = sx[t];
}

// one CTA per token: out[t][:] = sum over the token's local slots of weight * y[slot][:]   (bf16 in, fp32 sum, bf16 out)
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* y, long long ldy,
                                                          const int* inv, const float* wts, int k,
                                                          int d, __nv_bfloat16* out, long long ldo) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  const int t = blockIdx.x;
  __shared__ int slot_s[32];
  __shared__ float w_s[32];
  if (threadIdx.x < k) { slot_s[threadIdx.x] = inv[static_cast<size_t>(t) * k + threadIdx.x]; w_s[threadIdx.x] = wts[static_cast<size_t>(t) * k + threadIdx.x]; }
  __syncthreads();
  for (int c = threadIdx.x; c < d / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int s = slot_s[j];
      if (s < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(s) * ldy + c * 8);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      const float wt = w_s[j];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += wt * __uint_as_float(w[i] << 16);
        acc[2 * i + 1] += wt * __uint_as_float(w[i] & 0xffff0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pb = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      o[i] = *reinterpret_cast<const uint32_t*>(&pb);
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ldo + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_router_topk(const float* logits, long long ld, int M, int E, int k, int renorm, int* ids, float* wts,
                                cudaStream_t stream) {
  if (M <= 0) return 0;
  if (E <= 0 || E > 256 || k <= 0 || k > 32 || k > E) return -1;
  const int grid = (M + 3) / 4;
  if (E <= 32) launch_ex(router_topk_kernel<1>, dim3(grid), dim3(128), 0, stream, 0, logits, ld, M, E, k, renorm, ids, wts);
  else if (E <= 64) launch_ex(router_topk_kernel<2>, dim3(grid), dim3(128), 0, stream, 0, logits, ld, M, E, k, renorm, ids, wts);
  else if (E <= 128) launch_ex(router_topk_kernel<4>, dim3(grid), dim3(128), 0, stream, 0, logits, ld, M, E, k, renorm, ids, wts);
  else launch_ex(router_topk_kernel<8>, dim3(grid), dim3(128), 0, stream, 0, logits, ld, M, E, k, renorm, ids, wts);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_moe_align(const int* ids, int M, int k, int e0, int n_local, int* counts, int* offsets, int* slot_token,
                              int* inv, void* tiles, int* meta, cudaStream_t stream) {
  if (M <= 0 || n_local <= 0 || n_local > 1024) return -1;
  const size_t smem = static_cast<size_t>(3 * n_local + 1) * sizeof(int);
  launch_ex(moe_align_kernel, dim3(1), dim3(1024), smem, stream, 0, ids, M, k, e0, n_local, counts, offsets, slot_token, inv,
                                              static_cast<int4*>(tiles), meta);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_moe_gather(const void* xq, const float* sx, int d, const int* slot_token, const int* meta, int max_slots,
                               void* xq_perm, float* sx_perm, cudaStream_t stream) {
  if (max_slots <= 0) return 0;
  if (d % 16) return -1;
  launch_ex(moe_gather_kernel, dim3(max_slots), dim3(128), 0, stream, 0, static_cast<const int8_t*>(xq), sx, d, slot_token, meta,
                                                   static_cast<int8_t*>(xq_perm), sx_perm);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_moe_combine(const void* y, long long ldy, const int* inv, const float* wts, int M, int k, int d, void* out,
                                long long ldo, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (d % 8 || k > 32) return -1;
  launch_ex(moe_combine_kernel, dim3(M), dim3(256), 0, stream, 0, static_cast<const __nv_bfloat16*>(y), ldy, inv, wts, k, d,
                                            static_cast<__nv_bfloat16*>(out), ldo);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
