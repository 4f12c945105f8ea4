// Paged-KV decode attention (one query token per sequence, grouped-query heads).
//
// Grid (kv_head, sequence, split).  A CTA streams its slice of the sequence's K and V pages exactly once for the
// whole group of G query heads that share the KV head (the op is bound by those bytes), in sub-chunks of 256
// tokens with an online softmax.  With more than one split the CTAs write un-normalised partials and the last
// CTA to arrive for a (sequence, kv_head) merges them in the same launch.
//
//   phase 1  four lanes <-> token (each lane 32 dims = 4 x 16-byte loads, so a warp reads eight whole 256-byte
//            K rows per instruction group), partial dots with the G query vectors in smem, 2-step shuffle reduce
//   phase 2  warp <-> head: running max / sum, probabilities back to smem
//   phase 3  thread <-> (8 output dims, token slice): P.V with 16-byte V loads, then a cross-slice reduction
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"

namespace b200 {

constexpr int AD_THREADS = 128;
constexpr int AD_TC = 256;            // tokens per sub-chunk
constexpr int AD_D = 128;

struct DecodeParams {
  const __nv_bfloat16* q;             // [B][hq][128]
  const __nv_bfloat16* cache;         // [pages][2][hkv][page_size][128]
  const int* page_table;              // [B][max_pages]
  const int* seq_lens;                // [B]
  __nv_bfloat16* out;                 // [B][hq][128]
  float* part_acc;                    // [B][hq][splits][128]
  float* part_ml;                     // [B][hq][splits][2]
  unsigned* counters;                 // [B][hkv], zero between launches
  int hq, hkv, page_size, max_pages, splits;
  float scale_log2;                   // softmax scale * log2(e)
  int* status;                        // optional: ST_BAD_ARGUMENT when a length exceeds the page table row
};

__device__ __forceinline__ void bf16x8_to_float(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <int G>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(const DecodeParams p) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  __shared__ __align__(16) float q_s[G][4 * 36];     // four 32-dim parts, padded so the parts hit different banks
  __shared__ float sc[G][AD_TC];
  __shared__ float alpha_s[G], m_s[G], l_s[G];
  __shared__ __align__(16) float out_s[G][AD_D];
  __shared__ int last_flag;

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // A length beyond the sequence's page-table row would index the next row (or past the table): attend to what the
  // row can describe and say so in the status word.
  int len = p.seq_lens[b];
  if (len > p.max_pages * p.page_size) {
    if (tid == 0 && p.status) atomicCAS(p.status, 0, static_cast<int>(ST_BAD_ARGUMENT) | (8 << 8));
    len = p.max_pages * p.page_size;
  }
  if (len < 0) len = 0;
  const int per = ((len + p.splits - 1) / p.splits + 31) & ~31;
  const int t0 = split * per;
  const int t1 = min(len, t0 + per);
  const int* pt = p.page_table + static_cast<size_t>(b) * p.max_pages;
  const size_t page_stride = static_cast<size_t>(2) * p.hkv * p.page_size * AD_D;
  const size_t k_head_off = static_cast<size_t>(kvh) * p.page_size * AD_D;
  const size_t v_head_off = static_cast<size_t>(p.hkv + kvh) * p.page_size * AD_D;

  for (int i = tid; i < G * AD_D; i += AD_THREADS) {
    const int g = i / AD_D, d = i % AD_D;
    q_s[g][(d >> 5) * 36 + (d & 31)] = __bfloat162float(p.q[(static_cast<size_t>(b) * p.hq + kvh * G + g) * AD_D + d]) * p.scale_log2;
    out_s[g][d] = 0.f;
  }
  if (tid < G) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
  __syncthreads();

  const int dg = tid & 15, ts = tid >> 4;
  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[g][k] = 0.f;

  for (int c0 = t0; c0 < t1; c0 += AD_TC) {
    const int n = min(AD_TC, t1 - c0);
    // ---- phase 1: scores ----
    {
      const int part = lane & 3, tsub = lane >> 2;
#pragma unroll 2
      for (int tb = warp * 8; tb < n; tb += (AD_THREADS / 32) * 8) {
        const int tt = tb + tsub;
        const int tok = c0 + min(tt, n - 1);
        const int page = pt[tok / p.page_size];
        const uint4* kp = reinterpret_cast<const uint4*>(p.cache + static_cast<size_t>(page) * page_stride + k_head_off +
                                                          static_cast<size_t>(tok % p.page_size) * AD_D + part * 32);
        uint4 kr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) kr[i] = kp[i];
        float dot[G];
#pragma unroll
        for (int g = 0; g < G; ++g) dot[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float kf[8];
          bf16x8_to_float(kr[i], kf);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][part * 36 + 8 * i]);
            const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][part * 36 + 8 * i + 4]);
            dot[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
          }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 1);
          dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 2);
        }
        if (tt < n) {
#pragma unroll
          for (int g = 0; g < G; ++g)
            if ((g & 3) == part) sc[g][tt] = dot[g];
        }
      }
    }
    __syncthreads();
    // ---- phase 2: online softmax bookkeeping, one warp per head ----
    for (int g = warp; g < G; g += AD_THREADS / 32) {
      float mx = -INFINITY;
      for (int tt = lane; tt < n; tt += 32) mx = fmaxf(mx, sc[g][tt]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = m_s[g];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int tt = lane; tt < n; tt += 32) {
        const float e = exp2f(sc[g][tt] - m_new);
        sc[g][tt] = e;
        sum += e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        const float a = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m_new);
        alpha_s[g] = a;
        l_s[g] = l_s[g] * a + sum;
        m_s[g] = m_new;
      }
    }
    __syncthreads();
    // ---- phase 3: P.V ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float a = alpha_s[g];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[g][k] *= a;
    }
#pragma unroll 4
    for (int tt = ts; tt < n; tt += 8) {
      const int tok = c0 + tt;
      const int page = pt[tok / p.page_size];
      const uint4 vr = *(reinterpret_cast<const uint4*>(p.cache + static_cast<size_t>(page) * page_stride + v_head_off +
                                                             static_cast<size_t>(tok % p.page_size) * AD_D + 8 * dg));
      float vf[8];
      bf16x8_to_float(vr, vf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = sc[g][tt];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[g][k] += pr * vf[k];
      }
    }
    __syncthreads();
  }

  // ---- reduce the 8 token slices ----
  for (int s = 0; s < 8; ++s) {
    if (ts == s) {
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int k = 0; k < 8; ++k) out_s[g][8 * dg + k] += acc[g][k];
    }
    __syncthreads();
  }

  if (p.splits == 1) {
    for (int i = tid; i < G * AD_D; i += AD_THREADS) {
      const int g = i / AD_D, d = i % AD_D;
      const float l = l_s[g];
      p.out[(static_cast<size_t>(b) * p.hq + kvh * G + g) * AD_D + d] = __float2bfloat16(l > 0.f ? out_s[g][d] / l : 0.f);
    }
    return;
  }

  // ---- publish the partial, last CTA merges ----
  for (int i = tid; i < G * AD_D; i += AD_THREADS) {
    const int g = i / AD_D, d = i % AD_D;
    p.part_acc[((static_cast<size_t>(b) * p.hq + kvh * G + g) * p.splits + split) * AD_D + d] = out_s[g][d];
  }
  if (tid < G) {
    float* ml = p.part_ml + ((static_cast<size_t>(b) * p.hq + kvh * G + tid) * p.splits + split) * 2;
    ml[0] = m_s[tid];
    ml[1] = l_s[tid];
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned* ctr = p.counters + static_cast<size_t>(b) * p.hkv + kvh;
    const unsigned old = atomicAdd(ctr, 1u);
    last_flag = (old == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
    if (last_flag) *ctr = 0;
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  for (int i = tid; i < G * AD_D; i += AD_THREADS) {
    const int g = i / AD_D, d = i % AD_D;
    const size_t base = (static_cast<size_t>(b) * p.hq + kvh * G + g) * p.splits;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) m = fmaxf(m, __ldcg(p.part_ml + (base + s) * 2));
    float l = 0.f, o = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = __ldcg(p.part_ml + (base + s) * 2);
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      l += w * __ldcg(p.part_ml + (base + s) * 2 + 1);
      o += w * __ldcg(p.part_acc + (base + s) * AD_D + d);
    }
    p.out[(static_cast<size_t>(b) * p.hq + kvh * G + g) * AD_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
  }
}

}  // namespace b200

using namespace b200;

// scratch the split path needs: floats for (acc, m, l) partials
extern "C" size_t b200_attn_decode_scratch_floats(int B, int hq, int splits) {
  return static_cast<size_t>(B) * hq * splits * (AD_D + 2);
}

extern "C" int b200_attn_decode(const void* q, const void* cache, const int* page_table, const int* seq_lens, void* out,
                                float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size, int max_pages,
                                int splits, float scale, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (hq % hkv || page_size <= 0 || max_pages <= 0) return -1;
  const int G = hq / hkv;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!scratch || !counters)) return -1;
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.page_table = page_table; p.seq_lens = seq_lens; p.out = static_cast<__nv_bfloat16*>(out);
  p.part_acc = scratch;
  p.part_ml = scratch ? scratch + static_cast<size_t>(B) * hq * splits * AD_D : nullptr;
  p.counters = counters;
  p.hq = hq; p.hkv = hkv; p.page_size = page_size; p.max_pages = max_pages; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid(hkv, B, splits);
  switch (G) {
    case 1: launch_ex(attn_decode_kernel<1>, dim3(grid), dim3(AD_THREADS), 0, stream, 0, p); break;
    case 2: launch_ex(attn_decode_kernel<2>, dim3(grid), dim3(AD_THREADS), 0, stream, 0, p); break;
    case 4: launch_ex(attn_decode_kernel<4>, dim3(grid), dim3(AD_THREADS), 0, stream, 0, p); break;
    case 8: launch_ex(attn_decode_kernel<8>, dim3(grid), dim3(AD_THREADS), 0, stream, 0, p); break;
    case 16: launch_ex(attn_decode_kernel<16>, dim3(grid), dim3(AD_THREADS), 0, stream, 0, p); break;
    default: return -1;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared and documented in attn_decode_noalloc.h).
// ---------------------------------------------------------------------------------------------------------------
#include "attn_decode_noalloc.h"
#include <atomic>
#include <cstdio>

namespace b200 {

constexpr size_t ADN_MAX_COUNTERS = 4096;                       // (sequence, kv head) pairs
constexpr size_t ADN_MAX_FLOATS = 1u << 20;                     // split-KV partials: 4 MiB
constexpr size_t ADN_COUNTER_BYTES = ADN_MAX_COUNTERS * sizeof(unsigned);
constexpr size_t ADN_BYTES = ADN_COUNTER_BYTES + ADN_MAX_FLOATS * sizeof(float);
constexpr int ADN_MAX_DEVICES = 64;

// [counters | partials]; lives in every GPU that loads the library.  On the host this name is only a handle for
// cudaGetSymbolAddress: it must never be passed to a kernel as if it were a device pointer.
static __device__ __align__(256) unsigned char g_attn_decode_scratch[ADN_BYTES];

// device address of the array on the current device, looked up once per device
static int adn_scratch_address(unsigned char** out) {
  // Threads that make their first call on a device at the same time each look the address up and store the same
  // value; the atomic only makes that well defined.
  static std::atomic<unsigned char*> cached[ADN_MAX_DEVICES];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= ADN_MAX_DEVICES) return -3000 - static_cast<int>(e);
  if (!cached[dev].load(std::memory_order_acquire)) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_decode_scratch);        // resolves against the device that is current now
    if (e != cudaSuccess || !p) {
      std::fprintf(stderr, "b200_attn_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return -3000 - static_cast<int>(e);
    }
    cached[dev].store(static_cast<unsigned char*>(p), std::memory_order_release);
  }
  *out = cached[dev].load(std::memory_order_acquire);
  return 0;
}

}  // namespace b200

extern "C" int b200_attn_decode_noalloc(const void* q, const void* cache, const int* page_table, const int* seq_lens, void* out,
                                        int B, int hq, int hkv, int page_size, int max_pages, int splits, float scale,
                                        cudaStream_t stream) {
  if (B <= 0) return 0;
  if (hq <= 0 || hkv <= 0 || (hq % hkv)) return -1;
  if (splits < 1) splits = 1;
  // One split per sequence: the kernel touches neither the partials nor the counters, so no limit applies and
  // nothing has to be cleared.
  if (splits == 1)
    return b200_attn_decode(q, cache, page_table, seq_lens, out, nullptr, nullptr, B, hq, hkv, page_size, max_pages, 1, scale,
                            nullptr, stream);
  const size_t need_floats = b200_attn_decode_scratch_floats(B, hq, splits);
  const size_t need_counters = static_cast<size_t>(B) * hkv;
  if (need_floats > ADN_MAX_FLOATS || need_counters > ADN_MAX_COUNTERS) {
    std::fprintf(stderr,
                 "b200_attn_decode_noalloc: B=%d hq=%d hkv=%d splits=%d needs %zu scratch floats and %zu counters; the built-in "
                 "scratch holds %zu floats and %zu counters. Use fewer splits or b200_attn_decode with caller-owned scratch.\n",
                 B, hq, hkv, splits, need_floats, need_counters, static_cast<size_t>(ADN_MAX_FLOATS), static_cast<size_t>(ADN_MAX_COUNTERS));
    return B200_NOALLOC_TOO_LARGE;
  }
  unsigned char* base = nullptr;
  const int rc = adn_scratch_address(&base);
  if (rc) return rc;
  unsigned* counters = reinterpret_cast<unsigned*>(base);
  float* partials = reinterpret_cast<float*>(base + ADN_COUNTER_BYTES);
  // the arrival counters must start at zero; the array may hold anything a previous (possibly failed) call left
  cudaError_t e = cudaMemsetAsync(counters, 0, need_counters * sizeof(unsigned), stream);
  if (e != cudaSuccess) return -2000 - static_cast<int>(e);
  return b200_attn_decode(q, cache, page_table, seq_lens, out, partials, counters, B, hq, hkv, page_size, max_pages, splits,
                          scale, nullptr, stream);
}
