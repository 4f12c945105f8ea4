// Paged-KV decode attention, TMA-fed (page size 16): the form used when it applies; attn_decode.cu is the general one.
//
// Grid (kv_head, sequence, split), 160 threads: warp 4 is the producer, warps 0..3 consume.
//   * The producer walks the sequence's page table and issues one tiled TMA load per K block and per V block of a
//     page (16 tokens x 128 dims bf16 = 4 KiB each, viewed as 32 half-rows of 128 bytes with the 128-byte swizzle)
//     into a 6-stage ring: 48 KiB of loads in flight per CTA without holding a single register, three CTAs per SM.
//   * Each consumer warp owns every fourth page and keeps its own online-softmax state, so nothing in the main
//     loop synchronises the CTA.  For a page: lane (token t, half h) dots its 64 dims with the G query vectors
//     (all lanes read the same logical 16-byte unit, so the swizzle spreads them over all banks and the query reads
//     are broadcasts), a shuffle joins the halves, 16-lane shuffles give the row max / sum, and P.V accumulates
//     4 output dims per lane with V read as 8-byte words in token order.
//   * The four warps merge through shared memory; with several splits the last CTA merges the partials.
// All mbarrier waits are bounded.
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include <cuda.h>

namespace b200 {

constexpr int ADT_THREADS = 160;
constexpr int ADT_STAGES = 6;
constexpr int ADT_PS = 16;                 // tokens per page
constexpr int ADT_D = 128;
constexpr int ADT_BLOCK = ADT_PS * ADT_D * 2;   // 4 KiB: one K or V block
constexpr int ADT_MAX_PAGES = 256;              // page ids staged in shared memory per CTA (more are read on demand)

struct DecodeTmaParams {
  const __nv_bfloat16* q;
  const int* page_table;
  const int* seq_lens;
  __nv_bfloat16* out;
  float* part_acc;
  float* part_ml;
  unsigned* counters;
  int hq, hkv, max_pages, splits;
  float scale_log2;
  int* status;
  unsigned long long limit_ns;
};

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

template <int G>
__global__ void __launch_bounds__(ADT_THREADS) attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_kv,
                                                                      const DecodeTmaParams p) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [stage][K 4K | V 4K] ... then q, merge buffers, barriers
  float* q_s = reinterpret_cast<float*>(smem + ADT_STAGES * 2 * ADT_BLOCK);          // [G][128]
  float* mg_acc = q_s + G * ADT_D;                                                   // [4 warps][G][128]
  float* mg_ml = mg_acc + 4 * G * ADT_D;                                             // [4][G][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(mg_ml + 4 * G * 2 + 2);
  bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(bars) + 7) & ~uintptr_t(7));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * ADT_STAGES);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  int* page_s = last_flag + 1;                       // [ADT_MAX_PAGES] this CTA's slice of the page table
  const uint32_t ring = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (ADT_STAGES + s); };

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int len = p.seq_lens[b];
  if (len > p.max_pages * ADT_PS) {         // the page-table row cannot describe more tokens than this
    if (tid == 0 && p.status) atomicCAS(p.status, 0, (int)ST_BAD_ARGUMENT | (4 << 8));
    len = p.max_pages * ADT_PS;
  }
  if (len < 0) len = 0;
  const int total_pages = (len + ADT_PS - 1) / ADT_PS;
  const int per = (total_pages + p.splits - 1) / p.splits;
  const int pg0 = split * per, pg1 = min(total_pages, pg0 + per);
  const int npages = max(0, pg1 - pg0);
  const int* pt = p.page_table + static_cast<size_t>(b) * p.max_pages;

  if (tid == 0) {
    for (int s = 0; s < ADT_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < G * ADT_D; i += ADT_THREADS)
    q_s[i] = __bfloat162float(p.q[(static_cast<size_t>(b) * p.hq + kvh * G) * ADT_D + i]) * p.scale_log2;
  // the page ids are read once, in parallel, so the producer never waits on a global load between two TMA issues
  for (int i = tid; i < min(npages, ADT_MAX_PAGES); i += ADT_THREADS) page_s[i] = pt[pg0 + i];
  __syncthreads();

  float m_run[G], l_run[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f; }

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tmap_kv);
      bool ok = true;
      for (int i = 0; i < npages && ok; ++i) {
        const int s = i % ADT_STAGES;
        const uint32_t ph = (i / ADT_STAGES) & 1u;
        if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (4 << 8)), p.limit_ns)) { ok = false; break; }
        const int page = i < ADT_MAX_PAGES ? page_s[i] : pt[pg0 + i];
        // half-row index of the K block of (page, head): ((page*2 + 0)*hkv + head) * 32 ; V block: kv = 1
        const int rk = ((page * 2 + 0) * p.hkv + kvh) * (ADT_PS * 2);
        const int rv = ((page * 2 + 1) * p.hkv + kvh) * (ADT_PS * 2);
        mbar_expect_tx(full_bar(s), 2 * ADT_BLOCK);
        tma_load_2d(ring + s * 2 * ADT_BLOCK, &tmap_kv, full_bar(s), 0, rk);
        tma_load_2d(ring + s * 2 * ADT_BLOCK + ADT_BLOCK, &tmap_kv, full_bar(s), 0, rv);
      }
      if (!ok) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) { } }
    }
    __syncwarp();
  } else {
    const int t = lane & 15, half = lane >> 4;
    const int r_k = 2 * t + half;                       // half-row of this lane's K data inside the block
    bool ok = true;
    for (int i = warp; i < npages && ok; i += 4) {
      const int s = i % ADT_STAGES;
      const uint32_t ph = (i / ADT_STAGES) & 1u;
      if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (4 << 8)), p.limit_ns)) { ok = false; break; }
      const uint8_t* kblk = smem + s * 2 * ADT_BLOCK;
      const uint8_t* vblk = kblk + ADT_BLOCK;
      // ---- scores ----
      float dot[G];
#pragma unroll
      for (int g = 0; g < G; ++g) dot[g] = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kblk + r_k * 128 + ((u ^ (r_k & 7)) << 4));
        float kf[8];
        unpack8(raw, kf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(q_s + g * ADT_D + half * 64 + u * 8);
          const float4 qb = *reinterpret_cast<const float4*>(q_s + g * ADT_D + half * 64 + u * 8 + 4);
          dot[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
        }
      }
      const int tok = (pg0 + i) * ADT_PS + t;
      float pr[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sc = dot[g] + __shfl_xor_sync(0xffffffffu, dot[g], 16);
        if (tok >= len) sc = -INFINITY;
        float mx = sc;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run[g], mx);
        const float e = (m_new == -INFINITY) ? 0.f : exp2f(sc - m_new);
        float sum = e;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float alpha = (m_run[g] == -INFINITY) ? 0.f : exp2f(m_run[g] - m_new);
        l_run[g] = l_run[g] * alpha + sum;
        m_run[g] = m_new;
        acc[g][0] *= alpha; acc[g][1] *= alpha; acc[g][2] *= alpha; acc[g][3] *= alpha;
        pr[g] = e;                                       // lanes t and t+16 both hold p[t]
      }
      // ---- P.V: this lane owns output dims 4*lane .. 4*lane+3 ----
      const int vhalf = lane >> 4, vunit = (lane & 15) >> 1, vsub = (lane & 1) * 8;
#pragma unroll
      for (int tt = 0; tt < ADT_PS; ++tt) {
        const int r_v = 2 * tt + vhalf;
        const uint2 raw = *reinterpret_cast<const uint2*>(vblk + r_v * 128 + ((vunit ^ (r_v & 7)) << 4) + vsub);
        const float v0 = __uint_as_float(raw.x << 16), v1 = __uint_as_float(raw.x & 0xffff0000u);
        const float v2 = __uint_as_float(raw.y << 16), v3 = __uint_as_float(raw.y & 0xffff0000u);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pv = __shfl_sync(0xffffffffu, pr[g], tt);
          acc[g][0] += pv * v0; acc[g][1] += pv * v1; acc[g][2] += pv * v2; acc[g][3] += pv * v3;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));
    }
    // ---- publish this warp's state for the CTA merge ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
      *reinterpret_cast<float4*>(mg_acc + (warp * G + g) * ADT_D + 4 * lane) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      if (lane == 0) { mg_ml[(warp * G + g) * 2] = m_run[g]; mg_ml[(warp * G + g) * 2 + 1] = l_run[g]; }
    }
  }
  __syncthreads();

  // ---- merge the four warps: thread <-> (g, d) ----
  for (int i = tid; i < G * ADT_D; i += ADT_THREADS) {
    const int g = i / ADT_D, d = i % ADT_D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mg_ml[(w * G + g) * 2]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mg_ml[(w * G + g) * 2];
      const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      l += sc * mg_ml[(w * G + g) * 2 + 1];
      o += sc * mg_acc[(w * G + g) * ADT_D + d];
    }
    const size_t hrow = static_cast<size_t>(b) * p.hq + kvh * G + g;
    if (p.splits == 1) {
      p.out[hrow * ADT_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
    } else {
      p.part_acc[(hrow * p.splits + split) * ADT_D + d] = o;
      if (d == 0) { p.part_ml[(hrow * p.splits + split) * 2] = m; p.part_ml[(hrow * p.splits + split) * 2 + 1] = l; }
    }
  }
  if (p.splits == 1) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned* ctr = p.counters + static_cast<size_t>(b) * p.hkv + kvh;
    const unsigned old = atomicAdd(ctr, 1u);
    *last_flag = (old == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
    if (*last_flag) *ctr = 0;
  }
  __syncthreads();
  if (!*last_flag) return;
  __threadfence();
  for (int i = tid; i < G * ADT_D; i += ADT_THREADS) {
    const int g = i / ADT_D, d = i % ADT_D;
    const size_t base = (static_cast<size_t>(b) * p.hq + kvh * G + g) * p.splits;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) m = fmaxf(m, __ldcg(p.part_ml + (base + s) * 2));
    float l = 0.f, o = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = __ldcg(p.part_ml + (base + s) * 2);
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      l += w * __ldcg(p.part_ml + (base + s) * 2 + 1);
      o += w * __ldcg(p.part_acc + (base + s) * ADT_D + d);
    }
    p.out[(static_cast<size_t>(b) * p.hq + kvh * G + g) * ADT_D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int G>
static int launch_adt(const CUtensorMap& tm, const DecodeTmaParams& p, dim3 grid, cudaStream_t stream) {
  constexpr int SMEM = ADT_STAGES * 2 * ADT_BLOCK + (G * ADT_D + 4 * G * ADT_D + 4 * G * 2 + 2) * 4 + 2 * ADT_STAGES * 8 + 64 + ADT_MAX_PAGES * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(attn_decode_tma_kernel<G>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  launch_ex(attn_decode_tma_kernel<G>, dim3(grid), dim3(ADT_THREADS), SMEM, stream, 0, tm, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

}  // namespace b200

using namespace b200;

// Same contract as b200_attn_decode, for page_size 16 and G = hq/hkv in {1,2,4,8}; num_pages sizes the tensor map.
extern "C" int b200_attn_decode_tma(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                                    void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                                    int max_pages, int splits, float scale, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (page_size != ADT_PS || (hq % hkv)) return -3;
  const int G = hq / hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return -3;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!scratch || !counters)) return -1;
  if (reinterpret_cast<uintptr_t>(cache) & 127) return -2;
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) return -11;
    fn = reinterpret_cast<EncodeTiledFn2>(ptr);
  }
  // the cache as [half-rows][64 bf16]: one token row of 128 dims = two consecutive 128-byte half-rows
  CUtensorMap tm;
  cuuint64_t dims[2] = {64, static_cast<cuuint64_t>(num_pages) * 2 * hkv * ADT_PS * 2};
  cuuint64_t strides[1] = {128};
  cuuint32_t box[2] = {64, ADT_PS * 2};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -12;
  DecodeTmaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.page_table = page_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_acc = scratch;
  p.part_ml = scratch ? scratch + static_cast<size_t>(B) * hq * splits * ADT_D : nullptr;
  p.counters = counters; p.hq = hq; p.hkv = hkv; p.max_pages = max_pages; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.limit_ns = 2000000000ull;
  dim3 grid(hkv, B, splits);
  switch (G) {
    case 1: return launch_adt<1>(tm, p, grid, stream);
    case 2: return launch_adt<2>(tm, p, grid, stream);
    case 4: return launch_adt<4>(tm, p, grid, stream);
    default: return launch_adt<8>(tm, p, grid, stream);
  }
}
