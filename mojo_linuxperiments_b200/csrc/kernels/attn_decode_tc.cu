// Paged-KV decode attention on the tcgen05 tensor cores (page size 16, head dim 128, bf16, fp32 accumulate).
//
// The CUDA-core form (attn_decode_tma.cu) is bound by its instruction count (two FMAs per byte of KV for a group of
// four query heads); here the dot products are MMAs and the kernel is a pure HBM stream.
//
// Grid (kv_head, sequence, split), 192 threads, two CTAs per SM.  A CTA owns up to ADC_NB blocks of 128 cached tokens.
//   warp 0      TMA producer: for each block the 8 pages of K, then (second pass) the 8 pages of V, each page as two
//               [16 tokens x 64 dims] boxes (3-D tensor map over the cache, 128-byte swizzle) into a two-stage ring of
//               32 KiB tiles laid out exactly as the MMA wants them ([128 tokens][64 dims] x 2 halves)
//   warp 1      MMA issuer.  S^T[128 tokens x 16] = K_tile (A, K-major) . Q^T (B: the G query heads of this KV head
//               padded to 16 rows), one TMEM column block per token block; after the softmax warps have written
//               P (bf16, [16 heads x 128 tokens], K-major) O^T[128 dims x 16] += V_tile^T (A, MN-major) . P
//   warps 2..5  softmax, thread <-> token (TMEM lane): scores of all blocks stay in registers, the maximum and the
//               sum per head are combined across the four warps through shared memory, so P is computed once with
//               the final maximum and the PV accumulation needs no rescaling; then thread <-> output dim for O^T.
// Pages beyond the end of the sequence are replaced by the sequence's last valid page (an L2 hit) and masked.
// With several splits each CTA writes (o, m, l) partials and the last one to finish merges them.  All waits bounded.
// No counterpart in the reference (it has no attention or any other model kernel).
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include "hadamard.cuh"
#include <cuda.h>
#include <cstdlib>

namespace b200 {

constexpr int ADC_THREADS = 192;
constexpr int ADC_NB = 4;                       // token blocks (of 128) per CTA
constexpr int ADC_NB_LONG = 9;                  // fused form without a merge zone: up to 1,152 cached tokens per CTA
constexpr int ADC_D = 128;
constexpr int ADC_HALF = 128 * 128;             // bytes: 128 tokens x 64 dims bf16
constexpr int ADC_TILE = 2 * ADC_HALF;          // 32 KiB
constexpr int ADC_NH = 16;                      // MMA N: query heads padded to 16
constexpr int ADC_P_TILE = ADC_NH * 128 * 2;    // 4 KiB: P of one block
constexpr int ADC_Q_TILE = ADC_NH * ADC_D * 2;  // 4 KiB
constexpr int ADC_TMEM_COLS = 128;              // S: ADC_NB x 16 columns, O: 16 columns at 64
constexpr int ADC_O_COL = 64;

// Fused form (attn_decode_tc_kernel<G, true>): the kernel takes the raw q | k | v projections of the new token instead of
// a rotated q, applies the optional per-head RMSNorm and the rotary embedding itself, appends k and v to the paged
// cache, attends to the new token from registers (the cached tokens still arrive by TMA), and can finish with the
// block-128 Hadamard rotation + per-token int8 quantisation of the attention output, i.e. the operand of o_proj.
struct DecodeFuse {
  const __nv_bfloat16* qkv;        // [B][(hq + 2 hkv) * 128] (row pitch ld_qkv elements)
  long long ld_qkv;
  const int* positions;            // [B] position of the new token (seq_lens[b] counts it: cached tokens = seq_lens[b] - 1)
  const float* cos_tab;            // [max_pos][64]
  const float* sin_tab;
  int max_pos;
  const __nv_bfloat16* q_norm_w;   // [128] or nullptr
  const __nv_bfloat16* k_norm_w;
  float eps;
  __nv_bfloat16* cache;            // same storage the tensor map reads
  int num_pages;
  int8_t* xq;                      // [B][hq * 128] int8 rows (pitch ldq) or nullptr: no quantising epilogue
  long long ldq;
  float* sx;                       // [B] per-token scales
  float* rot_scratch;              // [B][hq][128] rotated rows, used when a token's heads span several CTAs (hkv > 1)
  float* blk_amax;                 // [B][hkv]
  unsigned* seq_counters;          // [B], zero between launches
  // Constant bytes that the next kernel streams (the o-projection's weights): its CTAs cannot be resident while this
  // kernel fills the SMs, so this kernel's CTAs ask for one slice each to be brought into L2 while HBM has slack.
  const uint8_t* next_w;
  unsigned long long next_w_bytes;
};

struct DecodeTcParams {
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
  // 1: the splits of a (sequence, kv head) are one thread-block cluster (cluster dims 1 x 1 x splits) and their partials
  // meet in the shared memory of the cluster's first CTA, which merges them: no global scratch, no counter, no fence
  int cluster_merge;
  int early_tiles;     // fused form: request the first two K / V tiles before the dependency wait
  DecodeFuse f;
};

constexpr int ADC_ZONE_ROW = ADC_D + 2;            // one partial row in the merge zone: 128 values, max, sum
constexpr int ADC_ZONE_MAX_SPLITS = 8;             // portable cluster size
constexpr int ADC_ZONE_MAX_G = 4;                  // the zone is sized for groups of up to four query heads

__device__ __forceinline__ void unpack8_bf16(const uint4& raw, float (&o)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
__device__ __forceinline__ uint4 pack8_bf16(const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&b);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

// One head (128 values) handled by 8 consecutive lanes: lane c holds elements 8c..8c+7 (lo) and 64+8c..64+8c+7 (hi).
// Optional RMSNorm over the head, then the rotate-half rotary embedding with the pairs (i, i + 64).  All 32 lanes of the
// warp must call this together (the reduction shuffles inside groups of 8 lanes).
__device__ __forceinline__ void head_norm_rope(float (&lo)[8], float (&hi)[8], const __nv_bfloat16* nw, float eps, int c,
                                               const float (&cs)[8], const float (&sn)[8]) {
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    const float r = rsqrtf(ss * (1.f / 128.f) + eps);
    float wl[8], wh[8];
    unpack8_bf16(*reinterpret_cast<const uint4*>(nw + 8 * c), wl);
    unpack8_bf16(*reinterpret_cast<const uint4*>(nw + 64 + 8 * c), wh);
#pragma unroll
    for (int j = 0; j < 8; ++j) { lo[j] *= r * wl[j]; hi[j] *= r * wh[j]; }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float a = lo[j], b = hi[j];
    lo[j] = a * cs[j] - b * sn[j];
    hi[j] = b * cs[j] + a * sn[j];
  }
}

template <int G, bool FUSED, int NB>
__global__ void __launch_bounds__(ADC_THREADS, 2)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmap_kv, const DecodeTcParams p) {
  // score columns of the NB blocks, then 16 columns of output; allocations are powers of two
  constexpr int O_COL_K = NB * ADC_NH;
  constexpr int TMEM_COLS_K = (NB * ADC_NH + ADC_NH <= 128) ? 128 : 256;
  pdl_launch_dependents();
  B200_TRACE_INIT();
  if (threadIdx.x == 0) B200_TRACE(TK_ATTN_DECODE, TP_START);
  // Fused form: only the new token's q / k / v come from the previous kernel.  Lengths, positions and page table were
  // settled before this step began and the cached tokens were written by earlier steps, so the first two K / V tiles are
  // requested before the dependency wait (below) and stream in while the previous kernel finishes.
  if constexpr (!FUSED) {
    pdl_wait();
    if (threadIdx.x == 0) B200_TRACE(TK_ATTN_DECODE, TP_DEPS);
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [ring 2 x 32K][P NB x 4K][Q 4K][exchange floats][barriers]
  uint8_t* pP = smem + 2 * ADC_TILE;
  uint8_t* pQ = pP + NB * ADC_P_TILE;
  float* xch = reinterpret_cast<float*>(pQ + ADC_Q_TILE);          // [2][4 warps][16]: per-warp max, then sum
  float* ml_s = xch + 128;                                         // [16][2]: final (m, l) per head
  uint64_t* bars = reinterpret_cast<uint64_t*>(ml_s + 32);
  enum { B_FULL = 0, B_EMPTY = 2, B_SFULL = 4, B_PFULL = 4 + NB, B_OFULL = 4 + 2 * NB, B_XCH = 5 + 2 * NB, B_COUNT = 6 + 2 * NB };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  int* page_s = last_flag + 1;                     // [NB * 8] page ids of this CTA's blocks
  // fused form only: the finished (bf16-rounded) output rows of this CTA's heads, v and the scores of the new token
  float* row_s = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(page_s + NB * 8) + 15) & ~uintptr_t(15));   // [G][128]
  float* vnew_s = row_s + G * ADC_D;               // [128]
  float* snew_s = vnew_s + ADC_D;                  // [16]
  float* amax_s = snew_s + 16;                     // [8]
  float* zone = amax_s + 8;                        // cluster merge: [splits][G][ADC_ZONE_ROW] (G <= 4 only)
  const uint32_t sRing = smem_u32(smem);
  const uint32_t sP = smem_u32(pP), sQ = smem_u32(pQ);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int len_total = p.seq_lens[b];
  // fused: the new token is not read from the cache, so the TMA path covers one token less
  int len = FUSED ? len_total - 1 : len_total;
  const bool has_new = FUSED && split == p.splits - 1 && len_total >= 1;
  if (len > p.max_pages * 16) {            // the page-table row cannot describe more tokens than this
    if (tid == 0 && p.status) atomicCAS(p.status, 0, (int)ST_BAD_ARGUMENT | (5 << 8));
    len = p.max_pages * 16;
  }
  if (len < 0) len = 0;
  const int total_pages = (len + 15) >> 4;
  const int total_blocks = (len + 127) >> 7;
  const int per = (total_blocks + p.splits - 1) / p.splits;
  const int blk0 = split * per;
  int nb = min(total_blocks, blk0 + per) - blk0;
  if (nb < 0) nb = 0;
  if (nb > NB) {                       // the host sized `splits` for a shorter maximum length
    if (tid == 0 && p.status) atomicCAS(p.status, 0, (int)ST_BAD_ARGUMENT | (5 << 8));
    nb = NB;
  }
  const int* pt = p.page_table + static_cast<size_t>(b) * p.max_pages;
  const uint64_t limit = p.limit_ns;

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), (i >= B_PFULL && i < B_PFULL + NB) || i == B_XCH ? 4 : 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS_K); tmem_relinquish(); }
  // Q^T operand: rows = heads, K-major, two 64-dim halves of [16 rows x 128 B], 128-byte swizzle.  Only the first G
  // rows of Q^T and of the P tiles are ever written: row n of a B operand feeds column n of the accumulator alone,
  // and the columns >= G of S^T and O^T are never read, so whatever the other rows hold is harmless.
  // Page ids are fetched once, in parallel, so the producer never waits on a global load between two TMA issues;
  // pages past the end of the sequence are replaced by its last page (already in L2) and masked in the softmax.
  if (tid < NB * 8 && total_pages > 0) page_s[tid] = pt[min(blk0 * 8 + tid, total_pages - 1)];
  // tile i of this CTA's stream (K blocks first, then V blocks) into ring stage i & 1
  auto issue_tile = [&](int i) {
    const int st = i & 1;
    const int blk = i < nb ? i : i - nb;
    const int kv = i < nb ? 0 : 1;
    mbar_expect_tx(bar(B_FULL + st), ADC_TILE);
    const uint32_t dst = sRing + st * ADC_TILE;
    const uint64_t pol = policy_evict_first();               // cached tokens are read once per step: they should not push
                                                             // the next kernels' weights out of L2
#pragma unroll 1
    for (int j = 0; j < 8; ++j) {
      const int page = page_s[blk * 8 + j];
      const int row = ((page * 2 + kv) * p.hkv + kvh) * 16;  // first token row of the block in the [rows][2][64] view
      tma_load_3d_hint(dst + j * 2048, &tmap_kv, bar(B_FULL + st), 0, 0, row, pol);
      tma_load_3d_hint(dst + ADC_HALF + j * 2048, &tmap_kv, bar(B_FULL + st), 0, 1, row, pol);
    }
  };
  if constexpr (!FUSED) {
    for (int i = tid; i < G * 16; i += ADC_THREADS) {
      const int g = i >> 4, c = i & 15;
      const uint4 v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(b) * p.hq + kvh * G + g) * ADC_D + c * 8);
      *reinterpret_cast<uint4*>(pQ + (c >> 3) * 2048 + (g >> 3) * 1024 + (g & 7) * 128 + (((c & 7) ^ (g & 7)) << 4)) = v;
    }
  } else {
    __syncthreads();                                 // barriers initialised, page ids in shared memory
    if (tid == 0 && nb > 0 && p.early_tiles) {
      prefetch_tmap(&tmap_kv);
      for (int i = 0; i < 2; ++i) issue_tile(i);     // first use of both ring stages: nothing to wait for (nb >= 1: 2 nb >= 2)
    }
    if (tid == 32 && p.f.next_w) {
      const unsigned long long ctas = static_cast<unsigned long long>(gridDim.x) * gridDim.y * gridDim.z;
      const unsigned long long me = blockIdx.x + gridDim.x * (blockIdx.y + static_cast<unsigned long long>(gridDim.y) * blockIdx.z);
      const unsigned long long chunk = ((p.f.next_w_bytes + ctas - 1) / ctas + 15) & ~15ull;
      const unsigned long long lo = me * chunk;
      if (lo < p.f.next_w_bytes) {
        const unsigned long long n = min(chunk, p.f.next_w_bytes - lo) & ~15ull;
        if (n) bulk_prefetch_l2(p.f.next_w + lo, static_cast<uint32_t>(n));
      }
    }
    pdl_wait();
    if (tid == 0) B200_TRACE(TK_ATTN_DECODE, TP_DEPS);
    // ---- rotate q (every CTA), and in the CTA that owns the new token: rotate k, append k and v to the cache, score ----
    const int pos = p.f.positions[b];
    const bool pos_ok = pos >= 0 && pos < p.f.max_pos;
    const __nv_bfloat16* row = p.f.qkv + static_cast<size_t>(b) * p.f.ld_qkv;
    // where the new token goes: refuse (status word) a position outside the tables or the pages of the sequence
    size_t cache_row = 0;
    bool store_ok = has_new && pos_ok && (pos >> 4) < p.max_pages;
    if (store_ok) {
      const int page = pt[pos >> 4];
      store_ok = page >= 0 && page < p.f.num_pages;
      cache_row = (static_cast<size_t>(page) * 2 * p.hkv + kvh) * 16 + (pos & 15);      // K row; the V row is hkv * 16 rows further
    }
    if (has_new && !store_ok && tid == 0 && p.status) atomicCAS(p.status, 0, (int)ST_BAD_ARGUMENT | (5 << 8));
    if (warp < (G * 8 + 31) / 32) {
      const bool act = tid < G * 8;
      const int g = act ? (tid >> 3) : 0, c = tid & 7;
      float cs[8], sn[8];
      if (pos_ok) {
        const float4 c0 = *reinterpret_cast<const float4*>(p.f.cos_tab + static_cast<size_t>(pos) * 64 + 8 * c);
        const float4 c1 = *reinterpret_cast<const float4*>(p.f.cos_tab + static_cast<size_t>(pos) * 64 + 8 * c + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(p.f.sin_tab + static_cast<size_t>(pos) * 64 + 8 * c);
        const float4 s1 = *reinterpret_cast<const float4*>(p.f.sin_tab + static_cast<size_t>(pos) * 64 + 8 * c + 4);
        cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { cs[j] = 1.f; sn[j] = 0.f; }
      }
      const __nv_bfloat16* qh = row + static_cast<size_t>(kvh * G + g) * ADC_D;
      float qlo[8], qhi[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(qh + 8 * c), qlo);
      unpack8_bf16(*reinterpret_cast<const uint4*>(qh + 64 + 8 * c), qhi);
      head_norm_rope(qlo, qhi, p.f.q_norm_w, p.f.eps, c, cs, sn);
      const uint4 qa = pack8_bf16(qlo), qb = pack8_bf16(qhi);
      if (act) {
        *reinterpret_cast<uint4*>(pQ + (g >> 3) * 1024 + (g & 7) * 128 + ((c ^ (g & 7)) << 4)) = qa;            // chunk c
        *reinterpret_cast<uint4*>(pQ + 2048 + (g >> 3) * 1024 + (g & 7) * 128 + ((c ^ (g & 7)) << 4)) = qb;     // chunk c + 8
      }
      if (has_new) {
        // every group of 8 lanes rotates the same k head; group 0 stores it
        const __nv_bfloat16* kh = row + static_cast<size_t>(p.hq + kvh) * ADC_D;
        float klo[8], khi[8];
        unpack8_bf16(*reinterpret_cast<const uint4*>(kh + 8 * c), klo);
        unpack8_bf16(*reinterpret_cast<const uint4*>(kh + 64 + 8 * c), khi);
        head_norm_rope(klo, khi, p.f.k_norm_w, p.f.eps, c, cs, sn);
        const uint4 ka = pack8_bf16(klo), kb = pack8_bf16(khi);
        if (act && g == 0 && store_ok) {
          __nv_bfloat16* dst = p.f.cache + cache_row * ADC_D;
          *reinterpret_cast<uint4*>(dst + 8 * c) = ka;
          *reinterpret_cast<uint4*>(dst + 64 + 8 * c) = kb;
        }
        // the score the tensor core would have produced: bf16 operands, fp32 sum
        float qr0[8], qr1[8], kr0[8], kr1[8];
        unpack8_bf16(qa, qr0); unpack8_bf16(qb, qr1); unpack8_bf16(ka, kr0); unpack8_bf16(kb, kr1);
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += qr0[j] * kr0[j] + qr1[j] * kr1[j];
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        if (act && c == 0) snew_s[g] = dot * p.scale_log2;
      }
    }
    if (has_new && tid >= 64 && tid < 80) {
      const int vc = tid - 64;
      const uint4 vv = *reinterpret_cast<const uint4*>(row + static_cast<size_t>(p.hq + p.hkv + kvh) * ADC_D + 8 * vc);
      float vf[8];
      unpack8_bf16(vv, vf);
#pragma unroll
      for (int j = 0; j < 8; ++j) vnew_s[8 * vc + j] = vf[j];
      if (store_ok) *reinterpret_cast<uint4*>(p.f.cache + (cache_row + static_cast<size_t>(p.hkv) * 16) * ADC_D + 8 * vc) = vv;
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool cmerge = p.cluster_merge != 0;
  if (cmerge) cluster_arrive_relaxed();          // "this CTA runs": waited for before the first store into a peer's zone

  if (warp == 0) {
    if (lane == 0 && nb > 0) {
      const bool early = FUSED && p.early_tiles;
      if (!early) prefetch_tmap(&tmap_kv);
      bool ok = true;
      for (int i = early ? 2 : 0; i < 2 * nb && ok; ++i) {            // fused: tiles 0 and 1 are already on their way
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1u;
        if (!mbar_wait(bar(B_EMPTY + st), ph ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (5 << 8)), limit)) { ok = false; break; }
        issue_tile(i);
      }
      if (!ok) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) { } }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && nb > 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(128, ADC_NH, 0, 0);
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, ADC_NH, 1, 0);      // A (= V^T) is MN-major
      bool ok = true;
      for (int i = 0; i < nb && ok; ++i) {
        const int st = i & 1;
        if (!mbar_wait(bar(B_FULL + st), (i >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (5 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + i * ADC_NH;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a = umma_desc_k_sw128(sRing + st * ADC_TILE + (kk >> 2) * ADC_HALF) + 2ull * (kk & 3);
          const uint64_t bd = umma_desc_k_sw128(sQ + (kk >> 2) * 2048) + 2ull * (kk & 3);
          umma_f16_ss(d, a, bd, IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(B_EMPTY + st));
        umma_commit(bar(B_SFULL + i));
      }
      for (int blk = 0; blk < nb && ok; ++blk) {
        const int i = nb + blk;
        const int st = i & 1;
        if (!mbar_wait(bar(B_PFULL + blk), 0, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (5 << 8)), limit)) { ok = false; break; }
        if (!mbar_wait(bar(B_FULL + st), (i >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (5 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + O_COL_K;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a = umma_desc_mn_sw128(sRing + st * ADC_TILE + kk * 2048, ADC_HALF, 1024);
          const uint64_t bd = umma_desc_k_sw128(sP + blk * ADC_P_TILE + (kk >> 2) * 2048) + 2ull * (kk & 3);
          umma_f16_ss(d, a, bd, IDESC_PV, (blk > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(B_EMPTY + st));
        if (blk == nb - 1) umma_commit(bar(B_OFULL));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ softmax / output warps ------------------------------
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                    // token inside a block, later output dim: the TMEM lane
    const int wi = warp - 2;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    float s[NB][G];
    float mx[G];
#pragma unroll
    for (int g = 0; g < G; ++g) mx[g] = -INFINITY;
    bool ok = nb > 0;
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) {
      if (blk < nb && ok) {
        if (!mbar_wait(bar(B_SFULL + blk), 0, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (5 << 8)), limit)) { ok = false; }
        else {
          tc_fence_after();
          uint32_t v[16];
          tmem_ld_x16(t_lane + blk * ADC_NH, v);
          tmem_ld_wait();
          const bool valid = (blk0 + blk) * 128 + r < len;
#pragma unroll
          for (int g = 0; g < G; ++g) {
            s[blk][g] = valid ? __uint_as_float(v[g]) * p.scale_log2 : -INFINITY;
            mx[g] = fmaxf(mx[g], s[blk][g]);
          }
        }
      } else {
#pragma unroll
        for (int g = 0; g < G; ++g) s[blk][g] = -INFINITY;
      }
    }
    if (tid == 64) B200_TRACE(TK_ATTN_DECODE, 2);           // all scores of this CTA are in registers
    if constexpr (FUSED) {
      if (has_new) {
#pragma unroll
        for (int g = 0; g < G; ++g) mx[g] = fmaxf(mx[g], snew_s[g]);
      }
    }
    // ---- maximum per head over the CTA's tokens: warp shuffle, then the four warps through shared memory ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xffffffffu, mx[g], o));
    }
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) xch[wi * 16 + g] = mx[g];
      mbar_arrive(bar(B_XCH));
    }
    if (ok && !mbar_wait(bar(B_XCH), 0, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (5 << 8)), limit)) ok = false;
    if (tid == 64) B200_TRACE(TK_ATTN_DECODE, 3);
    float m[G], sum[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = fmaxf(fmaxf(xch[g], xch[16 + g]), fmaxf(xch[32 + g], xch[48 + g]));
      sum[g] = 0.f;
    }
    // ---- probabilities with the final maximum -> bf16 -> P tiles (K-major rows = heads, swizzled) ----
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) {
      if (blk < nb && ok) {
        uint8_t* pt_blk = pP + blk * ADC_P_TILE + (r >> 6) * 2048;
        const int c = (r & 63) >> 3, e = (r & 7) * 2;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pr = (m[g] == -INFINITY) ? 0.f : exp2f(s[blk][g] - m[g]);
          const __nv_bfloat16 pb = __float2bfloat16(pr);
          sum[g] += __bfloat162float(pb);                 // what the MMA will actually see
          *reinterpret_cast<__nv_bfloat16*>(pt_blk + (g >> 3) * 1024 + (g & 7) * 128 + ((c ^ (g & 7)) << 4) + e) = pb;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_PFULL + blk));
      }
    }
    // ---- sum per head ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum[g] += __shfl_xor_sync(0xffffffffu, sum[g], o);
    }
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) xch[64 + wi * 16 + g] = sum[g];
      mbar_arrive(bar(B_XCH));
    }
    if (ok && !mbar_wait(bar(B_XCH), 1, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (5 << 8)), limit)) ok = false;
    float l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) l[g] = xch[64 + g] + xch[80 + g] + xch[96 + g] + xch[112 + g];
    // ---- output: thread <-> dim ----
    float o[G];
#pragma unroll
    for (int g = 0; g < G; ++g) o[g] = 0.f;
    if (nb > 0 && ok) {
      if (!mbar_wait(bar(B_OFULL), 0, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (5 << 8)), limit)) ok = false;
      else {
        tc_fence_after();
        uint32_t v[16];
        tmem_ld_x16(t_lane + O_COL_K, v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < G; ++g) o[g] = __uint_as_float(v[g]);
      }
    }
    if (tid == 64) B200_TRACE(TK_ATTN_DECODE, 5);           // P.V accumulator read back
    if (nb == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; }
    }
    if constexpr (FUSED) {
      if (has_new) {
        // the new token joins from registers: its probability with the final maximum, its value row from shared memory
        const float vr = vnew_s[r];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          if (nb == 0 || !ok) { m[g] = snew_s[g]; l[g] = 1.f; o[g] = vr; }
          else {
            const float pn = round_bf16(exp2f(snew_s[g] - m[g]));
            l[g] += pn;
            o[g] += pn * vr;
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const size_t hrow = static_cast<size_t>(b) * p.hq + kvh * G + g;
      if (p.splits == 1) {
        const __nv_bfloat16 ob = __float2bfloat16(l[g] > 0.f ? o[g] / l[g] : 0.f);
        if (p.out) p.out[hrow * ADC_D + r] = ob;
        if constexpr (FUSED) row_s[g * ADC_D + r] = __bfloat162float(ob);
      } else if (!cmerge) {
        p.part_acc[(hrow * p.splits + split) * ADC_D + r] = o[g];
        if (r == 0) { p.part_ml[(hrow * p.splits + split) * 2] = m[g]; p.part_ml[(hrow * p.splits + split) * 2 + 1] = l[g]; }
      }
    }
    if (cmerge && p.splits > 1) {
      // partial rows go straight into the shared memory of the cluster's first CTA
      cluster_wait_acquire();
      const uint32_t z0 = mapa_shared(smem_u32(zone), 0u);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint32_t zr = z0 + 4u * static_cast<uint32_t>((split * G + g) * ADC_ZONE_ROW);
        st_shared_cluster_u32(zr + 4u * r, __float_as_uint(o[g]));
        if (r == 0) { st_shared_cluster_u32(zr + 4u * ADC_D, __float_as_uint(m[g])); st_shared_cluster_u32(zr + 4u * (ADC_D + 1), __float_as_uint(l[g])); }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS_K); }
  if (tid == 0) B200_TRACE(TK_ATTN_DECODE, 6);
  if (p.splits == 1 && !(FUSED && p.f.xq)) { B200_TRACE_FLUSH(TK_ATTN_DECODE); return; }

  if (p.splits > 1 && cmerge) {
    // ---- cluster merge: every partial has landed in the first CTA's zone once the cluster barrier completes ----
    if (warp < 2) cluster_wait_acquire();            // the two service warps still owe the wait of the start-up arrive
    cluster_sync_all();
    if (split != 0) { B200_TRACE_FLUSH(TK_ATTN_DECODE); return; }
    if (tid == 0) B200_TRACE(TK_ATTN_DECODE, 7);
    for (int i = tid; i < G * ADC_D; i += ADC_THREADS) {
      const int g = i / ADC_D, d = i % ADC_D;
      float m = -INFINITY, l = 0.f, o = 0.f;
      for (int sI = 0; sI < p.splits; ++sI) m = fmaxf(m, zone[(sI * G + g) * ADC_ZONE_ROW + ADC_D]);
      for (int sI = 0; sI < p.splits; ++sI) {
        const float* zr = zone + (sI * G + g) * ADC_ZONE_ROW;
        const float w = (zr[ADC_D] == -INFINITY) ? 0.f : exp2f(zr[ADC_D] - m);
        l += w * zr[ADC_D + 1];
        o += w * zr[d];
      }
      const __nv_bfloat16 ob = __float2bfloat16(l > 0.f ? o / l : 0.f);
      if (p.out) p.out[(static_cast<size_t>(b) * p.hq + kvh * G + g) * ADC_D + d] = ob;
      if constexpr (FUSED) row_s[i] = __bfloat162float(ob);
    }
    if (tid == 0) B200_TRACE(TK_ATTN_DECODE, TP_EXIT);
  } else if (p.splits > 1) {
    // ---- the last CTA of this (sequence, kv head) merges the splits ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      unsigned* ctr = p.counters + static_cast<size_t>(b) * p.hkv + kvh;
      const unsigned old = atomicAdd(ctr, 1u);
      *last_flag = (old == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
      if (*last_flag) *ctr = 0;
    }
    __syncthreads();
    if (!*last_flag) { B200_TRACE_FLUSH(TK_ATTN_DECODE); return; }
    if (tid == 0) B200_TRACE(TK_ATTN_DECODE, 7);
    __threadfence();
    for (int i = tid; i < G * ADC_D; i += ADC_THREADS) {
      const int g = i / ADC_D, d = i % ADC_D;
      const size_t base = (static_cast<size_t>(b) * p.hq + kvh * G + g) * p.splits;
      float m = -INFINITY, l = 0.f, o = 0.f;
      if (p.splits <= 16) {
        // all partials are requested at once: the merge is a chain of L2 round trips otherwise
        float ms[16], ls[16], os[16];
#pragma unroll
        for (int sI = 0; sI < 16; ++sI) {
          ms[sI] = -INFINITY; ls[sI] = 0.f; os[sI] = 0.f;
          if (sI < p.splits) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (base + sI) * 2));
            ms[sI] = ml.x; ls[sI] = ml.y;
            os[sI] = __ldcg(p.part_acc + (base + sI) * ADC_D + d);
          }
        }
#pragma unroll
        for (int sI = 0; sI < 16; ++sI) m = fmaxf(m, ms[sI]);
#pragma unroll
        for (int sI = 0; sI < 16; ++sI) {
          const float w = (ms[sI] == -INFINITY) ? 0.f : exp2f(ms[sI] - m);
          l += w * ls[sI];
          o += w * os[sI];
        }
      } else {
        for (int sI = 0; sI < p.splits; ++sI) m = fmaxf(m, __ldcg(p.part_ml + (base + sI) * 2));
        for (int sI = 0; sI < p.splits; ++sI) {
          const float ms = __ldcg(p.part_ml + (base + sI) * 2);
          const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
          l += w * __ldcg(p.part_ml + (base + sI) * 2 + 1);
          o += w * __ldcg(p.part_acc + (base + sI) * ADC_D + d);
        }
      }
      const __nv_bfloat16 ob = __float2bfloat16(l > 0.f ? o / l : 0.f);
      if (p.out) p.out[(static_cast<size_t>(b) * p.hq + kvh * G + g) * ADC_D + d] = ob;
      if constexpr (FUSED) row_s[i] = __bfloat162float(ob);
    }
    if (tid == 0) B200_TRACE(TK_ATTN_DECODE, TP_EXIT);
  }

  if constexpr (!FUSED) { B200_TRACE_FLUSH(TK_ATTN_DECODE); }
  if constexpr (FUSED) {
    if (!p.f.xq) { B200_TRACE_FLUSH(TK_ATTN_DECODE); return; }
    // ---- epilogue: block-128 Hadamard rotation (one head = one block) + per-token int8 of the output row ----
    __syncthreads();                                   // row_s of all heads of this CTA is complete
    constexpr int NW = ADC_THREADS / 32;
    constexpr int GI = (G + NW - 1) / NW;               // heads per warp in the rotation (16 heads on 6 warps: 3)
    float v[GI < 2 ? 2 : GI][4];
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < (GI < 2 ? 2 : GI); ++i) {
      const int g = warp + i * NW;
      if (g < G) {
        const float4 x = *reinterpret_cast<const float4*>(row_s + g * ADC_D + 4 * lane);
        v[i][0] = x.x; v[i][1] = x.y; v[i][2] = x.z; v[i][3] = x.w;
        fwht128_lane4(v[i], lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) am = fmaxf(am, fabsf(v[i][j]));
      }
    }
    am = warp_max(am);
    if (lane == 0) amax_s[warp] = am;
    if (p.hkv == 1) {
      __syncthreads();
      float row_amax = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) row_amax = fmaxf(row_amax, amax_s[w]);
      const float scale = quant_scale_from_amax(row_amax), inv = quant_inv_scale(scale);
#pragma unroll
      for (int i = 0; i < (GI < 2 ? 2 : GI); ++i) {
        const int g = warp + i * NW;
        if (g < G) *reinterpret_cast<uint32_t*>(p.f.xq + static_cast<size_t>(b) * p.f.ldq + g * ADC_D + 4 * lane) = quant_pack4(v[i], inv);
      }
      if (tid == 0) p.f.sx[b] = scale;
    } else {
      // the token's heads are spread over hkv CTAs: park the rotated rows, the last CTA to arrive quantises the token
#pragma unroll
      for (int i = 0; i < (GI < 2 ? 2 : GI); ++i) {
        const int g = warp + i * NW;
        if (g < G)
          *reinterpret_cast<float4*>(p.f.rot_scratch + (static_cast<size_t>(b) * p.hq + kvh * G + g) * ADC_D + 4 * lane) =
              make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        float blk = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) blk = fmaxf(blk, amax_s[w]);
        p.f.blk_amax[static_cast<size_t>(b) * p.hkv + kvh] = blk;
        __threadfence();
        const unsigned old = atomicAdd(p.f.seq_counters + b, 1u);
        *last_flag = (old == static_cast<unsigned>(p.hkv - 1)) ? 1 : 0;
        if (*last_flag) p.f.seq_counters[b] = 0;
      }
      __syncthreads();
      if (!*last_flag) { B200_TRACE_FLUSH(TK_ATTN_DECODE); return; }
      __threadfence();
      float row_amax = 0.f;
      for (int k = 0; k < p.hkv; ++k) row_amax = fmaxf(row_amax, __ldcg(p.f.blk_amax + static_cast<size_t>(b) * p.hkv + k));
      const float scale = quant_scale_from_amax(row_amax), inv = quant_inv_scale(scale);
      for (int h = warp; h < p.hq; h += NW) {
        const float4 x = __ldcg(reinterpret_cast<const float4*>(p.f.rot_scratch + (static_cast<size_t>(b) * p.hq + h) * ADC_D + 4 * lane));
        const float xv[4] = {x.x, x.y, x.z, x.w};
        *reinterpret_cast<uint32_t*>(p.f.xq + static_cast<size_t>(b) * p.f.ldq + h * ADC_D + 4 * lane) = quant_pack4(xv, inv);
      }
      if (tid == 0) p.f.sx[b] = scale;
    }
    if (tid == 0) B200_TRACE(TK_ATTN_DECODE, 62);
    B200_TRACE_FLUSH(TK_ATTN_DECODE);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Persistent form: the grid is two CTAs per SM and every CTA walks the work items (kv_head, sequence, split) w =
// blockIdx.x, blockIdx.x + gridDim.x, ...  The three roles loop over the items independently, so the TMA producer runs
// ahead into the next item's K tiles while the softmax warps are still exchanging maxima or writing the output of the
// current one: the per-CTA set-up, the first-tile latency and the epilogue of the one-item kernel above are paid once
// per CTA instead of once per item, and there is no wave quantisation.  Extra hand-shakes: SFREE / OFREE tell the MMA
// warp that the softmax warps have copied the scores / the output out of TMEM, QFULL[2] double-buffers the Q^T
// operand (the softmax warps load the next item's queries while they wait for the current scores), page ids and
// sequence lengths are prefetched one and two items ahead.  Barriers that are not used by every item (an item of a
// short sequence may have fewer blocks, or none) keep their own use counters, which every role derives from the same
// sequence length.
// ------------------------------------------------------------------------------------------------------------------
struct ItemGeom { int kvh, b, split, len, total_pages, blk0, nb; };

__device__ __forceinline__ ItemGeom item_geom(int w, int len, const DecodeTcParams& p) {
  ItemGeom g;
  len = max(0, min(len, p.max_pages * 16));      // never index past the sequence's page-table row
  g.split = w % p.splits;
  const int rest = w / p.splits;
  g.kvh = rest % p.hkv;
  g.b = rest / p.hkv;
  g.len = len;
  g.total_pages = (len + 15) >> 4;
  const int total_blocks = (len + 127) >> 7;
  const int per = (total_blocks + p.splits - 1) / p.splits;
  g.blk0 = g.split * per;
  g.nb = min(max(min(total_blocks, g.blk0 + per) - g.blk0, 0), ADC_NB);
  return g;
}
__device__ __forceinline__ int item_seq(int w, const DecodeTcParams& p) { return w / (p.splits * p.hkv); }

template <int G>
__global__ void __launch_bounds__(ADC_THREADS, 2)
attn_decode_tcp_kernel(const __grid_constant__ CUtensorMap tmap_kv, const DecodeTcParams p, const int num_items) {
  pdl_launch_dependents();
  pdl_wait();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [ring 2 x 32K][P ADC_NB x 4K][Q 2 x 4K][exchange floats][barriers][flags][page ids 2 x 32]
  uint8_t* pP = smem + 2 * ADC_TILE;
  uint8_t* pQ = pP + ADC_NB * ADC_P_TILE;
  float* xch = reinterpret_cast<float*>(pQ + 2 * ADC_Q_TILE);
  uint64_t* bars = reinterpret_cast<uint64_t*>(xch + 64);
  enum { B_FULL = 0, B_EMPTY = 2, B_SFULL = 4, B_PFULL = 4 + ADC_NB, B_OFULL = 4 + 2 * ADC_NB, B_XCH = 5 + 2 * ADC_NB,
         B_SFREE = 6 + 2 * ADC_NB, B_OFREE = 8 + 2 * ADC_NB, B_QFULL = 10 + 2 * ADC_NB, B_COUNT = 12 + 2 * ADC_NB };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;
  int* page_s = const_cast<int*>(last_flag) + 1;   // [2][ADC_NB * 8]
  const uint32_t sRing = smem_u32(smem);
  const uint32_t sP = smem_u32(pP), sQ = smem_u32(pQ);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint64_t limit = p.limit_ns;
  const int stride = gridDim.x;
  const int w0 = blockIdx.x;

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) {
      const bool four = (i >= B_PFULL && i < B_PFULL + ADC_NB) || i == B_XCH || i >= B_SFREE;
      mbar_init(bar(i), four ? 4 : 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), ADC_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (whole warp: lanes prefetch page ids) ------------------------------
    prefetch_tmap(&tmap_kv);
    int len_cur = w0 < num_items ? p.seq_lens[item_seq(w0, p)] : 0;
    int len_nxt = w0 + stride < num_items ? p.seq_lens[item_seq(w0 + stride, p)] : 0;
    {
      const ItemGeom g = item_geom(w0, len_cur, p);
      if (w0 < num_items && g.total_pages > 0)
        page_s[lane] = p.page_table[static_cast<size_t>(g.b) * p.max_pages + min(g.blk0 * 8 + lane, g.total_pages - 1)];
    }
    __syncwarp();
    uint32_t t = 0;                                   // tiles issued so far: ring stage t & 1, use (t >> 1)
    bool ok = true;
    int it = 0;
    for (int w = w0; w < num_items && ok; w += stride, ++it) {
      const ItemGeom g = item_geom(w, len_cur, p);
      // page ids of the next item and the length of the one after it are requested now and consumed after this
      // item's tiles have been issued
      const int w1 = w + stride, w2 = w + 2 * stride;
      int pid_nxt = 0;
      ItemGeom g1 = g;
      if (w1 < num_items) {
        g1 = item_geom(w1, len_nxt, p);
        if (g1.total_pages > 0)
          pid_nxt = p.page_table[static_cast<size_t>(g1.b) * p.max_pages + min(g1.blk0 * 8 + lane, g1.total_pages - 1)];
      }
      const int len_nn = w2 < num_items ? p.seq_lens[item_seq(w2, p)] : 0;
      const int* pg = page_s + (it & 1) * (ADC_NB * 8);
      if (lane == 0) {
        for (int i = 0; i < 2 * g.nb && ok; ++i, ++t) {
          const int st = t & 1;
          const uint32_t ph = (t >> 1) & 1u;
          const int blk = i < g.nb ? i : i - g.nb;
          const int kv = i < g.nb ? 0 : 1;
          if (!mbar_wait(bar(B_EMPTY + st), ph ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (6 << 8)), limit)) { ok = false; break; }
          mbar_expect_tx(bar(B_FULL + st), ADC_TILE);
          const uint32_t dst = sRing + st * ADC_TILE;
#pragma unroll 1
          for (int j = 0; j < 8; ++j) {
            const int row = ((pg[blk * 8 + j] * 2 + kv) * p.hkv + g.kvh) * 16;
            tma_load_3d(dst + j * 2048, &tmap_kv, bar(B_FULL + st), 0, 0, row);
            tma_load_3d(dst + ADC_HALF + j * 2048, &tmap_kv, bar(B_FULL + st), 0, 1, row);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      t = __shfl_sync(0xffffffffu, t, 0);
      page_s[((it + 1) & 1) * (ADC_NB * 8) + lane] = pid_nxt;
      __syncwarp();
      len_cur = len_nxt;
      len_nxt = len_nn;
    }
    if (!ok && lane == 0) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) { } }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(128, ADC_NH, 0, 0);
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, ADC_NH, 1, 0);
      uint32_t t = 0, o_uses = 0;
      uint32_t blk_uses[ADC_NB];
#pragma unroll
      for (int i = 0; i < ADC_NB; ++i) blk_uses[i] = 0;
      int len_cur = w0 < num_items ? p.seq_lens[item_seq(w0, p)] : 0;
      bool ok = true;
      int it = 0;
      for (int w = w0; w < num_items && ok; w += stride, ++it) {
        const ItemGeom g = item_geom(w, len_cur, p);
        const int len_nxt = w + stride < num_items ? p.seq_lens[item_seq(w + stride, p)] : 0;
        const uint32_t sQb = sQ + (it & 1) * ADC_Q_TILE;
        if (!mbar_wait(bar(B_QFULL + (it & 1)), (it >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (6 << 8)), limit)) { ok = false; break; }
        // SFREE / OFREE alternate between two barriers: an item without blocks lets the softmax warps run one item
        // ahead, which must not complete the phase this warp is about to wait for
        if (it > 0 && !mbar_wait(bar(B_SFREE + ((it - 1) & 1)), ((it - 1) >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_EMPTY | (6 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int i = 0; i < g.nb && ok; ++i, ++t) {
          const int st = t & 1;
          if (!mbar_wait(bar(B_FULL + st), (t >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (6 << 8)), limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + i * ADC_NH;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a = umma_desc_k_sw128(sRing + st * ADC_TILE + (kk >> 2) * ADC_HALF) + 2ull * (kk & 3);
            const uint64_t bd = umma_desc_k_sw128(sQb + (kk >> 2) * 2048) + 2ull * (kk & 3);
            umma_f16_ss(d, a, bd, IDESC_S, kk > 0 ? 1u : 0u);
          }
          umma_commit(bar(B_EMPTY + st));
          umma_commit(bar(B_SFULL + i));
        }
        if (!ok) break;
        if (it > 0 && !mbar_wait(bar(B_OFREE + ((it - 1) & 1)), ((it - 1) >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_EMPTY | (6 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int blk = 0; blk < g.nb && ok; ++blk, ++t) {
          const int st = t & 1;
          if (!mbar_wait(bar(B_PFULL + blk), blk_uses[blk] & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (6 << 8)), limit)) { ok = false; break; }
          if (!mbar_wait(bar(B_FULL + st), (t >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (6 << 8)), limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + ADC_O_COL;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a = umma_desc_mn_sw128(sRing + st * ADC_TILE + kk * 2048, ADC_HALF, 1024);
            const uint64_t bd = umma_desc_k_sw128(sP + blk * ADC_P_TILE + (kk >> 2) * 2048) + 2ull * (kk & 3);
            umma_f16_ss(d, a, bd, IDESC_PV, (blk > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(bar(B_EMPTY + st));
          if (blk == g.nb - 1) umma_commit(bar(B_OFULL));
          ++blk_uses[blk];
        }
        if (ok && g.nb == 0) umma_commit(bar(B_OFULL));     // every item completes one OFULL phase: it paces the softmax warps
        ++o_uses;
        len_cur = len_nxt;
      }
      (void)o_uses;
    }
    __syncwarp();
  } else {
    // ------------------------------ softmax / output warps ------------------------------
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const int wi = warp - 2;
    const int st4 = tid - 64;                        // 0..127
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    uint32_t o_uses = 0, x_uses = 0;
    uint32_t blk_uses[ADC_NB];
#pragma unroll
    for (int i = 0; i < ADC_NB; ++i) blk_uses[i] = 0;
    int len_cur = w0 < num_items ? p.seq_lens[item_seq(w0, p)] : 0;
    auto load_q = [&](int w, int buf) {
      const int rest = w / p.splits;
      const int kvh = rest % p.hkv, b = rest / p.hkv;
      if (st4 < G * 16) {
        const int g = st4 >> 4, c = st4 & 15;
        const uint4 v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(b) * p.hq + kvh * G + g) * ADC_D + c * 8);
        *reinterpret_cast<uint4*>(pQ + buf * ADC_Q_TILE + (c >> 3) * 2048 + (g >> 3) * 1024 + (g & 7) * 128 + (((c & 7) ^ (g & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_QFULL + buf));
    };
    if (w0 < num_items) load_q(w0, 0);
    bool ok = true;
    int it = 0;
    for (int w = w0; w < num_items && ok; w += stride, ++it) {
      const ItemGeom gm = item_geom(w, len_cur, p);
      const int len_nxt = w + stride < num_items ? p.seq_lens[item_seq(w + stride, p)] : 0;
      if (w + stride < num_items) load_q(w + stride, (it + 1) & 1);
      const int nb = gm.nb;
      float s[ADC_NB][G];
      float mx[G];
#pragma unroll
      for (int g = 0; g < G; ++g) mx[g] = -INFINITY;
#pragma unroll
      for (int blk = 0; blk < ADC_NB; ++blk) {
        if (blk < nb && ok) {
          if (!mbar_wait(bar(B_SFULL + blk), blk_uses[blk] & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (6 << 8)), limit)) { ok = false; }
          else {
            tc_fence_after();
            uint32_t v[16];
            tmem_ld_x16(t_lane + blk * ADC_NH, v);
            tmem_ld_wait();
            const bool valid = (gm.blk0 + blk) * 128 + r < gm.len;
#pragma unroll
            for (int g = 0; g < G; ++g) {
              s[blk][g] = valid ? __uint_as_float(v[g]) * p.scale_log2 : -INFINITY;
              mx[g] = fmaxf(mx[g], s[blk][g]);
            }
          }
        } else {
#pragma unroll
          for (int g = 0; g < G; ++g) s[blk][g] = -INFINITY;
        }
      }
      // the scores are in registers: the MMA warp may overwrite the S columns with the next item's
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_SFREE + (it & 1)));
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xffffffffu, mx[g], o));
      }
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) xch[wi * 8 + g] = mx[g];
        mbar_arrive(bar(B_XCH));
      }
      if (ok && !mbar_wait(bar(B_XCH), x_uses & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (6 << 8)), limit)) ok = false;
      ++x_uses;
      float m[G], sum[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        m[g] = fmaxf(fmaxf(xch[g], xch[8 + g]), fmaxf(xch[16 + g], xch[24 + g]));
        sum[g] = 0.f;
      }
#pragma unroll
      for (int blk = 0; blk < ADC_NB; ++blk) {
        if (blk < nb && ok) {
          uint8_t* pt_blk = pP + blk * ADC_P_TILE + (r >> 6) * 2048;
          const int c = (r & 63) >> 3, e = (r & 7) * 2;
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pr = (m[g] == -INFINITY) ? 0.f : exp2f(s[blk][g] - m[g]);
            const __nv_bfloat16 pb = __float2bfloat16(pr);
            sum[g] += __bfloat162float(pb);
            *reinterpret_cast<__nv_bfloat16*>(pt_blk + (g >> 3) * 1024 + (g & 7) * 128 + ((c ^ (g & 7)) << 4) + e) = pb;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_PFULL + blk));
        }
        if (blk < nb) ++blk_uses[blk];
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum[g] += __shfl_xor_sync(0xffffffffu, sum[g], o);
      }
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) xch[32 + wi * 8 + g] = sum[g];
        mbar_arrive(bar(B_XCH));
      }
      if (ok && !mbar_wait(bar(B_XCH), x_uses & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (6 << 8)), limit)) ok = false;
      ++x_uses;
      float l[G];
#pragma unroll
      for (int g = 0; g < G; ++g) l[g] = xch[32 + g] + xch[40 + g] + xch[48 + g] + xch[56 + g];
      float o[G];
#pragma unroll
      for (int g = 0; g < G; ++g) o[g] = 0.f;
      if (ok) {
        if (!mbar_wait(bar(B_OFULL), o_uses & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (6 << 8)), limit)) ok = false;
        else if (nb > 0) {
          tc_fence_after();
          uint32_t v[16];
          tmem_ld_x16(t_lane + ADC_O_COL, v);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < G; ++g) o[g] = __uint_as_float(v[g]);
        }
      }
      ++o_uses;
      // the output is in registers: the MMA warp may start the next item's P.V
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_OFREE + (it & 1)));
      if (nb == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const size_t hrow = static_cast<size_t>(gm.b) * p.hq + gm.kvh * G + g;
        if (p.splits == 1) {
          p.out[hrow * ADC_D + r] = __float2bfloat16(l[g] > 0.f ? o[g] / l[g] : 0.f);
        } else {
          p.part_acc[(hrow * p.splits + gm.split) * ADC_D + r] = o[g];
          if (r == 0) { p.part_ml[(hrow * p.splits + gm.split) * 2] = m[g]; p.part_ml[(hrow * p.splits + gm.split) * 2 + 1] = l[g]; }
        }
      }
      if (p.splits > 1) {
        // ---- the last CTA to finish a (sequence, kv head) merges its splits; the four warps agree through XCH ----
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_XCH));
        if (ok && !mbar_wait(bar(B_XCH), x_uses & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (6 << 8)), limit)) ok = false;
        ++x_uses;
        if (st4 == 0) {
          unsigned* ctr = p.counters + static_cast<size_t>(gm.b) * p.hkv + gm.kvh;
          const unsigned old = atomicAdd(ctr, 1u);
          const int last = (old == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
          if (last) *ctr = 0;
          *last_flag = last;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_XCH));
        if (ok && !mbar_wait(bar(B_XCH), x_uses & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (6 << 8)), limit)) ok = false;
        ++x_uses;
        if (ok && *last_flag) {
          __threadfence();
          for (int i = st4; i < G * ADC_D; i += 128) {
            const int g = i / ADC_D, d = i % ADC_D;
            const size_t base = (static_cast<size_t>(gm.b) * p.hq + gm.kvh * G + g) * p.splits;
            float mm = -INFINITY;
            for (int sI = 0; sI < p.splits; ++sI) mm = fmaxf(mm, __ldcg(p.part_ml + (base + sI) * 2));
            float ll = 0.f, oo = 0.f;
            for (int sI = 0; sI < p.splits; ++sI) {
              const float ms = __ldcg(p.part_ml + (base + sI) * 2);
              const float wgt = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
              ll += wgt * __ldcg(p.part_ml + (base + sI) * 2 + 1);
              oo += wgt * __ldcg(p.part_acc + (base + sI) * ADC_D + d);
            }
            p.out[(static_cast<size_t>(gm.b) * p.hq + gm.kvh * G + g) * ADC_D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
          }
        }
      }
      len_cur = len_nxt;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, ADC_TMEM_COLS); }
}

typedef CUresult (*EncodeTiledFn3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// NB: 128-token blocks a CTA can hold.  4 with the merge zone (clusters of splits), 9 without it for a CTA that takes a
// whole sequence of up to 1,152 tokens - both sized for two CTAs per SM.
template <int G, bool FUSED, int NB>
static int launch_adc(const CUtensorMap& tm, const DecodeTcParams& p, dim3 grid, cudaStream_t stream) {
  // rows of the CTA's heads, the new token's value row, a few scalars, and (groups of up to four heads) the merge zone
  constexpr int SMEM = 2 * ADC_TILE + NB * ADC_P_TILE + ADC_Q_TILE + (128 + 32) * 4 + (6 + 2 * NB) * 8 + 64 + NB * 8 * 4 + 1024 +
                       (G * ADC_D + ADC_D + 32) * 4 + 16 +
                       ((G <= ADC_ZONE_MAX_G && NB <= ADC_NB) ? ADC_ZONE_MAX_SPLITS * G * ADC_ZONE_ROW * 4 : 0);
  static_assert(2 * (SMEM + 1024) <= 228 * 1024, "two CTAs per SM");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tc_kernel<G, FUSED, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(attn_decode_tc_kernel<G, FUSED, NB>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  if (p.cluster_merge) launch_ex_cluster(attn_decode_tc_kernel<G, FUSED, NB>, dim3(grid), dim3(ADC_THREADS), SMEM, stream, dim3(1, 1, grid.z), tm, p);
  else launch_ex(attn_decode_tc_kernel<G, FUSED, NB>, dim3(grid), dim3(ADC_THREADS), SMEM, stream, 0, tm, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}


template <int G>
static int launch_adcp(const CUtensorMap& tm, const DecodeTcParams& p, int num_items, int num_sms, cudaStream_t stream) {
  constexpr int SMEM = 2 * ADC_TILE + ADC_NB * ADC_P_TILE + 2 * ADC_Q_TILE + 64 * 4 + (12 + 2 * ADC_NB) * 8 + 64 + 2 * ADC_NB * 8 * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tcp_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(attn_decode_tcp_kernel<G>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  const int grid = num_items < 2 * num_sms ? num_items : 2 * num_sms;
  launch_ex(attn_decode_tcp_kernel<G>, dim3(grid), dim3(ADC_THREADS), SMEM, stream, 0, tm, p, num_items);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

}  // namespace b200

using namespace b200;

// Smallest split count this kernel accepts for sequences of up to max_len tokens (each CTA holds at most 4 x 128).
extern "C" int b200_attn_decode_tc_min_splits(int max_len) {
  const int blocks = (max_len + 127) / 128;
  return (blocks + ADC_NB - 1) / ADC_NB > 0 ? (blocks + ADC_NB - 1) / ADC_NB : 1;
}
// 128-token blocks one CTA can hold: 4, or 9 in the fused form (b200_attn_decode_fused) when the splits do not merge
// as a cluster
extern "C" int b200_attn_decode_tc_blocks_per_cta(int fused) { return fused ? ADC_NB_LONG : ADC_NB; }

static int attn_decode_tc_common(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                                 void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                                 int max_pages, int splits, float scale, int* status, int persistent, int num_sms,
                                 cudaStream_t stream, const DecodeFuse* fuse = nullptr) {
  if (B <= 0) return 0;
  if (page_size != 16 || (hq % hkv)) return -3;
  const int G = hq / hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return -3;
  if (G == 16 && persistent) return -3;               // sixteen heads per KV head: the one-item kernel only
  if (splits < 1) splits = 1;
  if (reinterpret_cast<uintptr_t>(cache) & 127) return -2;
  if (!fuse && (reinterpret_cast<uintptr_t>(q) & 15)) return -2;
  if (fuse) {
    if (persistent || !fuse->qkv || !fuse->positions || !fuse->cos_tab || !fuse->sin_tab || fuse->max_pos <= 0 || !fuse->cache) return -1;
    if ((reinterpret_cast<uintptr_t>(fuse->qkv) & 15) || (fuse->ld_qkv % 8) || (reinterpret_cast<uintptr_t>(fuse->cos_tab) & 15) ||
        (reinterpret_cast<uintptr_t>(fuse->sin_tab) & 15)) return -2;
    if (fuse->xq) {
      if (!fuse->sx || (fuse->ldq % 4) || (reinterpret_cast<uintptr_t>(fuse->xq) & 3)) return -2;
      if (hkv > 1 && (!fuse->rot_scratch || !fuse->blk_amax || !fuse->seq_counters || (reinterpret_cast<uintptr_t>(fuse->rot_scratch) & 15))) return -1;
    }
  }
  static EncodeTiledFn3 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) return -11;
    fn = reinterpret_cast<EncodeTiledFn3>(ptr);
  }
  // the cache as [token rows][2 halves][64 bf16]: box = 16 token rows of one half
  CUtensorMap tm;
  cuuint64_t dims[3] = {64, 2, static_cast<cuuint64_t>(num_pages) * 2 * hkv * 16};
  cuuint64_t strides[2] = {128, 256};
  cuuint32_t box[3] = {64, 1, 16};
  cuuint32_t estr[3] = {1, 1, 1};
  if (fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -12;
  DecodeTcParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.page_table = page_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_acc = scratch;
  p.part_ml = scratch ? scratch + static_cast<size_t>(B) * hq * splits * ADC_D : nullptr;
  p.counters = counters; p.hq = hq; p.hkv = hkv; p.max_pages = max_pages; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.limit_ns = 2000000000ull;
  if (fuse) p.f = *fuse; else p.f = DecodeFuse{};
  // splits of one (sequence, kv head) as a thread-block cluster that merges in shared memory (B200RT_ATTN_CLUSTER=0: off)
  static int cluster_env = -1;
  if (cluster_env < 0) { const char* e = std::getenv("B200RT_ATTN_CLUSTER"); cluster_env = (e && e[0] == '0') ? 0 : 1; }
  // Only while the grid is resident in one go (two CTAs per SM): with several waves of CTAs, clusters that have to be
  // placed whole are slower than independent CTAs that merge through global memory (measured: 768 CTAs, 583 vs 569 us
  // per four layers), while a one-wave grid saves the fence, the counter and the L2 round trips of that merge.
  static int sm_count = 0;
  if (!sm_count) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev); }
  static int early_env = -1;
  if (early_env < 0) { const char* e = std::getenv("B200RT_ATTN_EARLY_TILES"); early_env = (e && e[0] == '0') ? 0 : 1; }
  p.early_tiles = early_env;
  // blocks a CTA may meet: the page-table row bounds the sequence length
  const int blocks_max = (max_pages * 16 + 127) / 128, per_max = (blocks_max + splits - 1) / splits;
  const bool long_form = fuse && !persistent && per_max > ADC_NB && G <= 8;   // (sixteen heads: the scores of nine blocks would not fit the registers)        // whole (or half) sequences per CTA: no merge zone
  if (per_max > (long_form ? ADC_NB_LONG : ADC_NB)) return -1;
  p.cluster_merge = (!persistent && !long_form && cluster_env && G <= ADC_ZONE_MAX_G && splits >= 2 && splits <= ADC_ZONE_MAX_SPLITS &&
                     static_cast<long long>(B) * hkv * splits <= 2ll * sm_count) ? 1 : 0;
  if (splits > 1 && !p.cluster_merge && (!scratch || !counters)) return -1;
  if (persistent) {
    const int items = B * hkv * splits;
    switch (G) {
      case 1: return launch_adcp<1>(tm, p, items, num_sms, stream);
      case 2: return launch_adcp<2>(tm, p, items, num_sms, stream);
      case 4: return launch_adcp<4>(tm, p, items, num_sms, stream);
      default: return launch_adcp<8>(tm, p, items, num_sms, stream);
    }
  }
  dim3 grid(hkv, B, splits);
  if (long_form) {
    switch (G) {
      case 1: return launch_adc<1, true, ADC_NB_LONG>(tm, p, grid, stream);
      case 2: return launch_adc<2, true, ADC_NB_LONG>(tm, p, grid, stream);
      case 4: return launch_adc<4, true, ADC_NB_LONG>(tm, p, grid, stream);
      default: return launch_adc<8, true, ADC_NB_LONG>(tm, p, grid, stream);
    }
  }
  if (fuse) {
    switch (G) {
      case 1: return launch_adc<1, true, ADC_NB>(tm, p, grid, stream);
      case 2: return launch_adc<2, true, ADC_NB>(tm, p, grid, stream);
      case 4: return launch_adc<4, true, ADC_NB>(tm, p, grid, stream);
      case 8: return launch_adc<8, true, ADC_NB>(tm, p, grid, stream);
      default: return launch_adc<16, true, ADC_NB>(tm, p, grid, stream);
    }
  }
  switch (G) {
    case 1: return launch_adc<1, false, ADC_NB>(tm, p, grid, stream);
    case 2: return launch_adc<2, false, ADC_NB>(tm, p, grid, stream);
    case 4: return launch_adc<4, false, ADC_NB>(tm, p, grid, stream);
    case 8: return launch_adc<8, false, ADC_NB>(tm, p, grid, stream);
    default: return launch_adc<16, false, ADC_NB>(tm, p, grid, stream);
  }
}

// Decode attention with its neighbours folded in (one launch instead of rope_kv_write + attention + activation
// prologue of o_proj): qkv holds the new token's raw q | k | v projections, the kernel normalises / rotates q and k,
// appends k and v at positions[b] of the paged cache, attends to the seq_lens[b] - 1 cached tokens plus the new one, and,
// when xq is given, leaves the attention output rotated (block-128 Hadamard, one head = one block) and quantised
// per token in xq / sx; out (bf16 [B][hq][128]) is optional then.  rot_scratch (B * hq * 128 floats), blk_amax
// (B * hkv floats) and seq_counters (B zeroed uint32) are needed when hkv > 1 and xq is given.
extern "C" int b200_attn_decode_fused(const void* qkv, long long ld_qkv, const int* positions, const float* cos_tab,
                                      const float* sin_tab, int max_pos, const void* q_norm_w, const void* k_norm_w, float eps,
                                      void* cache, int num_pages, const int* page_table, const int* seq_lens, void* out,
                                      void* xq, long long ldq, float* sx, float* scratch, unsigned* counters,
                                      float* rot_scratch, float* blk_amax, unsigned* seq_counters, int B, int hq, int hkv,
                                      int page_size, int max_pages, int splits, float scale, int* status,
                                      const void* next_weights, unsigned long long next_weights_bytes, cudaStream_t stream) {
  DecodeFuse f;
  f.qkv = static_cast<const __nv_bfloat16*>(qkv); f.ld_qkv = ld_qkv; f.positions = positions; f.cos_tab = cos_tab; f.sin_tab = sin_tab;
  f.max_pos = max_pos; f.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_w); f.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_w);
  f.eps = eps; f.cache = static_cast<__nv_bfloat16*>(cache); f.num_pages = num_pages;
  f.xq = static_cast<int8_t*>(xq); f.ldq = ldq; f.sx = sx; f.rot_scratch = rot_scratch; f.blk_amax = blk_amax; f.seq_counters = seq_counters;
  static int l2_env = -1;
  if (l2_env < 0) { const char* e = std::getenv("B200RT_ATTN_NEXT_W"); l2_env = (e && e[0] == '1') ? 1 : 0; }
  const bool pf = l2_env && next_weights && next_weights_bytes >= 16 && (reinterpret_cast<uintptr_t>(next_weights) & 15) == 0;
  f.next_w = pf ? static_cast<const uint8_t*>(next_weights) : nullptr;
  f.next_w_bytes = pf ? next_weights_bytes : 0;
  return attn_decode_tc_common(nullptr, cache, num_pages, page_table, seq_lens, out, scratch, counters, B, hq, hkv, page_size,
                               max_pages, splits, scale, status, 0, 0, stream, &f);
}

// CTAs of the tensor-core decode attention (group size 4, plain form) one SM holds at once.
extern "C" int b200_attn_decode_tc_ctas_per_sm() {
  constexpr int SMEM = 2 * ADC_TILE + ADC_NB * ADC_P_TILE + ADC_Q_TILE + (128 + 32) * 4 + (6 + 2 * ADC_NB) * 8 + 64 + ADC_NB * 8 * 4 + 1024;
  cudaFuncSetAttribute(attn_decode_tc_kernel<4, false, ADC_NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  cudaFuncSetAttribute(attn_decode_tc_kernel<4, false, ADC_NB>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  int blocks = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attn_decode_tc_kernel<4, false, ADC_NB>, ADC_THREADS, SMEM);
  return blocks;
}

// Same contract as b200_attn_decode_tma.  splits must be at least b200_attn_decode_tc_min_splits(longest sequence).
extern "C" int b200_attn_decode_tc(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                                   void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                                   int max_pages, int splits, float scale, int* status, cudaStream_t stream) {
  return attn_decode_tc_common(q, cache, num_pages, page_table, seq_lens, out, scratch, counters, B, hq, hkv, page_size,
                               max_pages, splits, scale, status, 0, 0, stream);
}

// Persistent form of the same kernel: two CTAs per SM walk the (kv head, sequence, split) items.
extern "C" int b200_attn_decode_tcp(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                                    void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                                    int max_pages, int splits, float scale, int* status, int num_sms, cudaStream_t stream) {
  return attn_decode_tc_common(q, cache, num_pages, page_table, seq_lens, out, scratch, counters, B, hq, hkv, page_size,
                               max_pages, splits, scale, status, 1, num_sms > 0 ? num_sms : 148, stream);
}
