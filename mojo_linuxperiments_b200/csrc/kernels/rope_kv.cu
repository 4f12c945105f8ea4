// Token-wise glue kernels around attention:
//   rope_kv_write     (optional per-head RMSNorm of q/k) -> rotary embedding of q and k -> q to a dense buffer,
//                     k and v appended to the paged KV cache (and k optionally to a dense buffer for prefill)
//   embed_gather      token ids -> rows of the bf16 embedding table
//   argmax_rows       greedy sampling: (max, index) per row of a logits shard, plus an offset for vocab sharding
//   argmax_merge      combine per-rank (max, index) candidates gathered from all ranks
//
// KV cache layout: [num_pages][2 (k,v)][kv_heads][page_size][128] bf16, so one (page, head) holds page_size
// contiguous 256-byte rows; a sequence finds its pages through page_table[seq][pos / page_size].
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"

namespace b200 {

constexpr int HEAD_DIM = 128;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct RopeParams {
  const __nv_bfloat16* qkv;      // [M][(hq + 2 hkv) * 128]
  long long ld_qkv;
  const int* positions;          // [M] position of the token inside its sequence
  const int* seq_ids;            // [M] sequence of the token (nullptr: token i belongs to sequence i)
  const float* cos_tab;          // [max_pos][64]
  const float* sin_tab;          // [max_pos][64]
  const __nv_bfloat16* q_norm_w; // [128] or nullptr
  const __nv_bfloat16* k_norm_w; // [128] or nullptr
  float eps;
  __nv_bfloat16* q_out;          // [M][hq][128]
  __nv_bfloat16* k_out;          // [M][hkv][128] or nullptr
  __nv_bfloat16* v_out;          // [M][hkv][128] or nullptr
  __nv_bfloat16* cache;          // paged cache or nullptr
  const int* page_table;         // [num_seqs][max_pages]
  int max_pages, page_size;
  int hq, hkv, M;
  int max_pos;                   // rows of cos_tab / sin_tab
  int num_pages;                 // pages of the cache
  int* status;                   // optional status word: ST_BAD_ARGUMENT when a token is skipped
};

// grid (tokens, ceil(heads / 4)), 4 warps; a warp handles one head, lane l holds elements l, l+32, l+64, l+96
__global__ void __launch_bounds__(128) rope_kv_kernel(const RopeParams p) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  B200_TRACE_INIT();
  if (threadIdx.x == 0) B200_TRACE(TK_ROPE_KV, TP_START);
  pdl_wait();                // everything before this kernel in the stream has completed
  if (threadIdx.x == 0) B200_TRACE(TK_ROPE_KV, TP_DEPS);
  B200_TRACE_FLUSH(TK_ROPE_KV);

  const int tok = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[tok];
  const int seq = p.seq_ids ? p.seq_ids[tok] : tok;
  // A position beyond the tables or beyond the pages admitted for the sequence must not become a stray write: the
  // token is skipped (q_out keeps what it held) and the status word says so.
  bool bad = pos < 0 || pos >= p.max_pos || (p.cache && pos / p.page_size >= p.max_pages);
  int page = 0;
  if (!bad && p.cache) {
    page = p.page_table[static_cast<size_t>(seq) * p.max_pages + pos / p.page_size];
    bad = page < 0 || page >= p.num_pages;
  }
  if (bad) {
    if (threadIdx.x == 0 && blockIdx.y == 0 && p.status) atomicCAS(p.status, 0, static_cast<int>(ST_BAD_ARGUMENT) | (7 << 8));
    return;
  }
  const __nv_bfloat16* row = p.qkv + static_cast<size_t>(tok) * p.ld_qkv;
  const float c0 = p.cos_tab[static_cast<size_t>(pos) * 64 + lane], s0 = p.sin_tab[static_cast<size_t>(pos) * 64 + lane];
  const float c1 = p.cos_tab[static_cast<size_t>(pos) * 64 + lane + 32], s1 = p.sin_tab[static_cast<size_t>(pos) * 64 + lane + 32];
  size_t cache_row = 0;
  if (p.cache) cache_row = static_cast<size_t>(page) * 2 * p.hkv * p.page_size + (pos % p.page_size);
  const int nheads = p.hq + 2 * p.hkv;
  const int h = blockIdx.y * 4 + warp;
  if (h < nheads) {
    const __nv_bfloat16* x = row + static_cast<size_t>(h) * HEAD_DIM;
    float v0 = __bfloat162float(x[lane]), v1 = __bfloat162float(x[lane + 32]);
    float v2 = __bfloat162float(x[lane + 64]), v3 = __bfloat162float(x[lane + 96]);
    const bool is_q = h < p.hq, is_k = !is_q && h < p.hq + p.hkv;
    if (is_q || is_k) {
      const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
      if (nw) {
        const float ss = warp_sum_f(v0 * v0 + v1 * v1 + v2 * v2 + v3 * v3);
        const float r = rsqrtf(ss * (1.f / HEAD_DIM) + p.eps);
        v0 *= r * __bfloat162float(nw[lane]); v1 *= r * __bfloat162float(nw[lane + 32]);
        v2 *= r * __bfloat162float(nw[lane + 64]); v3 *= r * __bfloat162float(nw[lane + 96]);
      }
      // pairs (i, i+64): out[i] = x[i] cos_i - x[i+64] sin_i ; out[i+64] = x[i+64] cos_i + x[i] sin_i
      const float o0 = v0 * c0 - v2 * s0, o2 = v2 * c0 + v0 * s0;
      const float o1 = v1 * c1 - v3 * s1, o3 = v3 * c1 + v1 * s1;
      v0 = o0; v1 = o1; v2 = o2; v3 = o3;
    }
    const __nv_bfloat16 b0 = __float2bfloat16(v0), b1 = __float2bfloat16(v1), b2 = __float2bfloat16(v2), b3 = __float2bfloat16(v3);
    auto put = [&](__nv_bfloat16* dst) { dst[lane] = b0; dst[lane + 32] = b1; dst[lane + 64] = b2; dst[lane + 96] = b3; };
    if (is_q) {
      put(p.q_out + (static_cast<size_t>(tok) * p.hq + h) * HEAD_DIM);
    } else {
      const int kvh = is_k ? h - p.hq : h - p.hq - p.hkv;
      __nv_bfloat16* dense = is_k ? p.k_out : p.v_out;
      if (dense) put(dense + (static_cast<size_t>(tok) * p.hkv + kvh) * HEAD_DIM);
      if (p.cache) {
        // [page][k|v][head][slot][128]
        const size_t off = cache_row + (static_cast<size_t>(is_k ? 0 : 1) * p.hkv + kvh) * p.page_size;
        put(p.cache + off * HEAD_DIM);
      }
    }
  }
}

__global__ void embed_gather_kernel(const long long* ids, const __nv_bfloat16* table,
                                    __nv_bfloat16* out, int d, int vocab) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  const int tok = blockIdx.x;
  long long id = ids[tok];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * d);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(tok) * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

// grid (rows, chunks): CTA (r, c) scans columns [c*cs, (c+1)*cs) of row r and writes candidate [c][r];
// ties resolve to the lowest index (matches torch.argmax on a single device after the merge)
__global__ void __launch_bounds__(256) argmax_rows_kernel(const __nv_bfloat16* logits, long long ld, int n,
                                                          int chunk, int index_offset, float* out_val,
                                                          long long* out_idx) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  __shared__ float sv[8];
  __shared__ int si[8];
  const int row = blockIdx.x;
  const int c0 = blockIdx.y * chunk, c1 = min(n, c0 + chunk);
  const __nv_bfloat16* x = logits + static_cast<size_t>(row) * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto consider = [&](float v, int i) { if (v > best || (v == best && i < bi)) { best = v; bi = i; } };
  if (((reinterpret_cast<uintptr_t>(x) | static_cast<uintptr_t>(c0 * 2)) & 15) == 0) {
    const int nv = (c1 - c0) / 8;
    const uint4* xv = reinterpret_cast<const uint4*>(x + c0);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 raw = xv[i];
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        consider(__uint_as_float(w[k] << 16), c0 + i * 8 + 2 * k);
        consider(__uint_as_float(w[k] & 0xffff0000u), c0 + i * 8 + 2 * k + 1);
      }
    }
    for (int i = c0 + nv * 8 + threadIdx.x; i < c1; i += blockDim.x) consider(__bfloat162float(x[i]), i);
  } else {
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) consider(__bfloat162float(x[i]), i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    const size_t o = static_cast<size_t>(blockIdx.y) * gridDim.x + row;
    out_val[o] = best;
    out_idx[o] = static_cast<long long>(bi) + index_offset;
  }
}

// cand_val/cand_idx: [world][rows]; out: [rows]
__global__ void argmax_merge_kernel(const float* cand_val, const long long* cand_idx, int world,
                                    int rows, long long* out_idx) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float best = cand_val[r];
  long long bi = cand_idx[r];
  for (int w = 1; w < world; ++w) {
    const float v = cand_val[static_cast<size_t>(w) * rows + r];
    const long long i = cand_idx[static_cast<size_t>(w) * rows + r];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  out_idx[r] = bi;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rope_kv_write(const void* qkv, long long ld_qkv, const int* positions, const int* seq_ids,
                                  const float* cos_tab, const float* sin_tab, const void* q_norm_w, const void* k_norm_w,
                                  float eps, void* q_out, void* k_out, void* v_out, void* cache, const int* page_table,
                                  int max_pages, int page_size, int hq, int hkv, int M, int max_pos, int num_pages,
                                  int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (!qkv || !positions || !cos_tab || !sin_tab || !q_out || hq <= 0 || hkv <= 0 || max_pos <= 0) return -1;
  if (cache && (!page_table || page_size <= 0 || max_pages <= 0 || num_pages <= 0)) return -1;
  RopeParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv); p.ld_qkv = ld_qkv; p.positions = positions; p.seq_ids = seq_ids;
  p.cos_tab = cos_tab; p.sin_tab = sin_tab;
  p.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_w); p.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_w);
  p.eps = eps; p.q_out = static_cast<__nv_bfloat16*>(q_out); p.k_out = static_cast<__nv_bfloat16*>(k_out);
  p.v_out = static_cast<__nv_bfloat16*>(v_out);
  p.cache = static_cast<__nv_bfloat16*>(cache); p.page_table = page_table; p.max_pages = max_pages; p.page_size = page_size;
  p.hq = hq; p.hkv = hkv; p.M = M; p.max_pos = max_pos; p.num_pages = num_pages; p.status = status;
  launch_ex(rope_kv_kernel, dim3(dim3(M, (hq + 2 * hkv + 3) / 4)), dim3(128), 0, stream, 0, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_embed_gather(const long long* ids, const void* table, void* out, int M, int d, int vocab,
                                 cudaStream_t stream) {
  if (M <= 0) return 0;
  if (d % 8) return -1;
  launch_ex(embed_gather_kernel, dim3(M), dim3(128), 0, stream, 0, ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), d, vocab);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

// out_val / out_idx: [chunks][rows] candidates (merge them with b200_argmax_merge, world = chunks)
extern "C" int b200_argmax_rows(const void* logits, long long ld, int rows, int n, int index_offset, int chunks,
                                float* out_val, long long* out_idx, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (chunks < 1) chunks = 1;
  const int chunk = ((n + chunks - 1) / chunks + 7) & ~7;
  launch_ex(argmax_rows_kernel, dim3(dim3(rows, chunks)), dim3(256), 0, stream, 0, static_cast<const __nv_bfloat16*>(logits), ld, n, chunk, index_offset, out_val, out_idx);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_argmax_merge(const float* cand_val, const long long* cand_idx, int world, int rows, long long* out_idx,
                                 cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_ex(argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, 0, cand_val, cand_idx, world, rows, out_idx);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
