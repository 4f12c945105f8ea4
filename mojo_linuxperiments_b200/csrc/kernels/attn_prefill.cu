// Causal grouped-query flash attention for prefill on sm_100a tensor cores (bf16 in, fp32 accumulate).
//
// One CTA = 128 query rows of one head of one sequence; KV is walked in tiles of 128 tokens.
//   warp 0      TMA producer: Q once, then K and V tiles into two-stage rings (128-byte swizzle)
//   warp 1      MMA issuer:  S = Q.K^T (K-major x K-major) and PV = P.V (K-major P from smem x MN-major V),
//               both tcgen05.mma.kind::f16 with accumulators in TMEM: S and PV are each double buffered
//               (4 x 128 columns = the whole TMEM), so S of tile j+1 and PV of tile j run while the softmax
//               warps are busy with tile j
//   warps 2..5  softmax: thread <-> query row.  S is read with tcgen05.ld (twice: max pass, exp pass), P is
//               written to shared memory as bf16 in the swizzled K-major layout the MMA expects, the output
//               row lives in registers and is rescaled / accumulated from the PV buffer one tile late.
// Sequences are concatenated along the token axis (cu_seqlens); a tile may read rows of the next sequence,
// which the causal / length mask removes.  All waits are bounded.
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include <cuda.h>

namespace b200 {

constexpr int AP_THREADS = 192;
constexpr int AP_BM = 128, AP_BN = 128, AP_D = 128;
constexpr int AP_CHUNK_BYTES = 128 * 128;            // 128 rows x 64 bf16
constexpr int AP_TILE_BYTES = 2 * AP_CHUNK_BYTES;    // 128 x 128 bf16

struct PrefillParams {
  const int* cu_seqlens;      // [B+1]
  __nv_bfloat16* out;         // [tokens][hq][128]
  int hq, hkv;
  float scale_log2;
  int* status;
  unsigned long long limit_ns;
};

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes);

__global__ void __launch_bounds__(AP_THREADS, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [Q 32K][K0 32K][K1 32K][V0 32K][V1 32K][P 32K][barriers]
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + AP_TILE_BYTES;
  const uint32_t sV = sK + 2 * AP_TILE_BYTES;
  const uint32_t sP = sV + 2 * AP_TILE_BYTES;
  uint8_t* pP = smem + 5 * AP_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * AP_TILE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  enum { B_QFULL = 0, B_KFULL = 1, B_VFULL = 3, B_KEMPTY = 5, B_VEMPTY = 7, B_SFULL = 9, B_PFULL = 11, B_OFULL = 12, B_COUNT = 14 };
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;        // heavy (late) query tiles first
  const int head = blockIdx.y, b = blockIdx.z;
  const int seq0 = p.cu_seqlens[b];
  const int len = p.cu_seqlens[b + 1] - seq0;
  const int q0 = qt * AP_BM;
  if (q0 >= len) return;                            // uniform across the CTA, before any barrier / TMEM use
  const int n_tiles = qt + 1;                       // causal: kv tiles 0..qt
  const int kvh = head / (p.hq / p.hkv);
  const uint64_t limit = p.limit_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), (i == B_PFULL) ? 128 : 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_expect_tx(bar(B_QFULL), AP_TILE_BYTES);
      tma_load_2d(sQ, &tmap_q, bar(B_QFULL), head * AP_D, seq0 + q0);
      tma_load_2d(sQ + AP_CHUNK_BYTES, &tmap_q, bar(B_QFULL), head * AP_D + 64, seq0 + q0);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        const int row = seq0 + j * AP_BN;
        if (!mbar_wait(bar(B_KEMPTY + st), ph ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (3 << 8)), limit)) { ok = false; break; }
        mbar_expect_tx(bar(B_KFULL + st), AP_TILE_BYTES);
        tma_load_2d(sK + st * AP_TILE_BYTES, &tmap_k, bar(B_KFULL + st), kvh * AP_D, row);
        tma_load_2d(sK + st * AP_TILE_BYTES + AP_CHUNK_BYTES, &tmap_k, bar(B_KFULL + st), kvh * AP_D + 64, row);
        if (!mbar_wait(bar(B_VEMPTY + st), ph ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (3 << 8)), limit)) { ok = false; break; }
        mbar_expect_tx(bar(B_VFULL + st), AP_TILE_BYTES);
        tma_load_2d(sV + st * AP_TILE_BYTES, &tmap_v, bar(B_VFULL + st), kvh * AP_D, row);
        tma_load_2d(sV + st * AP_TILE_BYTES + AP_CHUNK_BYTES, &tmap_v, bar(B_VFULL + st), kvh * AP_D + 64, row);
      }
      if (!ok) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) { } }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, 128, 0, 1);     // B (= V) is MN-major
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t d = tmem_base + (j & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * AP_CHUNK_BYTES;
          const uint64_t a = umma_desc_k_sw128(sQ + off) + 2ull * (kk & 3);
          const uint64_t bd = umma_desc_k_sw128(sK + st * AP_TILE_BYTES + off) + 2ull * (kk & 3);
          umma_f16_ss(d, a, bd, IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(B_KEMPTY + st));
        umma_commit(bar(B_SFULL + (j & 1)));
      };
      bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (3 << 8)), limit) &&
                mbar_wait(bar(B_KFULL + 0), 0, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (3 << 8)), limit);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (j + 1 < n_tiles) {
          if (!mbar_wait(bar(B_KFULL + ((j + 1) & 1)), ((j + 1) >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (3 << 8)), limit)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(bar(B_PFULL), j & 1u, abort_flag, p.status, (ST_TIMEOUT_PEER_FLAG | (3 << 8)), limit)) { ok = false; break; }
        if (!mbar_wait(bar(B_VFULL + st), ph, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (3 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + 256 + (j & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a = umma_desc_k_sw128(sP + (kk >> 2) * AP_CHUNK_BYTES) + 2ull * (kk & 3);
          const uint64_t bd = umma_desc_mn_sw128(sV + st * AP_TILE_BYTES + kk * 2048, AP_CHUNK_BYTES, 1024);
          umma_f16_ss(d, a, bd, IDESC_PV, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(B_VEMPTY + st));
        umma_commit(bar(B_OFULL + (j & 1)));
      }
    }
    __syncwarp();
  } else {
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                    // row inside the tile == TMEM lane
    const int q_idx = q0 + r;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    float o[AP_D];
#pragma unroll
    for (int i = 0; i < AP_D; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    bool ok = true;
    uint8_t* p_row = pP + (r >> 3) * 1024 + (r & 7) * 128;
    const int sw = r & 7;

    auto o_update = [&](int j, float alpha) -> bool {
      if (!mbar_wait(bar(B_OFULL + (j & 1)), (j >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (3 << 8)), limit)) return false;
      tc_fence_after();
      const uint32_t t_pv = t_lane + 256 + (j & 1) * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_x32(t_pv + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
      return true;
    };

    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(bar(B_SFULL + (j & 1)), (j >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (3 << 8)), limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_s = t_lane + (j & 1) * 128;
      const int kv0 = j * AP_BN;
      const bool need_mask = (kv0 + AP_BN > q0) || (kv0 + AP_BN > len);
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_x32(t_s + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]);
          if (need_mask) { const int kv = kv0 + c * 32 + i; if (kv > q_idx || kv >= len) s = -INFINITY; }
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // the P buffer is free once the PV MMA of the previous tile has completed
      if (j > 0) {
        if (!mbar_wait(bar(B_OFULL + ((j - 1) & 1)), ((j - 1) >> 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (3 << 8)), limit)) { ok = false; break; }
      }
      // pass 2: probabilities -> bf16 -> swizzled shared memory
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_x32(t_s + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(v[i]), s1 = __uint_as_float(v[i + 1]);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv > q_idx || kv >= len) s0 = -INFINITY;
            if (kv + 1 > q_idx || kv + 1 >= len) s1 = -INFINITY;
          }
          const float e0 = exp2f(s0 * p.scale_log2 - m_use), e1 = exp2f(s1 * p.scale_log2 - m_use);
          const __nv_bfloat162 pb = __floats2bfloat162_rn(e0, e1);
          // sum what the MMA will actually see
          sum += __low2float(pb) + __high2float(pb);
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        // 32 columns = 4 sixteen-byte units; unit u of 128-byte row chunk lands at (u ^ (row & 7))
        uint8_t* chunk = p_row + (c >> 1) * AP_CHUNK_BYTES;
#pragma unroll
        for (int u4 = 0; u4 < 4; ++u4) {
          const int u = (c & 1) * 4 + u4;
          *reinterpret_cast<uint4*>(chunk + ((u ^ sw) << 4)) = make_uint4(pk[4 * u4], pk[4 * u4 + 1], pk[4 * u4 + 2], pk[4 * u4 + 3]);
        }
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(bar(B_PFULL));
      // while the tensor core works on PV of this tile, fold in PV of the previous one
      if (j > 0) { if (!o_update(j - 1, alpha_prev)) { ok = false; break; } }
      alpha_prev = alpha;
    }
    if (ok) ok = o_update(n_tiles - 1, alpha_prev);
    if (ok && q_idx < len) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(seq0 + q_idx) * p.hq + head) * AP_D);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const __nv_bfloat162 pb = __floats2bfloat162_rn(o[u * 8 + 2 * k] * inv, o[u * 8 + 2 * k + 1] * inv);
          w[k] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        dst[u] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bf16 row-major [rows][cols] with row pitch in bytes; box = 64 columns (128 bytes) x 128 rows, 128-byte swizzle
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) return -1;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r);
}

}  // namespace b200

using namespace b200;

// q [tokens][hq*128] (pitch ld_q elements), k / v [tokens][hkv*128] (pitches ld_k / ld_v), out [tokens][hq][128];
// cu_seqlens [B+1] device ints; max_len = longest sequence (host value, sizes the grid).
extern "C" int b200_attn_prefill(const void* q, long long ld_q, const void* k, long long ld_k, const void* v, long long ld_v,
                                 void* out, const int* cu_seqlens, int B, int total_tokens, int max_len, int hq, int hkv,
                                 float scale, int* status, cudaStream_t stream) {
  if (B <= 0 || total_tokens <= 0 || max_len <= 0) return 0;
  if (hq % hkv) return -1;
  if ((ld_q % 8) || (ld_k % 8) || (ld_v % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  CUtensorMap tq, tk, tv;
  if (make_tmap_2d_bf16(&tq, q, static_cast<uint64_t>(hq) * AP_D, total_tokens, static_cast<uint64_t>(ld_q) * 2)) return -11;
  if (make_tmap_2d_bf16(&tk, k, static_cast<uint64_t>(hkv) * AP_D, total_tokens, static_cast<uint64_t>(ld_k) * 2)) return -12;
  if (make_tmap_2d_bf16(&tv, v, static_cast<uint64_t>(hkv) * AP_D, total_tokens, static_cast<uint64_t>(ld_v) * 2)) return -13;
  PrefillParams p;
  p.cu_seqlens = cu_seqlens; p.out = static_cast<__nv_bfloat16*>(out); p.hq = hq; p.hkv = hkv;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.limit_ns = 2000000000ull;
  constexpr int SMEM = 6 * AP_TILE_BYTES + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  dim3 grid((max_len + AP_BM - 1) / AP_BM, hq, B);
  launch_ex(attn_prefill_kernel, dim3(grid), dim3(AP_THREADS), SMEM, stream, 0, tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
