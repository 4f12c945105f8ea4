// W8A8 GEMM for sm_100a:  Y[m,n] = (sum_k Xq[m,k] * Wq[n,k]) * sx[m] * sw[n]  (+ residual[m,n])
//
//   Xq int8 [M,K] (tokens, already Hadamard-rotated and per-token quantised), sx fp32 [M]
//   Wq int8 [N,K] (output channels, stored rotated), sw fp32 [N]
//
// Design (Blackwell-first):
//   * The weight tile is the tcgen05 "A" operand (128 output channels fill the MMA M dimension), the
//     token tile is the "B" operand (BN in {16,32,64,128,256} tokens fill the MMA N dimension).  The same
//     kernel therefore serves decode (M = 1..32 tokens: pure weight streaming) and prefill (M in the
//     thousands) without ever padding tokens up to 128.
//   * Operands arrive by TMA (2-D tiled, 128-byte swizzle, no cluster broadcast) into a STAGES-deep
//     ring of shared-memory stages guarded by full/empty mbarriers.
//   * One elected thread issues tcgen05.mma.kind::i8 (128 x BN x 32 per instruction); the int32
//     accumulator lives in TMEM and is double buffered so the epilogue of one tile overlaps the
//     main loop of the next.
//   * Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2..5 = epilogue
//     (each reads its 32-lane quarter of TMEM with tcgen05.ld).
//   * Persistent grid.  Work is the list of (tile, k-block) units.  Large problems give each CTA whole
//     tiles round-robin, rasterised so that concurrently running CTAs share token panels in L2.
//     Small-M problems (decode) use a stream-K split: every CTA gets an equal share of k-blocks;
//     partial tiles are summed exactly with int32 atomics into a scratch buffer and the CTA that
//     completes a tile applies the scales (and re-zeroes the scratch for the next launch).
//   * Every mbarrier wait is bounded; on a timeout the CTA records a status code, drains and exits.
#include "ptx.cuh"
#include "api.h"
#include <cuda.h>

namespace b200 {

constexpr int TILE_N = 128;     // output channels per tile  (MMA M)
constexpr int BLOCK_K = 128;    // int8 elements (= bytes) per k-block: one 128-byte swizzle row
constexpr int UMMA_K = 32;      // int8 elements per tcgen05.mma
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;      // token tiles per rasterisation group

struct GemmParams {
  int M, N, K;
  int m_tiles, n_tiles, kblocks, num_tiles;
  int mode;                     // 0: whole tiles round-robin, 1: stream-K
  long long total_units;
  const float* sx;
  const float* sw;
  void* y;
  const __nv_bfloat16* residual;
  int ldy;
  int out_fp32;
  int32_t* ws;                  // [m_tiles*BN][n_tiles*128] int32, zero between launches (mode 1)
  int ldws;
  uint32_t* counters;           // [num_tiles], zero between launches (mode 1)
  int* status;
  unsigned long long limit_ns;
};

struct Seg { int tile, kb0, kb1; };

struct WorkIter {
  int mode, next_tile, stride, num_tiles, kblocks;
  long long u, u_end;
  __device__ WorkIter(const GemmParams& p) {
    mode = p.mode; num_tiles = p.num_tiles; kblocks = p.kblocks;
    next_tile = blockIdx.x; stride = gridDim.x;
    u = p.total_units * blockIdx.x / gridDim.x;
    u_end = p.total_units * (blockIdx.x + 1) / gridDim.x;
  }
  __device__ bool next(Seg& s) {
    if (mode == 0) {
      if (next_tile >= num_tiles) return false;
      s.tile = next_tile; s.kb0 = 0; s.kb1 = kblocks; next_tile += stride;
      return true;
    }
    if (u >= u_end) return false;
    s.tile = static_cast<int>(u / kblocks);
    s.kb0 = static_cast<int>(u - static_cast<long long>(s.tile) * kblocks);
    long long take = kblocks - s.kb0;
    if (take > u_end - u) take = u_end - u;
    s.kb1 = s.kb0 + static_cast<int>(take);
    u += take;
    return true;
  }
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& m_tile, int& n_tile) {
  const int per_group = GROUP_M * p.n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(GROUP_M, p.m_tiles - first_m);
  const int r = tile - g * per_group;
  m_tile = first_m + r % gsize;
  n_tile = r / gsize;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const GemmParams p) {
  constexpr int A_BYTES = TILE_N * BLOCK_K;      // 16 KiB
  constexpr int B_BYTES = BN * BLOCK_K;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;   // power of two for BN in {16,...,256}
  constexpr uint32_t IDESC = umma_idesc_i8(TILE_N, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars: [0,STAGES) full, [STAGES,2*STAGES) empty, then tmem_full[2], tmem_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* fix_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
    *fix_slot = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint64_t limit = p.limit_ns;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tmap(&tmap_w);
      prefetch_tmap(&tmap_x);
      const uint64_t pol_w = (p.m_tiles == 1) ? policy_evict_first() : policy_evict_last();
      WorkIter it(p);
      Seg sg;
      int stage = 0; uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      while (ok && it.next(sg)) {
        int m_tile, n_tile;
        tile_coords(p, sg.tile, m_tile, n_tile);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY, limit)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          tma_load_2d_hint(a_dst, &tmap_w, full_bar(stage), kb * BLOCK_K, n_tile * TILE_N, pol_w);
          tma_load_2d(a_dst + A_BYTES, &tmap_x, full_bar(stage), kb * BLOCK_K, m_tile * BN);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies already in flight a bounded chance to land before the CTA's shared memory goes away.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }
      }
      (void)issued;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      WorkIter it(p);
      Seg sg;
      int stage = 0; uint32_t phase = 0;
      int seg_idx = 0;
      bool ok = true;
      while (ok && it.next(sg)) {
        const int a = seg_idx & 1;
        const uint32_t aphase = (seg_idx >> 1) & 1u;
        if (!mbar_wait(tempty_bar(a), aphase ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY, limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL, limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a_src);
          const uint64_t b_desc = umma_desc_k_sw128(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            // advancing 32 bytes along K inside the 128-byte swizzle row = +2 in 16-byte address units
            umma_i8_ss(d_tmem, a_desc + 2ull * k, b_desc + 2ull * k, IDESC, (kb > sg.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(a));
        ++seg_idx;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (4 warps) ------------------------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 64;        // 0..127
    WorkIter it(p);
    Seg sg;
    int seg_idx = 0;
    bool ok = true;
    while (ok && it.next(sg)) {
      const int a = seg_idx & 1;
      const uint32_t aphase = (seg_idx >> 1) & 1u;
      int m_tile, n_tile;
      tile_coords(p, sg.tile, m_tile, n_tile);
      if (!mbar_wait(tfull_bar(a), aphase, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL, limit)) { ok = false; break; }
      tc_fence_after();
      const int n = n_tile * TILE_N + q * 32 + lane;
      const bool n_ok = n < p.N;
      const int m0 = m_tile * BN;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * BN;
      const bool whole = (sg.kb0 == 0 && sg.kb1 == p.kblocks);
      const float swn = n_ok ? __ldg(p.sw + n) : 0.f;

      constexpr int CH = (BN >= 32) ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BN / CH; ++c) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_x32(t_addr + c * CH, r); else tmem_ld_x16(t_addr + c * CH, r);
        tmem_ld_wait();
        if (whole) {
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int m = m0 + c * CH + j;
              if (m < p.M) {
                float v = static_cast<float>(static_cast<int32_t>(r[j])) * swn * __ldg(p.sx + m);
                const size_t o = static_cast<size_t>(m) * p.ldy + n;
                if (p.residual) v += __bfloat162float(p.residual[o]);
                if (p.out_fp32) reinterpret_cast<float*>(p.y)[o] = v;
                else reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16(v);
              }
            }
          }
        } else {
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int m = m0 + c * CH + j;
              if (m < p.M) atomicAdd(p.ws + static_cast<size_t>(m) * p.ldws + n, static_cast<int32_t>(r[j]));
            }
          }
        }
      }
      // accumulator drained: hand the TMEM buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(a));

      if (!whole) {
        __threadfence();
        named_bar_sync(1, 128);
        if (et == 0) {
          const uint32_t add = static_cast<uint32_t>(sg.kb1 - sg.kb0);
          const uint32_t old = atomicAdd(p.counters + sg.tile, add);
          *fix_slot = (old + add == static_cast<uint32_t>(p.kblocks)) ? 1 : 0;
        }
        named_bar_sync(1, 128);
        const int last = *fix_slot;
        named_bar_sync(1, 128);     // everyone has read fix_slot before it can be rewritten
        if (last) {
          __threadfence();
          if (n_ok) {
            for (int j = 0; j < BN; ++j) {
              const int m = m0 + j;
              if (m >= p.M) break;
              int32_t* wp = p.ws + static_cast<size_t>(m) * p.ldws + n;
              const int32_t acc = __ldcg(wp);
              *wp = 0;
              float v = static_cast<float>(acc) * swn * __ldg(p.sx + m);
              const size_t o = static_cast<size_t>(m) * p.ldy + n;
              if (p.residual) v += __bfloat162float(p.residual[o]);
              if (p.out_fp32) reinterpret_cast<float*>(p.y)[o] = v;
              else reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16(v);
            }
          }
          if (et == 0) p.counters[sg.tile] = 0;
        }
      }
      ++seg_idx;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    if (qres != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D row-major byte matrix [rows][cols] with row pitch `pitch` bytes; box = 128 bytes x box_rows, 128-byte swizzle.
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r);
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int grid, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (TILE_N * BLOCK_K + BN * BLOCK_K) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  w8a8_gemm_kernel<BN, STAGES><<<grid, GEMM_THREADS, SMEM, stream>>>(tw, tx, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

int gemm_pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_w8a8_gemm_ws_bytes(int M, int N) {
  const int bn = gemm_pick_bn(M);
  const size_t m_pad = static_cast<size_t>((M + bn - 1) / bn) * bn;
  const size_t n_pad = static_cast<size_t>((N + TILE_N - 1) / TILE_N) * TILE_N;
  return m_pad * n_pad * sizeof(int32_t);
}

extern "C" int b200_w8a8_gemm(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                              const void* residual, int M, int N, int K, int ldy, int out_fp32,
                              void* ws, size_t ws_bytes, void* counters, int counters_len, int* status,
                              int num_sms, int force_mode, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 16) != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15)) return -2;
  const int bn = gemm_pick_bn(M);
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = (M + bn - 1) / bn;
  p.n_tiles = (N + TILE_N - 1) / TILE_N;
  p.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
  p.num_tiles = p.m_tiles * p.n_tiles;
  p.total_units = static_cast<long long>(p.num_tiles) * p.kblocks;
  p.sx = sx; p.sw = sw; p.y = y; p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldy = ldy; p.out_fp32 = out_fp32;
  p.ws = static_cast<int32_t*>(ws);
  p.ldws = p.n_tiles * TILE_N;
  p.counters = static_cast<uint32_t*>(counters);
  p.status = status;
  p.limit_ns = 2000000000ull;

  const size_t need_ws = static_cast<size_t>(p.m_tiles) * bn * p.ldws * sizeof(int32_t);
  const bool can_split = ws && counters && ws_bytes >= need_ws && counters_len >= p.num_tiles;
  int mode = 0;
  if (force_mode == 0 || force_mode == 1) mode = force_mode;
  else mode = (p.num_tiles < 2 * num_sms && p.m_tiles <= 2) ? 1 : 0;
  if (mode == 1 && !can_split) mode = 0;
  p.mode = mode;
  int grid;
  if (mode == 0) {
    grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  } else {
    long long g = p.total_units / 4;          // at least ~4 k-blocks per CTA
    if (g < 1) g = 1;
    if (g > num_sms) g = num_sms;
    if (g < p.num_tiles && p.num_tiles <= num_sms) g = p.num_tiles;
    grid = static_cast<int>(g);
  }

  CUtensorMap tw, tx;
  int r = make_tmap_2d_u8(&tw, wq, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), TILE_N);
  if (r) return -11;
  r = make_tmap_2d_u8(&tx, xq, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), bn);
  if (r) return -12;

  switch (bn) {
    case 16: return launch_gemm<16, 8>(tw, tx, p, grid, stream);
    case 32: return launch_gemm<32, 8>(tw, tx, p, grid, stream);
    case 64: return launch_gemm<64, 8>(tw, tx, p, grid, stream);
    case 128: return launch_gemm<128, 6>(tw, tx, p, grid, stream);
    default: return launch_gemm<256, 4>(tw, tx, p, grid, stream);
  }
}
