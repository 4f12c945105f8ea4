// W8A8 GEMM for sm_100a:  Y[m,n] = (sum_k Xq[m,k] * Wq[n,k]) * sx[m] * sw[n]  (+ residual[m,n])
//
//   Xq int8 [M,K] (tokens, already Hadamard-rotated and per-token quantised), sx fp32 [M]
//   Wq int8 [N,K] (output channels, stored rotated), sw fp32 [N]
//
// Design (Blackwell-first):
//   * Two orientations of one kernel.  SWAP (M <= 64 tokens, decode): the weight tile is the tcgen05 "A"
//     operand (128 output channels fill the MMA M dimension) and the token tile is the "B" operand
//     (BN in {16,32,64} tokens fill the MMA N dimension), so tokens are never padded up to 128 and the
//     kernel is pure weight streaming.  Normal (prefill): 128 tokens are the A rows and BN (64..256) output
//     channels the B rows, so each epilogue thread owns one token row and writes contiguous bf16.
//   * Operands arrive by TMA (2-D tiled, 128-byte swizzle, no cluster broadcast) into a STAGES-deep
//     ring of shared-memory stages guarded by full/empty mbarriers.
//   * One elected thread issues tcgen05.mma.kind::i8 (128 x BN x 32 per instruction); the int32
//     accumulator lives in TMEM and is double buffered so the epilogue of one tile overlaps the
//     main loop of the next.
//   * Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2..5 = epilogue
//     (each reads its 32-lane quarter of TMEM with tcgen05.ld).
//   * Persistent grid.  Work is the list of (tile, k-block) units.  Large problems give each CTA whole
//     tiles round-robin, rasterised so that concurrently running CTAs share token panels in L2.
//     Small-M problems (decode) use a stream-K split: every CTA gets an equal share of k-blocks; a CTA
//     that covers only part of a tile's K range stores its int32 partial into its own slab of a scratch
//     buffer (plain coalesced stores), and the last CTA to arrive for the tile sums the slabs exactly,
//     applies the scales and writes the output.
//   * Every mbarrier wait is bounded; on a timeout the CTA records a status code, drains and exits.
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include "gemm_common.cuh"

namespace b200 {

constexpr int GROUP_M = 8;      // token tiles per rasterisation group

struct GemmParams {
  int M, N, K;
  int m_tiles, n_tiles, kblocks, num_tiles;   // m_tiles: tiles along tokens, n_tiles: tiles along output channels
  int mode;                     // 0: whole tiles round-robin, 1: stream-K
  long long total_units;
  const float* sx;
  const float* sw;
  void* y;
  const __nv_bfloat16* residual;
  int ldy;
  int out_fp32;
  int32_t* ws;                  // stream-K partials: [num_tiles][max_segs][BN][128] int32 (mode 1); needs no zeroing
  int max_segs;
  uint32_t* counters;           // [num_tiles], zero between launches (mode 1); the finishing CTA re-zeroes
  int* status;
  unsigned long long limit_ns;
  // grouped (mixture-of-experts) form, normal orientation only: the token tiles come from a device table of
  // {expert, first row, rows, -}; *grp_meta_tiles of them are valid; expert e uses weight rows [e*N, (e+1)*N)
  const int4* grp_tiles;
  const int* grp_num_tiles;
};

struct Seg { int tile, kb0, kb1; };

struct WorkIter {
  int mode, next_tile, stride, num_tiles, kblocks;
  long long u, u_end;
  __device__ WorkIter(const GemmParams& p) {
    mode = p.mode; kblocks = p.kblocks;
    num_tiles = p.grp_tiles ? (*p.grp_num_tiles) * p.n_tiles : p.num_tiles;
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

// index of the CTA whose unit range [U*c/G, U*(c+1)/G) contains unit u
__device__ __forceinline__ int cta_of_unit(long long u, long long total_units, int grid) {
  int c = static_cast<int>(u * grid / total_units);
  while (c + 1 < grid && total_units * (c + 1) / grid <= u) ++c;
  return c;
}

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& m_tile, int& n_tile) {
  if (p.grp_tiles) { m_tile = tile / p.n_tiles; n_tile = tile - m_tile * p.n_tiles; return; }
  const int per_group = GROUP_M * p.n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(GROUP_M, p.m_tiles - first_m);
  const int r = tile - g * per_group;
  m_tile = first_m + r % gsize;
  n_tile = r / gsize;
}

// tmap_a covers the operand whose 128-row tiles fill the MMA M dimension (weights when SWAP, tokens otherwise),
// tmap_b the operand whose BN-row tiles fill the MMA N dimension.
template <int BN, int STAGES, bool SWAP>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

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
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      // weights streamed once (single token tile) should not displace anything; otherwise keep them
      const uint64_t pol_w = (p.m_tiles == 1) ? policy_evict_first() : policy_evict_last();
      WorkIter it(p);
      Seg sg;
      int stage = 0; uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      while (ok && it.next(sg)) {
        int m_tile, n_tile;
        tile_coords(p, sg.tile, m_tile, n_tile);
        int row0 = m_tile * TILE_N, wrow0 = 0;
        if (p.grp_tiles) { const int4 tt = p.grp_tiles[m_tile]; row0 = tt.y; wrow0 = tt.x * p.N; }
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (1 << 8)), limit)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          if constexpr (SWAP) {
            tma_load_2d_hint(a_dst, &tmap_a, full_bar(stage), kb * BLOCK_K, n_tile * TILE_N, pol_w);
            tma_load_2d(a_dst + A_BYTES, &tmap_b, full_bar(stage), kb * BLOCK_K, m_tile * BN);
          } else {
            tma_load_2d(a_dst, &tmap_a, full_bar(stage), kb * BLOCK_K, row0);
            tma_load_2d_hint(a_dst + A_BYTES, &tmap_b, full_bar(stage), kb * BLOCK_K, wrow0 + n_tile * BN, pol_w);
          }
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
        if (!mbar_wait(tempty_bar(a), aphase ^ 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_EMPTY | (1 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (1 << 8)), limit)) { ok = false; break; }
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
      if (!mbar_wait(tfull_bar(a), aphase, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (1 << 8)), limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * BN;
      const bool whole = (sg.kb0 == 0 && sg.kb1 == p.kblocks);
      constexpr int CH = (BN >= 32) ? 32 : 16;

      if constexpr (!SWAP) {
        // ---- normal orientation: this thread owns token row m and walks BN output channels ----
        int m = m_tile * TILE_N + q * 32 + lane;
        bool m_ok = m < p.M;
        const float* swg = p.sw;
        if (p.grp_tiles) {
          const int4 tt = p.grp_tiles[m_tile];
          m = tt.y + q * 32 + lane;
          m_ok = (q * 32 + lane) < tt.z;
          swg = p.sw + static_cast<size_t>(tt.x) * p.N;
        }
        const float sxm = m_ok ? p.sx[m] : 0.f;
        const int n0 = n_tile * BN;
        const size_t row_off = static_cast<size_t>(m_ok ? m : 0) * p.ldy;
        const bool vec_ok = !p.out_fp32 && (p.ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) &&
                            (!p.residual || (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_x32(t_addr + c * 32, r);
          tmem_ld_wait();
          const int nc = n0 + c * 32;
          if (vec_ok && nc + 32 <= p.N) {
            const float4* swp = reinterpret_cast<const float4*>(swg + nc);
            uint4 packed[4];
            uint32_t* pk = reinterpret_cast<uint32_t*>(packed);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const float4 w4 = __ldg(swp + g);
              const float f0 = static_cast<float>(static_cast<int32_t>(r[4 * g + 0])) * (w4.x * sxm);
              const float f1 = static_cast<float>(static_cast<int32_t>(r[4 * g + 1])) * (w4.y * sxm);
              const float f2 = static_cast<float>(static_cast<int32_t>(r[4 * g + 2])) * (w4.z * sxm);
              const float f3 = static_cast<float>(static_cast<int32_t>(r[4 * g + 3])) * (w4.w * sxm);
              __nv_bfloat162 lo = __floats2bfloat162_rn(f0, f1), hi = __floats2bfloat162_rn(f2, f3);
              pk[2 * g] = *reinterpret_cast<uint32_t*>(&lo);
              pk[2 * g + 1] = *reinterpret_cast<uint32_t*>(&hi);
            }
            if (m_ok) {
              __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(p.y) + row_off + nc;
              if (p.residual) {
                const uint4* rp = reinterpret_cast<const uint4*>(p.residual + row_off + nc);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint4 rv = rp[g];
                  const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
                  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&packed[g]);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 x = __bfloat1622float2(ob[e]), y2 = __bfloat1622float2(rb[e]);
                    ob[e] = __floats2bfloat162_rn(x.x + y2.x, x.y + y2.y);
                  }
                }
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) reinterpret_cast<uint4*>(yp)[g] = packed[g];
            }
          } else if (m_ok) {
            for (int j = 0; j < 32; ++j) {
              const int n = nc + j;
              if (n >= p.N) break;
              float v = static_cast<float>(static_cast<int32_t>(r[j])) * sxm * __ldg(swg + n);
              const size_t o = row_off + n;
              if (p.residual) v += __bfloat162float(p.residual[o]);
              if (p.out_fp32) reinterpret_cast<float*>(p.y)[o] = v;
              else reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16(v);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(a));
      } else {
        // ---- swapped orientation: this thread owns output channel n and walks BN tokens ----
        const int n = n_tile * TILE_N + q * 32 + lane;
        const bool n_ok = n < p.N;
        const int m0 = m_tile * BN;
        const float swn = n_ok ? __ldg(p.sw + n) : 0.f;
        int nseg = 1;
        int32_t* slab = nullptr;
        if (!whole) {
          const long long u_first = static_cast<long long>(sg.tile) * p.kblocks;
          const int c_first = cta_of_unit(u_first, p.total_units, gridDim.x);
          const int c_last = cta_of_unit(u_first + p.kblocks - 1, p.total_units, gridDim.x);
          nseg = c_last - c_first + 1;
          slab = p.ws + (static_cast<size_t>(sg.tile) * p.max_segs + (blockIdx.x - c_first)) * (BN * TILE_N);
        }
#pragma unroll 1
        for (int c = 0; c < BN / CH; ++c) {
          uint32_t r[CH];
          if constexpr (CH == 32) tmem_ld_x32(t_addr + c * CH, r); else tmem_ld_x16(t_addr + c * CH, r);
          tmem_ld_wait();
          const int mc = m0 + c * CH;
          const int jmax = min(CH, p.M - mc);
          if (!n_ok || jmax <= 0) continue;
          if (whole) {
            const float* sxp = p.sx + mc;
            const size_t o0 = static_cast<size_t>(mc) * p.ldy + n;
            if (p.out_fp32) {
              float* yp = reinterpret_cast<float*>(p.y) + o0;
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                if (j < jmax) {
                  float v = static_cast<float>(static_cast<int32_t>(r[j])) * swn * sxp[j];
                  if (p.residual) v += __bfloat162float(p.residual[o0 + static_cast<size_t>(j) * p.ldy]);
                  yp[static_cast<size_t>(j) * p.ldy] = v;
                }
              }
            } else {
              __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(p.y) + o0;
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                if (j < jmax) {
                  float v = static_cast<float>(static_cast<int32_t>(r[j])) * swn * sxp[j];
                  if (p.residual) v += __bfloat162float(p.residual[o0 + static_cast<size_t>(j) * p.ldy]);
                  yp[static_cast<size_t>(j) * p.ldy] = __float2bfloat16(v);
                }
              }
            }
          } else {
            // partial K range: park the int32 partial in this CTA's slab, [token][channel] so warps store 128 B rows
            int32_t* sp = slab + static_cast<size_t>(c * CH) * TILE_N + (q * 32 + lane);
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (j < jmax) __stcg(sp + j * TILE_N, static_cast<int32_t>(r[j]));
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
            const uint32_t old = atomicAdd(p.counters + sg.tile, 1u);
            *fix_slot = (old + 1u == static_cast<uint32_t>(nseg)) ? 1 : 0;
          }
          named_bar_sync(1, 128);
          const int last = *fix_slot;
          named_bar_sync(1, 128);     // everyone has read fix_slot before it can be rewritten
          if (last) {
            __threadfence();
            if (n_ok) {
              const int jmax = min(BN, p.M - m0);
              const int32_t* s0 = p.ws + static_cast<size_t>(sg.tile) * p.max_segs * (BN * TILE_N) + (q * 32 + lane);
              for (int j = 0; j < jmax; ++j) {
                int32_t acc = 0;
                for (int sgi = 0; sgi < nseg; ++sgi) acc += __ldcg(s0 + static_cast<size_t>(sgi) * (BN * TILE_N) + j * TILE_N);
                const int m = m0 + j;
                float v = static_cast<float>(acc) * swn * p.sx[m];
                const size_t o = static_cast<size_t>(m) * p.ldy + n;
                if (p.residual) v += __bfloat162float(p.residual[o]);
                if (p.out_fp32) reinterpret_cast<float*>(p.y)[o] = v;
                else reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16(v);
              }
            }
            if (et == 0) p.counters[sg.tile] = 0;
          }
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

template <int BN, int STAGES, bool SWAP>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (TILE_N * BLOCK_K + BN * BLOCK_K) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_gemm_kernel<BN, STAGES, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(w8a8_gemm_kernel<BN, STAGES, SWAP>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  launch_ex(w8a8_gemm_kernel<BN, STAGES, SWAP>, dim3(grid), dim3(GEMM_THREADS), SMEM, stream, 0, ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}


// token-tile width (swapped) or channel-tile width (normal)
int gemm_pick_bn(int M, int N, int num_sms) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= SWAP_MAX_M) return 64;
  const int m_tiles = (M + TILE_N - 1) / TILE_N;
  // rounds of the persistent grid times the cost of one tile (main loop ~ bn, plus a fixed part)
  int best = 256;
  long long best_cost = -1;
  for (int bn : {256, 128, 64}) {
    const long long tiles = static_cast<long long>(m_tiles) * ((N + bn - 1) / bn);
    const long long rounds = (tiles + num_sms - 1) / num_sms;
    const long long cost = rounds * (bn + 64);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace b200

using namespace b200;

// grid and slab count of the stream-K schedule for a swapped-orientation problem
static void streamk_plan(long long total_units, int kblocks, int num_sms, int* grid, int* max_segs) {
  long long g = total_units / 4;          // at least ~4 k-blocks per CTA
  if (g < 1) g = 1;
  if (g > num_sms) g = num_sms;
  *grid = static_cast<int>(g);
  const long long min_units = total_units / g;                 // every CTA gets at least this many units
  *max_segs = static_cast<int>((kblocks + min_units - 1) / (min_units > 0 ? min_units : 1)) + 1;
}

extern "C" size_t b200_w8a8_gemm_ws_bytes(int M, int N, int K, int num_sms) {
  if (M > SWAP_MAX_M) return 0;
  const int bn = gemm_pick_bn(M, N, num_sms);
  const long long tiles = static_cast<long long>((M + bn - 1) / bn) * ((N + TILE_N - 1) / TILE_N);
  const int kblocks = (K + BLOCK_K - 1) / BLOCK_K;
  int grid, max_segs;
  streamk_plan(tiles * kblocks, kblocks, num_sms, &grid, &max_segs);
  return static_cast<size_t>(tiles) * max_segs * bn * TILE_N * sizeof(int32_t);
}

extern "C" int b200_w8a8_gemm(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                              const void* residual, int M, int N, int K, int ldy, int out_fp32,
                              void* ws, size_t ws_bytes, void* counters, int counters_len, int* status,
                              int num_sms, int force_mode, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 16) != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15)) return -2;
  const bool swap = M <= SWAP_MAX_M;
  const int bn = gemm_pick_bn(M, N, num_sms);
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = swap ? (M + bn - 1) / bn : (M + TILE_N - 1) / TILE_N;
  p.n_tiles = swap ? (N + TILE_N - 1) / TILE_N : (N + bn - 1) / bn;
  p.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
  p.num_tiles = p.m_tiles * p.n_tiles;
  p.total_units = static_cast<long long>(p.num_tiles) * p.kblocks;
  p.sx = sx; p.sw = sw; p.y = y; p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldy = ldy; p.out_fp32 = out_fp32;
  p.ws = static_cast<int32_t*>(ws);
  p.max_segs = 1;
  p.counters = static_cast<uint32_t*>(counters);
  p.status = status;
  p.limit_ns = 2000000000ull;
  p.grp_tiles = nullptr;
  p.grp_num_tiles = nullptr;

  int mode = 0;
  int sk_grid = 1;
  if (swap) {
    streamk_plan(p.total_units, p.kblocks, num_sms, &sk_grid, &p.max_segs);
    const size_t need_ws = static_cast<size_t>(p.num_tiles) * p.max_segs * bn * TILE_N * sizeof(int32_t);
    const bool can_split = ws && counters && ws_bytes >= need_ws && counters_len >= p.num_tiles;
    if (force_mode == 0 || force_mode == 1) mode = force_mode;
    else mode = (p.num_tiles < 4 * num_sms) ? 1 : 0;
    if (mode == 1 && !can_split) mode = 0;
  }
  p.mode = mode;
  int grid;
  if (mode == 0) {
    grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  } else {
    grid = sk_grid;
  }

  CUtensorMap tw, tx;
  if (make_tmap_2d_u8(&tw, wq, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), swap ? TILE_N : bn)) return -11;
  if (make_tmap_2d_u8(&tx, xq, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), swap ? bn : TILE_N)) return -12;

  if (swap) {
    switch (bn) {
      case 16: return launch_gemm<16, 8, true>(tw, tx, p, grid, stream);
      case 32: return launch_gemm<32, 8, true>(tw, tx, p, grid, stream);
      default: return launch_gemm<64, 8, true>(tw, tx, p, grid, stream);
    }
  }
  switch (bn) {
    case 64: return launch_gemm<64, 8, false>(tx, tw, p, grid, stream);
    case 128: return launch_gemm<128, 6, false>(tx, tw, p, grid, stream);
    default: return launch_gemm<256, 4, false>(tx, tw, p, grid, stream);
  }
}

// Grouped form for mixture-of-experts prefill: xq [x_rows][K] holds the tokens in slot order, `tiles` (device, int4
// {expert, first row, rows <= 128, -}) lists the 128-row token tiles and *num_tiles how many are valid (at most
// max_tiles); expert e multiplies by wq[e*N : (e+1)*N].  N must be a multiple of 256.  Nothing syncs the host.
extern "C" int b200_w8a8_gemm_grouped(const void* xq, const float* sx, const void* wq, const float* sw, void* y, int x_rows,
                                      int N, int K, int ldy, int groups, const void* tiles, const int* num_tiles,
                                      int max_tiles, int* status, int num_sms, cudaStream_t stream) {
  if (x_rows <= 0 || N <= 0 || K <= 0 || (K % 16) || (N % 256) || groups <= 0 || max_tiles <= 0) return -1;
  GemmParams p;
  p.M = x_rows; p.N = N; p.K = K;
  p.m_tiles = max_tiles;
  p.n_tiles = N / 256;
  p.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
  p.num_tiles = max_tiles * p.n_tiles;
  p.total_units = static_cast<long long>(p.num_tiles) * p.kblocks;
  p.mode = 0;
  p.sx = sx; p.sw = sw; p.y = y; p.residual = nullptr; p.ldy = ldy; p.out_fp32 = 0;
  p.ws = nullptr; p.max_segs = 1; p.counters = nullptr; p.status = status; p.limit_ns = 2000000000ull;
  p.grp_tiles = static_cast<const int4*>(tiles);
  p.grp_num_tiles = num_tiles;
  CUtensorMap tw, tx;
  if (make_tmap_2d_u8(&tw, wq, static_cast<uint64_t>(K), static_cast<uint64_t>(groups) * N, static_cast<uint64_t>(K), 256)) return -11;
  if (make_tmap_2d_u8(&tx, xq, static_cast<uint64_t>(K), static_cast<uint64_t>(x_rows), static_cast<uint64_t>(K), TILE_N)) return -12;
  const int grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  return launch_gemm<256, 4, false>(tx, tw, p, grid, stream);
}
