// Tensor-parallel prefill forms of the W8A8 GEMM (tokens fill the MMA M dimension, see w8a8_gemm.cu for the tile
// pipeline), each ONE kernel that performs its collective over peer memory while the tensor cores run:
//
//   gather form  (column-parallel: QKV, gate|up)   Y[M, N_shard] = allgather_rows(Xq_local)[M, K] * Wq_shard^T
//     two extra "comm" warps per CTA copy this rank's R quantised rows (and their scales) into every rank's gather
//     buffer - one multimem.st per 16 bytes through the NVSwitch, or world plain peer stores - and publish one flag
//     per 128-row block; the TMA producer waits for the flags of the rows a tile needs right before loading it and the
//     tiles are walked starting with this rank's own rows, so the main loop overlaps the arrival of remote rows.
//
//   scatter form (row-parallel: o_proj, down)      out[R, N] = sum_ranks (Xq[M, K_shard] * Wq_shard^T)[my rows]
//     the epilogue stores each finished bf16 tile, re-laid through shared memory into 128-byte row segments, straight
//     into the receive slot of the rank that owns those token rows and adds the row count to that rank's arrival
//     counter; after its last tile the grid waits (bounded) for all world sources and sums the slots in rank order.
//
// No barrier, no second kernel, no library collective.  See tp_link.cuh for the buffer protocol.  The `phase` mask
// (1 tiles, 2 scatter tail, 4 gather push) exists so that a test can run several virtual ranks on one GPU as
// consecutive launches (all pushes, then all consumers): kernels that wait on each other must never be separate
// launches on one device.  Production launches use phase 7.
// The reference has no GEMM and no collective beyond the chain / butterfly sums of test_linux_threading.mojo:400-553;
// what is kept from it is the discipline of its ring reduce: a producer writes into memory the consumer can address,
// then opens a gate (threading/linux_threading.mojo:187-194).
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include "gemm_common.cuh"
#include "tp_link.cuh"

namespace b200 {

constexpr int TP_THREADS = 256;          // producer, MMA, 4 epilogue warps, 2 comm warps
constexpr int TP_GROUP_M = 8;
constexpr int TP_STG_BYTES = 4 * 4096;   // per epilogue warp: 32 rows x 128 bytes
constexpr int TP_READY_MAX = 1024;       // (source rank, 128-row block) pairs a gather may have

int gemm_pick_bn(int M, int N, int num_sms);

struct TpGemmParams {
  int M, N, K;
  int m_tiles, n_tiles, kblocks, num_tiles;
  int m_rot;                     // token tiles are visited starting at this one
  const float* sx;               // scatter / plain: per-token scales of the local operand
  const float* sw;
  void* y; int ldy;              // gather form output, bf16 [M, N]
  int gather, scatter, finish, phase;
  const int8_t* xq_local;        // gather: this rank's R quantised rows [R][K]
  const float* sx_local;         // gather: their scales
  int own_lo, own_hi;            // gather: global rows [own_lo, own_hi) are this rank's (read straight from xq_local)
  void* out; int ldo;            // scatter: bf16 [R, N]
  const __nv_bfloat16* residual; int ldr;   // optional addend of the scatter output
  int* status;
  unsigned long long limit_ns;
  AgLink ag;
  RsLink rs;
};

__device__ __forceinline__ void tp_tile_coords(const TpGemmParams& p, int tile, int& m_tile, int& n_tile) {
  const int per_group = TP_GROUP_M * p.n_tiles;
  const int g = tile / per_group;
  const int first_m = g * TP_GROUP_M;
  const int gsize = min(TP_GROUP_M, p.m_tiles - first_m);
  const int r = tile - g * per_group;
  m_tile = first_m + r % gsize + p.m_rot;
  if (m_tile >= p.m_tiles) m_tile -= p.m_tiles;
  n_tile = r / gsize;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TP_THREADS, 1)
w8a8_gemm_tp_kernel(const __grid_constant__ CUtensorMap tmap_a0, const __grid_constant__ CUtensorMap tmap_a1,
                    const __grid_constant__ CUtensorMap tmap_loc, const __grid_constant__ CUtensorMap tmap_b,
                    const TpGemmParams p) {
  // Stamps of the trace build (TK_GEMM_TP): 0 start, 1 dependency wait passed, 2 this rank's rows pushed to the peers,
  // 3 producer met a tile whose rows had not arrived (once per CTA, first time), 4 ... and they were there, 5 first tile's
  // accumulator complete, 6 last tile stored / scattered, 7 scatter tail: all partial rows have arrived, 8 tail summed,
  // 63 leaving.  Together they show how much of the exchange hides behind the tensor-core work.
  pdl_launch_dependents();
  B200_TRACE_INIT();
  if (threadIdx.x == 0) B200_TRACE(TK_GEMM_TP, TP_START);
  pdl_wait();
  if (threadIdx.x == 0) B200_TRACE(TK_GEMM_TP, TP_DEPS);

  constexpr int A_BYTES = TILE_N * BLOCK_K;
  constexpr int B_BYTES = BN * BLOCK_K;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = umma_idesc_i8(TILE_N, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stg = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg + TP_STG_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* misc_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [0] comm go-ahead, [1] tail go-ahead
  volatile uint32_t* mbox = reinterpret_cast<volatile uint32_t*>(tmem_slot + 4);   // [4] tiles stored so far, per epilogue warp
  volatile uint8_t* ready = reinterpret_cast<volatile uint8_t*>(tmem_slot + 8);    // [TP_READY_MAX] gather blocks seen complete

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
    misc_slot[0] = 0; misc_slot[1] = 0;
    for (int i = 0; i < 4; ++i) mbox[i] = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < TP_READY_MAX; i += TP_THREADS) ready[i] = 0;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint64_t limit = p.limit_ns;

  // epochs of this call (device-resident counters, advanced by the last CTA to leave)
  uint32_t ag_e = 0, rs_e = 0;
  if (p.gather) ag_e = *reinterpret_cast<volatile uint32_t*>(p.ag.words) + 1;
  if (p.scatter) rs_e = *reinterpret_cast<volatile uint32_t*>(p.rs.words) + 1;
  const int ag_par = static_cast<int>(ag_e & 1u), rs_par = static_cast<int>(rs_e & 1u);
  const float* sx = p.gather ? reinterpret_cast<const float*>(p.ag.t.data[p.ag.t.rank] + p.ag.s_off[ag_par]) : p.sx;
  const bool do_tiles = (p.phase & 1) != 0;
  const int num_tiles = do_tiles ? p.num_tiles : 0;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const CUtensorMap* ta = (p.gather && ag_par) ? &tmap_a1 : &tmap_a0;
      prefetch_tmap(ta);
      if (p.gather) prefetch_tmap(&tmap_loc);
      prefetch_tmap(&tmap_b);
      const uint64_t pol_w = policy_evict_last();
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      bool stamped_wait = false;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m_tile, n_tile;
        tp_tile_coords(p, tile, m_tile, n_tile);
        const int row0 = m_tile * TILE_N;
        // a tile made only of this rank's rows is read straight from the local operand: nothing to wait for
        const bool own = p.gather && row0 >= p.own_lo && min(row0 + TILE_N, p.M) <= p.own_hi;
        if (p.gather && !own) {
          // rows [row0, row0+128) come from source ranks s = row / R; each source publishes one flag per 128 of its
          // rows, which the comm warps of this CTA watch and mirror into shared memory
          const int R = p.ag.rows_per_rank;
          const int r_lo = row0, r_hi = min(row0 + TILE_N, p.M) - 1;
          for (int s = r_lo / R; ok && s <= r_hi / R; ++s) {
            const int a = max(r_lo, s * R) - s * R, b = min(r_hi, (s + 1) * R - 1) - s * R;
            for (int blk = a >> 7; ok && blk <= (b >> 7); ++blk) {
              const int i = s * p.ag.blk_cap + blk;
              if (ready[i]) continue;
              if (!stamped_wait) B200_TRACE(TK_GEMM_TP, 3);
              const uint64_t t0 = globaltimer_ns();
              uint32_t spins = 0;
              while (!ready[i]) {
                if ((++spins & 63u) == 0u) {
                  if (*abort_flag) { ok = false; break; }
                  if (globaltimer_ns() - t0 > limit) {
                    *abort_flag = 1;
                    if (p.status) atomicCAS(p.status, 0, (int)ST_TIMEOUT_PEER_FLAG | (3 << 8));
                    ok = false; break;
                  }
                }
              }
            }
          }
          if (!ok) break;
          if (!stamped_wait) { B200_TRACE(TK_GEMM_TP, 4); stamped_wait = true; }
          __threadfence_block();
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (3 << 8)), limit)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          if (own) tma_load_2d(a_dst, &tmap_loc, full_bar(stage), kb * BLOCK_K, row0 - p.own_lo);
          else tma_load_2d(a_dst, ta, full_bar(stage), kb * BLOCK_K, row0);
          tma_load_2d_hint(a_dst + A_BYTES, &tmap_b, full_bar(stage), kb * BLOCK_K, n_tile * BN, pol_w);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) { }      // bounded grace for copies in flight
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int seg_idx = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int a = seg_idx & 1;
        const uint32_t aphase = (seg_idx >> 1) & 1u;
        if (!mbar_wait(tempty_bar(a), aphase ^ 1u, abort_flag, p.status, (ST_TIMEOUT_TMEM_EMPTY | (3 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (3 << 8)), limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a_src);
          const uint64_t b_desc = umma_desc_k_sw128(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
            umma_i8_ss(d_tmem, a_desc + 2ull * k, b_desc + 2ull * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(a));
        ++seg_idx;
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ epilogue (4 warps) ------------------------------
    const int q = warp & 3;
    uint8_t* stg_w = stg + (warp - 2) * 4096;
    int seg_idx = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const int a = seg_idx & 1;
      const uint32_t aphase = (seg_idx >> 1) & 1u;
      int m_tile, n_tile;
      tp_tile_coords(p, tile, m_tile, n_tile);
      if (!mbar_wait(tfull_bar(a), aphase, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (3 << 8)), limit)) { ok = false; break; }
      tc_fence_after();
      if (seg_idx == 0 && threadIdx.x == 64) B200_TRACE(TK_GEMM_TP, 5);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * BN;
      const int m = m_tile * TILE_N + q * 32 + lane;
      const bool m_ok = m < p.M;
      // gathered scales were written by peers: read them past the L1
      float sxm = 0.f;
      if (m_ok) {
        if (!p.gather) sxm = sx[m];
        else if (m >= p.own_lo && m < p.own_hi) sxm = p.sx_local[m - p.own_lo];
        else sxm = __ldcg(sx + m);
      }
      const int n0 = n_tile * BN;

      // destination of the 8 rows this lane stores per 64-column chunk (after the re-layout through shared memory,
      // eight consecutive lanes store one 128-byte row segment)
      uint8_t* rowp[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int mm = m_tile * TILE_N + q * 32 + i * 4 + (lane >> 3);
        rowp[i] = nullptr;
        if (mm < p.M) {
          if (p.scatter) {
            const int R = p.rs.rows_per_rank;
            const int o = mm / R, lr = mm - o * R;
            rowp[i] = p.rs.t.data[o] + p.rs.recv_off[rs_par] +
                      (static_cast<size_t>(p.rs.t.rank) * p.rs.r_cap + lr) * p.N * 2 + (lane & 7) * 16;
          } else {
            rowp[i] = static_cast<uint8_t*>(p.y) + static_cast<size_t>(mm) * p.ldy * 2 + (lane & 7) * 16;
          }
        }
      }
#pragma unroll 1
      for (int c2 = 0; c2 < BN / 64; ++c2) {
        const int nc = n0 + c2 * 64;
        if (nc >= p.N) break;
        uint32_t r0[32], r1[32];
        tmem_ld_x32(t_addr + c2 * 64, r0);
        tmem_ld_x32(t_addr + c2 * 64 + 32, r1);
        tmem_ld_wait();
        const float4* swp = reinterpret_cast<const float4*>(p.sw + nc);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // 16-byte chunk j of this row = columns nc + 8j .. nc + 8j + 7
          const uint32_t* src = (j < 4) ? (r0 + 8 * j) : (r1 + 8 * (j - 4));
          const float4 wa = __ldg(swp + 2 * j), wb = __ldg(swp + 2 * j + 1);
          const float f0 = static_cast<float>(static_cast<int32_t>(src[0])) * (wa.x * sxm);
          const float f1 = static_cast<float>(static_cast<int32_t>(src[1])) * (wa.y * sxm);
          const float f2 = static_cast<float>(static_cast<int32_t>(src[2])) * (wa.z * sxm);
          const float f3 = static_cast<float>(static_cast<int32_t>(src[3])) * (wa.w * sxm);
          const float f4 = static_cast<float>(static_cast<int32_t>(src[4])) * (wb.x * sxm);
          const float f5 = static_cast<float>(static_cast<int32_t>(src[5])) * (wb.y * sxm);
          const float f6 = static_cast<float>(static_cast<int32_t>(src[6])) * (wb.z * sxm);
          const float f7 = static_cast<float>(static_cast<int32_t>(src[7])) * (wb.w * sxm);
          __nv_bfloat162 b0 = __floats2bfloat162_rn(f0, f1), b1 = __floats2bfloat162_rn(f2, f3);
          __nv_bfloat162 b2 = __floats2bfloat162_rn(f4, f5), b3 = __floats2bfloat162_rn(f6, f7);
          uint4 v;
          v.x = *reinterpret_cast<uint32_t*>(&b0); v.y = *reinterpret_cast<uint32_t*>(&b1);
          v.z = *reinterpret_cast<uint32_t*>(&b2); v.w = *reinterpret_cast<uint32_t*>(&b3);
          *reinterpret_cast<uint4*>(stg_w + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3);
          const uint4 v = *reinterpret_cast<const uint4*>(stg_w + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
          if (rowp[i]) *reinterpret_cast<uint4*>(rowp[i] + static_cast<size_t>(nc) * 2) = v;
        }
        __syncwarp();
      }
      // accumulator drained: hand the TMEM buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(a));

      if (p.scatter) {
        // hand the "stores of this tile are issued" event to the signalling thread of the comm warps: the system-scope
        // fence that must precede the arrival count then never stalls this warp
        __syncwarp();
        if (lane == 0) { __threadfence_block(); mbox[warp - 2] = static_cast<uint32_t>(seg_idx + 1); }
      }
      ++seg_idx;
    }
  } else {
    // ------------------------------ comm warps ------------------------------
    const int ct = threadIdx.x - 192;                  // 0..63
    if (p.gather) {
      const AgLink& g = p.ag;
      const PeerTable& t = g.t;
      const int R = g.rows_per_rank;
      if (p.phase & 4) {
        // ---- push my rows into every rank's gather buffer ----
        const int my_rows = max(0, min(R, p.M - t.rank * R));
        if (ct == 0) {
          // the buffer of this parity was last used two calls ago: every consumer must have finished that call
          const uint32_t* done = reinterpret_cast<const uint32_t*>(t.data[t.rank] + g.done_off);
          int good = 1;
          for (int r = 0; r < t.world && good; ++r)
            if (!wait_flag_ge(done + r, ag_e - 2u, p.status, limit)) good = 0;
          misc_slot[0] = good;
        }
        named_bar_sync(2, 64);
        const bool go = misc_slot[0] != 0;
        const size_t vec_per_row = static_cast<size_t>(p.K) / 16;
        const size_t row_base = static_cast<size_t>(t.rank) * R;
        const int nblk = (my_rows + 127) >> 7;
        // the CTAs split into nblk groups, one per 128-row block, so that each CTA pays for one system-scope fence
        const int G = static_cast<int>(gridDim.x);
        const int members = nblk > 0 && nblk <= G ? G / nblk : 1;
        const int first = nblk <= G ? static_cast<int>(blockIdx.x) / members : static_cast<int>(blockIdx.x);
        const int step = nblk <= G ? nblk : G;
        const size_t mtid = static_cast<size_t>(nblk <= G ? static_cast<int>(blockIdx.x) % members : 0) * 64 + ct;
        const size_t msz = static_cast<size_t>(members) * 64;
        for (int blk = first; blk < nblk; blk += step) {
          const int rows_b = min(128, my_rows - blk * 128);
          if (go) {
            const size_t v_end = static_cast<size_t>(rows_b) * vec_per_row;
            const uint4* src = reinterpret_cast<const uint4*>(p.xq_local + static_cast<size_t>(blk) * 128 * p.K);
            const size_t dst0 = g.q_off[ag_par] + (row_base + static_cast<size_t>(blk) * 128) * p.K;
            size_t v = mtid;
            for (; v + 7 * msz < v_end; v += 8 * msz) {     // eight independent 16-byte copies in flight
              uint4 x[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) x[u] = src[v + u * msz];
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const size_t off = dst0 + (v + u * msz) * 16;
                if (t.mc) multimem_st_16B(t.mc + off, x[u]);
                else for (int r = 0; r < t.world; ++r) *reinterpret_cast<uint4*>(t.data[r] + off) = x[u];
              }
            }
            for (; v < v_end; v += msz) {
              const uint4 x = src[v];
              const size_t off = dst0 + v * 16;
              if (t.mc) multimem_st_16B(t.mc + off, x);
              else for (int r = 0; r < t.world; ++r) *reinterpret_cast<uint4*>(t.data[r] + off) = x;
            }
            for (size_t i = mtid; i < static_cast<size_t>(rows_b); i += msz) {
              const float sc = p.sx_local[blk * 128 + i];
              const size_t off = g.s_off[ag_par] + (row_base + blk * 128 + i) * 4;
              for (int r = 0; r < t.world; ++r) *reinterpret_cast<float*>(t.data[r] + off) = sc;
            }
          }
          named_bar_sync(2, 64);
          if (ct == 0 && go) {
            fence_acq_rel_sys();
            const uint32_t old = atomicAdd(g.row_ctr + blk, 1u);
            if (old == static_cast<uint32_t>(members) - 1u) {   // every CTA of the block's group has stored its share
              g.row_ctr[blk] = 0;
              fence_acq_rel_sys();
              for (int r = 0; r < t.world; ++r)
                st_release_sys(reinterpret_cast<uint32_t*>(t.data[r] + g.flag_off) + t.rank * g.blk_cap + blk, ag_e);
            }
          }
        }
        if (ct == 0) B200_TRACE(TK_GEMM_TP, 2);
      }
      if (do_tiles) {
        // ---- watch the arrival flags (sources visited starting with this rank) and mirror them into shared memory ----
        const uint32_t* flags = reinterpret_cast<const uint32_t*>(t.data[t.rank] + g.flag_off);
        const int total = t.world * g.blk_cap;
        for (int j = ct; j < total; j += 64) {
          const int sj = j / g.blk_cap, blk = j - sj * g.blk_cap;
          int s = sj + t.rank;
          if (s >= t.world) s -= t.world;
          const int rows_s = max(0, min(R, p.M - s * R));
          if (blk * 128 >= rows_s) continue;
          if (*abort_flag) break;
          if (!wait_flag_ge(flags + s * g.blk_cap + blk, ag_e, p.status, limit)) { *abort_flag = 1; break; }
          __threadfence_block();
          ready[s * g.blk_cap + blk] = 1;
        }
      }
    }
    if (p.scatter && do_tiles && ct < 4) {
      // ---- one signalling thread per epilogue warp: fence, then add the delivered rows to the owners' counters ----
      const int q = (ct + 2) & 3;                        // TMEM lane quarter of epilogue warp ct + 2
      const int R = p.rs.rows_per_rank;
      uint32_t seq = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++seq) {
        const uint64_t t0 = globaltimer_ns();
        uint32_t spins = 0;
        while (mbox[ct] <= seq) {
          if ((++spins & 63u) == 0u) {
            if (*abort_flag) { ok = false; break; }
            if (globaltimer_ns() - t0 > limit) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0, (int)ST_TIMEOUT_DRAIN | (3 << 8));
              ok = false; break;
            }
          }
        }
        if (!ok) break;
        __threadfence_block();
        int m_tile, n_tile;
        tp_tile_coords(p, tile, m_tile, n_tile);
        const int m0 = m_tile * TILE_N + q * 32, m1 = min(m0 + 32, p.M);
        if (m0 < m1) {
          // red.release.sys orders the tile's stores (observed through the mailbox) before the count
          for (int o = m0 / R; o <= (m1 - 1) / R; ++o) {
            const int cnt = min(m1, (o + 1) * R) - max(m0, o * R);
            red_release_sys_add(reinterpret_cast<uint32_t*>(p.rs.t.data[o] + p.rs.ctr_off) + rs_par, static_cast<uint32_t>(cnt));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) B200_TRACE(TK_GEMM_TP, 6);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }

  // ------------------------------ scatter tail: sum the world receive slots of my rows ------------------------------
  if (p.scatter && (p.phase & 2)) {
    const RsLink& s = p.rs;
    const PeerTable& t = s.t;
    const int R = s.rows_per_rank;
    const int my_rows = max(0, min(R, p.M - t.rank * R));
    if (threadIdx.x == 0) {
      const uint32_t expected = static_cast<uint32_t>(t.world) * my_rows * p.n_tiles;
      int good = *abort_flag ? 0 : 1;
      if (good && my_rows > 0)
        good = wait_flag_ge(reinterpret_cast<const uint32_t*>(t.data[t.rank] + s.ctr_off) + rs_par, expected, p.status, limit) ? 1 : 0;
      misc_slot[1] = good;
      B200_TRACE(TK_GEMM_TP, 7);
    }
    __syncthreads();
    if (misc_slot[1]) {
      const size_t vec_per_row = static_cast<size_t>(p.N) / 8;
      const size_t total = static_cast<size_t>(my_rows) * vec_per_row;
      const size_t src_stride = static_cast<size_t>(s.r_cap) * p.N * 2;
      const uint8_t* base = t.data[t.rank] + s.recv_off[rs_par];
      const size_t gsz = static_cast<size_t>(gridDim.x) * TP_THREADS;
      auto addr = [&](size_t v) { const size_t row = v / vec_per_row, c8 = v - row * vec_per_row; return base + (row * p.N + c8 * 8) * 2; };
      auto finish = [&](size_t v, const uint4 (&x)[MAX_RANKS]) {
        const size_t row = v / vec_per_row, c8 = v - row * vec_per_row;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) if (r < t.world) add_bf16x8_to_f32(x[r], acc);
        if (p.residual) add_bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.residual + row * p.ldr + c8 * 8), acc);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + row * p.ldo + c8 * 8) = pack_f32x8_to_bf16(acc);
      };
      size_t v = static_cast<size_t>(blockIdx.x) * TP_THREADS + threadIdx.x;
      for (; v + gsz < total; v += 2 * gsz) {              // two vectors x world sources in flight per thread
        const uint8_t* a0 = addr(v);
        const uint8_t* a1 = addr(v + gsz);
        uint4 x0[MAX_RANKS], x1[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) if (r < t.world) { x0[r] = ld_peer_16B(a0 + r * src_stride); x1[r] = ld_peer_16B(a1 + r * src_stride); }
        finish(v, x0);
        finish(v + gsz, x1);
      }
      for (; v < total; v += gsz) {
        const uint8_t* a0 = addr(v);
        uint4 x0[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) if (r < t.world) x0[r] = ld_peer_16B(a0 + r * src_stride);
        finish(v, x0);
      }
    }
  }

  // ------------------------------ last CTA out: advance the epochs ------------------------------
  __syncthreads();
  if (threadIdx.x == 0 && p.scatter && (p.phase & 2)) B200_TRACE(TK_GEMM_TP, 8);
  if (threadIdx.x == 0) {
    uint32_t* exit_ctr = p.gather ? p.ag.words + 1 : p.rs.words + 1;
    __threadfence();
    const uint32_t old = atomicAdd(exit_ctr, 1u);
    if (old == gridDim.x - 1) {
      *exit_ctr = 0;
      if (p.scatter && (p.phase & 2)) {
        reinterpret_cast<uint32_t*>(p.rs.t.data[p.rs.t.rank] + p.rs.ctr_off)[rs_par] = 0;
        p.rs.words[0] = rs_e;
      }
      if (p.gather && p.finish && (p.phase & 1)) {
        // every CTA has finished reading the gather buffer of this epoch
        __threadfence_system();
        for (int r = 0; r < p.ag.t.world; ++r)
          st_relaxed_sys(reinterpret_cast<uint32_t*>(p.ag.t.data[r] + p.ag.done_off) + p.ag.t.rank, ag_e);
        p.ag.words[0] = ag_e;
      }
      __threadfence();
    }
    B200_TRACE(TK_GEMM_TP, TP_EXIT);
  }
  B200_TRACE_FLUSH(TK_GEMM_TP);
}

// Ends an epoch of the gather buffer without a consuming GEMM of this file (its readers were other kernels launched
// before this one in the stream): acknowledges to every rank and advances the epoch.  wait != 0 first waits for all
// blocks of all sources, which makes the whole buffer readable by ordinary kernels launched after this one.
__global__ void __launch_bounds__(256) ag_sync_kernel(const AgLink g, int M, int wait, int finish) {
  pdl_launch_dependents();
  pdl_wait();
  const PeerTable& t = g.t;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(g.words) + 1;
  __shared__ int good;
  if (threadIdx.x == 0) good = 1;
  __syncthreads();
  if (wait) {
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(t.data[t.rank] + g.flag_off);
    const int R = g.rows_per_rank;
    for (int i = threadIdx.x; i < t.world * g.blk_cap; i += blockDim.x) {
      const int s = i / g.blk_cap, blk = i - s * g.blk_cap;
      const int rows_s = max(0, min(R, M - s * R));
      if (blk * 128 < rows_s && !wait_flag_ge(flags + i, e, g.status, g.limit_ns)) good = 0;
    }
  }
  __syncthreads();
  if (finish && good && threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < t.world; ++r) st_relaxed_sys(reinterpret_cast<uint32_t*>(t.data[r] + g.done_off) + t.rank, e);
    g.words[0] = e;
    __threadfence();
  }
}

template <int BN, int STAGES>
static int launch_tp(const CUtensorMap& ta0, const CUtensorMap& ta1, const CUtensorMap& tl, const CUtensorMap& tb,
                     const TpGemmParams& p, int grid, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (TILE_N * BLOCK_K + BN * BLOCK_K) + TP_STG_BYTES + 1024 + 256 + TP_READY_MAX;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_gemm_tp_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(w8a8_gemm_tp_kernel<BN, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  launch_ex(w8a8_gemm_tp_kernel<BN, STAGES>, dim3(grid), dim3(TP_THREADS), SMEM, stream, 0, ta0, ta1, tl, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

static void fill_table(PeerTable& t, void* const* peer_data, void* mc_base, int world, int rank) {
  for (int r = 0; r < MAX_RANKS; ++r) {
    t.data[r] = r < world ? static_cast<uint8_t*>(peer_data[r]) : nullptr;
    t.flags[r] = nullptr;
  }
  t.mc = static_cast<uint8_t*>(mc_base); t.world = world; t.rank = rank;
}

static int run_tp(const CUtensorMap& ta0, const CUtensorMap& ta1, const CUtensorMap& tl, const void* wq, TpGemmParams& p, int num_sms,
                  cudaStream_t stream) {
  const int bn = gemm_pick_bn(p.M, p.N, num_sms);
  p.m_tiles = (p.M + TILE_N - 1) / TILE_N;
  p.n_tiles = (p.N + bn - 1) / bn;
  p.kblocks = (p.K + BLOCK_K - 1) / BLOCK_K;
  p.num_tiles = p.m_tiles * p.n_tiles;
  CUtensorMap tw;
  if (make_tmap_2d_u8(&tw, wq, static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.N), static_cast<uint64_t>(p.K), bn)) return -11;
  // every SM takes part in the push / the tail even when there are fewer tiles than SMs
  switch (bn) {
    case 64: return launch_tp<64, 8>(ta0, ta1, tl, tw, p, num_sms, stream);
    case 128: return launch_tp<128, 6>(ta0, ta1, tl, tw, p, num_sms, stream);
    default: return launch_tp<256, 4>(ta0, ta1, tl, tw, p, num_sms, stream);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_w8a8_gemm_ag(const void* xq_local, const float* sx_local, const void* wq, const float* sw, void* y,
                                 int M, int N, int K, int ldy, int rows_per_rank, void* const* peer_data, void* mc_base,
                                 int world, int rank, size_t q_off0, size_t q_off1, size_t s_off0, size_t s_off1,
                                 size_t flag_off, size_t done_off, int blk_cap, int m_cap, void* words, void* row_ctr,
                                 int finish, int phase, int* status, int limit_ms, int num_sms, cudaStream_t stream) {
  if (M <= 64 || N <= 0 || K <= 0 || (K % 128) || (N % 64) || (ldy % 8) || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || static_cast<long long>(rows_per_rank) * world < M || M > m_cap) return -1;
  if ((rows_per_rank + 127) / 128 > blk_cap || world * blk_cap > TP_READY_MAX) return -1;
  if ((q_off0 | q_off1) % 1024 || (s_off0 | s_off1 | flag_off | done_off) % 16) return -2;
  if ((reinterpret_cast<uintptr_t>(xq_local) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(y)) & 15) return -2;
  TpGemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.sx = nullptr; p.sw = sw; p.y = y; p.ldy = ldy;
  p.gather = 1; p.scatter = 0; p.finish = finish; p.phase = phase;
  p.xq_local = static_cast<const int8_t*>(xq_local); p.sx_local = sx_local;
  p.status = status;
  p.limit_ns = static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull;
  fill_table(p.ag.t, peer_data, mc_base, world, rank);
  p.ag.q_off[0] = q_off0; p.ag.q_off[1] = q_off1; p.ag.s_off[0] = s_off0; p.ag.s_off[1] = s_off1;
  p.ag.flag_off = flag_off; p.ag.done_off = done_off;
  p.ag.words = static_cast<uint32_t*>(words); p.ag.row_ctr = static_cast<uint32_t*>(row_ctr);
  p.ag.blk_cap = blk_cap; p.ag.rows_per_rank = rows_per_rank; p.ag.status = status; p.ag.limit_ns = p.limit_ns;
  p.m_rot = (rank * rows_per_rank) / TILE_N;              // start with the tile that holds my first row
  const int m_tiles = (M + TILE_N - 1) / TILE_N;
  if (p.m_rot >= m_tiles) p.m_rot = 0;
  CUtensorMap ta0, ta1;
  const uint8_t* mine = static_cast<const uint8_t*>(peer_data[rank]);
  if (make_tmap_2d_u8(&ta0, mine + q_off0, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), TILE_N)) return -12;
  if (make_tmap_2d_u8(&ta1, mine + q_off1, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), TILE_N)) return -12;
  // this rank's own rows, read without waiting for anything
  p.own_lo = rank * rows_per_rank < M ? rank * rows_per_rank : M;
  p.own_hi = p.own_lo + rows_per_rank < M ? p.own_lo + rows_per_rank : M;
  CUtensorMap tl = ta0;
  if (p.own_hi > p.own_lo &&
      make_tmap_2d_u8(&tl, xq_local, static_cast<uint64_t>(K), static_cast<uint64_t>(p.own_hi - p.own_lo), static_cast<uint64_t>(K), TILE_N)) return -12;
  return run_tp(ta0, ta1, tl, wq, p, num_sms, stream);
}

extern "C" int b200_w8a8_gemm_rs(const void* xq, const float* sx, const void* wq, const float* sw, void* out,
                                 const void* residual, int M, int N, int K, int ldo, int ldr, int rows_per_rank,
                                 void* const* peer_data, int world, int rank, size_t recv_off0, size_t recv_off1,
                                 size_t ctr_off, int r_cap, void* words, int phase, int* status, int limit_ms, int num_sms,
                                 cudaStream_t stream) {
  if (M <= 64 || N <= 0 || K <= 0 || (K % 16) || (N % 64) || (ldo % 8) || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank > r_cap || static_cast<long long>(rows_per_rank) * world < M) return -1;
  if ((recv_off0 | recv_off1 | ctr_off) % 16) return -2;
  if ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  if (residual && ((reinterpret_cast<uintptr_t>(residual) & 15) || (ldr % 8))) return -2;
  TpGemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.sx = sx; p.sw = sw; p.y = nullptr; p.ldy = 0;
  p.gather = 0; p.scatter = 1; p.finish = 0; p.phase = phase;
  p.out = out; p.ldo = ldo; p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.status = status;
  p.limit_ns = static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull;
  fill_table(p.rs.t, peer_data, nullptr, world, rank);
  p.rs.recv_off[0] = recv_off0; p.rs.recv_off[1] = recv_off1; p.rs.ctr_off = ctr_off;
  p.rs.words = static_cast<uint32_t*>(words); p.rs.r_cap = r_cap; p.rs.rows_per_rank = rows_per_rank;
  p.rs.status = status; p.rs.limit_ns = p.limit_ns;
  // my own rows come last: by then the other ranks, which started elsewhere, have delivered theirs
  const int m_tiles = (M + TILE_N - 1) / TILE_N;
  p.m_rot = (((rank + 1) % world) * rows_per_rank) / TILE_N;
  if (p.m_rot >= m_tiles) p.m_rot = 0;
  CUtensorMap ta;
  if (make_tmap_2d_u8(&ta, xq, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), TILE_N)) return -12;
  return run_tp(ta, ta, ta, wq, p, num_sms, stream);
}

extern "C" int b200_ag_sync(void* const* peer_data, int world, int rank, size_t flag_off, size_t done_off, int blk_cap,
                            int rows_per_rank, int M, void* words, int wait, int finish, int* status, int limit_ms,
                            cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || rows_per_rank <= 0) return -1;
  AgLink g = {};
  fill_table(g.t, peer_data, nullptr, world, rank);
  g.flag_off = flag_off; g.done_off = done_off; g.blk_cap = blk_cap; g.rows_per_rank = rows_per_rank;
  g.words = static_cast<uint32_t*>(words); g.row_ctr = nullptr; g.status = status;
  g.limit_ns = static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull;
  launch_ex(ag_sync_kernel, dim3(1), dim3(256), 0, stream, 0, g, M, wait, finish);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
