// W8A8 GEMM for decode (M <= 64 tokens): weight streaming with a split-K thread-block cluster.
//
//   Y[m,n] = (sum_k Xq[m,k] * Wq[n,k]) * sx[m] * sw[n]  (+ residual[m,n])
//
// The op is bound by the bytes of Wq, so the grid is shaped for bandwidth, not for the tensor core:
//   * one CTA = 128 output channels x (K / S) of the reduction; the S CTAs of a cluster share one output tile;
//   * shared memory is sized for two co-resident CTAs per SM (up to 32 tokens; the 64-token form takes the SM alone
//     with a deeper pipeline), which keeps > 150 KB of TMA loads in flight per SM and lets CTAs of different tiles
//     overlap head and tail.  The occupancy calculator answers "1 CTA per SM" for every kernel that allocates tensor
//     memory (tcgen05.alloc), whatever its other resources; in-kernel time stamps show two CTAs per SM running, so
//     the host doubles the calculator's cluster counts for the two-CTA forms;
//   * each CTA runs the usual TMA -> tcgen05.mma.kind::i8 -> TMEM pipeline (weights are the 128-row A operand, the
//     token tile of BN in {16,32,64} rows is the B operand);
//   * the S partial accumulators are combined through distributed shared memory: every CTA sends, for each of
//     the S row slices of the tile, its int32 partial to the CTA that owns the slice (16-byte st.shared::cluster
//     into an exchange buffer of its own, so nobody waits for a pipeline to drain), the cluster synchronises once,
//     and each CTA reduces and writes 128/S channels.  No global scratch, no atomics.  The "every CTA of the cluster
//     runs" barrier that distributed shared memory needs is arrived at when the kernel starts and waited for just
//     before the exchange, so its latency hides behind the weight stream.
//   * the host only uses a split whose clusters are all resident at once (occupancy query, with a margin for the
//     neighbouring kernels that programmatic dependent launch keeps on the SMs): a grid that needs a second wave of
//     clusters doubles the latency of an op that is all latency.
// All mbarrier waits are bounded; a CTA that gives up still reaches both cluster barriers, so peers never hang.
//
// Fused activation prologue (DecodeGemmParams::qp): residual add / RMSNorm / SwiGLU, Hadamard rotation and per-token
// int8 run in quantiser CTAs of the same launch (quant_row.cuh), so a linear is one launch from bf16 in to bf16 out.
//
// Fused all-reduce (row-parallel layers under tensor parallelism): with an `ArTail` the CTAs write their bf16 tile of
// the local partial product into this rank's symmetric buffer instead of y, the last CTA of the grid to finish
// signals every peer, and then *all* CTAs (the host only fuses when the whole grid is co-resident) wait for the
// peers' signals and sum the eight partials - through the NVSwitch with multimem.ld_reduce when the heap has a
// multicast mapping, with plain peer loads otherwise - straight into y.  GEMM, reduction and residual add are one
// launch; the partial buffers alternate between two slots so a fast rank never overwrites what a slow one reads.
#include "ptx.cuh"
#include "api.h"
#include "gemm_common.cuh"
#include "peer.cuh"
#include "launch.cuh"
#include "quant_row.cuh"
#include <cstdlib>
#include <algorithm>

namespace b200 {

struct ArTail {
  PeerTable t;
  size_t part_off[2];          // byte offsets of the two partial-product slots inside every heap ([M][N] bf16 each)
  uint32_t* words;             // device words of this rank: [0] epoch, [1] finished CTAs, [2] exited CTAs
  int enabled, use_nvls, limit_ms;
  // Low-latency form: every rank pushes its partial as 8-byte {2 x bf16, epoch} words into a receive area of every
  // rank ([source][M][N/2] words, two slots by epoch parity) and then sums the world copies that arrived locally:
  // one NVLink trip, no fence, no grid-wide counter.  recv_off: byte offsets of the two slots in every heap.
  int ll;
  size_t recv_off[2];
  // Two-hop form of the low-latency tail (more than a few tokens): the CTA that finishes a column slice sends its
  // partial only to the rank that owns the slice (slice index modulo world); the owner's CTA for that slice sums
  // the world partials and broadcasts the result as {2 x bf16, epoch} words into a second receive area ([M][N/2]
  // words, two slots by parity) of every rank.  Each rank then receives 2 x M x N/2 words instead of world x M x N/2,
  // for one more NVLink trip; every rank ends with the owner's bits.  recv2_off: byte offsets of the two slots.
  int two_hop;
  size_t recv2_off[2];
};

struct DecodeGemmParams {
  int M, N, K, kblocks, splits;
  const float* sx;
  const float* sw;
  void* y;
  const __nv_bfloat16* residual;
  int ldy, out_fp32;
  int* status;
  unsigned long long limit_ns;
  ArTail ar;
  // grouped (mixture-of-experts) form: blockIdx.z = local expert; its tokens are rows [grp_offsets[e], +grp_counts[e])
  // of xq / y, its weights are rows [e*N, (e+1)*N) of wq / sw
  const int* grp_offsets;
  const int* grp_counts;
  // Activation prologue inside the launch: the first qp.rows grid rows are quantiser CTAs (one token row each) that turn
  // the bf16 input into the int8 operand and publish a flag per row; the GEMM CTAs prefetch their weights meanwhile
  // and wait for the flags instead of for an earlier kernel.
  QuantProlog qp;
  // split-K exchange: 1 = partials travel as st.async counted on an mbarrier of the receiving CTA (it proceeds as soon
  // as its own bytes are there), 0 = plain distributed-shared-memory stores followed by a barrier of the whole cluster
  int async_x;
  int l2_prefetch;     // this many weight tiles beyond the shared-memory ring are requested into L2 before the dependency wait
  int narrow_epi;      // diagnostics: 1 = the unsplit epilogue stores 2 bytes per thread and token (the older form)
};

// Where a finished output element goes.  A plain struct of scalars (not a capturing lambda: called from the epilogue
// loops, that cost a chain of local-memory loads per element).
struct OutSink {
  int mode;                     // 0: y (+ residual), 1: shared-memory staging of the low-latency all-reduce, 2: bf16 partial in the heap
  float* vals; int cw, m0, n_base;
  __nv_bfloat16* part; int N;
  void* y; const __nv_bfloat16* residual; int ldy, out_fp32;
};
__device__ __forceinline__ void emit1(const OutSink& k, int m, int n, float v) {
  if (k.mode == 1) { k.vals[(m - k.m0) * k.cw + (n - k.n_base)] = v; return; }
  if (k.mode == 2) { k.part[static_cast<size_t>(m) * k.N + n] = __float2bfloat16(v); return; }
  const size_t o = static_cast<size_t>(m) * k.ldy + n;
  if (k.residual) v += __bfloat162float(k.residual[o]);
  if (k.out_fp32) reinterpret_cast<float*>(k.y)[o] = v;
  else reinterpret_cast<__nv_bfloat16*>(k.y)[o] = __float2bfloat16(v);
}
// two adjacent channels n (even), n + 1 of one token
__device__ __forceinline__ void emit2(const OutSink& k, int m, int n, float v0, float v1) {
  if (k.mode == 1) { *reinterpret_cast<float2*>(k.vals + (m - k.m0) * k.cw + (n - k.n_base)) = make_float2(v0, v1); return; }
  if (k.mode == 2) { *reinterpret_cast<__nv_bfloat162*>(k.part + static_cast<size_t>(m) * k.N + n) = __floats2bfloat162_rn(v0, v1); return; }
  const size_t o = static_cast<size_t>(m) * k.ldy + n;
  if (k.out_fp32 || (o & 1)) { emit1(k, m, n, v0); emit1(k, m, n + 1, v1); return; }
  if (k.residual) {
    const __nv_bfloat162 rb = *reinterpret_cast<const __nv_bfloat162*>(k.residual + o);
    v0 += __low2float(rb); v1 += __high2float(rb);
  }
  *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(k.y) + o) = __floats2bfloat162_rn(v0, v1);
}

// u / m for the handful of values the inline prologue meets (u < 8 unrolled, m = 1..4)
__device__ __forceinline__ int inl_div(int u, int m) {
  return m == 1 ? u : (m == 2 ? (u >> 1) : (m == 3 ? ((u * 11) >> 5) : (u >> 2)));
}

// inline prologue: [4 warps][4 rows][2] partial statistics of this CTA + [8 senders][4 rows][4] of the cluster
constexpr int STAT_BYTES = (32 + 128) * 4;
constexpr int INL_MAX_ROWS = 4;       // token rows the inline prologue handles
constexpr int INL_UNITS = 8;          // (k-block, row) pairs per quantising warp: their rotated values stay in registers

// dynamic shared memory: pipeline stages, split-K exchange buffer, channel / token scales, barriers, alignment slack
constexpr int decode_smem_bytes(int bn, int stages) {
  return stages * (TILE_N * BLOCK_K + bn * BLOCK_K) + (TILE_N + 16) * (bn + 4) * 4 + (TILE_N + 64) * 4 + STAT_BYTES + 1024 + 256;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, (BN == 64 ? 1 : 2))
w8a8_gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const DecodeGemmParams p) {
  constexpr int A_BYTES = TILE_N * BLOCK_K;
  constexpr int B_BYTES = BN * BLOCK_K;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t IDESC = umma_idesc_i8(TILE_N, BN);
  constexpr int XS = BN + 4;                      // words per channel row of the exchange buffer (16-byte aligned rows)
  constexpr int EX_ROWS = TILE_N + 16;            // S senders x (slice of at most 2 * ceil(64 / S) channels) <= 128 + 2 S
  constexpr int EX_BYTES = EX_ROWS * XS * 4;      // [sender][channel of the slice][token]
  static_assert(STAGES * STAGE_BYTES >= BN * TILE_N * 4, "the staging buffer of the all-reduce tail aliases the pipeline stages");

  pdl_launch_dependents();     // the next kernel may be scheduled: it only reads our output after its own pdl_wait
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int32_t* ex = reinterpret_cast<int32_t*>(smem + STAGES * STAGE_BYTES);          // split-K exchange buffer
  float* sw_s = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + EX_BYTES);  // [128] channel scales of this tile
  float* sx_s = sw_s + TILE_N;                                                     // [BN] token scales
  float* stat_s = sx_s + 64;                                                       // inline prologue: row statistics
  uint64_t* bars = reinterpret_cast<uint64_t*>(stat_s + STAT_BYTES / 4);           // full[S], empty[S], tfull
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
  const uint32_t xch_bar = bar_base + 8u * (2 * STAGES + 1);     // split-K exchange: bytes the other CTAs send to this one

  const int S = p.splits;
  const int rank = static_cast<int>(cluster_ctarank());          // == blockIdx.x: position along K
  const bool prolog = p.qp.mode != QR_NONE;
  const bool inl = BN == 16 && prolog && p.qp.rows == 0;     // a few tokens: this CTA quantises its own operand (below)
  if (prolog && static_cast<int>(blockIdx.y) < p.qp.rows) {
    // ---- quantiser CTA: one token row, then the row's flag ----
    B200_TRACE_INIT();
    if (threadIdx.x == 0) B200_TRACE(TK_GEMM_DECODE, 20);
    pdl_wait();                                   // the bf16 rows are the previous kernel's output
    if (threadIdx.x == 0) B200_TRACE(TK_GEMM_DECODE, 21);
    const int qrow = blockIdx.y * p.splits + static_cast<int>(cluster_ctarank());
    if (qrow < p.M) {
      const uint32_t ticket = quant_ticket(p.qp);
      quant_row_cta<GEMM_THREADS / 32>(p.qp, qrow, p.K, reinterpret_cast<float*>(smem), reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES));
      __syncthreads();                            // the release below is cumulative over what this barrier orders
      if (threadIdx.x == 0) { st_release_gpu(p.qp.flags + qrow, ticket); B200_TRACE(TK_GEMM_DECODE, 22); }
    }
    B200_TRACE_FLUSH(TK_GEMM_DECODE);
    return;
  }
  const int n_tile = blockIdx.y - (prolog ? p.qp.rows : 0);
  int m0 = blockIdx.z * BN, rows_valid = min(BN, p.M - m0), w_base = 0;
  const bool grouped = p.grp_counts != nullptr;
  if (grouped) {
    pdl_wait();                             // the work list comes from an earlier kernel of the stream
    rows_valid = min(BN, p.grp_counts[blockIdx.z]);
    if (rows_valid <= 0) return;            // same for every CTA of the cluster (they share blockIdx.z)
    m0 = p.grp_offsets[blockIdx.z];
    w_base = blockIdx.z * p.N;
  }
  const int kb0 = static_cast<int>(static_cast<long long>(p.kblocks) * rank / S);
  const int kb1 = static_cast<int>(static_cast<long long>(p.kblocks) * (rank + 1) / S);
  const uint64_t limit = p.limit_ns;

  if (threadIdx.x == 0) {
    // inline prologue: a stage is full when the weight tile has landed and a quantising warp has stored the rows
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), inl ? 2 : 1); mbar_init(empty_bar(s), 1); }
    mbar_init(tfull_bar, 1);
    mbar_init(xch_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    B200_TRACE_INIT();
    B200_TRACE(TK_GEMM_DECODE, TP_START);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  // channel scales never change: they are staged before the dependency wait
  if (threadIdx.x >= 64) {
    const int n = n_tile * TILE_N + (threadIdx.x - 64);
    sw_s[threadIdx.x - 64] = n < p.N ? __ldg(p.sw + w_base + n) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool async_x = S > 1 && p.async_x != 0;
  if (async_x && threadIdx.x == 0) {
    // every CTA of the cluster (this one included) sends its partial of this CTA's slice: whole token chunks, 4 bytes
    // each.  Expected before this CTA announces that it runs, so no sender's bytes can come first.
    constexpr int CHX = (BN >= 32) ? 32 : 16;
    const int my_cw = 2 * ((64 * (rank + 1) + S - 1) / S) - 2 * ((64 * rank + S - 1) / S);
    mbar_expect_tx(xch_bar, static_cast<uint32_t>(S * my_cw * ((rows_valid + CHX - 1) / CHX) * CHX * 4));
  }
  if (S > 1) cluster_arrive_relaxed();          // "this CTA runs": waited for just before the exchange

  // where a finished output element goes: y, or (fused all-reduce) this rank's slot of the symmetric partial buffer
  const bool fuse_ar = p.ar.enabled != 0;
  uint32_t ar_epoch = 0;              // set after the dependency wait: an earlier launch may still be bumping the word
  __nv_bfloat16* part = nullptr;
  // low-latency all-reduce: finished values are staged in shared memory (behind the exchange buffer) first
  const bool ll = fuse_ar && p.ar.ll != 0;
  float* vals = reinterpret_cast<float*>(smem);
  // The cluster's CTA r finishes channels [slice0(r), slice0(r + 1)) of the tile: even-sized slices (the all-reduce tail
  // packs channel pairs) that differ by at most two channels when S does not divide 128.
  auto slice0 = [S](int r) { return 2 * ((64 * r + S - 1) / S); };
  const int cw = slice0(rank + 1) - slice0(rank);                       // channels this CTA finishes
  const int n_base = n_tile * TILE_N + slice0(rank);

  // ---------------- inline activation prologue (up to INL_MAX_ROWS tokens) ----------------
  // Warps 2..5 turn rows [0, M) x this CTA's k-blocks of the bf16 input into the int8 B operand themselves.  A k-block
  // is one 128-block of the Hadamard rotation; k-block kb0 + i belongs to warp 2 + (i & 3), a lane holds four
  // consecutive elements, the rotated values stay in registers.  What a row needs from the other k-blocks - the sum of
  // squares for the norm, the maximum for the scale - is exchanged once through distributed shared memory: the
  // rotation is linear, so the values are rotated *before* the norm's scalar 1/rms is known and the maximum is scaled
  // afterwards.  Every cluster repeats the work for its own tile (a few thousand elements), which removes the
  // activation kernel and its boundary from the chain.  The weight tiles are requested before the dependency wait.
  uint32_t qw[INL_UNITS];
  const int nkb = kb1 - kb0, w4 = warp - 2, Mr = p.M;
  if (inl) {
    if (warp == 0 && lane == 0) {
      const uint64_t pol = policy_evict_first();
      prefetch_tmap(&tmap_w);
      const int pre = min(STAGES, nkb);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), A_BYTES);
        tma_load_2d_hint(smem_base + i * STAGE_BYTES, &tmap_w, full_bar(i), (kb0 + i) * BLOCK_K, w_base + n_tile * TILE_N, pol);
      }
    }
    pdl_wait();
    if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 21);
    const int mode = p.qp.mode;
    const bool norm = mode == QR_NORM || mode == QR_ADD_NORM;
    const int eti = threadIdx.x - 64;
    float v[INL_UNITS][4];
    float st_a = 0.f, st_b = 0.f;
    if (warp >= 2) {
      uint2 ra[INL_UNITS], rb[INL_UNITS], rg[INL_UNITS];
#pragma unroll
      for (int u = 0; u < INL_UNITS; ++u) {
        const int ib = inl_div(u, Mr), m = u - ib * Mr, i = 4 * ib + w4;
        ra[u] = make_uint2(0u, 0u); rb[u] = make_uint2(0u, 0u); rg[u] = make_uint2(0u, 0u);
        if (i < nkb) {
          const int k = (kb0 + i) * BLOCK_K + lane * 4;
          const __nv_bfloat16* xr = p.qp.x + static_cast<size_t>(m) * p.qp.ldx;
          ra[u] = *reinterpret_cast<const uint2*>(xr + k);
          if (mode == QR_SWIGLU) rb[u] = *reinterpret_cast<const uint2*>(xr + p.K + k);
          if (mode == QR_ADD_NORM) rb[u] = *reinterpret_cast<const uint2*>(p.qp.residual + static_cast<size_t>(m) * p.qp.ldr + k);
          if (norm) rg[u] = __ldg(reinterpret_cast<const uint2*>(p.qp.gamma + k));
        }
      }
      const bool keeper = n_tile == 0 && blockIdx.z == 0;       // one cluster writes the updated residual stream
      float ssr[INL_MAX_ROWS] = {0.f, 0.f, 0.f, 0.f}, amr[INL_MAX_ROWS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < INL_UNITS; ++u) {
        const int ib = inl_div(u, Mr), m = u - ib * Mr, i = 4 * ib + w4;
        if (i < nkb) {
          unpack4_bf16(ra[u], v[u]);
          if (mode == QR_SWIGLU) {
            float up[4];
            unpack4_bf16(rb[u], up);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[u][j] = __fdividef(v[u][j], 1.f + __expf(-v[u][j])) * up[j];
          } else if (mode == QR_ADD_NORM) {
            float r[4];
            unpack4_bf16(rb[u], r);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[u][j] = __bfloat162float(__float2bfloat16(__fadd_rn(v[u][j], r[j])));
            if (keeper) {
              const __nv_bfloat162 lo = __floats2bfloat162_rn(v[u][0], v[u][1]), hi = __floats2bfloat162_rn(v[u][2], v[u][3]);
              uint2 raw;
              raw.x = *reinterpret_cast<const uint32_t*>(&lo);
              raw.y = *reinterpret_cast<const uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(p.qp.residual_out + static_cast<size_t>(m) * p.qp.ldro + (kb0 + i) * BLOCK_K + lane * 4) = raw;
            }
          }
          float ss = 0.f;
          if (norm) {
            float g[4];
            unpack4_bf16(rg[u], g);
#pragma unroll
            for (int j = 0; j < 4; ++j) { ss += v[u][j] * v[u][j]; v[u][j] *= g[j]; }
          }
          fwht128_lane4(v[u], lane);
          float am = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) am = fmaxf(am, fabsf(v[u][j]));
#pragma unroll
          for (int mm = 0; mm < INL_MAX_ROWS; ++mm)
            if (m == mm) { ssr[mm] += ss; amr[mm] = fmaxf(amr[mm], am); }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) v[u][j] = 0.f;
        }
      }
#pragma unroll
      for (int mm = 0; mm < INL_MAX_ROWS; ++mm) {
        ssr[mm] = warp_sum(ssr[mm]);
        amr[mm] = warp_max(amr[mm]);
        if (lane == 0) { stat_s[(w4 * 4 + mm) * 2] = ssr[mm]; stat_s[(w4 * 4 + mm) * 2 + 1] = amr[mm]; }
      }
      named_bar_sync(1, 128);
      if (eti < INL_MAX_ROWS) {                  // thread `eti` owns row `eti`: this CTA's share of its statistics
#pragma unroll
        for (int w = 0; w < 4; ++w) { st_a += stat_s[(w * 4 + eti) * 2]; st_b = fmaxf(st_b, stat_s[(w * 4 + eti) * 2 + 1]); }
        if (S == 1) { stat_s[32 + eti * 4] = st_a; stat_s[32 + eti * 4 + 1] = st_b; }
      }
    }
    if (S > 1) {
      cluster_wait_acquire();                    // every CTA of the cluster runs (pairs with the arrival at kernel start)
      if (warp >= 2 && eti < INL_MAX_ROWS) {
        const uint32_t mine = smem_u32(stat_s + 32 + (rank * 4 + eti) * 4);
        for (int dst = 0; dst < S; ++dst)
          st_shared_cluster_v4(mapa_shared(mine, static_cast<uint32_t>(dst)), __float_as_uint(st_a), __float_as_uint(st_b), 0u, 0u);
      }
      cluster_arrive_release();
      cluster_wait_acquire();
      cluster_arrive_relaxed();                  // re-arms the barrier that the split-K exchange waits on
    } else if (warp >= 2) {
      named_bar_sync(1, 128);
    }
    if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 22);
    if (warp >= 2) {
      float inv[INL_MAX_ROWS], my_scale = 0.f;
#pragma unroll
      for (int mm = 0; mm < INL_MAX_ROWS; ++mm) {
        float tss = 0.f, tam = 0.f;
        for (int r = 0; r < S; ++r) { tss += stat_s[32 + (r * 4 + mm) * 4]; tam = fmaxf(tam, stat_s[32 + (r * 4 + mm) * 4 + 1]); }
        const float rstd = norm ? rsqrtf(tss / static_cast<float>(p.K) + p.qp.eps) : 1.f;
        const float sc = quant_scale_from_amax(tam * rstd);
        inv[mm] = rstd * quant_inv_scale(sc);
        if (eti == mm && mm < Mr) my_scale = sc;
      }
      if (eti < BN) sx_s[eti] = my_scale;         // token scales of the epilogue (rows beyond M: 0)
#pragma unroll
      for (int u = 0; u < INL_UNITS; ++u) {
        const int ib = inl_div(u, Mr), m = u - ib * Mr;
        float iv = inv[0];
#pragma unroll
        for (int mm = 1; mm < INL_MAX_ROWS; ++mm) if (m == mm) iv = inv[mm];
        qw[u] = quant_pack4(v[u], iv);
      }
    }
  }

  if (warp == 0) {
    const uint64_t pol_w = policy_evict_first();       // weights are read exactly once per launch
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    // Weights never change during inference, so the first ring-full of weight tiles is requested before waiting
    // for the previous kernel; the activation tiles (its output) are requested after the wait.
    const int pre = grouped ? 0 : min(STAGES, kb1 - kb0);
    const uint32_t stage_tx = inl ? A_BYTES : STAGE_BYTES;     // inline prologue: the token rows are stored, not loaded
    if (lane == 0 && !inl) {
      prefetch_tmap(&tmap_w);
      prefetch_tmap(&tmap_x);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), STAGE_BYTES);
        tma_load_2d_hint(smem_base + i * STAGE_BYTES, &tmap_w, full_bar(i), (kb0 + i) * BLOCK_K, w_base + n_tile * TILE_N, pol_w);
      }
      // The ring holds the first STAGES tiles; the rest of this CTA's weights are pulled into L2 meanwhile, so that once
      // the input is there the stream runs from L2 for as far as HBM got ahead while the previous kernel finished.
      if (p.l2_prefetch > 0)
        for (int kb = kb0 + pre; kb < min(kb1, kb0 + pre + p.l2_prefetch); ++kb) tma_prefetch_2d(&tmap_w, kb * BLOCK_K, w_base + n_tile * TILE_N);
    }
    if (!grouped && !inl) pdl_wait();
    if (prolog && !inl) {
      // the whole warp watches the row flags of this launch's quantiser CTAs (lane l: rows l and l + 32)
      const uint32_t ticket = quant_ticket(p.qp);
      const uint64_t t_start = globaltimer_ns();
      for (int r = lane; r < p.M; r += 32) {
        uint32_t spins = 0;
        while (*reinterpret_cast<const volatile uint32_t*>(p.qp.flags + r) != ticket) {
          if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > limit) {
            if (p.status) atomicCAS(p.status, 0, (ST_TIMEOUT_PEER_FLAG | (2 << 8)));
            ok = false;
            break;
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      __threadfence();                            // acquire side of the row flags (they were polled with plain loads)
      fence_proxy_async_all();                   // the rows were written with ordinary stores, TMA reads them
    }
    if (lane == 0 && ok) {
      B200_TRACE(TK_GEMM_DECODE, TP_DEPS);
      for (int i = 0; i < pre && !inl; ++i)
        tma_load_2d(smem_base + i * STAGE_BYTES + A_BYTES, &tmap_x, full_bar(i), (kb0 + i) * BLOCK_K, m0);
      if (pre == STAGES) phase = 1u; else stage = pre;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (2 << 8)), limit)) { ok = false; break; }
        mbar_expect_tx(full_bar(stage), stage_tx);
        const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
        tma_load_2d_hint(a_dst, &tmap_w, full_bar(stage), kb * BLOCK_K, w_base + n_tile * TILE_N, pol_w);
        if (!inl) tma_load_2d(a_dst + A_BYTES, &tmap_x, full_bar(stage), kb * BLOCK_K, m0);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    if (lane == 0 && !ok) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) { } }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (2 << 8)), limit)) { ok = false; break; }
        tc_fence_after();
        if (kb == kb0) B200_TRACE(TK_GEMM_DECODE, 2);
        const uint32_t a_src = smem_base + stage * STAGE_BYTES;
        const uint64_t a_desc = umma_desc_k_sw128(a_src);
        const uint64_t b_desc = umma_desc_k_sw128(a_src + A_BYTES);
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
          umma_i8_ss(tmem_base, a_desc + 2ull * k, b_desc + 2ull * k, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(empty_bar(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
      B200_TRACE(TK_GEMM_DECODE, 3);
    }
    __syncwarp();
  } else if (inl) {
    // warps 2..5: the quantised rows of their k-blocks go into the B half of the stages (128-byte rows, 16-byte chunk c
    // of row r stored at chunk c ^ (r & 7): the layout a swizzled TMA load would have produced)
    bool ok = true;
#pragma unroll
    for (int u = 0; u < INL_UNITS; ++u) {
      const int ib = inl_div(u, Mr), m = u - ib * Mr, i = 4 * ib + w4;
      if (i < nkb && ok) {
        const int stage = i % STAGES, use = i / STAGES;
        if (m == 0 && use > 0)
          ok = mbar_wait(empty_bar(stage), static_cast<uint32_t>(use - 1) & 1u, abort_flag, p.status, (ST_TIMEOUT_SMEM_EMPTY | (2 << 8)), limit);
        if (ok) {
          const uint32_t dst = smem_base + stage * STAGE_BYTES + A_BYTES + m * 128 + ((((lane >> 2) ^ m) & 7) << 4) + ((lane & 3) << 2);
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(qw[u]) : "memory");
          if (m == Mr - 1) {
            fence_proxy_async_smem();              // generic-proxy stores, read by the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar(stage));
          }
        }
      }
    }
  }

  if (!grouped && warp != 0) pdl_wait();
  if (fuse_ar) {
    // Every thread is past its dependency wait here, so all earlier launches of the stream (which advance the epoch
    // word when they finish) have completed.  The word is bumped again only after every CTA of this grid has exited.
    ar_epoch = *reinterpret_cast<volatile uint32_t*>(p.ar.words) + 1;
    part = reinterpret_cast<__nv_bfloat16*>(p.ar.t.data[p.ar.t.rank] + p.ar.part_off[ar_epoch & 1]);
  }

  // ---------------- epilogue warps: wait for the accumulator ----------------
  const bool epi = warp >= 2;
  const int q = warp & 3;
  const int et = threadIdx.x - 64;
  const int row = q * 32 + lane;                          // channel inside the tile == TMEM lane
  const int jmax = rows_valid;
  constexpr int CH = (BN >= 32) ? 32 : 16;
  bool acc_ok = false;
  if (epi) {
    // token scales: the previous kernel's output, readable now that the dependency wait is behind us
    if (!prolog && et < BN) sx_s[et] = et < jmax ? p.sx[m0 + et] : 0.f;       // (inline prologue: already there)
    acc_ok = (kb1 > kb0) && mbar_wait(tfull_bar, 0, abort_flag, p.status, (ST_TIMEOUT_TMEM_FULL | (2 << 8)), limit);
    tc_fence_after();
    // fused prologue: the scales are written by this launch's quantiser CTAs; the accumulator can only be complete
    // after the producer warp saw every row's flag, so they are there now (read past L1)
    if (prolog && !inl && et < BN) sx_s[et] = et < jmax ? __ldcg(p.sx + m0 + et) : 0.f;
    if (et == 0) B200_TRACE(TK_GEMM_DECODE, 4);
  }

  OutSink sink;
  sink.mode = ll ? 1 : (fuse_ar ? 2 : 0);
  sink.vals = vals; sink.cw = cw; sink.m0 = m0; sink.n_base = n_base; sink.part = part; sink.N = p.N;
  sink.y = p.y; sink.residual = p.residual; sink.ldy = p.ldy; sink.out_fp32 = p.out_fp32;

  if (S == 1) {
    if (epi) asm volatile("bar.sync 1, 128;" ::: "memory");          // sx_s is complete (epilogue warps only)
    if (epi) {
      // a wait gave up somewhere: one thread reads the flag, so all four warps take the same path below (they meet at
      // a barrier there)
      volatile int* verdict = abort_flag + 1;
      if (et == 0) *verdict = *abort_flag;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*verdict) acc_ok = false;
    }
    // Whole tile inside N, bf16 out, 16-byte aligned rows: the tile is turned through shared memory (the pipeline
    // stages are idle now) so that every thread stores 16 bytes of one token row instead of 2 bytes of BN rows.
    __nv_bfloat16* const wdst = sink.mode == 2 ? part : reinterpret_cast<__nv_bfloat16*>(p.y);
    const int wld = sink.mode == 2 ? p.N : p.ldy;
    const __nv_bfloat16* const wres = sink.mode == 0 ? p.residual : nullptr;
    const bool wide = !p.narrow_epi && sink.mode != 1 && !p.out_fp32 && n_tile * TILE_N + TILE_N <= p.N && (wld % 8) == 0 &&
                      (reinterpret_cast<uintptr_t>(wdst) & 15) == 0 && (reinterpret_cast<uintptr_t>(wres) & 15) == 0;
    if (epi && acc_ok && wide) {
      constexpr int TP = TILE_N + 4;                       // floats per token row of the turned tile
      float* tile_f = reinterpret_cast<float*>(smem);
      const float swn = sw_s[row];
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / CH; ++c) {
        if (c * CH >= jmax) break;
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_x32(t_addr + c * CH, r); else tmem_ld_x16(t_addr + c * CH, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; ++j)
          tile_f[(c * CH + j) * TP + row] = static_cast<float>(static_cast<int32_t>(r[j])) * swn * sx_s[c * CH + j];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const size_t col0 = static_cast<size_t>(n_tile) * TILE_N;
      for (int ch = et; ch < jmax * (TILE_N / 8); ch += 128) {
        const int j = ch >> 4, c8 = ch & 15;
        const float4 lo = *reinterpret_cast<const float4*>(tile_f + j * TP + c8 * 8);
        const float4 hi = *reinterpret_cast<const float4*>(tile_f + j * TP + c8 * 8 + 4);
        float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const size_t o = static_cast<size_t>(m0 + j) * wld + col0 + c8 * 8;
        if (wres) {
          const uint4 rv = *reinterpret_cast<const uint4*>(wres + o);
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { f[2 * e] += __uint_as_float(rw[e] << 16); f[2 * e + 1] += __uint_as_float(rw[e] & 0xffff0000u); }
        }
        uint4 out;
        __nv_bfloat162 b2;
        b2 = __floats2bfloat162_rn(f[0], f[1]); out.x = *reinterpret_cast<uint32_t*>(&b2);
        b2 = __floats2bfloat162_rn(f[2], f[3]); out.y = *reinterpret_cast<uint32_t*>(&b2);
        b2 = __floats2bfloat162_rn(f[4], f[5]); out.z = *reinterpret_cast<uint32_t*>(&b2);
        b2 = __floats2bfloat162_rn(f[6], f[7]); out.w = *reinterpret_cast<uint32_t*>(&b2);
        *reinterpret_cast<uint4*>(wdst + o) = out;
      }
    } else if (epi && acc_ok) {
      const int n = n_tile * TILE_N + row;
      const bool n_ok = n < p.N;
      const float swn = sw_s[row];
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / CH; ++c) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_x32(t_addr + c * CH, r); else tmem_ld_x16(t_addr + c * CH, r);
        tmem_ld_wait();
        const int mc = m0 + c * CH;
        const int jm = min(CH, jmax - c * CH);
        if (!n_ok || jm <= 0) continue;
#pragma unroll
        for (int j = 0; j < CH; ++j)
          if (j < jm) emit1(sink, mc + j, n, static_cast<float>(static_cast<int32_t>(r[j])) * swn * sx_s[c * CH + j]);
      }
    }
  } else {
    cluster_wait_acquire();                                 // every CTA of the cluster runs: its shared memory exists
    if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 5);
    if (epi) {
      // exchange buffer in the owner CTA: [sender][channel in the owner's slice][token] int32, XS words per channel row
      const int owner = ((row >> 1) * S) >> 6, row_in = row - slice0(owner);
      const int cw_owner = slice0(owner + 1) - slice0(owner);
      const uint32_t remote = mapa_shared(smem_u32(ex), static_cast<uint32_t>(owner)) +
                              4u * static_cast<uint32_t>((rank * cw_owner + row_in) * XS);
      const uint32_t remote_bar = mapa_shared(xch_bar, static_cast<uint32_t>(owner));
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / CH; ++c) {
        uint32_t r[CH];
        if (acc_ok) {
          if constexpr (CH == 32) tmem_ld_x32(t_addr + c * CH, r); else tmem_ld_x16(t_addr + c * CH, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < CH; ++j) r[j] = 0u;           // empty K range (or aborted): contributes nothing
        }
        if (c * CH < jmax) {                                // token rows beyond the batch are never read back
#pragma unroll
          for (int j = 0; j < CH; j += 4) {
            if (async_x) st_async_cluster_v4(remote + 4u * (c * CH + j), r[j], r[j + 1], r[j + 2], r[j + 3], remote_bar);
            else st_shared_cluster_v4(remote + 4u * (c * CH + j), r[j], r[j + 1], r[j + 2], r[j + 3]);
          }
        }
      }
    }
    if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 10);
    tc_fence_before();
    bool x_ok = true;
    if (async_x) {
      cluster_arrive_relaxed();      // "my stores are issued": waited for just before this CTA leaves (below), so that no
                                     // CTA exits while a peer may still write into it
      x_ok = mbar_wait(xch_bar, 0, abort_flag, p.status, (ST_TIMEOUT_SMEM_FULL | (2 << 8)), limit);
    } else {
      cluster_sync_all();
    }
    if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 6);
    if (x_ok) {
      // All six warps finish blocks of 4 tokens x 8 channel pairs: shared-memory reads spread over the banks (2-way
      // conflicts at worst) and every token row gets 32 contiguous bytes, i.e. whole sectors.  With one warp per
      // scheduler every instruction's latency is exposed, so the loop avoids integer division and works on two
      // independent blocks at a time (all loads first, then the arithmetic and the stores).
      const int pairs = cw >> 1, jt_n = (jmax + 3) >> 2, blocks = jt_n * ((pairs + 7) >> 3);
      const int sw_off = n_base - n_tile * TILE_N;
      const uint32_t inv_jt = (65536u + jt_n - 1) / jt_n;            // blk / jt_n == (blk * inv_jt) >> 16 for blk < 4096
      const int lj = lane & 3, lp = lane >> 2;
      constexpr int NWARP = GEMM_THREADS / 32;
      constexpr int UB = 3;                       // blocks per round: with the sender loop unrolled, all their loads fly together
      for (int blk0 = warp; blk0 < blocks; blk0 += UB * NWARP) {
        int32_t a[UB][2];
        int jj[UB], rr[UB];
        bool on[UB];
#pragma unroll
        for (int u = 0; u < UB; ++u) {
          const int blk = blk0 + u * NWARP;
          const int pt = static_cast<int>((static_cast<uint32_t>(blk) * inv_jt) >> 16), jt = blk - pt * jt_n;
          jj[u] = 4 * jt + lj;
          rr[u] = 2 * (8 * pt + lp);
          on[u] = blk < blocks && jj[u] < jmax && rr[u] < cw;
          a[u][0] = 0; a[u][1] = 0;
        }
        int32_t ld[UB][8][2];
#pragma unroll
        for (int u = 0; u < UB; ++u)
#pragma unroll
          for (int sdr = 0; sdr < 8; ++sdr) {
            ld[u][sdr][0] = 0; ld[u][sdr][1] = 0;
            if (on[u] && sdr < S) {
              ld[u][sdr][0] = ex[(sdr * cw + rr[u]) * XS + jj[u]];
              ld[u][sdr][1] = ex[(sdr * cw + rr[u] + 1) * XS + jj[u]];
            }
          }
#pragma unroll
        for (int u = 0; u < UB; ++u)
#pragma unroll
          for (int sdr = 0; sdr < 8; ++sdr) { a[u][0] += ld[u][sdr][0]; a[u][1] += ld[u][sdr][1]; }
#pragma unroll
        for (int u = 0; u < UB; ++u) {
          if (!on[u]) continue;
          const int n = n_base + rr[u];
          const float sxj = sx_s[jj[u]];
          const float v0 = static_cast<float>(a[u][0]) * sw_s[sw_off + rr[u]] * sxj;
          const float v1 = static_cast<float>(a[u][1]) * sw_s[sw_off + rr[u] + 1] * sxj;
          if (n + 1 < p.N) emit2(sink, m0 + jj[u], n, v0, v1);
          else if (n < p.N) emit1(sink, m0 + jj[u], n, v0);
        }
      }
      if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 11);
    }
    if (async_x) cluster_wait_acquire();
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 64) B200_TRACE(TK_GEMM_DECODE, 7);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }

  if (ll) {
    // ---- low-latency all-reduce: push {payload, epoch} words, then sum what arrived here ----
    const PeerTable& t = p.ar.t;
    const int half = cw / 2, words = half * jmax;
    const size_t slot = p.ar.recv_off[ar_epoch & 1];
    const size_t src_stride = static_cast<size_t>(p.M) * (p.N / 2) * 8;          // bytes per source rank
    const bool two_hop = p.ar.two_hop != 0;
    // debug build: both receive areas must lie inside the heap (a violation is recorded and the tail does nothing)
    bool heap_fine = B200_DBG_RANGE(p.ar.recv_off[0], t.world * src_stride, p.status) && B200_DBG_RANGE(p.ar.recv_off[1], t.world * src_stride, p.status);
    if (two_hop) heap_fine = B200_DBG_RANGE(p.ar.recv2_off[0], src_stride, p.status) && B200_DBG_RANGE(p.ar.recv2_off[1], src_stride, p.status) && heap_fine;
    // two-hop: who reduces this CTA's column slice
    const int unit = n_tile * S + rank;
    const int owner = two_hop ? unit % t.world : t.rank;
    const bool own = owner == t.rank;
    __syncthreads();                                                             // vals complete
    if (epi && heap_fine) {
      for (int w = et; w < words; w += 128) {
        const int j = w / half, c2 = w - j * half;
        const int n = n_base + 2 * c2;
        if (n >= p.N) continue;
        const __nv_bfloat162 pb = __floats2bfloat162_rn(vals[j * cw + 2 * c2], vals[j * cw + 2 * c2 + 1]);
        const uint32_t payload = *reinterpret_cast<const uint32_t*>(&pb);
        const size_t off = slot + t.rank * src_stride + (static_cast<size_t>(m0 + j) * (p.N / 2) + n / 2) * 8;
        if (two_hop) st_ll_peer(t.data[owner] + off, payload, ar_epoch);
        else if (p.ar.use_nvls) multimem_st_ll(t.mc + off, payload, ar_epoch);
        else for (int r = 0; r < t.world; ++r) st_ll_peer(t.data[r] + off, payload, ar_epoch);
      }
      if (et == 0) B200_TRACE(TK_GEMM_DECODE, 8);
      const uint8_t* mine = t.data[t.rank] + slot;
      const size_t slot2 = p.ar.recv2_off[ar_epoch & 1];
      const uint64_t t_start = globaltimer_ns();
      bool good = true;
      for (int w = et; w < words && good; w += 128) {
        const int j = w / half, c2 = w - j * half;
        const int n = n_base + 2 * c2;
        if (n >= p.N) continue;
        const size_t eoff = (static_cast<size_t>(m0 + j) * (p.N / 2) + n / 2) * 8;
        float a0 = 0.f, a1 = 0.f;
        if (own) {
          // all sources are requested at once so their latencies overlap; words that have not arrived are re-read
          uint2 v[MAX_RANKS];
#pragma unroll
          for (int r = 0; r < MAX_RANKS; ++r)
            if (r < t.world) v[r] = ld_ll(mine + r * src_stride + eoff);
          uint32_t spins = 0;
          while (good) {
            bool all = true;
#pragma unroll
            for (int r = 0; r < MAX_RANKS; ++r)
              if (r < t.world && v[r].y != ar_epoch) { all = false; v[r] = ld_ll(mine + r * src_stride + eoff); }
            if (all) break;
            if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > limit) {
              if (p.status) atomicCAS(p.status, 0, (ST_TIMEOUT_PEER_FLAG | (2 << 8)));
              good = false;
            }
          }
          if (!good) break;
#pragma unroll
          for (int r = 0; r < MAX_RANKS; ++r)                                    // fixed order: same bits on every rank
            if (r < t.world) { a0 += __uint_as_float(v[r].x << 16); a1 += __uint_as_float(v[r].x & 0xffff0000u); }
          if (two_hop) {
            // the owner's rounding is what every rank gets
            const __nv_bfloat162 fb = __floats2bfloat162_rn(a0, a1);
            const uint32_t fin = *reinterpret_cast<const uint32_t*>(&fb);
            if (p.ar.use_nvls) multimem_st_ll(t.mc + slot2 + eoff, fin, ar_epoch);
            else for (int r = 0; r < t.world; ++r) if (r != t.rank) st_ll_peer(t.data[r] + slot2 + eoff, fin, ar_epoch);
            a0 = __low2float(fb); a1 = __high2float(fb);
          }
        } else {
          uint2 v = ld_ll(t.data[t.rank] + slot2 + eoff);
          uint32_t spins = 0;
          while (v.y != ar_epoch) {
            if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > limit) {
              if (p.status) atomicCAS(p.status, 0, (ST_TIMEOUT_PEER_FLAG | (2 << 8)));
              good = false;
              break;
            }
            v = ld_ll(t.data[t.rank] + slot2 + eoff);
          }
          if (!good) break;
          a0 = __uint_as_float(v.x << 16); a1 = __uint_as_float(v.x & 0xffff0000u);
        }
        const size_t o = static_cast<size_t>(m0 + j) * p.ldy + n;
        if (p.residual) {
          const __nv_bfloat162 rb = *reinterpret_cast<const __nv_bfloat162*>(p.residual + o);
          a0 += __low2float(rb); a1 += __high2float(rb);
        }
        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.y) + o) = __floats2bfloat162_rn(a0, a1);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      B200_TRACE(TK_GEMM_DECODE, 9);
      const unsigned total_ctas = gridDim.x * gridDim.y * gridDim.z;
      const unsigned old = atomicAdd(p.ar.words + 2, 1u);
      if (old == total_ctas - 1) { p.ar.words[2] = 0; __threadfence(); p.ar.words[0] = ar_epoch; }
    }
  } else if (fuse_ar) {
    // ---- all-reduce tail: every CTA of the (co-resident) grid takes part ----
    const PeerTable& t = p.ar.t;
    const unsigned total_ctas = gridDim.x * gridDim.y * gridDim.z;
    const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const bool heap_fine = B200_DBG_RANGE(p.ar.part_off[0], static_cast<size_t>(p.M) * p.N * 2, p.status) &&
                           B200_DBG_RANGE(p.ar.part_off[1], static_cast<size_t>(p.M) * p.N * 2, p.status);
    __shared__ int ar_ok;
    __threadfence_system();                       // this CTA's part of the partial product is visible to peers
    __syncthreads();
    if (threadIdx.x == 0) {
      ar_ok = 1;
      const unsigned old = atomicAdd(p.ar.words + 1, 1u);
      if (old == total_ctas - 1) {                // the whole local partial is complete: tell everyone
        p.ar.words[1] = 0;
        __threadfence_system();
        for (int r = 0; r < t.world; ++r) st_release_sys(flag_ptr(t, r, 0, t.rank), ar_epoch);
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) { if (!wait_all(t, 0, ar_epoch, threadIdx.x, p.status, limit)) ar_ok = 0; }
    __syncthreads();
    if (ar_ok && heap_fine) {
      const size_t nvec = static_cast<size_t>(p.M) * p.N / 8;            // N is a multiple of 8
      const size_t v0 = nvec * cta / total_ctas, v1 = nvec * (cta + 1) / total_ctas;
      const size_t off = p.ar.part_off[ar_epoch & 1];
      const int vec_per_row = p.N / 8;
      for (size_t i = v0 + threadIdx.x; i < v1; i += GEMM_THREADS) {
        float acc[8];
        if (p.ar.use_nvls) {
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] = 0.f;
          add_bf16x8_to_f32(multimem_ld_reduce_bf16x8(t.mc + off + i * 16), acc);
        } else {
          reduce_p2p_bf16x8(t, off + i * 16, acc);
        }
        const size_t m = i / vec_per_row, nv = i - m * vec_per_row;
        const size_t o = m * p.ldy + nv * 8;
        if (p.residual) add_bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.residual + o), acc);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y) + o) = pack_f32x8_to_bf16(acc);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned old = atomicAdd(p.ar.words + 2, 1u);
      if (old == total_ctas - 1) { p.ar.words[2] = 0; __threadfence(); p.ar.words[0] = ar_epoch; }
    }
  }
  B200_TRACE_FLUSH(TK_GEMM_DECODE);
}

template <int BN, int STAGES>
static int launch_decode(const CUtensorMap& tw, const CUtensorMap& tx, const DecodeGemmParams& p, dim3 grid, cudaStream_t stream) {
  constexpr int SMEM = decode_smem_bytes(BN, STAGES);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_gemm_decode_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
    // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
    cudaFuncSetAttribute(w8a8_gemm_decode_kernel<BN, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return -1000 - static_cast<int>(e);
    configured = true;
  }
  cudaError_t e = launch_ex(w8a8_gemm_decode_kernel<BN, STAGES>, grid, dim3(GEMM_THREADS), SMEM, stream, static_cast<int>(grid.x), tw, tx, p);
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

// How many clusters of `s` CTAs of this kernel the GPU can hold at once (cached per instantiation and cluster size).
static int resident_clusters_reported(int bn, int s);

template <int BN, int STAGES>
static int max_resident_clusters(int s) {
  static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (s < 1 || s > 8) return 0;
  if (cache[s] > 0) return cache[s];
  constexpr int SMEM = decode_smem_bytes(BN, STAGES);
  cudaFuncSetAttribute(w8a8_gemm_decode_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
  // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
  cudaFuncSetAttribute(w8a8_gemm_decode_kernel<BN, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s, 64, 1);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = s; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, w8a8_gemm_decode_kernel<BN, STAGES>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cache[s] = n > 0 ? n : -1;
  return cache[s];
}

// CTAs of the decode GEMM one SM really holds: two when twice the shared memory (plus the per-CTA reservation) fits
static int ctas_per_sm(int bn) {
  const int smem = bn <= 16 ? decode_smem_bytes(16, 5) : (bn <= 32 ? decode_smem_bytes(32, 4) : decode_smem_bytes(64, 7));
  return 2 * (smem + 1024) <= 228 * 1024 ? 2 : 1;
}

static int resident_clusters(int bn, int s) {
  return resident_clusters_reported(bn, s) * ctas_per_sm(bn);
}

static int resident_clusters_reported(int bn, int s) {
  switch (bn) {
    case 16: return max_resident_clusters<16, 5>(s);
    case 32: return max_resident_clusters<32, 4>(s);
    default: return max_resident_clusters<64, 7>(s);
  }
}

// Split along K: the largest cluster size (1..8, any value: slices need not divide the tile evenly) whose grid of
// tiles x S CTAs (a) fits the SMs (two CTAs each for up to 32 tokens), (b) leaves every CTA at least two k-blocks, and (c) is resident at
// once according to the occupancy query, with `margin` spare clusters.
// quant_rows > 0: the launch also carries ceil(quant_rows / S) clusters of quantiser CTAs.
// min_kb: fewest k-blocks a CTA should keep.
int decode_pick_splits(int tiles, int kblocks, int num_sms, int bn, int margin, int quant_rows = 0, int min_kb = 2) {
  static int limit_env = -1;
  if (limit_env < 0) { const char* e = std::getenv("B200RT_GEMM_MAX_CTAS"); limit_env = e ? std::atoi(e) : 0; }
  const int limit = limit_env > 0 ? limit_env : num_sms * ctas_per_sm(bn);
  int best = 1;
  for (int s = 2; s <= 8; ++s) {
    const int all = tiles + (quant_rows + s - 1) / s;
    if (all * s > limit || kblocks < min_kb * s) break;
    if (all + margin <= resident_clusters(bn, s)) best = s;
  }
  return best;
}

}  // namespace b200

using namespace b200;

// groups > 0: M is the bound on tokens per expert and on the rows of xq, wq holds groups*N rows
static int decode_gemm_impl(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                            const void* residual, int M, int N, int K, int ldy, int out_fp32, int* status,
                            int num_sms, int force_splits, const ArTail* ar, cudaStream_t stream,
                            int groups = 0, const int* grp_offsets = nullptr, const int* grp_counts = nullptr,
                            int x_rows = 0, const QuantProlog* qp = nullptr) {
  // Plain calls may bring several token tiles of 64 (one grid layer each; every layer streams the weights again, so this
  // is for narrow outputs such as a router); the grouped, fused-prologue and all-reduce forms take one tile.
  constexpr int MULTI_TILE_MAX_M = 4 * SWAP_MAX_M;
  if (M <= 0 || N <= 0 || K <= 0 || (K % 16) != 0) return -1;
  if (M > ((groups > 0 || qp || ar) ? SWAP_MAX_M : MULTI_TILE_MAX_M)) return -1;
  if (qp) {
    // the quantiser CTAs park a row as floats in the pipeline's stage memory and work in whole 128-blocks
    if (groups > 0 || force_splits > 0 || (K % 128) || K * 4 > 80 * 1024 || qp->mode < QR_PLAIN || qp->mode > QR_SWIGLU) return -1;
    if (!qp->x || !qp->q || !qp->scale || !qp->flags || !qp->step) return -1;
    if ((qp->mode == QR_NORM || qp->mode == QR_ADD_NORM) && !qp->gamma) return -1;
    if (qp->mode == QR_ADD_NORM && !qp->residual) return -1;
    if (qp->residual_out && ((qp->ldro % 4) || (reinterpret_cast<uintptr_t>(qp->residual_out) & 7))) return -2;
    if ((qp->ldx % 4) || (qp->ldr % 4) || (reinterpret_cast<uintptr_t>(qp->x) & 7) || (reinterpret_cast<uintptr_t>(qp->residual) & 7) ||
        (reinterpret_cast<uintptr_t>(qp->gamma) & 7)) return -2;
  }
  if (groups > 0 && ((N % TILE_N) || !grp_offsets || !grp_counts || ar)) return -1;
  if ((reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15)) return -2;
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  DecodeGemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
  const int n_tiles = (N + TILE_N - 1) / TILE_N, m_tiles = groups > 0 ? groups : (M + bn - 1) / bn;
  // A split whose clusters do not all fit on the GPU at once runs as two waves: twice the latency for an op that is
  // nothing but latency.  (Grouped launches have one grid row per expert and are multi-wave by nature.)
  // Up to INL_MAX_ROWS tokens the GEMM CTAs quantise their own operand (inline prologue) when a warp's share of
  // (k-block, row) pairs fits its registers; otherwise the launch carries quantiser CTAs.
  bool inl = false;
  int s = 0;
  if (qp && M <= INL_MAX_ROWS && qp->allow_inline && !(qp->mode == QR_ADD_NORM && (!qp->residual_out || qp->residual_out == qp->residual))) {
    s = decode_pick_splits(n_tiles * m_tiles, p.kblocks, num_sms, bn, 1, 0);
    if (ar) while (s >= 1 && n_tiles * m_tiles + 1 > resident_clusters(bn, s)) --s;
    if (s >= 1 && (((p.kblocks + s - 1) / s + 3) / 4) * M <= INL_UNITS) inl = true;
  }
  // With the all-reduce tail every CTA also pushes, polls and sums its slice of the output: a launch of few CTAs (the
  // o-projection's 1/8 shard has four k-blocks) is bound by that tail, so there a CTA may keep a single k-block (4 GPUs,
  // 32 tokens, K shard 512: 12.9 us against 15.0 us with two k-blocks per CTA; B200RT_AR_MIN_KBLOCKS=2 restores that).
  static int ar_min_kb = -1;
  if (ar_min_kb < 0) { const char* e = std::getenv("B200RT_AR_MIN_KBLOCKS"); ar_min_kb = e ? std::max(1, std::atoi(e)) : 1; }
  if (!inl) s = force_splits > 0 ? force_splits : decode_pick_splits(n_tiles * m_tiles, p.kblocks, num_sms, bn, groups > 0 ? -100000 : 1, qp ? M : 0,
                                                                     ar ? ar_min_kb : 2);
  if (s < 1 || s > 8) return -1;
  p.splits = s;
  p.sx = sx; p.sw = sw; p.y = y; p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldy = ldy; p.out_fp32 = out_fp32; p.status = status; p.limit_ns = 2000000000ull;
  if (ar) p.ar = *ar; else { p.ar = ArTail{}; p.ar.enabled = 0; }
  p.grp_offsets = groups > 0 ? grp_offsets : nullptr;
  p.grp_counts = groups > 0 ? grp_counts : nullptr;
  const int w_rows = groups > 0 ? groups * N : N;
  const int xr = groups > 0 ? x_rows : M;
  if (ar) {
    // Every CTA waits for the peers, so the whole grid has to be resident at once: ask the occupancy calculator how
    // many clusters of this size fit (clusters are placed per GPC, so this is less than SMs x CTAs-per-SM / size)
    // and narrow the split until the grid fits, keeping a margin of one cluster.
    if ((N % 8) || (ldy % 8) || out_fp32) return -2;
    while (s >= 1 && n_tiles * m_tiles + ((qp && !inl) ? (M + s - 1) / s : 0) + 1 > resident_clusters(bn, s)) --s;
    if (s < 1) return -20;
    p.splits = s;
    // The two-hop tail pays for its second NVLink trip by spreading the owner's work over many CTAs; a launch split
    // into fewer CTAs than this per tile keeps the one-trip tail (B200RT_AR_TWO_HOP_MIN_SPLITS, default 1: no limit).
    static int th_min_s = -1;
    if (th_min_s < 0) { const char* e = std::getenv("B200RT_AR_TWO_HOP_MIN_SPLITS"); th_min_s = e ? std::max(1, std::atoi(e)) : 1; }
    if (s < th_min_s) p.ar.two_hop = 0;
    p.limit_ns = static_cast<unsigned long long>(ar->limit_ms > 0 ? ar->limit_ms : 2000) * 1000000ull;
  }
  static int async_env = -1;
  if (async_env < 0) { const char* e = std::getenv("B200RT_GEMM_ASYNC_X"); async_env = (e && e[0] == '0') ? 0 : 1; }
  p.async_x = async_env;
  static int l2_env = -1;
  if (l2_env < 0) { const char* e = std::getenv("B200RT_L2_PREFETCH_TILES"); l2_env = e ? std::atoi(e) : 0; }
  p.l2_prefetch = (groups > 0) ? 0 : l2_env;
  static int narrow_env = -1;
  if (narrow_env < 0) { const char* e = std::getenv("B200RT_GEMM_NARROW_EPI"); narrow_env = (e && e[0] == '1') ? 1 : 0; }
  p.narrow_epi = narrow_env;
  p.qp = QuantProlog{};
  int q_rows = 0;
  if (qp) {
    static uint32_t launch_counter = 0;          // distinguishes the launches of one step (see quant_ticket)
    p.qp = *qp;
    p.qp.launch_id = ++launch_counter;
    q_rows = inl ? 0 : (M + s - 1) / s;
    p.qp.rows = q_rows;
    if (!p.qp.residual_out) { p.qp.residual_out = p.qp.residual; p.qp.ldro = p.qp.ldr; }
    if (m_tiles != 1) return -1;
  }
  CUtensorMap tw, tx;
  if (make_tmap_2d_u8(&tw, wq, static_cast<uint64_t>(K), static_cast<uint64_t>(w_rows), static_cast<uint64_t>(K), TILE_N)) return -11;
  if (make_tmap_2d_u8(&tx, xq, static_cast<uint64_t>(K), static_cast<uint64_t>(xr), static_cast<uint64_t>(K), bn)) return -12;
  dim3 grid(s, n_tiles + q_rows, m_tiles);
  switch (bn) {
    case 16: return launch_decode<16, 5>(tw, tx, p, grid, stream);
    case 32: return launch_decode<32, 4>(tw, tx, p, grid, stream);
    default: return launch_decode<64, 7>(tw, tx, p, grid, stream);
  }
}

template <int BN, int STAGES>
static void occupancy_facts(int* out) {
  constexpr int SMEM = decode_smem_bytes(BN, STAGES);
  cudaFuncSetAttribute(w8a8_gemm_decode_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  // ask for the largest shared-memory carveout: with the default preference the occupancy calculator (and the
  // launch) may settle for a split of the L1 / shared array that holds fewer CTAs per SM than the kernel was sized for
  cudaFuncSetAttribute(w8a8_gemm_decode_kernel<BN, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  int blocks = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, w8a8_gemm_decode_kernel<BN, STAGES>, GEMM_THREADS, SMEM);
  cudaFuncAttributes a{};
  cudaFuncGetAttributes(&a, w8a8_gemm_decode_kernel<BN, STAGES>);
  out[0] = blocks; out[1] = static_cast<int>(a.sharedSizeBytes); out[2] = a.numRegs; out[3] = SMEM;
}
// Occupancy facts of the decode GEMM for `m` tokens: {CTAs per SM without clusters, static shared bytes, registers per
// thread, dynamic shared bytes}.
extern "C" void b200_w8a8_gemm_decode_occupancy(int m, int* out4) {
  if (m <= 16) occupancy_facts<16, 5>(out4); else if (m <= 32) occupancy_facts<32, 4>(out4); else occupancy_facts<64, 7>(out4);
}

// Occupancy calculator's answer for the 32-token decode GEMM at an arbitrary dynamic shared-memory size (diagnostics).
extern "C" int b200_w8a8_gemm_decode_blocks_at(int smem_bytes) {
  int blocks = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, w8a8_gemm_decode_kernel<32, 4>, GEMM_THREADS, smem_bytes);
  return blocks;
}

// How many clusters of `splits` CTAs of the decode GEMM for `m` tokens this GPU holds at once (occupancy query).
extern "C" int b200_w8a8_gemm_decode_resident_clusters(int m, int splits) {
  return resident_clusters(m <= 16 ? 16 : (m <= 32 ? 32 : 64), splits);
}

static QuantProlog to_prolog(const b200_quant_prolog& c) {
  QuantProlog q{};
  q.mode = c.mode;
  q.x = static_cast<const __nv_bfloat16*>(c.x); q.ldx = c.ldx;
  q.residual = static_cast<__nv_bfloat16*>(c.residual); q.ldr = c.ldr;
  q.gamma = static_cast<const __nv_bfloat16*>(c.gamma); q.eps = c.eps;
  q.q = static_cast<int8_t*>(c.q); q.scale = c.scale;
  q.flags = static_cast<uint32_t*>(c.flags); q.step = static_cast<const uint32_t*>(c.step);
  q.residual_out = static_cast<__nv_bfloat16*>(c.residual_out); q.ldro = c.ldro;
  q.allow_inline = c.allow_inline;
  return q;
}

// One launch from bf16 activations to the bf16 result: the prologue (prolog->mode: 1 rotate + quantise, 2 RMSNorm first,
// 3 residual add + RMSNorm first, 4 SwiGLU of [M][2K] first) runs in quantiser CTAs of the same launch.
extern "C" int b200_w8a8_gemm_decode_p(const b200_quant_prolog* prolog, const void* wq, const float* sw, void* y,
                                       const void* residual, int M, int N, int K, int ldy, int out_fp32, int* status,
                                       int num_sms, cudaStream_t stream) {
  if (!prolog) return -1;
  const QuantProlog q = to_prolog(*prolog);
  return decode_gemm_impl(q.q, q.scale, wq, sw, y, residual, M, N, K, ldy, out_fp32, status, num_sms, 0, nullptr, stream, 0, nullptr,
                          nullptr, 0, &q);
}

extern "C" int b200_w8a8_gemm_decode(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                                     const void* residual, int M, int N, int K, int ldy, int out_fp32, int* status,
                                     int num_sms, int force_splits, cudaStream_t stream) {
  return decode_gemm_impl(xq, sx, wq, sw, y, residual, M, N, K, ldy, out_fp32, status, num_sms, force_splits, nullptr, stream);
}

// Grouped form for mixture-of-experts decode: `groups` local experts, expert e multiplies rows
// [grp_offsets[e], +grp_counts[e]) of xq (x_rows rows in total, at most max_tokens per expert, max_tokens <= 64) by
// wq[e*N : (e+1)*N] and writes the same rows of y.  Offsets and counts are device arrays: nothing syncs the host.
extern "C" int b200_w8a8_gemm_decode_grouped(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                                             int max_tokens, int x_rows, int N, int K, int ldy, int groups,
                                             const int* grp_offsets, const int* grp_counts, int* status, int num_sms,
                                             cudaStream_t stream) {
  return decode_gemm_impl(xq, sx, wq, sw, y, nullptr, max_tokens, N, K, ldy, 0, status, num_sms, 0, nullptr, stream, groups,
                          grp_offsets, grp_counts, x_rows);
}

// Row-parallel linear fused with its all-reduce: y[m,n] = sum over ranks of (xq_r . wq_r^T * sx_r * sw) (+ residual).
// part_off0/1: byte offsets (same on every rank) of two [M][N] bf16 slots in the symmetric heap; words: >= 4 zeroed
// device uint32 of this rank.  Returns -20 when the grid would not be co-resident (use the unfused path then).
static int decode_ar_impl(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                          const void* residual, int M, int N, int K, int ldy, int* status, int num_sms,
                          void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                          size_t part_off0, size_t part_off1, void* words, int limit_ms, int ll,
                          size_t recv_off0, size_t recv_off1, size_t recv_bytes, int two_hop,
                          size_t recv2_off0, size_t recv2_off1, size_t recv2_bytes, cudaStream_t stream, const QuantProlog* qp) {
  if (world < 1 || world > MAX_RANKS) return -1;
  ArTail ar;
  for (int r = 0; r < MAX_RANKS; ++r) {
    ar.t.data[r] = r < world ? static_cast<uint8_t*>(peer_data[r]) : nullptr;
    ar.t.flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  ar.t.mc = static_cast<uint8_t*>(mc_base); ar.t.world = world; ar.t.rank = rank;
  ar.part_off[0] = part_off0; ar.part_off[1] = part_off1;
  ar.words = static_cast<uint32_t*>(words);
  ar.enabled = 1; ar.use_nvls = mc_base != nullptr; ar.limit_ms = limit_ms;
  ar.ll = ll; ar.recv_off[0] = recv_off0; ar.recv_off[1] = recv_off1;
  ar.two_hop = (ll && two_hop && world > 1) ? 1 : 0; ar.recv2_off[0] = recv2_off0; ar.recv2_off[1] = recv2_off1;
  if (ll) {
    if ((recv_off0 % 8) || (recv_off1 % 8) || (N % 2)) return -2;
    if (static_cast<size_t>(world) * M * (N / 2) * 8 > recv_bytes) return -21;       // receive slot too small
  }
  if (ar.two_hop) {
    if ((recv2_off0 % 8) || (recv2_off1 % 8)) return -2;
    if (static_cast<size_t>(M) * (N / 2) * 8 > recv2_bytes) return -21;
    // every rank has to own a slice, or the slot-reuse argument (a rank cannot run two launches ahead) breaks
    if ((N + TILE_N - 1) / TILE_N < world) ar.two_hop = 0;
  }
  if ((part_off0 % 16) || (part_off1 % 16)) return -2;
  return decode_gemm_impl(xq, sx, wq, sw, y, residual, M, N, K, ldy, 0, status, num_sms, 0, &ar, stream, 0, nullptr, nullptr, 0, qp);
}

extern "C" int b200_w8a8_gemm_decode_ar(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                                        const void* residual, int M, int N, int K, int ldy, int* status, int num_sms,
                                        void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                                        size_t part_off0, size_t part_off1, void* words, int limit_ms, int ll,
                                        size_t recv_off0, size_t recv_off1, size_t recv_bytes, int two_hop,
                                        size_t recv2_off0, size_t recv2_off1, size_t recv2_bytes, cudaStream_t stream) {
  return decode_ar_impl(xq, sx, wq, sw, y, residual, M, N, K, ldy, status, num_sms, peer_data, peer_flags, mc_base, world, rank,
                        part_off0, part_off1, words, limit_ms, ll, recv_off0, recv_off1, recv_bytes, two_hop, recv2_off0,
                        recv2_off1, recv2_bytes, stream, nullptr);
}

// The fused GEMM + all-reduce with the activation prologue in the same launch (see b200_w8a8_gemm_decode_p).
extern "C" int b200_w8a8_gemm_decode_ar_p(const b200_quant_prolog* prolog, const void* wq, const float* sw, void* y,
                                          const void* residual, int M, int N, int K, int ldy, int* status, int num_sms,
                                          void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                                          size_t part_off0, size_t part_off1, void* words, int limit_ms, int ll,
                                          size_t recv_off0, size_t recv_off1, size_t recv_bytes, int two_hop,
                                          size_t recv2_off0, size_t recv2_off1, size_t recv2_bytes, cudaStream_t stream) {
  if (!prolog) return -1;
  const QuantProlog q = to_prolog(*prolog);
  return decode_ar_impl(q.q, q.scale, wq, sw, y, residual, M, N, K, ldy, status, num_sms, peer_data, peer_flags, mc_base, world, rank,
                        part_off0, part_off1, words, limit_ms, ll, recv_off0, recv_off1, recv_bytes, two_hop, recv2_off0,
                        recv2_off1, recv2_bytes, stream, &q);
}
