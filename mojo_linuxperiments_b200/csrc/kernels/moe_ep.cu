// Expert-parallel dispatch and combine for token-sharded prefill: the all-to-all of a mixture-of-experts layer done
// with stores into the receivers' symmetric heaps (buffers and epoch protocol of tp_link.cuh).
//
// Each rank owns R token rows.  After the router ran on those rows:
//   dispatch   one CTA per owned row.  The row's int8 activations and scale are stored only into the heaps of the
//              ranks that own at least one of its top-k experts (a token reaches ~5.3 of 8 ranks for top-8 of 128), its
//              (expert id, weight) list is stored into every heap (64 bytes per token); the last row of each 128-row
//              block publishes flag[source][block] = epoch on every rank.
//   wait       every rank waits (bounded) for all blocks of all sources and copies the routing lists of all M tokens
//              out of the epoch's buffer; from there the existing work-list / grouped-GEMM kernels run unchanged and
//              `gather` fetches exactly the rows that were sent here.
//   combine    one CTA per token that used a local expert: the weighted sum of its local expert outputs is stored
//              (bf16) into receive slot [this rank][row] of the token's owner; every 128-row block of an owner is
//              reported with one remote add of its row count.
//   reduce     the owner waits until all world ranks reported all of its rows and sums, per row, the slots of exactly
//              those ranks its own routing list says contributed.
// No barrier and no library collective; every wait is bounded and reports through the status word.
// No counterpart in the reference (it has no model code); the transport is the same store-then-gate pattern as its
// ring reduce (test_linux_threading.mojo:400-414).
#include "ptx.cuh"
#include "api.h"
#include "launch.cuh"
#include "tp_link.cuh"

namespace b200 {

constexpr int EP_KMAX = 8;       // routing slots per token in the exchange buffers

struct EpDispatchParams {
  AgLink g;                      // gather buffers, flags, done words, epoch words, row counters
  size_t ids_off[2], wts_off[2]; // int32 / fp32 [m_cap][EP_KMAX] per parity
  const int8_t* xq_local;        // [my_rows][K]
  const float* sx_local;
  const int* ids_local;          // [my_rows][k]
  const float* wts_local;
  int M, K, k, experts_per_rank;
};

__global__ void __launch_bounds__(128) ep_dispatch_kernel(const EpDispatchParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const AgLink& g = p.g;
  const PeerTable& t = g.t;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(g.words) + 1;
  const int par = static_cast<int>(e & 1u);
  const int R = g.rows_per_rank;
  const int my_rows = max(0, min(R, p.M - t.rank * R));
  const int row = blockIdx.x;
  if (row >= my_rows) return;
  const int tid = threadIdx.x;
  __shared__ int need_s[MAX_RANKS];
  __shared__ int ok_s;
  if (tid == 0) ok_s = 1;
  if (tid < MAX_RANKS) need_s[tid] = 0;
  __syncthreads();
  // the buffer of this parity was last used two calls ago: every consumer must have finished that call
  if (tid < t.world) {
    if (!wait_flag_ge(reinterpret_cast<const uint32_t*>(t.data[t.rank] + g.done_off) + tid, e - 2u, g.status, g.limit_ns)) ok_s = 0;
  }
  if (tid < p.k) {
    const int ex = p.ids_local[static_cast<size_t>(row) * p.k + tid];
    const int dst = ex / p.experts_per_rank;
    if (dst >= 0 && dst < t.world) need_s[dst] = 1;            // benign race: all writers store 1
  }
  __syncthreads();
  const size_t grow = static_cast<size_t>(t.rank) * R + row;
  // debug build: every store of this row (int8 row, scale, routing lists) must land inside the peers' heaps
  const bool heap_fine = B200_DBG_RANGE(g.q_off[par] + grow * p.K, static_cast<size_t>(p.K), g.status) &&
                         B200_DBG_RANGE(g.s_off[par] + grow * 4, 4, g.status) &&
                         B200_DBG_RANGE(p.ids_off[par] + grow * EP_KMAX * 4, EP_KMAX * 4, g.status) &&
                         B200_DBG_RANGE(p.wts_off[par] + grow * EP_KMAX * 4, EP_KMAX * 4, g.status);
  if (ok_s && heap_fine) {
    // routing list to every rank, padded to EP_KMAX with id -1
    if (tid < EP_KMAX) {
      const int id = tid < p.k ? p.ids_local[static_cast<size_t>(row) * p.k + tid] : -1;
      const float w = tid < p.k ? p.wts_local[static_cast<size_t>(row) * p.k + tid] : 0.f;
      for (int r = 0; r < t.world; ++r) {
        reinterpret_cast<int*>(t.data[r] + p.ids_off[par])[grow * EP_KMAX + tid] = id;
        reinterpret_cast<float*>(t.data[r] + p.wts_off[par])[grow * EP_KMAX + tid] = w;
      }
    }
    // the row itself only to the ranks that own one of its experts
    const uint4* src = reinterpret_cast<const uint4*>(p.xq_local + static_cast<size_t>(row) * p.K);
    const size_t off = g.q_off[par] + grow * p.K;
    for (int v = tid; v < p.K / 16; v += blockDim.x) {
      const uint4 x = src[v];
      for (int r = 0; r < t.world; ++r)
        if (need_s[r]) *reinterpret_cast<uint4*>(t.data[r] + off + static_cast<size_t>(v) * 16) = x;
    }
    if (tid < t.world && need_s[tid]) *reinterpret_cast<float*>(t.data[tid] + g.s_off[par] + grow * 4) = p.sx_local[row];
  }
  __syncthreads();
  if (tid == 0 && ok_s) {
    const int blk = row >> 7;
    const int rows_b = min(128, my_rows - blk * 128);
    fence_acq_rel_sys();
    const uint32_t old = atomicAdd(g.row_ctr + blk, 1u);
    if (old == static_cast<uint32_t>(rows_b) - 1u) {
      g.row_ctr[blk] = 0;
      fence_acq_rel_sys();
      for (int r = 0; r < t.world; ++r)
        st_release_sys(reinterpret_cast<uint32_t*>(t.data[r] + g.flag_off) + t.rank * g.blk_cap + blk, e);
    }
  }
}

// waits for every block of every source, then copies the routing lists of all M tokens into ordinary tensors
__global__ void __launch_bounds__(256) ep_wait_kernel(const AgLink g, size_t ids_off0, size_t ids_off1, size_t wts_off0,
                                                      size_t wts_off1, int M, int k, int* ids_out, float* wts_out) {
  pdl_launch_dependents();
  pdl_wait();
  const PeerTable& t = g.t;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(g.words) + 1;
  const int par = static_cast<int>(e & 1u);
  __shared__ int good;
  if (threadIdx.x == 0) good = 1;
  __syncthreads();
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(t.data[t.rank] + g.flag_off);
  const int R = g.rows_per_rank;
  for (int i = threadIdx.x; i < t.world * g.blk_cap; i += blockDim.x) {
    const int s = i / g.blk_cap, blk = i - s * g.blk_cap;
    const int rows_s = max(0, min(R, M - s * R));
    if (blk * 128 < rows_s && !wait_flag_ge(flags + i, e, g.status, g.limit_ns)) good = 0;
  }
  __syncthreads();
  if (!good) return;
  const int* ids = reinterpret_cast<const int*>(t.data[t.rank] + (par ? ids_off1 : ids_off0));
  const float* wts = reinterpret_cast<const float*>(t.data[t.rank] + (par ? wts_off1 : wts_off0));
  const size_t total = static_cast<size_t>(M) * k;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t m = i / k, j = i - m * k;
    ids_out[i] = __ldcg(ids + m * EP_KMAX + j);
    wts_out[i] = __ldcg(wts + m * EP_KMAX + j);
  }
}

// moe_gather over the gather buffer of the current epoch: slot s <- token row slot_token[s]
__global__ void __launch_bounds__(128) ep_gather_kernel(const uint8_t* heap, size_t q_off0, size_t q_off1, size_t s_off0,
                                                        size_t s_off1, const uint32_t* words, int d, const int* slot_token,
                                                        const int* meta, int8_t* xq_perm, float* sx_perm) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= meta[0]) return;
  const int par = static_cast<int>((*reinterpret_cast<const volatile uint32_t*>(words) + 1) & 1u);
  const int tkn = slot_token[s];
  const uint4* src = reinterpret_cast<const uint4*>(heap + (par ? q_off1 : q_off0) + static_cast<size_t>(tkn) * d);
  uint4* dst = reinterpret_cast<uint4*>(xq_perm + static_cast<size_t>(s) * d);
  for (int i = threadIdx.x; i < d / 16; i += blockDim.x) dst[i] = __ldcg(src + i);
  if (threadIdx.x == 0) sx_perm[s] = __ldcg(reinterpret_cast<const float*>(heap + (par ? s_off1 : s_off0)) + tkn);
}

struct EpCombineParams {
  RsLink s;
  const __nv_bfloat16* y; long long ldy;      // expert outputs in slot order
  const int* inv;                              // [M][k] slot of (token, j) or -1
  const float* wts;                            // [M][k]
  uint32_t* blk_ctr;                           // local: [world * blk_cap] rows handled per (owner, 128-row block)
  int blk_cap;
  int M, k, d;
};

// one CTA per token
__global__ void __launch_bounds__(256) ep_combine_scatter_kernel(const EpCombineParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const PeerTable& t = p.s.t;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.s.words) + 1;
  const int par = static_cast<int>(e & 1u);
  const int m = blockIdx.x;
  const int R = p.s.rows_per_rank;
  const int owner = m / R, lr = m - owner * R;
  __shared__ int slot_s[32];
  __shared__ float w_s[32];
  __shared__ int any_s;
  if (threadIdx.x == 0) any_s = 0;
  __syncthreads();
  if (threadIdx.x < p.k) {
    const int sl = p.inv[static_cast<size_t>(m) * p.k + threadIdx.x];
    slot_s[threadIdx.x] = sl;
    w_s[threadIdx.x] = p.wts[static_cast<size_t>(m) * p.k + threadIdx.x];
    if (sl >= 0) any_s = 1;
  }
  __syncthreads();
  if (any_s) {
    uint8_t* dst = t.data[owner] + p.s.recv_off[par] + (static_cast<size_t>(t.rank) * p.s.r_cap + lr) * p.d * 2;
    for (int c = threadIdx.x; c < p.d / 8; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < p.k; ++j) {
        const int sl = slot_s[j];
        if (sl < 0) continue;
        const uint4 raw = *reinterpret_cast<const uint4*>(p.y + static_cast<size_t>(sl) * p.ldy + c * 8);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        const float wt = w_s[j];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += wt * __uint_as_float(w[i] << 16);
          acc[2 * i + 1] += wt * __uint_as_float(w[i] & 0xffff0000u);
        }
      }
      *reinterpret_cast<uint4*>(dst + static_cast<size_t>(c) * 16) = pack_f32x8_to_bf16(acc);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // every row of the owner is reported, sent or not; the last row of a 128-row block makes the remote add
    const int rows_o = max(0, min(R, p.M - owner * R));
    const int blk = lr >> 7;
    const int rows_b = min(128, rows_o - blk * 128);
    fence_acq_rel_sys();
    uint32_t* c = p.blk_ctr + owner * p.blk_cap + blk;
    const uint32_t old = atomicAdd(c, 1u);
    if (old == static_cast<uint32_t>(rows_b) - 1u) {
      *c = 0;
      red_release_sys_add(reinterpret_cast<uint32_t*>(t.data[owner] + p.s.ctr_off) + par, static_cast<uint32_t>(rows_b));
    }
  }
}

struct EpReduceParams {
  RsLink s;
  const int* ids_local;          // [my_rows][k]: this rank's own routing decides which sources contributed
  int M, k, d, experts_per_rank;
  __nv_bfloat16* out; long long ldo;
};

__global__ void __launch_bounds__(256) ep_combine_reduce_kernel(const EpReduceParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const PeerTable& t = p.s.t;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.s.words) + 1;
  const int par = static_cast<int>(e & 1u);
  const int R = p.s.rows_per_rank;
  const int my_rows = max(0, min(R, p.M - t.rank * R));
  __shared__ int good;
  __shared__ int need_s[MAX_RANKS];
  uint32_t* ctr = reinterpret_cast<uint32_t*>(t.data[t.rank] + p.s.ctr_off) + par;
  if (threadIdx.x == 0)
    good = (my_rows == 0 || wait_flag_ge(ctr, static_cast<uint32_t>(t.world) * my_rows, p.s.status, p.s.limit_ns)) ? 1 : 0;
  __syncthreads();
  if (good) {
    const uint8_t* base = t.data[t.rank] + p.s.recv_off[par];
    const size_t src_stride = static_cast<size_t>(p.s.r_cap) * p.d * 2;
    for (int row = blockIdx.x; row < my_rows; row += gridDim.x) {
      if (threadIdx.x < MAX_RANKS) need_s[threadIdx.x] = 0;
      __syncthreads();
      if (threadIdx.x < p.k) {
        const int dst = p.ids_local[static_cast<size_t>(row) * p.k + threadIdx.x] / p.experts_per_rank;
        if (dst >= 0 && dst < t.world) need_s[dst] = 1;
      }
      __syncthreads();
      for (int c = threadIdx.x; c < p.d / 8; c += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 x[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < t.world && need_s[r]) x[r] = ld_peer_16B(base + r * src_stride + (static_cast<size_t>(row) * p.d + c * 8) * 2);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < t.world && need_s[r]) add_bf16x8_to_f32(x[r], acc);
        *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(row) * p.ldo + c * 8) = pack_f32x8_to_bf16(acc);
      }
      __syncthreads();
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(p.s.words + 1, 1u);
    if (old == gridDim.x - 1) {
      p.s.words[1] = 0;
      *ctr = 0;
      p.s.words[0] = e;
      __threadfence();
    }
  }
}

static void fill_table_ep(PeerTable& t, void* const* peer_data, int world, int rank) {
  for (int r = 0; r < MAX_RANKS; ++r) {
    t.data[r] = r < world ? static_cast<uint8_t*>(peer_data[r]) : nullptr;
    t.flags[r] = nullptr;
  }
  t.mc = nullptr; t.world = world; t.rank = rank;
}

}  // namespace b200

using namespace b200;

static unsigned long long ep_limit(int limit_ms) { return static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull; }

extern "C" int b200_ep_dispatch(const void* xq_local, const float* sx_local, const int* ids_local, const float* wts_local,
                                int M, int K, int k, int experts_per_rank, int rows_per_rank, void* const* peer_data,
                                int world, int rank, size_t q_off0, size_t q_off1, size_t s_off0, size_t s_off1,
                                size_t ids_off0, size_t ids_off1, size_t wts_off0, size_t wts_off1, size_t flag_off,
                                size_t done_off, int blk_cap, void* words, void* row_ctr, int* status, int limit_ms,
                                cudaStream_t stream) {
  if (M <= 0 || K <= 0 || (K % 16) || k < 1 || k > EP_KMAX || experts_per_rank < 1 || world < 1 || world > MAX_RANKS ||
      rank < 0 || rank >= world || rows_per_rank <= 0 || static_cast<long long>(rows_per_rank) * world < M) return -1;
  if ((rows_per_rank + 127) / 128 > blk_cap) return -1;
  if ((q_off0 | q_off1 | s_off0 | s_off1 | ids_off0 | ids_off1 | wts_off0 | wts_off1 | flag_off | done_off) % 16) return -2;
  EpDispatchParams p = {};
  fill_table_ep(p.g.t, peer_data, world, rank);
  p.g.q_off[0] = q_off0; p.g.q_off[1] = q_off1; p.g.s_off[0] = s_off0; p.g.s_off[1] = s_off1;
  p.g.flag_off = flag_off; p.g.done_off = done_off; p.g.words = static_cast<uint32_t*>(words);
  p.g.row_ctr = static_cast<uint32_t*>(row_ctr); p.g.blk_cap = blk_cap; p.g.rows_per_rank = rows_per_rank;
  p.g.status = status; p.g.limit_ns = ep_limit(limit_ms);
  p.ids_off[0] = ids_off0; p.ids_off[1] = ids_off1; p.wts_off[0] = wts_off0; p.wts_off[1] = wts_off1;
  p.xq_local = static_cast<const int8_t*>(xq_local); p.sx_local = sx_local; p.ids_local = ids_local; p.wts_local = wts_local;
  p.M = M; p.K = K; p.k = k; p.experts_per_rank = experts_per_rank;
  int my_rows = M - rank * rows_per_rank;
  if (my_rows > rows_per_rank) my_rows = rows_per_rank;
  if (my_rows <= 0) return 0;
  launch_ex(ep_dispatch_kernel, dim3(my_rows), dim3(128), 0, stream, 0, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_ep_wait(void* const* peer_data, int world, int rank, size_t ids_off0, size_t ids_off1, size_t wts_off0,
                            size_t wts_off1, size_t flag_off, int blk_cap, int rows_per_rank, int M, int k, void* words,
                            int* ids_out, float* wts_out, int* status, int limit_ms, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || M <= 0 || k < 1 || k > EP_KMAX) return -1;
  AgLink g = {};
  fill_table_ep(g.t, peer_data, world, rank);
  g.flag_off = flag_off; g.blk_cap = blk_cap; g.rows_per_rank = rows_per_rank; g.words = static_cast<uint32_t*>(words);
  g.status = status; g.limit_ns = ep_limit(limit_ms);
  int ctas = (M * k + 255) / 256;
  if (ctas > 64) ctas = 64;
  launch_ex(ep_wait_kernel, dim3(ctas), dim3(256), 0, stream, 0, g, ids_off0, ids_off1, wts_off0, wts_off1, M, k, ids_out, wts_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_ep_gather(const void* heap_base, size_t q_off0, size_t q_off1, size_t s_off0, size_t s_off1,
                              const void* words, int d, const int* slot_token, const int* meta, int max_slots,
                              void* xq_perm, float* sx_perm, cudaStream_t stream) {
  if (max_slots <= 0) return 0;
  if (d % 16) return -1;
  launch_ex(ep_gather_kernel, dim3(max_slots), dim3(128), 0, stream, 0, static_cast<const uint8_t*>(heap_base), q_off0, q_off1,
            s_off0, s_off1, static_cast<const uint32_t*>(words), d, slot_token, meta, static_cast<int8_t*>(xq_perm), sx_perm);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_ep_combine_scatter(const void* y, long long ldy, const int* inv, const float* wts, int M, int k, int d,
                                       int rows_per_rank, void* const* peer_data, int world, int rank, size_t recv_off0,
                                       size_t recv_off1, size_t ctr_off, int r_cap, void* words, void* blk_ctr, int blk_cap,
                                       int* status, int limit_ms, cudaStream_t stream) {
  if (M <= 0 || k < 1 || k > 32 || (d % 8) || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank > r_cap || static_cast<long long>(rows_per_rank) * world < M) return -1;
  if ((rows_per_rank + 127) / 128 > blk_cap) return -1;
  EpCombineParams p = {};
  fill_table_ep(p.s.t, peer_data, world, rank);
  p.s.recv_off[0] = recv_off0; p.s.recv_off[1] = recv_off1; p.s.ctr_off = ctr_off; p.s.words = static_cast<uint32_t*>(words);
  p.s.r_cap = r_cap; p.s.rows_per_rank = rows_per_rank; p.s.status = status; p.s.limit_ns = ep_limit(limit_ms);
  p.y = static_cast<const __nv_bfloat16*>(y); p.ldy = ldy; p.inv = inv; p.wts = wts;
  p.blk_ctr = static_cast<uint32_t*>(blk_ctr); p.blk_cap = blk_cap; p.M = M; p.k = k; p.d = d;
  launch_ex(ep_combine_scatter_kernel, dim3(M), dim3(256), 0, stream, 0, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

extern "C" int b200_ep_combine_reduce(const int* ids_local, int M, int k, int d, int experts_per_rank, int rows_per_rank,
                                      void* const* peer_data, int world, int rank, size_t recv_off0, size_t recv_off1,
                                      size_t ctr_off, int r_cap, void* words, void* out, long long ldo, int* status,
                                      int limit_ms, int num_sms, cudaStream_t stream) {
  if (M <= 0 || k < 1 || k > 32 || (d % 8) || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (rows_per_rank <= 0 || rows_per_rank > r_cap) return -1;
  EpReduceParams p = {};
  fill_table_ep(p.s.t, peer_data, world, rank);
  p.s.recv_off[0] = recv_off0; p.s.recv_off[1] = recv_off1; p.s.ctr_off = ctr_off; p.s.words = static_cast<uint32_t*>(words);
  p.s.r_cap = r_cap; p.s.rows_per_rank = rows_per_rank; p.s.status = status; p.s.limit_ns = ep_limit(limit_ms);
  p.ids_local = ids_local; p.M = M; p.k = k; p.d = d; p.experts_per_rank = experts_per_rank;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  int my_rows = M - rank * rows_per_rank;
  if (my_rows > rows_per_rank) my_rows = rows_per_rank;
  int ctas = my_rows < 1 ? 1 : (my_rows < 2 * num_sms ? my_rows : 2 * num_sms);
  launch_ex(ep_combine_reduce_kernel, dim3(ctas), dim3(256), 0, stream, 0, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
