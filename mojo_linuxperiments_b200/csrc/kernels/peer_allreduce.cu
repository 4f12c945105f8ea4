// All-reduce (sum) over peer-mapped memory, one kernel per call, several algorithms:
//   0  one-shot, plain peer loads: every rank reads every rank's contribution (latency-optimal for small messages)
//   1  one-shot NVLS: multimem.ld_reduce lets the NVSwitch add the eight copies, each rank receives only the sum
//   2  two-shot NVLS: each rank reduces 1/world of the message through the switch and multimem.st broadcasts it
//      (bandwidth-optimal), result written back in place into every rank's heap
//   3  chain towards rank 0 (reference: test_linux_threading.mojo:400-476): rank r waits for r+1, adds, signals r-1
//   4  butterfly / recursive doubling (reference: test_linux_threading.mojo:478-553): log2(world) exchange rounds
// Contributions live in each rank's symmetric heap at the same offset.  dtype: 0 bf16, 1 fp32, 2 fp64 (algorithms
// 3 and 4 and fp64 use plain peer loads).  Epochs come from a device-resident counter that the kernel advances, so a
// captured launch can be replayed without host involvement.
#include "peer.cuh"
#include "api.h"
#include "launch.cuh"

namespace b200 {

struct ArParams {
  PeerTable t;
  size_t in_off;            // byte offset of the contribution inside the heap
  size_t scratch_off;       // byte offset of per-round scratch inside the heap (algorithms 3, 4): world * 16 bytes... rounds * n
  void* out;                // local output (may be nullptr for in-place algorithm 2)
  const void* residual;     // optional bf16 addend (dtype 0 only)
  size_t n;                 // elements
  int dtype, algo;
  uint32_t* epoch;          // device counter: [0] epoch, [1] exit counter
  int* status;
  unsigned long long limit_ns;
  int trailing_barrier;     // 1: do not return before every rank finished reading (the heap region may be reused at once)
};

__device__ __forceinline__ void finish_launch(const ArParams& p, uint32_t epochs_used) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(p.epoch + 1, 1u);
    if (old == gridDim.x - 1) {
      p.epoch[1] = 0;
      p.epoch[0] += epochs_used;
      __threadfence();
    }
  }
}

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const ArParams p) {
  pdl_launch_dependents();   // the next kernel may start its prologue now
  pdl_wait();                // everything before this kernel in the stream has completed

  const PeerTable& t = p.t;
  {
    // debug build: the message and (low-latency form) the receive slots must lie inside the heap on every rank; a
    // launch that would not is recorded and does nothing (its peers run into their bounded waits)
    const size_t esz = p.dtype == 0 ? 2 : (p.dtype == 1 ? 4 : 8);
    bool fine = B200_DBG_RANGE(p.in_off, p.n * esz, p.status);
    if (p.algo == 5) fine = B200_DBG_RANGE(p.scratch_off, 2 * static_cast<size_t>(t.world) * (p.n / 2) * 8, p.status) && fine;
    if (!fine) return;
  }
  const uint32_t e0 = *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1;     // same on every CTA: bumped only at exit
  const int tid = threadIdx.x;
  __shared__ int ok_s;
  if (tid == 0) ok_s = 1;
  __syncthreads();

  if (p.algo == 5) {
    // Low-latency form for small bf16 messages: no barrier at all.  Every rank pushes its contribution as 8-byte
    // {2 x bf16, epoch} words into slot (epoch & 1) of every rank's receive area ([source][n/2] words at scratch_off)
    // and sums the world copies that arrive in its own.  The contribution was written by earlier kernels of the stream.
    const size_t nw = p.n / 2;
    const size_t src_stride = nw * 8;
    const size_t slot = p.scratch_off + static_cast<size_t>(e0 & 1) * t.world * src_stride;
    const uint32_t* mine_in = reinterpret_cast<const uint32_t*>(t.data[t.rank] + p.in_off);
    const size_t g0 = static_cast<size_t>(blockIdx.x) * blockDim.x + tid, gs = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = g0; i < nw; i += gs) {
      const size_t off = slot + t.rank * src_stride + i * 8;
      const uint32_t payload = mine_in[i];
      if (t.mc) multimem_st_ll(t.mc + off, payload, e0);
      else for (int r = 0; r < t.world; ++r) st_ll_peer(t.data[r] + off, payload, e0);
    }
    const uint8_t* mine = t.data[t.rank] + slot;
    const uint64_t t_start = globaltimer_ns();
    bool good = true;
    for (size_t i = g0; i < nw && good; i += gs) {
      uint2 v[MAX_RANKS];
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) if (r < t.world) v[r] = ld_ll(mine + r * src_stride + i * 8);
      uint32_t spins = 0;
      while (good) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < t.world && v[r].y != e0) { all = false; v[r] = ld_ll(mine + r * src_stride + i * 8); }
        if (all) break;
        if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > p.limit_ns) {
          if (p.status) atomicCAS(p.status, 0, (int)ST_TIMEOUT_PEER_FLAG);
          good = false;
        }
      }
      if (!good) break;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) if (r < t.world) { a0 += __uint_as_float(v[r].x << 16); a1 += __uint_as_float(v[r].x & 0xffff0000u); }
      if (p.residual) {
        const __nv_bfloat162 rb = reinterpret_cast<const __nv_bfloat162*>(p.residual)[i];
        a0 += __low2float(rb); a1 += __high2float(rb);
      }
      reinterpret_cast<__nv_bfloat162*>(p.out)[i] = __floats2bfloat162_rn(a0, a1);
    }
    finish_launch(p, 1);
    return;
  }

  // ---- barrier: every rank's contribution is in place.  The contribution was written by earlier kernels of this
  // stream, whose completion made it visible, so the signal needs no fence of its own. ----
  if (blockIdx.x == 0 && tid < 32) signal_all_relaxed(t, 0, e0, tid);
  if (tid < 32) { if (!wait_all(t, 0, e0, tid, p.status, p.limit_ns)) ok_s = 0; }
  __syncthreads();
  const bool ok = ok_s != 0;

  const size_t esz = p.dtype == 0 ? 2 : (p.dtype == 1 ? 4 : 8);
  const size_t nvec = p.n * esz / 16;                                       // whole 16-byte vectors
  const size_t gtid = static_cast<size_t>(blockIdx.x) * blockDim.x + tid, gsz = static_cast<size_t>(gridDim.x) * blockDim.x;

  if (ok && p.algo == 0) {
    for (size_t i = gtid; i < nvec; i += gsz) {
      const size_t off = p.in_off + i * 16;
      if (p.dtype == 0) {
        float acc[8];
        reduce_p2p_bf16x8(t, off, acc);
        if (p.residual) add_bf16x8_to_f32(*reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.residual) + i * 16), acc);
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + i * 16) = pack_f32x8_to_bf16(acc);
      } else if (p.dtype == 1) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < t.world; ++r) {
          const uint4 v = ld_peer_16B(t.data[r] + off);
          a.x += __uint_as_float(v.x); a.y += __uint_as_float(v.y); a.z += __uint_as_float(v.z); a.w += __uint_as_float(v.w);
        }
        *reinterpret_cast<float4*>(static_cast<uint8_t*>(p.out) + i * 16) = a;
      } else {
        double a0 = 0.0, a1 = 0.0;
        for (int r = 0; r < t.world; ++r) {
          const uint4 v = ld_peer_16B(t.data[r] + off);
          a0 += __hiloint2double(static_cast<int>(v.y), static_cast<int>(v.x));
          a1 += __hiloint2double(static_cast<int>(v.w), static_cast<int>(v.z));
        }
        double* o = reinterpret_cast<double*>(static_cast<uint8_t*>(p.out) + i * 16);
        o[0] = a0; o[1] = a1;
      }
    }
    // tail elements (message not a multiple of 16 bytes)
    const size_t done = nvec * 16 / esz;
    for (size_t i = done + gtid; i < p.n; i += gsz) {
      if (p.dtype == 0) {
        float a = 0.f;
        for (int r = 0; r < t.world; ++r) a += __bfloat162float(*reinterpret_cast<const volatile __nv_bfloat16*>(t.data[r] + p.in_off + i * 2));
        if (p.residual) a += __bfloat162float(static_cast<const __nv_bfloat16*>(p.residual)[i]);
        static_cast<__nv_bfloat16*>(p.out)[i] = __float2bfloat16(a);
      } else if (p.dtype == 1) {
        float a = 0.f;
        for (int r = 0; r < t.world; ++r) a += *reinterpret_cast<const volatile float*>(t.data[r] + p.in_off + i * 4);
        static_cast<float*>(p.out)[i] = a;
      } else {
        double a = 0.0;
        for (int r = 0; r < t.world; ++r) a += *reinterpret_cast<const volatile double*>(t.data[r] + p.in_off + i * 8);
        static_cast<double*>(p.out)[i] = a;
      }
    }
  } else if (ok && p.algo == 1) {
    for (size_t i = gtid; i < nvec; i += gsz) {
      const uint8_t* a = t.mc + p.in_off + i * 16;
      if (p.dtype == 0) {
        uint4 v = multimem_ld_reduce_bf16x8(a);
        if (p.residual) {
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          add_bf16x8_to_f32(v, acc);
          add_bf16x8_to_f32(*reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.residual) + i * 16), acc);
          v = pack_f32x8_to_bf16(acc);
        }
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + i * 16) = v;
      } else {
        *reinterpret_cast<float4*>(static_cast<uint8_t*>(p.out) + i * 16) = multimem_ld_reduce_f32x4(a);
      }
    }
  } else if (ok && p.algo == 2) {
    // my slice of the vectors: [v0, v1)
    const size_t v0 = nvec * t.rank / t.world, v1 = nvec * (t.rank + 1) / t.world;
    size_t i = v0 + gtid;
    if (p.dtype == 0) {
      for (; i + gsz < v1; i += 2 * gsz) {                 // two independent vectors in flight per thread
        uint8_t* a = t.mc + p.in_off + i * 16;
        uint8_t* b = a + gsz * 16;
        const uint4 va = multimem_ld_reduce_bf16x8(a), vb = multimem_ld_reduce_bf16x8(b);
        multimem_st_16B(a, va);
        multimem_st_16B(b, vb);
      }
    }
    for (; i < v1; i += gsz) {
      uint8_t* a = t.mc + p.in_off + i * 16;
      if (p.dtype == 0) {
        multimem_st_16B(a, multimem_ld_reduce_bf16x8(a));
      } else {
        const float4 f = multimem_ld_reduce_f32x4(a);
        multimem_st_16B(a, make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w)));
      }
    }
    // every rank has broadcast its slice: second barrier, then (optionally) copy out with the residual
    __threadfence_system();
    __syncthreads();
    // the barrier must cover all CTAs of this rank: count them on the exit counter's sibling word
    if (tid == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(p.epoch + 2, 1u);
      if (old == gridDim.x - 1) {
        p.epoch[2] = 0;
        __threadfence_system();
        for (int r = 0; r < t.world; ++r) st_relaxed_sys(flag_ptr(t, r, 1, t.rank), e0);
      }
    }
    if (tid < 32) { if (!wait_all(t, 1, e0, tid, p.status, p.limit_ns)) ok_s = 0; }
    __syncthreads();
    if (ok_s && p.out) {
      for (size_t i = gtid; i < nvec; i += gsz) {
        uint4 v = ld_peer_16B(t.data[t.rank] + p.in_off + i * 16);
        if (p.dtype == 0 && p.residual) {
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          add_bf16x8_to_f32(v, acc);
          add_bf16x8_to_f32(*reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.residual) + i * 16), acc);
          v = pack_f32x8_to_bf16(acc);
        }
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + i * 16) = v;
      }
    }
  } else if (ok && (p.algo == 3 || p.algo == 4) && blockIdx.x == 0) {
    // small messages only (scalars to a few KB), fp32 / fp64, handled by one CTA.
    // scratch layout in every heap: slot k (k = 0..rounds) holds the running value after k rounds, n elements each
    const size_t bytes = p.n * esz;
    auto slot = [&](int r, int k) { return t.data[r] + p.scratch_off + static_cast<size_t>(k) * bytes; };
    // slot 0 = own contribution
    for (size_t i = tid; i < p.n; i += blockDim.x) {
      if (p.dtype == 1) reinterpret_cast<float*>(slot(t.rank, 0))[i] = *reinterpret_cast<const float*>(t.data[t.rank] + p.in_off + i * 4);
      else reinterpret_cast<double*>(slot(t.rank, 0))[i] = *reinterpret_cast<const double*>(t.data[t.rank] + p.in_off + i * 8);
    }
    __threadfence_system();
    __syncthreads();
    if (p.algo == 3) {
      // chain: kind-2 flag word 0 of rank r is written by rank r+1 once its running sum (slot 1) is final
      const int up = chain_upstream(t.rank, t.world), down = chain_downstream(t.rank);
      bool good = true;
      if (up >= 0) {
        if (tid == 0) good = wait_flag_ge(flag_ptr(t, t.rank, 2, 0), e0, p.status, p.limit_ns);
        good = __syncthreads_and(good ? 1 : 0) != 0;
      }
      for (size_t i = tid; i < p.n && good; i += blockDim.x) {
        if (p.dtype == 1) {
          float a = reinterpret_cast<const float*>(slot(t.rank, 0))[i];
          if (up >= 0) a += *reinterpret_cast<const volatile float*>(slot(up, 1) + i * 4);
          reinterpret_cast<float*>(slot(t.rank, 1))[i] = a;
          if (t.rank == 0 && p.out) static_cast<float*>(p.out)[i] = a;
        } else {
          double a = reinterpret_cast<const double*>(slot(t.rank, 0))[i];
          if (up >= 0) a += *reinterpret_cast<const volatile double*>(slot(up, 1) + i * 8);
          reinterpret_cast<double*>(slot(t.rank, 1))[i] = a;
          if (t.rank == 0 && p.out) static_cast<double*>(p.out)[i] = a;
        }
      }
      __threadfence_system();
      __syncthreads();
      if (tid == 0 && down >= 0) st_release_sys(flag_ptr(t, down, 2, 0), e0);
    } else {
      const int rounds = butterfly_rounds(t.world);
      bool good = is_pow2(t.world);
      for (int k = 0; k < rounds && good; ++k) {
        const int partner = butterfly_partner(t.rank, k);
        // tell the partner that my slot k is final, wait for the partner's
        if (tid == 0) {
          st_release_sys(flag_ptr(t, partner, 2, 1 + k), e0);
          good = wait_flag_ge(flag_ptr(t, t.rank, 2, 1 + k), e0, p.status, p.limit_ns);
        }
        good = __syncthreads_and(good ? 1 : 0) != 0;
        if (!good) break;
        for (size_t i = tid; i < p.n; i += blockDim.x) {
          if (p.dtype == 1) {
            const float a = reinterpret_cast<const float*>(slot(t.rank, k))[i], b = *reinterpret_cast<const volatile float*>(slot(partner, k) + i * 4);
            // add in rank order so both partners round identically
            reinterpret_cast<float*>(slot(t.rank, k + 1))[i] = (t.rank < partner) ? a + b : b + a;
          } else {
            const double a = reinterpret_cast<const double*>(slot(t.rank, k))[i], b = *reinterpret_cast<const volatile double*>(slot(partner, k) + i * 8);
            reinterpret_cast<double*>(slot(t.rank, k + 1))[i] = (t.rank < partner) ? a + b : b + a;
          }
        }
        __threadfence_system();
        __syncthreads();
      }
      if (good && p.out) {
        for (size_t i = tid; i < p.n; i += blockDim.x) {
          if (p.dtype == 1) static_cast<float*>(p.out)[i] = reinterpret_cast<const float*>(slot(t.rank, rounds))[i];
          else static_cast<double*>(p.out)[i] = reinterpret_cast<const double*>(slot(t.rank, rounds))[i];
        }
      }
    }
  }

  if (p.trailing_barrier) {
    // nobody may overwrite its contribution before every rank has finished reading it
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(p.epoch + 3, 1u);
      if (old == gridDim.x - 1) {
        p.epoch[3] = 0;
        for (int r = 0; r < t.world; ++r) st_relaxed_sys(flag_ptr(t, r, 3, t.rank), e0);      // "done reading": no data to publish
      }
    }
    if (blockIdx.x == 0 && tid < 32) wait_all(t, 3, e0, tid, p.status, p.limit_ns);
  }
  finish_launch(p, 1);
}

// Greedy sampling across vocabulary shards: every rank has written its candidates (fp32 value, int64 index) for each
// row into its heap ([ncand][rows] values at val_off, indices at idx_off); after the barrier every rank reads all
// world*ncand candidates and keeps the largest value (lowest index on ties), so all ranks agree without a broadcast.
struct ArgmaxParams {
  PeerTable t;
  size_t val_off, idx_off;       // val_off: receive area (2 slots x world x rows x 16 bytes); idx_off unused
  const float* cand_val;         // local candidates [ncand][rows]
  const long long* cand_idx;
  int ncand, rows;
  long long* out_idx;
  uint32_t* epoch;
  int* status;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(128) peer_argmax_kernel(const ArgmaxParams p) {
  pdl_launch_dependents();
  pdl_wait();
  // Low-latency exchange: every rank reduces its own candidates to one (value, index) per row, pushes it as two
  // 8-byte {payload, epoch} words into every rank's receive area and picks the best of the world pairs that arrive
  // in its own - one NVLink trip, no barrier.  Receive area: val_off, two slots by epoch parity, [source][row][2].
  const PeerTable& t = p.t;
  const uint32_t e0 = *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1;
  const size_t src_stride = static_cast<size_t>(p.rows) * 16;
  const size_t slot = p.val_off + static_cast<size_t>(e0 & 1) * t.world * src_stride;
  if (!B200_DBG_RANGE(p.val_off, 2 * static_cast<size_t>(t.world) * src_stride, p.status)) return;
  const uint64_t t_start = globaltimer_ns();
  for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
    float best = -INFINITY;
    long long bi = 0x7fffffffll;
    for (int c = 0; c < p.ncand; ++c) {
      const float val = p.cand_val[static_cast<size_t>(c) * p.rows + r];
      const long long idx = p.cand_idx[static_cast<size_t>(c) * p.rows + r];
      if (val > best || (val == best && idx < bi)) { best = val; bi = idx; }
    }
    const size_t off = slot + t.rank * src_stride + static_cast<size_t>(r) * 16;
    for (int w = 0; w < t.world; ++w) {
      st_ll_peer(t.data[w] + off, __float_as_uint(best), e0);
      st_ll_peer(t.data[w] + off + 8, static_cast<uint32_t>(bi), e0);
    }
  }
  for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
    float best = -INFINITY;
    long long bi = 0x7fffffffll;
    bool good = true;
    for (int w = 0; w < t.world && good; ++w) {
      const uint8_t* src = t.data[t.rank] + slot + w * src_stride + static_cast<size_t>(r) * 16;
      uint2 a = ld_ll(src), b = ld_ll(src + 8);
      uint32_t spins = 0;
      while (a.y != e0 || b.y != e0) {
        if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > p.limit_ns) {
          if (p.status) atomicCAS(p.status, 0, (int)ST_TIMEOUT_PEER_FLAG);
          good = false;
          break;
        }
        a = ld_ll(src); b = ld_ll(src + 8);
      }
      if (!good) break;
      const float val = __uint_as_float(a.x);
      const long long idx = static_cast<long long>(b.x);
      if (val > best || (val == best && idx < bi)) { best = val; bi = idx; }
    }
    p.out_idx[r] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence(); p.epoch[0] = e0; }
}

}  // namespace b200

using namespace b200;

// cand_val / cand_idx: this rank's local candidates [ncand][rows] (ordinary device memory); recv_off: byte offset of a
// receive area of 2 * world * rows * 16 bytes in every heap.  Indices must fit 31 bits.
extern "C" int b200_peer_argmax(void* const* peer_data, void* const* peer_flags, int world, int rank, size_t recv_off,
                                const float* cand_val, const long long* cand_idx, int ncand, int rows, long long* out_idx,
                                void* epoch_words, int* status, int limit_ms, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rows <= 0 || ncand <= 0 || (recv_off % 8)) return -1;
  ArgmaxParams p;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.t.data[r] = r < world ? static_cast<uint8_t*>(peer_data[r]) : nullptr;
    p.t.flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  p.t.mc = nullptr; p.t.world = world; p.t.rank = rank;
  p.val_off = recv_off; p.idx_off = 0; p.cand_val = cand_val; p.cand_idx = cand_idx; p.ncand = ncand; p.rows = rows; p.out_idx = out_idx;
  p.epoch = static_cast<uint32_t*>(epoch_words); p.status = status;
  p.limit_ns = static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull;
  launch_ex(peer_argmax_kernel, dim3(1), dim3(128), 0, stream, 0, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}

// peer_data / peer_flags: host arrays [world] of device pointers (each rank's heap base and flag block as mapped here)
extern "C" int b200_peer_allreduce(void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                                   size_t in_off, size_t scratch_off, void* out, const void* residual, size_t n, int dtype,
                                   int algo, void* epoch_words, int* status, int limit_ms, int trailing_barrier, int max_ctas,
                                   cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || n == 0) return -1;
  if (dtype < 0 || dtype > 2 || algo < 0 || algo > 5) return -1;
  if (algo == 5 && (dtype != 0 || (n % 2) || !out || (scratch_off % 8))) return -3;
  if ((algo == 1 || algo == 2) && (!mc_base || dtype == 2)) return -3;
  if ((algo == 3 || algo == 4) && dtype == 0) return -3;
  if ((algo == 0 || algo == 1) && !out) return -1;
  if (in_off % 16) return -2;
  const size_t esz = dtype == 0 ? 2 : (dtype == 1 ? 4 : 8);
  if ((algo == 1 || algo == 2) && (n * esz) % 16) return -2;
  ArParams p;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.t.data[r] = r < world ? static_cast<uint8_t*>(peer_data[r]) : nullptr;
    p.t.flags[r] = r < world ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
  }
  p.t.mc = static_cast<uint8_t*>(mc_base); p.t.world = world; p.t.rank = rank;
  p.in_off = in_off; p.scratch_off = scratch_off; p.out = out; p.residual = residual; p.n = n; p.dtype = dtype; p.algo = algo;
  p.epoch = static_cast<uint32_t*>(epoch_words); p.status = status;
  p.limit_ns = static_cast<unsigned long long>(limit_ms > 0 ? limit_ms : 2000) * 1000000ull;
  p.trailing_barrier = trailing_barrier;
  const size_t nvec = (n * esz + 15) / 16;
  int ctas = static_cast<int>((nvec + 255) / 256);
  if (algo == 2) ctas = static_cast<int>((nvec / world + 255) / 256);
  if (algo >= 3) ctas = 1;
  if (ctas < 1) ctas = 1;
  if (max_ctas < 1) max_ctas = 64;
  if (ctas > max_ctas) ctas = max_ctas;        // every CTA spins on flags: keep the grid well inside one wave
  launch_ex(peer_allreduce_kernel, dim3(ctas), dim3(256), 0, stream, 0, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -2000 - static_cast<int>(e);
}
