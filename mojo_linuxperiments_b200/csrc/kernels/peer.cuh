// Device-side building blocks for collectives over peer-mapped (symmetric) memory.
//
// Every rank maps the same-sized allocation of every other rank; `PeerTable` carries the per-rank base pointers of
// the data heap and of the flag block, plus the NVLS multicast mapping of the data heap when there is one.
// Signals are monotonically increasing epochs (never reset), written with st.release.sys into the *receiver's*
// flag block and polled with ld.acquire.sys; a wait gives up after limit_ns and records ST_TIMEOUT_PEER_FLAG.
// This is the GPU form of the reference's MutexGate (threading/linux_threading.mojo:174-198) and of its join-all
// barrier (test_linux_threading.mojo:533-534), without their unbounded waits.
#pragma once
#include "ptx.cuh"
#include "fabric/protocol.h"

namespace b200 {

constexpr int MAX_RANKS = 8;
constexpr int FLAG_KINDS = 4;               // independent flag rows per rank (ready, done, round flags, ...)
constexpr int FLAGS_PER_RANK = FLAG_KINDS * 16;   // uint32 words per flag block row, padded

struct PeerTable {
  uint8_t* data[MAX_RANKS];                 // base of rank r's symmetric heap as mapped on this GPU
  uint32_t* flags[MAX_RANKS];               // base of rank r's flag block as mapped on this GPU
  uint8_t* mc;                              // multicast (NVLS) mapping of the heap, or nullptr
  int world, rank;
};

// flag word `src` of row `kind` in the block of the receiver
__device__ __forceinline__ uint32_t* flag_ptr(const PeerTable& t, int receiver, int kind, int src) {
  return t.flags[receiver] + kind * 16 + src;
}

// one thread per destination rank: tell every rank (including ourselves) that we reached `epoch`
__device__ __forceinline__ void signal_all(const PeerTable& t, int kind, uint32_t epoch, int lane) {
  if (lane < t.world) st_release_sys(flag_ptr(t, lane, kind, t.rank), epoch);
}
// Same without the release fence: for signals that publish no data of this kernel ("the buffers an earlier kernel
// of my stream wrote are ready" - kernel completion already made them visible - or "I have finished reading").
__device__ __forceinline__ void signal_all_relaxed(const PeerTable& t, int kind, uint32_t epoch, int lane) {
  if (lane < t.world) st_relaxed_sys(flag_ptr(t, lane, kind, t.rank), epoch);
}
// one thread per source rank: wait until every rank reached `epoch`; returns false on timeout (lanes >= world: true)
__device__ __forceinline__ bool wait_all(const PeerTable& t, int kind, uint32_t epoch, int lane, int* status, uint64_t limit_ns) {
  if (lane >= t.world) return true;
  return wait_flag_ge(flag_ptr(t, t.rank, kind, lane), epoch, status, limit_ns);
}

// ---- NVLS (multimem) primitives: the switch reduces / broadcasts ----
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16B(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 8-byte "LL" words {payload, flag}: one store carries data and its own arrival flag, so no fence or separate
// signal is needed; the receiver polls the word until the flag equals the epoch it expects.
__device__ __forceinline__ void st_ll_peer(void* p, uint32_t payload, uint32_t flag) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(flag) : "memory");
}
__device__ __forceinline__ void multimem_st_ll(void* mc_addr, uint32_t payload, uint32_t flag) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};"
               ::"l"(mc_addr), "f"(__uint_as_float(payload)), "f"(__uint_as_float(flag)) : "memory");
}
__device__ __forceinline__ uint2 ld_ll(const void* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// ---- plain peer loads ----
__device__ __forceinline__ uint4 ld_peer_16B(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void add_bf16x8_to_f32(const uint4& raw, float (&acc)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(w[i] << 16);
    acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack_f32x8_to_bf16(const float (&acc)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 pb = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&pb);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Sum of the same 16-byte bf16x8 vector of every rank's heap at byte offset `off`, ranks visited in a fixed order
// so that every rank computes bit-identical results.
__device__ __forceinline__ void reduce_p2p_bf16x8(const PeerTable& t, size_t off, float (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  uint4 v[MAX_RANKS];
#pragma unroll
  for (int r = 0; r < MAX_RANKS; ++r)
    if (r < t.world) v[r] = ld_peer_16B(t.data[r] + off);
#pragma unroll
  for (int r = 0; r < MAX_RANKS; ++r)
    if (r < t.world) add_bf16x8_to_f32(v[r], acc);
}

}  // namespace b200
