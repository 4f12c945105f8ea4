#include "w8a8_host.hpp"

#include <immintrin.h>

#include <cstring>
#include <vector>

#include "heap_move_array.hpp"
#include "pool.hpp"
#include "sys.hpp"
#include "team.hpp"

namespace hostrt {

namespace {

inline float bf16_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return static_cast<uint16_t>((u >> 16) | ((u & 0xffffu) ? 0x40u : 0u));   // inf / nan
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

// in-place fast Walsh-Hadamard transform of 128 floats in Sylvester order, scaled by 1/sqrt(128)
inline void fwht128(float* v) {
  for (int h = 1; h < 128; h <<= 1)
    for (int i = 0; i < 128; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        const float a = v[j], b = v[j + h];
        v[j] = a + b;
        v[j + h] = a - b;
      }
  const float s = 0.08838834764831845f;
  for (int i = 0; i < 128; ++i) v[i] *= s;
}

struct QuantJob {
  const uint16_t* x; int K; int m0, m1;
  int8_t* q; uint8_t* qu; float* sx;
  int simd;                      // 1: AVX-512 rotation / quantisation (same butterflies, same bits as the scalar code)
};

// The same transform on eight 16-float registers: stages 1..8 inside a register (partner = lane ^ h through a
// permute, the lower element of a pair takes the sum, the upper one lower - upper), stages 16..64 between registers.
__attribute__((target("avx512f,avx512bw")))
inline void fwht128_avx512(__m512 (&z)[8]) {
  const __m512i lane = _mm512_set_epi32(15, 14, 13, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0);
  const __mmask16 upper[4] = {0xAAAA, 0xCCCC, 0xF0F0, 0xFF00};
  for (int st = 0; st < 4; ++st) {
    const __m512i idx = _mm512_xor_si512(lane, _mm512_set1_epi32(1 << st));
    for (int i = 0; i < 8; ++i) {
      const __m512 t = _mm512_permutexvar_ps(idx, z[i]);
      z[i] = _mm512_mask_blend_ps(upper[st], _mm512_add_ps(z[i], t), _mm512_sub_ps(t, z[i]));
    }
  }
  for (int h = 1; h < 8; h <<= 1)
    for (int i = 0; i < 8; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        const __m512 a = z[j], b = z[j + h];
        z[j] = _mm512_add_ps(a, b);
        z[j + h] = _mm512_sub_ps(a, b);
      }
  const __m512 s = _mm512_set1_ps(0.08838834764831845f);
  for (int i = 0; i < 8; ++i) z[i] = _mm512_mul_ps(z[i], s);
}

__attribute__((target("avx512f,avx512bw")))
inline void load_block_avx512(const uint16_t* xr, __m512 (&z)[8]) {
  for (int i = 0; i < 8; ++i) {
    const __m256i h = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(xr + 16 * i));
    z[i] = _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(h), 16));      // bf16 -> fp32
  }
}

__attribute__((target("avx512f,avx512bw")))
void quant_rows_avx512(const QuantJob& j) {
  for (int m = j.m0; m < j.m1; ++m) {
    const uint16_t* xr = j.x + static_cast<size_t>(m) * j.K;
    __m512 vmax = _mm512_setzero_ps();
    __m512 z[8];
    for (int b = 0; b < j.K; b += 128) {
      load_block_avx512(xr + b, z);
      fwht128_avx512(z);
      for (int i = 0; i < 8; ++i) vmax = _mm512_max_ps(vmax, _mm512_abs_ps(z[i]));
    }
    const float amax = _mm512_reduce_max_ps(vmax);
    const float s = amax > 0.f ? amax / 127.f : 1.f;
    j.sx[m] = s;
    const __m512 vs = _mm512_set1_ps(s);
    const __m512i lo = _mm512_set1_epi32(-127), hi = _mm512_set1_epi32(127), bias = _mm512_set1_epi32(128);
    int8_t* qr = j.q + static_cast<size_t>(m) * j.K;
    uint8_t* qur = j.qu + static_cast<size_t>(m) * j.K;
    for (int b = 0; b < j.K; b += 128) {
      load_block_avx512(xr + b, z);
      fwht128_avx512(z);
      for (int i = 0; i < 8; ++i) {
        __m512i qi = _mm512_cvtps_epi32(_mm512_div_ps(z[i], vs));            // round to nearest even
        qi = _mm512_min_epi32(_mm512_max_epi32(qi, lo), hi);
        _mm_storeu_si128(reinterpret_cast<__m128i*>(qr + b + 16 * i), _mm512_cvtepi32_epi8(qi));
        _mm_storeu_si128(reinterpret_cast<__m128i*>(qur + b + 16 * i), _mm512_cvtepi32_epi8(_mm512_add_epi32(qi, bias)));
      }
    }
  }
}

// rows [m0, m1): rotate, quantise, and also store the +128-biased copy the VNNI path multiplies
void quant_worker(uint64_t a0, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) {
  QuantJob& j = *reinterpret_cast<QuantJob*>(a0);
  if (j.simd) { quant_rows_avx512(j); return; }
  float blk[128];
  for (int m = j.m0; m < j.m1; ++m) {
    const uint16_t* xr = j.x + static_cast<size_t>(m) * j.K;
    float amax = 0.f;
    // pass 1: the row maximum of the rotated values
    for (int b = 0; b < j.K; b += 128) {
      for (int i = 0; i < 128; ++i) blk[i] = bf16_to_f32(xr[b + i]);
      fwht128(blk);
      for (int i = 0; i < 128; ++i) {           // no libm calls on pool threads
        const float a = blk[i] < 0.f ? -blk[i] : blk[i];
        amax = a > amax ? a : amax;
      }
    }
    const float s = amax > 0.f ? amax / 127.f : 1.f;
    j.sx[m] = s;
    // pass 2: quantise (the rotation is recomputed: it is cheap next to keeping K floats per row around)
    int8_t* qr = j.q + static_cast<size_t>(m) * j.K;
    uint8_t* qur = j.qu + static_cast<size_t>(m) * j.K;
    for (int b = 0; b < j.K; b += 128) {
      for (int i = 0; i < 128; ++i) blk[i] = bf16_to_f32(xr[b + i]);
      fwht128(blk);
      for (int i = 0; i < 128; ++i) {
        int qi = _mm_cvtss_si32(_mm_set_ss(blk[i] / s));      // round to nearest even (default MXCSR mode)
        qi = qi > 127 ? 127 : (qi < -127 ? -127 : qi);
        qr[b + i] = static_cast<int8_t>(qi);
        qur[b + i] = static_cast<uint8_t>(qi + 128);
      }
    }
  }
}

struct GemmJob {
  const int8_t* q; const uint8_t* qu; const float* sx;
  const int8_t* wq; const float* sw;
  uint16_t* y; int32_t* acc_out;
  int M, K, N, n0, n1, vnni;     // vnni: 0 scalar, 1 AVX-512 VNNI, 2 AMX int8 tiles
  const int8_t* q_pack;          // AMX: activations as [M/16 blocks][K/4][16 tokens][4] (zero padded)
};

inline void finish(const GemmJob& j, int m, int n, int32_t acc) {
  if (j.acc_out) j.acc_out[static_cast<size_t>(m) * j.N + n] = acc;
  j.y[static_cast<size_t>(m) * j.N + n] = f32_to_bf16_rne(static_cast<float>(acc) * (j.sw[n] * j.sx[m]));
}

void gemm_scalar(const GemmJob& j) {
  for (int n = j.n0; n < j.n1; ++n) {
    const int8_t* w = j.wq + static_cast<size_t>(n) * j.K;
    for (int m = 0; m < j.M; ++m) {
      const int8_t* q = j.q + static_cast<size_t>(m) * j.K;
      int32_t acc = 0;
      for (int k = 0; k < j.K; ++k) acc += static_cast<int32_t>(q[k]) * static_cast<int32_t>(w[k]);
      finish(j, m, n, acc);
    }
  }
}

constexpr int MB = 16;   // token rows per register block

__attribute__((target("avx512f,avx512bw,avx512vnni")))
void gemm_vnni(const GemmJob& j) {
  const __m512i ones = _mm512_set1_epi8(1);
  for (int n = j.n0; n < j.n1; ++n) {
    const int8_t* w = j.wq + static_cast<size_t>(n) * j.K;
    // 128 * sum_k w[k]: what the +128 bias of the activations adds to every dot product with this channel
    __m512i ws = _mm512_setzero_si512();
    for (int k = 0; k < j.K; k += 64) ws = _mm512_dpbusd_epi32(ws, ones, _mm512_loadu_si512(w + k));
    const int32_t corr = 128 * _mm512_reduce_add_epi32(ws);
    for (int m0 = 0; m0 < j.M; m0 += MB) {
      const int mb = j.M - m0 < MB ? j.M - m0 : MB;
      __m512i acc[MB];
      for (int i = 0; i < MB; ++i) acc[i] = _mm512_setzero_si512();
      for (int k = 0; k < j.K; k += 64) {
        const __m512i wv = _mm512_loadu_si512(w + k);
        for (int i = 0; i < mb; ++i)
          acc[i] = _mm512_dpbusd_epi32(acc[i], _mm512_loadu_si512(j.qu + static_cast<size_t>(m0 + i) * j.K + k), wv);
      }
      for (int i = 0; i < mb; ++i) finish(j, m0 + i, n, _mm512_reduce_add_epi32(acc[i]) - corr);
    }
  }
}

// AMX: C[16 channels][16 tokens] += W[16 channels][64 k] . A[16 k-groups][16 tokens x 4 k], signed x signed.  The
// weights are tile-loaded straight from their row-major layout (row stride K); four token blocks share one weight tile.
struct alignas(64) TileCfg {
  uint8_t palette, start_row, reserved[14];
  uint16_t colsb[16];
  uint8_t rows[16];
};

__attribute__((target("amx-tile,amx-int8,avx512f")))
void gemm_amx(const GemmJob& j) {
  TileCfg cfg{};
  cfg.palette = 1;
  for (int t = 0; t < 6; ++t) { cfg.colsb[t] = 64; cfg.rows[t] = 16; }
  _tile_loadconfig(&cfg);
  alignas(64) int32_t cbuf[4][16][16];
  alignas(64) int8_t wtail[16][64];
  const int mblocks = (j.M + 15) / 16;
  const size_t blk_stride = static_cast<size_t>(j.K / 4) * 64;      // bytes of one packed token block
  for (int n0 = j.n0; n0 < j.n1; n0 += 16) {
    const int nrows = j.n1 - n0 < 16 ? j.n1 - n0 : 16;
    for (int mb0 = 0; mb0 < mblocks; mb0 += 4) {
      const int nmb = mblocks - mb0 < 4 ? mblocks - mb0 : 4;
      _tile_zero(0); _tile_zero(1); _tile_zero(2); _tile_zero(3);
      for (int k = 0; k < j.K; k += 64) {
        if (nrows == 16) {
          _tile_loadd(4, j.wq + static_cast<size_t>(n0) * j.K + k, j.K);
        } else {                                                    // last, partial channel block: stage with zero rows
          for (int r = 0; r < 16; ++r)
            for (int c = 0; c < 64; ++c) wtail[r][c] = r < nrows ? j.wq[static_cast<size_t>(n0 + r) * j.K + k + c] : 0;
          _tile_loadd(4, wtail, 64);
        }
        const int8_t* a = j.q_pack + static_cast<size_t>(mb0) * blk_stride + static_cast<size_t>(k / 4) * 64;
        _tile_loadd(5, a, 64); _tile_dpbssd(0, 4, 5);
        if (nmb > 1) { _tile_loadd(5, a + blk_stride, 64); _tile_dpbssd(1, 4, 5); }
        if (nmb > 2) { _tile_loadd(5, a + 2 * blk_stride, 64); _tile_dpbssd(2, 4, 5); }
        if (nmb > 3) { _tile_loadd(5, a + 3 * blk_stride, 64); _tile_dpbssd(3, 4, 5); }
      }
      _tile_stored(0, cbuf[0], 64);
      if (nmb > 1) _tile_stored(1, cbuf[1], 64);
      if (nmb > 2) _tile_stored(2, cbuf[2], 64);
      if (nmb > 3) _tile_stored(3, cbuf[3], 64);
      for (int b = 0; b < nmb; ++b)
        for (int r = 0; r < nrows; ++r)
          for (int c = 0; c < 16; ++c) {
            const int m = (mb0 + b) * 16 + c;
            if (m < j.M) finish(j, m, n0 + r, cbuf[b][r][c]);
          }
    }
  }
  _tile_release();
}

void gemm_worker(uint64_t a0, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t) {
  const GemmJob& j = *reinterpret_cast<GemmJob*>(a0);
  if (j.vnni == 2 && (j.K % 64) == 0) gemm_amx(j);
  else if (j.vnni == 1 && (j.K % 64) == 0) gemm_vnni(j);
  else gemm_scalar(j);
}

}  // namespace

namespace {

// `run(fn, args)` executes fn(args[i]) on worker i for i < total and returns 0 or -errno
template <typename Run>
W8A8HostResult linear_core(int total, Run&& run, const uint16_t* x, int M, int K, const int8_t* wq, const float* sw, int N,
                           uint16_t* y, int force_scalar, int8_t* q_out, float* sx_out, int32_t* acc_out,
                           const NodeShardedWeights* shards = nullptr) {
  W8A8HostResult res{};
  if (M <= 0 || N <= 0 || K <= 0 || (K % 128) != 0 || !x || (!wq && !shards) || !sw || !y) { res.status = -err::kINVAL; return res; }
  if (shards && (shards->workers() != total || shards->N() != N || shards->K() != K)) { res.status = -err::kINVAL; return res; }
  if (total <= 0) { res.status = -err::kNOENT; return res; }
  res.workers = total;
  // force_scalar: 0 best available, 1 scalar, 2 at most AVX-512 VNNI
  res.used_vnni = (force_scalar != 1 && __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bw")) ? 1 : 0;
  if (res.used_vnni && force_scalar == 0 && __builtin_cpu_supports("amx-int8") && __builtin_cpu_supports("amx-tile")) {
    // the tile registers are an opt-in extended state: ask the kernel once for the whole process (ARCH_REQ_XCOMP_PERM,
    // feature 18 = XTILEDATA); without the permission the first tile instruction would fault
    if (raw_syscall(158 /* arch_prctl */, 0x1023, 18) == 0) res.used_vnni = 2;
  }

  std::vector<int8_t> q_own;
  std::vector<float> sx_own;
  int8_t* q = q_out;
  float* sx = sx_out;
  if (!q) { q_own.resize(static_cast<size_t>(M) * K); q = q_own.data(); }
  if (!sx) { sx_own.resize(M); sx = sx_own.data(); }
  std::vector<uint8_t> qu(static_cast<size_t>(M) * K);
  std::vector<uint64_t> args(total);

  // phase 1: rows split over the workers
  std::vector<QuantJob> qjobs(total);
  for (int w = 0; w < total; ++w) {
    qjobs[w] = QuantJob{x, K, static_cast<int>(static_cast<long>(M) * w / total), static_cast<int>(static_cast<long>(M) * (w + 1) / total), q, qu.data(), sx,
                        res.used_vnni ? 1 : 0};
    args[w] = reinterpret_cast<uint64_t>(&qjobs[w]);
  }
  long t0 = sys_clock_monotonic_ns();
  res.status = run(&quant_worker, args.data());
  res.quant_ns = sys_clock_monotonic_ns() - t0;
  if (res.status != 0) return res;

  // AMX wants the activations in groups of four k per token: [token block of 16][k / 4][token][4]
  std::vector<int8_t> q_pack;
  if (res.used_vnni == 2) {
    const int mblocks = (M + 15) / 16;
    q_pack.assign(static_cast<size_t>(mblocks) * (K / 4) * 64 + 64, 0);
    for (int m = 0; m < M; ++m)
      for (int k = 0; k < K; ++k)
        q_pack[(static_cast<size_t>(m / 16) * (K / 4) + k / 4) * 64 + (m % 16) * 4 + (k % 4)] = q[static_cast<size_t>(m) * K + k];
  }

  // phase 2: output channels split over the workers
  std::vector<GemmJob> gjobs(total);
  for (int w = 0; w < total; ++w) {
    gjobs[w] = GemmJob{q, qu.data(), sx, shards ? shards->base_for(w) : wq, sw, y, acc_out, M, K, N, static_cast<int>(static_cast<long>(N) * w / total),
                       static_cast<int>(static_cast<long>(N) * (w + 1) / total), res.used_vnni, q_pack.data()};
    args[w] = reinterpret_cast<uint64_t>(&gjobs[w]);
  }
  t0 = sys_clock_monotonic_ns();
  res.status = run(&gemm_worker, args.data());
  res.gemm_ns = sys_clock_monotonic_ns() - t0;
  return res;
}

}  // namespace

W8A8HostResult w8a8_linear_host(const NumaInfo& info, const uint16_t* x, int M, int K, const int8_t* wq, const float* sw,
                                int N, uint16_t* y, int max_workers_per_node, int force_scalar, int8_t* q_out,
                                float* sx_out, int32_t* acc_out) {
  const int nn = info.num_nodes();
  std::vector<int> per_node(nn > 0 ? nn : 0);
  int total = 0;
  for (int k = 0; k < nn; ++k) {
    int c = static_cast<int>(info.nodes()[k].cpu_ids.size());
    if (max_workers_per_node > 0 && c > max_workers_per_node) c = max_workers_per_node;
    per_node[k] = c;
    total += c;
  }
  HeapMoveArray<ThreadPool> pools(nn > 0 ? nn : 1);
  bool pools_ok = nn > 0;
  for (int k = 0; k < nn && pools_ok; ++k) {
    const int node = info.nodes()[k].id;
    auto m = info.get_node_mask<128>(node);
    pools.emplace(per_node[k], m.ptr(), size_t(128), node, stack_size::DEFAULT);
    if (!pools[k]) pools_ok = false;
  }
  if (!pools_ok) { W8A8HostResult r{}; r.status = nn > 0 ? -err::kNOMEM : -err::kNOENT; return r; }
  auto run = [&](WorkerFn fn, const uint64_t* args) -> long {        // one fresh thread per job, as the pool does it
    int w = 0;
    long st = 0;
    for (int k = 0; k < nn; ++k)
      for (int i = 0; i < per_node[k]; ++i, ++w)
        if (pools[k].launch(fn, args[w]) < 0) st = -err::kAGAIN;
    for (int k = 0; k < nn; ++k) if (pools[k].wait_all(120'000'000'000l) != 0) st = -err::kTIMEDOUT;
    return st;
  };
  return linear_core(total, run, x, M, K, wq, sw, N, y, force_scalar, q_out, sx_out, acc_out);
}

NodeShardedWeights::NodeShardedWeights(const WorkerTeam& team, const int8_t* wq, int N, int K)
    : arenas_(team.size() > 0 ? team.size() : 1), N_(N), K_(K) {
  const int total = team.size();
  if (total <= 0 || N <= 0 || K <= 0 || !wq) return;
  bases_.assign(total, nullptr);
  firsts_.assign(total, nullptr);
  nodes_.assign(total, -1);
  // one arena per run of consecutive workers on the same node (workers are ordered node by node)
  int w = 0;
  while (w < total) {
    int w_end = w;
    const int node = team.node_of(w);
    while (w_end < total && team.node_of(w_end) == node) ++w_end;
    const long n_lo = static_cast<long>(N) * w / total, n_hi = static_cast<long>(N) * w_end / total;
    const size_t bytes = static_cast<size_t>(n_hi - n_lo) * K;
    arenas_.emplace(node, bytes + 4096, size_t(64), page_size::THP_2MB);
    NumaArena& a = arenas_[arenas_.size() - 1];
    if (!a) return;
    int8_t* dst = bytes ? a.alloc<int8_t>(bytes) : nullptr;
    if (bytes && !dst) return;
    if (bytes) __builtin_memcpy(dst, wq + static_cast<size_t>(n_lo) * K, bytes);      // first touch happens here, on the bound node
    for (int i = w; i < w_end; ++i) {
      const long n0 = static_cast<long>(N) * i / total;
      bases_[i] = dst ? dst - static_cast<size_t>(n_lo) * K : nullptr;   // so that base + n*K addresses global row n
      firsts_[i] = dst ? dst + static_cast<size_t>(n0 - n_lo) * K : nullptr;
      nodes_[i] = node;
    }
    w = w_end;
  }
  valid_ = true;
}

int NodeShardedWeights::misplaced() const {
  int bad = 0;
  for (size_t i = 0; i < firsts_.size(); ++i) {
    const long n0 = static_cast<long>(N_) * static_cast<long>(i) / static_cast<long>(firsts_.size());
    const long n1 = static_cast<long>(N_) * static_cast<long>(i + 1) / static_cast<long>(firsts_.size());
    if (!firsts_[i] || n1 <= n0) continue;
    const long where = sys_move_pages_query(const_cast<int8_t*>(firsts_[i]));
    if (where < 0) return -1;
    if (where != nodes_[i]) ++bad;
  }
  return bad;
}

W8A8HostResult w8a8_linear_team_sharded(WorkerTeam& team, const NodeShardedWeights& w, const uint16_t* x, int M, const float* sw,
                                        uint16_t* y, int force_scalar, int8_t* q_out, float* sx_out, int32_t* acc_out) {
  auto run = [&](WorkerFn fn, const uint64_t* args) -> long { return team.run(fn, args); };
  return linear_core(team ? team.size() : 0, run, x, M, w.K(), nullptr, sw, w.N(), y, force_scalar, q_out, sx_out, acc_out, &w);
}

W8A8HostResult w8a8_linear_team(WorkerTeam& team, const uint16_t* x, int M, int K, const int8_t* wq, const float* sw, int N,
                                uint16_t* y, int force_scalar, int8_t* q_out, float* sx_out, int32_t* acc_out) {
  auto run = [&](WorkerFn fn, const uint64_t* args) -> long { return team.run(fn, args); };
  return linear_core(team ? team.size() : 0, run, x, M, K, wq, sw, N, y, force_scalar, q_out, sx_out, acc_out);
}

}  // namespace hostrt
