// C ABI of the sm_100a kernel library (loaded from Python with ctypes; usable from any C/C++ host).
// Conventions: every function returns 0 on success and a negative value on a rejected argument or a
// launch error; nothing here synchronises the stream; pointers are device pointers unless noted.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- W8A8 linear -----------------------------------------------------------------------------------
// Scratch bytes the stream-K path of b200_w8a8_gemm wants for an [M,N] problem (int32 partial sums).
size_t b200_w8a8_gemm_ws_bytes(int M, int N, int K, int num_sms);
// y[m,n] = (sum_k xq[m,k]*wq[n,k]) * sx[m] * sw[n] (+ residual[m,n]); y is bf16 (or fp32 when out_fp32).
// counters must be zero on entry and are left zero on exit (ws needs no initialisation); force_mode: -1 auto, 0 whole tiles, 1 stream-K.
int b200_w8a8_gemm(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                   const void* residual, int M, int N, int K, int ldy, int out_fp32,
                   void* ws, size_t ws_bytes, void* counters, int counters_len, int* status,
                   int num_sms, int force_mode, cudaStream_t stream);

// Decode form (M <= 64): split-K thread-block clusters reduced through distributed shared memory; no scratch.
// force_splits: 0 auto, else 1/2/4/8 CTAs per cluster along K.
int b200_w8a8_gemm_decode(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                          const void* residual, int M, int N, int K, int ldy, int out_fp32, int* status,
                          int num_sms, int force_splits, cudaStream_t stream);

int b200_w8a8_gemm_decode_resident_clusters(int m, int splits);

// Activation prologue carried inside a decode GEMM launch (quantiser CTAs of the same grid, see quant_row.cuh).
// mode: 1 rotate + quantise x [M][K]; 2 RMSNorm(gamma, eps) first; 3 residual += x (bf16, in place) then RMSNorm of the
// residual; 4 x is [M][2K] = gate | up and silu(gate) * up is quantised.  q [M][K] int8 and scale [M] are written by the
// launch (and are what its GEMM CTAs consume); flags: M uint32 words; step: a device uint32 that the caller changes
// between two replays of a captured launch (within one step every launch tags the flags with its own number).
typedef struct b200_quant_prolog {
  int mode;
  const void* x; long long ldx;
  void* residual; long long ldr;
  const void* gamma; float eps;
  void* q; float* scale;
  void* flags; const void* step;
  void* residual_out; long long ldro;   // mode 3: where residual + x is written (NULL: in place, which rules out the
                                        // inline form)
  int allow_inline;                     // up to four tokens: let the GEMM CTAs quantise their own operand (no quantiser
                                        // CTAs, row statistics exchanged inside the split-K cluster) when the shape allows
} b200_quant_prolog;
int b200_w8a8_gemm_decode_p(const b200_quant_prolog* prolog, const void* wq, const float* sw, void* y,
                            const void* residual, int M, int N, int K, int ldy, int out_fp32, int* status, int num_sms,
                            cudaStream_t stream);
int b200_w8a8_gemm_decode_ar_p(const b200_quant_prolog* prolog, const void* wq, const float* sw, void* y,
                               const void* residual, int M, int N, int K, int ldy, int* status, int num_sms,
                               void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                               size_t part_off0, size_t part_off1, void* words, int limit_ms, int ll,
                               size_t recv_off0, size_t recv_off1, size_t recv_bytes, int two_hop, size_t recv2_off0,
                               size_t recv2_off1, size_t recv2_bytes, cudaStream_t stream);

// Same, fused with the tensor-parallel all-reduce over peer memory (one launch).  -20: grid not co-resident, use
// b200_w8a8_gemm_decode followed by b200_peer_allreduce instead.  ll: low-latency {payload, epoch} words; two_hop
// (with ll): partials go only to the rank owning the column slice, which sums and broadcasts them through a second
// receive area of M * N/2 words per slot (recv2_off0/1) - less NVLink traffic at more than a few tokens.
int b200_w8a8_gemm_decode_ar(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                             const void* residual, int M, int N, int K, int ldy, int* status, int num_sms,
                             void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                             size_t part_off0, size_t part_off1, void* words, int limit_ms, int ll,
                             size_t recv_off0, size_t recv_off1, size_t recv_bytes, int two_hop, size_t recv2_off0,
                             size_t recv2_off1, size_t recv2_bytes, cudaStream_t stream);

// Mixture-of-experts grouped forms (device-side offsets / tile tables, no host sync).
int b200_w8a8_gemm_decode_grouped(const void* xq, const float* sx, const void* wq, const float* sw, void* y,
                                  int max_tokens, int x_rows, int N, int K, int ldy, int groups,
                                  const int* grp_offsets, const int* grp_counts, int* status, int num_sms,
                                  cudaStream_t stream);
int b200_w8a8_gemm_grouped(const void* xq, const float* sx, const void* wq, const float* sw, void* y, int x_rows,
                           int N, int K, int ldy, int groups, const void* tiles, const int* num_tiles,
                           int max_tiles, int* status, int num_sms, cudaStream_t stream);
int b200_router_topk(const float* logits, long long ld, int M, int E, int k, int renorm, int* ids, float* wts,
                     cudaStream_t stream);
int b200_moe_align(const int* ids, int M, int k, int e0, int n_local, int* counts, int* offsets, int* slot_token,
                   int* inv, void* tiles, int* meta, cudaStream_t stream);
int b200_moe_gather(const void* xq, const float* sx, int d, const int* slot_token, const int* meta, int max_slots,
                    void* xq_perm, float* sx_perm, cudaStream_t stream);
int b200_moe_combine(const void* y, long long ldy, const int* inv, const float* wts, int M, int k, int d, void* out,
                     long long ldo, cudaStream_t stream);

// ---- activation prologue ---------------------------------------------------------------------------
int b200_act_quant(const void* x, long long ldx, void* residual, long long ldr, const void* gamma, float eps,
                   void* q, long long ldq, float* scale, void* xn_out, long long ldn, int M, int K, int mode,
                   cudaStream_t stream);

// ---- attention and token-wise glue ---------------------------------------------------------------------
// max_pos: rows of cos_tab / sin_tab; num_pages: pages of the cache.  A token whose position is outside the tables,
// outside the max_pages pages of its sequence, or whose page id is not a page of the cache is skipped and
// ST_BAD_ARGUMENT is recorded in *status (optional) - never a stray write.
int b200_rope_kv_write(const void* qkv, long long ld_qkv, const int* positions, const int* seq_ids,
                       const float* cos_tab, const float* sin_tab, const void* q_norm_w, const void* k_norm_w,
                       float eps, void* q_out, void* k_out, void* v_out, void* cache, const int* page_table,
                       int max_pages, int page_size, int hq, int hkv, int M, int max_pos, int num_pages, int* status,
                       cudaStream_t stream);
int b200_embed_gather(const long long* ids, const void* table, void* out, int M, int d, int vocab, cudaStream_t stream);
int b200_argmax_rows(const void* logits, long long ld, int rows, int n, int index_offset, int chunks, float* out_val,
                     long long* out_idx, cudaStream_t stream);
int b200_argmax_merge(const float* cand_val, const long long* cand_idx, int world, int rows, long long* out_idx,
                      cudaStream_t stream);
size_t b200_attn_decode_scratch_floats(int B, int hq, int splits);
// seq_lens[b] > max_pages * page_size is clamped to that and ST_BAD_ARGUMENT is recorded in *status (optional).
int b200_attn_decode(const void* q, const void* cache, const int* page_table, const int* seq_lens, void* out,
                     float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size, int max_pages,
                     int splits, float scale, int* status, cudaStream_t stream);
int b200_attn_decode_tma(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                         void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                         int max_pages, int splits, float scale, int* status, cudaStream_t stream);
// Tensor-core form of the same (tcgen05 MMAs, scores in TMEM); needs splits >= b200_attn_decode_tc_min_splits(longest sequence).
int b200_attn_decode_tc_min_splits(int max_len);
int b200_attn_decode_tc(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                        void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                        int max_pages, int splits, float scale, int* status, cudaStream_t stream);
// The same kernel with its neighbours folded in: raw q | k | v of the new token in, (optional per-head RMSNorm,) rotary
// embedding, KV append, attention over the cache plus the new token, and (xq given) Hadamard rotation + per-token int8
// of the output out.  seq_lens[b] counts the new token; positions[b] is where it goes.  See attn_decode_tc.cu.
int b200_attn_decode_fused(const void* qkv, long long ld_qkv, const int* positions, const float* cos_tab,
                           const float* sin_tab, int max_pos, const void* q_norm_w, const void* k_norm_w, float eps,
                           void* cache, int num_pages, const int* page_table, const int* seq_lens, void* out, void* xq,
                           long long ldq, float* sx, float* scratch, unsigned* counters, float* rot_scratch,
                           float* blk_amax, unsigned* seq_counters, int B, int hq, int hkv, int page_size, int max_pages,
                           int splits, float scale, int* status, const void* next_weights,
                           unsigned long long next_weights_bytes, cudaStream_t stream);
// Persistent form: two CTAs per SM walk the (kv head, sequence, split) items, loads of the next item overlap the
// softmax / output phase of the current one.
int b200_attn_decode_tcp(const void* q, const void* cache, int num_pages, const int* page_table, const int* seq_lens,
                         void* out, float* scratch, unsigned* counters, int B, int hq, int hkv, int page_size,
                         int max_pages, int splits, float scale, int* status, int num_sms, cudaStream_t stream);
int b200_attn_prefill(const void* q, long long ld_q, const void* k, long long ld_k, const void* v, long long ld_v,
                      void* out, const int* cu_seqlens, int B, int total_tokens, int max_len, int hq, int hkv,
                      float scale, int* status, cudaStream_t stream);

// Split-KV form of b200_attn_prefill: every `chunk` KV tiles (of 128 tokens) of a query tile are one CTA; partial rows go
// through `scratch` (b200_attn_prefill_split_scratch_floats floats) and a merge kernel.
size_t b200_attn_prefill_split_scratch_floats(int B, int hq, int max_len, int chunk);
int b200_attn_prefill_split(const void* q, long long ld_q, const void* k, long long ld_k, const void* v, long long ld_v,
                            void* out, const int* cu_seqlens, int B, int total_tokens, int max_len, int hq, int hkv,
                            float scale, int chunk, float* scratch, int* status, cudaStream_t stream);

// ---- in-kernel time stamps (trace.cuh; only in the library variant built with -DB200RT_TRACE) -----------------------
int b200_debug_compiled(void);
int b200_debug_set_heap_extent(size_t bytes);
int b200_trace_compiled(void);
int b200_trace_set(void* ring, unsigned capacity);

// ---- locality query: every CTA writes {sm id, number of sm ids, rank_tag, cta index} (int32 [ctas][4]) -------------
int b200_where_am_i(int* out, int ctas, int rank_tag, cudaStream_t stream);

// ---- config-1 workload: counter-RNG fill + sum ------------------------------------------------------------
int b200_fill_uniform_reduce(float* out, unsigned long long begin, unsigned long long end, unsigned long long seed,
                             double* partials, int max_ctas, unsigned* counter, double* result, cudaStream_t stream);

// ---- collectives over peer-mapped memory ---------------------------------------------------------------
// peer_data / peer_flags: host arrays [world] of device pointers (rank r's heap base / flag block as mapped here).
// algo: 0 one-shot peer loads, 1 one-shot NVLS, 2 two-shot NVLS (in place), 3 chain to rank 0, 4 butterfly,
// 5 low-latency push of {payload, epoch} words (bf16, receive area of 2 * world * n * 4 bytes at scratch_off).
int b200_peer_allreduce(void* const* peer_data, void* const* peer_flags, void* mc_base, int world, int rank,
                        size_t in_off, size_t scratch_off, void* out, const void* residual, size_t n, int dtype,
                        int algo, void* epoch_words, int* status, int limit_ms, int trailing_barrier, int max_ctas,
                        cudaStream_t stream);

int b200_peer_argmax(void* const* peer_data, void* const* peer_flags, int world, int rank, size_t recv_off,
                     const float* cand_val, const long long* cand_idx, int ncand, int rows, long long* out_idx,
                     void* epoch_words, int* status, int limit_ms, cudaStream_t stream);

// ---- tensor-parallel prefill linears fused with their collective (token-sharded layout between blocks) ----------
// All offsets are byte offsets into every rank's symmetric heap (peer_data[r] = rank r's heap as mapped here).
// Rank r owns token rows [r*rows_per_rank, (r+1)*rows_per_rank) of the M rows.  phase: 7 in production (1 tiles,
// 2 scatter tail, 4 gather push; subsets only for single-device tests that run virtual ranks as consecutive launches).
//
// All-gather -> GEMM: y[M,N] = gathered(xq_local)[M,K] * wq[N,K]^T, scaled.  Gather buffers (two, by epoch parity):
// int8 [m_cap][K] at q_off*, fp32 [m_cap] at s_off*; flags uint32 [world][blk_cap] at flag_off; done words uint32
// [world] at done_off; words: 2 local uint32 (epoch, exit counter), row_ctr: blk_cap local uint32, all zero at first.
// finish != 0 acknowledges the epoch at exit; with 0 the gather buffer stays valid until b200_ag_sync(finish=1).
int b200_w8a8_gemm_ag(const void* xq_local, const float* sx_local, const void* wq, const float* sw, void* y,
                      int M, int N, int K, int ldy, int rows_per_rank, void* const* peer_data, void* mc_base,
                      int world, int rank, size_t q_off0, size_t q_off1, size_t s_off0, size_t s_off1,
                      size_t flag_off, size_t done_off, int blk_cap, int m_cap, void* words, void* row_ctr,
                      int finish, int phase, int* status, int limit_ms, int num_sms, cudaStream_t stream);
// GEMM -> reduce-scatter: out[my rows, N] = sum over ranks of (xq[M,K_shard] * wq^T) (+ residual[my rows]).
// Receive slots (two, by parity): bf16 [world][r_cap][N] at recv_off*; arrival counters uint32 [2] at ctr_off (zero at
// first); words: 2 local uint32.
int b200_w8a8_gemm_rs(const void* xq, const float* sx, const void* wq, const float* sw, void* out,
                      const void* residual, int M, int N, int K, int ldo, int ldr, int rows_per_rank,
                      void* const* peer_data, int world, int rank, size_t recv_off0, size_t recv_off1,
                      size_t ctr_off, int r_cap, void* words, int phase, int* status, int limit_ms, int num_sms,
                      cudaStream_t stream);
int b200_ag_sync(void* const* peer_data, int world, int rank, size_t flag_off, size_t done_off, int blk_cap,
                 int rows_per_rank, int M, void* words, int wait, int finish, int* status, int limit_ms,
                 cudaStream_t stream);

// ---- expert-parallel dispatch / combine for token-sharded prefill (buffers of the all-gather / reduce-scatter links) ----
// dispatch: this rank's rows go (int8 + scale) to the ranks owning one of their top-k experts, the routing lists
// (ids / weights padded to 8 per token at ids_off* / wts_off*) to every rank; flags as in b200_w8a8_gemm_ag.
int b200_ep_dispatch(const void* xq_local, const float* sx_local, const int* ids_local, const float* wts_local,
                     int M, int K, int k, int experts_per_rank, int rows_per_rank, void* const* peer_data,
                     int world, int rank, size_t q_off0, size_t q_off1, size_t s_off0, size_t s_off1,
                     size_t ids_off0, size_t ids_off1, size_t wts_off0, size_t wts_off1, size_t flag_off,
                     size_t done_off, int blk_cap, void* words, void* row_ctr, int* status, int limit_ms,
                     cudaStream_t stream);
// wait for all sources, then copy the routing lists of all M tokens to ids_out / wts_out [M][k]
int b200_ep_wait(void* const* peer_data, int world, int rank, size_t ids_off0, size_t ids_off1, size_t wts_off0,
                 size_t wts_off1, size_t flag_off, int blk_cap, int rows_per_rank, int M, int k, void* words,
                 int* ids_out, float* wts_out, int* status, int limit_ms, cudaStream_t stream);
// b200_moe_gather over the gather buffer of the current epoch (heap_base: this rank's heap)
int b200_ep_gather(const void* heap_base, size_t q_off0, size_t q_off1, size_t s_off0, size_t s_off1,
                   const void* words, int d, const int* slot_token, const int* meta, int max_slots,
                   void* xq_perm, float* sx_perm, cudaStream_t stream);
// combine: weighted local expert outputs of each token -> receive slot of the token's owner; blk_ctr: world*blk_cap
// local uint32, zero at first.  reduce: the owner sums the slots of the ranks its own routing names -> out[my rows][d].
int b200_ep_combine_scatter(const void* y, long long ldy, const int* inv, const float* wts, int M, int k, int d,
                            int rows_per_rank, void* const* peer_data, int world, int rank, size_t recv_off0,
                            size_t recv_off1, size_t ctr_off, int r_cap, void* words, void* blk_ctr, int blk_cap,
                            int* status, int limit_ms, cudaStream_t stream);
int b200_ep_combine_reduce(const int* ids_local, int M, int k, int d, int experts_per_rank, int rows_per_rank,
                           void* const* peer_data, int world, int rank, size_t recv_off0, size_t recv_off1,
                           size_t ctr_off, int r_cap, void* words, void* out, long long ldo, int* status,
                           int limit_ms, int num_sms, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
