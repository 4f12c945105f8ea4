// Allocation-free entry point of the paged decode attention.
//
// This function has no counterpart in the reference project; it exists for hosts that embed the kernel library but
// must never reach the CUDA allocator: a serving process that has handed every byte of HBM to its own arena (so a
// late cudaMalloc can fail, or stall the device with its implicit synchronisation, in the middle of a request), or a
// plain C / C++ host that links neither PyTorch nor any pooling allocator and has nowhere to get scratch from.
// Such callers pass only inputs and outputs; the split-KV partials and the per-(sequence, head) arrival counters the
// kernel needs live in a fixed device array inside the library (about 4 MiB per GPU that loads it, held until exit).
//
// Contract
//   * Same arguments and result as b200_attn_decode (attn_decode.cu), minus the scratch and counter pointers.
//   * Limits (splits > 1 only): B * hq * splits * 130 floats must fit 1 Mi floats (4 MiB) and B * hkv must not
//     exceed 4096.  A call beyond either limit is rejected with B200_NOALLOC_TOO_LARGE and a message on stderr;
//     nothing is launched.  With splits == 1 the kernel uses no scratch at all, so any batch is accepted and nothing
//     is cleared.
//   * The first call with splits > 1 on each device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and caches it for the life of the process; make that first call outside any stream
//     capture.  First calls may come from several host threads at once.  The address belongs to the device that is
//     current at the call: `stream` must be a stream of that device.  A cudaDeviceReset invalidates the cached
//     address; do not call this function again in a process that reset the device.
//   * A sequence length beyond max_pages * page_size is treated as max_pages * page_size (the page-table row cannot
//     describe more); b200_attn_decode reports the same case through its status word.
//   * Every call on a device uses the same array.  The counters are cleared on the stream at the start of each call;
//     the partials are fully rewritten before they are read.  Two calls whose kernels can overlap on the GPU (different
//     streams without an ordering between them) race on the array: serialise them.
//   * Nothing in this path calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_NOALLOC_TOO_LARGE (-30)

int b200_attn_decode_noalloc(const void* q, const void* cache, const int* page_table, const int* seq_lens, void* out,
                             int B, int hq, int hkv, int page_size, int max_pages, int splits, float scale,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
