// ilb_attention_decode_static: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference; it exists for callers of this
// library that are not allowed to allocate device memory.
//
// Who that is.  The ordinary entry point, ilb_attention_decode, needs a scratch buffer (the
// per-chunk partial results and one counter per (sequence, kv head)) that its caller
// allocates.  Some callers cannot: a host program that hands this library a fixed budget of
// device memory at start-up and forbids any allocation afterwards; code that runs between
// the capture and the replay of a CUDA graph, where an allocation would change addresses
// the graph has recorded; a real-time loop that must never meet the implicit device-wide
// synchronisation of cudaMalloc/cudaFree; a plain C, C++ or Rust caller that links the
// shared library without torch and so has no caching allocator to lean on.  For them the
// scratch lives in a static array inside the library.
//
// What it costs.  The array is kStaticScratchBytes (16 MiB + 16 KiB) of device memory on
// EVERY GPU on which this library is loaded, from the moment the module is loaded there
// until the process exits, whether or not this entry point is ever called.
//
// Limits.  The call is refused with an error (return -1, message via ilb_last_error) when
//   n_seqs * nkv * max_chunks * (nq / nkv) * (d + 2)  >  kStaticScratchFloats   (4 Mi floats)
//   n_seqs * nkv                                        >  kStaticTickets         (4096)
// Everything else is as for ilb_attention_decode (same kernel, same arguments, same result).
//
// Set-up.  The first call on each device looks up the device address of the array
// (cudaGetSymbolAddress) with that device current and remembers it; make that first call
// before any stream capture begins on that device.  No call allocates or frees memory.
//
// Sharing.  All calls on a device use the same array, and the array keeps what the last
// call left in it.  The counters must be zero when a launch starts, so every call clears
// them on `stream` first (cudaMemsetAsync); the partial results need no clearing because
// each launch writes what it later reads.  Two calls whose kernels may overlap on the GPU
// (different streams without an ordering between them) race on the array: order them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { kStaticScratchFloats = 4 * 1024 * 1024, kStaticTickets = 4096 };
enum { kStaticScratchBytes = kStaticScratchFloats * 4 + kStaticTickets * 4 };

// Arguments as ilb_attention_decode without scratch, scratch_floats, tickets, n_tickets.
// Returns 0, or -1 with a message in ilb_last_error().
int ilb_attention_decode_static(const void* q, void* out, const void* k_cache, const void* v_cache,
                                const int* positions, const int* cu_q, const int* block_table,
                                int max_blocks, int page_size, int num_pages, int window, float scale,
                                int n_seqs, int nq, int nkv, int d, int q_stride, int out_stride,
                                int chunk, int max_chunks, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
