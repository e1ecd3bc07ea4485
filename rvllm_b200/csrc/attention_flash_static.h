// rv_flash_attention_static - paged flash attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project; it exists for users of this
// library.
//
// Who needs it.  rv_flash_attention splits the keys of a sequence over several CTAs when a
// batch alone cannot fill the GPU, and the partial results of the splits need scratch memory
// that the caller passes in.  Some callers have no way to provide it:
//   * a host program (C, Rust, a plug-in) that loads this shared library directly and has
//     handed all device memory to its own arena at start-up - the engine around these kernels
//     sizes its cache to fill the GPU, so a later cudaMalloc may simply fail;
//   * code on a latency path or inside a region where cudaMalloc is not allowed, because it
//     synchronises the device and may block for an unbounded time;
//   * callers without the tensor library whose allocator the Python wrappers use.
// For them the scratch is a fixed array inside the library.
//
// What it costs.  The array has RV_FLASH_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on
// which a process loads this library holds that much until the process exits, whether or not
// this function is ever called.  A call needs num_splits * n_tokens * num_heads * (HEAD_DIM + 2)
// floats when num_splits > 1 (nothing otherwise); a call that needs more is refused with
// RV_ERR_SCRATCH_TOO_LARGE and a message in `err` - use fewer splits, or rv_flash_attention.
//
// Rules.
//   * The function calls no cudaMalloc, cudaFree or any allocating routine.  Inputs and outputs
//     are the caller's, exactly as for rv_flash_attention (q_filter is always 0: every sequence).
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it, and raises the kernels'
//     shared-memory limit on that device.  Make that first call before any stream capture on that
//     device.  The remembered address is kept per device without a lock: two host threads that
//     make the first call on a device at the same moment both look it up and store the same value.
//   * n_tokens must be the number of rows that the sequences cover (cu_seqlens[num_seqs]) and
//     max_q_len at least the longest sequence's rows.  Output rows beyond the sequences, or beyond
//     an understated max_q_len, are undefined: with key splits they are merged from whatever an
//     earlier call left in the shared array.
//   * All calls share the one array, which keeps whatever the last call left in it.  Nothing in
//     it has to be zero: each call overwrites every element it later reads.  Two calls that
//     overlap on the GPU (different streams, no ordering between them) race on it - order them.
//   * Return value: 0, a negative RV_ERR_* code for sizes it refuses, or a positive cudaError_t.
//     `err` (may be null) receives a one-line message of at most err_len bytes on failure.
#pragma once
#include <cuda_runtime.h>

#define RV_FLASH_STATIC_SCRATCH_FLOATS (1 << 20)
#define RV_ERR_SCRATCH_TOO_LARGE (-5)

extern "C" int rv_flash_attention_static(const void* q, const void* cache, const int* block_tables,
                                         const int* cu_seqlens, const int* ctx_lens, void* out, int n_tokens,
                                         int num_seqs, int nh, int nkv, int hd, int page_size, int max_blocks,
                                         float scale, int window, int mode, int max_q_len, int num_splits,
                                         cudaStream_t stream, char* err, int err_len);
