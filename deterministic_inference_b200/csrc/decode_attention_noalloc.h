// Split-KV decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for
// hosts of this library that cannot call cudaMalloc at the time they need
// attention: real-time or embedded hosts that fix all their device memory at
// start-up, processes whose device memory is fully committed to other owners,
// and plug-ins that run under an allocator they do not own and may not re-enter.
// The regular entry point
// (dib_decode_attention_bf16) leaves the scratch for the per-split partial
// results to its caller, who normally gets it from an allocator; this one keeps
// that scratch inside the library instead.
//
// What it computes is what dib_decode_attention_bf16 computes: for each of the first
// `num_seqs` sequences of a batch, one query token attends over the sequence's keys in
// the paged cache, in splits of 128 keys that a second kernel adds in split order.  Its
// first stage is the kernel that copies keys and values row by row; the regular entry
// point takes that kernel only for shapes its page-wise TMA kernels refuse (or when it
// is called with num_pages = 0).  Against that form the results agree in every bit;
// against the TMA kernels, which exponentiate against a split-wide maximum instead of
// a per-warp one, they agree within the rounding of bfloat16 probabilities.  The caller
// still passes every input and the output; only the scratch is internal.
//
// The scratch is a file-scope device array of DIB_NOALLOC_SCRATCH_FLOATS floats
// (16 MiB), aligned to 256 bytes.  Every GPU on which this library is loaded holds
// that array from the moment the module is loaded on it until the process exits.
// A call needs num_seqs * Hq * max_splits * (D + 1) floats of it; a call that
// needs more is refused with DIB_BAD_SIZE (-2) and launches nothing.
//
// Set-up: the first call on a device (with that device current) looks up the
// device address of the array with cudaGetSymbolAddress and remembers it for that
// device, and the first call for a head size on a device raises that kernel's
// shared-memory limit.  Neither is a stream operation, so make the first call for each
// head size on each device before any stream capture begins.  Where the CUDA runtime
// loads modules lazily, that first look-up is also what loads this library's module
// onto the device, which is when the driver reserves the array: "no call allocates"
// holds from the second call on a device on.  No call calls cudaMalloc, cudaFree or
// a library routine that allocates.
//
// Sharing: all calls on a device use the same array, and it keeps what the last
// call left in it.  Nothing in it has to start at zero: every element stage 2 reads
// was written by stage 1 of the same call.  Two calls whose kernels overlap on the
// GPU (different streams, or the same stream in different graphs that run
// concurrently) race on the array and give wrong results; order them.
#pragma once
#include <cuda_runtime.h>

#define DIB_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Floats of scratch a call with these sizes needs.
long long dib_decode_attention_noalloc_scratch_needed(int num_seqs, int max_splits, int Hq, int D);

// q, out: bfloat16 [num_seqs, Hq, D]; cache: bfloat16 [pages, 2, Hkv, page_size, D];
// block_table: int32 [num_seqs (or more), max_blocks]; seq_lens: int32 [num_seqs];
// max_splits >= ceil(longest sequence / 128) (a smaller value never reads beyond the
// scratch: the splits beyond it are left out of the result).  Returns 0, or a negative
// dib_status: -2 sizes refused (head_dim not a multiple of 16 up to 128, group ratio
// above 16, or more scratch needed than the array holds), -4 launch or set-up failed.
int dib_decode_attention_bf16_noalloc(const void* q, void* out, const void* cache,
                                      const int* block_table, int max_blocks,
                                      const int* seq_lens, int num_seqs, int max_splits, int Hq,
                                      int Hkv, int D, int page_size, float scale, int window,
                                      cudaStream_t stream);

// This library's own error word: 0, or 1 if a bounded wait inside one of its kernels ran
// out since the last clear (the output of that call is not valid).  Reading it
// synchronises with the device.  -1: the word could not be read.
int dib_decode_attention_noalloc_status(void);
int dib_decode_attention_noalloc_status_clear(void);

#ifdef __cplusplus
}
#endif
