// dib_decode_attention_bf16_noalloc: the split-KV decode attention with its
// scratch memory inside the library, for callers that cannot allocate (see
// decode_attention_noalloc.h).  The kernels are the row-copy first stage and the merge
// that the regular entry point launches for shapes its TMA kernels do not take.
#include "decode_attention_noalloc.h"

#include "attention_bf16_kernels.cuh"

// The scratch: per-split partial outputs [num_seqs, Hq, max_splits, D] followed by
// their log-sum-exp values [num_seqs, Hq, max_splits].  In host code this name is
// only a handle; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float dib_noalloc_scratch[DIB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* scratch_address[MAX_DEVICES] = {nullptr};

// Device address of the scratch on the current device; looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return DIB_LAUNCH_FAILED;
  if (scratch_address[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, dib_noalloc_scratch) != cudaSuccess || p == nullptr)
      return DIB_LAUNCH_FAILED;
    scratch_address[dev] = static_cast<float*>(p);
  }
  *out = scratch_address[dev];
  return DIB_OK;
}
}  // namespace

extern "C" {

int dib_decode_attention_noalloc_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, dib_attention_error_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
int dib_decode_attention_noalloc_status_clear(void) {
  const int v = 0;
  return cudaMemcpyToSymbol(dib_attention_error_word, &v, sizeof(int)) == cudaSuccess ? 0 : -1;
}

long long dib_decode_attention_noalloc_scratch_needed(int num_seqs, int max_splits, int Hq, int D) {
  return (long long)num_seqs * Hq * max_splits * ((long long)D + 1);
}

int dib_decode_attention_bf16_noalloc(const void* q, void* out, const void* cache,
                                      const int* block_table, int max_blocks,
                                      const int* seq_lens, int num_seqs, int max_splits, int Hq,
                                      int Hkv, int D, int page_size, float scale, int window,
                                      cudaStream_t st) {
  if (num_seqs == 0) return DIB_OK;
  if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16 || num_seqs > 65535 || max_splits > 65535 ||
      max_splits < 1 || num_seqs < 0 || D < 1)
    return DIB_BAD_SIZE;
  if (dib_decode_attention_noalloc_scratch_needed(num_seqs, max_splits, Hq, D) >
      (long long)DIB_NOALLOC_SCRATCH_FLOATS)
    return DIB_BAD_SIZE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != DIB_OK) return rc;
  float* part_o = scratch;
  float* part_lse = scratch + (size_t)num_seqs * Hq * max_splits * D;
#define CALL(DD)                                                                                  \
  launch_decode<DD>(q, out, cache, block_table, max_blocks, seq_lens, part_o, part_lse, num_seqs, \
                    max_splits, Hq, Hkv, page_size, scale, window, st)
  DIB_DISPATCH_D(D, CALL)
#undef CALL
}

}  // extern "C"
