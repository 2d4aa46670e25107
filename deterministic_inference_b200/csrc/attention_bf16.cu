// Entry points of the bfloat16 tensor-core attention kernels (the kernels and
// their launch templates are in attention_bf16_kernels.cuh).
#include "attention_bf16_kernels.cuh"

extern "C" {

int dib_attention_bf16_split_size() { return DEC_SPLIT; }

// 0, or 1 if a bounded wait inside a kernel of this library ever ran out (the
// results of that launch are then not valid).  Synchronises with the device.
int dib_attention_bf16_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, dib_attention_error_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
int dib_attention_bf16_tile_rows() { return EXT_M; }

// Sequences with more than one new token.  q/out are the step's full [T, Hq, D]
// tensors; tiles name (sequence, first token of the tile among its new tokens), with
// floor(64 / (Hq/Hkv)) tokens per tile.
int dib_extend_attention_bf16(const void* q, void* out, const void* cache, const int* block_table,
                              int max_blocks, const int* cu_q_lens, const int* seq_lens,
                              const int* tile_seq, const int* tile_start, int num_tiles, int Hq,
                              int Hkv, int D, int page_size, float scale, int window,
                              cudaStream_t st) {
  if (num_tiles == 0) return DIB_OK;
  if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > EXT_M || Hkv > 65535) return DIB_BAD_SIZE;
#define CALL(DD)                                                                              \
  launch_extend<DD>(q, out, cache, block_table, max_blocks, cu_q_lens, seq_lens, tile_seq,   \
                    tile_start, num_tiles, Hq, Hkv, page_size, scale, window, st)
  DIB_DISPATCH_D(D, CALL)
#undef CALL
}

// The first num_seqs sequences of the batch, one token each (token index = sequence
// index).  part_o: float32 [num_seqs, Hq, max_splits, D]; part_lse: [num_seqs, Hq,
// max_splits]; max_splits >= ceil(longest sequence / 128).
int dib_decode_attention_bf16(const void* q, void* out, const void* cache, const int* block_table,
                              int max_blocks, const int* seq_lens, float* part_o, float* part_lse,
                              int num_seqs, int max_splits, int Hq, int Hkv, int D, int page_size,
                              float scale, int window, cudaStream_t st) {
  if (num_seqs == 0) return DIB_OK;
  if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16 || num_seqs > 65535 || max_splits > 65535 ||
      max_splits < 1)
    return DIB_BAD_SIZE;
#define CALL(DD)                                                                                  \
  launch_decode<DD>(q, out, cache, block_table, max_blocks, seq_lens, part_o, part_lse, num_seqs, \
                    max_splits, Hq, Hkv, page_size, scale, window, st)
  DIB_DISPATCH_D(D, CALL)
#undef CALL
}

}  // extern "C"
