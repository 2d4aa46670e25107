// The merge of the split-KV decode attention's partial results, as ONE function that every
// kernel which merges them calls (the two stage-2 kernels, and the output projection that
// merges while it loads its operand), so that all of them give the same bits.
//
// A sequence's splits s0..s1 (128 keys each) are taken in chunks of MERGE_CH = 16 (chunk c =
// splits 16c .. 16c+15): with M the largest log-sum-exp of the range and w_s = exp(lse_s - M),
// a chunk's sums are acc_c = fma(w_s, o_s, acc_c) and den_c = den_c + w_s in split order from
// 0; the chunks' sums are added in chunk order; the result is total / total_den.  The order
// depends on the sequence's own length (and window) only.
#pragma once
#include "common.cuh"

constexpr int MERGE_CH = 16;
constexpr int MERGE_SPLIT = 128;     // keys per split (DEC_SPLIT of the attention kernels)
constexpr float MERGE_NEG_BIG = -1e30f;

// The range of splits a sequence of kv_len keys has results for: [s0, s1], clamped to the
// max_splits the scratch holds.
__device__ __forceinline__ void merge_range(int kv_len, int window, int max_splits, int& s0, int& s1) {
  const int pos = kv_len - 1;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  s0 = first_key / MERGE_SPLIT;
  s1 = min(pos / MERGE_SPLIT, max_splits - 1);
}

// The weight of a split whose log-sum-exp is lse, against the range's largest one.
__device__ __forceinline__ float merge_weight(float lse, float M) { return expf(__fsub_rn(lse, M)); }

// One chunk's contribution for V consecutive dimensions: w[j] (the weights), o[j][v] hold the
// chunk's 16 splits (entries outside [s0, s1] are ignored).
template <int V>
__device__ __forceinline__ void merge_chunk_weighted(const float (&w)[MERGE_CH], const float (&o)[MERGE_CH][V],
                                                     int c, int s0, int s1, float (&acc)[V], float& den) {
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  den = 0.f;
#pragma unroll
  for (int j = 0; j < MERGE_CH; ++j) {
    const int s = c * MERGE_CH + j;
    if (s >= s0 && s <= s1) {
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = __fmaf_rn(w[j], o[j][v], acc[v]);
      den = __fadd_rn(den, w[j]);
    }
  }
}
// The same from the log-sum-exps (the weight of a split is computed where it is used).
template <int V>
__device__ __forceinline__ void merge_chunk(const float (&lse)[MERGE_CH], const float (&o)[MERGE_CH][V],
                                            int c, int s0, int s1, float M, float (&acc)[V], float& den) {
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  den = 0.f;
#pragma unroll
  for (int j = 0; j < MERGE_CH; ++j) {
    const int s = c * MERGE_CH + j;
    if (s >= s0 && s <= s1) {
      const float w = merge_weight(lse[j], M);
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = __fmaf_rn(w, o[j][v], acc[v]);
      den = __fadd_rn(den, w);
    }
  }
}

// total (+)= chunk, in chunk order; first: this is the range's first chunk.
template <int V>
__device__ __forceinline__ void merge_add(bool first, const float (&acc)[V], float den,
                                          float (&total)[V], float& total_den) {
#pragma unroll
  for (int v = 0; v < V; ++v) total[v] = first ? acc[v] : __fadd_rn(total[v], acc[v]);
  total_den = first ? den : __fadd_rn(total_den, den);
}

__device__ __forceinline__ float merge_finish(float total, float total_den) {
  return __fdiv_rn(total, total_den);
}
