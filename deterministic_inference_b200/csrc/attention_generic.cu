// Generic paged attention: one warp per (token, query head), float32 arithmetic
// throughout (expf, not the fast intrinsic), any head_dim up to 256, any number
// of heads and groups, any page size, optional window.  It is the attention of
// the 32-bit path, and the fallback of the bfloat16 path for head sizes the
// tensor-core kernels refuse.
//
// Every token of the step is one query: token t belongs to sequence
// token_seq[t], stands at absolute position positions[t] and sees the keys
// max(0, pos-window+1) .. pos of its sequence, all read from the paged cache
// through the sequence's row of the block table (this step's keys were written
// before the launch).  Keys are visited in tiles of 32 anchored at position 0,
// so the order of the reduction for a query depends on its position alone:
// the same token gives the same bits however the prompt was cut into steps,
// whatever else is in the batch and whichever pages hold its keys.
//
// Cache layout of a layer: [num_pages, 2, num_kv_heads, page_size, head_dim].
#include "common.cuh"

namespace {

constexpr int MAX_D = 256;
constexpr int WARPS = 4;
constexpr float NEG_BIG = -1e30f;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out,
                               const T* __restrict__ kv_cache,
                               const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ token_seq,
                               const int* __restrict__ positions, int T_tokens, int Hq, int Hkv,
                               int D, int page_size, float scale, int window) {
  pdl_prologue(q, kv_cache, block_table, token_seq, positions);
  __shared__ float sq[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)T_tokens * Hq) return;
  const int t = (int)(item / Hq), h = (int)(item % Hq);
  const int group = Hq / Hkv;
  const int kvh = h / group;
  const int seq = token_seq[t];
  const int pos = positions[t];
  const int* bt = block_table + (size_t)seq * max_blocks;

  const T* qrow = q + ((size_t)t * Hq + h) * D;
  for (int d = lane; d < D; d += 32) sq[warp][d] = Elem<T>::load(qrow + d);
  __syncwarp();

  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  float m = NEG_BIG, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  const size_t head_stride = (size_t)page_size * D;          // one head inside a page
  const size_t kv_stride = (size_t)Hkv * head_stride;        // keys -> values inside a page
  const size_t page_stride = 2 * kv_stride;

  for (int k0 = (first / 32) * 32; k0 <= pos; k0 += 32) {
    const int key = k0 + lane;
    const bool visible = key >= first && key <= pos;
    float s = NEG_BIG;
    const T* vrow = nullptr;
    if (visible) {
      const int page = bt[key / page_size];
      const T* krow = kv_cache + (size_t)page * page_stride + (size_t)kvh * head_stride +
                      (size_t)(key % page_size) * D;
      vrow = krow + kv_stride;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(sq[warp][d], Elem<T>::load(krow + d), dot);
      s = dot * scale;
    }
    const float tile_max = warp_max(s);
    const float m_new = fmaxf(m, tile_max);   // the tile holds at least one visible key
    const float p = visible ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
    // P.V: keys in order, each lane owns dims lane, lane+32, ...
    const unsigned long long vaddr = (unsigned long long)vrow;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const unsigned long long va = __shfl_sync(0xffffffffu, vaddr, j);
      if (va == 0ull) continue;   // warp-uniform
      const T* vr = (const T*)va;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pj, Elem<T>::load(vr + d), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* orow = out + ((size_t)t * Hq + h) * D;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) Elem<T>::store(orow + d, acc[i] * inv);
  }
}

}  // namespace

extern "C" int dib_paged_attention_generic(const void* q, void* out, const void* kv_cache,
                                           const int* block_table, int max_blocks,
                                           const int* token_seq, const int* positions, int T,
                                           int Hq, int Hkv, int D, int page_size, float scale,
                                           int window, int dtype, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (D < 1 || D > MAX_D || Hkv < 1 || Hq % Hkv != 0 || page_size < 1) return DIB_BAD_SIZE;
  const long long items = (long long)T * Hq;
  const int blocks = ceil_div_host(items, WARPS);
  if (dtype == 0)
    dib_launch(paged_attention_generic_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, st, 
        (const float*)q, (float*)out, (const float*)kv_cache, block_table, max_blocks, token_seq,
        positions, T, Hq, Hkv, D, page_size, scale, window);
  else if (dtype == 1)
    dib_launch(paged_attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, st, 
        (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kv_cache, block_table,
        max_blocks, token_seq, positions, T, Hq, Hkv, D, page_size, scale, window);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}
