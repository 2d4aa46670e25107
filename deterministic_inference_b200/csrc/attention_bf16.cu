// Entry points of the bfloat16 tensor-core attention kernels (the kernels and
// their launch templates are in attention_bf16_kernels.cuh).
#include <cuda.h>

#include <map>
#include <tuple>

#include "attention_bf16_kernels.cuh"

// ------------------------------------------------------------------------------
// Decode stage 1 with page-granular TMA loads.  The cache of a layer is a 2-D
// matrix [pages * 2 * kv_heads * page_size rows, head_dim]; the keys (or values) of
// one head in one page are page_size consecutive rows, fetched as boxes of
// [page_size rows x 64 columns] (128 bytes per row) with the 128-byte swizzle, so
// ldmatrix reads them without bank conflicts: the 16-byte chunk c of row r lies at
// chunk c ^ (r & 7).  One CTA issues 2 * (128 / page_size) * head_dim / 64 copies
// instead of one copy per key row.  head_dim 64 or 128, page_size 8..128 dividing 128.
namespace {

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)),
      "r"(c0), "r"(c1)
      : "memory");
}

// element offset of (row, d) in a [halves][128 rows][64] bf16 tile with the swizzle
__device__ __forceinline__ int sw_off(int row, int d) {
  return (d >> 6) * (DEC_SPLIT * 64) + row * 64 + ((((d & 63) >> 3) ^ (row & 7)) << 3);
}

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_stage1_tma_kernel(const __grid_constant__ CUtensorMap map,
                                   const __nv_bfloat16* __restrict__ q,
                                   const int* __restrict__ block_table, int max_blocks,
                                   const int* __restrict__ seq_lens, float* __restrict__ part_o,
                                   float* __restrict__ part_lse, int max_splits, int Hq, int Hkv,
                                   int page_size, float scale, int window) {
  // Keys and values of earlier steps do not depend on the kernel before this one
  // (which only writes the new token's slot), nor do the block table and the
  // lengths: their loads start at once; only the page that holds the new token, and
  // the query, wait for that kernel.
  pdl_trigger();
  constexpr int HALVES = D / 64;
  constexpr int TILE = DEC_SPLIT * D;   // elements of the K (or V) tile
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sV = sK + TILE;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + (size_t)2 * TILE * 2);

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int k0 = split * DEC_SPLIT;
  const int* bt = block_table + (size_t)b * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The sequence length and this thread's block-table entry are fetched side by side
  // (neither address depends on the other), so the copies can start one memory
  // round-trip after the kernel does.  An entry beyond the table reads page 0.
  const int pages = DEC_SPLIT / page_size;
  const int pi = threadIdx.x / (2 * HALVES);
  const int kv_len = seq_lens[b];
  int page = 0;
  if (threadIdx.x < pages * 2 * HALVES) {
    const int idx = k0 / page_size + pi;
    page = idx < max_blocks ? bt[idx] : 0;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  __syncthreads();
  const int pos = kv_len - 1;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (k0 > pos || k0 + DEC_SPLIT <= first_key) return;
  const int nvalid = min(DEC_SPLIT, kv_len - k0);
  const int valid_pages = (nvalid + page_size - 1) / page_size;
  if (threadIdx.x == 0) {
    mbar_expect_tx(&bars[0], (unsigned)valid_pages * page_size * D * 2);
    mbar_expect_tx(&bars[1], (unsigned)valid_pages * page_size * D * 2);
  }
  // thread t issues the copy of (page t / (2*HALVES), key-or-value, 64-column half):
  // before the wait if the page lies wholly before the new token's position
  const bool issuer = threadIdx.x < pages * 2 * HALVES && pi < valid_pages;
  const bool early = (k0 / page_size + pi) < pos / page_size;
  const int kv = (threadIdx.x / HALVES) & 1;
  const int half = threadIdx.x % HALVES;
  const int row0 = (((page * 2 + kv) * Hkv) + kvh) * page_size;
  __nv_bfloat16* dst = (kv ? sV : sK) + half * (DEC_SPLIT * 64) + pi * page_size * 64;
  if (issuer && early) tma_load_2d(dst, &map, half * 64, row0, &bars[kv]);
  pdl_wait();
  if (issuer && !early) tma_load_2d(dst, &map, half * 64, row0, &bars[kv]);

  unsigned qf[D / 16][4];
  {
    const __nv_bfloat16* qb = q + ((size_t)b * Hq + (size_t)kvh * G) * D;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d = ks * 16 + c0;
      qf[ks][0] = r0 < G ? *reinterpret_cast<const unsigned*>(qb + (size_t)r0 * D + d) : 0u;
      qf[ks][1] = r0 + 8 < G ? *reinterpret_cast<const unsigned*>(qb + (size_t)(r0 + 8) * D + d) : 0u;
      qf[ks][2] = r0 < G ? *reinterpret_cast<const unsigned*>(qb + (size_t)r0 * D + d + 8) : 0u;
      qf[ks][3] =
          r0 + 8 < G ? *reinterpret_cast<const unsigned*>(qb + (size_t)(r0 + 8) * D + d + 8) : 0u;
    }
  }
  int lo[2] = {first_key, first_key}, hi[2] = {pos, pos};
  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[dt][i] = 0.f;
  float mrow[2] = {NEG_BIG, NEG_BIG}, lrow[2] = {0.f, 0.f};
  const int krow0 = warp * DEC_WARP_KEYS;
  const int m = lane >> 3, r = lane & 7;

  // ---- scores of this warp's 32 keys (keys beyond the sequence are masked, whatever
  // the tile holds there)
  if (!mbar_wait(&bars[0], 0)) atomicExch(&dib_attention_error_word, 1);
  float s[DEC_WARP_KEYS / 8][4];
#pragma unroll
  for (int nt = 0; nt < DEC_WARP_KEYS / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < DEC_WARP_KEYS / 16; ++np) {
      unsigned bf[4];
      ldmatrix_x4(bf, sK + sw_off(krow0 + np * 16 + (m >> 1) * 8 + r, ks * 16 + (m & 1) * 8));
      mma_16816(s[np * 2], qf[ks], bf[0], bf[1]);
      mma_16816(s[np * 2 + 1], qf[ks], bf[2], bf[3]);
    }
  }
  softmax_tile<D, DEC_WARP_KEYS>(s, o, mrow, lrow, k0 + krow0, lo, hi, scale * LOG2E, lane);

  // ---- P.V; value rows beyond the sequence are zeroed first (their probability is 0,
  // but 0 * garbage must stay 0)
  if (!mbar_wait(&bars[1], 0)) atomicExch(&dib_attention_error_word, 1);
  if (nvalid < DEC_SPLIT) {
    const int row = threadIdx.x;
    if (row >= nvalid) {
#pragma unroll
      for (int c = 0; c < D / 8; ++c)
        *reinterpret_cast<uint4*>(sV + sw_off(row, c * 8)) = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
  }
#pragma unroll
  for (int kk = 0; kk < DEC_WARP_KEYS / 16; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(s[kk * 2][0], s[kk * 2][1]);
    a[1] = pack_bf16(s[kk * 2][2], s[kk * 2][3]);
    a[2] = pack_bf16(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
    a[3] = pack_bf16(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      unsigned bf[4];
      ldmatrix_x4_trans(bf, sV + sw_off(krow0 + kk * 16 + (m & 1) * 8 + r, dp * 16 + (m >> 1) * 8));
      mma_16816(o[dp * 2], a, bf[0], bf[1]);
      mma_16816(o[dp * 2 + 1], a, bf[2], bf[3]);
    }
  }
  __syncthreads();  // the K tile is reused for the merge

  float* sO = reinterpret_cast<float*>(smem_raw);
  float* sM = sO + 4 * 16 * D;
  float* sL = sM + 4 * 16;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = (lane >> 2) + rr * 8;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      const int d = dt * 8 + (lane & 3) * 2;
      sO[(warp * 16 + row) * D + d] = o[dt][rr * 2];
      sO[(warp * 16 + row) * D + d + 1] = o[dt][rr * 2 + 1];
    }
    if ((lane & 3) == 0) {
      sM[warp * 16 + row] = mrow[rr];
      sL[warp * 16 + row] = lrow[rr];
    }
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int row = threadIdx.x;
    float M = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 16 + row]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = fast_exp2(sM[w * 16 + row] - M);
      L += sL[w * 16 + row] * f;
      sM[w * 16 + row] = f;
    }
    sL[row] = 1.0f / L;
    const size_t prow = ((size_t)b * Hq + (size_t)kvh * G + row) * max_splits + split;
    part_lse[prow] = (M + log2f(L)) / LOG2E;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += DEC_THREADS) {
    const int row = idx / D, d = idx % D;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) acc += sO[(w * 16 + row) * D + d] * sM[w * 16 + row];
    const size_t prow = ((size_t)b * Hq + (size_t)kvh * G + row) * max_splits + split;
    part_o[prow * D + d] = acc * sL[row];
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a cache layer, made once per (pointer, shape) and kept.
const CUtensorMap* cache_map(const void* cache, long long num_pages, int Hkv, int page_size, int D) {
  static EncodeTiledFn enc = nullptr;
  static std::map<std::tuple<const void*, long long, int, int, int>, CUtensorMap> maps;
  if (enc == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      return nullptr;
    enc = reinterpret_cast<EncodeTiledFn>(p);
  }
  const auto key = std::make_tuple(cache, num_pages, Hkv, page_size, D);
  auto it = maps.find(key);
  if (it != maps.end()) return &it->second;
  CUtensorMap m;
  const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * 2 * Hkv * page_size};
  const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return nullptr;
  return &maps.emplace(key, m).first->second;
}

template <int D>
int launch_decode_tma(const void* q, void* out, const void* cache, long long num_pages,
                      const int* bt, int max_blocks, const int* seq_lens, float* part_o,
                      float* part_lse, int num_seqs, int max_splits, int Hq, int Hkv, int page_size,
                      float scale, int window, cudaStream_t st) {
  const CUtensorMap* map = cache_map(cache, num_pages, Hkv, page_size, D);
  if (map == nullptr) return DIB_LAUNCH_FAILED;
  const size_t smem = (size_t)2 * DEC_SPLIT * D * 2 + 16 + 1024;
  auto kern = decode_attention_stage1_tma_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set = true;
  }
  dib_launch(kern, dim3(Hkv, num_seqs, max_splits), dim3(DEC_THREADS), smem, st, *map,
             (const __nv_bfloat16*)q, bt, max_blocks, seq_lens, part_o, part_lse, max_splits, Hq, Hkv,
             page_size, scale, window);
  DIB_CHECK_LAUNCH();
  const int th = D < 32 ? 32 : (D + 31) / 32 * 32;
  dib_launch(decode_attention_stage2_kernel, dim3(num_seqs, Hq), dim3(th), 0, st, part_o, part_lse,
             seq_lens, (__nv_bfloat16*)out, max_splits, Hq, D, window);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // namespace

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
  if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > EXT_M || num_tiles > 65535) return DIB_BAD_SIZE;
#define CALL(DD)                                                                              \
  launch_extend<DD>(q, out, cache, block_table, max_blocks, cu_q_lens, seq_lens, tile_seq,   \
                    tile_start, num_tiles, Hq, Hkv, page_size, scale, window, st)
  DIB_DISPATCH_D(D, CALL)
#undef CALL
}

// The first num_seqs sequences of the batch, one token each (token index = sequence
// index).  part_o: float32 [num_seqs, Hq, max_splits, D]; part_lse: [num_seqs, Hq,
// max_splits]; max_splits >= ceil(longest sequence / 128).
int dib_decode_attention_bf16(const void* q, void* out, const void* cache, long long num_pages,
                              const int* block_table, int max_blocks, const int* seq_lens,
                              float* part_o, float* part_lse, int num_seqs, int max_splits, int Hq,
                              int Hkv, int D, int page_size, float scale, int window,
                              cudaStream_t st) {
  if (num_seqs == 0) return DIB_OK;
  if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16 || num_seqs > 65535 || max_splits > 65535 ||
      max_splits < 1)
    return DIB_BAD_SIZE;
  // page-granular TMA loads where the shape allows them (num_pages <= 0 forces the
  // row-copy kernel)
  if (num_pages > 0 && (D == 64 || D == 128) && page_size >= 8 && page_size <= DEC_SPLIT &&
      DEC_SPLIT % page_size == 0 &&
      (long long)num_pages * 2 * Hkv * page_size < (1ll << 31) &&
      reinterpret_cast<uintptr_t>(cache) % 16 == 0) {
    if (D == 128)
      return launch_decode_tma<128>(q, out, cache, num_pages, block_table, max_blocks, seq_lens,
                                    part_o, part_lse, num_seqs, max_splits, Hq, Hkv, page_size, scale,
                                    window, st);
    return launch_decode_tma<64>(q, out, cache, num_pages, block_table, max_blocks, seq_lens, part_o,
                                 part_lse, num_seqs, max_splits, Hq, Hkv, page_size, scale, window, st);
  }
#define CALL(DD)                                                                                  \
  launch_decode<DD>(q, out, cache, block_table, max_blocks, seq_lens, part_o, part_lse, num_seqs, \
                    max_splits, Hq, Hkv, page_size, scale, window, st)
  DIB_DISPATCH_D(D, CALL)
#undef CALL
}

}  // extern "C"
