// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// float32 accumulation; scores, softmax statistics and the output accumulator are
// float32).
//
// Two kernels share the tile machinery:
//
//  * extend: sequences that bring more than one token (prompt portions, with or
//    without a cached prefix).  The rows of a 64-row tile are (token, query head of
//    one kv group) pairs, so one CTA serves every query head of a kv head and K/V
//    tiles are loaded once per group.  Key tiles of 64 are anchored at absolute
//    position 0, so the order of a query's reduction depends on its position alone.
//
//  * decode: sequences that bring one token.  Split-KV: a CTA takes one (sequence,
//    kv head, split of 128 keys); its 4 warps take 32 keys each and merge in shared
//    memory; stage 2 merges the splits in index order.  The split size is fixed, so
//    the reduction order depends on the sequence's own length only.
//
// Cache layout of a layer: [num_pages, 2, num_kv_heads, page_size, head_dim].
// head_dim: multiples of 16 up to 128.  Group ratio: up to 64 (extend), 16 (decode).
#pragma once
#include "attention_merge.cuh"
#include "common.cuh"

namespace {

constexpr float NEG_BIG = -1e30f;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int PAD = 8;  // bf16 elements of padding per shared-memory row (16 bytes)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- mbarrier + bulk copy (global -> shared, completion counted in bytes)
__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes,
                                         unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Set when a bounded wait ran out; read by dib_attention_bf16_status().
__device__ int dib_attention_error_word = 0;

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                          unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Load `nkeys` keys starting at absolute key index k0 of one kv head into shared
// memory rows [nkeys][D + PAD], K and V, 16 bytes per cp.async.  Keys at or beyond
// kv_len are zero-filled.
template <int D, int NTHREADS>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* sK, __nv_bfloat16* sV,
                                             const __nv_bfloat16* __restrict__ cache,
                                             const int* __restrict__ bt, int k0, int nkeys,
                                             int kv_len, int kvh, int Hkv, int page_size) {
  constexpr int CH = D / 8;  // 16-byte chunks per row
  const size_t head_stride = (size_t)page_size * D;
  const size_t kv_stride = (size_t)Hkv * head_stride;
  for (int c = threadIdx.x; c < nkeys * CH; c += NTHREADS) {
    const int r = c / CH, ch = c % CH;
    const int key = k0 + r;
    const bool valid = key < kv_len;
    const __nv_bfloat16* src = cache;
    if (valid) {
      const int page = bt[key / page_size];
      src = cache + (size_t)page * 2 * kv_stride + (size_t)kvh * head_stride +
            (size_t)(key % page_size) * D + ch * 8;
    }
    cp_async16(sK + r * (D + PAD) + ch * 8, src, valid);
    cp_async16(sV + r * (D + PAD) + ch * 8, valid ? src + kv_stride : src, valid);
  }
}

// One warp: S[16 x NK] = Q[16 x D] K^T for NK keys held in shared memory rows
// [key][D+PAD] starting at row `krow0`.  s[nt] holds the m16n8 accumulator of keys
// nt*8 .. nt*8+7.
template <int D, int NK>
__device__ __forceinline__ void qk_tile(float (&s)[NK / 8][4], const unsigned (&qf)[D / 16][4],
                                        const __nv_bfloat16* sK, int krow0, int lane) {
#pragma unroll
  for (int nt = 0; nt < NK / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
  const int m = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < NK / 16; ++np) {
      unsigned b[4];
      const __nv_bfloat16* p =
          sK + (krow0 + np * 16 + (m >> 1) * 8 + r) * (D + PAD) + ks * 16 + (m & 1) * 8;
      ldmatrix_x4(b, p);
      mma_16816(s[np * 2], qf[ks], b[0], b[1]);
      mma_16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
    }
  }
}

// One warp: O[16 x D] += P[16 x NK] V[NK x D], P given as the (already
// exponentiated) score accumulators, V in shared memory rows [key][D+PAD].
template <int D, int NK>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&p)[NK / 8][4],
                                        const __nv_bfloat16* sV, int krow0, int lane) {
  const int m = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < NK / 16; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(p[kk * 2][0], p[kk * 2][1]);
    a[1] = pack_bf16(p[kk * 2][2], p[kk * 2][3]);
    a[2] = pack_bf16(p[kk * 2 + 1][0], p[kk * 2 + 1][1]);
    a[3] = pack_bf16(p[kk * 2 + 1][2], p[kk * 2 + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      unsigned b[4];
      const __nv_bfloat16* ptr =
          sV + (krow0 + kk * 16 + (m & 1) * 8 + r) * (D + PAD) + dp * 16 + (m >> 1) * 8;
      ldmatrix_x4_trans(b, ptr);
      mma_16816(o[dp * 2], a, b[0], b[1]);
      mma_16816(o[dp * 2 + 1], a, b[2], b[3]);
    }
  }
}

// Mask, running max, exponentials and running sum for the two rows a thread holds
// (row0 = lane/4, row1 = row0 + 8).  Scores arrive as raw dot products; they leave as
// exp2((s*scale - m) * log2e).  `o` is rescaled.  key index of s[nt][i]:
// kbase + nt*8 + (lane%4)*2 + (i&1), row (i>>1).
template <int D, int NK, bool FIRST = false>   // FIRST: o is still zero, nothing to rescale
__device__ __forceinline__ void softmax_tile(float (&s)[NK / 8][4], float (&o)[D / 8][4],
                                             float (&mrow)[2], float (&lrow)[2], int kbase,
                                             const int (&lo)[2], const int (&hi)[2],
                                             float scale_log2, int lane) {
  float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
  for (int nt = 0; nt < NK / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = kbase + nt * 8 + (lane & 3) * 2 + (i & 1);
      const int rr = i >> 1;
      const bool vis = key >= lo[rr] && key <= hi[rr];
      s[nt][i] = vis ? s[nt][i] * scale_log2 : NEG_BIG;
      mx[rr] = fmaxf(mx[rr], s[nt][i]);
    }
  float alpha[2], msafe[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
    mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
    const float mnew = fmaxf(mrow[rr], mx[rr]);
    msafe[rr] = mnew <= -1e29f ? 0.f : mnew;  // nothing visible yet: exponentials become 0
    alpha[rr] = fast_exp2(mrow[rr] - msafe[rr]);
    mrow[rr] = mnew;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nt = 0; nt < NK / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float e = fast_exp2(s[nt][i] - msafe[i >> 1]);
      s[nt][i] = e;
      sum[i >> 1] += e;
    }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 1);
    sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 2);
    lrow[rr] = lrow[rr] * alpha[rr] + sum[rr];
  }
  if (!FIRST) {
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o[dt][0] *= alpha[0];
      o[dt][1] *= alpha[0];
      o[dt][2] *= alpha[1];
      o[dt][3] *= alpha[1];
    }
  }
}

// ------------------------------------------------------------------ extend kernel
constexpr int EXT_M = 64, EXT_N = 64, EXT_THREADS = 128;

template <int D>
__global__ void __launch_bounds__(EXT_THREADS)
extend_attention_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                        const __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ cu_q_lens, const int* __restrict__ seq_lens,
                        const int* __restrict__ tile_seq, const int* __restrict__ tile_start,
                        int Hq, int Hkv, int page_size, float scale, int window) {
  pdl_prologue(q, cache);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sK0 = sQ + EXT_M * (D + PAD);
  constexpr int TILE_ELEMS = EXT_N * (D + PAD);
  // stage s: K at sK0 + s*2*TILE_ELEMS, V right behind it

  // tiles are listed in order of position; the ones with the most keys run first
  const int tile = gridDim.y - 1 - blockIdx.y, kvh = blockIdx.x;
  const int G = Hq / Hkv;
  const int tokens_per_tile = EXT_M / G;
  const int seq = tile_seq[tile];
  const int tok0 = tile_start[tile];  // first token of the tile among the sequence's new tokens
  const int q_begin = cu_q_lens[seq];
  const int q_len = cu_q_lens[seq + 1] - q_begin;
  const int kv_len = seq_lens[seq];
  const int prefix = kv_len - q_len;
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int* bt = block_table + (size_t)seq * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Q tile -> shared memory (rows beyond the tile's tokens are zero)
  constexpr int CH = D / 8;
  for (int c = threadIdx.x; c < EXT_M * CH; c += EXT_THREADS) {
    const int r = c / CH, ch = c % CH;
    const int tl = r / G, g = r % G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tl < ntok) {
      const size_t t = (size_t)(q_begin + tok0 + tl);
      v = *reinterpret_cast<const uint4*>(q + (t * Hq + (size_t)kvh * G + g) * D + ch * 8);
    }
    *reinterpret_cast<uint4*>(sQ + r * (D + PAD) + ch * 8) = v;
  }

  const int first_pos = prefix + tok0, last_pos = prefix + tok0 + ntok - 1;
  const int first_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
  const int j0 = first_key / EXT_N, j1 = last_pos / EXT_N;

  load_kv_tile<D, EXT_THREADS>(sK0, sK0 + TILE_ELEMS, cache, bt, j0 * EXT_N, EXT_N, kv_len, kvh, Hkv,
                               page_size);
  cp_async_commit();
  __syncthreads();  // sQ visible

  unsigned qf[D / 16][4];
  {
    const int m = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(qf[ks], sQ + (warp * 16 + (m & 1) * 8 + r) * (D + PAD) + ks * 16 + (m >> 1) * 8);
  }
  // rows of this thread and what they may see
  int lo[2], hi[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = warp * 16 + (lane >> 2) + rr * 8;
    const int tl = r / G;
    if (tl < ntok) {
      hi[rr] = prefix + tok0 + tl;
      lo[rr] = (window > 0 && hi[rr] - window + 1 > 0) ? hi[rr] - window + 1 : 0;
    } else {
      hi[rr] = -1;  // sees nothing
      lo[rr] = 0;
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[dt][i] = 0.f;
  float mrow[2] = {NEG_BIG, NEG_BIG}, lrow[2] = {0.f, 0.f};
  const float scale_log2 = scale * LOG2E;

  for (int j = j0; j <= j1; ++j) {
    const int stage = (j - j0) & 1;
    __nv_bfloat16* sK = sK0 + stage * 2 * TILE_ELEMS;
    __nv_bfloat16* sV = sK + TILE_ELEMS;
    if (j + 1 <= j1) {
      __nv_bfloat16* nK = sK0 + (stage ^ 1) * 2 * TILE_ELEMS;
      load_kv_tile<D, EXT_THREADS>(nK, nK + TILE_ELEMS, cache, bt, (j + 1) * EXT_N, EXT_N, kv_len,
                                   kvh, Hkv, page_size);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[EXT_N / 8][4];
    qk_tile<D, EXT_N>(s, qf, sK, 0, lane);
    softmax_tile<D, EXT_N>(s, o, mrow, lrow, j * EXT_N, lo, hi, scale_log2, lane);
    pv_tile<D, EXT_N>(o, s, sV, 0, lane);
    __syncthreads();  // the stage is overwritten by the load of tile j+2
  }

  // write the valid rows
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = warp * 16 + (lane >> 2) + rr * 8;
    const int tl = r / G, g = r % G;
    if (tl >= ntok) continue;
    const float inv = 1.0f / lrow[rr];
    const size_t t = (size_t)(q_begin + tok0 + tl);
    __nv_bfloat16* dst = out + (t * Hq + (size_t)kvh * G + g) * D + (lane & 3) * 2;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<__nv_bfloat162*>(dst + dt * 8) =
          __floats2bfloat162_rn(o[dt][rr * 2] * inv, o[dt][rr * 2 + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------ decode kernels
constexpr int DEC_SPLIT = 128, DEC_THREADS = 128, DEC_WARP_KEYS = 32;

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_stage1_kernel(const __nv_bfloat16* __restrict__ q,
                               const __nv_bfloat16* __restrict__ cache,
                               const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ seq_lens, float* __restrict__ part_o,
                               float* __restrict__ part_lse, int max_splits, int Hq, int Hkv,
                               int page_size, float scale, int window) {
  pdl_prologue(q, cache);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sV = sK + DEC_SPLIT * (D + PAD);

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int kv_len = seq_lens[b];
  const int pos = kv_len - 1;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int k0 = split * DEC_SPLIT;
  if (k0 > pos || k0 + DEC_SPLIT <= first_key) return;  // nothing visible in this split
  const int* bt = block_table + (size_t)b * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // K and V rows of the split by bulk copies: thread r owns key k0 + r and issues
  // one copy for its K row and one for its V row (the keys of a head inside a page
  // are contiguous, so a row is D*2 contiguous bytes).  Two barriers count the
  // bytes, so the scores can start while V is still arriving.  Rows at or beyond
  // the sequence's length are zero-filled by their thread.
  static_assert(DEC_SPLIT == MERGE_SPLIT, "one split size");
  static_assert(DEC_THREADS == DEC_SPLIT, "one thread per key row");
  unsigned long long* bars =
      reinterpret_cast<unsigned long long*>(smem_raw + (size_t)2 * DEC_SPLIT * (D + PAD) * 2);
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  __syncthreads();
  {
    const int nvalid = min(DEC_SPLIT, kv_len - k0);
    if (threadIdx.x == 0) {
      mbar_expect_tx(&bars[0], (unsigned)nvalid * D * 2);
      mbar_expect_tx(&bars[1], (unsigned)nvalid * D * 2);
    }
    const int r = threadIdx.x;
    __nv_bfloat16* dk = sK + r * (D + PAD);
    __nv_bfloat16* dv = sV + r * (D + PAD);
    if (r < nvalid) {
      const int key = k0 + r;
      const size_t head_stride = (size_t)page_size * D;
      const size_t kv_stride = (size_t)Hkv * head_stride;
      const int page = bt[key / page_size];
      const __nv_bfloat16* src = cache + (size_t)page * 2 * kv_stride + (size_t)kvh * head_stride +
                                 (size_t)(key % page_size) * D;
      bulk_g2s(dk, src, D * 2, &bars[0]);
      bulk_g2s(dv, src + kv_stride, D * 2, &bars[1]);
    } else {
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        *reinterpret_cast<uint4*>(dk + c * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  }

  // Q fragments straight from global memory: rows are the G heads of the group
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

  __syncthreads();  // zero-filled rows are visible
  if (!mbar_wait(&bars[0], 0)) atomicExch(&dib_attention_error_word, 1);
  float s[DEC_WARP_KEYS / 8][4];
  qk_tile<D, DEC_WARP_KEYS>(s, qf, sK, warp * DEC_WARP_KEYS, lane);
  softmax_tile<D, DEC_WARP_KEYS>(s, o, mrow, lrow, k0 + warp * DEC_WARP_KEYS, lo, hi,
                                 scale * LOG2E, lane);
  if (!mbar_wait(&bars[1], 0)) atomicExch(&dib_attention_error_word, 1);
  pv_tile<D, DEC_WARP_KEYS>(o, s, sV, warp * DEC_WARP_KEYS, lane);
  __syncthreads();  // sK is reused for the merge

  // merge the 4 warps: sO[warp][row][D], sM/sL[warp][row]
  float* sO = reinterpret_cast<float*>(smem_raw);
  float* sM = sO + 4 * 16 * D;
  float* sL = sM + 4 * 16;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = (lane >> 2) + rr * 8;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      const int d = dt * 8 + (lane & 3) * 2;
      sO[(warp * 16 + r) * D + d] = o[dt][rr * 2];
      sO[(warp * 16 + r) * D + d + 1] = o[dt][rr * 2 + 1];
    }
    if ((lane & 3) == 0) {
      sM[warp * 16 + r] = mrow[rr];
      sL[warp * 16 + r] = lrow[rr];
    }
  }
  __syncthreads();
  // per row: the common maximum, each warp's factor (kept in sM) and 1/L (in sL[0])
  if (threadIdx.x < G) {
    const int r = threadIdx.x;
    float M = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 16 + r]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = fast_exp2(sM[w * 16 + r] - M);
      L += sL[w * 16 + r] * f;
      sM[w * 16 + r] = f;
    }
    sL[r] = 1.0f / L;
    const size_t row = ((size_t)b * Hq + (size_t)kvh * G + r) * max_splits + split;
    part_lse[row] = (M + log2f(L)) / LOG2E;  // natural-log domain
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += DEC_THREADS) {
    const int r = idx / D, d = idx % D;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) acc += sO[(w * 16 + r) * D + d] * sM[w * 16 + r];
    const size_t row = ((size_t)b * Hq + (size_t)kvh * G + r) * max_splits + split;
    part_o[row * D + d] = acc * sL[r];
  }
}

// Stage 2: merge the splits of one (sequence, head).  The order of the sums depends on
// the sequence's own length only: the splits are taken in chunks of 16 (chunk c = splits
// 16c .. 16c+15), a chunk is added up in split order, and the chunks' sums are added in
// chunk order.  Two kernels do this: the first with one thread per output dimension,
// for steps whose longest sequence has few chunks; the second with a group of threads per
// chunk, for long sequences.  Both give the same bits for a sequence, whatever else is in
// the batch.  The partial results of the first chunk are requested before the
// sequence's length is known (what lies beyond its last split is read but not used), so
// a sequence of one chunk waits for memory once.
__global__ void decode_attention_stage2_kernel(const float* __restrict__ part_o,
                                               const float* __restrict__ part_lse,
                                               const int* __restrict__ seq_lens,
                                               __nv_bfloat16* __restrict__ out, int max_splits,
                                               int Hq, int D, int window) {
  pdl_prologue(part_o, part_lse);
  constexpr int CH = MERGE_CH;
  const int b = blockIdx.x, h = blockIdx.y;
  const size_t row = ((size_t)b * Hq + h) * max_splits;
  const int kv_len = seq_lens[b];
  float lse_r[CH], o_r[CH][1];
#pragma unroll
  for (int j = 0; j < CH; ++j) lse_r[j] = j < max_splits ? part_lse[row + j] : NEG_BIG;
#pragma unroll
  for (int j = 0; j < CH; ++j)
    o_r[j][0] = (j < max_splits && (int)threadIdx.x < D) ? part_o[(row + j) * D + threadIdx.x] : 0.f;
  // (a caller that passes fewer splits than the sequence has keys for gets a result over
  // the splits there are, never a read beyond the row)
  int s0, s1;
  merge_range(kv_len, window, max_splits, s0, s1);
  const int c0 = s0 / CH, c1 = s1 / CH;
  float M = NEG_BIG;
#pragma unroll
  for (int j = 0; j < CH; ++j)
    if (j >= s0 && j <= s1) M = fmaxf(M, lse_r[j]);
  for (int s = max(s0, CH); s <= s1; ++s) M = fmaxf(M, part_lse[row + s]);
  bool first = true;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float total[1] = {0.f}, total_den = 0.f;
    for (int c = c0; c <= c1; ++c) {
      if (c > 0 || !first) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int s = c * CH + j;
          const bool in = s >= s0 && s <= s1;
          lse_r[j] = in ? part_lse[row + s] : NEG_BIG;
          o_r[j][0] = in ? part_o[(row + s) * D + d] : 0.f;
        }
      }
      float acc[1], den;
      merge_chunk<1>(lse_r, o_r, c, s0, s1, M, acc, den);
      merge_add<1>(c == c0, acc, den, total, total_den);
    }
    out[((size_t)b * Hq + h) * D + d] = __float2bfloat16_rn(merge_finish(total[0], total_den));
    first = false;
  }
}

// The kernel for long sequences: chunk c belongs to group c % 8 of the block's groups of
// D threads (a block has as many groups as the step's longest sequence has chunks, 8 at
// most); a group leaves each of its chunks' sums in shared memory, and the first group
// adds them in chunk order.  For at most MERGE_MAX_CHUNKS chunks of a sequence's range.
constexpr int MERGE_GROUPS = 8, MERGE_MAX_CHUNKS = 64;
__global__ void __launch_bounds__(1024)
decode_attention_stage2_wide_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_lse,
                                    const int* __restrict__ seq_lens,
                                    __nv_bfloat16* __restrict__ out, int max_splits, int Hq, int D,
                                    int window) {
  pdl_prologue(part_o, part_lse);
  constexpr int CH = MERGE_CH;
  __shared__ float s_acc[MERGE_MAX_CHUNKS][128];
  __shared__ float s_den[MERGE_MAX_CHUNKS];
  __shared__ float s_max[MERGE_GROUPS];
  const int b = blockIdx.x, h = blockIdx.y;
  const int d = threadIdx.x, g = threadIdx.y;
  const int groups = blockDim.y;
  const size_t row = ((size_t)b * Hq + h) * max_splits;
  const int kv_len = seq_lens[b];
  // chunk g is requested before the sequence's length is known: it is this group's
  // first chunk unless a window has moved the range past it
  float lse_r[CH], o_r[CH][1];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int s = g * CH + j;
    lse_r[j] = s < max_splits ? part_lse[row + s] : NEG_BIG;
    o_r[j][0] = (s < max_splits && d < D) ? part_o[(row + s) * D + d] : 0.f;
  }
  int s0, s1;
  merge_range(kv_len, window, max_splits, s0, s1);
  const int c0 = s0 / CH, c1 = s1 / CH;
  // the largest lse of the sequence's splits (a maximum does not depend on the order):
  // every thread of a group over the group's chunks, then over the groups
  float m = NEG_BIG;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int s = g * CH + j;
    if (s >= s0 && s <= s1) m = fmaxf(m, lse_r[j]);
  }
  for (int c = g + MERGE_GROUPS; c <= c1; c += MERGE_GROUPS)
    for (int j = 0; j < CH; ++j) {
      const int s = c * CH + j;
      if (s >= s0 && s <= s1) m = fmaxf(m, part_lse[row + s]);
    }
  if (d == 0) s_max[g] = m;
  __syncthreads();
  float M = NEG_BIG;
  for (int k = 0; k < groups; ++k) M = fmaxf(M, s_max[k]);

  for (int c = g; c <= c1; c += MERGE_GROUPS) {
    if (c < c0) continue;
    if (c != g) {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int s = c * CH + j;
        const bool in = s >= s0 && s <= s1;
        lse_r[j] = in ? part_lse[row + s] : NEG_BIG;
        o_r[j][0] = (in && d < D) ? part_o[(row + s) * D + d] : 0.f;
      }
    }
    float acc[1], den;
    merge_chunk<1>(lse_r, o_r, c, s0, s1, M, acc, den);
    if (c0 == c1) {      // one chunk: its sum is the result
      if (d < D) out[((size_t)b * Hq + h) * D + d] = __float2bfloat16_rn(merge_finish(acc[0], den));
    } else {
      if (d < D) s_acc[c - c0][d] = acc[0];
      if (d == 0) s_den[c - c0] = den;
    }
  }
  if (c0 == c1) return;    // uniform over the block
  __syncthreads();
  if (g == 0 && d < D) {
    float total = s_acc[0][d], total_den = s_den[0];
    for (int k = 1; k <= c1 - c0; ++k) {
      total = __fadd_rn(total, s_acc[k][d]);
      total_den = __fadd_rn(total_den, s_den[k]);
    }
    out[((size_t)b * Hq + h) * D + d] = __float2bfloat16_rn(merge_finish(total, total_den));
  }
}

// From how many splits on the merge runs as the kernel with a group of threads per chunk
// (measurements and tests change it through dib_attention_bf16_set_merge_wide_from).
static inline int& merge_wide_from() {
  static int v = 49;
  return v;
}

// Stage 2 of the split-KV decode attention: the kernel for at most 16 splits, or the
// wide one.
static inline void launch_decode_merge(const float* part_o, const float* part_lse, const int* seq_lens,
                                       void* out, int num_seqs, int max_splits, int Hq, int D,
                                       int window, cudaStream_t st) {
  const int th = D < 32 ? 32 : (D + 31) / 32 * 32;
  const int chunks = (max_splits + 15) / 16;
  const int wide_from = merge_wide_from();
  if (max_splits >= wide_from && max_splits > MERGE_CH && th <= 128 && chunks <= MERGE_MAX_CHUNKS)
    dib_launch(decode_attention_stage2_wide_kernel, dim3(num_seqs, Hq),
               dim3(th, chunks < MERGE_GROUPS ? chunks : MERGE_GROUPS), 0, st,
               part_o, part_lse, seq_lens, (__nv_bfloat16*)out, max_splits, Hq, D, window);
  else
    dib_launch(decode_attention_stage2_kernel, dim3(num_seqs, Hq), dim3(th), 0, st, part_o, part_lse,
               seq_lens, (__nv_bfloat16*)out, max_splits, Hq, D, window);
}

template <int D>
int launch_extend(const void* q, void* out, const void* cache, const int* bt, int max_blocks,
                  const int* cu_q_lens, const int* seq_lens, const int* tile_seq,
                  const int* tile_start, int num_tiles, int Hq, int Hkv, int page_size, float scale,
                  int window, cudaStream_t st) {
  const size_t smem = (size_t)(EXT_M + 4 * EXT_N) * (D + PAD) * sizeof(__nv_bfloat16);
  auto kern = extend_attention_kernel<D>;
  static DeviceOnce attr_set;  // once per instantiation and device; never during a stream capture
  if (smem > 40 * 1024 && !attr_set.done()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  dim3 grid(Hkv, num_tiles);   // x-then-y order: all kv heads of the longest tile first
  dib_launch(kern, dim3(grid), dim3(EXT_THREADS), smem, st, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                                        (const __nv_bfloat16*)cache, bt, max_blocks, cu_q_lens,
                                        seq_lens, tile_seq, tile_start, Hq, Hkv, page_size, scale,
                                        window);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

template <int D>
int launch_decode(const void* q, void* out, const void* cache, const int* bt, int max_blocks,
                  const int* seq_lens, float* part_o, float* part_lse, int num_seqs, int max_splits,
                  int Hq, int Hkv, int page_size, float scale, int window, cudaStream_t st) {
  size_t smem = (size_t)2 * DEC_SPLIT * (D + PAD) * sizeof(__nv_bfloat16) + 16;  // + 2 barriers
  const size_t merge = (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float);
  if (merge > smem) smem = merge;
  auto kern = decode_attention_stage1_kernel<D>;
  static DeviceOnce attr_set;
  if (smem > 40 * 1024 && !attr_set.done()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  dim3 grid(Hkv, num_seqs, max_splits);
  dib_launch(kern, dim3(grid), dim3(DEC_THREADS), smem, st, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, bt,
                                        max_blocks, seq_lens, part_o, part_lse, max_splits, Hq, Hkv,
                                        page_size, scale, window);
  DIB_CHECK_LAUNCH();
  if (out != nullptr) {
    launch_decode_merge(part_o, part_lse, seq_lens, out, num_seqs, max_splits, Hq, D, window, st);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // namespace

#define DIB_DISPATCH_D(D, CALL)            \
  switch (D) {                             \
    case 16: return CALL(16);              \
    case 32: return CALL(32);              \
    case 48: return CALL(48);              \
    case 64: return CALL(64);              \
    case 80: return CALL(80);              \
    case 96: return CALL(96);              \
    case 112: return CALL(112);            \
    case 128: return CALL(128);            \
    default: return DIB_BAD_SIZE;          \
  }

