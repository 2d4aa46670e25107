// Prefill / extend attention over the paged cache on the 5th-generation tensor
// cores: S = Q K^T and O_j = P V by tcgen05.mma with accumulators in tensor memory,
// K and V pages fetched by TMA into 128-byte-swizzled tiles, softmax in float32 by
// one thread per query row.  Two kernels: the one described first (one query tile per
// CTA), and the default, which gives a CTA two query tiles (described at its definition).
//
// First kernel.  A CTA owns 128 rows = (token, query head of one kv group) pairs of one sequence and
// walks the key tiles of 128 keys from position 0 (or the window's start) to its last
// token, so the order of a row's reduction depends on its position alone.  Ten warps:
//   warps 0-7  softmax: two threads share a row (tensor-memory lane = row; warp w reads
//              lanes 32(w%4).., and half w/4 of the columns).  Both read all of S_j for
//              the row's maximum; each computes the probabilities of its 64 keys against
//              a reference maximum, writes them (bf16) to shared memory as the A operand
//              of the second product and keeps the sum of its half.  O stays in tensor
//              memory and is accumulated there by the MMA; a row's O is rescaled (read,
//              multiplied, written back) only when the reference maximum has to rise.
//   warp 8     TMA: one copy per (page, key-or-value, 64-column half) of a tile, two
//              stages.
//   warp 9     MMA issue: S is double-buffered in tensor memory, so S_{j+1} = Q K_{j+1}^T
//              runs while the softmax threads work on S_j; O += P_j V_j follows as soon
//              as P_j is in shared memory.
// Operand layouts (all 128-byte swizzle): Q, K, P K-major [halves][rows][64]; V is
// read as the MN-major B operand straight from its [key][dim] tile.  head_dim 128,
// group ratio dividing 128, page_size dividing 128 (at least 8).  Every mbarrier wait
// is bounded; a wait that runs out sets the error word and the kernel unwinds.
#include <cuda.h>

#include <map>
#include <tuple>

#include "attention_bf16_kernels.cuh"

namespace {

constexpr int TC_M = 128, TC_N = 128, TC_D = 128, TC_THREADS = 320;
constexpr int TMA_WARP = 8, MMA_WARP = 9;
constexpr int PAIR_THREADS = 384, PAIR_V_WARP = 10;   // the pair kernel fetches keys (warp 8) and values apart
// Registers are handed out to groups of four warps.  The pair kernel's third group (keys,
// products, values, one warp without work) gives most of its registers back and the two
// groups of softmax threads, each of which holds a row of 128 scores, take them.
constexpr int PAIR_REGS_FEW = 56, PAIR_REGS_MANY = 224;      // 128 * 56 + 256 * 224 = 64,512
template <int N> __device__ __forceinline__ void regs_give() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void regs_take() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
constexpr int TILE_BYTES = 128 * 128 * 2;   // a [128 x 128] bf16 tile (two 64-column halves)
constexpr int HALF_BYTES = 128 * 64 * 2;

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)),
      "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long desc_a,
                                       unsigned long long desc_b, unsigned idesc, unsigned accum) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accum), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 consecutive columns of this thread's lane; the values are valid after tc_wait_ld().
__device__ __forceinline__ void tc_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
      "%12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ void tc_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
      "%12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31, %32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
      "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// K-major operand, rows of 128 bytes, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_k_major(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
// MN-major operand (V as [key][dim] rows of 128 bytes per 64-dim half): 64 dims are
// contiguous, the next 64 dims lie `half_stride` bytes on (leading byte offset), 8-key
// groups are 1024 bytes apart (stride byte offset).
__device__ __forceinline__ unsigned long long desc_mn_major(unsigned addr, unsigned half_stride) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)((half_stride >> 4) & 0x3FFFu) << 16;
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
constexpr unsigned idesc_f16(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_mn_major << 16) |
         ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

// byte offset of (row, 16-byte chunk c of the row's 128 elements) in a [2][128][64] bf16 tile
__device__ __forceinline__ int sw_chunk_off(int row, int c) {
  return (c >> 3) * HALF_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(TC_THREADS, 1)
extend_attention_tc_kernel(const __grid_constant__ CUtensorMap map,
                           const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                           const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ cu_q_lens, const int* __restrict__ seq_lens,
                           const int* __restrict__ tile_seq, const int* __restrict__ tile_start,
                           int Hq, int Hkv, int page_size, float scale, int window) {
  if (threadIdx.x == 0) prefetch_tensormap(&map);
  pdl_prologue(q);
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;                       // 32 KB
  unsigned char* sP = smem + TILE_BYTES;          // 32 KB
  unsigned char* sKV = smem + 2 * TILE_BYTES;     // 2 stages x (K 32 KB + V 32 KB)
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + 6 * TILE_BYTES);
  unsigned long long* kv_full = bars;             // [2] K and V of a tile are in shared memory
  unsigned long long* kv_empty = bars + 2;        // [2] both products of the tile have read them
  unsigned long long* s_full = bars + 4;          // [2] S_j is in tensor memory (buffer j & 1)
  unsigned long long* s_free = bars + 6;          // [2] the softmax threads have read it (256)
  unsigned long long* p_full = bars + 8;          // P_j is in shared memory, O is rescaled (256)
  unsigned long long* o_done = bars + 9;          // O += P_j V_j has completed
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 10);

  // blocks are handed out in x-then-y order: y counts the tiles from the longest down
  const int tile = gridDim.y - 1 - blockIdx.y, kvh = blockIdx.x;
  const int G = Hq / Hkv;
  const int tokens_per_tile = TC_M / G;
  const int seq = tile_seq[tile];
  const int tok0 = tile_start[tile];
  const int q_begin = cu_q_lens[seq];
  const int q_len = cu_q_lens[seq + 1] - q_begin;
  const int kv_len = seq_lens[seq];
  const int prefix = kv_len - q_len;
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int* bt = block_table + (size_t)seq * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int first_pos = prefix + tok0, last_pos = prefix + tok0 + ntok - 1;
  const int first_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
  const int j0 = first_key / TC_N, j1 = last_pos / TC_N;
  const int ntiles = j1 - j0 + 1;

  if (warp == MMA_WARP && lane == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
    }
    mbar_init(p_full, 256);
    mbar_init(o_done, 1);
    mbar_fence_init();
  }
  if (warp == TMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  // Q tile -> shared memory, swizzled; rows beyond the tile's tokens are zero
  for (int c = threadIdx.x; c < TC_M * 16; c += TC_THREADS) {
    const int r = c >> 4, ch = c & 15;
    const int tl = r / G, g = r % G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tl < ntok) {
      const size_t t = (size_t)(q_begin + tok0 + tl);
      v = *reinterpret_cast<const uint4*>(q + (t * Hq + (size_t)kvh * G + g) * TC_D + ch * 8);
    }
    *reinterpret_cast<uint4*>(sQ + sw_chunk_off(r, ch)) = v;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q is read by the MMA unit
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_slot;
  const unsigned tmem_o = tmem + 256;   // columns 0..127: S (even tiles), 128..255: S (odd), 256..383: O
  bool ok = true;

  if (warp == TMA_WARP) {
    // ---- TMA: one copy per (page, K or V, half); lanes share the copies of a tile
    const int pages = TC_N / page_size;
    const int ops = pages * 4;
    for (int i = 0; i < ntiles && ok; ++i) {
      const int st = i & 1;
      if (i >= 2) ok = mbar_wait(&kv_empty[st], ((i >> 1) - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) mbar_expect_tx(&kv_full[st], 2 * TILE_BYTES);
      __syncwarp();
      const int k0 = (j0 + i) * TC_N;
      for (int op = lane; op < ops; op += 32) {
        const int pi = op >> 2, kv = (op >> 1) & 1, half = op & 1;
        const int idx = k0 / page_size + pi;
        const int page = idx < max_blocks ? bt[idx] : 0;
        const int row0 = (((page * 2 + kv) * Hkv) + kvh) * page_size;
        unsigned char* dst = sKV + st * 2 * TILE_BYTES + kv * TILE_BYTES + half * HALF_BYTES +
                             pi * page_size * 128;
        tma_load_2d(dst, &map, half * 64, row0, &kv_full[st]);
      }
    }
  } else if (warp == MMA_WARP) {
    // ---- MMA issue (one lane).  S of the next tile is issued before P V of this one, so
    // it runs while the softmax threads work on this tile.
    if (lane == 0) {
      constexpr unsigned idesc_s = idesc_f16(TC_M, TC_N, 0);
      constexpr unsigned idesc_o = idesc_f16(TC_M, TC_D, 1);
      const unsigned q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int i) {
        const unsigned k_addr = smem_u32(sKV + (i & 1) * 2 * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < TC_D / 16; ++ks) {
          const unsigned off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          tc_mma(tmem + (i & 1) * 128, desc_k_major(q_addr + off), desc_k_major(k_addr + off),
                 idesc_s, ks > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[i & 1]);
      };
      ok = mbar_wait(&kv_full[0], 0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int i = 0; i < ntiles && ok; ++i) {
        if (i + 1 < ntiles) {
          ok = mbar_wait(&kv_full[(i + 1) & 1], ((i + 1) >> 1) & 1);
          if (ok && i + 1 >= 2) ok = mbar_wait(&s_free[(i + 1) & 1], (((i + 1) >> 1) - 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_s(i + 1);
        }
        ok = mbar_wait(p_full, i & 1);   // P_i is in shared memory, O is rescaled
        if (!ok) break;
        tc_fence_after();
        const unsigned v_addr = smem_u32(sKV + (i & 1) * 2 * TILE_BYTES + TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < TC_N / 16; ++ks) {
          const unsigned a_off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;   // 16 keys of P
          const unsigned b_off = ks * 16 * 128;                            // 16 key rows of V
          tc_mma(tmem_o, desc_k_major(p_addr + a_off), desc_mn_major(v_addr + b_off, HALF_BYTES),
                 idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
        }
        tc_commit(o_done);
        tc_commit(&kv_empty[i & 1]);
      }
    }
  } else {
    // ---- softmax: two threads per row, each with half of the keys and of the dims.
    // The exponentials are taken against a reference maximum that is only raised when the
    // tile's maximum exceeds it by more than 2^8; O (in tensor memory) and the sum are
    // rescaled then.  The result is the same sum, scaled by a common factor that the
    // final division removes.
    const int r = threadIdx.x & 127;
    const int hf = threadIdx.x >> 7;                 // 0: keys/dims 0..63, 1: 64..127
    const int tl = r / G, g = r % G;
    const bool valid = tl < ntok;
    const int hi = valid ? prefix + tok0 + tl : -1;
    const int lo = (valid && window > 0 && hi - window + 1 > 0) ? hi - window + 1 : 0;
    const float scale_log2 = scale * LOG2E;
    const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    float m_ref = NEG_BIG, l = 0.f;
    for (int i = 0; i < ntiles && ok; ++i) {
      const unsigned tmem_s = tmem + (i & 1) * 128;
      ok = mbar_wait(&s_full[i & 1], (i >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int kbase = (j0 + i) * TC_N;
      const bool full = kbase >= lo && kbase + TC_N - 1 <= hi;   // no key of the tile is masked
      // pass 1: the row's maximum over all 128 keys (both threads of the row)
      float mx = NEG_BIG;
#pragma unroll
      for (int c = 0; c < TC_N / 64; ++c) {
        unsigned v0[32], v1[32];
        tc_ld32(tmem_s + lane_base + c * 64, v0);
        tc_ld32(tmem_s + lane_base + c * 64 + 32, v1);
        tc_wait_ld();
        if (full) {
#pragma unroll
          for (int k = 0; k < 32; ++k)
            mx = fmaxf(mx, fmaxf(__uint_as_float(v0[k]), __uint_as_float(v1[k])));
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int key = kbase + c * 64 + k;
            if (key >= lo && key <= hi) mx = fmaxf(mx, __uint_as_float(v0[k]));
            if (key + 32 >= lo && key + 32 <= hi) mx = fmaxf(mx, __uint_as_float(v1[k]));
          }
        }
      }
      mx = mx <= -1e29f ? NEG_BIG : mx * scale_log2;   // scale is positive
      // raise the reference only when it must be (or at the first visible key)
      float factor = 1.0f;
      bool rescale = false;
      if (mx > m_ref + 8.0f) {
        rescale = m_ref > -1e29f;
        factor = rescale ? fast_exp2(m_ref - mx) : 0.f;
        m_ref = mx;
        l *= factor;
      }
      const float m_use = m_ref <= -1e29f ? 0.f : m_ref;
      // pass 2: probabilities of this thread's 64 keys, 32 at a time
      unsigned pk[32];
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        unsigned v[32];
        tc_ld32(tmem_s + lane_base + hf * 64 + c * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          const int key = kbase + hf * 64 + c * 32 + k;
          const bool vis0 = full || (key >= lo && key <= hi);
          const bool vis1 = full || (key + 1 >= lo && key + 1 <= hi);
          const float p0 = vis0 ? fast_exp2(__uint_as_float(v[k]) * scale_log2 - m_use) : 0.f;
          const float p1 = vis1 ? fast_exp2(__uint_as_float(v[k + 1]) * scale_log2 - m_use) : 0.f;
          sum += p0 + p1;
          pk[c * 16 + (k >> 1)] = pack_bf16(p0, p1);
        }
      }
      l += sum;
      tc_fence_before();
      mbar_arrive(&s_free[i & 1]);            // S_i has been read: S_{i+2} may overwrite it
      // P_{i-1} V_{i-1} must have completed before P is overwritten and O is touched
      if (i > 0) {
        ok = mbar_wait(o_done, (i - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          unsigned v[32];
          tc_ld32(tmem_o + lane_base + hf * 64 + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * (rescale ? factor : 1.0f));
          tc_st32(tmem_o + lane_base + hf * 64 + c * 32, v);
        }
        tc_wait_st();
      }
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(sP + sw_chunk_off(r, hf * 8 + ch)) =
            make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(p_full);
    }
    // the last product, then O / (sum of the row's two halves)
    if (ok) {
      ok = mbar_wait(o_done, (ntiles - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    tc_fence_after();
    float* sL = reinterpret_cast<float*>(sP);       // free now
    sL[hf * 128 + r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_row = sL[r] + sL[128 + r];
    if (ok) {
      const float inv = 1.0f / l_row;
      const size_t t = (size_t)(q_begin + tok0 + tl);
      __nv_bfloat16* dst = out + (t * Hq + (size_t)kvh * G + g) * TC_D + hf * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        unsigned v[32];
        tc_ld32(tmem_o + lane_base + hf * 64 + c * 32, v);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 o4;
            o4.x = pack_bf16(__uint_as_float(v[ch * 8 + 0]) * inv, __uint_as_float(v[ch * 8 + 1]) * inv);
            o4.y = pack_bf16(__uint_as_float(v[ch * 8 + 2]) * inv, __uint_as_float(v[ch * 8 + 3]) * inv);
            o4.z = pack_bf16(__uint_as_float(v[ch * 8 + 4]) * inv, __uint_as_float(v[ch * 8 + 5]) * inv);
            o4.w = pack_bf16(__uint_as_float(v[ch * 8 + 6]) * inv, __uint_as_float(v[ch * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + ch * 8) = o4;
          }
        }
      }
    }
  }
  if (!ok) atomicExch(&dib_attention_error_word, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == TMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
}

// ------------------------------------------------------------------------------
// Two query tiles per CTA.  The CTA owns two tiles A and B of 128 rows (same sequence,
// same kv head, anywhere in it), which share every key/value tile they both need.
// Warps 0-3 are the softmax threads of A, warps 4-7 those of B: ONE thread per row,
// the row's 128 scores in registers, so maximum, exponentials and sum need no
// exchange.  The probabilities go back to tensor memory, packed as bfloat16 over the
// scores they came from, and are the A operand of the second product straight from
// there (no shared memory, no proxy fence).  The MMA warp staggers the two tiles:
// after O_A += P_A V it issues S_A of the next key tile at once, then turns to B, so
// each tile's softmax runs while the tensor core works for the other tile.
// Warp 8 fetches the keys, warp 10 the values (each refills a stage as soon as it is
// free; both send for the first two key tiles before Q is loaded), warp 9 issues the
// products.  When one tile has had its last key tile, or has none (B = -1), the other
// runs alone and takes the idle tile's score columns as a second buffer (see solo_from).
// Tensor memory: S_A/P_A columns 0..127, S_B/P_B 128..255, O_A 256..383, O_B 384..511.
__device__ __forceinline__ void tc_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long desc_b,
                                          unsigned idesc, unsigned accum) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accum), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

// 2^x for x <= ~8 on the FMA and integer pipes, two values at once with the packed float32
// instructions (the special-function unit makes 16 exponentials per clock and SM, which
// would bound the softmax of a tile): x = n + f with n the nearest integer, 2^f by a cubic
// (relative error 1e-4, below the bfloat16 step of the probabilities), 2^n by adding n to
// the exponent bits.  The packed operations round each half as the single ones do.
__device__ __forceinline__ float2 exp2_fma2(float2 x) {
  x.x = fmaxf(x.x, -125.0f);
  x.y = fmaxf(x.y, -125.0f);
  const float2 magic = make_float2(12582912.0f, 12582912.0f);
  const float2 xf = __fadd2_rn(x, magic);
  const float2 t = __fadd2_rn(xf, make_float2(-12582912.0f, -12582912.0f));
  const float2 f = __ffma2_rn(t, make_float2(-1.0f, -1.0f), x);
  float2 p = __ffma2_rn(f, make_float2(0.05500893f, 0.05500893f), make_float2(0.24221095f, 0.24221095f));
  p = __ffma2_rn(p, f, make_float2(0.6932829f, 0.6932829f));
  p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(xf.x) << 23)),
                     __int_as_float(__float_as_int(p.y) + (__float_as_int(xf.y) << 23)));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__global__ void __launch_bounds__(PAIR_THREADS, 1)
extend_attention_tc_pair_kernel(const __grid_constant__ CUtensorMap map,
                                const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                                const int* __restrict__ block_table, int max_blocks,
                                const int* __restrict__ cu_q_lens, const int* __restrict__ seq_lens,
                                const int* __restrict__ tile_seq, const int* __restrict__ tile_start,
                                const int* __restrict__ tile_start_b, int Hq, int Hkv,
                                int page_size, float scale, int window,
                                int chunk_tiles, const int* __restrict__ tile_chunk, int max_chunks,
                                float* __restrict__ part_o, float* __restrict__ part_ml) {
  if (threadIdx.x == 0) prefetch_tensormap(&map);
  pdl_prologue(q);
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;                       // [2] x 32 KB
  unsigned char* sKV = smem + 2 * TILE_BYTES;     // 2 stages x (K 32 KB + V 32 KB)
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + 6 * TILE_BYTES);
  unsigned long long* k_full = bars;              // [2] the keys of a key tile are in shared memory
  unsigned long long* k_empty = bars + 2;         // [2] both score products have read them
  unsigned long long* v_full = bars + 4;          // [2] the values of a key tile are in shared memory
  unsigned long long* v_empty = bars + 6;         // [2] both output products have read them
  unsigned long long* s_full = bars + 8;          // [2: A, B] the tile's scores are in tensor memory
  unsigned long long* p_full = bars + 10;         // [2] its probabilities are, and O is rescaled (128)
  unsigned long long* o_final = bars + 12;        // [2] its last product has completed
  unsigned long long* pv_done = bars + 14;        // an output product of the tile that runs alone has completed
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 15);

  const int tile = gridDim.y - 1 - blockIdx.y, kvh = blockIdx.x;
  const int G = Hq / Hkv;
  const int npt = TC_M / G;                       // tokens of one query tile
  const int seq = tile_seq[tile];
  const int tokx[2] = {tile_start[tile], tile_start_b[tile]};   // first token of A and of B (-1: no B)
  const int q_begin = cu_q_lens[seq];
  const int q_len = cu_q_lens[seq + 1] - q_begin;
  const int kv_len = seq_lens[seq];
  const int prefix = kv_len - q_len;
  const int* bt = block_table + (size_t)seq * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Per query tile: its tokens and the key tiles it needs.  With chunk_tiles > 0 the key
  // range is cut into chunks of that many key tiles, anchored at key 0, and this CTA
  // takes the chunk its list entry names: a tile whose range spans several chunks gets
  // partial results (unnormalised O, reference maximum, sum) that a second kernel
  // merges; a tile whose range lies in one chunk is finished here.
  int ntok[2], jf[2], jl[2];
  bool whole[2];
  const int chunk = chunk_tiles > 0 ? tile_chunk[tile] : 0;
  const int c_lo = chunk * chunk_tiles;
  const int c_hi = chunk_tiles > 0 ? c_lo + chunk_tiles - 1 : 0x7fffffff;
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int t0 = tokx[x];
    ntok[x] = t0 >= 0 ? max(0, min(npt, q_len - t0)) : 0;
    const int first_pos = prefix + t0, last_pos = prefix + t0 + ntok[x] - 1;
    const int first_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int f = first_key / TC_N;
    const int l = ntok[x] > 0 ? last_pos / TC_N : -1;     // an empty tile is never active
    whole[x] = chunk_tiles <= 0 || f / chunk_tiles == l / chunk_tiles;
    jf[x] = max(f, c_lo);
    jl[x] = min(l, c_hi);
  }
  const bool any0 = jl[0] >= jf[0], any1 = jl[1] >= jf[1];
  if (!any0 && !any1) return;     // nothing of this chunk concerns the pair
  const int j0 = any0 && any1 ? min(jf[0], jf[1]) : (any0 ? jf[0] : jf[1]);
  const int ntiles = max(any0 ? jl[0] : -1, any1 ? jl[1] : -1) - j0 + 1;
  auto active = [&](int x, int i) { return j0 + i >= jf[x] && j0 + i <= jl[x]; };
  // Once one tile has had its last key tile, the other runs alone (a tile early in a
  // prompt beside one late in it).  Alone it would wait for the tensor core and the
  // tensor core for it, in turn; so from key tile `solo_from` on it takes the finished
  // tile's score columns as a second buffer: the scores of key tile i + 1 are computed
  // while its softmax works on tile i.  solo_x is that tile, 1 - solo_x the finished one.
  const int solo_x = (any1 && (!any0 || jl[1] >= jl[0])) ? 1 : 0;
  const int n_other = (solo_x ? any0 : any1) ? jl[1 - solo_x] - jf[1 - solo_x] + 1 : 0;   // its key tiles
  const int solo_from = max((solo_x ? any0 : any1) ? jl[1 - solo_x] - j0 + 1 : 0, jf[solo_x] - j0);

  bool ok = true;
  // The warp that fetches the keys and the one that fetches the values each prepare
  // their own barriers and send for the first two key tiles at once, beside the loading
  // of Q below.  Lane l takes half (64 dimensions) l & 1 of page l >> 1 of a key tile.
  const int tile_ops = TC_N / page_size * 2;
  auto fetch = [&](int kv, int i, int page) {
    const int st = i & 1;
    unsigned long long* full = kv ? &v_full[st] : &k_full[st];
    if (lane == 0) mbar_expect_tx(full, TILE_BYTES);
    __syncwarp();
    if (lane < tile_ops) {
      const int pi = lane >> 1, half = lane & 1;
      const int row0 = (((page * 2 + kv) * Hkv) + kvh) * page_size;
      unsigned char* dst = sKV + st * 2 * TILE_BYTES + kv * TILE_BYTES + half * HALF_BYTES +
                           pi * page_size * 128;
      tma_load_2d(dst, &map, half * 64, row0, full);
    }
  };
  auto page_of = [&](int i) {      // this lane's page of key tile i
    const int idx = (j0 + i) * (TC_N / page_size) + (lane >> 1);
    return (lane < tile_ops && i < ntiles && idx < max_blocks) ? bt[idx] : 0;
  };
  if (warp == TMA_WARP || warp == PAIR_V_WARP) {
    const int kv = warp == PAIR_V_WARP;
    if (lane == 0) {
      for (int i = 0; i < 2; ++i) {
        mbar_init(kv ? &v_full[i] : &k_full[i], 1);
        mbar_init(kv ? &v_empty[i] : &k_empty[i], 1);
      }
      mbar_fence_init();
    }
    __syncwarp();
    const int p0 = page_of(0), p1 = page_of(1);
    fetch(kv, 0, p0);
    if (ntiles > 1) fetch(kv, 1, p1);
  }
  if (warp == MMA_WARP) {
    if (lane == 0) {
      mbar_init(pv_done, 1);
      for (int i = 0; i < 2; ++i) {
        mbar_init(&s_full[i], 1);
        mbar_init(&p_full[i], 128);
        mbar_init(&o_final[i], 1);
      }
      mbar_fence_init();
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  // both Q tiles -> shared memory, swizzled; rows beyond a tile's tokens are zero.  All of
  // a thread's loads go out before its first store (one memory round-trip, not thirteen).
  {
    constexpr int LOADERS = 256;      // the softmax threads: the other warps are busy with keys, values and tensor memory
    constexpr int PER_THREAD = 2 * TC_M * 16 / LOADERS;
    uint4 v[PER_THREAD];
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int c = threadIdx.x + it * LOADERS;
      const int x = c >> 11, r = (c >> 4) & 127, ch = c & 15;
      const int tl = r / G, g = r % G;
      v[it] = make_uint4(0, 0, 0, 0);
      if (threadIdx.x < LOADERS && tl < ntok[x]) {
        const size_t t = (size_t)(q_begin + tokx[x] + tl);
        v[it] = *reinterpret_cast<const uint4*>(q + (t * Hq + (size_t)kvh * G + g) * TC_D + ch * 8);
      }
    }
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int c = threadIdx.x + it * LOADERS;
      const int x = c >> 11, r = (c >> 4) & 127, ch = c & 15;
      if (threadIdx.x < LOADERS) *reinterpret_cast<uint4*>(sQ + x * TILE_BYTES + sw_chunk_off(r, ch)) = v[it];
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q is read by the MMA unit
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_slot;

  if (warp >= TMA_WARP) {
  regs_give<PAIR_REGS_FEW>();
  if (warp == TMA_WARP || warp == PAIR_V_WARP) {
    // Keys and values of a key tile are fetched, waited for and handed back apart, each
    // by a warp of its own: the keys are free again after the score products, long
    // before the values, and neither waits for the other's stage.  The page ids of the
    // next key tile are read while the warp waits for its stage.
    const int kv = warp == PAIR_V_WARP;
    for (int i = 2; i < ntiles && ok; ++i) {
      const int page = page_of(i);
      ok = mbar_wait(kv ? &v_empty[i & 1] : &k_empty[i & 1], ((i >> 1) - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fetch(kv, i, page);
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr unsigned idesc_s = idesc_f16(TC_M, TC_N, 0);
      constexpr unsigned idesc_o = idesc_f16(TC_M, TC_D, 1);
      // Descriptors are made once: the issuing thread is alone, and what it computes
      // between two products delays the next one.  A descriptor's low bits hold the
      // address in 16-byte units, so a step inside a tile is an addition.
      unsigned long long q_desc[2][TC_D / 16];
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int ks = 0; ks < TC_D / 16; ++ks)
          q_desc[x][ks] = desc_k_major(smem_u32(sQ + x * TILE_BYTES) + (ks >> 2) * HALF_BYTES + (ks & 3) * 32);
      unsigned long long k_desc[2], v_desc[2];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
        k_desc[st] = desc_k_major(smem_u32(sKV + st * 2 * TILE_BYTES));
        v_desc[st] = desc_mn_major(smem_u32(sKV + st * 2 * TILE_BYTES + TILE_BYTES), HALF_BYTES);
      }
      auto issue_s_to = [&](int x, int buf, int i) {     // scores of tile x, key tile i -> columns of buf
        const unsigned long long kd = k_desc[i & 1];
#pragma unroll
        for (int ks = 0; ks < TC_D / 16; ++ks)
          tc_mma(tmem + buf * 128, x ? q_desc[1][ks] : q_desc[0][ks],
                 kd + (unsigned long long)(((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4), idesc_s,
                 ks > 0 ? 1u : 0u);
        tc_commit(&s_full[buf]);
      };
      auto issue_s = [&](int x, int i) { issue_s_to(x, x, i); };
      int uses[2] = {0, 0};     // completed phases of p_full[x]
      int have_k = 0;           // keys of key tiles 0..have_k have been waited for
      int have_v = -1;          // values likewise
      ok = mbar_wait(&k_full[0], 0);
      if (ok) {
        tc_fence_after();
        if (active(0, 0)) issue_s(0, 0);
        if (active(1, 0)) issue_s(1, 0);
        tc_commit(&k_empty[0]);
      }
      const int paired_end = min(ntiles, solo_from);
      // Keys and values come by TMA and are read by the tensor core, both through the async
      // proxy: their barrier orders them and no tcgen05 fence follows it.  They have long
      // arrived as a rule, so they are looked at before the waits for the probabilities,
      // off the path from a tile's probabilities to its next scores.
      for (int i = 0; i < paired_end && ok; ++i) {
        if (have_v < i) {
          ok = mbar_wait(&v_full[i & 1], (i >> 1) & 1);
          have_v = i;
        }
        if (ok && i + 1 < ntiles && have_k < i + 1) {
          ok = mbar_wait(&k_full[(i + 1) & 1], ((i + 1) >> 1) & 1);
          have_k = i + 1;
        }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!ok) break;
          if (active(x, i)) {
            ok = mbar_wait(&p_full[x], uses[x] & 1);
            if (!ok) break;
            ++uses[x];
            tc_fence_after();
            const unsigned long long vd = v_desc[i & 1];
            const bool first = j0 + i == jf[x];
#pragma unroll
            for (int ks = 0; ks < TC_N / 16; ++ks)
              tc_mma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8,
                        vd + (unsigned long long)((ks * 16 * 128) >> 4), idesc_o,
                        (!first || ks > 0) ? 1u : 0u);
            if (j0 + i == jl[x]) tc_commit(&o_final[x]);
          }
          if (x == 1) tc_commit(&v_empty[i & 1]);   // both output products of key tile i have been issued
          if (i + 1 < ntiles && active(x, i + 1)) issue_s(x, i + 1);
          if (x == 1 && i + 1 < ntiles) tc_commit(&k_empty[(i + 1) & 1]);   // both score products of key tile i+1
        }
      }
      // ---- one tile alone: its scores of key tile i are in buffer (i - solo_from) & 1
      // (0: its own columns, 1: the finished tile's); those of i + 1 go to the other one
      // before this loop waits for the probabilities of i.
      for (int i = solo_from; i < ntiles && ok; ++i) {
        const int x = solo_x;
        const int buf = ((i - solo_from) & 1) ? 1 - x : x;
        if (i + 1 < ntiles) {
          if (have_k < i + 1) {
            ok = mbar_wait(&k_full[(i + 1) & 1], ((i + 1) >> 1) & 1);
            if (!ok) break;
            have_k = i + 1;
          }
          issue_s_to(x, 1 - buf, i + 1);
          tc_commit(&k_empty[(i + 1) & 1]);
        }
        if (have_v < i) {
          ok = mbar_wait(&v_full[i & 1], (i >> 1) & 1);
          if (!ok) break;
          have_v = i;
        }
        ok = mbar_wait(&p_full[buf], uses[buf] & 1);
        if (!ok) break;
        ++uses[buf];
        tc_fence_after();
        const unsigned long long vd = v_desc[i & 1];
        const bool first = j0 + i == jf[x];
#pragma unroll
        for (int ks = 0; ks < TC_N / 16; ++ks)
          tc_mma_ts(tmem + 256 + x * 128, tmem + buf * 128 + ks * 8,
                    vd + (unsigned long long)((ks * 16 * 128) >> 4), idesc_o,
                    (!first || ks > 0) ? 1u : 0u);
        tc_commit(&v_empty[i & 1]);
        tc_commit(pv_done);
        if (i == ntiles - 1) tc_commit(&o_final[x]);
      }
    }
  }
  } else {
    regs_take<PAIR_REGS_MANY>();
    // ---- softmax: thread r of group x owns row r of tile x
    const int x = threadIdx.x >> 7, r = threadIdx.x & 127;
    const int tl = r / G, g = r % G;
    const bool valid = tl < ntok[x];
    const int hi = valid ? prefix + tokx[x] + tl : -1;
    const int lo = (valid && window > 0 && hi - window + 1 > 0) ? hi - window + 1 : 0;
    const float scale_log2 = scale * LOG2E;
    const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    const unsigned tmem_o = tmem + lane_base + 256 + x * 128;
    float m_ref = NEG_BIG, l = 0.f;
    // completed phases of s_full[own columns] and s_full[the other tile's]: the latter has
    // served the other tile's key tiles before this one borrows it
    int uses_own = 0, uses_other = n_other;
    const int my_solo = x == solo_x ? solo_from : 0x7fffffff;
    for (int i = 0; i < ntiles && ok; ++i) {
      if (!active(x, i)) continue;
      const bool borrowed = i >= my_solo && ((i - my_solo) & 1);
      const int buf = borrowed ? 1 - x : x;
      const unsigned tmem_s = tmem + lane_base + buf * 128;
      ok = mbar_wait(&s_full[buf], (borrowed ? uses_other : uses_own) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (borrowed) ++uses_other; else ++uses_own;
      tc_fence_after();
      const int kbase = (j0 + i) * TC_N;
      const bool full = kbase >= lo && kbase + TC_N - 1 <= hi;   // no key of the tile is masked
      unsigned v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld32(tmem_s + c * 32, v[c]);
      tc_wait_ld();
      // Four independent chains for the maximum and for the sum (a thread has few warps
      // beside it to hide the latency of one long chain).  Tiles without a masked key,
      // nearly all of them, take a path without the per-key tests.
      float m4[4] = {NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG};
      if (!full) {
        // keys outside [lo, hi] get the score NEG_BIG: one subtraction and one unsigned
        // comparison each; their exponentials below are exactly zero
        const int a = lo - kbase, b = hi - kbase;
        const int first_vis = b >= a ? a : (1 << 20);
        const unsigned span = b >= a ? (unsigned)(b - a) : 0u;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if ((unsigned)(c * 32 + k - first_vis) > span) v[c][k] = __float_as_uint(NEG_BIG);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < 32; k += 8)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            m4[j] = max3(m4[j], __uint_as_float(v[c][k + 2 * j]), __uint_as_float(v[c][k + 2 * j + 1]));
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      mx = mx <= -1e29f ? NEG_BIG : mx * scale_log2;   // scale is positive
      // the reference maximum rises only when it must (or at the first visible key)
      float factor = 1.0f;
      bool rescale = false;
      if (mx > m_ref + 8.0f) {
        rescale = m_ref > -1e29f;
        factor = rescale ? fast_exp2(m_ref - mx) : 0.f;
        m_ref = mx;
        l *= factor;
      }
      const float m_use = m_ref <= -1e29f ? 0.f : m_ref;
      // Two keys in eight (positions 6 and 7 mod 8) take their exponentials on the FMA pipe,
      // the others on the special-function unit: about what keeps both pipes equally busy.
      // Scaling, the polynomial and the sums use the packed float32 instructions (two values
      // an instruction, each rounded as by the single one): a warp alone on its scheduler is
      // bound by the instructions it can issue.  Eight chains of sums: chain j takes the keys
      // at positions j mod 8.
      float2 s8[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      if (full) {
        const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_use, -m_use);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int k = 0; k < 32; k += 8) {
            float2 p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              p[j] = __ffma2_rn(make_float2(__uint_as_float(v[c][k + 2 * j]), __uint_as_float(v[c][k + 2 * j + 1])),
                                sc2, nm2);
#pragma unroll
            for (int j = 0; j < 3; ++j) p[j] = make_float2(fast_exp2(p[j].x), fast_exp2(p[j].y));
            p[3] = exp2_fma2(p[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              s8[j] = __fadd2_rn(s8[j], p[j]);
              v[c >> 1][(c & 1) * 16 + (k >> 1) + j] = pack_bf16(p[j].x, p[j].y);   // 64 packed pairs in v[0], v[1]
            }
          }
      } else {
        // a tile with masked keys: every exponential on the special-function unit, whose
        // result for a masked score (NEG_BIG) is exactly zero
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            float pj[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              pj[j] = fast_exp2(fmaf(__uint_as_float(v[c][k + j]), scale_log2, -m_use));
            s8[(k >> 1) & 2] = __fadd2_rn(s8[(k >> 1) & 2], make_float2(pj[0], pj[1]));
            s8[((k >> 1) & 2) + 1] = __fadd2_rn(s8[((k >> 1) & 2) + 1], make_float2(pj[2], pj[3]));
            v[c >> 1][(c & 1) * 16 + (k >> 1)] = pack_bf16(pj[0], pj[1]);
            v[c >> 1][(c & 1) * 16 + (k >> 1) + 1] = pack_bf16(pj[2], pj[3]);
          }
      }
      const float sum = ((s8[0].x + s8[0].y) + (s8[1].x + s8[1].y)) + ((s8[2].x + s8[2].y) + (s8[3].x + s8[3].y));
      l += sum;
      // O of this tile is rescaled when a row of the warp raised its reference.  Its last
      // product completed before these scores did, except where the tile runs alone: there
      // the scores of key tile i were issued before the product of i - 1, which is waited
      // for here (phase i - 1 - my_solo of pv_done; that of i - 2 completed before the scores).
      if (__any_sync(0xffffffffu, rescale)) {
        if (i > my_solo) {
          ok = mbar_wait(pv_done, (i - 1 - my_solo) & 1);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tc_ld32(tmem_o + c * 32, v[2]);
          tc_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k)
            v[2][k] = __float_as_uint(__uint_as_float(v[2][k]) * (rescale ? factor : 1.0f));
          tc_st32(tmem_o + c * 32, v[2]);
        }
      }
      tc_st32(tmem_s, v[0]);          // probabilities over the scores they came from
      tc_st32(tmem_s + 32, v[1]);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[buf]);
    }
    if (ok && jl[x] >= jf[x]) {
      ok = mbar_wait(&o_final[x], 0);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      if (ok && !whole[x]) {
        // a partial result of this chunk: O as accumulated (against m_ref), m_ref, l
        const size_t t = (size_t)(q_begin + tokx[x] + tl);
        const size_t row = (t * Hq + (size_t)kvh * G + g) * max_chunks + chunk;
        float* dst = part_o + row * TC_D;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          unsigned o[32];
          tc_ld32(tmem_o + c * 32, o);
          tc_wait_ld();
          if (valid) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              *reinterpret_cast<uint4*>(dst + c * 32 + ch * 4) =
                  make_uint4(o[ch * 4], o[ch * 4 + 1], o[ch * 4 + 2], o[ch * 4 + 3]);
          }
        }
        if (valid) *reinterpret_cast<float2*>(part_ml + row * 2) = make_float2(m_ref, l);
      } else if (ok) {
        const float inv = 1.0f / l;
        const size_t t = (size_t)(q_begin + tokx[x] + tl);
        __nv_bfloat16* dst = out + (t * Hq + (size_t)kvh * G + g) * TC_D;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          unsigned o[32];
          tc_ld32(tmem_o + c * 32, o);
          tc_wait_ld();
          if (valid) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint4 o4;
              o4.x = pack_bf16(__uint_as_float(o[ch * 8 + 0]) * inv, __uint_as_float(o[ch * 8 + 1]) * inv);
              o4.y = pack_bf16(__uint_as_float(o[ch * 8 + 2]) * inv, __uint_as_float(o[ch * 8 + 3]) * inv);
              o4.z = pack_bf16(__uint_as_float(o[ch * 8 + 4]) * inv, __uint_as_float(o[ch * 8 + 5]) * inv);
              o4.w = pack_bf16(__uint_as_float(o[ch * 8 + 6]) * inv, __uint_as_float(o[ch * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + ch * 8) = o4;
            }
          }
        }
      }
    }
  }
  if (!ok) atomicExch(&dib_attention_error_word, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
}

// Rows whose key range spans several chunks: out = sum_c O_c 2^(m_c - M) / sum_c l_c
// 2^(m_c - M) over the chunks of the row's query tile, in chunk order.  A warp takes a
// token (a lane four dimensions) and walks its query heads; tokens that the attention
// kernel finished itself cost one look at their lengths.
constexpr int MERGE_MAX = 16;     // chunks of one row
__global__ void __launch_bounds__(256)
extend_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                              __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q_lens,
                              const int* __restrict__ seq_lens, const int* __restrict__ token_seq,
                              int t_first, int num_tokens, int Hq, int Hkv, int max_chunks,
                              int chunk_tiles, int window) {
  pdl_prologue(part_o, part_ml);
  const int lane = threadIdx.x & 31;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= num_tokens) return;
  const int t = t_first + idx;
  const int seq = token_seq[t];
  const int q_begin = cu_q_lens[seq];
  const int q_len = cu_q_lens[seq + 1] - q_begin;
  const int prefix = seq_lens[seq] - q_len;
  const int npt = TC_M / (Hq / Hkv);
  const int tile_tok0 = (t - q_begin) / npt * npt;
  const int first_pos = prefix + tile_tok0;
  const int last_pos = first_pos + min(npt, q_len - tile_tok0) - 1;
  const int first_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
  const int c0 = first_key / TC_N / chunk_tiles, c1 = last_pos / TC_N / chunk_tiles;
  if (c0 == c1) return;     // finished by the attention kernel itself
  // Lane j first works out head j's (and j+32's, ...) weights of the chunks, all heads'
  // loads in flight together; then the warp walks the heads, four at a time, with the
  // weights handed round by shuffles.
  for (int h0 = 0; h0 < Hq; h0 += 32) {
    const int hl = h0 + lane;
    float w[MERGE_MAX], inv = 0.f;     // at most MERGE_MAX chunks of a row are merged here (see the launcher)
    {
      float m[MERGE_MAX], l[MERGE_MAX], M = NEG_BIG, L = 0.f;
#pragma unroll
      for (int c = 0; c < MERGE_MAX; ++c) {
        m[c] = NEG_BIG;
        l[c] = 0.f;
        if (hl < Hq && c0 + c <= c1) {
          const float2 ml = *reinterpret_cast<const float2*>(
              part_ml + (((size_t)t * Hq + hl) * max_chunks + c0 + c) * 2);
          m[c] = ml.x;
          l[c] = ml.y;
        }
        M = fmaxf(M, m[c]);
      }
#pragma unroll
      for (int c = 0; c < MERGE_MAX; ++c) {
        w[c] = m[c] <= -1e29f ? 0.f : fast_exp2(m[c] - M);
        L += l[c] * w[c];
      }
      inv = 1.0f / L;
    }
    const int nh = min(32, Hq - h0);
    for (int hb = 0; hb < nh; hb += 4) {
      float4 acc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < MERGE_MAX; ++c) {
        if (c0 + c > c1) break;     // uniform
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int src = min(hb + j, nh - 1);
          const float f = __shfl_sync(0xffffffffu, w[c], src);
          if (hb + j < nh) {
            const float4 o = *reinterpret_cast<const float4*>(
                part_o + (((size_t)t * Hq + h0 + hb + j) * max_chunks + c0 + c) * TC_D + lane * 4);
            acc[j].x += o.x * f;
            acc[j].y += o.y * f;
            acc[j].z += o.z * f;
            acc[j].w += o.w * f;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float iv = __shfl_sync(0xffffffffu, inv, min(hb + j, nh - 1));
        if (hb + j < nh) {
          uint2 packed;
          packed.x = pack_bf16(acc[j].x * iv, acc[j].y * iv);
          packed.y = pack_bf16(acc[j].z * iv, acc[j].w * iv);
          *reinterpret_cast<uint2*>(out + ((size_t)t * Hq + h0 + hb + j) * TC_D + lane * 4) = packed;
        }
      }
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

}  // namespace

extern "C" {

int dib_attention_prefill_tc_tile_rows() { return TC_M; }

int dib_attention_prefill_tc_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, dib_attention_error_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
int dib_attention_prefill_tc_status_clear() {
  const int v = 0;
  return cudaMemcpyToSymbol(dib_attention_error_word, &v, sizeof(int)) == cudaSuccess ? 0 : -1;
}

// Sequences with more than one new token; tiles name (sequence, first token of the
// tile among its new tokens) with 128 / (Hq/Hkv) tokens per tile.  Returns -2 for
// shapes this kernel does not take (the caller then uses the mma.sync kernel).
int dib_extend_attention_tc(const void* q, void* out, const void* cache, long long num_pages,
                            const int* block_table, int max_blocks, const int* cu_q_lens,
                            const int* seq_lens, const int* tile_seq, const int* tile_start,
                            int num_tiles, int Hq, int Hkv, int D, int page_size, float scale,
                            int window, cudaStream_t st) {
  if (num_tiles == 0) return DIB_OK;
  if (D != TC_D || Hkv < 1 || Hq % Hkv != 0 || TC_M % (Hq / Hkv) != 0 || page_size < 8 ||
      page_size > TC_N || TC_N % page_size != 0 || num_tiles > 65535 ||
      (long long)num_pages * 2 * Hkv * page_size >= (1ll << 31) ||
      reinterpret_cast<uintptr_t>(cache) % 16 != 0 || reinterpret_cast<uintptr_t>(q) % 16 != 0)
    return DIB_BAD_SIZE;
  const CUtensorMap* map = cache_map(cache, num_pages, Hkv, page_size, D);
  if (map == nullptr) return DIB_LAUNCH_FAILED;
  const size_t smem = 6 * TILE_BYTES + 10 * 8 + 16 + 1024;
  static DeviceOnce attr_set;
  if (!attr_set.done()) {
    if (cudaFuncSetAttribute(extend_attention_tc_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  dib_launch(extend_attention_tc_kernel, dim3(Hkv, num_tiles), dim3(TC_THREADS), smem, st, *map,
             (const __nv_bfloat16*)q, (__nv_bfloat16*)out, block_table, max_blocks, cu_q_lens,
             seq_lens, tile_seq, tile_start, Hq, Hkv, page_size, scale, window);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The same with two query tiles of one sequence per CTA: a list entry names the sequence
// and the first tokens of tile A and of tile B (128 / (Hq/Hkv) tokens each; -1: no B).  The
// two share the key tiles that both need; the caller pairs a tile early in a prompt with
// one late in it, so that every CTA has about the same number of key tiles.
// chunk_tiles > 0: the key range is cut into chunks of that many tiles of 128 keys and a
// list entry names (sequence, first token, chunk tile_chunk[i] < max_chunks): several CTAs
// share a pair of query tiles (the caller lists every chunk a pair may need, longest
// first); part_o (float32 [T, Hq, max_chunks, 128])
// and part_ml ([T, Hq, max_chunks, 2]) take the partial results, which a second kernel
// merges for the tokens t_first .. t_first + num_tokens - 1 (the step's prompt tokens;
// token_seq names their sequences).
int dib_extend_attention_tc_pair(const void* q, void* out, const void* cache, long long num_pages,
                                 const int* block_table, int max_blocks, const int* cu_q_lens,
                                 const int* seq_lens, const int* tile_seq, const int* tile_start,
                                 const int* tile_start_b, int num_tiles, int Hq, int Hkv, int D,
                                 int page_size, float scale, int window, int chunk_tiles, const int* tile_chunk, int max_chunks,
                                 float* part_o, float* part_ml, const int* token_seq, int t_first,
                                 int num_tokens, cudaStream_t st) {
  if (num_tiles == 0) return DIB_OK;
  if (D != TC_D || Hkv < 1 || Hq % Hkv != 0 || TC_M % (Hq / Hkv) != 0 || page_size < 8 ||
      page_size > TC_N || TC_N % page_size != 0 || num_tiles > 65535 ||
      (long long)num_pages * 2 * Hkv * page_size >= (1ll << 31) ||
      reinterpret_cast<uintptr_t>(cache) % 16 != 0 || reinterpret_cast<uintptr_t>(q) % 16 != 0)
    return DIB_BAD_SIZE;
  const CUtensorMap* map = cache_map(cache, num_pages, Hkv, page_size, D);
  if (map == nullptr) return DIB_LAUNCH_FAILED;
  const size_t smem = 6 * TILE_BYTES + 15 * 8 + 16 + 1024;
  static DeviceOnce attr_set;
  if (!attr_set.done()) {
    if (cudaFuncSetAttribute(extend_attention_tc_pair_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  if (chunk_tiles <= 0) {
    chunk_tiles = 0;
    max_chunks = 1;
  } else if (max_chunks < 1 || max_chunks > MERGE_MAX || tile_chunk == nullptr || part_o == nullptr || part_ml == nullptr ||
             token_seq == nullptr || num_tokens < 1) {
    return DIB_BAD_SIZE;
  }
  dib_launch(extend_attention_tc_pair_kernel, dim3(Hkv, num_tiles), dim3(PAIR_THREADS), smem, st, *map,
             (const __nv_bfloat16*)q, (__nv_bfloat16*)out, block_table, max_blocks, cu_q_lens, seq_lens,
             tile_seq, tile_start, tile_start_b, Hq, Hkv, page_size, scale, window, chunk_tiles,
             tile_chunk, max_chunks, part_o, part_ml);
  DIB_CHECK_LAUNCH();
  if (chunk_tiles > 0 && max_chunks > 1) {
    dib_launch(extend_attention_merge_kernel, dim3((num_tokens + 7) / 8), dim3(256), 0, st,
               (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, cu_q_lens, seq_lens,
               token_seq, t_first, num_tokens, Hq, Hkv, max_chunks, chunk_tiles, window);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // extern "C"
