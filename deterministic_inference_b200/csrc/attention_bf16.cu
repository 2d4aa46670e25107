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

// A named barrier over one group of 128 threads (id 0 with 128 threads is the whole
// CTA of the one-split kernel).
__device__ __forceinline__ void group_sync(int id) {
  asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Orders this thread's generic-proxy accesses to shared memory before later writes of
// the async proxy (a bulk tensor copy into the same bytes).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// A bounded wait that, once one wait of this thread has run out, waits no more: the
// launch is reported as failed (the error word keeps the first `where`), and its
// remaining work only has to end.
__device__ __forceinline__ void mbar_wait_once(unsigned long long* bar, unsigned parity, bool& dead,
                                               int where) {
  if (dead) return;
  if (!mbar_wait(bar, parity)) {
    dead = true;
    atomicCAS(&dib_attention_error_word, 0, where);
  }
}
// A barrier over a group of 128 threads that also tells every thread whether any of
// them has given up, so that the group leaves together.
__device__ __forceinline__ bool group_sync_any(int id, bool flag) {
  unsigned out;
  asm volatile(
      "{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.or.pred p, %2, 128, q; selp.u32 %0, 1, 0, p; }"
      : "=r"(out)
      : "r"((unsigned)flag), "r"(id)
      : "memory");
  return out != 0;
}

constexpr int Q_ROW_PAD = 8;            // elements between query rows in shared memory (16 bytes)
constexpr int P_STRIDE = DEC_SPLIT + 8;  // elements per row of the probability tile (272 bytes)
// a group's exchange area: probabilities [16][P_STRIDE] bf16, then row maxima and row
// sums of the four warps [2][4][16] float
constexpr int EXCH_BYTES = 16 * P_STRIDE * 2 + 2 * 4 * 16 * 4;

// One split of one (sequence, kv head): the 128 keys k0 .. k0+127 against the G query
// heads of the group, by 128 threads (tid 0..127), from the swizzled tiles sK / sV
// whose copies complete on bar_k / bar_v.  Writes the split's partial output and
// log-sum-exp.  The arithmetic depends on nothing but the split itself, so both
// kernels below give the same bits for it.
//
// Each warp scores 32 keys; the row maxima go through shared memory, so every warp
// exponentiates against the split's maximum; the probabilities (bfloat16, as the
// tensor cores take them) go through shared memory too, and each warp multiplies all
// 128 of them with its own quarter of the value columns, so the outputs need no merge:
// they leave from registers.
//
// sQ: the group's query rows in shared memory (row stride D + Q_ROW_PAD; they arrive
// with the keys), or nullptr to read them from q.  exch: EXCH_BYTES of this group's own.
// PIPE: each warp hands the K tile back (rel_k) after its scores and the V tile
// (rel_v) after its products; both barriers count the four warps.
template <int D, bool PIPE>
__device__ __forceinline__ void decode_split_compute(
    __nv_bfloat16* sK, __nv_bfloat16* sV, const __nv_bfloat16* sQ, unsigned char* exch,
    unsigned long long* bar_k, unsigned parity_k, unsigned long long* bar_v, unsigned parity_v,
    unsigned long long* rel_k, unsigned long long* rel_v, int tid, int bar_id, bool& dead,
    const __nv_bfloat16* __restrict__ q, int b, int kvh, int split, int kv_len,
    float* __restrict__ part_o, float* __restrict__ part_lse, int max_splits, int Hq, int Hkv,
    float scale, int window) {
  constexpr int WCOLS = D / 4;    // value columns of one warp
  const int G = Hq / Hkv;
  const int k0 = split * DEC_SPLIT;
  const int warp = tid >> 5, lane = tid & 31;
  const int pos = kv_len - 1;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int nvalid = min(DEC_SPLIT, kv_len - k0);
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(exch);
  float* sM = reinterpret_cast<float*>(exch + 16 * P_STRIDE * 2);   // [4][16]
  float* sL = sM + 4 * 16;

  unsigned qf[D / 16][4];
  const int r0 = lane >> 2, c0 = (lane & 3) * 2;
  if (sQ == nullptr) {
    const __nv_bfloat16* qb = q + ((size_t)b * Hq + (size_t)kvh * G) * D;
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
  const int krow0 = warp * DEC_WARP_KEYS;
  const int m = lane >> 3, r = lane & 7;

  // ---- scores of this warp's 32 keys
  mbar_wait_once(bar_k, parity_k, dead, 1);
  if (sQ != nullptr) {
    constexpr int QS = D + Q_ROW_PAD;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d = ks * 16 + c0;
      qf[ks][0] = r0 < G ? *reinterpret_cast<const unsigned*>(sQ + r0 * QS + d) : 0u;
      qf[ks][1] = r0 + 8 < G ? *reinterpret_cast<const unsigned*>(sQ + (r0 + 8) * QS + d) : 0u;
      qf[ks][2] = r0 < G ? *reinterpret_cast<const unsigned*>(sQ + r0 * QS + d + 8) : 0u;
      qf[ks][3] = r0 + 8 < G ? *reinterpret_cast<const unsigned*>(sQ + (r0 + 8) * QS + d + 8) : 0u;
    }
  }
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
  if (PIPE) {   // this warp has read its keys (and the query rows)
    __syncwarp();
    if (lane == 0) mbar_arrive(rel_k);
  }

  // ---- mask (keys outside [first_key, pos] whatever the tile holds there), scale, and
  // the maximum of each row over the split
  const float scale_log2 = scale * LOG2E;
  float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
  for (int nt = 0; nt < DEC_WARP_KEYS / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = k0 + krow0 + nt * 8 + c0 + (i & 1);
      const bool vis = key >= first_key && key <= pos;
      s[nt][i] = vis ? s[nt][i] * scale_log2 : NEG_BIG;
      mx[i >> 1] = fmaxf(mx[i >> 1], s[nt][i]);
    }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
    mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
    if ((lane & 3) == 0 && r0 + rr * 8 < G) sM[warp * 16 + r0 + rr * 8] = mx[rr];
  }
  group_sync(bar_id);
  float M[2], msafe[2], sum[2] = {0.f, 0.f};
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = r0 + rr * 8;
    M[rr] = NEG_BIG;
    if (row < G) {
#pragma unroll
      for (int w = 0; w < 4; ++w) M[rr] = fmaxf(M[rr], sM[w * 16 + row]);
    }
    msafe[rr] = M[rr] <= -1e29f ? 0.f : M[rr];   // nothing visible: the exponentials become 0
  }
#pragma unroll
  for (int nt = 0; nt < DEC_WARP_KEYS / 8; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[nt][i] = fast_exp2(s[nt][i] - msafe[i >> 1]);
      sum[i >> 1] += s[nt][i];
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
      if (r0 + rr * 8 < G)
        *reinterpret_cast<unsigned*>(sP + (r0 + rr * 8) * P_STRIDE + krow0 + nt * 8 + c0) =
            pack_bf16(s[nt][rr * 2], s[nt][rr * 2 + 1]);
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 1);
    sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 2);
    if ((lane & 3) == 0 && r0 + rr * 8 < G) sL[warp * 16 + r0 + rr * 8] = sum[rr];
  }

  // ---- values; rows beyond the sequence are zeroed first (their probability is 0,
  // but 0 * garbage must stay 0)
  mbar_wait_once(bar_v, parity_v, dead, 2);
  if (nvalid < DEC_SPLIT && tid >= nvalid) {
#pragma unroll
    for (int c = 0; c < D / 8; ++c)
      *reinterpret_cast<uint4*>(sV + sw_off(tid, c * 8)) = make_uint4(0, 0, 0, 0);
  }
  dead = group_sync_any(bar_id, dead);   // probabilities, sums and zeroed rows are in place
  if (dead) return;   // a wait ran out somewhere in the group: nothing of this split is written

  // ---- O[16 x WCOLS] = P[16 x 128] V[128 x this warp's columns]; rows >= G of P are
  // never written and what they give is never read
  float o[WCOLS / 8][4];
#pragma unroll
  for (int nt = 0; nt < WCOLS / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nt][i] = 0.f;
#pragma unroll
  for (int kk = 0; kk < DEC_SPLIT / 16; ++kk) {
    unsigned a[4];
    ldmatrix_x4(a, sP + ((m & 1) * 8 + r) * P_STRIDE + kk * 16 + (m >> 1) * 8);
#pragma unroll
    for (int dp = 0; dp < WCOLS / 16; ++dp) {
      unsigned bf[4];
      ldmatrix_x4_trans(bf, sV + sw_off(kk * 16 + (m & 1) * 8 + r, warp * WCOLS + dp * 16 + (m >> 1) * 8));
      mma_16816(o[dp * 2], a, bf[0], bf[1]);
      mma_16816(o[dp * 2 + 1], a, bf[2], bf[3]);
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = r0 + rr * 8;
    if (row < G) {
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) L += sL[w * 16 + row];
      const float inv = 1.0f / L;
      const size_t prow = ((size_t)b * Hq + (size_t)kvh * G + row) * max_splits + split;
      float* dst = part_o + prow * D + warp * WCOLS + c0;
#pragma unroll
      for (int nt = 0; nt < WCOLS / 8; ++nt)
        *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][rr * 2] * inv, o[nt][rr * 2 + 1] * inv);
      if (warp == 0 && (lane & 3) == 0) part_lse[prow] = (M[rr] + log2f(L)) / LOG2E;
    }
  }
  if (PIPE) {
    // rows of the V tile may have been zeroed: order that before the producer's next
    // copy into it, then hand it back
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(rel_v);
  }
}

// ---- one split per CTA: grid (kv heads, sequences, splits)
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
  if (threadIdx.x == 0) prefetch_tensormap(&map);
  constexpr int HALVES = D / 64;
  constexpr int TILE = DEC_SPLIT * D;   // elements of the K (or V) tile
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sV = sK + TILE;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + (size_t)2 * TILE * 2);
  unsigned char* exch = reinterpret_cast<unsigned char*>(bars + 2);

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int k0 = split * DEC_SPLIT;
  const int* bt = block_table + (size_t)b * max_blocks;
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
  pdl_wait(q);
  if (issuer && !early) tma_load_2d(dst, &map, half * 64, row0, &bars[kv]);

  bool dead = false;
  decode_split_compute<D, false>(sK, sV, nullptr, exch, &bars[0], 0, &bars[1], 0, nullptr, nullptr,
                                 threadIdx.x, 0, dead, q, b, kvh, split, kv_len, part_o, part_lse,
                                 max_splits, Hq, Hkv, scale, window);
}

// ---- many splits per CTA, pipelined.  One CTA per SM walks the step's splits
// (flattened (sequence, split, kv head), every gridDim.x-th one).  A producer warp
// finds the splits, and keeps the key tiles, the value tiles and the query rows of
// the next ones in flight (a ring of STAGES key buffers and one of value buffers, each
// handed back as soon as its readers have done with it); GROUPS groups of four warps
// take the splits in turn.  So neither the length / block-table / query round-trips
// nor the arithmetic of a split stand between two copies.  Each split is computed
// exactly as by the kernel above.
struct DecodeItem { int b, kvh, split, kv_len; };
constexpr int gcd_c(int a, int b) { return b == 0 ? a : gcd_c(b, a % b); }

// The next split at or after flat index idx that belongs to this CTA and lies inside
// its sequence's visible range; false when there is none.  idx is left on the item.
__device__ __forceinline__ bool decode_next_item(unsigned& idx, unsigned total, unsigned max_splits,
                                                 unsigned Hkv, int window,
                                                 const int* __restrict__ seq_lens, DecodeItem& it) {
  const unsigned grid = gridDim.x, bid = blockIdx.x;
  while (idx < total) {
    const unsigned t = idx / Hkv;
    const unsigned b = t / max_splits, split = t % max_splits;
    const int kv_len = seq_lens[b];
    const int pos = kv_len - 1;
    const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int s0 = first_key / DEC_SPLIT, s1 = pos / DEC_SPLIT;
    unsigned base;
    if (kv_len <= 0 || (int)split > s1) base = (b + 1) * max_splits * Hkv;      // next sequence
    else if ((int)split < s0) base = (b * max_splits + (unsigned)s0) * Hkv;     // the window's first split
    else {
      it.b = (int)b; it.kvh = (int)(idx % Hkv); it.split = (int)split; it.kv_len = kv_len;
      return true;
    }
    idx = base + (bid + grid - base % grid) % grid;   // this CTA's first index >= base
  }
  return false;
}

template <int D, int KS, int VS, int GROUPS>
__global__ void __launch_bounds__(GROUPS * DEC_THREADS + 64, 1)
decode_attention_stage1_pipe_kernel(const __grid_constant__ CUtensorMap map,
                                    const __nv_bfloat16* __restrict__ q,
                                    const int* __restrict__ block_table, int max_blocks,
                                    const int* __restrict__ seq_lens, float* __restrict__ part_o,
                                    float* __restrict__ part_lse, int num_seqs, int max_splits,
                                    int Hq, int Hkv, int page_size, float scale, int window) {
  pdl_trigger();
  if (threadIdx.x == 0) prefetch_tensormap(&map);
  constexpr int HALVES = D / 64;
  constexpr int TILE = DEC_SPLIT * D;
  constexpr int QS = D + Q_ROW_PAD;
  const int G = Hq / Hkv;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* k_tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [KS][TILE]
  __nv_bfloat16* v_tiles = k_tiles + (size_t)KS * TILE;                     // [VS][TILE]
  __nv_bfloat16* q_rows = v_tiles + (size_t)VS * TILE;                      // [KS][G][QS]
  unsigned char* tail = reinterpret_cast<unsigned char*>(q_rows + (size_t)KS * G * QS);
  tail = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tail) + 15) & ~(uintptr_t)15);
  // "full" barriers exist once per (tile of the ring, consumer group): a wait names a
  // phase by its parity alone, so a barrier must have one waiter that takes its phases
  // in order; a tile that serves the groups in turn has one barrier for each.
  unsigned long long* full_k = reinterpret_cast<unsigned long long*>(tail);   // [KS][GROUPS]
  unsigned long long* empty_k = full_k + KS * GROUPS;                         // [KS]
  unsigned long long* full_v = empty_k + KS;                                  // [VS][GROUPS]
  unsigned long long* empty_v = full_v + VS * GROUPS;                         // [VS]
  DecodeItem* info = reinterpret_cast<DecodeItem*>(empty_v + VS);           // [KS]
  unsigned char* exch = reinterpret_cast<unsigned char*>(info + KS);        // [GROUPS][EXCH_BYTES]
  if (threadIdx.x == 0) {
    for (int i = 0; i < KS * GROUPS; ++i) mbar_init(&full_k[i], 1);
    for (int i = 0; i < VS * GROUPS; ++i) mbar_init(&full_v[i], 1);
    for (int i = 0; i < KS; ++i) mbar_init(&empty_k[i], 4);
    for (int i = 0; i < VS; ++i) mbar_init(&empty_v[i], 4);
    mbar_fence_init();
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bool dead = false;

  if (warp >= GROUPS * 4) {
    // ---------------- two producer warps, one for the ring of key tiles (with the
    // query rows and the item itself), one for the ring of value tiles; each walks the
    // same list of splits.  Lane c issues the copy of (page c / HALVES, 64-column half
    // c % HALVES); lanes 0..G-1 of the key warp the query rows.
    // part 0: the byte count and the pages that lie wholly before the new token;
    // part 1: the page that holds the new token (written by the kernel before this
    // one); part 2: everything, with the query rows.  The first splits' query rows are
    // read from global memory by the consumers instead: a copy of them would queue
    // behind all the tiles sent before it.
    const bool is_k = warp == GROUPS * 4;
    const int ring = is_k ? KS : VS;
    unsigned long long* full = is_k ? full_k : full_v;
    unsigned long long* empty = is_k ? empty_k : empty_v;
    __nv_bfloat16* tiles = is_k ? k_tiles : v_tiles;
    const unsigned total = (unsigned)num_seqs * max_splits * Hkv;
    const int copies = (DEC_SPLIT / page_size) * HALVES;   // at most 32 (page size 8, head size 128)
    const int pi = lane / HALVES, half = lane % HALVES;
    auto page_of = [&](const DecodeItem& it) {
      const int e = it.split * DEC_SPLIT / page_size + pi;
      return (lane < copies && e < max_blocks) ? block_table[(size_t)it.b * max_blocks + e] : 0;
    };
    auto send = [&](int n, const DecodeItem& it, int page, int part) {
      const int stage = n % ring;
      unsigned long long* full_bar = &full[stage * GROUPS + (n % GROUPS)];
      const int k0 = it.split * DEC_SPLIT;
      const int pos = it.kv_len - 1;
      const int valid_pages = (min(DEC_SPLIT, it.kv_len - k0) + page_size - 1) / page_size;
      const bool issuer = lane < copies && pi < valid_pages;
      const bool early = k0 / page_size + pi < pos / page_size;
      const bool mine = issuer && (part == 2 || (part == 0) == early);
      const unsigned tile_bytes = (unsigned)valid_pages * page_size * D * 2;
      if (part == 2 && n >= ring) mbar_wait_once(&empty[stage], ((n / ring) - 1) & 1, dead, is_k ? 3 : 4);
      dead = __any_sync(0xffffffffu, dead);
      if (dead) return;
      if (part != 1) {
        if (lane == 0) {
          if (is_k) info[stage] = it;
          mbar_expect_tx(full_bar, tile_bytes + (is_k && part == 2 ? (unsigned)G * D * 2 : 0u));
        }
        __syncwarp();
      }
      if (mine)
        tma_load_2d(tiles + (size_t)stage * TILE + half * (DEC_SPLIT * 64) + pi * page_size * 64, &map,
                    half * 64, (((page * 2 + (is_k ? 0 : 1)) * Hkv) + it.kvh) * page_size, full_bar);
      if (is_k && part == 2 && lane < G)
        bulk_g2s(q_rows + ((size_t)stage * G + lane) * QS,
                 q + ((size_t)it.b * Hq + (size_t)it.kvh * G + lane) * D, D * 2, full_bar);
    };
    // the first splits (as many as the ring holds): what does not depend on the kernel
    // before this one goes out before the dependency wait, the rest after it
    constexpr int FIRST = KS > VS ? KS : VS;
    DecodeItem first_it[FIRST];
    int first_page[FIRST];
    unsigned idx = blockIdx.x;
    int n = 0;
#pragma unroll
    for (int j = 0; j < FIRST; ++j) {
      if (n == j && j < ring && decode_next_item(idx, total, max_splits, Hkv, window, seq_lens, first_it[j])) {
        first_page[j] = page_of(first_it[j]);
        ++n;
        idx += gridDim.x;
      }
    }
#pragma unroll
    for (int j = 0; j < FIRST; ++j)
      if (j < n) send(j, first_it[j], first_page[j], 0);
    pdl_wait(q);
#pragma unroll
    for (int j = 0; j < FIRST; ++j)
      if (j < n) send(j, first_it[j], first_page[j], 1);
    // the rest: the next split is found, and its block-table entry fetched, while the
    // current one's copies go out
    if (n == ring) {
      DecodeItem cur, nxt;
      bool has = decode_next_item(idx, total, max_splits, Hkv, window, seq_lens, cur);
      int page = has ? page_of(cur) : 0;
      while (has && !dead) {
        idx += gridDim.x;
        const bool has_next = decode_next_item(idx, total, max_splits, Hkv, window, seq_lens, nxt);
        const int page_next = has_next ? page_of(nxt) : 0;
        send(n, cur, page, 2);
        ++n;
        cur = nxt;
        page = page_next;
        has = has_next;
      }
    }
    // one end mark for each group, in the key ring
    for (int e = 0; is_k && e < GROUPS && !dead; ++e, ++n) {
      const int stage = n % KS;
      if (n >= KS) mbar_wait_once(&empty_k[stage], ((n / KS) - 1) & 1, dead, 5);
      dead = __any_sync(0xffffffffu, dead);
      if (dead) break;
      if (lane == 0) {
        info[stage].b = -1;
        mbar_arrive(&full_k[stage * GROUPS + (n % GROUPS)]);
      }
      __syncwarp();
    }
    return;
  }

  // ---------------- consumers: group g takes this CTA's splits g, g + GROUPS, ...
  const int g = warp >> 2, tid = threadIdx.x & (DEC_THREADS - 1);
  pdl_wait(q);   // transitively, everything this kernel writes over has been read
  for (int n = g;; n += GROUPS) {
    const int ks = n % KS, vs = n % VS;
    // this group's own count of uses of the tile: item m uses stage m % KS for group
    // m % GROUPS, so the pair (stage, group) comes again every lcm(KS, GROUPS) items
    constexpr int LCM_K = KS * GROUPS / gcd_c(KS, GROUPS), LCM_V = VS * GROUPS / gcd_c(VS, GROUPS);
    const unsigned par_k = (n / LCM_K) & 1;
    const unsigned par_v = (n / LCM_V) & 1;
    unsigned long long* fk = &full_k[ks * GROUPS + g];
    unsigned long long* fv = &full_v[vs * GROUPS + g];
    mbar_wait_once(fk, par_k, dead, 7);
    dead = group_sync_any(1 + g, dead);
    if (dead) break;
    const DecodeItem it = info[ks];
    if (it.b < 0) break;
    decode_split_compute<D, true>(k_tiles + (size_t)ks * TILE, v_tiles + (size_t)vs * TILE,
                                  n < KS ? nullptr : q_rows + (size_t)ks * G * QS,
                                  exch + (size_t)g * EXCH_BYTES,
                                  fk, par_k, fv, par_v, &empty_k[ks],
                                  &empty_v[vs], tid, 1 + g, dead, q, it.b,
                                  it.kvh, it.split, it.kv_len, part_o, part_lse, max_splits, Hq, Hkv,
                                  scale, window);
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

int sm_count_of_current_device() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
      sms = 0;
  }
  return sms;
}

// pipelined: 0 never, 1 always, 2 where it measured faster than one split per CTA: more
// than four splits per SM, sequences of eight splits (1,024 keys) or more, and groups
// of at most four query heads.
template <int D>
int launch_decode_tma(const void* q, void* out, const void* cache, long long num_pages,
                      const int* bt, int max_blocks, const int* seq_lens, float* part_o,
                      float* part_lse, int num_seqs, int max_splits, int Hq, int Hkv, int page_size,
                      float scale, int window, int pipelined, cudaStream_t st) {
  const CUtensorMap* map = cache_map(cache, num_pages, Hkv, page_size, D);
  if (map == nullptr) return DIB_LAUNCH_FAILED;
  const int sms = sm_count_of_current_device();
  const long long items = (long long)num_seqs * max_splits * Hkv;
  const int G = Hq / Hkv;
  if (sms > 0 && items < (1ll << 31) && (pipelined == 1 || (pipelined == 2 && items > 4ll * sms && max_splits >= 8 && G <= 4))) {
    constexpr int KS = D == 128 ? 3 : 6, VS = KS;   // tiles in the key ring and in the value ring
    constexpr int GROUPS = 2;
    const size_t smem = (size_t)(KS + VS) * DEC_SPLIT * D * 2 +                   // the two rings
                        (size_t)KS * G * (D + Q_ROW_PAD) * 2 + 16 +               // query rows
                        (size_t)(KS + VS) * 3 * 8 + KS * sizeof(DecodeItem) +     // barriers, items
                        (size_t)GROUPS * EXCH_BYTES + 1024;
    auto kern = decode_attention_stage1_pipe_kernel<D, KS, VS, GROUPS>;
    static size_t attr_smem = 0;   // grows with the group size (warm-up reaches it before any capture)
    if (smem > attr_smem) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess)
        return DIB_LAUNCH_FAILED;
      attr_smem = smem;
    }
    const int grid = (int)(items < sms ? items : sms);
    dib_launch(kern, dim3(grid), dim3(GROUPS * DEC_THREADS + 64), smem, st, *map,
               (const __nv_bfloat16*)q, bt, max_blocks, seq_lens, part_o, part_lse, num_seqs, max_splits,
               Hq, Hkv, page_size, scale, window);
    DIB_CHECK_LAUNCH();
  } else {
    const size_t smem = (size_t)2 * DEC_SPLIT * D * 2 + 16 + EXCH_BYTES + 1024;
    auto kern = decode_attention_stage1_tma_kernel<D>;
    static DeviceOnce attr_set;
    if (!attr_set.done()) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess)
        return DIB_LAUNCH_FAILED;
      attr_set.mark();
    }
    dib_launch(kern, dim3(Hkv, num_seqs, max_splits), dim3(DEC_THREADS), smem, st, *map,
               (const __nv_bfloat16*)q, bt, max_blocks, seq_lens, part_o, part_lse, max_splits, Hq, Hkv,
               page_size, scale, window);
    DIB_CHECK_LAUNCH();
  }
  if (out != nullptr) {   // (no output: the caller merges the partial results itself)
    launch_decode_merge(part_o, part_lse, seq_lens, out, num_seqs, max_splits, Hq, D, window, st);
    DIB_CHECK_LAUNCH();
  }
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
int dib_attention_bf16_status_clear() {
  const int v = 0;
  return cudaMemcpyToSymbol(dib_attention_error_word, &v, sizeof(int)) == cudaSuccess ? 0 : -1;
}
int dib_attention_bf16_tile_rows() { return EXT_M; }
// From how many splits on stage 2 runs as the kernel with a group of threads per chunk
// (both kernels give the same bits; 49 unless set).
void dib_attention_bf16_set_merge_wide_from(int n) { merge_wide_from() = n; }

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

// Stage 2 alone: out [num_seqs, Hq, D] from the partial results of a call that was made
// without an output.
int dib_decode_attention_merge(const float* part_o, const float* part_lse, const int* seq_lens,
                               void* out, int num_seqs, int max_splits, int Hq, int D, int window,
                               cudaStream_t st) {
  if (num_seqs == 0) return DIB_OK;
  if (num_seqs > 65535 || max_splits < 1 || D < 1 || D > 1024) return DIB_BAD_SIZE;
  launch_decode_merge(part_o, part_lse, seq_lens, out, num_seqs, max_splits, Hq, D, window, st);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The first num_seqs sequences of the batch, one token each (token index = sequence
// index).  part_o: float32 [num_seqs, Hq, max_splits, D]; part_lse: [num_seqs, Hq,
// max_splits]; max_splits >= ceil(longest sequence / 128).  out == nullptr: only the
// partial results are made (the caller merges them, see dib_decode_attention_merge).
int dib_decode_attention_bf16(const void* q, void* out, const void* cache, long long num_pages,
                              const int* block_table, int max_blocks, const int* seq_lens,
                              float* part_o, float* part_lse, int num_seqs, int max_splits, int Hq,
                              int Hkv, int D, int page_size, float scale, int window,
                              int pipelined, cudaStream_t st) {
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
                                    window, pipelined, st);
    return launch_decode_tma<64>(q, out, cache, num_pages, block_table, max_blocks, seq_lens, part_o,
                                 part_lse, num_seqs, max_splits, Hq, Hkv, page_size, scale, window,
                                 pipelined, st);
  }
#define CALL(DD)                                                                                  \
  launch_decode<DD>(q, out, cache, block_table, max_blocks, seq_lens, part_o, part_lse, num_seqs, \
                    max_splits, Hq, Hkv, page_size, scale, window, st)
  DIB_DISPATCH_D(D, CALL)
#undef CALL
}

}  // extern "C"
