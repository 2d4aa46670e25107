// bfloat16 matrix product out[M, N] = X[M, K] * W[N, K]^T on the 5th-generation
// tensor cores: tcgen05.mma with the accumulator in tensor memory, operands staged
// in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a ring of
// mbarrier-guarded stages, float32 accumulation.
//
// "Swap-AB" form for few tokens (decode and the head): the 128 rows of the MMA are
// rows of W (output features), its N is the token count padded to 16..128, so a
// handful of tokens fills the tensor core and the kernel streams W once.  A CTA owns
// one (128 output features) x (BN tokens) tile and a contiguous range of k-blocks;
// when there are fewer tiles than SMs the k range is split across CTAs and every CTA
// writes its float32 partial tile to partial[split][token][feature].  The partials
// are added IN SPLIT ORDER by whoever reads them: the next kernel of the layer
// (residual-add + norm, q/k norm, SiLU gate) or a plain sum kernel, so no CTA waits
// for another and the result does not depend on their timing.  Neither the k order
// nor the split depends on M.
//
// Roles inside a CTA of 128 threads: warp 0 allocates tensor memory and one of its
// lanes issues the TMA loads; one lane of warp 1 issues the MMAs; all four warps read
// the accumulator back (tcgen05.ld: warp w owns lanes 32w..32w+31) and store it.
// Every mbarrier wait is bounded; a wait that runs out sets an error word that the
// host reads with dib_gemm_bf16_status(), tensor memory is still freed, and the kernel
// returns.
#include <cuda.h>

#include <cstdlib>

#include "attention_merge.cuh"
#include "common.cuh"

namespace {

constexpr int BM = 128;      // W rows per tile = MMA M
constexpr int BK = 64;       // k per stage: 64 bf16 = 128 bytes = one swizzle atom
constexpr int UMMA_K = 16;   // k per tcgen05.mma for 16-bit inputs
constexpr int THREADS = 128;

__device__ int dib_gemm_error_word = 0;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)),
      "r"(c0), "r"(c1)
      : "memory");
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
// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major.
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
__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
      "%12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes
// (one 128-byte swizzle atom wide): 8-row groups lie 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);   // start address
  d |= (unsigned long long)(1024u >> 4) << 32;         // stride between 8-row groups
  d |= 1ull << 46;                                     // descriptor version of sm_100
  d |= 2ull << 61;                                     // layout: 128-byte swizzle
  return d;
}

// kind::f16 instruction descriptor: float32 accumulator, bf16 A and B, both K-major.
constexpr unsigned make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

// ---- thread-block clusters: the CTAs that share one output tile (one per slice of k)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
// a float at the same shared-memory offset in the cluster's CTA `rank`
__device__ __forceinline__ float ld_peer_smem(const float* local, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// ---- the token operand made inside the kernel.  Instead of fetching X by TMA, the CTA
// computes the columns of X it needs (its range of k) from what the kernel before it left,
// and writes them to shared memory in the layout the TMA would have produced (rows of 128
// bytes per k-block, 128-byte swizzle), so the kernel that would have made X, and the trip
// of X through memory, are gone.  Two forms:
//   PRO_GATE:  X = silu(gate) * up of a gated feed-forward whose [gate | up] product lies
//              in memory as `S` float32 partial products of a split k (the sums in split
//              order, rounded to bfloat16 as stored products, then the gate, as the
//              kernel that reads such partials computes it);
//   PRO_MERGE: X = the split-KV decode attention's output, merged from the per-split partial
//              results (merge_chunk / merge_add of attention_merge.cuh, as its second stage
//              computes it).
// Either gives, bit for bit, the X the separate kernel writes.
enum { PRO_TMA = 0, PRO_GATE = 1, PRO_MERGE = 2 };
struct Operand {
  // PRO_GATE: parts [S][M][2 * I] float32
  const float* parts;
  int S;
  long long split_stride;
  // PRO_MERGE: part_o [M][Hq][max_splits][D], part_lse [M][Hq][max_splits], seq_lens [M]
  const float* part_o;
  const float* part_lse;
  const int* seq_lens;
  int max_splits, D, window;
};

// byte offset of the 16-byte chunk c8 (8 elements) of row r in k-block kb of the operand
// slab [k-blocks][BN rows][64 elements], 128-byte swizzle (the slab starts on 1,024 bytes)
template <int BN> __device__ __forceinline__ int slab_off(int kb, int r, int c8) {
  return kb * (BN * 128) + r * 128 + ((c8 ^ (r & 7)) << 4);
}
// The whole slab to zero: columns beyond K (the last k-block of a width that is no multiple
// of 64) and rows beyond M must not hold what shared memory happened to hold (the weights'
// columns beyond K are zero, and 0 times a NaN is a NaN).
template <int BN> __device__ __forceinline__ void slab_clear(unsigned char* slab, int nkb) {
  for (int i = threadIdx.x; i < nkb * BN * 8; i += THREADS)
    *reinterpret_cast<uint4*>(slab + (size_t)i * 16) = make_uint4(0, 0, 0, 0);
}
__device__ __forceinline__ unsigned pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Both forms first bring what they read into shared memory with bulk copies that are all in
// flight together (one trip to memory, whatever the number of splits), then compute from
// there.  `stage` is that buffer, `bar` the barrier its copies complete on.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes,
                                         unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// X[m][k0 .. k0 + nkb*64) for m < M of the gated feed-forward; K = I.
// stage: [S][M][2 (gate, up)][len] float32, len = the CTA's columns.
template <int BN>
__device__ __forceinline__ bool operand_gate(unsigned char* slab, float* stage, unsigned long long* bar,
                                             const Operand& op, int M, int K, int k0, int nkb) {
  const int len = min(nkb * 64, K - k0);            // a multiple of 8
  const int copies = op.S * M * 2;
  if (threadIdx.x == 0) mbar_expect_tx(bar, (unsigned)copies * len * 4);
  slab_clear<BN>(slab, nkb);
  __syncthreads();
  for (int c = threadIdx.x; c < copies; c += THREADS) {
    const int gu = c & 1, m = (c >> 1) % M, sp = (c >> 1) / M;
    bulk_g2s(stage + (size_t)c * len, op.parts + sp * op.split_stride + (size_t)m * 2 * K + gu * K + k0,
             (unsigned)len * 4, bar);
  }
  const bool ok = mbar_wait(bar, 0);
  const int quads = len / 4;
  for (int id = threadIdx.x; id < M * quads; id += THREADS) {     // a thread takes 4 columns of a row
    const int r = id / quads, col = (id % quads) * 4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
    for (int sp = 0; sp < op.S; ++sp) {              // the sums in split order
      const float* p = stage + ((size_t)(sp * M + r) * 2) * len + col;
      const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + len);
      g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
      u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
    }
    const float y0 = silu_gate<__nv_bfloat16>(round_to<__nv_bfloat16>(g.x), round_to<__nv_bfloat16>(u.x));
    const float y1 = silu_gate<__nv_bfloat16>(round_to<__nv_bfloat16>(g.y), round_to<__nv_bfloat16>(u.y));
    const float y2 = silu_gate<__nv_bfloat16>(round_to<__nv_bfloat16>(g.z), round_to<__nv_bfloat16>(u.z));
    const float y3 = silu_gate<__nv_bfloat16>(round_to<__nv_bfloat16>(g.w), round_to<__nv_bfloat16>(u.w));
    *reinterpret_cast<uint2*>(slab + slab_off<BN>(col >> 6, r, (col & 63) >> 3) + ((col >> 2) & 1) * 8) =
        ok ? make_uint2(pack2_bf16(y0, y1), pack2_bf16(y2, y3)) : make_uint2(0, 0);
  }
  return ok;
}

// X[m][k0 .. ) = merged attention output of sequence m, column k = head * D + dim; K = Hq * D.
// The CTA's columns are `seg` consecutive dimensions of each of `nh` heads (seg = D when the
// range covers whole heads, else the range lies inside one head).
// stage: [M][nh][max_splits][seg] float32, then the log-sum-exps and the weights
// [M][nh][max_splits] each, and the sequences' lengths [M].
template <int BN>
__device__ __forceinline__ bool operand_merge(unsigned char* slab, float* stage, unsigned long long* bar,
                                              const Operand& op, int M, int K, int k0, int nkb) {
  constexpr int CH = MERGE_CH;
  const int D = op.D, Hq = K / D, S = op.max_splits;
  const int len = min(nkb * 64, K - k0);
  const int h0 = k0 / D, d0 = k0 % D;
  const int seg = min(D - d0, len), nh = (len + seg - 1) / seg;     // (the launcher checks the fit)
  float* s_lse = stage + (size_t)M * nh * S * seg;
  float* s_w = s_lse + (size_t)M * nh * S;                             // the splits' weights
  int* s_len = reinterpret_cast<int*>(s_w + (size_t)M * nh * S);       // the sequences' lengths
  // whole heads: one copy per (sequence, head) of all its splits; part of a head: one per split
  const int per_copy = seg == D ? S : 1;
  const int copies = M * nh * (S / per_copy);
  if (threadIdx.x == 0) mbar_expect_tx(bar, (unsigned)(M * nh * S) * seg * 4);
  slab_clear<BN>(slab, nkb);
  __syncthreads();
  for (int c = threadIdx.x; c < copies; c += THREADS) {
    const int unit = c * per_copy;                  // index of (m, head, split) in stage order
    const int sp = unit % S, hh = (unit / S) % nh, m = unit / (S * nh);
    bulk_g2s(stage + (size_t)unit * seg,
             op.part_o + ((((size_t)m * Hq + h0 + hh) * S + sp) * D + d0), (unsigned)(per_copy * seg) * 4, bar);
  }
  for (int e = threadIdx.x; e < M * nh * S; e += THREADS) {
    const int sp = e % S, hh = (e / S) % nh, m = e / (S * nh);
    s_lse[e] = op.part_lse[((size_t)m * Hq + h0 + hh) * S + sp];
  }
  for (int e = threadIdx.x; e < M; e += THREADS) s_len[e] = op.seq_lens[e];
  const bool ok = mbar_wait(bar, 0);
  __syncthreads();                                   // the log-sum-exps and lengths are in place
  // every split's weight once
  for (int e = threadIdx.x; e < M * nh * S; e += THREADS) {
    const int sp = e % S, m = e / (S * nh);
    int s0, s1;
    merge_range(s_len[m], op.window, S, s0, s1);
    float w = 0.f;
    if (sp >= s0 && sp <= s1) {
      const float* pl = s_lse + (e - sp);
      float M_lse = MERGE_NEG_BIG;
      for (int t = s0; t <= s1; ++t) M_lse = fmaxf(M_lse, pl[t]);
      w = merge_weight(pl[sp], M_lse);
    }
    s_w[e] = w;
  }
  __syncthreads();
  // a thread takes V dimensions of a row: 4 when that keeps every thread busy, else 1
  const bool four = M * len >= 4 * THREADS;
  const int per_row = four ? len / 4 : len;
  for (int id = threadIdx.x; id < M * per_row; id += THREADS) {
    const int r = id / per_row, col = (id % per_row) * (four ? 4 : 1);
    const int hh = col / seg, d = col % seg;       // seg is a multiple of 4: the 4 dimensions share a head
    const float* po = stage + ((size_t)(r * nh + hh) * S) * seg + d;
    const float* pw = s_w + (size_t)(r * nh + hh) * S;
    int s0, s1;
    merge_range(s_len[r], op.window, S, s0, s1);
    const int c0 = s0 / CH, c1 = s1 / CH;
    float total[4] = {0.f, 0.f, 0.f, 0.f}, total_den = 0.f;
    for (int c = c0; c <= c1; ++c) {
      float w[CH], o[CH][4];
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int sp = c * CH + j;
        const bool in = sp >= s0 && sp <= s1;
        w[j] = in ? pw[sp] : 0.f;
        if (four) {
          const float4 v = in ? *reinterpret_cast<const float4*>(po + (size_t)sp * seg)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
          o[j][0] = v.x; o[j][1] = v.y; o[j][2] = v.z; o[j][3] = v.w;
        } else {
          o[j][0] = in ? po[(size_t)sp * seg] : 0.f;
          o[j][1] = o[j][2] = o[j][3] = 0.f;
        }
      }
      float acc[4], den;
      merge_chunk_weighted<4>(w, o, c, s0, s1, acc, den);
      merge_add<4>(c == c0, acc, den, total, total_den);
    }
    unsigned char* dst = slab + slab_off<BN>(col >> 6, r, (col & 63) >> 3) + (col & 7) * 2;
    if (four) {
      *reinterpret_cast<uint2*>(dst) =
          ok ? make_uint2(pack2_bf16(merge_finish(total[0], total_den), merge_finish(total[1], total_den)),
                          pack2_bf16(merge_finish(total[2], total_den), merge_finish(total[3], total_den)))
             : make_uint2(0, 0);
    } else {
      *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(ok ? merge_finish(total[0], total_den) : 0.f);
    }
  }
  return ok;
}

// GATED: w is [gate rows ; up rows] of a gated feed-forward ([2N, K]); a tile holds 64
// gate rows and the 64 up rows of the same features, and the epilogue writes
// silu(gate) * up, [M, N], so the gate/up product never goes to memory.
// CLUSTER: the `splits` CTAs of a tile (grid z) form a thread-block cluster; each leaves
// its partial tile in its shared memory, and each then adds up, over all of them in split
// order, its share of the tile's rows through distributed shared memory and writes the
// finished values: no partial products in global memory, and a gate can follow a split k.
template <int BN, typename OutT, bool GATED, int STAGES, bool CLUSTER, int PRO = PRO_TMA>
__global__ void __launch_bounds__(THREADS)
gemm_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 OutT* __restrict__ out, float* __restrict__ partial, int M, int N, int num_kb,
                 int kb_per_split, int splits, int K, const Operand op) {
  static_assert(PRO == PRO_TMA || (!GATED && !CLUSTER), "an operand made in the kernel: plain product only");
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = PRO == PRO_TMA ? BN * BK * 2 : 0;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // with an operand made in the kernel: its slab first (kb_per_split k-blocks of BN rows of
  // 128 bytes, rounded up to 1,024 bytes), then the ring of weight stages
  unsigned char* slab = smem;
  if (PRO != PRO_TMA) smem += ((size_t)kb_per_split * BN * 128 + 1023) & ~(size_t)1023;
  unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* accum = empty + STAGES;
  unsigned long long* stage_bar = accum + 1;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(stage_bar + 1);
  float* stage = reinterpret_cast<float*>(tmem_slot + 4);     // 16-byte aligned; only with PRO

  pdl_trigger();   // the kernel after this one may set itself up (and fetch its weights) beside this one
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_w);
    if (PRO == PRO_TMA) prefetch_tensormap(&map_x);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * (GATED ? BM / 2 : BM), m0 = blockIdx.y * BN, split = blockIdx.z;
  const int kb_begin = split * kb_per_split;
  const int nkb = min(kb_per_split, num_kb - kb_begin);

  if (warp == 1 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    mbar_init(stage_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((unsigned)TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_slot;
  bool ok = true;
  const int pre = nkb < STAGES ? nkb : STAGES;

  if (PRO != PRO_TMA) {
    // The weights of the first stages are sent for, then every thread waits for the kernel
    // before this one and the CTA builds its slab of the token operand; the roles follow.
    if (warp == 0 && lane == 0) {
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], STAGE_BYTES);
        tma_load_2d(smem + i * STAGE_BYTES, &map_w, (kb_begin + i) * BK, n0, &full[i]);
      }
    }
    pdl_wait();
    bool made;
    if (PRO == PRO_GATE) made = operand_gate<BN>(slab, stage, stage_bar, op, M, K, kb_begin * BK, nkb);
    else made = operand_merge<BN>(slab, stage, stage_bar, op, M, K, kb_begin * BK, nkb);
    if (!made) atomicExch(&dib_gemm_error_word, 1);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the slab is read by the MMA unit
    __syncthreads();
  }

  if (warp == 0 && lane == 0) {
    // ---- TMA producer.  The weights do not depend on the kernel before this one, so
    // their loads for the first stages start before the wait for that kernel; the
    // activations follow after it.
    if (PRO == PRO_TMA) {
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], STAGE_BYTES);
        if (GATED) {
          tma_load_2d(smem + i * STAGE_BYTES, &map_w, (kb_begin + i) * BK, n0, &full[i]);
          tma_load_2d(smem + i * STAGE_BYTES + A_BYTES / 2, &map_w, (kb_begin + i) * BK, N + n0,
                      &full[i]);
        } else {
          tma_load_2d(smem + i * STAGE_BYTES, &map_w, (kb_begin + i) * BK, n0, &full[i]);
        }
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + i * STAGE_BYTES + A_BYTES, &map_x, (kb_begin + i) * BK, m0, &full[i]);
    }
    for (int i = pre; i < nkb && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(&empty[s], ((i / STAGES) - 1) & 1);
      if (!ok) break;
      mbar_expect_tx(&full[s], STAGE_BYTES);
      unsigned char* a = smem + s * STAGE_BYTES;
      const int k = (kb_begin + i) * BK;
      tma_load_2d(a, &map_w, k, n0, &full[s]);
      if (GATED) tma_load_2d(a + A_BYTES / 2, &map_w, k, N + n0, &full[s]);
      if (PRO == PRO_TMA) tma_load_2d(a + A_BYTES, &map_x, k, m0, &full[s]);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer
    constexpr unsigned idesc = make_idesc(BM, BN);
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(&full[s], (i / STAGES) & 1);
      if (!ok) break;
      tc_fence_after();
      const unsigned a = smem_u32(smem + s * STAGE_BYTES);
      const unsigned b = PRO == PRO_TMA ? a + A_BYTES : smem_u32(slab) + i * (BN * 128);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        tc_mma(tmem, smem_desc_sw128(a + k * UMMA_K * 2), smem_desc_sw128(b + k * UMMA_K * 2), idesc,
               (i > 0 || k > 0) ? 1u : 0u);
      tc_commit(&empty[s]);   // the stage is free once these MMAs have read it
    }
    if (ok) tc_commit(accum);  // the accumulator is complete once all MMAs are done
  }
  if (!ok) atomicExch(&dib_gemm_error_word, 1);
  __syncwarp();
  pdl_wait();   // nothing is stored before the kernel before this one has finished

  // ---- epilogue: accumulator D[n (lane), token (column)] -> out[token][n]
  bool acc_ok = mbar_wait(accum, 0);
  acc_ok = __all_sync(0xffffffffu, acc_ok);   // tcgen05.ld below is warp-wide
  if (!acc_ok) atomicExch(&dib_gemm_error_word, 1);
  tc_fence_after();
  const int n = n0 + warp * 32 + lane;
  if (CLUSTER) {
    // the pipeline stages are free (every MMA has completed): this CTA's partial tile
    // goes there as [128 rows][BN + 1] float
    constexpr int LD = BN + 1;
    float* stg = reinterpret_cast<float*>(smem);
#pragma unroll 1
    for (int c = 0; c < BN / 16; ++c) {
      unsigned r[16];
      if (acc_ok) {
        tc_ld16(tmem + ((unsigned)(warp * 32) << 16) + c * 16, r);
        tc_wait_ld();
      }
#pragma unroll
      for (int j = 0; j < 16; ++j)
        stg[(warp * 32 + lane) * LD + c * 16 + j] = acc_ok ? __uint_as_float(r[j]) : 0.f;
    }
    cluster_sync_all();
    const unsigned rank = blockIdx.z;
    const int cols = min(BN, M - m0);
    if (GATED) {
      // feature pairs (gate row p, up row 64 + p): this CTA's share of the 64
      const int per = (BM / 2 + splits - 1) / splits;
      const int p0 = rank * per, np = max(0, min(BM / 2, p0 + per) - p0);
      for (int e = threadIdx.x; e < np * cols; e += THREADS) {
        const int p = p0 + e % np, col = e / np;
        if (n0 + p >= N) continue;
        float g = 0.f, u = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
          g += ld_peer_smem(stg + p * LD + col, sp);
          u += ld_peer_smem(stg + (BM / 2 + p) * LD + col, sp);
        }
        g = round_to<__nv_bfloat16>(g);
        u = round_to<__nv_bfloat16>(u);
        Elem<OutT>::store(out + (size_t)(m0 + col) * N + n0 + p, silu_gate<OutT>(g, u));
      }
    } else {
      const int per = (BM + splits - 1) / splits;
      const int r0 = rank * per, nr = max(0, min(BM, r0 + per) - r0);
      for (int e = threadIdx.x; e < nr * cols; e += THREADS) {
        const int row = r0 + e % nr, col = e / nr;
        if (n0 + row >= N) continue;
        float acc = 0.f;
        for (int sp = 0; sp < splits; ++sp) acc += ld_peer_smem(stg + row * LD + col, sp);
        Elem<OutT>::store(out + (size_t)(m0 + col) * N + n0 + row, acc);
      }
    }
    cluster_sync_all();   // nobody leaves while a peer may still read its tile
  } else if (GATED) {
    // rows 0..63 of the tile are gate rows (warps 0, 1), rows 64..127 the up rows of
    // the same features (warps 2, 3): the up values go through shared memory (the
    // pipeline stages are free: every MMA has completed)
    float* ex = reinterpret_cast<float*>(smem);   // [64][17]
    const int pr = (warp & 1) * 32 + lane;         // pair index inside the tile
#pragma unroll 1
    for (int c = 0; c < BN / 16; ++c) {
      unsigned r[16];
      if (acc_ok) {
        tc_ld16(tmem + ((unsigned)(warp * 32) << 16) + c * 16, r);
        tc_wait_ld();
      }
      if (warp >= 2) {
#pragma unroll
        for (int j = 0; j < 16; ++j) ex[pr * 17 + j] = __uint_as_float(r[j]);
      }
      __syncthreads();
      if (warp < 2 && acc_ok && n0 + pr < N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + c * 16 + j;
          if (m >= M) break;
          const float g = round_to<__nv_bfloat16>(__uint_as_float(r[j]));
          const float u = round_to<__nv_bfloat16>(ex[pr * 17 + j]);
          Elem<OutT>::store(out + (size_t)m * N + n0 + pr, silu_gate<OutT>(g, u));
        }
      }
      __syncthreads();
    }
  } else if (acc_ok) {
#pragma unroll
    for (int c = 0; c < BN / 16; ++c) {
      unsigned r[16];
      tc_ld16(tmem + ((unsigned)(warp * 32) << 16) + c * 16, r);
      tc_wait_ld();
      if (n < N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + c * 16 + j;
          if (m >= M) break;
          const float v = __uint_as_float(r[j]);
          if (splits == 1) Elem<OutT>::store(out + (size_t)m * N + n, v);
          else partial[((size_t)split * M + m) * N + n] = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"((unsigned)TMEM_COLS));
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a row-major bf16 matrix [rows, K] with boxes of box_rows x 64
// elements, 128-byte swizzle; out-of-range elements read as zero.
bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// STAGES: 4 keeps several CTAs on an SM (grids with many more CTAs than SMs overlap one
// CTA's ramp-up with another's stream); 8 keeps more bytes in flight for a CTA that has
// the SM to itself and a long range of k to walk.
template <int BN, typename OutT, bool GATED, int STAGES, bool CLUSTER>
int launch_swap_stages(const CUtensorMap& mw, const CUtensorMap& mx, void* out, float* partial,
                       int M, int N, int num_kb, int kb_per_split, int splits, dim3 grid,
                       cudaStream_t st) {
  constexpr size_t ring = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2);
  static_assert(!CLUSTER || ring >= (size_t)BM * (BN + 1) * 4, "the partial tile must fit in the ring");
  constexpr size_t smem = ring + (2 * STAGES + 2) * 8 + 16 + 1024;
  auto kern = gemm_swap_kernel<BN, OutT, GATED, STAGES, CLUSTER>;
  static DeviceOnce attr_set;
  if (!attr_set.done()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  if (CLUSTER) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dib_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, mw, mx, (OutT*)out, partial, M, N, num_kb, kb_per_split, splits, 0,
                       Operand{});
  } else {
    dib_launch(kern, dim3(grid), dim3(THREADS), smem, st, mw, mx, (OutT*)out, partial, M, N, num_kb,
               kb_per_split, splits, 0, Operand{});
  }
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The product with its token operand made in the kernel (PRO_GATE / PRO_MERGE): one tile of
// tokens, a slab of at most MAX_SLAB bytes, four weight stages.
constexpr size_t MAX_OPERAND_SMEM = 220 * 1024;     // slab + staged inputs + ring + barriers
template <int BN, typename OutT, int PRO>
int launch_operand(const CUtensorMap& mw, void* out, float* partial, int M, int N, int K, int num_kb,
                   int kb_per_split, int splits, const Operand& op, size_t stage_bytes,
                   cudaStream_t st) {
  constexpr int STAGES = 4;
  constexpr size_t ring = (size_t)STAGES * (BM * BK * 2);
  const size_t slab = ((size_t)kb_per_split * BN * 128 + 1023) & ~(size_t)1023;
  const size_t smem = slab + ring + (2 * STAGES + 2) * 8 + 32 + stage_bytes + 1024;
  if (smem > MAX_OPERAND_SMEM) return DIB_BAD_SIZE;
  auto kern = gemm_swap_kernel<BN, OutT, false, STAGES, false, PRO>;
  static DeviceOnce attr_set;
  if (!attr_set.done()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)MAX_OPERAND_SMEM) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  dib_launch(kern, dim3((N + BM - 1) / BM, 1, splits), dim3(THREADS), smem, st, mw, mw, (OutT*)out, partial,
             M, N, num_kb, kb_per_split, splits, K, op);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

template <int BN, typename OutT, bool GATED = false>
int launch_swap(const CUtensorMap& mw, const CUtensorMap& mx, void* out, float* partial, int M,
                int N, int num_kb, int kb_per_split, int splits, dim3 grid, int sm_count,
                bool cluster, cudaStream_t st) {
  // a deep ring where a CTA has its SM to itself; else four stages, so that several
  // CTAs share an SM and stream side by side
  const long long ctas = (long long)grid.x * grid.y * grid.z;
  constexpr int DEEP = BN <= 32 ? 8 : (BN <= 64 ? 6 : 5);
  if (cluster) {
    if (kb_per_split >= 6 && ctas <= sm_count)
      return launch_swap_stages<BN, OutT, GATED, DEEP, true>(mw, mx, out, partial, M, N, num_kb,
                                                             kb_per_split, splits, grid, st);
    return launch_swap_stages<BN, OutT, GATED, 4, true>(mw, mx, out, partial, M, N, num_kb,
                                                        kb_per_split, splits, grid, st);
  }
  if (kb_per_split >= 6 && ctas <= sm_count)
    return launch_swap_stages<BN, OutT, GATED, DEEP, false>(mw, mx, out, partial, M, N, num_kb,
                                                            kb_per_split, splits, grid, st);
  return launch_swap_stages<BN, OutT, GATED, 4, false>(mw, mx, out, partial, M, N, num_kb,
                                                       kb_per_split, splits, grid, st);
}

}  // namespace

namespace {

// The time of a product, in units of one SM streaming one k-block of a weight tile.
// The CTAs spread over the SMs, up to RESIDENT of them on an SM at a time (four-stage
// ring, small token tile); an SM's time is its k-blocks plus a start-up per round of
// resident CTAs, which weighs more on a CTA that is alone on its SM (nothing else
// streams while its first block is on the way).  Splitting k makes more, shorter CTAs:
// the SMs get equal loads and the start-ups hide behind one another.  Measured on the
// layer shapes of the 0.6B, 8B and 32B presets.  Depends on N, K and the number of SMs
// only, never on the number of rows, so a row's order of summation does not depend on
// the batch.
constexpr int RESIDENT = 3;
constexpr int START_ALONE_KB = 7, START_SHARED_KB = 3;
constexpr int READER_KB = 8;     // the kernel that reads split gate_up partials and gates
long long cost_of(long long ctas, int per, int sm_count) {
  if (ctas <= sm_count) return per + START_ALONE_KB;
  const long long on_sm = (ctas + sm_count - 1) / sm_count;
  const long long rounds = (on_sm + RESIDENT - 1) / RESIDENT;
  return on_sm * per + START_SHARED_KB * rounds;
}
// The CTAs of a tile as a thread-block cluster (8 at most) that adds its partial tiles up
// itself, instead of partial products in global memory that the next kernel adds.  Off
// unless DIB200_GEMM_CLUSTER=1: it measured slower on B200 (N=4096, K=1024, 8 splits: 6.2
// against 2.7 us with 8 rows, 18.7 against 4.7 us with 64 rows; the cluster launch and
// its two barriers alone cost 2 us, the reads from the peers' shared memory the rest).
int& cluster_option() {
  static int v = -1;     // -1: not yet read from the environment (read once)
  return v;
}
bool cluster_enabled() {
  int& v = cluster_option();
  if (v < 0) {
    const char* e = getenv("DIB200_GEMM_CLUSTER");
    v = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}
int& forced_splits_option() {
  static int v = -1;     // -1: not yet read; 0: the model's choice
  return v;
}
constexpr int MAX_CLUSTER = 8;

long long plan_cost(int n_tiles, int num_kb, int sm_count, int* per_out) {
  long long best = -1;
  int best_per = num_kb;
  if (sm_count < 1) sm_count = 1;
  const int max_splits = cluster_enabled() ? MAX_CLUSTER : 16;
  for (int s = 1; s <= max_splits && s <= num_kb; ++s) {
    const int per = (num_kb + s - 1) / s;
    const int real = (num_kb + per - 1) / per;
    if (real != s) continue;   // the same cut as a smaller s
    // In twentieths of a unit.  A split also writes and reads its partial products:
    // counted for 32 rows (the plan must not know the real number), 8 bytes per
    // element and split against the 16 KB of a weight k-block, spread over the SMs.
    long long cost = cost_of((long long)n_tiles * real, per, sm_count) * 20;
    if (s > 1 && !cluster_enabled()) cost += 20ll * s * 32 * n_tiles * BM * 8 / (BM * BK * 2) / sm_count;
    if (best < 0 || cost < best) {
      best = cost;
      best_per = per;
    }
  }
  *per_out = best_per;
  return best;
}

// k-blocks per split: the model's choice, or a forced number of splits (DIB200_GEMM_SPLITS=n
// in the environment when the library is first used, or dib_gemm_bf16_configure)
int planned_per(int n_tiles, int num_kb, int sm_count) {
  int per = num_kb;
  plan_cost(n_tiles, num_kb, sm_count, &per);
  int& forced = forced_splits_option();
  if (forced < 0) {
    const char* e = getenv("DIB200_GEMM_SPLITS");
    forced = e != nullptr ? atoi(e) : 0;
    if (forced < 0) forced = 0;
  }
  if (forced >= 1) {
    per = (num_kb + forced - 1) / forced;
    if (per < 1) per = 1;
  }
  return per;
}

}  // namespace

extern "C" {

int dib_gemm_bf16_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, dib_gemm_error_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
// Measurement and test switches (both are read from the environment once, at first use):
// cluster 0/1: the CTAs of a tile add their partial tiles up as a thread-block cluster;
// forced_splits 0: the model's choice of the split of k, n >= 1: n splits.  A negative
// value leaves a switch as it is.
void dib_gemm_bf16_configure(int cluster, int forced_splits) {
  cluster_enabled();
  if (cluster >= 0) cluster_option() = cluster ? 1 : 0;
  if (forced_splits >= 0) forced_splits_option() = forced_splits;
  else if (forced_splits_option() < 0) forced_splits_option() = 0;
}
// Sets the error word back to 0 (after the failure has been reported).
int dib_gemm_bf16_status_clear() {
  const int v = 0;
  return cudaMemcpyToSymbol(dib_gemm_error_word, &v, sizeof(int)) == cudaSuccess ? 0 : -1;
}

// How the product of these sizes is cut: tokens per tile, k-blocks per split, number
// of splits.  A function of (M, N, K, number of SMs) only; the split of k depends on
// N and K, never on M.
void dib_gemm_bf16_plan(int M, int N, int K, int sm_count, int* bn, int* kb_per_split,
                        int* splits) {
  int b = 16;
  while (b < M && b < 128) b <<= 1;
  const int n_tiles = (N + BM - 1) / BM;
  const int num_kb = (K + BK - 1) / BK;
  const int per = planned_per(n_tiles, num_kb, sm_count);
  *bn = b;
  *kb_per_split = per;
  *splits = (num_kb + per - 1) / per;
}

// 1 if the gate_up product of intermediate size I is better run as one kernel with the
// gate in its epilogue (one CTA per 64 features, k not split) than as the split product
// followed by the kernel that adds the partials and applies the gate.
int dib_gemm_bf16_gated_pays(int I, int K, int sm_count) {
  if (sm_count < 1) return 0;
  if (cluster_enabled()) return 1;   // the gate follows the cluster's sum: no second kernel either way
  const int num_kb = (K + BK - 1) / BK;
  const int ctas = I / 64;
  const long long gated = cost_of(ctas, num_kb, sm_count) * 20;
  int per;
  const long long split = plan_cost((2 * I + BM - 1) / BM, num_kb, sm_count, &per) + READER_KB * 20;
  return gated <= split ? 1 : 0;
}

// x[M, K] * w[N, K]^T, bf16 inputs, float32 accumulation.  With `splits` == 1 (as
// dib_gemm_bf16_plan says, or forced by passing partial == nullptr) the product goes to
// out [M, N], bf16 (out_fp32 = 0) or float32.  Otherwise out is not touched and
// partial [splits, M, N] float32 receives the partial products, to be added in split
// order by the reader.  K must be a multiple of 8 (TMA wants 16-byte row strides); x
// and w must be 16-byte aligned.
// 1 if a product of these sizes has its split of k added up inside the kernel (by the
// cluster of a tile's CTAs), so that it comes out finished although k is split.
int dib_gemm_bf16_cluster_reduces(int N, int K, int sm_count) {
  if (!cluster_enabled()) return 0;
  int bn, per, splits;
  dib_gemm_bf16_plan(1, N, K, sm_count, &bn, &per, &splits);
  return splits >= 2 && splits <= MAX_CLUSTER ? 1 : 0;
}

int dib_gemm_bf16(const void* x, const void* w, void* out, int M, int N, int K, int out_fp32,
                  float* partial, int sm_count, cudaStream_t st) {
  if (M == 0 || N == 0) return DIB_OK;
  if (K < 8 || K % 8 != 0) return DIB_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16 != 0) return DIB_BAD_ALIGN;
  int bn, per, splits;
  dib_gemm_bf16_plan(M, N, K, sm_count, &bn, &per, &splits);
  const int n_tiles = (N + BM - 1) / BM, m_tiles = (M + bn - 1) / bn;
  const int num_kb = (K + BK - 1) / BK;
  // no buffer for partial products: the finished product is wanted, from the tile's
  // cluster if the plan splits k and clusters are on, else from one CTA that walks all of k
  const bool cluster = partial == nullptr && splits >= 2 && splits <= MAX_CLUSTER && cluster_enabled();
  if (partial == nullptr && !cluster) {
    splits = 1;
    per = num_kb;
  }
  if (m_tiles > 65535 || splits > 65535) return DIB_BAD_SIZE;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, BM) || !make_map(&mx, x, M, K, bn)) return DIB_LAUNCH_FAILED;
  dim3 grid(n_tiles, m_tiles, splits);
#define CALL(BNV)                                                                              \
  (out_fp32 ? launch_swap<BNV, float>(mw, mx, out, partial, M, N, num_kb, per, splits, grid, sm_count, \
                                      cluster, st)                                                \
            : launch_swap<BNV, __nv_bfloat16>(mw, mx, out, partial, M, N, num_kb, per, splits,  \
                                              grid, sm_count, cluster, st))
  switch (bn) {
    case 16: return CALL(16);
    case 32: return CALL(32);
    case 64: return CALL(64);
    default: return CALL(128);
  }
#undef CALL
}

// The product out[M, N] = X[M, K] * w[N, K]^T whose X is not in memory yet: the kernel makes
// the columns of X it needs while it waits for its weights.
//   pro 1: X = silu(gate) * up, [gate | up] given as float32 partial products of a split k,
//          parts [S][M][2K] (split_stride elements apart);
//   pro 2: X = the split-KV decode attention's output [M][Hq * D], given as its per-split
//          partial results part_o [M][Hq][max_splits][D], part_lse [M][Hq][max_splits] and
//          the sequences' lengths (seq_lens [M], window).
// The split of k is the one dib_gemm_bf16_plan gives for (N, K); out / partial as in
// dib_gemm_bf16.  Returns -2 for shapes it does not take (more than 128 rows, inputs of X
// that do not fit a CTA's shared memory, widths that are no multiples of 8): the caller then makes X with the
// kernel of its own and calls dib_gemm_bf16.
int dib_gemm_bf16_operand(int pro, const void* w, void* out, int M, int N, int K, int out_fp32,
                          float* partial, int sm_count, const float* parts, int S,
                          long long split_stride, const float* part_o, const float* part_lse,
                          const int* seq_lens, int max_splits, int D, int window, cudaStream_t st) {
  if (M == 0 || N == 0) return DIB_OK;
  if (K < 8 || K % 8 != 0 || M > 128) return DIB_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(w) % 16 != 0) return DIB_BAD_ALIGN;
  Operand op = {};
  if (pro == PRO_GATE) {
    if (parts == nullptr || S < 1 || split_stride % 4 != 0 || reinterpret_cast<uintptr_t>(parts) % 16 != 0)
      return DIB_BAD_SIZE;
    op.parts = parts; op.S = S; op.split_stride = split_stride;
  } else if (pro == PRO_MERGE) {
    if (part_o == nullptr || part_lse == nullptr || seq_lens == nullptr || max_splits < 1 || D < 4 ||
        D % 4 != 0 || K % D != 0 || reinterpret_cast<uintptr_t>(part_o) % 16 != 0)
      return DIB_BAD_SIZE;
    op.part_o = part_o; op.part_lse = part_lse; op.seq_lens = seq_lens;
    op.max_splits = max_splits; op.D = D; op.window = window;
  } else {
    return DIB_BAD_SIZE;
  }
  int bn, per, splits;
  dib_gemm_bf16_plan(M, N, K, sm_count, &bn, &per, &splits);
  const int num_kb = (K + BK - 1) / BK;
  if (partial == nullptr) {
    splits = 1;
    per = num_kb;
  }
  if (splits > 65535) return DIB_BAD_SIZE;
  // what a CTA stages of the inputs of X: its columns (at most per * 64) of every row
  const long long len = per * BK < K ? per * BK : K;
  size_t stage_bytes;
  if (pro == PRO_GATE) {
    stage_bytes = (size_t)S * M * 2 * len * 4;
  } else {
    // the range of a CTA is whole heads, or lies inside one head
    if (!((per * BK) % D == 0 || D % (per * BK) == 0)) return DIB_BAD_SIZE;
    const long long seg = len < D ? len : D, nh = (len + seg - 1) / seg;
    stage_bytes = (size_t)M * nh * max_splits * (seg + 2) * 4 + (size_t)M * 4;
    if ((seg * 4) % 16 != 0) return DIB_BAD_SIZE;
  }
  CUtensorMap mw;
  if (!make_map(&mw, w, N, K, BM)) return DIB_LAUNCH_FAILED;
#define CALL(BNV, PROV)                                                                                \
  (out_fp32 ? launch_operand<BNV, float, PROV>(mw, out, partial, M, N, K, num_kb, per, splits, op,    \
                                               stage_bytes, st)                                       \
            : launch_operand<BNV, __nv_bfloat16, PROV>(mw, out, partial, M, N, K, num_kb, per, splits, \
                                                       op, stage_bytes, st))
#define CALL_BN(PROV)                  \
  switch (bn) {                        \
    case 16: return CALL(16, PROV);    \
    case 32: return CALL(32, PROV);    \
    case 64: return CALL(64, PROV);    \
    default: return CALL(128, PROV);   \
  }
  if (pro == PRO_GATE) { CALL_BN(PRO_GATE) }
  CALL_BN(PRO_MERGE)
#undef CALL_BN
#undef CALL
}

// out[M, I] = silu(x w_gate^T) * (x w_up^T) with w = [w_gate ; w_up] of shape [2I, K]
// (bf16 in, bf16 out; the two products are rounded to bf16 before the gate, as stored
// products would be).  I must be a multiple of 64, K of 8.
int dib_gemm_bf16_gated(const void* x, const void* w, void* out, int M, int I, int K,
                        int sm_count, cudaStream_t st) {
  if (M == 0 || I == 0) return DIB_OK;
  if (K < 8 || K % 8 != 0 || I % 64 != 0) return DIB_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16 != 0) return DIB_BAD_ALIGN;
  int bn = 16;
  while (bn < M && bn < 128) bn <<= 1;
  const int m_tiles = (M + bn - 1) / bn, num_kb = (K + BK - 1) / BK;
  if (m_tiles > 65535) return DIB_BAD_SIZE;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, 2ll * I, K, BM / 2) || !make_map(&mx, x, M, K, bn)) return DIB_LAUNCH_FAILED;
  // k is split over a cluster of CTAs per tile where that fills the GPU better
  int per = num_kb, splits = 1;
  if (cluster_enabled()) {
    per = planned_per(I / 64, num_kb, sm_count);
    splits = (num_kb + per - 1) / per;
    if (splits > MAX_CLUSTER) { splits = 1; per = num_kb; }
  }
  const bool cluster = splits > 1;
  dim3 grid(I / 64, m_tiles, splits);
#define CALL(BNV) \
  launch_swap<BNV, __nv_bfloat16, true>(mw, mx, out, nullptr, M, I, num_kb, per, splits, grid, sm_count, cluster, st)
  switch (bn) {
    case 16: return CALL(16);
    case 32: return CALL(32);
    case 64: return CALL(64);
    default: return CALL(128);
  }
#undef CALL
}

}  // extern "C"
