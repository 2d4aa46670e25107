// bfloat16 matrix product out[M, N] = X[M, K] * W[N, K]^T for many rows (prompt portions) on
// the 5th-generation tensor cores: persistent kernels, one CTA per SM, that walk output
// tiles.  Two kernels: one CTA on a tile of 128 tokens x 256 (or 128) features, described
// first, and a pair of CTAs on a tile of 256 x 256 (tcgen05.mma.cta_group::2, described at
// its definition), which large products take: each SM then fetches a third less per
// k-block, and the rate at which L2 feeds the SMs is what bounds these products.
// tcgen05.mma (M 128, N 256, K 16) with the accumulator
// in tensor memory, operands staged by TMA (128-byte swizzle) through a ring of four
// mbarrier-guarded stages of 48 KB, float32 accumulation over all of k in one pass, in the
// same order for every tile and tile shape: a row's bits do not depend on how many rows the
// step has.
//
// The accumulator is double-buffered (2 x 256 of the 512 tensor-memory columns): while the
// four epilogue warps read tile i back (tcgen05.ld: a thread owns one token row), round it
// and store it, the MMA warp already works on tile i + 1.  Tiles are taken in an order that
// keeps the CTAs that run side by side on the same 256 weight rows (they differ in their
// token tile), so a weight tile comes from DRAM once and from L2 afterwards.
//
// GATED: W = [gate rows ; up rows] of a gated feed-forward ([2N, K]); a tile holds 128
// gate rows and the 128 up rows of the same features, and the epilogue writes
// silu(gate) * up, [M, N]: the [gate | up] product and the gate kernel's pass over it are
// gone.  The two products are rounded to bfloat16 first, as stored products would be, and
// the gate is silu_gate<bf16> of common.cuh, so the bits are those of the two-kernel path.
//
// Roles in a CTA of 384 threads: warp 0 issues the TMA loads (the weights of the first
// stages before the programmatic dependency wait, the tokens after it), warp 1 allocates
// tensor memory and issues the MMAs, warps 2 and 3 have no work, warps 4-11 are the epilogue
// (two warps to each quarter of the tile's rows, half of its columns each).  Every mbarrier wait is
// bounded; a wait that runs out sets the error word (dib_gemm_bf16_large_status), tensor
// memory is still freed and the kernel returns.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int BM = 128;       // tokens per tile = MMA M
constexpr int BK = 64;        // k per stage: 128 bytes = one swizzle atom
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
// Three groups of four warps: warp 0 copies, warp 1 issues the products (2 and 3 have no
// work), warps 4-11 are the epilogue.  Registers are handed out to groups of four warps: in
// the QKV form the first group gives most of its registers back (setmaxnreg) and the epilogue
// warps take them, so that the q/k arithmetic of eight rows at a time fits without spills.
constexpr int THREADS = 384;
constexpr int EPI_WARP0 = 4;
constexpr int EPI_WARPS = 8;
constexpr int REGS_FEW = 40, REGS_MANY = 232;      // 128 * 40 + 256 * 232 = 64,512 registers
template <int N> __device__ __forceinline__ void regs_give() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void regs_take() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
// Features per tile = MMA N: 256 (GATED: 128 gate + 128 up rows), or 128 for products with so
// few tiles of 256 that they would leave SMs idle.  Stages of the ring: what fits.
// (QKV: the epilogue that norms and rotates heads stages 8 KB a warp instead of 4, a stage of
// the ring less)
template <int BNL, bool QKV = false> struct Tile {
  static constexpr int B_BYTES = BNL * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BNL == 256 ? 4 : 6) - (QKV ? 1 : 0);
  static constexpr int EPI_BYTES = EPI_WARPS * 4096 * (QKV ? 2 : 1);
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
};

__device__ int dib_gemm_large_error_word = 0;

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
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// K-major bf16 tile, rows of 128 bytes, 128-byte swizzle: 8-row groups 1,024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
// kind::f16: float32 accumulator, bf16 A and B, both K-major.
constexpr unsigned make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ unsigned pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// ---- the epilogue.  A warp owns 32 token rows (its quarter of the tile's tensor-memory lanes)
// and one half of the tile's columns.  It reads them in blocks of 128 bytes of output a row
// (64 bfloat16 or 32 float32 values), puts a block's 32 rows into its own 4 KB of shared
// memory in the 128-byte-swizzled layout, and hands that to a TMA store, which writes whole
// rows of the block and clips what lies beyond M or N.  (A thread that stores its own row
// 16 bytes at a time makes every store instruction touch 32 cache lines: 4 us for a tile's
// epilogue instead of 1.)
constexpr int EPI_STAGE_BYTES = 32 * 128;
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// 16-byte piece c (0..7) of this lane's row of the warp's staging block
__device__ __forceinline__ void stage_piece(unsigned char* stage, int lane, int c, uint4 v) {
  *reinterpret_cast<uint4*>(stage + lane * 128 + ((c ^ (lane & 7)) << 4)) = v;
}
// What the epilogue of a fused q/k/v projection needs beside the product (QKV form): the rows
// of the product are tokens, its columns the heads of 128 of q, then k, then v; a warp's half
// of a tile's 256 columns is one head.  The epilogue rounds the product to bfloat16 as a
// stored projection would be, applies the q/k RMSNorm and the rotation with the arithmetic of
// the q/k kernels of elementwise.cu (sumsq4 in the butterfly's order, rms_rstd, norm_scale,
// rope_first/second: the same bits), and writes q rows to the output and k, v rows to the
// tokens' cache slots.
struct QkvEpilogue {
  const float* q_norm_w;        // [128] or null
  const float* k_norm_w;
  float eps;
  const float* cos_sin;         // [max_pos, 128] rows cos | sin, or null
  int max_pos;
  const int* positions;         // [M]
  const int* slot_mapping;      // [M] page * page_size + offset, or negative
  __nv_bfloat16* cache;         // [pages, 2, Hkv, page_size, 128] or null
  __nv_bfloat16* q_out;         // [M, Hq, 128]
  long long num_pages;
  int page_size, Hq, Hkv, M;
};

// The QKV epilogue of a warp's 32 token rows and one head (see QkvEpilogue), in two stages.
// First every lane rounds its own row of the product to bfloat16 and puts it into the warp's
// 8 KB of shared memory (two blocks of 32 rows x 128 bytes, swizzled).  Then the warp takes
// the rows back four at a time, eight lanes a row (lane l: the dimensions 8l..8l+7 and
// 64+8l..64+8l+7, a rotation pair in one lane), runs qk_row128 of common.cuh on them, the
// function the q/k kernels run, and writes whole rows of 128 bytes: the norm weights, the
// rotation table and the stores are then read and written by neighbouring lanes together.
//
// What does not depend on the product is found before the warp waits for it
// (qkv_rows_prepare): where each row goes, its table row, and the table values of the first
// QKV_AHEAD rounds of four rows; in the loop the values of round it + QKV_AHEAD are asked for
// while round it is worked on (a table row comes from L2: several hundred cycles, a round's
// arithmetic takes a hundred or two).
constexpr int QKV_AHEAD = 8;
struct QkvRows {
  long long my_dst;       // lane r: element offset of row r's result from q_out or the cache, or -1
  int my_pos;             // lane r: row r's table row
  int head;
  bool active, is_q, is_k, rotate;
  float4 tv[QKV_AHEAD][4];
};
__device__ __forceinline__ void qkv_table(const QkvRows& R, int it, int lane, const QkvEpilogue& qk, float4 (&t)[4]) {
  if (R.rotate) {
    const int p = __shfl_sync(0xffffffffu, R.my_pos, it * 4 + (lane >> 3));
    const float* tab = qk.cos_sin + (size_t)p * 128 + (lane & 7) * 8;
    t[0] = *reinterpret_cast<const float4*>(tab);
    t[1] = *reinterpret_cast<const float4*>(tab + 4);
    t[2] = *reinterpret_cast<const float4*>(tab + 64);
    t[3] = *reinterpret_cast<const float4*>(tab + 68);
  }
}
__device__ __forceinline__ void qkv_rows_prepare(QkvRows& R, int lane, int row0, int n0, int half,
                                                 const QkvEpilogue& qk) {
  R.head = (n0 >> 7) + half;
  R.active = R.head < qk.Hq + 2 * qk.Hkv;          // else the tile's second half lies beyond the last head
  R.is_q = R.head < qk.Hq;
  R.is_k = !R.is_q && R.head < qk.Hq + qk.Hkv;
  R.rotate = R.active && qk.cos_sin != nullptr && (R.is_q || R.is_k);
  R.my_dst = -1;
  R.my_pos = 0;
  if (!R.active) return;
  const int token = row0 + lane;
  if (token < qk.M) {
    if (R.rotate) {
      const int p = qk.positions[token];
      R.my_pos = p < 0 ? 0 : (p >= qk.max_pos ? qk.max_pos - 1 : p);
    }
    if (R.is_q) {
      R.my_dst = ((long long)token * qk.Hq + R.head) * 128;
    } else if (qk.cache != nullptr) {
      const int slot = qk.slot_mapping[token];
      if (slot >= 0) {
        const long long page = slot / qk.page_size;
        if (page < qk.num_pages) {
          const int h = R.is_k ? R.head - qk.Hq : R.head - qk.Hq - qk.Hkv;
          R.my_dst = ((((page * 2 + (R.is_k ? 0 : 1)) * qk.Hkv + h) * qk.page_size) + (slot - page * qk.page_size)) * 128;
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < QKV_AHEAD; ++a) {
    R.tv[a][0] = R.tv[a][1] = R.tv[a][2] = R.tv[a][3] = make_float4(0.f, 0.f, 0.f, 0.f);
    qkv_table(R, a, lane, qk, R.tv[a]);
  }
}
__device__ __forceinline__ void store_rows_qkv(unsigned src, unsigned char* stage, int lane, int half,
                                               const QkvEpilogue& qk, QkvRows& R, const CUtensorMap* map_q,
                                               int row0) {
  if (!R.active) return;
  const unsigned acc = src + half * 128;
  // the stores of the tile before this one must have read the staging blocks
  if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  __syncwarp();
  // While a lane has its own row in hand it also takes the row's sum of squares (of the
  // rounded values), in the order of the butterfly of qk_row128: vector j (elements 4j..4j+3,
  // sumsq4) is added to vector j + 16, the sixteen sums 8 apart, then 4, 2, 1 apart.  Every
  // lane works on a row of its own here; eight lanes a row would each redo the chain of a
  // division, a root and a reciprocal, with shuffles between.
  const float* nw = R.is_q ? qk.q_norm_w : (R.is_k ? qk.k_norm_w : nullptr);
  const bool norm = nw != nullptr;
  float t16[16];
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      unsigned v[32];
      tc_ld32(acc + blk * 64 + h * 32, v);
      tc_wait_ld();
      unsigned p[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) p[k] = pack2_bf16(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
#pragma unroll
      for (int q = 0; q < 4; ++q)
        stage_piece(stage + blk * EPI_STAGE_BYTES, lane, h * 4 + q,
                    make_uint4(p[q * 4], p[q * 4 + 1], p[q * 4 + 2], p[q * 4 + 3]));
      if (norm) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {     // vector blk * 16 + h * 8 + j of the row
          const float sv = sumsq4(__uint_as_float(p[2 * j] << 16), __uint_as_float(p[2 * j] & 0xffff0000u),
                                  __uint_as_float(p[2 * j + 1] << 16), __uint_as_float(p[2 * j + 1] & 0xffff0000u));
          if (blk == 0) t16[h * 8 + j] = sv;
          else t16[h * 8 + j] = __fadd_rn(t16[h * 8 + j], sv);
        }
      }
    }
  }
  float my_rstd = 0.f;
  if (norm) {
#pragma unroll
    for (int w = 8; w > 0; w >>= 1)
#pragma unroll
      for (int j = 0; j < w; ++j) t16[j] = __fadd_rn(t16[j], t16[j + w]);
    my_rstd = rms_rstd(t16[0], 128, qk.eps);
  }
  __syncwarp();
  const int l = lane & 7;
  __nv_bfloat16* base = R.is_q ? qk.q_out : qk.cache;
  float wa[8] = {}, wb[8] = {};
  if (norm) qk_row128_weights(nw, l, wa, wb);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3);
    uint4 lo = *reinterpret_cast<const uint4*>(stage + r * 128 + ((l ^ (r & 7)) << 4));
    uint4 hi = *reinterpret_cast<const uint4*>(stage + EPI_STAGE_BYTES + r * 128 + ((l ^ (r & 7)) << 4));
    float4(&tv)[4] = R.tv[it % QKV_AHEAD];
    const float c[8] = {tv[0].x, tv[0].y, tv[0].z, tv[0].w, tv[1].x, tv[1].y, tv[1].z, tv[1].w};
    const float sn[8] = {tv[2].x, tv[2].y, tv[2].z, tv[2].w, tv[3].x, tv[3].y, tv[3].z, tv[3].w};
    if (it + QKV_AHEAD < 8) qkv_table(R, it + QKV_AHEAD, lane, qk, tv);
    const long long d = __shfl_sync(0xffffffffu, R.my_dst, r);
    const float rstd = __shfl_sync(0xffffffffu, my_rstd, r);
    if (R.is_q || R.is_k) qk_row128_apply(lo, hi, norm, rstd, wa, wb, R.rotate, c, sn);
    if (R.is_q) {
      // back to where they were staged: the q rows of the warp leave as two stores of
      // 32 rows x 128 bytes by the copy engine, which clips the rows beyond M
      *reinterpret_cast<uint4*>(stage + r * 128 + ((l ^ (r & 7)) << 4)) = lo;
      *reinterpret_cast<uint4*>(stage + EPI_STAGE_BYTES + r * 128 + ((l ^ (r & 7)) << 4)) = hi;
    } else if (d >= 0) {
      *reinterpret_cast<uint4*>(base + d + l * 8) = lo;
      *reinterpret_cast<uint4*>(base + d + 64 + l * 8) = hi;
    }
  }
  if (R.is_q) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_q, stage, R.head * 128, row0);
      tma_store_2d(map_q, stage + EPI_STAGE_BYTES, R.head * 128 + 64, row0);
    }
  }
}

template <typename OutT, bool GATED, int BNL>
__device__ __forceinline__ void store_rows(unsigned src, const CUtensorMap* map_out, unsigned char* stage,
                                           int lane, int row0, int n0, int half) {
  constexpr int PER_BLOCK = 128 / (int)sizeof(OutT);            // output values per row of a block
  constexpr int OUT_COLS = GATED ? BNL / 2 : BNL;               // output columns of a tile
  // a gated tile of 64 + 64 rows has one block of output columns: the first half's warps take it
  constexpr bool ONE_HALF = GATED && OUT_COLS == PER_BLOCK;
  constexpr int BLOCKS = ONE_HALF ? 1 : OUT_COLS / 2 / PER_BLOCK;   // blocks of this warp's half
  if (ONE_HALF && half == 1) return;
#pragma unroll 1
  for (int blk = 0; blk < BLOCKS; ++blk) {
    const int col = (ONE_HALF ? 0 : half * (OUT_COLS / 2)) + blk * PER_BLOCK;    // first output column of the block
    // the store before this one must have read the staging block
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
    if (GATED) {
      // accumulator columns 0..BNL/2-1: gate, the other half: up, of the same features
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        unsigned g[32], u[32];
        tc_ld32(src + col + h * 32, g);
        tc_ld32(src + BNL / 2 + col + h * 32, u);
        tc_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float y[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            y[e] = silu_gate<__nv_bfloat16>(round_to<__nv_bfloat16>(__uint_as_float(g[q * 8 + e])),
                                            round_to<__nv_bfloat16>(__uint_as_float(u[q * 8 + e])));
          stage_piece(stage, lane, h * 4 + q,
                      make_uint4(pack2_bf16(y[0], y[1]), pack2_bf16(y[2], y[3]), pack2_bf16(y[4], y[5]),
                                 pack2_bf16(y[6], y[7])));
        }
      }
    } else if (sizeof(OutT) == 2) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        unsigned v[32];
        tc_ld32(src + col + h * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q)
          stage_piece(stage, lane, h * 4 + q,
                      make_uint4(pack2_bf16(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1])),
                                 pack2_bf16(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3])),
                                 pack2_bf16(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5])),
                                 pack2_bf16(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]))));
      }
    } else {
      unsigned v[32];
      tc_ld32(src + col, v);
      tc_wait_ld();
#pragma unroll
      for (int q = 0; q < 8; ++q)
        stage_piece(stage, lane, q, make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the TMA reads what the lanes wrote
    __syncwarp();
    if (lane == 0) tma_store_2d(map_out, stage, n0 + col, row0);
  }
}
// before a CTA ends, its stores must have read their staging blocks
__device__ __forceinline__ void stores_done(int lane) {
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncwarp();
}

template <typename OutT, bool GATED, int BNL, bool QKV = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_large_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_out, int M, int N, int K, int m_tiles, int n_tiles,
                  const __grid_constant__ QkvEpilogue qk) {
  // (gated: a tile holds BNL / 2 gate rows and the BNL / 2 up rows of the same features)
  using TL = Tile<BNL, QKV>;
  constexpr int B_BYTES = TL::B_BYTES, STAGE_BYTES = TL::STAGE_BYTES, STAGES = TL::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* epi_stage = smem + STAGES * STAGE_BYTES;      // 4 KB to each epilogue warp
  unsigned long long* full = reinterpret_cast<unsigned long long*>(epi_stage + TL::EPI_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;     // [2] a tile's accumulator is complete
  unsigned long long* acc_empty = acc_full + 2;      // [2] the epilogue has read it (128 arrivals)
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);

  pdl_trigger();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_out);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int tiles = m_tiles * n_tiles;
  // tile t: token tile t % m_tiles of feature tile t / m_tiles; this CTA takes
  // blockIdx.x, blockIdx.x + gridDim.x, ...
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_slot;
  bool ok = true;

  if (warp < EPI_WARP0) {
    if (QKV) regs_give<REGS_FEW>();
    if (warp == 0) {
      if (lane == 0) {
        // ---- TMA producer.  The ring runs on across this CTA's tiles: load number c is
        // k-block c % num_kb of its tile number c / num_kb and goes to stage c % STAGES.  The
        // weights do not depend on the kernel before this one, so those of the first STAGES
        // loads are sent for before the wait for that kernel, the tokens after it.
        const int my_tiles = tiles > (int)blockIdx.x ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
        const int total = my_tiles * num_kb;
        auto load_w = [&](int c) {
          const int t = blockIdx.x + (c / num_kb) * gridDim.x, kb = c % num_kb;
          const int n0 = (t / m_tiles) * (GATED ? BNL / 2 : BNL);
          unsigned char* b = smem + (c % STAGES) * STAGE_BYTES + A_BYTES;
          tma_load_2d(b, &map_w, kb * BK, n0, &full[c % STAGES]);
          if (BNL == 256 || GATED)     // (the weight map's boxes are 128 rows, or BNL / 2 for a gated tile)
            tma_load_2d(b + B_BYTES / 2, &map_w, kb * BK, GATED ? N + n0 : n0 + 128, &full[c % STAGES]);
        };
        auto load_x = [&](int c) {
          const int t = blockIdx.x + (c / num_kb) * gridDim.x, kb = c % num_kb;
          tma_load_2d(smem + (c % STAGES) * STAGE_BYTES, &map_x, kb * BK, (t % m_tiles) * BM, &full[c % STAGES]);
        };
        const int pre = total < STAGES ? total : STAGES;
        for (int c = 0; c < pre; ++c) {
          mbar_expect_tx(&full[c], STAGE_BYTES);
          load_w(c);
        }
        pdl_wait();
        for (int c = 0; c < pre; ++c) load_x(c);
        for (int c = pre; c < total && ok; ++c) {
          ok = mbar_wait(&empty[c % STAGES], ((c / STAGES) - 1) & 1);
          if (!ok) break;
          mbar_expect_tx(&full[c % STAGES], STAGE_BYTES);
          load_w(c);
          load_x(c);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        // ---- MMA issuer
        constexpr unsigned idesc = make_idesc(BM, BNL);
        int count = 0, local = 0;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
          const int buf = local & 1;
          if (local >= 2) {     // the epilogue must have read this buffer's earlier tile
            ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1);
            if (!ok) break;
            tc_fence_after();
          }
          for (int kb = 0; kb < num_kb && ok; ++kb, ++count) {
            const int s = count % STAGES;
            ok = mbar_wait(&full[s], (count / STAGES) & 1);
            if (!ok) break;
            tc_fence_after();
            const unsigned a = smem_u32(smem + s * STAGE_BYTES), b = a + A_BYTES;
  #pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              tc_mma(tmem + buf * BNL, smem_desc_sw128(a + k * UMMA_K * 2), smem_desc_sw128(b + k * UMMA_K * 2),
                     idesc, (kb > 0 || k > 0) ? 1u : 0u);
            tc_commit(&empty[s]);
          }
          if (ok) tc_commit(&acc_full[buf]);
        }
      }
    }
  } else {
    if (QKV) regs_take<REGS_MANY>();
    // ---- epilogue: warps 4..11; a warp reads the 32 lanes (token rows) 32 * (warp % 4) ..,
    // warps 4-7 the first half of the columns, warps 8-11 the second
    pdl_wait();      // nothing is stored before the kernel before this one has finished
    const int quarter = warp & 3, half = (warp - EPI_WARP0) >> 2;
    const unsigned lane_base = (unsigned)(quarter * 32) << 16;
    int local = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * (GATED ? BNL / 2 : BNL);
      // (QKV tiles of 128 columns are one head: the warps of the second half have no part in them)
      const bool works = !(QKV && BNL == 128 && half == 1);
      QkvRows rows;
      if (QKV && works) qkv_rows_prepare(rows, lane, m0 + quarter * 32, n0, half, qk);
      bool got = ok && mbar_wait(&acc_full[buf], (local >> 1) & 1);
      got = __all_sync(0xffffffffu, got);     // tcgen05.ld below is warp-wide
      if (!got) { ok = false; break; }
      tc_fence_after();
      if (QKV) {
        if (works)
          store_rows_qkv(tmem + buf * BNL + lane_base, epi_stage + (warp - EPI_WARP0) * 2 * EPI_STAGE_BYTES, lane, half, qk,
                         rows, &map_out, m0 + quarter * 32);
      } else {
        store_rows<OutT, GATED, BNL>(tmem + buf * BNL + lane_base, &map_out, epi_stage + (warp - EPI_WARP0) * EPI_STAGE_BYTES,
                                     lane, m0 + quarter * 32, n0, half);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    stores_done(lane);
  }
  if (!ok) atomicExch(&dib_gemm_large_error_word, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
}

// ---------------------------------------------------------------- two CTAs on one tile
// The same product with a pair of CTAs (a cluster of two, on the two SMs of a TPC) on a tile
// of 256 tokens x BNL features: tcgen05.mma.cta_group::2 (M 256, N BNL, K 16), issued by the
// pair's first CTA alone, reads each CTA's own 128 token rows and HALF of the weight rows
// from each CTA's shared memory and accumulates each CTA's 128 x BNL tile in that CTA's
// tensor memory.  A CTA so fetches 16 KB of tokens and 16 KB (BNL 256) of weights per k-block
// instead of 16 + 32 KB: the rate at which L2 feeds the SMs bounds these products, not
// the tensor cores.  GATED: the first CTA fetches the 128 gate rows, the second the 128 up rows.
//
// Protocol, per stage s of the ring (same offsets in both CTAs):
//   full[s]    of the FIRST CTA counts the bytes of both CTAs' loads (its producer expects
//              them all; the second CTA's copies signal it through cp.async.bulk.tensor
//              .cta_group::2);
//   empty[s]   in each CTA, signalled by the first CTA's tcgen05.commit (multicast to both);
//   acc_full[b] likewise; acc_empty[b] of the first CTA takes one arrival per epilogue warp
//              of both CTAs (the second CTA's arrive remotely).
// The pair synchronises as a cluster after the set-up and before tensor memory is freed.
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of `local` in the CTA of rank `rank`
__device__ __forceinline__ unsigned cluster_addr(unsigned local, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
// a TMA load into this CTA's shared memory whose bytes are counted by the barrier at
// `bar_cluster_address`, which may be the other CTA's of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1,
                                                 unsigned bar_cluster_address) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar_cluster_address),
      "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(unsigned long long* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((unsigned short)3)
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned tmem_d, unsigned long long desc_a,
                                            unsigned long long desc_b, unsigned idesc, unsigned accum) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accum)
      : "memory");
}

template <int BNL, bool QKV = false> struct PairTile {
  static constexpr int B_BYTES = (BNL / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // per CTA
  static constexpr int STAGES = QKV ? 5 : 6;
  static constexpr int EPI_BYTES = EPI_WARPS * 4096 * (QKV ? 2 : 1);
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
};

template <typename OutT, bool GATED, int BNL, bool QKV = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, int M, int N, int K, int m_tiles, int n_tiles,
                 const __grid_constant__ QkvEpilogue qk) {
  static_assert(!GATED || BNL == 256, "the gated epilogue pairs 128 gate rows with 128 up rows");
  using TL = PairTile<BNL, QKV>;
  constexpr int STAGE_BYTES = TL::STAGE_BYTES, STAGES = TL::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* epi_stage = smem + STAGES * STAGE_BYTES;      // 4 KB to each epilogue warp
  unsigned long long* full = reinterpret_cast<unsigned long long*>(epi_stage + TL::EPI_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;     // [2]
  unsigned long long* acc_empty = acc_full + 2;      // [2]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_out);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_rank();              // 0: the CTA that issues the products
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int num_kb = (K + BK - 1) / BK;
  const int tiles = m_tiles * n_tiles;               // tiles of 256 tokens x BNL features
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // both CTAs' barriers and tensor memory exist before either is used
  tc_fence_after();
  const unsigned tmem = *tmem_slot;
  bool ok = true;

  if (warp < EPI_WARP0) {
    if (QKV) regs_give<REGS_FEW>();
    if (warp == 0) {
      if (lane == 0) {
        // ---- TMA producer of this CTA's halves.  Load number c is k-block c % num_kb of the
        // pair's tile number c / num_kb and goes to stage c % STAGES.
        const int my_tiles = tiles > pair ? (tiles - pair + pairs - 1) / pairs : 0;
        const int total = my_tiles * num_kb;
        const unsigned full0 = cluster_addr(smem_u32(full), 0);   // the first CTA's full[0], as a cluster address
        auto load_w = [&](int c) {
          const int t = pair + (c / num_kb) * pairs, kb = c % num_kb;
          const int n0 = (t / m_tiles) * (GATED ? BNL / 2 : BNL);
          const int row = GATED ? (rank ? N + n0 : n0) : n0 + (int)rank * (BNL / 2);
          tma_load_2d_pair(smem + (c % STAGES) * STAGE_BYTES + A_BYTES, &map_w, kb * BK, row, full0 + (c % STAGES) * 8);
        };
        auto load_x = [&](int c) {
          const int t = pair + (c / num_kb) * pairs, kb = c % num_kb;
          tma_load_2d_pair(smem + (c % STAGES) * STAGE_BYTES, &map_x, kb * BK,
                           (t % m_tiles) * 2 * BM + (int)rank * BM, full0 + (c % STAGES) * 8);
        };
        const int pre = total < STAGES ? total : STAGES;
        for (int c = 0; c < pre; ++c) {
          if (rank == 0) mbar_expect_tx(&full[c], 2 * STAGE_BYTES);
          load_w(c);
        }
        pdl_wait();
        for (int c = 0; c < pre; ++c) load_x(c);
        for (int c = pre; c < total && ok; ++c) {
          ok = mbar_wait(&empty[c % STAGES], ((c / STAGES) - 1) & 1);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(&full[c % STAGES], 2 * STAGE_BYTES);
          load_w(c);
          load_x(c);
        }
      }
    } else if (warp == 1) {
      if (lane == 0 && rank == 0) {
        // ---- MMA issuer of the pair
        constexpr unsigned idesc = make_idesc(2 * BM, BNL);
        int count = 0, local = 0;
        for (int t = pair; t < tiles && ok; t += pairs, ++local) {
          const int buf = local & 1;
          if (local >= 2) {     // both CTAs' epilogues must have read this buffer's earlier tile
            ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1);
            if (!ok) break;
            tc_fence_after();
          }
          for (int kb = 0; kb < num_kb && ok; ++kb, ++count) {
            const int s = count % STAGES;
            ok = mbar_wait(&full[s], (count / STAGES) & 1);
            if (!ok) break;
            tc_fence_after();
            const unsigned a = smem_u32(smem + s * STAGE_BYTES), b = a + A_BYTES;
  #pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              tc_mma_pair(tmem + buf * BNL, smem_desc_sw128(a + k * UMMA_K * 2),
                          smem_desc_sw128(b + k * UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            tc_commit_pair(&empty[s]);
          }
          if (ok) tc_commit_pair(&acc_full[buf]);
        }
      }
    }
  } else {
    if (QKV) regs_take<REGS_MANY>();
    // ---- epilogue of this CTA's 128 token rows
    pdl_wait();
    const int quarter = warp & 3, half = (warp - EPI_WARP0) >> 2;
    const unsigned lane_base = (unsigned)(quarter * 32) << 16;
    const unsigned acc_empty0 = cluster_addr(smem_u32(acc_empty), 0);   // the first CTA's acc_empty[0]
    int local = 0;
    for (int t = pair; t < tiles; t += pairs, ++local) {
      const int buf = local & 1;
      const int m0 = (t % m_tiles) * 2 * BM + (int)rank * BM, n0 = (t / m_tiles) * (GATED ? BNL / 2 : BNL);
      QkvRows rows;
      if (QKV) qkv_rows_prepare(rows, lane, m0 + quarter * 32, n0, half, qk);
      bool got = ok && mbar_wait(&acc_full[buf], (local >> 1) & 1);
      got = __all_sync(0xffffffffu, got);     // tcgen05.ld below is warp-wide
      if (!got) { ok = false; break; }
      tc_fence_after();
      if (QKV)
        store_rows_qkv(tmem + buf * BNL + lane_base, epi_stage + (warp - EPI_WARP0) * 2 * EPI_STAGE_BYTES, lane, half, qk, rows,
                       &map_out, m0 + quarter * 32);
      else
        store_rows<OutT, GATED, BNL>(tmem + buf * BNL + lane_base, &map_out, epi_stage + (warp - EPI_WARP0) * EPI_STAGE_BYTES,
                                     lane, m0 + quarter * 32, n0, half);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + buf * 8);
    }
    stores_done(lane);
  }
  if (!ok) atomicExch(&dib_gemm_large_error_word, 1);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // the other CTA's products and arrivals may still touch this one
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
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

// Row-major bf16 matrix [rows, K], boxes of box_rows x 64 elements, 128-byte swizzle;
// out-of-range elements read as zero.
bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The output [M, N] (bfloat16 or float32), boxes of 32 rows x 128 bytes, 128-byte swizzle; a
// store clips what lies beyond the matrix.
template <typename OutT>
bool make_out_map(CUtensorMap* map, void* ptr, long long M, long long N) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)N * sizeof(OutT)};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / sizeof(OutT)), 32};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, sizeof(OutT) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr,
             dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// (QKV: `out` is the q rows [M, out_cols]; the k and v rows go where `qk` says)
template <typename OutT, bool GATED, int BNL, bool QKV = false>
int launch_large(const void* x, const void* w, void* out, int M, int N, int K, int sm_count,
                 cudaStream_t st, const QkvEpilogue& qk = QkvEpilogue{}) {
  CUtensorMap mx, mw, mo;
  if (!make_map(&mx, x, M, K, BM) || !make_map(&mw, w, GATED ? 2ll * N : (long long)N, K, GATED ? BNL / 2 : 128) ||
      !make_out_map<OutT>(&mo, out, M, QKV ? (long long)qk.Hq * 128 : (long long)N))
    return DIB_LAUNCH_FAILED;
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + (GATED ? BNL / 2 : BNL) - 1) / (GATED ? BNL / 2 : BNL);
  const long long tiles = (long long)m_tiles * n_tiles;
  if (tiles > (1ll << 30)) return DIB_BAD_SIZE;
  auto kern = gemm_large_kernel<OutT, GATED, BNL, QKV>;
  constexpr size_t SMEM_BYTES = Tile<BNL, QKV>::SMEM_BYTES;
  static DeviceOnce attr_set;
  if (!attr_set.done()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  const int grid = (int)(tiles < sm_count ? tiles : sm_count);
  dib_launch(kern, dim3(grid), dim3(THREADS), SMEM_BYTES, st, mx, mw, mo, M, N, K, m_tiles, n_tiles, qk);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

template <typename OutT, bool GATED, int BNL, bool QKV = false>
int launch_pair(const void* x, const void* w, void* out, int M, int N, int K, int sm_count,
                cudaStream_t st, const QkvEpilogue& qk = QkvEpilogue{}) {
  CUtensorMap mx, mw, mo;
  if (!make_map(&mx, x, M, K, BM) || !make_map(&mw, w, GATED ? 2ll * N : (long long)N, K, BNL / 2) ||
      !make_out_map<OutT>(&mo, out, M, QKV ? (long long)qk.Hq * 128 : (long long)N))
    return DIB_LAUNCH_FAILED;
  const int m_tiles = (M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = (N + (GATED ? BNL / 2 : BNL) - 1) / (GATED ? BNL / 2 : BNL);
  const long long tiles = (long long)m_tiles * n_tiles;
  if (tiles > (1ll << 30) || sm_count < 2) return DIB_BAD_SIZE;
  auto kern = gemm_pair_kernel<OutT, GATED, BNL, QKV>;
  constexpr size_t SMEM_BYTES = PairTile<BNL, QKV>::SMEM_BYTES;
  static DeviceOnce attr_set;
  if (!attr_set.done()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_set.mark();
  }
  const int pairs = (int)(tiles < sm_count / 2 ? tiles : sm_count / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dib_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kern, mx, mw, mo, M, N, K, m_tiles, n_tiles, qk);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// Tile shape forced for measurements and tests (-1: the choice of tile_shape): 0: 128 x 128,
// 1: 128 x 256 by one CTA; 2: 256 x 256 by a pair of CTAs.
int& forced_shape() {
  static int v = -1;
  return v;
}
// A function of the sizes and the SM count alone (the order in which a row's k is added up
// is the same for all three, so the choice never changes a bit of the result).  The pair of
// CTAs where its tiles of 256 x 256 keep two thirds of the SMs busy or more; else tiles of
// 128 x 256, or of 128 x 128 where twice as many tiles still get an SM each (two rounds of
// half tiles are no shorter than one round of whole ones).
int tile_shape(int M, int n_rows, int sm_count) {
  if (forced_shape() >= 0) return forced_shape();
  const long long pair_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((n_rows + 255) / 256);
  if (sm_count >= 2 && 3 * pair_tiles >= sm_count) return 2;
  const long long tiles256 = (long long)((M + BM - 1) / BM) * ((n_rows + 255) / 256);
  return 2 * tiles256 <= sm_count && n_rows > 128 ? 0 : 1;
}

}  // namespace

extern "C" {

void dib_gemm_bf16_large_force_shape(int shape) { forced_shape() = shape; }

int dib_gemm_bf16_large_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, dib_gemm_large_error_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
int dib_gemm_bf16_large_status_clear() {
  const int v = 0;
  return cudaMemcpyToSymbol(dib_gemm_large_error_word, &v, sizeof(int)) == cudaSuccess ? 0 : -1;
}

// out[M, N] = x[M, K] * w[N, K]^T; bf16 inputs, float32 accumulation over k in one pass;
// out bf16 (out_fp32 = 0) or float32.  K a multiple of 8 and N of 8 (bf16 output) or 4
// (float32) (TMA wants 16-byte row strides); x, w and out 16-byte aligned.
int dib_gemm_bf16_large(const void* x, const void* w, void* out, int M, int N, int K, int out_fp32,
                        int sm_count, cudaStream_t st) {
  if (M == 0 || N == 0) return DIB_OK;
  if (K < 8 || K % 8 != 0 || sm_count < 1 || N % (out_fp32 ? 4 : 8) != 0) return DIB_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
    return DIB_BAD_ALIGN;
  const int shape = tile_shape(M, N, sm_count);
  if (out_fp32) {
    if (shape == 2) return launch_pair<float, false, 256>(x, w, out, M, N, K, sm_count, st);
    if (shape == 0) return launch_large<float, false, 128>(x, w, out, M, N, K, sm_count, st);
    return launch_large<float, false, 256>(x, w, out, M, N, K, sm_count, st);
  }
  if (shape == 2) return launch_pair<__nv_bfloat16, false, 256>(x, w, out, M, N, K, sm_count, st);
  if (shape == 0) return launch_large<__nv_bfloat16, false, 128>(x, w, out, M, N, K, sm_count, st);
  return launch_large<__nv_bfloat16, false, 256>(x, w, out, M, N, K, sm_count, st);
}

// out[M, I] = silu(x w_gate^T) * (x w_up^T) with w = [w_gate ; w_up] of shape [2I, K]; bf16 in
// and out.  I a multiple of 8, K of 8.
int dib_gemm_bf16_large_gated(const void* x, const void* w, void* out, int M, int I, int K,
                              int sm_count, cudaStream_t st) {
  if (M == 0 || I == 0) return DIB_OK;
  if (K < 8 || K % 8 != 0 || I % 8 != 0 || sm_count < 1) return DIB_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
    return DIB_BAD_ALIGN;
  const int shape = tile_shape(M, 2 * I, sm_count);
  if (shape == 2) return launch_pair<__nv_bfloat16, true, 256>(x, w, out, M, I, K, sm_count, st);
  if (shape == 0) return launch_large<__nv_bfloat16, true, 128>(x, w, out, M, I, K, sm_count, st);
  return launch_large<__nv_bfloat16, true, 256>(x, w, out, M, I, K, sm_count, st);
}

// The fused q/k/v projection of a prompt portion: x [M, K] times w [(Hq + 2 Hkv) * 128, K]^T,
// each head's row rounded to bfloat16, q and k normed (weights [128], or null) and rotated
// (table [max_pos, 128] rows cos | sin, or null) as by dib_qk_norm_rope_cache; q rows to q_out
// [M, Hq, 128], k and v rows to the tokens' cache slots (cache null: not written).  Heads of
// 128 only; K a multiple of 8; pointers 16-byte aligned.
int dib_gemm_bf16_large_qkv(const void* x, const void* w, void* q_out, int M, int K, int Hq, int Hkv,
                            const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_sin,
                            int max_pos, const int* positions, const int* slot_mapping, void* cache,
                            long long num_pages, int page_size, int sm_count, cudaStream_t st) {
  if (M == 0) return DIB_OK;
  const int N = (Hq + 2 * Hkv) * 128;
  if (K < 8 || K % 8 != 0 || sm_count < 1 || Hq < 1 || Hkv < 1 || page_size < 1) return DIB_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(q_out) |
       reinterpret_cast<uintptr_t>(cache)) % 16 != 0)
    return DIB_BAD_ALIGN;
  QkvEpilogue qk = {};
  qk.q_norm_w = q_norm_w; qk.k_norm_w = k_norm_w; qk.eps = eps; qk.cos_sin = cos_sin; qk.max_pos = max_pos;
  qk.positions = positions; qk.slot_mapping = slot_mapping; qk.cache = (__nv_bfloat16*)cache;
  qk.q_out = (__nv_bfloat16*)q_out;
  qk.num_pages = num_pages; qk.page_size = page_size; qk.Hq = Hq; qk.Hkv = Hkv; qk.M = M;
  // (tiles of one head where tiles of two would be fewer than the SMs: a prompt portion of up to
  // about a thousand tokens)
  const int shape = tile_shape(M, N, sm_count);
  if (shape == 2) return launch_pair<__nv_bfloat16, false, 256, true>(x, w, q_out, M, N, K, sm_count, st, qk);
  if (shape == 0) return launch_large<__nv_bfloat16, false, 128, true>(x, w, q_out, M, N, K, sm_count, st, qk);
  return launch_large<__nv_bfloat16, false, 256, true>(x, w, q_out, M, N, K, sm_count, st, qk);
}

}  // extern "C"
