// Row-wise and element-wise kernels: embedding gather, RMSNorm, fused
// residual-add + RMSNorm, per-head q/k RMSNorm fused with rotary position
// encoding and the write into the paged cache, SiLU-gate, row gather.
//
// All arithmetic is float32; storage is float32 or bfloat16 (template T).  Norm
// weights and the rotary table are always float32.
//
// Paged cache layout of one layer: [num_pages, 2 (key,value), num_kv_heads,
// page_size, head_dim], so the keys (or values) of one head inside one page are
// contiguous.
#include <cstdlib>

#include "common.cuh"

namespace {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 T* __restrict__ out, int H, int V) {
  pdl_prologue(ids);
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;
  const T* src = table + (size_t)(ok ? id : 0) * H;
  T* dst = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    if (ok) dst[i] = src[i];
    else Elem<T>::store(dst + i, 0.f);
  }
}

// Rows copied 16 bytes a thread: out row r = src row idx[r] (rows of row_bytes, a multiple
// of 16; an index outside [0, rows_in) gives zeros if zero_bad, else is clamped).
__global__ void copy_rows16_kernel(const uint4* __restrict__ src, const int* __restrict__ idx,
                                   uint4* __restrict__ out, int vecs, int rows_in, int zero_bad) {
  pdl_prologue(src, idx);
  const int r = blockIdx.x;
  int id = idx[r];
  const bool bad = id < 0 || id >= rows_in;
  if (bad) id = id < 0 ? 0 : rows_in - 1;
  const uint4* s = src + (size_t)id * vecs;
  uint4* d = out + (size_t)r * vecs;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x)
    d[i] = (bad && zero_bad) ? make_uint4(0, 0, 0, 0) : s[i];
}

// ---------------------------------------------------------------- RMSNorm
// y = x * 1/sqrt(mean(x^2) + eps) * w; one block per row; the row is staged in
// shared memory as float32.  With ADD: residual += x first (stored rounded to T),
// and the norm reads the unrounded float32 sum; y overwrites x.  This form serves row
// widths the vector kernels do not take (not a multiple of the vector width); which form a
// width gets never depends on the number of rows.
template <typename T, bool ADD>
__global__ void rms_norm_kernel(T* __restrict__ x, T* __restrict__ residual,
                                const float* __restrict__ w, T* __restrict__ out,
                                int H, float eps) {
  pdl_prologue(x, residual);
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = Elem<T>::load(x + base + i);
    if (ADD) {
      v += Elem<T>::load(residual + base + i);
      Elem<T>::store(residual + base + i, v);
    }
    row[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rms_rstd(total, H, eps);
  T* dst = ADD ? x : out;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    Elem<T>::store(dst + base + i, norm_scale(row[i], rstd, w[i]));
  }
}

// Vector path of the same kernel: 16-byte loads, the row kept in registers.  Used
// when the row width is a multiple of the vector width and fits ITERS passes.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 x;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = x;
  }
};

template <typename T, bool ADD, int ITERS>
__global__ void rms_norm_vec_kernel(T* __restrict__ x, T* __restrict__ residual,
                                    const float* __restrict__ w, T* __restrict__ out, int H,
                                    float eps) {
  pdl_prologue(x, residual);
  constexpr int N = Vec<T>::N, VPT = N / 4;
  __shared__ float scratch[256];   // groups of 128 elements: at most 4096 vectors of N
  const size_t base = (size_t)blockIdx.x * H;
  float v[ITERS][N];
  float ss[ITERS][VPT];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * N;
#pragma unroll
    for (int k = 0; k < VPT; ++k) ss[it][k] = 0.f;
    if (i < H) {
      Vec<T>::load(x + base + i, v[it]);
      if (ADD) {
        float r[N];
        Vec<T>::load(residual + base + i, r);
#pragma unroll
        for (int k = 0; k < N; ++k) v[it][k] = __fadd_rn(v[it][k], r[k]);
        Vec<T>::store(residual + base + i, v[it]);
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k)
        ss[it][k] = sumsq4(v[it][4 * k], v[it][4 * k + 1], v[it][4 * k + 2], v[it][4 * k + 3]);
    }
  }
  const float total = sumsq_row<ITERS, VPT>(ss, H / 4, scratch);
  const float rstd = rms_rstd(total, H, eps);
  T* dst = ADD ? x : out;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * N;
    if (i < H) {
      float y[N];
#pragma unroll
      for (int k = 0; k < N; k += 4) {
        const float4 ww = *reinterpret_cast<const float4*>(w + i + k);
        y[k] = norm_scale(v[it][k], rstd, ww.x);
        y[k + 1] = norm_scale(v[it][k + 1], rstd, ww.y);
        y[k + 2] = norm_scale(v[it][k + 2], rstd, ww.z);
        y[k + 3] = norm_scale(v[it][k + 3], rstd, ww.w);
      }
      Vec<T>::store(dst + base + i, y);
    }
  }
}

// ------------------------------------------- q/k norm + rotary + cache write
// One warp per (token, head) of the fused qkv row.  Heads 0..Hq-1 are queries
// (written to q_out), then Hkv key heads, then Hkv value heads (written to the
// cache page slot of the token).  Norm is applied when its weight pointer is
// non-null, the rotation when the table pointer is non-null; the rotation is
// rotate-half over the first rotary_dim dims: (x[d], x[d+r/2]) rotated by
// angle(pos, d) with the table row [cos(r/2) | sin(r/2)].
template <typename T>
__global__ void qk_norm_rope_cache_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ kv_cache,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ cos_sin, int rotary_dim, int max_pos,
    const int* __restrict__ positions, const int* __restrict__ slot_mapping,
    int T_tokens, int Hq, int Hkv, int D, int page_size, long long num_pages) {
  pdl_prologue(qkv, positions, slot_mapping);
  extern __shared__ float smem[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)T_tokens * heads) return;
  const int t = (int)(item / heads);
  const int head = (int)(item % heads);
  float* s = smem + (size_t)warp * D;

  const T* src = qkv + ((size_t)t * heads + head) * D;
  const bool is_q = head < Hq;
  const bool is_k = !is_q && head < Hq + Hkv;
  const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);

  // destination
  T* dst = nullptr;
  if (is_q) {
    dst = q_out + ((size_t)t * Hq + head) * D;
  } else {
    if (kv_cache == nullptr) return;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const long long page = slot / page_size;
    if (page >= num_pages) return;
    const int off = slot % page_size;
    const int kv = is_k ? 0 : 1;
    const int h = is_k ? head - Hq : head - Hq - Hkv;
    dst = kv_cache + ((((size_t)page * 2 + kv) * Hkv + h) * page_size + off) * D;
  }

  float ss = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float v = Elem<T>::load(src + d);
    s[d] = v;
    ss += v * v;
  }
  if (nw != nullptr) {
    ss = warp_sum(ss);
    const float rstd = rms_rstd(ss, D, eps);
    __syncwarp();
    for (int d = lane; d < D; d += 32) s[d] = norm_scale(s[d], rstd, nw[d]);
  }
  __syncwarp();

  const bool rotate = (cos_sin != nullptr) && (is_q || is_k);
  if (rotate) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* tab = cos_sin + (size_t)pos * rotary_dim;
    const int half = rotary_dim >> 1;
    for (int d = lane; d < half; d += 32) {
      const float c = tab[d], sn = tab[half + d];
      const float x1 = s[d], x2 = s[d + half];
      Elem<T>::store(dst + d, rope_first(x1, x2, c, sn));
      Elem<T>::store(dst + d + half, rope_second(x1, x2, c, sn));
    }
    for (int d = rotary_dim + lane; d < D; d += 32) Elem<T>::store(dst + d, s[d]);
  } else {
    for (int d = lane; d < D; d += 32) Elem<T>::store(dst + d, s[d]);
  }
}

// Vector path of the kernel above for head sizes that are multiples of 64 with a
// rotation over the whole head (or none): each lane owns EPL = D/32 contiguous
// elements, so the partner of a rotation pair (d, d + D/2) sits in lane ^ 16 and
// nothing goes through shared memory.
template <typename T, int EPL>
struct alignas((sizeof(T) * EPL) <= 16 ? (sizeof(T) * EPL) : 16) Pack {
  T e[EPL];
};

template <typename T, int EPL, int ITEMS>
__global__ void qk_norm_rope_cache_vec_kernel(
    const T* __restrict__ qkv, const float* __restrict__ parts, int S, long long split_stride,
    T* __restrict__ q_out, T* __restrict__ kv_cache,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ cos_sin, int max_pos, const int* __restrict__ positions,
    const int* __restrict__ slot_mapping, int T_tokens, int Hq, int Hkv, int page_size,
    long long num_pages) {
  pdl_prologue(qkv, parts, positions, slot_mapping);
  constexpr int D = EPL * 32;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  const long long total = (long long)T_tokens * heads;
  const long long item0 = ((long long)blockIdx.x * warps_per_block + warp) * ITEMS;
  if (item0 >= total) return;

  // A warp takes ITEMS consecutive (token, head) items and issues the loads of all of
  // them before it works on any, so their memory round-trips overlap.
  float v[ITEMS][EPL];
  int tok[ITEMS], head[ITEMS], pos[ITEMS], slot[ITEMS];
  bool act[ITEMS];
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const long long item = item0 + it;
    act[it] = item < total;
    tok[it] = act[it] ? (int)(item / heads) : 0;
    head[it] = act[it] ? (int)(item % heads) : 0;
    pos[it] = 0;
    slot[it] = -1;
    if (!act[it]) continue;
    if (parts == nullptr) {
      const T* src = qkv + ((size_t)tok[it] * heads + head[it]) * D + lane * EPL;
      const Pack<T, EPL> in = *reinterpret_cast<const Pack<T, EPL>*>(src);
#pragma unroll
      for (int k = 0; k < EPL; ++k) v[it][k] = Elem<T>::load(&in.e[k]);
    } else {
      // the row is a sum of split-k partial products, added in split order and rounded
      // to T as a stored projection output would be
      const float* src = parts + ((size_t)tok[it] * heads + head[it]) * D + lane * EPL;
#pragma unroll
      for (int k = 0; k < EPL; ++k) v[it][k] = 0.f;
      // up to 8 splits' loads go out together, then the sums in split order
      for (int sp0 = 0; sp0 < S; sp0 += 8) {
        Pack<float, EPL> in[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (sp0 + j < S)
            in[j] = *reinterpret_cast<const Pack<float, EPL>*>(src + (sp0 + j) * split_stride);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (sp0 + j < S) {
#pragma unroll
            for (int k = 0; k < EPL; ++k) v[it][k] += in[j].e[k];
          }
        }
      }
#pragma unroll
      for (int k = 0; k < EPL; ++k) v[it][k] = round_to<T>(v[it][k]);
    }
    if (cos_sin != nullptr && head[it] < Hq + Hkv) {
      const int p = positions[tok[it]];
      pos[it] = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    }
    if (head[it] >= Hq && kv_cache != nullptr) slot[it] = slot_mapping[tok[it]];
  }

#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    if (!act[it]) continue;
    const bool is_q = head[it] < Hq;
    const bool is_k = !is_q && head[it] < Hq + Hkv;
    const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    T* dst = nullptr;
    if (is_q) {
      dst = q_out + ((size_t)tok[it] * Hq + head[it]) * D;
    } else {
      if (slot[it] < 0) continue;
      const long long page = slot[it] / page_size;
      if (page >= num_pages) continue;
      const int off = slot[it] % page_size;
      const int kv = is_k ? 0 : 1;
      const int h = is_k ? head[it] - Hq : head[it] - Hq - Hkv;
      dst = kv_cache + ((((size_t)page * 2 + kv) * Hkv + h) * page_size + off) * D;
    }
    if (nw != nullptr) {
      // a lane's EPL consecutive elements as a chain of fused multiply-adds, the lanes by
      // the butterfly: for heads of 128 (EPL 4) this is the order of a row's norm statistic
      float ss = __fmul_rn(v[it][0], v[it][0]);
#pragma unroll
      for (int k = 1; k < EPL; ++k) ss = __fmaf_rn(v[it][k], v[it][k], ss);
      const float one[1] = {ss};
      ss = sumsq_group<1>(one);
      const float rstd = rms_rstd(ss, D, eps);
#pragma unroll
      for (int k = 0; k < EPL; ++k) v[it][k] = norm_scale(v[it][k], rstd, nw[lane * EPL + k]);
    }
    if (cos_sin != nullptr && (is_q || is_k)) {
      const float* tab = cos_sin + (size_t)pos[it] * D;
      const int j0 = (lane & 15) * EPL;
      const bool upper = lane >= 16;
#pragma unroll
      for (int k = 0; k < EPL; ++k) {
        const float partner = __shfl_xor_sync(0xffffffffu, v[it][k], 16);
        const float c = tab[j0 + k], sn = tab[D / 2 + j0 + k];
        v[it][k] = upper ? rope_second(partner, v[it][k], c, sn) : rope_first(v[it][k], partner, c, sn);
      }
    }
    Pack<T, EPL> o;
#pragma unroll
    for (int k = 0; k < EPL; ++k) Elem<T>::store(&o.e[k], v[it][k]);
    *reinterpret_cast<Pack<T, EPL>*>(dst + lane * EPL) = o;
  }
}

// The same for many rows of bfloat16 heads of 128 with a full rotation (prompt
// portions): eight lanes share a (token, head) row, each with the elements 8l..8l+7 and
// 64+8l..64+8l+7, so a rotation pair lies in one lane (no exchange), every load and
// store moves 16 bytes, and a warp has four rows in flight; each group of eight lanes
// takes ROWS rows and issues all their loads first.
template <int ROWS>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_rows128_kernel(
    const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
    __nv_bfloat16* __restrict__ kv_cache, const float* __restrict__ q_norm_w,
    const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_sin, int max_pos,
    const int* __restrict__ positions, const int* __restrict__ slot_mapping, int T_tokens, int Hq,
    int Hkv, int page_size, long long num_pages) {
  pdl_prologue(qkv, positions, slot_mapping);
  constexpr int D = 128;
  const int heads = Hq + 2 * Hkv;
  const int total = T_tokens * heads;            // the launcher keeps this below 2^31
  const int l = threadIdx.x & 7;
  const int group = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3);
  const int row0 = group * ROWS;
  const unsigned mask = 0xffu << (threadIdx.x & 24);   // the eight lanes of this group

  // Three rounds of loads, each issued for all ROWS rows before anything waits for them:
  // the row itself with its token's position and slot; the rotation table's row; then
  // the arithmetic and the stores.
  uint4 lo[ROWS], hi[ROWS];
  int tok[ROWS], head[ROWS], pos[ROWS], slot[ROWS];
  bool act[ROWS];
#pragma unroll
  for (int it = 0; it < ROWS; ++it) {
    const int row = row0 + it;
    act[it] = row < total;
    tok[it] = act[it] ? row / heads : 0;
    head[it] = act[it] ? row - tok[it] * heads : 0;
    pos[it] = 0;
    slot[it] = -1;
    if (act[it]) {
      const __nv_bfloat16* src = qkv + ((size_t)tok[it] * heads + head[it]) * D + l * 8;
      lo[it] = *reinterpret_cast<const uint4*>(src);
      hi[it] = *reinterpret_cast<const uint4*>(src + 64);
      if (head[it] < Hq + Hkv && cos_sin != nullptr) pos[it] = positions[tok[it]];
      if (head[it] >= Hq && kv_cache != nullptr) slot[it] = slot_mapping[tok[it]];
    }
  }
  float4 c0[ROWS], c1[ROWS], s0[ROWS], s1[ROWS];
#pragma unroll
  for (int it = 0; it < ROWS; ++it) {
    if (act[it] && head[it] < Hq + Hkv && cos_sin != nullptr) {
      const int p = pos[it] < 0 ? 0 : (pos[it] >= max_pos ? max_pos - 1 : pos[it]);
      const float* tab = cos_sin + (size_t)p * D + l * 8;
      c0[it] = *reinterpret_cast<const float4*>(tab);
      c1[it] = *reinterpret_cast<const float4*>(tab + 4);
      s0[it] = *reinterpret_cast<const float4*>(tab + 64);
      s1[it] = *reinterpret_cast<const float4*>(tab + 68);
    }
  }
#pragma unroll
  for (int it = 0; it < ROWS; ++it) {
    if (!act[it]) continue;   // uniform over the group
    const bool is_q = head[it] < Hq;
    const bool is_k = !is_q && head[it] < Hq + Hkv;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = q_out + ((size_t)tok[it] * Hq + head[it]) * D;
    } else {
      if (slot[it] < 0) continue;
      const int page = slot[it] / page_size;
      if (page >= num_pages) continue;
      const int h = is_k ? head[it] - Hq : head[it] - Hq - Hkv;
      dst = kv_cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * Hkv + h) * page_size +
                        (slot[it] - page * page_size)) * D;
    }
    if (is_q || is_k) {
      const float c[8] = {c0[it].x, c0[it].y, c0[it].z, c0[it].w, c1[it].x, c1[it].y, c1[it].z, c1[it].w};
      const float sn[8] = {s0[it].x, s0[it].y, s0[it].z, s0[it].w, s1[it].x, s1[it].y, s1[it].z, s1[it].w};
      qk_row128(lo[it], hi[it], l, mask, is_q ? q_norm_w : k_norm_w, eps, cos_sin != nullptr, c, sn);
    }
    *reinterpret_cast<uint4*>(dst + l * 8) = lo[it];
    *reinterpret_cast<uint4*>(dst + 64 + l * 8) = hi[it];
  }
}

// ------------------------------------------------ standalone cache write
// k, v: [T, Hkv, D] -> the page slot of each token (slot < 0: skipped).
template <typename T>
__global__ void reshape_and_cache_kernel(const T* __restrict__ k, const T* __restrict__ v,
                                         T* __restrict__ kv_cache,
                                         const int* __restrict__ slot_mapping, int Hkv, int D,
                                         int page_size, long long num_pages) {
  pdl_prologue(k, v, slot_mapping);
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const long long page = slot / page_size;
  if (page >= num_pages) return;
  const int off = slot % page_size;
  for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
    const int h = i / D, d = i % D;
    const size_t kd = ((((size_t)page * 2 + 0) * Hkv + h) * page_size + off) * D + d;
    const size_t vd = ((((size_t)page * 2 + 1) * Hkv + h) * page_size + off) * D + d;
    kv_cache[kd] = k[(size_t)t * Hkv * D + i];
    kv_cache[vd] = v[(size_t)t * Hkv * D + i];
  }
}

// ---------------------------------------------------------------- SiLU gate
// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z)).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total,
                                int I) {
  pdl_prologue(gu);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / I;
  const int i = (int)(idx % I);
  const float g = Elem<T>::load(gu + t * 2 * I + i);
  const float u = Elem<T>::load(gu + t * 2 * I + I + i);
  Elem<T>::store(out + idx, silu_gate<T>(g, u));
}

// blockIdx.x names ROWS consecutive tokens, blockIdx.y and the thread a vector of the row
// (no division); a thread sends for its vectors of all ROWS tokens before it computes.
template <typename T, int ROWS>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int T_rows,
                                    int I) {
  pdl_prologue(gu);
  constexpr int N = Vec<T>::N;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * N;
  if (i >= I) return;
  const long long t0 = (long long)blockIdx.x * ROWS;
  float g[ROWS][N], u[ROWS][N];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
    if (t0 + r < T_rows) {
      Vec<T>::load(gu + (t0 + r) * 2 * I + i, g[r]);
      Vec<T>::load(gu + (t0 + r) * 2 * I + I + i, u[r]);
    }
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
    if (t0 + r < T_rows) {
      float y[N];
#pragma unroll
      for (int k = 0; k < N; ++k) y[k] = silu_gate<T>(g[r][k], u[r][k]);
      Vec<T>::store(out + (t0 + r) * I + i, y);
    }
}

// ------------------------------------------------ readers of split-k partials
// A matrix product with split k leaves `S` float32 partial products
// parts[s][row][col]; its readers add them in split order and round the sum to T,
// which is what reading a stored product would give.

template <typename T>
__global__ void sum_split_kernel(const float* __restrict__ parts, T* __restrict__ out,
                                 long long total4, long long split_stride, int S) {
  pdl_prologue(parts);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp = 0; sp < S; ++sp) {
    const float4 p = *reinterpret_cast<const float4*>(parts + sp * split_stride + i * 4);
    a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
  }
  Pack<T, 4> o;
  Elem<T>::store(&o.e[0], a.x);
  Elem<T>::store(&o.e[1], a.y);
  Elem<T>::store(&o.e[2], a.z);
  Elem<T>::store(&o.e[3], a.w);
  *reinterpret_cast<Pack<T, 4>*>(out + i * 4) = o;
}

// residual += x (stored rounded), out = rms_norm(unrounded sum), x given as partials.
template <typename T, int ITERS>
__global__ void __launch_bounds__(ITERS >= 4 ? 1024 : 512)
add_rms_norm_split_kernel(const float* __restrict__ parts, int S,
                                          long long split_stride, T* __restrict__ residual,
                                          const float* __restrict__ w, T* __restrict__ out, int H,
                                          float eps) {
  pdl_prologue(parts, residual);
  __shared__ float scratch[128];
  const size_t base = (size_t)blockIdx.x * H;
  float v[ITERS][4];
  float ss[ITERS][1];
  // The kernel is a chain of memory round-trips, so it makes few of them: the residual
  // and up to 16 partials of an element are requested together, then added in split order.
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    ss[it][0] = 0.f;
    if (i < H) {
      const Pack<T, 4> r = *reinterpret_cast<const Pack<T, 4>*>(residual + base + i);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      constexpr int BATCH = ITERS == 1 ? 16 : ITERS == 2 ? 8 : 4;   // what the block's registers hold
      for (int sp0 = 0; sp0 < S; sp0 += BATCH) {
        float4 p[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j)
          if (sp0 + j < S)
            p[j] = *reinterpret_cast<const float4*>(parts + (sp0 + j) * split_stride + base + i);
#pragma unroll
        for (int j = 0; j < BATCH; ++j)
          if (sp0 + j < S) { a.x += p[j].x; a.y += p[j].y; a.z += p[j].z; a.w += p[j].w; }
      }
      v[it][0] = __fadd_rn(round_to<T>(a.x), Elem<T>::load(&r.e[0]));
      v[it][1] = __fadd_rn(round_to<T>(a.y), Elem<T>::load(&r.e[1]));
      v[it][2] = __fadd_rn(round_to<T>(a.z), Elem<T>::load(&r.e[2]));
      v[it][3] = __fadd_rn(round_to<T>(a.w), Elem<T>::load(&r.e[3]));
      Pack<T, 4> o;
#pragma unroll
      for (int k = 0; k < 4; ++k) Elem<T>::store(&o.e[k], v[it][k]);
      ss[it][0] = sumsq4(v[it][0], v[it][1], v[it][2], v[it][3]);
      *reinterpret_cast<Pack<T, 4>*>(residual + base + i) = o;
    }
  }
  float4 ww[ITERS];     // requested before the reduction, used after it
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    ww[it] = i < H ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float total = sumsq_row<ITERS, 1>(ss, H / 4, scratch);
  const float rstd = rms_rstd(total, H, eps);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < H) {
      Pack<T, 4> o;
      Elem<T>::store(&o.e[0], norm_scale(v[it][0], rstd, ww[it].x));
      Elem<T>::store(&o.e[1], norm_scale(v[it][1], rstd, ww[it].y));
      Elem<T>::store(&o.e[2], norm_scale(v[it][2], rstd, ww[it].z));
      Elem<T>::store(&o.e[3], norm_scale(v[it][3], rstd, ww[it].w));
      *reinterpret_cast<Pack<T, 4>*>(out + base + i) = o;
    }
  }
}

template <typename T>
__global__ void silu_mul_split_kernel(const float* __restrict__ parts, int S, long long split_stride,
                                      T* __restrict__ out, long long vecs, int I) {
  pdl_prologue(parts);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= vecs) return;
  const int per_row = I / 4;
  const long long t = idx / per_row;
  const int i = (int)(idx % per_row) * 4;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
  // up to 8 splits' loads go out together (one memory round-trip), then the sums in split order
  for (int sp0 = 0; sp0 < S; sp0 += 8) {
    float4 a[8], b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (sp0 + j < S) {
        const float* row = parts + (sp0 + j) * split_stride + t * 2 * I;
        a[j] = *reinterpret_cast<const float4*>(row + i);
        b[j] = *reinterpret_cast<const float4*>(row + I + i);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (sp0 + j < S) {
        g.x += a[j].x; g.y += a[j].y; g.z += a[j].z; g.w += a[j].w;
        u.x += b[j].x; u.y += b[j].y; u.z += b[j].z; u.w += b[j].w;
      }
    }
  }
  const float gg[4] = {round_to<T>(g.x), round_to<T>(g.y), round_to<T>(g.z), round_to<T>(g.w)};
  const float uu[4] = {round_to<T>(u.x), round_to<T>(u.y), round_to<T>(u.z), round_to<T>(u.w)};
  Pack<T, 4> o;
#pragma unroll
  for (int k = 0; k < 4; ++k) Elem<T>::store(&o.e[k], silu_gate<T>(gg[k], uu[k]));
  *reinterpret_cast<Pack<T, 4>*>(out + t * I + i) = o;
}

// ------------------------------------------------ token hand-over on the device
// ids[dst[i]] = prev[src[i]] for every i with dst[i] >= 0: the tokens a step sampled
// become the next step's inputs without a trip to the host.
__global__ void patch_ids_kernel(int* __restrict__ ids, const int* __restrict__ dst,
                                 const int* __restrict__ src, const int* __restrict__ prev, int n,
                                 int num_ids, int num_prev) {
  pdl_prologue(dst, src, prev);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = dst[i], sidx = src[i];
  if (d >= 0 && d < num_ids && sidx >= 0 && sidx < num_prev) ids[d] = prev[sidx];
}

// ---------------------------------------------------------------- row gather
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ idx,
                                   T* __restrict__ out, int H, int T_rows) {
  pdl_prologue(x, idx);
  const int r = blockIdx.x;
  int src = idx[r];
  src = src < 0 ? 0 : (src >= T_rows ? T_rows - 1 : src);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)r * H + i] = x[(size_t)src * H + i];
}

int pick_threads(int n) {
  int t = 32;
  while (t < n && t < 1024) t <<= 1;
  return t;
}

template <typename T, bool ADD>
int launch_rms(void* x, void* res, const float* w, void* out, int rows, int H, float eps,
                      cudaStream_t st) {
  constexpr int N = Vec<T>::N;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                       (res == nullptr || reinterpret_cast<uintptr_t>(res) % 16 == 0) &&
                       (out == nullptr || reinterpret_cast<uintptr_t>(out) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(w) % 16 == 0);
  // few rows: a wide block (more loads in flight per row); many rows: 256 threads.  The
  // block's width changes who holds which elements, not the order of the row's sums.
  const int th_max = rows <= 64 ? 1024 : 256;
  if (H % N == 0 && aligned && H / N <= 4096) {   // at most 4 (16) vectors per thread
    const int vecs = H / N;
    int th = 32;
    while (th < vecs && th < th_max) th <<= 1;
    const int iters = (vecs + th - 1) / th;
#define DIB_RMS(IT) \
  dib_launch(rms_norm_vec_kernel<T, ADD, IT>, dim3(rows), dim3(th), 0, st, (T*)x, (T*)res, w, (T*)out, H, eps)
    if (iters == 1) DIB_RMS(1);
    else if (iters == 2) DIB_RMS(2);
    else if (iters <= 4) DIB_RMS(4);
    else if (iters <= 8) DIB_RMS(8);
    else DIB_RMS(16);
#undef DIB_RMS
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return DIB_BAD_SIZE;
  auto kern = rms_norm_kernel<T, ADD>;
  static size_t attr_smem = 0;  // raised when a wider row comes; never shrinks
  if (smem > 40 * 1024 && smem > attr_smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    attr_smem = smem;
  }
  int th = pick_threads(H);
  if (th > 512) th = 512;
  dib_launch(kern, dim3(rows), dim3(th), smem, st, (T*)x, (T*)res, w, (T*)out, H, eps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // namespace

extern "C" {

int dib_embedding(const void* table, const int* ids, void* out, int T, int H, int V, int dtype,
                  cudaStream_t st) {
  if (T == 0) return DIB_OK;
  const int th = pick_threads(H) > 256 ? 256 : pick_threads(H);
  const size_t row_bytes = (size_t)H * (dtype == 0 ? 4 : 2);
  if ((dtype == 0 || dtype == 1) && row_bytes % 16 == 0 && V > 0 &&
      (reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
    const int vecs = (int)(row_bytes / 16);
    dib_launch(copy_rows16_kernel, dim3(T), dim3(vecs < 256 ? pick_threads(vecs) : 256), 0, st,
               (const uint4*)table, ids, (uint4*)out, vecs, V, 1);
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  if (dtype == 0)
    dib_launch(embedding_kernel<float>, dim3(T), dim3(th), 0, st, (const float*)table, ids, (float*)out, H, V);
  else if (dtype == 1)
    dib_launch(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(th), 0, st, (const __nv_bfloat16*)table, ids,
                                                      (__nv_bfloat16*)out, H, V);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_rms_norm(const void* x, const float* w, void* out, int rows, int H, float eps, int dtype,
                 cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (dtype == 0) return launch_rms<float, false>((void*)x, nullptr, w, out, rows, H, eps, st);
  if (dtype == 1)
    return launch_rms<__nv_bfloat16, false>((void*)x, nullptr, w, out, rows, H, eps, st);
  return DIB_BAD_DTYPE;
}

int dib_add_rms_norm(void* x, void* residual, const float* w, int rows, int H, float eps,
                     int dtype, cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (dtype == 0) return launch_rms<float, true>(x, residual, w, nullptr, rows, H, eps, st);
  if (dtype == 1) return launch_rms<__nv_bfloat16, true>(x, residual, w, nullptr, rows, H, eps, st);
  return DIB_BAD_DTYPE;
}

int dib_qk_norm_rope_cache_split(const void* qkv, const float* parts, int S, long long split_stride,
                                 void* q_out, void* kv_cache, const float* q_norm_w,
                                 const float* k_norm_w, float eps, const float* cos_sin,
                                 int rotary_dim, int max_pos, const int* positions,
                                 const int* slot_mapping, int T, int Hq, int Hkv, int D,
                                 int page_size, long long num_pages, int dtype, cudaStream_t st);

int dib_qk_norm_rope_cache(const void* qkv, void* q_out, void* kv_cache, const float* q_norm_w,
                           const float* k_norm_w, float eps, const float* cos_sin, int rotary_dim,
                           int max_pos, const int* positions, const int* slot_mapping, int T,
                           int Hq, int Hkv, int D, int page_size, long long num_pages, int dtype,
                           cudaStream_t st) {
  return dib_qk_norm_rope_cache_split(qkv, nullptr, 0, 0, q_out, kv_cache, q_norm_w, k_norm_w, eps,
                                      cos_sin, rotary_dim, max_pos, positions, slot_mapping, T, Hq,
                                      Hkv, D, page_size, num_pages, dtype, st);
}

// With parts != nullptr the fused projection rows are sums of S split-k partials
// (float32 [S, T, (Hq+2Hkv)*D]); only head sizes 64, 128, 256 with a full rotation
// take that form (-2 otherwise: the caller sums the partials first).
int dib_qk_norm_rope_cache_split(const void* qkv, const float* parts, int S, long long split_stride,
                                 void* q_out, void* kv_cache, const float* q_norm_w,
                           const float* k_norm_w, float eps, const float* cos_sin, int rotary_dim,
                           int max_pos, const int* positions, const int* slot_mapping, int T,
                           int Hq, int Hkv, int D, int page_size, long long num_pages, int dtype,
                           cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (D < 2 || D > 1024 || (rotary_dim & 1) || rotary_dim > D) return DIB_BAD_SIZE;
  const int warps = 4;
  const long long items = (long long)T * (Hq + 2 * Hkv);
  const int blocks = ceil_div_host(items, warps);
  const bool aligned = reinterpret_cast<uintptr_t>(qkv) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(parts) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(q_out) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(kv_cache) % 16 == 0;
  if (aligned && parts == nullptr && dtype == 1 && D == 128 && (cos_sin == nullptr || rotary_dim == D) &&
      items >= 2048 && items < (1ll << 31) - 4096 &&
      reinterpret_cast<uintptr_t>(q_norm_w) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(k_norm_w) % 16 == 0 && reinterpret_cast<uintptr_t>(cos_sin) % 16 == 0) {
    // one row per group of eight lanes: with two, the registers of the second cost more
    // threads per multiprocessor than its loads in flight gain (12.2 us against 9.7 us for
    // 2,048 tokens of 16 + 2 x 8 heads)
    dib_launch(qk_norm_rope_cache_rows128_kernel<1>, dim3(ceil_div_host(items * 8, 256)), dim3(256),
               0, st, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_cache,
               q_norm_w, k_norm_w, eps, cos_sin, max_pos, positions, slot_mapping, T, Hq, Hkv,
               page_size, num_pages);
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  if (aligned && (D == 64 || D == 128 || D == 256) && (cos_sin == nullptr || rotary_dim == D) &&
      (dtype == 0 || dtype == 1)) {
    // many items: 4 per warp (their loads overlap); few items: one per warp
    const bool many = parts == nullptr && items >= 8192;
    const int vblocks = many ? ceil_div_host(items, warps * 4) : blocks;
#define DIB_QK_VEC(TT, EPL)                                                                      \
  if (many)                                                                                      \
    dib_launch(qk_norm_rope_cache_vec_kernel<TT, EPL, 4>, dim3(vblocks), dim3(warps * 32), 0, st, \
      (const TT*)qkv, parts, S, split_stride, (TT*)q_out, (TT*)kv_cache, q_norm_w, k_norm_w,   \
      eps, cos_sin, max_pos,                                                                    \
      positions, slot_mapping, T, Hq, Hkv, page_size, num_pages);                              \
  else                                                                                           \
  dib_launch(qk_norm_rope_cache_vec_kernel<TT, EPL, 1>, dim3(blocks), dim3(warps * 32), 0, st,                         \
      (const TT*)qkv, parts, S, split_stride, (TT*)q_out, (TT*)kv_cache, q_norm_w, k_norm_w,   \
      eps, cos_sin, max_pos,                                                                    \
      positions, slot_mapping, T, Hq, Hkv, page_size, num_pages)
    if (dtype == 0) {
      if (D == 64) DIB_QK_VEC(float, 2);
      else if (D == 128) DIB_QK_VEC(float, 4);
      else DIB_QK_VEC(float, 8);
    } else {
      if (D == 64) DIB_QK_VEC(__nv_bfloat16, 2);
      else if (D == 128) DIB_QK_VEC(__nv_bfloat16, 4);
      else DIB_QK_VEC(__nv_bfloat16, 8);
    }
#undef DIB_QK_VEC
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  if (parts != nullptr) return DIB_BAD_SIZE;
  const size_t smem = (size_t)warps * D * sizeof(float);
  if (dtype == 0)
    dib_launch(qk_norm_rope_cache_kernel<float>, dim3(blocks), dim3(warps * 32), smem, st, 
        (const float*)qkv, (float*)q_out, (float*)kv_cache, q_norm_w, k_norm_w, eps, cos_sin,
        rotary_dim, max_pos, positions, slot_mapping, T, Hq, Hkv, D, page_size, num_pages);
  else if (dtype == 1)
    dib_launch(qk_norm_rope_cache_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, st, 
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_cache, q_norm_w,
        k_norm_w, eps, cos_sin, rotary_dim, max_pos, positions, slot_mapping, T, Hq, Hkv, D,
        page_size, num_pages);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_reshape_and_cache(const void* k, const void* v, void* kv_cache, const int* slot_mapping,
                          int T, int Hkv, int D, int page_size, long long num_pages, int dtype,
                          cudaStream_t st) {
  if (T == 0) return DIB_OK;
  int th = pick_threads(Hkv * D);
  if (th > 256) th = 256;
  if (dtype == 0)
    dib_launch(reshape_and_cache_kernel<float>, dim3(T), dim3(th), 0, st, (const float*)k, (const float*)v,
                                                      (float*)kv_cache, slot_mapping, Hkv, D,
                                                      page_size, num_pages);
  else if (dtype == 1)
    dib_launch(reshape_and_cache_kernel<__nv_bfloat16>, dim3(T), dim3(th), 0, st, 
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)kv_cache, slot_mapping,
        Hkv, D, page_size, num_pages);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_silu_mul(const void* gu, void* out, int T, int I, int dtype, cudaStream_t st) {
  const long long total = (long long)T * I;
  if (total == 0) return DIB_OK;
  const int th = 256;
  const bool aligned = reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  if (aligned && dtype == 1 && I % 8 == 0 && I / 8 <= 65535 * 32) {
    const int per_row = I / 8;
    const int tx = per_row >= 256 ? 128 : pick_threads(per_row);
    const dim3 grid1(T, ceil_div_host(per_row, tx)), grid2((T + 1) / 2, ceil_div_host(per_row, tx));
    if ((long long)T * per_row >= 2 * 148 * 2048ll)
      dib_launch(silu_mul_vec_kernel<__nv_bfloat16, 2>, grid2, dim3(tx), 0, st,
                 (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I);
    else
      dib_launch(silu_mul_vec_kernel<__nv_bfloat16, 1>, grid1, dim3(tx), 0, st,
                 (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I);
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  if (aligned && dtype == 0 && I % 4 == 0 && I / 4 <= 65535 * 32) {
    const int per_row = I / 4;
    const int tx = per_row >= 256 ? 128 : pick_threads(per_row);
    dib_launch(silu_mul_vec_kernel<float, 1>, dim3(T, ceil_div_host(per_row, tx)), dim3(tx), 0, st,
               (const float*)gu, (float*)out, T, I);
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  const int blocks = ceil_div_host(total, th);
  if (dtype == 0)
    dib_launch(silu_mul_kernel<float>, dim3(blocks), dim3(th), 0, st, (const float*)gu, (float*)out, total, I);
  else if (dtype == 1)
    dib_launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(th), 0, st, (const __nv_bfloat16*)gu,
                                                          (__nv_bfloat16*)out, total, I);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_gather_rows(const void* x, const int* idx, void* out, int R, int H, int T_rows, int dtype,
                    cudaStream_t st) {
  if (R == 0) return DIB_OK;
  int th = pick_threads(H);
  if (th > 256) th = 256;
  const size_t row_bytes = (size_t)H * (dtype == 0 ? 4 : 2);
  if ((dtype == 0 || dtype == 1) && row_bytes % 16 == 0 && T_rows > 0 &&
      (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
    const int vecs = (int)(row_bytes / 16);
    dib_launch(copy_rows16_kernel, dim3(R), dim3(vecs < 256 ? pick_threads(vecs) : 256), 0, st,
               (const uint4*)x, idx, (uint4*)out, vecs, T_rows, 0);
    DIB_CHECK_LAUNCH();
    return DIB_OK;
  }
  if (dtype == 0)
    dib_launch(gather_rows_kernel<float>, dim3(R), dim3(th), 0, st, (const float*)x, idx, (float*)out, H, T_rows);
  else if (dtype == 1)
    dib_launch(gather_rows_kernel<__nv_bfloat16>, dim3(R), dim3(th), 0, st, (const __nv_bfloat16*)x, idx,
                                                        (__nv_bfloat16*)out, H, T_rows);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// out[i] = round(sum over s of parts[s][i]); total elements a multiple of 4.
int dib_sum_split(const float* parts, int S, long long split_stride, void* out, long long total,
                  int dtype, cudaStream_t st) {
  if (total == 0) return DIB_OK;
  if (total % 4 != 0 || S < 1) return DIB_BAD_SIZE;
  const long long v = total / 4;
  const int th = 256;
  if (dtype == 0)
    dib_launch(sum_split_kernel<float>, dim3(ceil_div_host(v, th)), dim3(th), 0, st, parts, (float*)out, v, split_stride, S);
  else if (dtype == 1)
    dib_launch(sum_split_kernel<__nv_bfloat16>, dim3(ceil_div_host(v, th)), dim3(th), 0, st, parts, (__nv_bfloat16*)out, v,
                                                                      split_stride, S);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// add_rms_norm with x given as split-k partials [S, rows, H]; out [rows, H] is new.
int dib_add_rms_norm_split(const float* parts, int S, long long split_stride, void* residual,
                           const float* w, void* out, int rows, int H, float eps, int dtype,
                           cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (H % 4 != 0 || S < 1) return DIB_BAD_SIZE;
  const int vecs = H / 4;
  // Few rows: wide blocks, but 1,024 threads (64 registers each) only where 512 x 4 is too few.
  const int th_max = rows <= 128 ? (vecs > 2048 ? 1024 : 512) : 256;
  if (vecs > 4 * th_max) return DIB_BAD_SIZE;                           // at most 4 per thread
  int th = 32;
  while (th < vecs && th < th_max) th <<= 1;
  const int iters = (vecs + th - 1) / th;
#define DIB_ARS(TT, IT)                                                                         \
  dib_launch(add_rms_norm_split_kernel<TT, IT>, dim3(rows), dim3(th), 0, st, parts, S, split_stride, (TT*)residual, w, \
                                                         (TT*)out, H, eps)
  if (dtype == 0) {
    if (iters == 1) DIB_ARS(float, 1); else if (iters == 2) DIB_ARS(float, 2); else DIB_ARS(float, 4);
  } else if (dtype == 1) {
    if (iters == 1) DIB_ARS(__nv_bfloat16, 1);
    else if (iters == 2) DIB_ARS(__nv_bfloat16, 2);
    else DIB_ARS(__nv_bfloat16, 4);
  } else return DIB_BAD_DTYPE;
#undef DIB_ARS
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// silu_mul with [gate | up] given as split-k partials [S, T, 2I].
int dib_silu_mul_split(const float* parts, int S, long long split_stride, void* out, int T, int I,
                       int dtype, cudaStream_t st) {
  const long long total = (long long)T * I;
  if (total == 0) return DIB_OK;
  if (I % 4 != 0 || S < 1) return DIB_BAD_SIZE;
  const long long v = total / 4;
  const int th = 256;
  if (dtype == 0)
    dib_launch(silu_mul_split_kernel<float>, dim3(ceil_div_host(v, th)), dim3(th), 0, st, parts, S, split_stride,
                                                                    (float*)out, v, I);
  else if (dtype == 1)
    dib_launch(silu_mul_split_kernel<__nv_bfloat16>, dim3(ceil_div_host(v, th)), dim3(th), 0, st, 
        parts, S, split_stride, (__nv_bfloat16*)out, v, I);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_patch_ids(int* ids, const int* dst, const int* src, const int* prev, int n, int num_ids,
                  int num_prev, cudaStream_t st) {
  if (n == 0) return DIB_OK;
  dib_launch(patch_ids_kernel, dim3(ceil_div_host(n, 128)), dim3(128), 0, st, ids, dst, src, prev, n,
             num_ids, num_prev);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // extern "C"
