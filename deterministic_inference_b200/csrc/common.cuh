// Shared device helpers for the sm_100a kernels of this package.
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes
// and a stream, validates what it can on the host, launches, and returns 0 or a
// negative code (see dib_status below); the Python wrappers turn codes into
// exceptions.  dtype codes: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

enum dib_status : int {
  DIB_OK = 0,
  DIB_BAD_DTYPE = -1,
  DIB_BAD_SIZE = -2,      // a size this kernel refuses (message printed by the wrapper)
  DIB_BAD_ALIGN = -3,
  DIB_LAUNCH_FAILED = -4,
};

#define DIB_CHECK_LAUNCH()                                   \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return DIB_LAUNCH_FAILED;        \
  } while (0)

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// silu(g) * u in float32.  For float32 storage with the library's exponential and a true
// division; for bfloat16 storage with the special-function unit's 2^x and reciprocal
// (relative error about 1e-6, far below the bfloat16 step of the stored result), which
// is a third of the instructions: at prompt sizes the gate is bound by them, not by memory.
// Every kernel that gates (the separate gate, the reader of split products, the matrix
// product's epilogue) uses this one form, so they agree in every bit.
template <typename T> __device__ __forceinline__ float silu_gate(float g, float u);
template <> __device__ __forceinline__ float silu_gate<float>(float g, float u) {
  return g / (1.0f + expf(-g)) * u;
}
template <> __device__ __forceinline__ float silu_gate<__nv_bfloat16>(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * r * u;
}

// Round a float32 value to the storage type and back (what a store followed by
// a load would give).
template <typename T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Fixed-order butterfly reductions: the same lanes always combine in the same
// order, so a row's result never depends on what else is in the launch.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed order: warp butterflies, then warp 0 adds the
// per-warp partials in index order.  `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// ---- the one order in which a row's sum of squares (the RMSNorm statistic) is added up,
// whatever kernel, block size or launch form computes it, so that a row's norm never
// depends on what else is in the launch: the row is cut into vectors of 4 consecutive
// elements; a vector's sum is the chain fma(x3,x3, fma(x2,x2, fma(x1,x1, x0*x0))); 32
// consecutive vectors (128 elements) form a group, added by the butterfly over the vector
// index (partners 16, 8, 4, 2, 1 apart, missing vectors count as 0); the groups' sums are
// added one after the other in index order.
__device__ __forceinline__ float sumsq4(float x0, float x1, float x2, float x3) {
  return __fmaf_rn(x3, x3, __fmaf_rn(x2, x2, __fmaf_rn(x1, x1, __fmul_rn(x0, x0))));
}
// VPT vectors per thread: thread `lane` of a warp holds the vectors VPT*lane .. VPT*lane +
// VPT-1 of 32*VPT consecutive ones (VPT 1 or 2).  Returns the sum of the group this lane's
// vectors belong to: the whole warp (VPT 1) or its half-warp (VPT 2).
template <int VPT> __device__ __forceinline__ float sumsq_group(const float (&s)[VPT]);
template <> __device__ __forceinline__ float sumsq_group<1>(const float (&s)[1]) {
  float v = s[0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <> __device__ __forceinline__ float sumsq_group<2>(const float (&s)[2]) {
  float a = s[0], b = s[1];     // vector indices 2*lane and 2*lane + 1 inside the half-warp's group
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {   // partners 16, 8, 4, 2 vectors apart: 8, 4, 2, 1 lanes
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, o));
    b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, o));
  }
  return __fadd_rn(a, b);             // partner 1 vector apart: in this thread
}
// Block-wide: thread t holds, for iteration it, the vectors VPT*(it*blockDim.x + t) ..; the
// block's threads cover the row's `num_vectors` vectors.  `scratch` holds at least
// ceil(num_vectors / 32) floats.  Every thread gets the row's total.
template <int ITERS, int VPT>
__device__ __forceinline__ float sumsq_row(const float (&s)[ITERS][VPT], int num_vectors,
                                           float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();   // scratch may still be read from a previous call
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const float g = sumsq_group<VPT>(s[it]);
    const int group = (it * nwarps + warp) * VPT + (VPT == 2 ? (lane >> 4) : 0);
    if ((lane & (VPT == 2 ? 15 : 31)) == 0 && group * 32 < num_vectors) scratch[group] = g;
  }
  __syncthreads();
  const int groups = (num_vectors + 31) >> 5;
  float total = scratch[0];
  for (int g = 1; g < groups; ++g) total = __fadd_rn(total, scratch[g]);
  return total;
}
// y = x * rstd * w and the rotate-half pair, with every rounding spelled out so that all
// kernels that norm and rotate give the same bits.
__device__ __forceinline__ float norm_scale(float x, float rstd, float w) {
  return __fmul_rn(__fmul_rn(x, rstd), w);
}
__device__ __forceinline__ float rope_first(float x1, float x2, float c, float sn) {   // x1 cos - x2 sin
  return __fmaf_rn(x1, c, -__fmul_rn(x2, sn));
}
__device__ __forceinline__ float rope_second(float x1, float x2, float c, float sn) {  // x2 cos + x1 sin
  return __fmaf_rn(x2, c, __fmul_rn(x1, sn));
}
__device__ __forceinline__ float rms_rstd(float sumsq, int n, float eps) {
  return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, (float)n), eps)));
}

// One (token, head) row of 128 bfloat16 values held by eight lanes: lane l (0..7; `mask` names
// the eight) has the elements 8l..8l+7 in `lo` and 64+8l..64+8l+7 in `hi`, so a rotation pair
// lies in one lane.  RMSNorm with the weight nw [128] (or null: none), then the rotate-half
// rotation by c / sn (the position's cosines and sines of the dimensions 8l..8l+7) if
// `rotate`.  The sum of squares is taken in the order of the one-warp-per-row kernel (a lane
// there holds 4 consecutive elements, lanes combine 16, 8, 4, 2, 1 apart: this lane holds
// that kernel's lanes 2l, 2l+1 (lo) and 2l+16, 2l+17 (hi)), so every kernel that norms a head
// of 128 gives the same bits.
// (In three steps, so that a kernel with several rows in hand can take the steps of all of
// them together: the row's 1/rms; the lane's norm weights; norm, rotation and rounding.)
__device__ __forceinline__ void qk_row128_unpack(const uint4& lo, const uint4& hi, float (&a)[8], float (&b)[8]) {
  const __nv_bfloat162* pl = reinterpret_cast<const __nv_bfloat162*>(&lo);
  const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&hi);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 x = __bfloat1622float2(pl[k]), y = __bfloat1622float2(ph[k]);
    a[2 * k] = x.x; a[2 * k + 1] = x.y;
    b[2 * k] = y.x; b[2 * k + 1] = y.y;
  }
}
// this lane's two sums of the butterfly: lanes combine them 4, 2, 1 apart, then e + o
__device__ __forceinline__ void qk_row128_sums(const uint4& lo, const uint4& hi, float& e, float& o) {
  float a[8], b[8];
  qk_row128_unpack(lo, hi, a, b);
  e = __fadd_rn(sumsq4(a[0], a[1], a[2], a[3]), sumsq4(b[0], b[1], b[2], b[3]));
  o = __fadd_rn(sumsq4(a[4], a[5], a[6], a[7]), sumsq4(b[4], b[5], b[6], b[7]));
}
__device__ __forceinline__ float qk_row128_rstd(const uint4& lo, const uint4& hi, unsigned mask, float eps) {
  float e, o;
  qk_row128_sums(lo, hi, e, o);
#pragma unroll
  for (int sh = 4; sh > 0; sh >>= 1) {
    e = __fadd_rn(e, __shfl_xor_sync(mask, e, sh));
    o = __fadd_rn(o, __shfl_xor_sync(mask, o, sh));
  }
  return rms_rstd(__fadd_rn(e, o), 128, eps);
}
__device__ __forceinline__ void qk_row128_weights(const float* nw, int l, float (&wa)[8], float (&wb)[8]) {
  const float4 w0 = *reinterpret_cast<const float4*>(nw + l * 8);
  const float4 w1 = *reinterpret_cast<const float4*>(nw + l * 8 + 4);
  const float4 w2 = *reinterpret_cast<const float4*>(nw + 64 + l * 8);
  const float4 w3 = *reinterpret_cast<const float4*>(nw + 64 + l * 8 + 4);
  wa[0] = w0.x; wa[1] = w0.y; wa[2] = w0.z; wa[3] = w0.w; wa[4] = w1.x; wa[5] = w1.y; wa[6] = w1.z; wa[7] = w1.w;
  wb[0] = w2.x; wb[1] = w2.y; wb[2] = w2.z; wb[3] = w2.w; wb[4] = w3.x; wb[5] = w3.y; wb[6] = w3.z; wb[7] = w3.w;
}
__device__ __forceinline__ void qk_row128_apply(uint4& lo, uint4& hi, bool norm, float rstd, const float (&wa)[8],
                                                const float (&wb)[8], bool rotate, const float (&c)[8],
                                                const float (&sn)[8]) {
  float a[8], b[8];
  qk_row128_unpack(lo, hi, a, b);
  if (norm) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a[k] = norm_scale(a[k], rstd, wa[k]);
      b[k] = norm_scale(b[k], rstd, wb[k]);
    }
  }
  if (rotate) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x = a[k], y = b[k];
      a[k] = rope_first(x, y, c[k], sn[k]);
      b[k] = rope_second(x, y, c[k], sn[k]);
    }
  }
  __nv_bfloat162* ql = reinterpret_cast<__nv_bfloat162*>(&lo);
  __nv_bfloat162* qh = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    ql[k] = __floats2bfloat162_rn(a[2 * k], a[2 * k + 1]);
    qh[k] = __floats2bfloat162_rn(b[2 * k], b[2 * k + 1]);
  }
}
__device__ __forceinline__ void qk_row128(uint4& lo, uint4& hi, int l, unsigned mask, const float* nw, float eps,
                                          bool rotate, const float (&c)[8], const float (&sn)[8]) {
  float wa[8] = {}, wb[8] = {};
  float rstd = 0.f;
  if (nw != nullptr) {
    rstd = qk_row128_rstd(lo, hi, mask, eps);
    qk_row128_weights(nw, l, wa, wb);
  }
  qk_row128_apply(lo, hi, nw != nullptr, rstd, wa, wb, rotate, c, sn);
}

static inline int ceil_div_host(long long a, long long b) { return (int)((a + b - 1) / b); }

// "Done once on the current device": a kernel's attributes (its shared-memory limit) are
// kept per device, so a set-up step done on one device has to be done again on the next.
struct DeviceOnce {
  unsigned long long mask[4] = {0, 0, 0, 0};   // devices 0..255
  static int current() {
    int dev = 0;
    return cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 256 ? dev : -1;
  }
  bool done() const {
    const int d = current();
    return d >= 0 && ((mask[d >> 6] >> (d & 63)) & 1ull);
  }
  void mark() {
    const int d = current();
    if (d >= 0) mask[d >> 6] |= 1ull << (d & 63);
  }
};

// ---- programmatic dependent launch
// Every kernel of this package is launched with the attribute that lets it start
// while the kernel before it on the stream is still draining (its blocks are
// scheduled, its prologue runs), and every kernel waits with griddepcontrol.wait for
// that predecessor to have finished and flushed its memory before it reads or writes
// anything the predecessor may touch.  Only constants (weights, tables, tensor maps)
// are read before the wait.  In a chain A, B, C each kernel waits for the one before
// it, which itself only finished after its own wait, so C also sees A complete.  Set
// DIB200_PDL=0 to launch the plain way.
//
// The wait takes the pointers through which the kernel reads what its predecessor
// wrote, and hands them back as values the compiler knows nothing about.  Without
// that, a load through a `const T* __restrict__` parameter counts as a load of data
// that never changes while the kernel runs, and the compiler may move it above the
// wait (it did, in the kernel that merges the splits of decode attention: the partial
// results were read before the kernel that writes them had finished).
template <typename P> __device__ __forceinline__ void pdl_fresh(P& p) { asm volatile("" : "+l"(p)); }
template <typename... P> __device__ __forceinline__ void pdl_wait(P&... p) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  (pdl_fresh(p), ...);
}
// Ask for a tensor map (a kernel parameter) ahead of the first copy that uses it.
__device__ __forceinline__ void prefetch_tensormap(const void* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(map)) : "memory");
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::); }
template <typename... P> __device__ __forceinline__ void pdl_prologue(P&... p) {
  pdl_trigger();
  pdl_wait(p...);
}

static inline bool dib_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("DIB200_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <typename... KArgs, typename... Args>
static inline void dib_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dib_pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- bounded wait on a shared-memory mbarrier.  A copy or a tensor-core operation
// completes within microseconds; a wait that has lasted `limit_ns` (a second unless the
// caller says otherwise) means the kernel's bookkeeping is broken.  It then gives up and
// reports false, so that the kernel can set its error word and end instead of spinning
// for good.
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity,
                                          unsigned long long limit_ns = 1000000000ull) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(bar);
  unsigned long long t0 = 0;
  for (unsigned i = 1;; ++i) {
    unsigned ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; "
        "selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 63u) == 0) {
      const unsigned long long t = global_timer_ns();
      if (t0 == 0) t0 = t;
      else if (t - t0 > limit_ns) return false;
    }
  }
}
