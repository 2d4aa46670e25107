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

static inline int ceil_div_host(long long a, long long b) { return (int)((a + b - 1) / b); }

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
// completes within microseconds; a wait that has lasted a second means the kernel's
// bookkeeping is broken.  It then gives up and reports false, so that the kernel can
// set its error word and end instead of spinning for good.
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
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
    if ((i & 255u) == 0) {
      const unsigned long long t = global_timer_ns();
      if (t0 == 0) t0 = t;
      else if (t - t0 > 1000000000ull) return false;
    }
  }
}
