// Sampling kernels over float32 logits [R, V]: argmax (lowest index wins ties)
// and temperature sampling by position-seeded Gumbel-max.
//
// Gumbel-max: p = softmax(logits / temperature); token = argmax over kept ids of
// log(p + 1e-10) + g(seed, pos, id), with g = -log(-log(u + 1e-10) + 1e-10) and u
// the low 24 bits of a 64-bit wrap-around hash of (seed, pos, id) divided by
// 2^24.  The noise is a pure function of (seed, position of the generated token,
// vocabulary id), so a draw does not depend on the batch.  Rows with
// temperature <= 0 take the argmax.  `keep` (optional, uint8 [R, V]) masks ids
// dropped by top-k / top-p.
#include "common.cuh"

namespace {

struct Best {
  float v;
  int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  // larger value wins; equal values: lower index wins
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ Best block_best(Best b, Best* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    b = better(b, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = b;
  __syncthreads();
  Best r = scratch[0];
  for (int w = 1; w < nwarps; ++w) r = better(r, scratch[w]);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < nwarps; ++w) r = fmaxf(r, scratch[w]);
  return r;
}

constexpr int INT_MAX_ = 0x7fffffff;

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  pdl_prologue();
  __shared__ Best scratch[32];
  const float* row = logits + (size_t)blockIdx.x * V;
  Best b{-INFINITY, INT_MAX_};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    Best c{row[i], i};
    b = better(b, c);
  }
  b = block_best(b, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = b.i == INT_MAX_ ? 0 : b.i;
}

// Two-stage argmax for wide rows: a row is cut into chunks of ARGMAX_CHUNK ids,
// one block per (row, chunk) writes its best (value, index); a second kernel picks
// the best chunk.  Ties go to the lowest index in both stages.
constexpr int ARGMAX_CHUNK = 4096;

__global__ void argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ pv,
                                      int* __restrict__ pi, int V, int chunks) {
  pdl_prologue();
  __shared__ Best scratch[32];
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const int lo = c * ARGMAX_CHUNK, hi = min(V, lo + ARGMAX_CHUNK);
  Best b{-INFINITY, INT_MAX_};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) b = better(b, Best{row[i], i});
  b = block_best(b, scratch);
  if (threadIdx.x == 0) {
    pv[(size_t)r * chunks + c] = b.v;
    pi[(size_t)r * chunks + c] = b.i;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi,
                                    int* __restrict__ out, int chunks) {
  pdl_prologue();
  __shared__ Best scratch[32];
  const int r = blockIdx.x;
  Best b{-INFINITY, INT_MAX_};
  for (int c = threadIdx.x; c < chunks; c += blockDim.x)
    b = better(b, Best{pv[(size_t)r * chunks + c], pi[(size_t)r * chunks + c]});
  b = block_best(b, scratch);
  if (threadIdx.x == 0) out[r] = b.i == INT_MAX_ ? 0 : b.i;
}

__device__ __forceinline__ float seeded_gumbel(long long seed, long long pos, int col) {
  const unsigned long long step =
      ((unsigned long long)seed * 19349663ull) ^ ((unsigned long long)pos * 73856093ull);
  const unsigned long long hashed =
      (step * 8589934591ull) ^ ((unsigned long long)col * 479001599ull);
  const float u = (float)(unsigned)(hashed & 0xffffffull) / 16777216.0f;
  return -logf(-logf(u + 1e-10f) + 1e-10f);
}

__global__ void gumbel_sample_kernel(const float* __restrict__ logits,
                                     const float* __restrict__ temperatures,
                                     const long long* __restrict__ seeds,
                                     const long long* __restrict__ sample_pos,
                                     const unsigned char* __restrict__ keep,
                                     int* __restrict__ out, int V) {
  pdl_prologue();
  __shared__ Best bscratch[32];
  __shared__ float fscratch[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float temp = temperatures[r];
  if (temp <= 0.f) {
    Best b{-INFINITY, INT_MAX_};
    for (int i = threadIdx.x; i < V; i += blockDim.x) b = better(b, Best{row[i], i});
    b = block_best(b, bscratch);
    if (threadIdx.x == 0) out[r] = b.i == INT_MAX_ ? 0 : b.i;
    return;
  }
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] / temp);
  mx = block_max(mx, fscratch);
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) sum += expf(row[i] / temp - mx);
  sum = block_sum(sum, fscratch);
  const long long seed = seeds[r], pos = sample_pos[r];
  const unsigned char* krow = keep ? keep + (size_t)r * V : nullptr;
  Best b{-INFINITY, INT_MAX_};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (krow && !krow[i]) continue;
    const float p = expf(row[i] / temp - mx) / sum;
    const float score = logf(p + 1e-10f) + seeded_gumbel(seed, pos, i);
    b = better(b, Best{score, i});
  }
  b = block_best(b, bscratch);
  if (threadIdx.x == 0) out[r] = b.i == INT_MAX_ ? 0 : b.i;
}
// Wide rows in chunks of ARGMAX_CHUNK ids, one block per (row, chunk), three kernels:
// the chunk's maximum of logits / temperature and its sum of exponentials against that
// maximum; then, with the row's maximum and sum put together from the chunks' in chunk
// order (a row's normaliser never depends on the batch), the chunk's best score; then
// the best chunk (argmax_final_kernel).
__global__ void gumbel_stats_kernel(const float* __restrict__ logits,
                                    const float* __restrict__ temperatures,
                                    float* __restrict__ cmax, float* __restrict__ csum, int V,
                                    int chunks) {
  pdl_prologue();
  __shared__ float fscratch[32];
  const int r = blockIdx.y, c = blockIdx.x;
  const float temp = temperatures[r];
  if (temp <= 0.f) return;     // a greedy row needs no normaliser
  const float* row = logits + (size_t)r * V;
  const int lo = c * ARGMAX_CHUNK, hi = min(V, lo + ARGMAX_CHUNK);
  float mx = -INFINITY;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) mx = fmaxf(mx, row[i] / temp);
  mx = block_max(mx, fscratch);
  float sum = 0.f;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) sum += expf(row[i] / temp - mx);
  sum = block_sum(sum, fscratch);
  if (threadIdx.x == 0) {
    cmax[(size_t)r * chunks + c] = mx;
    csum[(size_t)r * chunks + c] = sum;
  }
}

__global__ void gumbel_pick_kernel(const float* __restrict__ logits,
                                   const float* __restrict__ temperatures,
                                   const long long* __restrict__ seeds,
                                   const long long* __restrict__ sample_pos,
                                   const unsigned char* __restrict__ keep,
                                   const float* __restrict__ cmax, const float* __restrict__ csum,
                                   float* __restrict__ pv, int* __restrict__ pi, int V, int chunks) {
  pdl_prologue();
  __shared__ Best bscratch[32];
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const int lo = c * ARGMAX_CHUNK, hi = min(V, lo + ARGMAX_CHUNK);
  const float temp = temperatures[r];
  Best b{-INFINITY, INT_MAX_};
  if (temp <= 0.f) {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) b = better(b, Best{row[i], i});
  } else {
    float mx = -INFINITY;
    for (int k = 0; k < chunks; ++k) mx = fmaxf(mx, cmax[(size_t)r * chunks + k]);
    float sum = 0.f;
    for (int k = 0; k < chunks; ++k)
      sum += csum[(size_t)r * chunks + k] * expf(cmax[(size_t)r * chunks + k] - mx);
    const long long seed = seeds[r], pos = sample_pos[r];
    const unsigned char* krow = keep ? keep + (size_t)r * V : nullptr;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      if (krow && !krow[i]) continue;
      const float p = expf(row[i] / temp - mx) / sum;
      b = better(b, Best{logf(p + 1e-10f) + seeded_gumbel(seed, pos, i), i});
    }
  }
  b = block_best(b, bscratch);
  if (threadIdx.x == 0) {
    pv[(size_t)r * chunks + c] = b.v;
    pi[(size_t)r * chunks + c] = b.i;
  }
}

}  // namespace

extern "C" {

int dib_argmax(const float* logits, int* out, int R, int V, cudaStream_t st) {
  if (R == 0) return DIB_OK;
  if (V < 1) return DIB_BAD_SIZE;
  dib_launch(argmax_kernel, dim3(R), dim3(1024), 0, st, logits, out, V);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_argmax_chunks(int V) { return (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK; }

// scratch_v / scratch_i: [R, dib_argmax_chunks(V)]
int dib_argmax_two_stage(const float* logits, float* scratch_v, int* scratch_i, int* out, int R,
                         int V, cudaStream_t st) {
  if (R == 0) return DIB_OK;
  if (V < 1 || R > 65535) return DIB_BAD_SIZE;
  const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
  dib_launch(argmax_partial_kernel, dim3(dim3(chunks, R)), dim3(256), 0, st, logits, scratch_v, scratch_i, V, chunks);
  DIB_CHECK_LAUNCH();
  dib_launch(argmax_final_kernel, dim3(R), dim3(64), 0, st, scratch_v, scratch_i, out, chunks);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_gumbel_sample(const float* logits, const float* temperatures, const long long* seeds,
                      const long long* sample_pos, const unsigned char* keep, int* out, int R,
                      int V, cudaStream_t st) {
  if (R == 0) return DIB_OK;
  if (V < 1) return DIB_BAD_SIZE;
  dib_launch(gumbel_sample_kernel, dim3(R), dim3(1024), 0, st, logits, temperatures, seeds, sample_pos, keep, out, V);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The same in chunks (see gumbel_stats_kernel).  scratch_f: float [3, R, chunks];
// scratch_i: int [R, chunks], chunks = dib_argmax_chunks(V).
int dib_gumbel_sample_chunked(const float* logits, const float* temperatures, const long long* seeds,
                              const long long* sample_pos, const unsigned char* keep,
                              float* scratch_f, int* scratch_i, int* out, int R, int V,
                              cudaStream_t st) {
  if (R == 0) return DIB_OK;
  if (V < 1 || R > 65535) return DIB_BAD_SIZE;
  const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
  float* cmax = scratch_f;
  float* csum = scratch_f + (size_t)R * chunks;
  float* pv = scratch_f + 2 * (size_t)R * chunks;
  dib_launch(gumbel_stats_kernel, dim3(chunks, R), dim3(256), 0, st, logits, temperatures, cmax, csum, V,
             chunks);
  DIB_CHECK_LAUNCH();
  dib_launch(gumbel_pick_kernel, dim3(chunks, R), dim3(256), 0, st, logits, temperatures, seeds,
             sample_pos, keep, (const float*)cmax, (const float*)csum, pv, scratch_i, V, chunks);
  DIB_CHECK_LAUNCH();
  dib_launch(argmax_final_kernel, dim3(R), dim3(64), 0, st, (const float*)pv, (const int*)scratch_i, out,
             chunks);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // extern "C"
