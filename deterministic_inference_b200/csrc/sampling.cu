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
  pdl_prologue(logits);
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
  pdl_prologue(logits);
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
  pdl_prologue(pv, pi);
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
  pdl_prologue(logits, temperatures, seeds, sample_pos, keep);
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
                                    float* __restrict__ cmax, float* __restrict__ csum,
                                    unsigned* __restrict__ hist_cnt,
                                    unsigned long long* __restrict__ hist_mass, int R, int V,
                                    int chunks) {
  pdl_prologue(logits, temperatures);
  __shared__ float fscratch[32];
  const int r = blockIdx.y, c = blockIdx.x;
  // the row's top-k / top-p histograms (4 passes x 256 bins) start from zero: the blocks
  // of the row share the zeroing
  if (hist_cnt != nullptr) {
    for (int e = c * blockDim.x + threadIdx.x; e < 4 * 256; e += chunks * blockDim.x) {
      const size_t at = ((size_t)(e >> 8) * R + r) * 256 + (e & 255);
      hist_cnt[at] = 0u;
      hist_mass[at] = 0ull;
    }
  }
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

// The row's maximum and sum of exponentials from its chunks', in chunk order: every
// kernel that needs a probability forms it from these two, with the same expression, so
// all of them see the same bits.
__device__ __forceinline__ void row_normaliser(const float* __restrict__ cmax,
                                               const float* __restrict__ csum, int r, int chunks,
                                               float& mx, float& sum) {
  mx = -INFINITY;
  for (int k = 0; k < chunks; ++k) mx = fmaxf(mx, cmax[(size_t)r * chunks + k]);
  sum = 0.f;
  for (int k = 0; k < chunks; ++k)
    sum += csum[(size_t)r * chunks + k] * expf(cmax[(size_t)r * chunks + k] - mx);
}
__device__ __forceinline__ float row_probability(float logit, float temp, float mx, float sum) {
  return expf(logit / temp - mx) / sum;
}

// top-k / top-p without a sort.  In the order of a descending sort a token stays when
// its rank is below k and the probability mass before it is at most top_p (rank 0 always
// stays).  Rank and mass before are both non-increasing in the token's probability, so
// the kept set is {p >= t} for one threshold t: found by a radix descent over the 32
// bits of the probability, 8 bits a pass, with a histogram of counts and of masses per
// pass.  Masses are added as 40-bit fixed point, so that the order of the additions
// (atomics) cannot change a bit.  Tokens that tie with the threshold all stay (a sort
// would keep some of them).  A pass is one kernel with a block per chunk of a row; the
// histograms of the four passes lie in global memory ([4][R][256] counts and masses,
// zeroed by the kernel that computes the normaliser), and every block works out the
// bits fixed so far from the histograms of the passes before its own.
constexpr float MASS_ONE = 1099511627776.0f;     // 2^40

struct FilterState {
  unsigned prefix;                      // the threshold's bits found so far
  unsigned long long cnt_above, mass_above;   // tokens (and their mass) above the chosen bins
};

// Warp 0 of the block: the state after `passes` passes, from their histograms.
__device__ __forceinline__ FilterState filter_descend(const unsigned* __restrict__ hist_cnt,
                                                      const unsigned long long* __restrict__ hist_mass,
                                                      int R, int r, int passes, unsigned long long k,
                                                      unsigned long long P) {
  const int lane = threadIdx.x & 31;
  FilterState st{0u, 0ull, 0ull};
  for (int pass = 0; pass < passes; ++pass) {
    const unsigned* hc = hist_cnt + ((size_t)pass * R + r) * 256 + lane * 8;
    const unsigned long long* hm = hist_mass + ((size_t)pass * R + r) * 256 + lane * 8;
    unsigned c[8];
    unsigned long long m[8], csum = 0ull, msum = 0ull;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      c[j] = __ldcg(hc + j);
      m[j] = __ldcg(hm + j);
      csum += c[j];
      msum += m[j];
    }
    // counts and masses of the bins of higher lanes (an exclusive suffix sum)
    unsigned long long ca = 0ull, ma = 0ull;
    {
      unsigned long long c_run = csum, m_run = msum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long c_up = __shfl_down_sync(0xffffffffu, c_run, o);
        const unsigned long long m_up = __shfl_down_sync(0xffffffffu, m_run, o);
        if (lane + o < 32) {
          c_run += c_up;
          m_run += m_up;
        }
      }
      ca = st.cnt_above + c_run - csum;     // inclusive suffix minus own
      ma = st.mass_above + m_run - msum;
    }
    // this lane's bins from the highest down: the lowest non-empty bin that is entered
    // while fewer than k tokens, weighing at most P, lie above it
    int best = 256;
    unsigned long long best_ca = 0ull, best_ma = 0ull;
#pragma unroll
    for (int j = 7; j >= 0; --j) {
      if (c[j] != 0u && ca < k && ma <= P) {
        best = lane * 8 + j;
        best_ca = ca;
        best_ma = ma;
      }
      ca += c[j];
      ma += m[j];
    }
    int chosen = best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) chosen = min(chosen, __shfl_xor_sync(0xffffffffu, chosen, o));
    if (chosen == 256) chosen = 0;      // an empty histogram (cannot happen for a row that is filtered)
    const int owner = chosen >> 3;
    st.cnt_above = __shfl_sync(0xffffffffu, best == chosen ? best_ca : 0ull, owner);
    st.mass_above = __shfl_sync(0xffffffffu, best == chosen ? best_ma : 0ull, owner);
    st.prefix |= (unsigned)chosen << (24 - 8 * pass);
  }
  return st;
}

__device__ __forceinline__ bool row_is_filtered(float temp, long long top_k, float top_p) {
  return temp > 0.f && (top_k > 0 || top_p < 1.0f);
}

__global__ void __launch_bounds__(256)
filter_histogram_kernel(const float* __restrict__ logits, const float* __restrict__ temperatures,
                        const long long* __restrict__ top_ks, const float* __restrict__ top_ps,
                        const float* __restrict__ cmax, const float* __restrict__ csum,
                        unsigned* __restrict__ hist_cnt, unsigned long long* __restrict__ hist_mass,
                        int pass, int R, int V, int chunks) {
  pdl_prologue(logits, temperatures, top_ks, top_ps, cmax, csum);
  __shared__ unsigned s_cnt[256];
  __shared__ unsigned long long s_mass[256];
  __shared__ unsigned s_prefix;
  const int r = blockIdx.y, c = blockIdx.x;
  const float temp = temperatures[r];
  const long long top_k = top_ks[r];
  const float top_p = top_ps[r];
  if (!row_is_filtered(temp, top_k, top_p)) return;
  const unsigned long long k = top_k > 0 ? (unsigned long long)top_k : (unsigned long long)V + 1;
  const unsigned long long P = top_p >= 1.0f ? ~0ull : (unsigned long long)(top_p * MASS_ONE);
  s_cnt[threadIdx.x] = 0u;
  s_mass[threadIdx.x] = 0ull;
  if (threadIdx.x < 32) {
    const FilterState st = filter_descend(hist_cnt, hist_mass, R, r, pass, k, P);
    if (threadIdx.x == 0) s_prefix = st.prefix;
  }
  __syncthreads();
  const unsigned prefix = s_prefix;
  const int shift = 24 - 8 * pass;
  const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
  const float* row = logits + (size_t)r * V;
  float mx, sum;
  row_normaliser(cmax, csum, r, chunks, mx, sum);
  const int lo = c * ARGMAX_CHUNK, hi = min(V, lo + ARGMAX_CHUNK);
  // In the first pass nearly all of a warp's 32 tokens fall into one or two bins (the top
  // bits of small probabilities): the lanes of a bin add up among themselves and one of
  // them updates the histogram, instead of 32 atomics on one address.
  for (int i0 = lo; i0 < hi; i0 += 256) {
    const int i = i0 + threadIdx.x;
    unsigned bin = 0xffffffffu;               // no bin: outside the chunk or the prefix
    unsigned long long m = 0ull;
    if (i < hi) {
      const float p = row_probability(row[i], temp, mx, sum);
      const unsigned key = __float_as_uint(p);
      if ((key & mask) == prefix) {
        bin = (key >> shift) & 255u;
        m = (unsigned long long)(p * MASS_ONE);
      }
    }
    const unsigned peers = __match_any_sync(0xffffffffu, bin);
    if (bin == 0xffffffffu) continue;
    // the group's mass: 40-bit values as two halves that 32-bit warp sums can take
    const unsigned lo20 = __reduce_add_sync(peers, (unsigned)(m & 0xfffffull));
    const unsigned hi20 = __reduce_add_sync(peers, (unsigned)(m >> 20));
    if ((threadIdx.x & 31) == __ffs(peers) - 1) {
      atomicAdd(&s_cnt[bin], (unsigned)__popc(peers));
      atomicAdd(&s_mass[bin], ((unsigned long long)hi20 << 20) + lo20);
    }
  }
  __syncthreads();
  if (s_cnt[threadIdx.x] != 0u) {
    const size_t at = ((size_t)pass * R + r) * 256 + threadIdx.x;
    atomicAdd(&hist_cnt[at], s_cnt[threadIdx.x]);
    atomicAdd(&hist_mass[at], s_mass[threadIdx.x]);
  }
}

__global__ void gumbel_pick_kernel(const float* __restrict__ logits,
                                   const float* __restrict__ temperatures,
                                   const long long* __restrict__ seeds,
                                   const long long* __restrict__ sample_pos,
                                   const unsigned char* __restrict__ keep,
                                   const long long* __restrict__ top_ks,
                                   const float* __restrict__ top_ps,
                                   const unsigned* __restrict__ hist_cnt,
                                   const unsigned long long* __restrict__ hist_mass,
                                   unsigned* __restrict__ thresh,
                                   const float* __restrict__ cmax, const float* __restrict__ csum,
                                   float* __restrict__ pv, int* __restrict__ pi, int R, int V,
                                   int chunks) {
  pdl_prologue(logits, temperatures, seeds, sample_pos, keep, top_ks, top_ps, hist_cnt, hist_mass, cmax,
               csum);
  __shared__ Best bscratch[32];
  __shared__ unsigned s_thresh;
  const int r = blockIdx.y, c = blockIdx.x;
  // the threshold of top-k / top-p: all four passes' histograms are complete
  if (threadIdx.x < 32) {
    unsigned t = 0u;
    if (thresh != nullptr) {
      const long long top_k = top_ks[r];
      const float top_p = top_ps[r];
      if (row_is_filtered(temperatures[r], top_k, top_p)) {
        const unsigned long long k = top_k > 0 ? (unsigned long long)top_k : (unsigned long long)V + 1;
        const unsigned long long P = top_p >= 1.0f ? ~0ull : (unsigned long long)(top_p * MASS_ONE);
        t = filter_descend(hist_cnt, hist_mass, R, r, 4, k, P).prefix;
      }
      if (threadIdx.x == 0 && c == 0) thresh[r] = t;
    }
    if (threadIdx.x == 0) s_thresh = t;
  }
  __syncthreads();
  const float* row = logits + (size_t)r * V;
  const int lo = c * ARGMAX_CHUNK, hi = min(V, lo + ARGMAX_CHUNK);
  const float temp = temperatures[r];
  Best b{-INFINITY, INT_MAX_};
  if (temp <= 0.f) {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) b = better(b, Best{row[i], i});
  } else {
    float mx, sum;
    row_normaliser(cmax, csum, r, chunks, mx, sum);
    const long long seed = seeds[r], pos = sample_pos[r];
    const unsigned char* krow = keep ? keep + (size_t)r * V : nullptr;
    const unsigned t = s_thresh;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      if (krow && !krow[i]) continue;
      const float p = row_probability(row[i], temp, mx, sum);
      if (__float_as_uint(p) < t) continue;
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
// top_ks / top_ps (both or neither): per-row top-k (<= 0: off) and top-p (>= 1: off),
// applied by a threshold found without a sort.  thresh: unsigned [R], receives the bits of
// each row's smallest kept probability (0 = all kept); hist: scratch of 4 * R * 256 * 12
// bytes, 8-byte aligned (masses first, then counts).
int dib_gumbel_sample_chunked(const float* logits, const float* temperatures, const long long* seeds,
                              const long long* sample_pos, const unsigned char* keep,
                              const long long* top_ks, const float* top_ps, unsigned* thresh,
                              void* hist, float* scratch_f, int* scratch_i, int* out, int R, int V,
                              cudaStream_t st) {
  if (R == 0) return DIB_OK;
  if (V < 1 || R > 65535) return DIB_BAD_SIZE;
  const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
  float* cmax = scratch_f;
  float* csum = scratch_f + (size_t)R * chunks;
  float* pv = scratch_f + 2 * (size_t)R * chunks;
  const bool filtered = top_ks != nullptr && top_ps != nullptr && thresh != nullptr && hist != nullptr;
  if (filtered && reinterpret_cast<uintptr_t>(hist) % 8 != 0) return DIB_BAD_ALIGN;
  unsigned long long* hist_mass = filtered ? reinterpret_cast<unsigned long long*>(hist) : nullptr;
  unsigned* hist_cnt = filtered ? reinterpret_cast<unsigned*>(hist_mass + (size_t)4 * R * 256) : nullptr;
  dib_launch(gumbel_stats_kernel, dim3(chunks, R), dim3(256), 0, st, logits, temperatures, cmax, csum,
             hist_cnt, hist_mass, R, V, chunks);
  DIB_CHECK_LAUNCH();
  if (filtered) {
    for (int pass = 0; pass < 4; ++pass) {
      dib_launch(filter_histogram_kernel, dim3(chunks, R), dim3(256), 0, st, logits, temperatures, top_ks,
                 top_ps, (const float*)cmax, (const float*)csum, hist_cnt, hist_mass, pass, R, V, chunks);
      DIB_CHECK_LAUNCH();
    }
  }
  dib_launch(gumbel_pick_kernel, dim3(chunks, R), dim3(256), 0, st, logits, temperatures, seeds,
             sample_pos, keep, top_ks, top_ps, (const unsigned*)hist_cnt,
             (const unsigned long long*)hist_mass, filtered ? thresh : (unsigned*)nullptr,
             (const float*)cmax, (const float*)csum, pv, scratch_i, R, V, chunks);
  DIB_CHECK_LAUNCH();
  dib_launch(argmax_final_kernel, dim3(R), dim3(64), 0, st, (const float*)pv, (const int*)scratch_i, out,
             chunks);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // extern "C"
