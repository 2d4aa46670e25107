// True float32 matrix product on the CUDA cores: C[M,N] = A[M,K] * W[N,K]^T.
//
// This is the matrix product of the 32-bit path: plain FMA, no tensor cores and
// no reduced-precision mode.  Every output element is the sum over k in index
// order 0..K-1 in one accumulator, so a row's result does not depend on M or on
// the tile it falls in: the same token gives the same bits in any batch.
//
// Tile 64x64x16, 256 threads, 4x4 outputs per thread.  Any M, N, K.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_fp32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                 int M, int N, int K) {
  pdl_prologue(A);
  __shared__ float sA[BK][BM + 4];
  __shared__ float sW[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / BK, kk = idx % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      sA[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.f;
      sW[kk][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = sA[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = sW[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn < N) C[(size_t)gm * N + gn] = acc[i][j];
    }
  }
}

}  // namespace

extern "C" int dib_gemm_fp32(const float* A, const float* W, float* C, int M, int N, int K,
                             cudaStream_t st) {
  if (M == 0 || N == 0) return DIB_OK;
  if (K <= 0) return DIB_BAD_SIZE;
  dim3 grid(ceil_div_host(N, BN), ceil_div_host(M, BM));
  if (grid.y > 65535) return DIB_BAD_SIZE;
  dib_launch(gemm_fp32_kernel, dim3(grid), dim3(256), 0, st, A, W, C, M, N, K);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}
