// Test-only kernel: a bounded wait of the package (mbar_wait of csrc/common.cuh) on an
// mbarrier that nothing ever arrives on and that no copy targets.  After `limit_ns` the
// wait gives up, the thread sets this library's error word and the kernel returns: the
// launch ends, the context stays usable, and the host learns of it from the word.  With
// `arrive` set the thread arrives on the barrier itself first, so the wait succeeds.
#include "common.cuh"

__device__ int test_wait_error_word = 0;

__global__ void wait_kernel(unsigned long long limit_ns, int arrive) {
  __shared__ unsigned long long bar;
  if (threadIdx.x != 0) return;
  const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(1));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (arrive) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
  if (!mbar_wait(&bar, 0, limit_ns)) atomicExch(&test_wait_error_word, 7);
}

extern "C" {

int test_wait_launch(unsigned long long limit_ns, int arrive, cudaStream_t st) {
  wait_kernel<<<1, 32, 0, st>>>(limit_ns, arrive);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
int test_wait_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, test_wait_error_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
int test_wait_status_clear() {
  const int v = 0;
  return cudaMemcpyToSymbol(test_wait_error_word, &v, sizeof(int)) == cudaSuccess ? 0 : -1;
}

}  // extern "C"
