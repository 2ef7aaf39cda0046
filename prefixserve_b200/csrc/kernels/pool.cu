// The device memory of the cache pages, owned by this library rather than by a tensor library's caching allocator:
// one allocation per cache entry, made once when the cache manager is built and freed when it goes, at an address
// that never moves (captured steps have it baked in) and that no allocator can hand to anything else in between.
// The reference keeps its pool in one tensor of its engine (prefixserve/llama_engine.py:114-117 of PrefixServe); the
// survey of it asked for the pool to belong to the native side.  Python wraps the address without copying.
#include "common.cuh"

// Allocates ``bytes`` and fills them with zeros.  *out receives the address.
PSB_API int psb_pool_alloc(long long bytes, void** out) {
  if (bytes < 1 || !out) PSB_REFUSE("pool_alloc: %lld bytes", bytes);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();  // an allocation that fails is an answer, not a state to stay in
    PSB_REFUSE("pool_alloc: cannot allocate %.2f GB for cache pages: %s", bytes / 1e9, cudaGetErrorString(e));
  }
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    PSB_REFUSE("pool_alloc: cannot clear the pages: %s", cudaGetErrorString(e));
  }
  *out = p;
  return 0;
}

PSB_API int psb_pool_free(void* p) {
  if (!p) return 0;
  cudaError_t e = cudaFree(p);  // waits for the device: nothing that still reads the pages is cut short
  if (e != cudaSuccess) PSB_REFUSE("pool_free: %s", cudaGetErrorString(e));
  return 0;
}
