// C[M,N] (+)= A[M,K] * W[N,K]^T with float32 multiply-adds on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no
// reduced-precision mode), and the fallback for operand type mixes the
// tensor-core kernels do not take (e.g. bfloat16 activations against a weight
// the checkpoint stores in float32).  Every output element is the sum over k
// in increasing order, whatever M and N are and wherever the tile lies, so a
// token's result does not depend on what else is in the batch.
//
// Stands where the reference calls F.linear (prefixserve/model/llama.py:113,
// :117, :120, :121, :126).
#include "common.cuh"

namespace {

constexpr int TILE = 64;   // output tile is TILE x TILE
constexpr int BK = 16;
constexpr int THREADS = 256;  // 16 x 16 threads, 4 x 4 outputs each

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(THREADS)
gemm_nt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
               int64_t lda, int64_t ldw, int64_t ldc, int accumulate) {
  __shared__ float sa[BK][TILE + 4];
  __shared__ float sw[BK][TILE + 4];
  pdl_trigger();
  pdl_wait();
  const int m0 = blockIdx.y * TILE, n0 = blockIdx.x * TILE;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  // each thread loads 4 elements of each tile per step: row = id / 4 ... 64 rows x 16 cols = 1024 = 256 * 4
  const int lrow = threadIdx.x >> 2;          // 0..63
  const int lcol = (threadIdx.x & 3) * 4;     // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lcol + j;
      const int m = m0 + lrow, n = n0 + lrow;
      sa[lcol + j][lrow] = (m < M && k < K) ? to_float<TA>(A[(size_t)m * lda + k]) : 0.f;
      sw[lcol + j][lrow] = (n < N && k < K) ? to_float<TW>(W[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sa[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sw[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      TC* c = C + (size_t)m * ldc + n;
      float v = acc[i][j];
      if (accumulate) v += to_float<TC>(*c);
      *c = from_float<TC>(v);
    }
  }
}

template <typename TA, typename TW>
int launch_c(const void* a, const void* w, void* c, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldw,
             int64_t ldc, int accumulate, cudaStream_t stream) {
  dim3 grid((N + TILE - 1) / TILE, (M + TILE - 1) / TILE);
  if (grid.y > 65535) PSB_REFUSE("gemm_nt: M=%d is too large for this kernel", M);
  PSB_DISPATCH_DTYPE(c_dtype, TC, {
    psb_launch(gemm_nt_kernel<TA, TW, TC>, grid, dim3(THREADS), 0, stream, (const TA*)a, (const TW*)w, (TC*)c, M, N, K, lda, ldw, ldc, accumulate);
  });
  return 0;
}

}  // namespace

PSB_API int psb_gemm_nt(const void* a, int a_dtype, const void* w, int w_dtype, void* c, int c_dtype, int M, int N, int K,
                        int64_t lda, int64_t ldw, int64_t ldc, int accumulate, cudaStream_t stream) {
  if (M < 0 || N < 1 || K < 1) PSB_REFUSE("gemm_nt: bad sizes M=%d N=%d K=%d", M, N, K);
  if (lda < K || ldw < K || ldc < N) PSB_REFUSE("gemm_nt: a leading dimension is smaller than its row");
  if (M == 0) return 0;
  int rc = 0;
  PSB_DISPATCH_DTYPE(a_dtype, TA, {
    PSB_DISPATCH_DTYPE(w_dtype, TW, {
      rc = launch_c<TA, TW>(a, w, c, c_dtype, M, N, K, lda, ldw, ldc, accumulate, stream);
    });
  });
  if (rc) return rc;
  PSB_LAUNCH_CHECK("gemm_nt");
  return 0;
}
