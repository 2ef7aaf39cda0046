// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores, for many rows (prefill).
//
// Persistent, warp-specialised CTAs (one per SM), 192 threads:
//   warp 0      producer: one lane issues TMA loads (cp.async.bulk.tensor.2d) of a 128x64 tile of A and two 128x64
//               tiles of W per stage into 128-byte-swizzled shared memory; completion by mbarrier transaction bytes;
//   warp 1      MMA: one lane issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=256, K=16; four per stage) with
//               shared-memory matrix descriptors; accumulators are float32 in tensor memory (two buffers of 256
//               columns, so the epilogue of one tile overlaps the main loop of the next); tcgen05.commit hands stages
//               back to the producer and finished accumulators to the epilogue;
//   warps 2..5  epilogue: tcgen05.ld (32 lanes x 32 columns per instruction) -> registers -> bfloat16 -> global.
// The two W tiles of a stage are rows [n0, n0+128) and [n1, n1+128): for a plain product n1 = n0 + 128; for the
// gated feed-forward n0 indexes the gate rows and n1 the matching up rows, and the epilogue writes
// silu(gate) * up, so the [T, 2I] intermediate never exists (prefixserve/model/llama.py:120-121 of PrefixServe;
// F.linear at :113, :117).
//
// Rows of A past M, rows of W past N and columns past K are filled with zeros by the TMA unit (K only needs to be a
// multiple of 8: a 16-byte row pitch).  No cluster, no multicast: every CTA loads its own tiles.
//
// Every wait on an mbarrier is bounded.  If one runs out, the CTA raises a flag that all its warps poll, stops
// issuing work, pauses long enough for copies in flight to land, frees its tensor memory and returns; the host finds
// a non-zero status word (psb_tcgen05_status) and raises.  That path has never been taken in testing; it exists so
// that a defect cannot hang the GPU.
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BN_HALF = 128, BN = 2 * BN_HALF, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int B_BYTES = BN * BK * 2;        // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;              // two accumulator buffers of BN float32 columns

// shared memory: [stages][A | B] (1024-byte aligned), then barriers and the tensor-memory address
struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + (int)sizeof(Barriers);

// status word: 0 ok; otherwise which wait gave up (1 producer, 2 mma, 3 epilogue, 4 mma/acc)
using namespace tc;
constexpr uint32_t INSTR_DESC = instr_desc(BM, BN, false);  // M=128, N=256, both operands K-major

// gated: 0 plain (C[M, N], tile columns [n0, n0+128) and [n0+128, n0+256)); 1 gated (C[M, I], W = [gate; up], tile
// columns [n0, n0+128) of the gate and the same of the up rows).
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    __nv_bfloat16* __restrict__ C, int M, int N_out, int K, int ldc, int up_offset, int gated) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(tiles + STAGES * STAGE_BYTES);
  volatile uint32_t* abort = &bars->abort;
  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;  // the warp's role is the same for all its lanes

  const int n_span = gated ? BN_HALF : BN;  // output columns one tile covers
  const int m_blocks = (M + BM - 1) / BM;
  const int n_blocks = (N_out + n_span - 1) / n_span;
  const int tiles_total = m_blocks * n_blocks;
  const int k_blocks = (K + BK - 1) / BK;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 4);  // one arrival per epilogue warp
    }
    bars->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {  // one warp allocates (and later frees) the tensor memory
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  pdl_wait();  // A is the preceding kernel's output

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tiles_total; tile += gridDim.x) {
        const int m0 = (tile % m_blocks) * BM;
        const int n0 = (tile / m_blocks) * n_span;
        const int n1 = gated ? up_offset + n0 : n0 + BN_HALF;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&bars->empty[stage], phase ^ 1, abort, 1);
          if (!ok) break;
          unsigned char* a_dst = tiles + stage * STAGE_BYTES;
          unsigned char* b_dst = a_dst + A_BYTES;
          mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, kb * BK, m0, &bars->full[stage]);
          tma_load_2d(b_dst, &map_w, kb * BK, n0, &bars->full[stage]);
          tma_load_2d(b_dst + BN_HALF * BK * 2, &map_w, kb * BK, n1, &bars->full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA
    // The whole warp runs this loop and waits on the barriers; each tensor-core instruction is issued by one elected
    // lane (tcgen05.cuh says why).
    {
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tiles_total; tile += gridDim.x, ++local) {
        const uint32_t buf = local & 1, use = local >> 1;  // accumulator buffer and how often it has been used
        ok = mbar_wait(&bars->acc_empty[buf], (use & 1) ^ 1, abort, 4);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after();
        const uint32_t acc = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&bars->full[stage], phase, abort, 2);  // filled by TMA: no tensor-memory fence needed
          if (!ok) break;
          const uint64_t da = smem_desc(smem_u32(tiles + stage * STAGE_BYTES));
          const uint64_t db = smem_desc(smem_u32(tiles + stage * STAGE_BYTES + A_BYTES));
          const uint32_t hi = (uint32_t)(da >> 32), a_lo = (uint32_t)da, b_lo = (uint32_t)db;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 elements = 32 bytes further along K inside the swizzled 128-byte rows: 2 in the address field
            if (elect_one()) mma_f16_split(acc, a_lo + 2 * k, hi, b_lo + 2 * k, hi, INSTR_DESC, (kb | k) != 0);
          }
          if (elect_one()) mma_commit(&bars->empty[stage]);  // arrives when the MMAs that read this stage are done
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) mma_commit(&bars->acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // a warp may only read tensor-memory lanes [32*(warp%4), +32)
    uint32_t local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < tiles_total; tile += gridDim.x, ++local) {
      const uint32_t buf = local & 1, use = local >> 1;
      const int m0 = (tile % m_blocks) * BM;
      const int n0 = (tile / m_blocks) * n_span;
      ok = mbar_wait(&bars->acc_full[buf], use & 1, abort, 3);
      if (!ok) break;
      fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      __nv_bfloat16* crow = C + (size_t)row * ldc;
      if (gated) {
#pragma unroll 1
        for (int c = 0; c < BN_HALF; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c, g);
          tmem_ld32(taddr + BN_HALF + c, u);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n0 + c + j;
              uint32_t packed[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                // the reference rounds both projections to bfloat16 before the activation
                const float g0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j + 2 * q])));
                const float g1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j + 2 * q + 1])));
                const float u0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j + 2 * q])));
                const float u1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j + 2 * q + 1])));
                packed[q] = pack2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
              }
              if (col + 8 <= N_out && (ldc & 7) == 0) {
                *reinterpret_cast<uint4*>(crow + col) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              } else {
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(packed);
                for (int q = 0; q < 8; ++q)
                  if (col + q < N_out) crow[col + q] = e[q];
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + c, v);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n0 + c + j;
              uint32_t packed[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) packed[q] = pack2(__uint_as_float(v[j + 2 * q]), __uint_as_float(v[j + 2 * q + 1]));
              if (col + 8 <= N_out && (ldc & 7) == 0) {
                *reinterpret_cast<uint4*>(crow + col) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              } else {
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(packed);
                for (int q = 0; q < 8; ++q)
                  if (col + q < N_out) crow[col + q] = e[q];
              }
            }
          }
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);  // this warp has read its part of the buffer
    }
  }

  if (*abort) {
    // something gave up: give copies in flight time to land before the shared memory is handed to another CTA
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  fence_before();
  __syncthreads();
  if (warp == 2) {
    fence_after();
    tmem_free(tmem_base, TMEM_COLS);
  }
}

// ---- host side -----------------------------------------------------------------------------------------------
// row-major [rows, K] bfloat16 matrix, box of 64 columns x box_rows rows
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  const int r = make_map_bf16(map, base, (uint64_t)rows, (uint64_t)K, (uint64_t)K, box_rows);
  if (r == -1) PSB_REFUSE("gemm_tcgen05: the driver does not export cuTensorMapEncodeTiled");
  if (r != 0) PSB_REFUSE("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d)", r, rows, K);
  return 0;
}

int launch(const void* a, const void* w, void* c, int M, int w_rows, int N_out, int K, int up_offset, int gated, int sms,
           cudaStream_t stream) {
  if (M < 1 || N_out < 1 || K < 8 || K % 8) PSB_REFUSE("gemm_tcgen05: needs K a multiple of 8 (M=%d N=%d K=%d)", M, N_out, K);
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15) PSB_REFUSE("gemm_tcgen05: operands must be 16-byte aligned");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) PSB_REFUSE("gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  CUtensorMap map_a, map_w;
  if (int rc = make_map(&map_a, a, M, K, BM)) return rc;
  if (int rc = make_map(&map_w, w, w_rows, K, BN_HALF)) return rc;
  const int n_span = gated ? BN_HALF : BN;
  const int tiles = ((M + BM - 1) / BM) * ((N_out + n_span - 1) / n_span);
  const int grid = tiles < sms ? tiles : sms;
  psb_launch(gemm_tcgen05_kernel, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, stream, map_a, map_w, (__nv_bfloat16*)c, M,
             N_out, K, N_out, up_offset, gated);
  PSB_LAUNCH_CHECK("gemm_tcgen05");
  return 0;
}

}  // namespace

// C[M,N] = A[M,K] W[N,K]^T, all bfloat16 row-major, K % 8 == 0.  sms: CTAs to launch at most (the SM count).
PSB_API int psb_gemm_tcgen05(const void* a, const void* w, void* c, int M, int N, int K, int sms, cudaStream_t stream) {
  return launch(a, w, c, M, N, N, K, 0, 0, sms, stream);
}

// act[M,I] = silu(A Wg^T) * (A Wu^T) for W = [Wg; Wu] of shape [2I, K].
PSB_API int psb_gemm_tcgen05_gated(const void* a, const void* w, void* act, int M, int I, int K, int sms, cudaStream_t stream) {
  return launch(a, w, act, M, 2 * I, I, K, I, 1, sms, stream);
}

// 0 while no bounded wait has ever run out on the current device; reading it synchronises with the device.
PSB_API int psb_tcgen05_status() {
  return tc::read_status();
}
