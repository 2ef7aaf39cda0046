// y[M,N] = x[M,K] * W[N,K]^T for a handful of rows (decode): bound by reading W once from HBM.
//
// The product is computed transposed on the tensor cores (mma.sync m16n8k16, float32
// accumulation): 16 rows of W are the "A" tile, 8 rows of x the "B" tile, so one warp
// instruction yields y^T[16 x 8].  Weights go from global memory straight into operand
// registers, 16 bytes per lane: lane (g, t) reads 8 consecutive k of W rows g and g+8,
// and the same 8 k of x row g; since a dot product may add its terms in any order, those
// 8 values serve as the (2t, 2t+1, 2t+8, 2t+9) slots of two consecutive k16 steps.  Every
// W row is therefore read in whole 64-byte runs, and nothing is staged in shared memory.
//
// A CTA works on one 16-row tile of W at a time (two tiles in the gated variant: the gate rows
// and the matching up rows); its warps split K among themselves and add their partial tiles
// through shared memory in a fixed order, so the result does not depend on timing.
//
// Variants: plain store (bfloat16 or float32 output), and gate/up with act(gate)*up in
// the epilogue, which writes [M, I] directly (prefixserve/model/llama.py:120-121 of
// PrefixServe; F.linear at :113, :117, :126).  (A variant with one CTA per tile, for up to 64
// rows, was measured against the library product at 17 to 64 rows, lost at every shape, and
// is gone.)
#include "common.cuh"

namespace {


__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// weights are read once: keep them out of L1 so that x stays there
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

}  // namespace

// ------------------------------------------------------------------------------------------------------------------
// Streaming variant for at most 16 rows of x: persistent CTAs (one per SM) of 16 warps that split K; every lane feeds
// the 16-byte pieces it will need through a ring of its own in shared memory with cp.async, so the loads of the next
// row tile are already in flight while the current one is reduced and stored.  Same operand layout and the same
// fixed-order reduction as above.
namespace {

constexpr int SW = 16;  // warps per CTA

template <int MT, int TILES>
struct StreamShape {
  static constexpr int PIECES = 2 * TILES + MT;                 // per lane per k chunk
  static constexpr int STAGES = PIECES <= 3 ? 8 : (PIECES == 4 ? 6 : (PIECES == 5 ? 4 : 3));  // ring + partials <= 227 KB
  static constexpr int RING_BYTES = SW * STAGES * PIECES * 32 * 16;
  static constexpr int PART_BYTES = 2 * SW * TILES * 16 * (8 * MT + 1) * 4;  // two buffers of partial tiles
  static constexpr int SMEM_BYTES = RING_BYTES + PART_BYTES;
};

__device__ __forceinline__ void cp16_cg(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp16_ca_zfill(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

template <int MT, int TILES, typename TOut>
__global__ void __launch_bounds__(SW * 32, 1)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, TOut* __restrict__ y, int M, int N,
                   int K, int ldy, int up_offset, int act) {
  using Shape = StreamShape<MT, TILES>;
  constexpr int STAGES = Shape::STAGES, PIECES = Shape::PIECES;
  constexpr uint32_t STAGE_BYTES = PIECES * 32 * 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // this lane's ring: slot(stage, piece) = ring0 + stage*STAGE_BYTES + piece*512
  const uint32_t ring0 = (uint32_t)__cvta_generic_to_shared(smem_raw) + (uint32_t)warp * STAGES * STAGE_BYTES + lane * 16;
  typedef float PartTile[TILES][16][8 * MT + 1];
  PartTile* part = reinterpret_cast<PartTile*>(smem_raw + Shape::RING_BYTES);  // [2][SW]

  const int tiles = (N + 15) / 16;
  const int my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int chunks = K / 32;
  const int per = chunks / SW, extra = chunks % SW;
  const int c_begin = warp * per + min(warp, extra);
  const int cpw = per + (warp < extra ? 1 : 0);  // chunks of every tile that fall to this warp
  const int units = my_tiles * cpw;

  // sources, advanced as units are issued (no divisions in the loop)
  const __nv_bfloat16* xsrc[MT];
  int xbytes[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    const int m = 8 * j + g;
    xbytes[j] = m < M ? 16 : 0;  // rows past M are zero-filled
    xsrc[j] = x + (size_t)(m < M ? m : 0) * K + c_begin * 32 + t * 8;
  }
  const __nv_bfloat16* wsrc[2];   // rows g and g+8 of the tile being issued (first of the TILES row groups)
  auto tile_rows = [&](int ti) {
    const int row0 = (blockIdx.x + ti * gridDim.x) * 16;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int row = row0 + g + 8 * r;
      row = row < N ? row : N - 1;  // rows past N are computed on a copy of the last row and never stored
      wsrc[r] = W + (size_t)row * K + c_begin * 32 + t * 8;
    }
  };
  const size_t up_elems = (size_t)up_offset * K;
  int issued = 0, issue_c = 0, issue_ti = 0;
  uint32_t issue_slot = ring0;
  int issue_stage = 0;
  if (units > 0) tile_rows(0);
  // with_x false: only the weights (they never change; x comes from the preceding kernel and must wait for it)
  auto issue = [&](bool with_w, bool with_x) {
    if (with_w) {
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        cp16_cg(issue_slot + (2 * tl) * 512, wsrc[0] + tl * up_elems + issue_c * 32);
        cp16_cg(issue_slot + (2 * tl + 1) * 512, wsrc[1] + tl * up_elems + issue_c * 32);
      }
    }
    if (with_x) {
#pragma unroll
      for (int j = 0; j < MT; ++j) cp16_ca_zfill(issue_slot + (2 * TILES + j) * 512, xsrc[j] + issue_c * 32, xbytes[j]);
    }
    ++issued;
    if (++issue_c == cpw) {
      issue_c = 0;
      if (++issue_ti < my_tiles) tile_rows(issue_ti);
    }
    if (++issue_stage == STAGES) { issue_stage = 0; issue_slot = ring0; } else issue_slot += STAGE_BYTES;
  };
  // The ring is primed in two passes over the same first STAGES-1 units: weights before the dependency wait,
  // x after it.  All of it lands in the first commit groups, which the first wait_group covers.
  pdl_trigger();
#pragma unroll
  for (int u = 0; u < STAGES - 1; ++u)
    if (issued < units) issue(true, false);
  pdl_wait();
  issued = 0; issue_c = 0; issue_ti = 0; issue_slot = ring0; issue_stage = 0;
  if (units > 0) tile_rows(0);
#pragma unroll
  for (int u = 0; u < STAGES - 1; ++u) {
    if (issued < units) issue(false, true);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }

  uint32_t read_slot = ring0;
  int read_stage = 0;
  for (int ti = 0; ti < my_tiles; ++ti) {
    float acc[TILES][MT][4];
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[tl][j][0] = acc[tl][j][1] = acc[tl][j][2] = acc[tl][j][3] = 0.f;
    for (int cc = 0; cc < cpw; ++cc) {
      if (issued < units) issue(true, true);
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1) : "memory");
      uint4 wv[TILES][2], xv[MT];
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        wv[tl][0] = lds16(read_slot + (2 * tl) * 512);
        wv[tl][1] = lds16(read_slot + (2 * tl + 1) * 512);
      }
#pragma unroll
      for (int j = 0; j < MT; ++j) xv[j] = lds16(read_slot + (2 * TILES + j) * 512);
      if (++read_stage == STAGES) { read_stage = 0; read_slot = ring0; } else read_slot += STAGE_BYTES;
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          mma_bf16(acc[tl][j], wv[tl][0].x, wv[tl][1].x, wv[tl][0].y, wv[tl][1].y, xv[j].x, xv[j].y);
          mma_bf16(acc[tl][j], wv[tl][0].z, wv[tl][1].z, wv[tl][0].w, wv[tl][1].w, xv[j].z, xv[j].w);
        }
    }
    PartTile* mine = part + (size_t)(ti & 1) * SW;
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        mine[warp][tl][g][8 * j + 2 * t] = acc[tl][j][0];
        mine[warp][tl][g][8 * j + 2 * t + 1] = acc[tl][j][1];
        mine[warp][tl][g + 8][8 * j + 2 * t] = acc[tl][j][2];
        mine[warp][tl][g + 8][8 * j + 2 * t + 1] = acc[tl][j][3];
      }
    __syncthreads();  // one barrier per tile: the two buffers alternate
    const int row0 = (blockIdx.x + ti * gridDim.x) * 16;
    for (int idx = threadIdx.x; idx < 16 * 8 * MT; idx += SW * 32) {
      const int r = idx & 15, m = idx >> 4;
      const int row = row0 + r;
      if (m >= M || row >= N) continue;
      float v[TILES];
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SW; ++w) sum += mine[w][tl][r][m];
        v[tl] = sum;
      }
      float out;
      if (TILES == 2) {
        const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
        const float up = __bfloat162float(__float2bfloat16_rn(v[TILES - 1]));
        out = gate_act(gate, act) * up;
      } else {
        out = v[0];
      }
      y[(size_t)m * ldy + row] = from_float<TOut>(out);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <int MT, int TILES, typename TOut>
int launch_stream(const void* x, const void* W, void* y, int M, int N, int K, int ldy, int up_offset, int act, int sms, cudaStream_t stream) {
  using Shape = StreamShape<MT, TILES>;
  static PsbPerDevice configured; 
  if (!configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<MT, TILES, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Shape::SMEM_BYTES);
    if (e != cudaSuccess) PSB_REFUSE("gemm_stream: cannot reserve %d bytes of shared memory: %s", Shape::SMEM_BYTES, cudaGetErrorString(e));
    configured.set(); 
  }
  const int tiles = (N + 15) / 16;
  const int grid = tiles < sms ? tiles : sms;
  psb_launch(gemm_stream_kernel<MT, TILES, TOut>, dim3(grid), dim3(SW * 32), (size_t)Shape::SMEM_BYTES, stream,
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)W, (TOut*)y, M, N, K, ldy, up_offset, act);
  return 0;
}

}  // namespace

// y[M,N] = x[M,K] W[N,K]^T for M <= 16 with the streaming kernel; sms: CTAs to launch at most (the SM count).
PSB_API int psb_gemm_stream(const void* x, const void* W, void* y, int out_dtype, int M, int N, int K, int sms, cudaStream_t stream) {
  if (M < 0 || M > 16 || N < 1 || K < 32 || K % 32 || sms < 1) PSB_REFUSE("gemm_stream: needs M <= 16 and K a multiple of 32 (M=%d N=%d K=%d)", M, N, K);
  if (M == 0) return 0;
  int rc;
  if (out_dtype == PSB_F32) rc = M <= 8 ? launch_stream<1, 1, float>(x, W, y, M, N, K, N, 0, 0, sms, stream) : launch_stream<2, 1, float>(x, W, y, M, N, K, N, 0, 0, sms, stream);
  else if (out_dtype == PSB_BF16) rc = M <= 8 ? launch_stream<1, 1, __nv_bfloat16>(x, W, y, M, N, K, N, 0, 0, sms, stream) : launch_stream<2, 1, __nv_bfloat16>(x, W, y, M, N, K, N, 0, 0, sms, stream);
  else PSB_REFUSE("gemm_stream: unknown output dtype %d", out_dtype);
  if (rc) return rc;
  PSB_LAUNCH_CHECK("gemm_stream");
  return 0;
}

PSB_API int psb_gemm_stream_gated(const void* x, const void* W, void* act, int M, int I, int K, int sms, int activation,
                                  cudaStream_t stream) {
  if (!psb_activation_known(activation)) PSB_REFUSE("gemm_stream_gated: activation code %d is not built", activation);
  if (M < 0 || M > 16 || I < 1 || K < 32 || K % 32 || sms < 1) PSB_REFUSE("gemm_stream_gated: needs M <= 16 and K a multiple of 32 (M=%d I=%d K=%d)", M, I, K);
  if (M == 0) return 0;
  const int rc = M <= 8 ? launch_stream<1, 2, __nv_bfloat16>(x, W, act, M, I, K, I, I, activation, sms, stream)
                        : launch_stream<2, 2, __nv_bfloat16>(x, W, act, M, I, K, I, I, activation, sms, stream);
  if (rc) return rc;
  PSB_LAUNCH_CHECK("gemm_stream_gated");
  return 0;
}

// ------------------------------------------------------------------------------------------------------------------
// The streaming product with the preceding residual add + RMSNorm folded in (decode):
//   v = h[rows[m]] + pending[rows[m]]        (float32; written to h_out by CTA 0 when pending is given and rows is not)
//   y[m, n] = rsqrt(mean(v^2) + eps) * sum_k W[n, k] * bf16(v[k] * gain[k])
// A warp's share of K is the same for every row tile it visits, so it computes its bfloat16 operand fragments of
// v * gain once, keeps them in registers, and the ring in shared memory carries weights only.  Each warp also adds up
// the squares of its share of v; the 16 partial sums per row meet in shared memory at the first tile's barrier and
// the scale is applied to the finished sums.  (RMSNorm: prefixserve/model/llama.py:63-69 of PrefixServe; the
// reference rounds the normalised row to bfloat16 and multiplies by the gain, this rounds v * gain and scales after
// the product: the same number of roundings.)
namespace {

template <int MT, int TILES>
struct NormStreamShape {
  static constexpr int PIECES = 2 * TILES;
  static constexpr int STAGES = TILES == 1 ? 8 : (MT == 1 ? 5 : 4);
  static constexpr int RING_BYTES = SW * STAGES * PIECES * 32 * 16;
  static constexpr int PART_BYTES = 2 * SW * TILES * 16 * (8 * MT + 1) * 4;
  static constexpr int SSQ_BYTES = SW * 8 * MT * 4;
  static constexpr int SMEM_BYTES = RING_BYTES + PART_BYTES + SSQ_BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "beyond a CTA's shared memory");
};

template <typename TP>
__device__ __forceinline__ void load8_any(const TP* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8_any<float>(const float* p, float (&o)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_any<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h2[k]);
    o[2 * k] = f.x; o[2 * k + 1] = f.y;
  }
}

// CPW: most k chunks (of 32) a warp may own (K <= 512 * CPW).  ROPE: the epilogue rotates and appends (TILES == 1).
template <int MT, int TILES, int CPW, typename TOut, bool ROPE = false>
__global__ void __launch_bounds__(SW * 32, 1)
gemm_stream_norm_kernel(const float* __restrict__ h_in, const __nv_bfloat16* __restrict__ pending, const float* __restrict__ gain,
                        const int32_t* __restrict__ rows, float* __restrict__ h_out, const __nv_bfloat16* __restrict__ W,
                        TOut* __restrict__ y, int M, int N, int K, int ldy, int up_offset, int act, float eps, RopeArgs rope) {
  using Shape = NormStreamShape<MT, TILES>;
  constexpr int STAGES = Shape::STAGES, PIECES = Shape::PIECES;
  constexpr uint32_t STAGE_BYTES = PIECES * 32 * 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t ring0 = (uint32_t)__cvta_generic_to_shared(smem_raw) + (uint32_t)warp * STAGES * STAGE_BYTES + lane * 16;
  typedef float PartTile[TILES][16][8 * MT + 1];
  PartTile* part = reinterpret_cast<PartTile*>(smem_raw + Shape::RING_BYTES);  // [2][SW]
  float(*ssq_part)[8 * MT] = reinterpret_cast<float(*)[8 * MT]>(smem_raw + Shape::RING_BYTES + Shape::PART_BYTES);  // [SW]

  const int tiles = (N + 15) / 16;
  const int my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int chunks = K / 32;
  const int per = chunks / SW, extra = chunks % SW;
  const int c_begin = warp * per + min(warp, extra);
  const int cpw = per + (warp < extra ? 1 : 0);
  const int units = my_tiles * cpw;

  const __nv_bfloat16* wsrc[2];
  auto tile_rows = [&](int ti) {
    const int row0 = (blockIdx.x + ti * gridDim.x) * 16;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int row = row0 + g + 8 * r;
      row = row < N ? row : N - 1;
      wsrc[r] = W + (size_t)row * K + c_begin * 32 + t * 8;
    }
  };
  const size_t up_elems = (size_t)up_offset * K;
  int issued = 0, issue_c = 0, issue_ti = 0, issue_stage = 0;
  uint32_t issue_slot = ring0;
  if (units > 0) tile_rows(0);
  auto issue = [&]() {
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl) {
      cp16_cg(issue_slot + (2 * tl) * 512, wsrc[0] + tl * up_elems + issue_c * 32);
      cp16_cg(issue_slot + (2 * tl + 1) * 512, wsrc[1] + tl * up_elems + issue_c * 32);
    }
    ++issued;
    if (++issue_c == cpw) {
      issue_c = 0;
      if (++issue_ti < my_tiles) tile_rows(issue_ti);
    }
    if (++issue_stage == STAGES) { issue_stage = 0; issue_slot = ring0; } else issue_slot += STAGE_BYTES;
  };
  // weights never change: prime the ring before waiting for the preceding kernel
  pdl_trigger();
#pragma unroll
  for (int u = 0; u < STAGES - 1; ++u) {
    if (issued < units) issue();
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  // So are the step's own inputs: the thread that will rotate and store pair j of token m (see the epilogue) looks up
  // the token's position and page now, and the angles of each tile while the tile's products run.
  int ep_pos = 0, ep_page = -1;
  float ep_cos = 1.f, ep_sin = 0.f;
  const bool ep_thread = ROPE && threadIdx.x < 8 * 8 * MT && (int)(threadIdx.x >> 3) < M;
  if constexpr (ROPE) {
    if (ep_thread) {
      const int m = threadIdx.x >> 3;
      ep_pos = rope.positions[m];
      ep_page = rope.table[(size_t)rope.token_item[m] * rope.table_width + (ep_pos >> rope.page_shift)];
    }
  }
  pdl_wait();

  // ---- this warp's operand fragments of v * gain, and its share of sum(v^2)
  uint4 xf[CPW][MT];
  {
    float ssq[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) ssq[j] = 0.f;
#pragma unroll
    for (int cc = 0; cc < CPW; ++cc) {
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        const int m = 8 * j + g;
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (cc < cpw && m < M) {
          const int src = rows ? rows[m] : m;
          const size_t at = (size_t)src * K + (size_t)(c_begin + cc) * 32 + t * 8;
          float v[8], gn[8];
          load8_any<float>(h_in + at, v);
          if (pending) {
            float p[8];
            load8_any<__nv_bfloat16>(pending + at, p);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] += p[k];
            if (h_out && blockIdx.x == 0) {
              *reinterpret_cast<float4*>(h_out + at) = make_float4(v[0], v[1], v[2], v[3]);
              *reinterpret_cast<float4*>(h_out + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
          }
          load8_any<float>(gain + (size_t)(c_begin + cc) * 32 + t * 8, gn);
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            ssq[j] += v[2 * k] * v[2 * k] + v[2 * k + 1] * v[2 * k + 1];
            o2[k] = __floats2bfloat162_rn(v[2 * k] * gn[2 * k], v[2 * k + 1] * gn[2 * k + 1]);
          }
        }
        xf[cc][j] = packed;
      }
    }
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      float s = ssq[j];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (t == 0) ssq_part[warp][8 * j + g] = s;
    }
  }

  uint32_t read_slot = ring0;
  int read_stage = 0;
  for (int ti = 0; ti < my_tiles; ++ti) {
    if constexpr (ROPE) {
      const int row0 = (blockIdx.x + ti * gridDim.x) * 16;
      if (ep_thread && rope.cos_t && row0 < (rope.hq + rope.hkv) * rope.D) {
        const int block = (row0 % rope.D) >> 4, j = threadIdx.x & 7;
        const int safe = ep_pos < 0 ? 0 : (ep_pos >= rope.max_positions ? rope.max_positions - 1 : ep_pos);
        ep_cos = rope.cos_t[(size_t)safe * (rope.D >> 1) + block * 8 + j];
        ep_sin = rope.sin_t[(size_t)safe * (rope.D >> 1) + block * 8 + j];
      }
    }
    float acc[TILES][MT][4];
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[tl][j][0] = acc[tl][j][1] = acc[tl][j][2] = acc[tl][j][3] = 0.f;
#pragma unroll
    for (int cc = 0; cc < CPW; ++cc) {
      if (cc < cpw) {
        if (issued < units) issue();
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1) : "memory");
        uint4 wv[TILES][2];
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
          wv[tl][0] = lds16(read_slot + (2 * tl) * 512);
          wv[tl][1] = lds16(read_slot + (2 * tl + 1) * 512);
        }
        if (++read_stage == STAGES) { read_stage = 0; read_slot = ring0; } else read_slot += STAGE_BYTES;
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            mma_bf16(acc[tl][j], wv[tl][0].x, wv[tl][1].x, wv[tl][0].y, wv[tl][1].y, xf[cc][j].x, xf[cc][j].y);
            mma_bf16(acc[tl][j], wv[tl][0].z, wv[tl][1].z, wv[tl][0].w, wv[tl][1].w, xf[cc][j].z, xf[cc][j].w);
          }
      }
    }
    PartTile* mine = part + (size_t)(ti & 1) * SW;
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        mine[warp][tl][g][8 * j + 2 * t] = acc[tl][j][0];
        mine[warp][tl][g][8 * j + 2 * t + 1] = acc[tl][j][1];
        mine[warp][tl][g + 8][8 * j + 2 * t] = acc[tl][j][2];
        mine[warp][tl][g + 8][8 * j + 2 * t + 1] = acc[tl][j][3];
      }
    __syncthreads();  // also makes every warp's sum of squares visible (written before the first of these barriers)
    const int row0 = (blockIdx.x + ti * gridDim.x) * 16;
    if constexpr (ROPE) {
      // a thread takes one pair (rows j and j+8 of the tile) of one token (8 * 8 * MT <= the CTA's threads)
      if (ep_thread && row0 < N) {
        const int j = threadIdx.x & 7, m = threadIdx.x >> 3;
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < SW; ++w) total += ssq_part[w][m];
        const float inv = rsqrtf(total / (float)K + eps);
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int w = 0; w < SW; ++w) { lo += mine[w][0][j][m]; hi += mine[w][0][j + 8][m]; }
        // what a separate projection would have stored in bfloat16 before the rotary kernel read it
        lo = __bfloat162float(__float2bfloat16_rn(lo * inv));
        hi = __bfloat162float(__float2bfloat16_rn(hi * inv));
        const int D = rope.D, q_cols = rope.hq * D, k_cols = rope.hkv * D;
        const int pos = ep_pos, page = ep_page;
        if (row0 < q_cols + k_cols) {
          const int within = row0 < q_cols ? row0 : row0 - q_cols;
          const int head = within / D, block = (within - head * D) >> 4;
          if (rope.cos_t) {
            float a, b;
            rotate_pair(lo, hi, ep_cos, ep_sin, a, b);
            lo = a; hi = b;
          }
          __nv_bfloat16* dst = nullptr;
          if (row0 < q_cols) {
            dst = rope.q_out + ((size_t)m * rope.hq + head) * D;
          } else {
            if (page >= 0 && page < rope.num_pages)  // the host checks tables before launch; a bad id is skipped
              dst = rope.kv + ((((size_t)page * 2) * rope.hkv + head) << rope.page_shift) * D + (size_t)(pos & ((1 << rope.page_shift) - 1)) * D;
          }
          if (dst) {
            dst[block * 16 + j] = __float2bfloat16_rn(lo);
            dst[block * 16 + 8 + j] = __float2bfloat16_rn(hi);
          }
        } else {
          const int within = row0 - q_cols - k_cols;
          const int head = within / D, d0 = within - head * D;
          if (page >= 0 && page < rope.num_pages) {
            __nv_bfloat16* dst = rope.kv + ((((size_t)page * 2 + 1) * rope.hkv + head) << rope.page_shift) * D +
                                 (size_t)(pos & ((1 << rope.page_shift) - 1)) * D;
            dst[d0 + j] = __float2bfloat16_rn(lo);
            dst[d0 + 8 + j] = __float2bfloat16_rn(hi);
          }
        }
      }
    } else {
    for (int idx = threadIdx.x; idx < 16 * 8 * MT; idx += SW * 32) {
      const int r = idx & 15, m = idx >> 4;
      const int row = row0 + r;
      if (m >= M || row >= N) continue;
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < SW; ++w) total += ssq_part[w][m];
      const float inv = rsqrtf(total / (float)K + eps);
      float v[TILES];
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SW; ++w) sum += mine[w][tl][r][m];
        v[tl] = sum * inv;
      }
      float out;
      if (TILES == 2) {
        const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
        const float up = __bfloat162float(__float2bfloat16_rn(v[TILES - 1]));
        out = gate_act(gate, act) * up;
      } else {
        out = v[0];
      }
      y[(size_t)m * ldy + row] = from_float<TOut>(out);
    }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <int MT, int TILES, int CPW, typename TOut, bool ROPE = false>
int launch_norm_stream(const void* h_in, const void* pending, const void* gain, const void* rows, void* h_out, const void* W,
                       void* y, int M, int N, int K, int ldy, int up_offset, int act, float eps, int sms, cudaStream_t stream,
                       const RopeArgs& rope = RopeArgs{}) {
  using Shape = NormStreamShape<MT, TILES>;
  static PsbPerDevice configured; 
  if (!configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_norm_kernel<MT, TILES, CPW, TOut, ROPE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Shape::SMEM_BYTES);
    if (e != cudaSuccess) PSB_REFUSE("gemm_stream_norm: cannot reserve %d bytes of shared memory: %s", Shape::SMEM_BYTES, cudaGetErrorString(e));
    configured.set(); 
  }
  const int tiles = (N + 15) / 16;
  const int grid = tiles < sms ? tiles : sms;
  psb_launch(gemm_stream_norm_kernel<MT, TILES, CPW, TOut, ROPE>, dim3(grid), dim3(SW * 32), (size_t)Shape::SMEM_BYTES, stream,
             (const float*)h_in, (const __nv_bfloat16*)pending, (const float*)gain, (const int32_t*)rows, (float*)h_out,
             (const __nv_bfloat16*)W, (TOut*)y, M, N, K, ldy, up_offset, act, eps, rope);
  return 0;
}

template <int TILES, typename TOut>
int dispatch_norm_stream(const void* h_in, const void* pending, const void* gain, const void* rows, void* h_out, const void* W,
                         void* y, int M, int N, int K, int ldy, int up_offset, int act, float eps, int sms, cudaStream_t stream) {
  const int cpw = (K / 32 + SW - 1) / SW;  // the most chunks any warp owns
#define PSB_NS(MT, CPW) launch_norm_stream<MT, TILES, CPW, TOut>(h_in, pending, gain, rows, h_out, W, y, M, N, K, ldy, up_offset, act, eps, sms, stream)
  if (M <= 8) {
    if (cpw <= 4) return PSB_NS(1, 4);
    if (cpw <= 8) return PSB_NS(1, 8);
    if (cpw <= 16) return PSB_NS(1, 16);
  } else if (M <= 16) {
    if (cpw <= 4) return PSB_NS(2, 4);
    if (cpw <= 8) return PSB_NS(2, 8);
  }
#undef PSB_NS
  PSB_REFUSE("gemm_stream_norm: M=%d K=%d is beyond this kernel (M <= 8 with K <= 8192, or M <= 16 with K <= 4096)", M, K);
}

int dispatch_norm_stream_rope(const void* h_in, const void* pending, const void* gain, void* h_out, const void* W, int M, int N,
                              int K, float eps, int sms, cudaStream_t stream, const RopeArgs& rope) {
  const int cpw = (K / 32 + SW - 1) / SW;
#define PSB_NSR(MT, CPW) launch_norm_stream<MT, 1, CPW, __nv_bfloat16, true>(h_in, pending, gain, nullptr, h_out, W, nullptr, M, N, K, N, 0, 0, eps, sms, stream, rope)
  if (M <= 8) {
    if (cpw <= 4) return PSB_NSR(1, 4);
    if (cpw <= 8) return PSB_NSR(1, 8);
    if (cpw <= 16) return PSB_NSR(1, 16);
  } else if (M <= 16) {
    if (cpw <= 4) return PSB_NSR(2, 4);
    if (cpw <= 8) return PSB_NSR(2, 8);
  }
#undef PSB_NSR
  PSB_REFUSE("gemm_stream_norm_rope: M=%d K=%d is beyond this kernel (M <= 8 with K <= 8192, or M <= 16 with K <= 4096)", M, K);
}

}  // namespace

// 1 if psb_gemm_stream_norm takes the shape, else 0.
PSB_API int psb_gemm_stream_norm_supported(int M, int K) {
  if (M < 1 || K < 32 || K % 32) return 0;
  const int cpw = (K / 32 + SW - 1) / SW;
  return (M <= 8 && cpw <= 16) || (M <= 16 && cpw <= 8) ? 1 : 0;
}

// y[M,N] = rmsnorm(h_in[rows] + pending[rows]; gain, eps) W[N,K]^T; h_out (optional, rows absent) receives the sum.
PSB_API int psb_gemm_stream_norm(const void* h_in, const void* pending, const void* gain, const void* rows, void* h_out,
                                 const void* W, void* y, int out_dtype, int M, int N, int K, float eps, int sms,
                                 cudaStream_t stream) {
  if (!psb_gemm_stream_norm_supported(M, K) || N < 1 || sms < 1) PSB_REFUSE("gemm_stream_norm: shape M=%d N=%d K=%d is not taken", M, N, K);
  if (rows && h_out) PSB_REFUSE("gemm_stream_norm: the stream cannot be updated through a row selection");
  if (!(eps > 0.f)) PSB_REFUSE("gemm_stream_norm: eps must be positive");
  int rc;
  if (out_dtype == PSB_F32) rc = dispatch_norm_stream<1, float>(h_in, pending, gain, rows, h_out, W, y, M, N, K, N, 0, 0, eps, sms, stream);
  else if (out_dtype == PSB_BF16) rc = dispatch_norm_stream<1, __nv_bfloat16>(h_in, pending, gain, rows, h_out, W, y, M, N, K, N, 0, 0, eps, sms, stream);
  else PSB_REFUSE("gemm_stream_norm: unknown output dtype %d", out_dtype);
  if (rc) return rc;
  PSB_LAUNCH_CHECK("gemm_stream_norm");
  return 0;
}

// act[M,I] = f(x Wg^T) * (x Wu^T), f the activation named by its code, with x = rmsnorm(h_in + pending) as above, W = [Wg; Wu].
PSB_API int psb_gemm_stream_norm_gated(const void* h_in, const void* pending, const void* gain, void* h_out, const void* W,
                                       void* act, int M, int I, int K, float eps, int sms, int activation, cudaStream_t stream) {
  if (!psb_activation_known(activation)) PSB_REFUSE("gemm_stream_norm_gated: activation code %d is not built", activation);
  if (!psb_gemm_stream_norm_supported(M, K) || I < 1 || sms < 1) PSB_REFUSE("gemm_stream_norm_gated: shape M=%d I=%d K=%d is not taken", M, I, K);
  if (!(eps > 0.f)) PSB_REFUSE("gemm_stream_norm_gated: eps must be positive");
  if (int rc = dispatch_norm_stream<2, __nv_bfloat16>(h_in, pending, gain, nullptr, h_out, W, act, M, I, K, I, I, activation, eps, sms, stream)) return rc;
  PSB_LAUNCH_CHECK("gemm_stream_norm_gated");
  return 0;
}

// The fused projection of an attention layer for few tokens: rmsnorm(h_in + pending) W^T with W = [queries; keys;
// values] in the pair-interleaved row order described at RopeArgs, queries rotated into q_out [M, hq, D], keys rotated
// and values as they are stored at the tokens' positions in the pages (what psb_gemm_stream_norm followed by
// psb_rope_append in its paired form would do, in one kernel).  cos_t/sin_t null: no rotation.
PSB_API int psb_gemm_stream_norm_rope(const void* h_in, const void* pending, const void* gain, void* h_out, const void* W, int M,
                                      int K, float eps, int sms, const void* positions, const void* token_item, const void* table,
                                      int table_width, const void* cos_t, const void* sin_t, void* kv, void* q_out, int hq, int hkv,
                                      int D, int page_size, int num_pages, int max_positions, cudaStream_t stream) {
  const int N = (hq + 2 * hkv) * D;
  if (!psb_gemm_stream_norm_supported(M, K) || sms < 1) PSB_REFUSE("gemm_stream_norm_rope: shape M=%d K=%d is not taken", M, K);
  if (hq < 1 || hkv < 1 || D < 16 || D % 16) PSB_REFUSE("gemm_stream_norm_rope: needs a head size that is a multiple of 16 (hq=%d hkv=%d D=%d)", hq, hkv, D);
  if (page_size < 1 || (page_size & (page_size - 1)) || num_pages < 1 || table_width < 1) PSB_REFUSE("gemm_stream_norm_rope: page size %d must be a power of two (pages=%d, width=%d)", page_size, num_pages, table_width);
  if (!positions || !token_item || !table || !kv || !q_out) PSB_REFUSE("gemm_stream_norm_rope: cache arguments missing");
  if ((cos_t == nullptr) != (sin_t == nullptr) || (cos_t && max_positions < 1)) PSB_REFUSE("gemm_stream_norm_rope: angle tables incomplete");
  if (!(eps > 0.f)) PSB_REFUSE("gemm_stream_norm_rope: eps must be positive");
  RopeArgs rope;
  rope.positions = (const int32_t*)positions; rope.token_item = (const int32_t*)token_item; rope.table = (const int32_t*)table;
  rope.cos_t = (const float*)cos_t; rope.sin_t = (const float*)sin_t; rope.kv = (__nv_bfloat16*)kv; rope.q_out = (__nv_bfloat16*)q_out;
  rope.table_width = table_width; rope.hq = hq; rope.hkv = hkv; rope.D = D; rope.num_pages = num_pages; rope.max_positions = max_positions;
  rope.page_shift = 0;
  while ((1 << rope.page_shift) < page_size) ++rope.page_shift;
  if (int rc = dispatch_norm_stream_rope(h_in, pending, gain, h_out, W, M, N, K, eps, sms, stream, rope)) return rc;
  PSB_LAUNCH_CHECK("gemm_stream_norm_rope");
  return 0;
}
