// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 for a few dozen rows (up to 64: decoding with that many requests, short
// prompt portions).  Such a product is bound by reading W once, and a kernel that tiles the output 128 rows at a time
// would fill a quarter of every instruction and of few SMs.  Here the roles are swapped and the contraction is shared:
//   * W is the instruction's M operand: an output tile is 128 rows of W by all MT (32 or 64) rows of A, which sit in
//     the instruction's N dimension, so the tensor memory accumulator has the features in its lanes and the tokens in
//     its columns (prefixserve/model/llama.py:113-126 of PrefixServe: the same F.linear calls);
//   * the contraction is cut into `ks` (1..8) ranges, one CTA each, the CTAs of a tile forming a thread-block cluster:
//     N/128 tiles times ks ranges keep 120 to 148 SMs streaming their own slice of W through a ring of TMA stages;
//   * every CTA leaves its partial sums in its own shared memory, the cluster meets at its barrier, and CTA r adds up,
//     in rank order (so the result does not depend on timing), the partial sums of tokens r, r+ks, ... read from its
//     peers' shared memory (distributed shared memory), then does the epilogue's job for them: plain store, the gated
//     activation (W = [gate; up], a tile = 64 gate rows and the 64 up rows that go with them), or the rotation and the
//     append to the cache pages (RopeArgs in common.cuh; the tile's features are then in the pair-interleaved order,
//     so the partners of a thread's four elements sit two lanes away).
// The RMSNorm between two such products needs no kernel of its own (prefixserve/model/llama.py:63-69, :117-121 of
// PrefixServe).  The product in front of it (O or down) adds its sums, rounded to bfloat16 as a stored product would
// be, to the float32 stream, writes the stream back, writes v * gain in bfloat16 for the product behind the norm, and
// leaves its tile's share of every row's sum(v^2); the product behind it (QKV, gate/up) adds those shares up in tile
// order and scales its own sums by rsqrt(mean + eps): the same order of roundings as the streaming kernels' norm.
// 192 threads: warp 0 producer (W before the dependency wait, since weights do not depend on the preceding kernel;
// A after it), warp 1 issues tcgen05.mma (M=128, N=MT, K=16), warps 2..5 read the accumulator and do the reduction.
// Every mbarrier wait is bounded (tcgen05.cuh); the cluster barriers are reached by every thread whatever happened.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int FEATURES = 128, BK = 64, THREADS = 192, STAGES = 9;
constexpr int W_BYTES = FEATURES * BK * 2;  // 16 KB a stage

template <int MT>
struct Shape {
  static_assert(MT == 32 || MT == 64, "row tiles built");  // (a tile of 16 rows was no faster for 9 to 16 of them)
  static constexpr int X_BYTES = MT * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int PART_BYTES = MT * FEATURES * 4;  // [token][feature] float32
  // the partial sums take the place of the first stages once the last instruction has read them
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
  static_assert(PART_BYTES <= STAGES * STAGE_BYTES, "the partial sums lie over the ring");
  static_assert(SMEM_BYTES <= 227 * 1024, "beyond a CTA's shared memory");
};

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  uint32_t abort;
};
static_assert(sizeof(Barriers) <= 256, "room kept for the barriers");

enum : int { MODE_PLAIN = 0, MODE_GATED = 1, MODE_ROPE = 2 };

constexpr int SSQ_PITCH = 64;  // floats per tile in the array of partial sums of squares: one per row of A

// The norm around a product (all null: none).  Behind a norm: ssq_in [ssq_parts][SSQ_PITCH] float32, the tiles' shares of
// every row's sum of squares; the row's sums are scaled by rsqrt(sum / width + eps).  In front of a norm (plain products
// only): stream [M, N] float32 is read, added to and written; gained [M, N] bfloat16 takes v * gain; ssq_out
// [tiles][SSQ_PITCH] this product's shares.
struct NormArgs {
  const float* ssq_in;
  int ssq_parts;
  float eps, inv_width;
  float* stream;
  const float* gain;
  __nv_bfloat16* gained;
  float* ssq_out;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// four floats at the same shared-memory offset in CTA `rank` of this cluster.  No memory clobber: the partial sums
// do not change between the two cluster barriers, and a thread's loads must be free to overlap one another (one
// load at a time, each waited for, made the reduction cost more than the product).
__device__ __forceinline__ float4 peer_float4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
  return v;
}
// the sum over the cluster's CTAs, in rank order, of four neighbouring partial sums
__device__ __forceinline__ float4 cluster_sum4(uint32_t local_addr, uint32_t ks) {
  float4 v[8];
#pragma unroll
  for (uint32_t r = 0; r < 8; ++r)
    if (r < ks) v[r] = peer_float4(local_addr, r);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (uint32_t r = 0; r < 8; ++r)
    if (r < ks) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
  return acc;
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// four neighbouring outputs: one 8-byte store where the row pitch and the edge allow it
__device__ __forceinline__ void store4(__nv_bfloat16* row, int col, int limit, bool aligned, const float (&o)[4]) {
  if (aligned && col + 4 <= limit) {
    *reinterpret_cast<uint2*>(row + col) = make_uint2(pack2(o[0], o[1]), pack2(o[2], o[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (col + i < limit) row[col + i] = __float2bfloat16_rn(o[i]);
  }
}

// status word: 0 ok; otherwise which wait gave up (1 producer, 2 mma, 3 accumulator)
template <int MT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_fewrows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    __nv_bfloat16* __restrict__ C, int M, int N_out, int K, int ldc, int up_offset, int mode, int activation,
                    const RopeArgs rope, const NormArgs norm) {
  using S = Shape<MT>;
  constexpr uint32_t INSTR_DESC = instr_desc(FEATURES, MT, false);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* part = reinterpret_cast<float*>(tiles);  // over the ring: written only after the accumulator is complete
  Barriers* bars = reinterpret_cast<Barriers*>(tiles + STAGES * S::STAGE_BYTES);
  volatile uint32_t* abort = &bars->abort;
  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank(), ks = gridDim.x;  // the cluster is the grid's x extent
  const bool gated = mode == MODE_GATED;
  const int tile = blockIdx.y;
  const int n_span = gated ? FEATURES / 2 : FEATURES;  // output columns a tile covers
  const int n0 = tile * n_span;
  const int r0 = n0, r1 = gated ? up_offset + n0 : n0 + FEATURES / 2;  // first rows of the two 64-row boxes of W
  const int k_blocks = (K + BK - 1) / BK;
  const int kb0 = (int)(((long)rank * k_blocks) / ks), kb1 = (int)(((long)(rank + 1) * k_blocks) / ks);
  const int nkb = kb1 - kb0;

  __shared__ float row_factor[SSQ_PITCH];  // behind a norm: rsqrt(mean(v^2) + eps) of every row
  constexpr int EARLY = 4;                 // in front of a norm: rows whose piece of the stream a thread fetches ahead
  float4 early_h[EARLY], early_gain = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int it = 0; it < EARLY; ++it) early_h[it] = make_float4(0.f, 0.f, 0.f, 0.f);

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full, 1);
    bars->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc(&bars->tmem_base, MT);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      const int early = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < early; ++i) {  // the ring's first round: nothing to wait for, and W may come before the wait
        unsigned char* w_dst = tiles + i * S::STAGE_BYTES;
        mbar_expect_tx(&bars->full[i], S::STAGE_BYTES);
        tma_load_2d(w_dst, &map_w, (kb0 + i) * BK, r0, &bars->full[i]);
        tma_load_2d(w_dst + W_BYTES / 2, &map_w, (kb0 + i) * BK, r1, &bars->full[i]);
      }
      pdl_wait();  // A is the preceding kernel's output
      for (int i = 0; i < early; ++i)
        tma_load_2d(tiles + i * S::STAGE_BYTES + W_BYTES, &map_x, (kb0 + i) * BK, 0, &bars->full[i]);
      bool ok = true;
      for (int i = early; ok && i < nkb; ++i) {
        const int stage = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(&bars->empty[stage], phase ^ 1, abort, 1);
        if (!ok) break;
        unsigned char* w_dst = tiles + stage * S::STAGE_BYTES;
        mbar_expect_tx(&bars->full[stage], S::STAGE_BYTES);
        tma_load_2d(w_dst, &map_w, (kb0 + i) * BK, r0, &bars->full[stage]);
        tma_load_2d(w_dst + W_BYTES / 2, &map_w, (kb0 + i) * BK, r1, &bars->full[stage]);
        tma_load_2d(w_dst + W_BYTES, &map_x, (kb0 + i) * BK, 0, &bars->full[stage]);
      }
    }
    __syncwarp();
    pdl_wait();
  } else if (warp == 1) {
    // ----------------------------------------------------------------------- MMA
    pdl_wait();
    bool ok = true;
    for (int i = 0; ok && i < nkb; ++i) {
      const int stage = i % STAGES;
      const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
      ok = mbar_wait(&bars->full[stage], phase, abort, 2);
      if (!ok) break;
      const uint64_t da = smem_desc(smem_u32(tiles + stage * S::STAGE_BYTES));
      const uint64_t db = smem_desc(smem_u32(tiles + stage * S::STAGE_BYTES + W_BYTES));
      const uint32_t hi = (uint32_t)(da >> 32), a_lo = (uint32_t)da, b_lo = (uint32_t)db;
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) {
        if (elect_one()) mma_f16_split(tmem_base, a_lo + 2 * k, hi, b_lo + 2 * k, hi, INSTR_DESC, (i | k) != 0);
      }
      if (elect_one()) mma_commit(&bars->empty[stage]);
    }
    if (ok && elect_one()) mma_commit(&bars->acc_full);
  } else {
    // ------------------------------------------------- this CTA's partial sums: tensor memory -> shared memory
    pdl_wait();
    const int quarter = warp & 3;  // a warp may only read tensor-memory lanes [32*(warp%4), +32)
    const int feature = quarter * 32 + lane;
    // What the reduction below needs of the norm around this product does not depend on the product: it is fetched
    // now, while the instructions run.  Behind a norm: every row's factor, into shared memory (the cluster barrier
    // below publishes it).  In front of one: this thread's pieces of the stream and of the gain, into registers.
    {
      const int e = threadIdx.x - 64;
      if (norm.ssq_in && e < M && e < SSQ_PITCH) {
        float total = 0.f;
#pragma unroll 8
        for (int p = 0; p < norm.ssq_parts; ++p) total += __ldg(norm.ssq_in + p * SSQ_PITCH + e);
        row_factor[e] = rsqrtf(total * norm.inv_width + norm.eps);
      }
      if (norm.stream) {
        const int col = n0 + (e & 31) * 4;
        const bool whole = col + 4 <= N_out && (ldc & 3) == 0;
        early_gain = whole ? __ldg(reinterpret_cast<const float4*>(norm.gain + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int it = 0; it < EARLY; ++it) {
          const int t = (int)rank + (int)ks * ((e >> 5) + 4 * it);
          early_h[it] = (whole && t < M) ? *reinterpret_cast<const float4*>(norm.stream + (size_t)t * ldc + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
    if (mbar_wait(&bars->acc_full, 0, abort, 3)) {
      fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
      for (int c = 0; c < MT; c += 32) {
        uint32_t v[32];
        tmem_ld32(taddr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) part[(c + j) * FEATURES + feature] = __uint_as_float(v[j]);
      }
    }
    fence_before();
  }

  // every thread of every CTA of the cluster, whatever happened above
  cluster_sync_all();

  if (warp >= 2 && !*abort) {
    const int e = threadIdx.x - 64;  // 0..127
    const uint32_t part_addr = smem_u32(part);
    const bool aligned = (ldc & 3) == 0;
    // behind a norm: the factor of row t
    auto row_scale = [&](int t) { return norm.ssq_in ? row_factor[t] : 1.f; };
    if (gated) {
      // 64 output columns a tile: features 4g..4g+3 of the gate half go with 64+4g.. of the up half; sixteen threads
      // a token, eight tokens at a time
      const int f = (e & 15) * 4, col = n0 + f;
#pragma unroll 2
      for (int t = (int)rank + (int)ks * (e >> 4); t < M; t += 8 * (int)ks) {
        const float4 g4 = cluster_sum4(part_addr + (uint32_t)(t * FEATURES + f) * 4u, ks);
        const float4 u4 = cluster_sum4(part_addr + (uint32_t)(t * FEATURES + 64 + f) * 4u, ks);
        const float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
        const float inv = row_scale(t);
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)  // the reference rounds both projections to bfloat16 before the activation
          o[i] = gate_act(round_bf16(g[i] * inv), activation) * round_bf16(u[i] * inv);
        store4(C + (size_t)t * ldc, col, N_out, aligned, o);
      }
    } else {
      // features 4g..4g+3 of a token a thread; a warp a token (so the shuffle below is safe), four tokens at a time
      const int f = (e & 31) * 4, col = n0 + f;
#pragma unroll 2
      for (int t = (int)rank + (int)ks * (e >> 5); t < M; t += 4 * (int)ks) {
        const float4 v4 = cluster_sum4(part_addr + (uint32_t)(t * FEATURES + f) * 4u, ks);
        const float inv = row_scale(t);
        float o[4] = {v4.x * inv, v4.y * inv, v4.z * inv, v4.w * inv};
        if (mode == MODE_PLAIN) {
          if (norm.stream) {
            // in front of a norm: the residual sum, the gained rows and this tile's share of the row's sum of squares
            float ss = 0.f;
            float gained[4] = {0.f, 0.f, 0.f, 0.f};
            float* hrow = norm.stream + (size_t)t * ldc;
            const int it = (t - (int)rank) / (int)ks / 4;  // which of this thread's rows
            if (col + 4 <= N_out && aligned && it < EARLY) {
              float4 hv = early_h[0];
#pragma unroll
              for (int k = 1; k < EARLY; ++k)
                if (it == k) hv = early_h[k];
              const float v[4] = {hv.x + round_bf16(o[0]), hv.y + round_bf16(o[1]), hv.z + round_bf16(o[2]), hv.w + round_bf16(o[3])};
              *reinterpret_cast<float4*>(hrow + col) = make_float4(v[0], v[1], v[2], v[3]);
              gained[0] = v[0] * early_gain.x; gained[1] = v[1] * early_gain.y; gained[2] = v[2] * early_gain.z; gained[3] = v[3] * early_gain.w;
              ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (col + i < N_out) {
                  const float v = hrow[col + i] + round_bf16(o[i]);
                  hrow[col + i] = v;
                  gained[i] = v * __ldg(norm.gain + col + i);
                  ss += v * v;
                }
            }
            store4(norm.gained + (size_t)t * ldc, col, N_out, aligned, gained);
            ss = warp_sum(ss);  // a warp a token
            if ((e & 31) == 0) norm.ssq_out[tile * SSQ_PITCH + t] = ss;
          } else {
            store4(C + (size_t)t * ldc, col, N_out, aligned, o);
          }
          continue;
        }
        // the projection of an attention layer: what rope_store_row of the many-row kernel does.  A block of 16
        // features holds 8 first-half elements and then the 8 they are rotated with: the partners of this thread's
        // four sit two lanes away.
        float other[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          o[i] = round_bf16(o[i]);  // what a separate projection would have stored
          other[i] = __shfl_xor_sync(0xffffffffu, o[i], 2);
        }
        if (col >= N_out) continue;
        const int D = rope.D, q_cols = rope.hq * D, k_cols = rope.hkv * D;
        const int pos = rope.positions[t];
        const int page = rope.table[(size_t)rope.token_item[t] * rope.table_width + (pos >> rope.page_shift)];
        const bool page_ok = page >= 0 && page < rope.num_pages;
        const size_t in_page = (size_t)(pos & ((1 << rope.page_shift) - 1)) * D;
        __nv_bfloat16* dst = nullptr;
        if (col < q_cols + k_cols) {
          const int within = col < q_cols ? col : col - q_cols;
          const int head = within / D, off = within - head * D;
          if (rope.cos_t) {
            const int safe = pos < 0 ? 0 : (pos >= rope.max_positions ? rope.max_positions - 1 : pos);
            const int pair = (off >> 4) * 8 + (off & 7);  // a multiple of 4
            const float4 c4 = __ldg(reinterpret_cast<const float4*>(rope.cos_t + (size_t)safe * (D >> 1) + pair));
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(rope.sin_t + (size_t)safe * (D >> 1) + pair));
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
            const bool second = (off & 8) != 0;  // this thread holds the elements that are rotated with those two lanes below
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float a, b;
              rotate_pair(second ? other[i] : o[i], second ? o[i] : other[i], cs[i], sn[i], a, b);
              o[i] = second ? b : a;
            }
          }
          if (col < q_cols) dst = rope.q_out + ((size_t)t * rope.hq + head) * D + off;
          else if (page_ok) dst = rope.kv + ((((size_t)page * 2) * rope.hkv + head) << rope.page_shift) * D + in_page + off;
        } else {
          const int within = col - q_cols - k_cols;
          const int head = within / D, off = within - head * D;
          if (page_ok) dst = rope.kv + ((((size_t)page * 2 + 1) * rope.hkv + head) << rope.page_shift) * D + in_page + off;
        }
        if (dst) *reinterpret_cast<uint2*>(dst) = make_uint2(pack2(o[0], o[1]), pack2(o[2], o[3]));
      }
    }
  }

  cluster_sync_all();  // nobody leaves while a peer may still read its shared memory

  if (*abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // copies in flight land before the shared memory is handed on
  }
  fence_before();
  __syncthreads();
  if (warp == 2) {
    fence_after();
    tmem_free(tmem_base, MT);
  }
}

// ---- host side -----------------------------------------------------------------------------------------------
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  const int r = make_map_bf16(map, base, (uint64_t)rows, (uint64_t)K, (uint64_t)K, box_rows);
  if (r == -1) PSB_REFUSE("gemm_fewrows: the driver does not export cuTensorMapEncodeTiled");
  if (r != 0) PSB_REFUSE("gemm_fewrows: cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d)", r, rows, K);
  return 0;
}

template <int MT>
cudaError_t launch_kernel(dim3 grid, cudaStream_t stream, const CUtensorMap& map_w, const CUtensorMap& map_x, __nv_bfloat16* c,
                          int M, int N_out, int K, int ldc, int up_offset, int mode, int activation, const RopeArgs& rope,
                          const NormArgs& norm) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = Shape<MT>::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = grid.x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (psb_pdl_enabled) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  return cudaLaunchKernelEx(&cfg, gemm_fewrows_kernel<MT>, map_w, map_x, c, M, N_out, K, ldc, up_offset, mode, activation, rope, norm);
}

// How many clusters of `ks` CTAs the device holds at once (one CTA an SM, a cluster inside one GPC); asked once per
// device and size.
template <int MT>
int resident_clusters(int ks) {
  static int known[PsbPerDevice::kMaxDevices][9] = {};
  const int dev = PsbPerDevice::current();
  if (dev < 0) return 1;
  if (known[dev][ks] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ks, 64);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = Shape<MT>::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_fewrows_kernel<MT>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 1;
    }
    known[dev][ks] = n;
  }
  return known[dev][ks];
}

int g_forced_splits = 0;  // 0: the launcher chooses; 1..8: tests compare them

// Ranges of the contraction: as many as make the tiles' clusters fill the device in one round, each range paying a
// fixed share (first loads, the reduction) on top of its blocks.
template <int MT>
int choose_splits(int tiles, int k_blocks) {
  int best = 1;
  long best_cost = -1;
  for (int ks = 1; ks <= 8 && ks <= k_blocks; ks *= 2) {  // other cluster sizes found fewer SMs (six CTAs: twice the time of four)
    if (g_forced_splits && ks != g_forced_splits && g_forced_splits <= k_blocks) continue;
    const int resident = resident_clusters<MT>(ks);
    const long rounds = (tiles + resident - 1) / resident;
    const long cost = rounds * ((k_blocks + ks - 1) / ks + 3) + (ks > 1 ? 1 : 0);
    if (best_cost < 0 || cost < best_cost) {
      best = ks;
      best_cost = cost;
    }
  }
  return best;
}

template <int MT>
int launch_shape(const void* a, const void* w, void* c, int M, int w_rows, int N_out, int K, int up_offset, int mode, int activation,
                 cudaStream_t stream, const RopeArgs& rope, const NormArgs& norm) {
  static PsbPerDevice configured;  // more than 48 KB of dynamic shared memory has to be asked for once
  if (!configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fewrows_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<MT>::SMEM_BYTES);
    if (e != cudaSuccess) PSB_REFUSE("gemm_fewrows: cannot reserve %d bytes of shared memory: %s", Shape<MT>::SMEM_BYTES, cudaGetErrorString(e));
    configured.set();
  }
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, w, w_rows, K, FEATURES / 2)) return rc;
  if (int rc = make_map(&map_x, a, M, K, MT)) return rc;
  const int n_span = mode == MODE_GATED ? FEATURES / 2 : FEATURES;
  const int tiles = (N_out + n_span - 1) / n_span;
  const int k_blocks = (K + BK - 1) / BK;
  const int ks = choose_splits<MT>(tiles, k_blocks);
  cudaError_t e = launch_kernel<MT>(dim3(ks, tiles), stream, map_w, map_x, (__nv_bfloat16*)c, M, N_out, K, N_out, up_offset, mode,
                                    activation, rope, norm);
  if (e != cudaSuccess) {
    cudaGetLastError();
    PSB_REFUSE("gemm_fewrows: launch failed: %s (M=%d N=%d K=%d ranges=%d)", cudaGetErrorString(e), M, N_out, K, ks);
  }
  return 0;
}

int launch(const void* a, const void* w, void* c, int M, int w_rows, int N_out, int K, int up_offset, int mode, int activation,
           cudaStream_t stream, const RopeArgs& rope = RopeArgs{}, const NormArgs& norm = NormArgs{}) {
  if (norm.ssq_in && (norm.ssq_parts < 1 || !(norm.eps > 0.f))) PSB_REFUSE("gemm_fewrows: the norm in front needs its parts and a positive eps");
  if (norm.stream && (mode != MODE_PLAIN || !norm.gain || !norm.gained || !norm.ssq_out || (((uintptr_t)norm.stream | (uintptr_t)norm.gained) & 15)))
    PSB_REFUSE("gemm_fewrows: a product in front of a norm is a plain one with stream, gain, gained rows and shares given (16-byte aligned)");
  if (M < 1 || M > 64 || N_out < 1 || K < 8 || K % 8) PSB_REFUSE("gemm_fewrows: needs 1..64 rows and K a multiple of 8 (M=%d N=%d K=%d)", M, N_out, K);
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15) PSB_REFUSE("gemm_fewrows: operands must be 16-byte aligned");
  if (M <= 32) return launch_shape<32>(a, w, c, M, w_rows, N_out, K, up_offset, mode, activation, stream, rope, norm);
  return launch_shape<64>(a, w, c, M, w_rows, N_out, K, up_offset, mode, activation, stream, rope, norm);
}

}  // namespace

// C[M,N] = A[M,K] W[N,K]^T, all bfloat16 row-major, M <= 64, K % 8 == 0.
PSB_API int psb_gemm_fewrows(const void* a, const void* w, void* c, int M, int N, int K, cudaStream_t stream) {
  return launch(a, w, c, M, N, N, K, 0, MODE_PLAIN, 0, stream);
}

// act[M,I] = f(A Wg^T) * (A Wu^T) for W = [Wg; Wu] of shape [2I, K], f the activation named by its code (PsbAct).
PSB_API int psb_gemm_fewrows_gated(const void* a, const void* w, void* act, int M, int I, int K, int activation, cudaStream_t stream) {
  if (!psb_activation_known(activation)) PSB_REFUSE("gemm_fewrows_gated: activation code %d is not built", activation);
  return launch(a, w, act, M, 2 * I, I, K, I, MODE_GATED, activation, stream);
}

// The projection of an attention layer for a few dozen tokens: as psb_gemm_tcgen05_rope (W in the pair-interleaved
// row order, queries rotated into q_out, keys rotated and values stored at the tokens' positions in the pages).
PSB_API int psb_gemm_fewrows_rope(const void* a, const void* w, int M, int K, const void* positions, const void* token_item,
                                  const void* table, int table_width, const void* cos_t, const void* sin_t, void* kv, void* q_out,
                                  int hq, int hkv, int D, int page_size, int num_pages, int max_positions, cudaStream_t stream) {
  if (hq < 1 || hkv < 1 || D < 16 || D % 16) PSB_REFUSE("gemm_fewrows_rope: needs a head size that is a multiple of 16 (hq=%d hkv=%d D=%d)", hq, hkv, D);
  if (page_size < 1 || (page_size & (page_size - 1)) || num_pages < 1 || table_width < 1) PSB_REFUSE("gemm_fewrows_rope: page size %d must be a power of two (pages=%d, width=%d)", page_size, num_pages, table_width);
  if (!positions || !token_item || !table || !kv || !q_out) PSB_REFUSE("gemm_fewrows_rope: cache arguments missing");
  if ((cos_t == nullptr) != (sin_t == nullptr) || (cos_t && max_positions < 1)) PSB_REFUSE("gemm_fewrows_rope: angle tables incomplete");
  if (((uintptr_t)kv | (uintptr_t)q_out | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) PSB_REFUSE("gemm_fewrows_rope: cache, queries and angle tables must be 16-byte aligned");
  RopeArgs rope;
  rope.positions = (const int32_t*)positions; rope.token_item = (const int32_t*)token_item; rope.table = (const int32_t*)table;
  rope.cos_t = (const float*)cos_t; rope.sin_t = (const float*)sin_t; rope.kv = (__nv_bfloat16*)kv; rope.q_out = (__nv_bfloat16*)q_out;
  rope.table_width = table_width; rope.hq = hq; rope.hkv = hkv; rope.D = D; rope.num_pages = num_pages; rope.max_positions = max_positions;
  rope.page_shift = 0;
  while ((1 << rope.page_shift) < page_size) ++rope.page_shift;
  const int N = (hq + 2 * hkv) * D;
  return launch(a, w, q_out, M, N, N, K, 0, MODE_ROPE, 0, stream, rope);
}

namespace {
NormArgs behind_norm(const void* ssq_in, int ssq_parts, float eps, int width) {
  NormArgs n{};
  n.ssq_in = (const float*)ssq_in; n.ssq_parts = ssq_parts; n.eps = eps; n.inv_width = 1.f / (float)width;
  return n;
}
}  // namespace

// The same three products behind a norm whose rows arrive as v * gain (bfloat16) with the shares of their sums of squares
// (ssq_in [ssq_parts][64] float32, from psb_gemm_fewrows_add_norm): every sum is scaled by rsqrt(sum(v^2) / K + eps).
PSB_API int psb_gemm_fewrows_scaled(const void* a, const void* w, void* c, int M, int N, int K, const void* ssq_in, int ssq_parts,
                                    float eps, cudaStream_t stream) {
  return launch(a, w, c, M, N, N, K, 0, MODE_PLAIN, 0, stream, RopeArgs{}, behind_norm(ssq_in, ssq_parts, eps, K));
}
PSB_API int psb_gemm_fewrows_gated_scaled(const void* a, const void* w, void* act, int M, int I, int K, int activation,
                                          const void* ssq_in, int ssq_parts, float eps, cudaStream_t stream) {
  if (!psb_activation_known(activation)) PSB_REFUSE("gemm_fewrows_gated: activation code %d is not built", activation);
  return launch(a, w, act, M, 2 * I, I, K, I, MODE_GATED, activation, stream, RopeArgs{}, behind_norm(ssq_in, ssq_parts, eps, K));
}
PSB_API int psb_gemm_fewrows_rope_scaled(const void* a, const void* w, int M, int K, const void* positions, const void* token_item,
                                         const void* table, int table_width, const void* cos_t, const void* sin_t, void* kv,
                                         void* q_out, int hq, int hkv, int D, int page_size, int num_pages, int max_positions,
                                         const void* ssq_in, int ssq_parts, float eps, cudaStream_t stream) {
  if (hq < 1 || hkv < 1 || D < 16 || D % 16) PSB_REFUSE("gemm_fewrows_rope: needs a head size that is a multiple of 16 (hq=%d hkv=%d D=%d)", hq, hkv, D);
  if (page_size < 1 || (page_size & (page_size - 1)) || num_pages < 1 || table_width < 1) PSB_REFUSE("gemm_fewrows_rope: page size %d must be a power of two (pages=%d, width=%d)", page_size, num_pages, table_width);
  if (!positions || !token_item || !table || !kv || !q_out) PSB_REFUSE("gemm_fewrows_rope: cache arguments missing");
  if ((cos_t == nullptr) != (sin_t == nullptr) || (cos_t && max_positions < 1)) PSB_REFUSE("gemm_fewrows_rope: angle tables incomplete");
  if (((uintptr_t)kv | (uintptr_t)q_out | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) PSB_REFUSE("gemm_fewrows_rope: cache, queries and angle tables must be 16-byte aligned");
  RopeArgs rope;
  rope.positions = (const int32_t*)positions; rope.token_item = (const int32_t*)token_item; rope.table = (const int32_t*)table;
  rope.cos_t = (const float*)cos_t; rope.sin_t = (const float*)sin_t; rope.kv = (__nv_bfloat16*)kv; rope.q_out = (__nv_bfloat16*)q_out;
  rope.table_width = table_width; rope.hq = hq; rope.hkv = hkv; rope.D = D; rope.num_pages = num_pages; rope.max_positions = max_positions;
  rope.page_shift = 0;
  while ((1 << rope.page_shift) < page_size) ++rope.page_shift;
  const int N = (hq + 2 * hkv) * D;
  return launch(a, w, q_out, M, N, N, K, 0, MODE_ROPE, 0, stream, rope, behind_norm(ssq_in, ssq_parts, eps, K));
}

// A product in front of a norm: stream[M,N] += bfloat16(A W^T) (float32, in place); gained[M,N] = bfloat16(stream * gain);
// ssq_out [ceil(N/128)][64] float32 takes each tile's share of every row's sum of stream^2.  Returns the number of tiles
// through *tiles_out.
PSB_API int psb_gemm_fewrows_add_norm(const void* a, const void* w, void* stream_io, const void* gain, void* gained, void* ssq_out,
                                      int M, int N, int K, cudaStream_t stream) {
  NormArgs n{};
  n.stream = (float*)stream_io; n.gain = (const float*)gain; n.gained = (__nv_bfloat16*)gained; n.ssq_out = (float*)ssq_out;
  return launch(a, w, gained, M, N, N, K, 0, MODE_PLAIN, 0, stream, RopeArgs{}, n);
}

// For tests: 1, 2, 4 or 8 makes every later product cut the contraction into that many ranges (where it has that many
// blocks of 64), 0 gives the choice back.
PSB_API int psb_gemm_fewrows_splits(int splits) {
  if (splits < 0 || splits > 8 || (splits & (splits - 1))) PSB_REFUSE("gemm_fewrows: 0, 1, 2, 4 or 8 ranges, not %d", splits);
  g_forced_splits = splits;
  return 0;
}

// 0 while no bounded wait has ever run out on the current device; reading it synchronises with the device.
PSB_API int psb_gemm_fewrows_status() {
  return tc::read_status();
}
