// Split-KV decode attention over the paged cache with the keys and values brought in by the TMA unit.
//
// Decode attention is nothing but memory traffic: per request and key/value head one row of queries per head of the
// group meets thousands of keys.  What limits it is how many bytes an SM keeps in flight and how many instructions
// it spends per byte.  Here one producer warp asks the TMA unit for whole 16-key tiles (cp.async.bulk.tensor.2d, one
// box of keys and one of values per tile, 128-byte swizzle, completion on an mbarrier) into a ring of a dozen
// stages, and four consumer warps take the tiles in turn: ldmatrix out of the swizzled rows straight into
// mma.sync operand order, scores, running softmax in float32, P V.  No thread copies data; the ring is deep
// enough that the SM always has tens of kilobytes on the way.
//
// grid (key ranges, key/value heads, items), 160 threads.  Each CTA walks the keys [range*chunk, +chunk) of one
// request that its query may see; warps keep a running (maximum, sum, output) each, the CTA combines them and writes
// either the output row (one range) or a partial result for the merge kernel of attention_mma.cu (same layout:
// part_o[item][head][range][D], part_ml[item][head][range][2]).  The mathematics is that of
// prefixserve/model/attention.py:68-121 of PrefixServe (grouped heads, scores scaled by 1/sqrt(D), softmax in
// float32, probabilities rounded to bfloat16 before P V).
//
// Rows of a tile past the request's last key belong to nobody (or to an earlier owner of the page): their scores are
// masked and their value rows are cleared in shared memory before P V, so that 0 x (whatever lies there) is 0.
//
// Every wait on an mbarrier is bounded (tcgen05.cuh); if one runs out the CTA stops, lets copies in flight land and
// returns, and the host reads a non-zero status word.
#include <cfloat>

#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int CONSUMERS = 4;                 // warps that compute
constexpr int THREADS = 32 * (CONSUMERS + 1);
constexpr int KEYS = 16;                     // keys per tile
constexpr float LOG2E_F = 1.4426950408889634f;

template <int D>
struct Shape {
  static constexpr int DS = D / 64;                      // boxes of 64 head dims per tile
  static constexpr int BOX_BYTES = KEYS * 128;           // [16 keys x 64 dims] bfloat16
  static constexpr int K_BYTES = DS * BOX_BYTES;
  static constexpr int STAGE_BYTES = 2 * K_BYTES;        // keys, then values
  // A stage must always come back to the warp that used it last (stage j % STAGES, warp j % CONSUMERS): a parity wait
  // only tells the phase in progress from the one before it, so a warp that could reach a stage a whole round ahead of
  // another warp's turn at it would take that warp's unfinished phase for its own finished one.
  static constexpr int STAGES = D == 64 ? 12 : 8;
  static_assert(STAGES % CONSUMERS == 0, "every stage belongs to one consumer warp");
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int MERGE_BYTES = CONSUMERS * 16 * (D + 4 + 2) * 4;
  static constexpr int BAR_OFF = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
  static constexpr int SMEM_BYTES = BAR_OFF + 1024 /* alignment slack */ + 2 * STAGES * 8 + 16;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// where the 16-byte chunk `chunk` (8 head dims) of key row `row` lies inside a tile of DS swizzled boxes
__device__ __forceinline__ uint32_t chunk_at(uint32_t base, int row, int chunk) {
  return base + (uint32_t)((chunk >> 3) * (KEYS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// status codes: 1 producer, 2 consumer
template <int D>
__global__ void __launch_bounds__(THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const __nv_bfloat16* __restrict__ q,
                            const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ item_start,
                            const int32_t* __restrict__ kv_len, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                            float* __restrict__ part_ml, int hq, int hkv, int page_shift, int window, float scale, int chunk,
                            int max_splits, int all_single) {
  using Sh = Shape<D>;
  constexpr int STAGES = Sh::STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Sh::BAR_OFF);
  uint64_t* empty = full + STAGES;
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(empty + STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_trigger();
  // lengths and page tables are inputs of the step: readable before the preceding kernel has finished
  const int item = blockIdx.z, h = blockIdx.y, split = blockIdx.x;
  int t0 = item;
  bool mine = true;
  if (!all_single) {
    t0 = item_start[item];
    mine = item_start[item + 1] - t0 == 1;  // otherwise not a decode item: a prefill kernel has it
  }
  const int G = hq / hkv;
  const int kvl = kv_len[item];
  const int p = kvl - 1;
  const int lo_key = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int k_begin = (lo_key & ~15) + split * chunk;
  if (!mine || k_begin >= kvl) {  // the merge kernel knows how many ranges this item has
    pdl_wait();
    return;
  }
  const int k_end = min(k_begin + chunk, kvl);
  const int n_tiles = (k_end - k_begin + KEYS - 1) / KEYS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const uint32_t ring = smem_u32(smem);
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const int g = lane >> 2, t = lane & 3;

  if (warp == CONSUMERS) {
    // ---------------------------------------------------------------------------------------------- producer
    const int32_t* pages = table + (size_t)item * table_width;
    const int page_mask = (1 << page_shift) - 1;
    int ids = 0;
    bool ok = true, waited = false;
    for (int j = 0; ok && j < n_tiles; ++j) {
      if ((j & 31) == 0) {  // page ids of the next 32 tiles, one per lane: a load in the issue path costs a full latency
        const int jj = j + lane;
        ids = jj < n_tiles ? __ldg(pages + ((k_begin + jj * KEYS) >> page_shift)) : 0;
      }
      const int pid = __shfl_sync(0xffffffffu, ids, j & 31);
      const int key0 = k_begin + j * KEYS;
      // tiles of earlier steps do not change during this one: they may be asked for before the preceding kernel (which
      // writes this step's key and value, and the queries) has finished; the tile that holds position p may not
      if (!waited && (key0 + KEYS > p || j >= STAGES)) {
        pdl_wait();
        waited = true;
      }
      const int stage = j % STAGES;
      if (j >= STAGES) {
        ok = mbar_wait(&empty[stage], ((j / STAGES) - 1) & 1, abort, 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (lane == 0) {
        const int row_k = ((pid * 2) * hkv + h) * (1 << page_shift) + (key0 & page_mask);
        const int row_v = row_k + hkv * (1 << page_shift);
        unsigned char* dst = smem + stage * Sh::STAGE_BYTES;
        mbar_expect_tx(&full[stage], (uint32_t)Sh::STAGE_BYTES);
#pragma unroll
        for (int b = 0; b < Sh::DS; ++b) {
          tma_load_2d(dst + b * Sh::BOX_BYTES, &map_kv, 64 * b, row_k, &full[stage]);
          tma_load_2d(dst + Sh::K_BYTES + b * Sh::BOX_BYTES, &map_kv, 64 * b, row_v, &full[stage]);
        }
      }
      __syncwarp();
    }
    if (!waited) pdl_wait();
  } else {
    // --------------------------------------------------------------------------------------------- consumers
    pdl_wait();  // the queries are the preceding kernel's output
    uint32_t qa[D / 16][4];
    {
      const uint32_t* r0 = g < G ? reinterpret_cast<const uint32_t*>(q + ((size_t)t0 * hq + h * G + g) * D) : nullptr;
      const uint32_t* r1 = g + 8 < G ? reinterpret_cast<const uint32_t*>(q + ((size_t)t0 * hq + h * G + g + 8) * D) : nullptr;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qa[ks][0] = r0 ? __ldg(r0 + 8 * ks + t) : 0u;
        qa[ks][1] = r1 ? __ldg(r1 + 8 * ks + t) : 0u;
        qa[ks][2] = r0 ? __ldg(r0 + 8 * ks + 4 + t) : 0u;
        qa[ks][3] = r1 ? __ldg(r1 + 8 * ks + 4 + t) : 0u;
      }
    }
    const float sl2 = scale * LOG2E_F;
    const int lm = lane >> 3, lr = lane & 7;  // which of an ldmatrix's four matrices this lane addresses, and which row
    bool ok = true;
    for (int j = warp; ok && j < n_tiles; j += CONSUMERS) {
      const int stage = j % STAGES;
      const int key0 = k_begin + j * KEYS;
      ok = mbar_wait(&full[stage], (j / STAGES) & 1, abort, 2);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t kbase = ring + stage * Sh::STAGE_BYTES, vbase = kbase + Sh::K_BYTES;
      const int valid = kvl - key0;  // rows of the tile that hold this request's keys
      if (valid < KEYS) {
        // clear the value rows that are not this request's: 0 x (what an earlier owner of the page left) must be 0
        for (int idx = lane; idx < (KEYS - valid) * (D / 8); idx += 32) {
          const int row = valid + idx / (D / 8), ch = idx % (D / 8);
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(chunk_at(vbase, row, ch)), "r"(0u) : "memory");
        }
        fence_async_smem();  // these writes come before the TMA unit's next use of the stage
        __syncwarp();
      }
      // key fragments: B operand of S = Q K^T, n = key, k = head dim
      uint32_t kb[2][D / 16][2];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int qd = 0; qd < D / 32; ++qd) {
          uint32_t r[4];
          ldmatrix_x4(r, chunk_at(kbase, half * 8 + lr, 4 * qd + lm));
          kb[half][2 * qd][0] = r[0]; kb[half][2 * qd][1] = r[1];
          kb[half][2 * qd + 1][0] = r[2]; kb[half][2 * qd + 1][1] = r[3];
        }
      // value fragments: B operand of O += P V, k = key, n = head dim (transposed on the way out of shared memory)
      uint32_t vb[D / 8][2];
#pragma unroll
      for (int c = 0; c < D / 8; c += 2) {
        uint32_t r[4];
        ldmatrix_x4_trans(r, chunk_at(vbase, (lm & 1) * 8 + lr, c + (lm >> 1)));
        vb[c][0] = r[0]; vb[c][1] = r[1];
        vb[c + 1][0] = r[2]; vb[c + 1][1] = r[3];
      }
      float s[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        s[half][0] = s[half][1] = s[half][2] = s[half][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) mma_bf16(s[half], qa[ks], kb[half][ks][0], kb[half][ks][1]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);  // the tile is in registers: its stage may be filled again
      if (key0 + KEYS - 1 > p || key0 < lo_key) {
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int key = key0 + half * 8 + 2 * t + (i & 1);
            if (key > p || key < lo_key) s[half][i] = -INFINITY;
          }
      }
      float pr[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r == 1 && G <= 8) continue;  // rows 8..15 of the tile are padding when a group has at most 8 query heads
        float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx * sl2);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen nothing yet
        const float alpha = ex2(m_run[r] - m_safe);
        m_run[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float e = ex2(fmaf(s[half][2 * r + i], sl2, -m_safe));
            pr[half][2 * r + i] = e;
            sum += e;
          }
        l_run[r] = l_run[r] * alpha + sum;
#pragma unroll
        for (int jn = 0; jn < D / 8; ++jn) {
          o[jn][2 * r] *= alpha;
          o[jn][2 * r + 1] *= alpha;
        }
      }
      uint32_t pa[4];
      pa[0] = pack2(pr[0][0], pr[0][1]);
      pa[1] = pack2(pr[0][2], pr[0][3]);
      pa[2] = pack2(pr[1][0], pr[1][1]);
      pa[3] = pack2(pr[1][2], pr[1][3]);
#pragma unroll
      for (int jn = 0; jn < D / 8; ++jn) mma_bf16(o[jn], pa, vb[jn][0], vb[jn][1]);
    }
  }

  if (*abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // copies in flight must land before the memory changes hands
  }
  __syncthreads();  // every warp is done with the ring: the same memory now carries the merge of the warps' results

  float(*sh_m)[16] = reinterpret_cast<float(*)[16]>(smem);
  float(*sh_l)[16] = reinterpret_cast<float(*)[16]>(smem + CONSUMERS * 16 * 4);
  float(*sh_o)[16][D + 4] = reinterpret_cast<float(*)[16][D + 4]>(smem + 2 * CONSUMERS * 16 * 4);
  if (warp < CONSUMERS) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_run[r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int row = g + 8 * r;
      if (row < G) {
        if (t == 0) { sh_m[warp][row] = m_run[r]; sh_l[warp][row] = l; }
#pragma unroll
        for (int jn = 0; jn < D / 8; ++jn) {
          sh_o[warp][row][8 * jn + 2 * t] = o[jn][2 * r];
          sh_o[warp][row][8 * jn + 2 * t + 1] = o[jn][2 * r + 1];
        }
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, sh_m[w][row]);
    const float m_safe = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) {
      const float a = ex2(sh_m[w][row] - m_safe);
      l += a * sh_l[w][row];
      acc += a * sh_o[w][row][d];
    }
    const int head = h * G + row;
    if (max_splits == 1) {
      out[((size_t)t0 * hq + head) * D + d] = __float2bfloat16_rn(acc / l);
    } else {
      const size_t slot = ((size_t)item * hq + head) * max_splits + split;
      part_o[slot * D + d] = acc;
      if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
    }
  }
}

template <int D>
int launch(const CUtensorMap& map, const void* q, const void* table, int table_width, const void* item_start, const void* kv_len,
           void* out, void* part_o, void* part_ml, int num_items, int hq, int hkv, int page_shift, int window, float scale,
           int chunk, int max_splits, int all_single, cudaStream_t stream) {
  static PsbPerDevice configured;
  if (!configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<D>::SMEM_BYTES);
    if (e != cudaSuccess) PSB_REFUSE("attention_decode_tma: cannot reserve shared memory: %s", cudaGetErrorString(e));
    configured.set();
  }
  psb_launch(attention_decode_tma_kernel<D>, dim3(max_splits, hkv, num_items), dim3(THREADS), (size_t)Shape<D>::SMEM_BYTES, stream,
             map, (const __nv_bfloat16*)q, (const int32_t*)table, table_width, (const int32_t*)item_start, (const int32_t*)kv_len,
             (__nv_bfloat16*)out, (float*)part_o, (float*)part_ml, hq, hkv, page_shift, window, scale, chunk, max_splits, all_single);
  return 0;
}

}  // namespace

// 1 if this kernel takes the shape, else 0 (the caller then uses the kernel of attention_mma.cu).
PSB_API int psb_attention_decode_tma_supported(int hq, int hkv, int D, int page_size) {
  if (D != 64 && D != 128) return 0;
  if (hkv < 1 || hq % hkv || hq / hkv > 16) return 0;
  return page_size >= KEYS && (page_size & (page_size - 1)) == 0 ? 1 : 0;
}

// The decode kernel alone: arguments as psb_attention_decode_bf16 (attention_mma.cu) plus the number of pages of the
// cache entry (for the tensor map).  With more than one key range the caller launches that file's merge afterwards
// (psb_attention_decode_merge_bf16).
PSB_API int psb_attention_decode_tma_bf16(const void* q, const void* kv, const void* table, int table_width, const void* item_start,
                                          const void* kv_len, void* out, void* part_o, void* part_ml, int num_items, int hq,
                                          int hkv, int D, int page_size, long long num_pages, int window, float scale, int chunk,
                                          int max_splits, int all_single, cudaStream_t stream) {
  if (!psb_attention_decode_tma_supported(hq, hkv, D, page_size))
    PSB_REFUSE("attention_decode_tma: hq=%d hkv=%d D=%d pages of %d are not built (heads of 64 or 128, groups up to 16, pages a power of two from 16)", hq, hkv, D, page_size);
  if (window < 0 || table_width < 1 || num_pages < 1) PSB_REFUSE("attention_decode_tma: bad sizes (window=%d table_width=%d)", window, table_width);
  if (chunk < KEYS || chunk % KEYS) PSB_REFUSE("attention_decode_tma: key range %d is not a multiple of %d", chunk, KEYS);
  if (max_splits < 1 || max_splits > 1024 || (max_splits > 1 && (!part_o || !part_ml)))
    PSB_REFUSE("attention_decode_tma: %d key ranges (at most 1024), or their scratch is missing", max_splits);
  if (num_items <= 0) return 0;
  if (num_items > 65535 || hkv > 65535) PSB_REFUSE("attention_decode_tma: batch too large");
  const long long kv_rows = num_pages * 2 * hkv * page_size;
  if (kv_rows > 0x7fffffffLL) PSB_REFUSE("attention_decode_tma: the cache entry has %lld rows, beyond a TMA coordinate", kv_rows);
  if (((uintptr_t)q | (uintptr_t)kv) & 15) PSB_REFUSE("attention_decode_tma: operands must be 16-byte aligned");
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap map;
  const int r = make_map_bf16(&map, kv, (uint64_t)kv_rows, (uint64_t)D, (uint64_t)D, KEYS);
  if (r == -1) PSB_REFUSE("attention_decode_tma: the driver does not export cuTensorMapEncodeTiled");
  if (r != 0) PSB_REFUSE("attention_decode_tma: cuTensorMapEncodeTiled failed with code %d", r);
  int rc;
  if (D == 64) rc = launch<64>(map, q, table, table_width, item_start, kv_len, out, part_o, part_ml, num_items, hq, hkv, page_shift, window, scale, chunk, max_splits, all_single, stream);
  else rc = launch<128>(map, q, table, table_width, item_start, kv_len, out, part_o, part_ml, num_items, hq, hkv, page_shift, window, scale, chunk, max_splits, all_single, stream);
  if (rc) return rc;
  PSB_LAUNCH_CHECK("attention_decode_tma");
  return 0;
}

// 0 while no bounded wait of this kernel has ever run out on the current device; reading it synchronises with the device.
PSB_API int psb_attention_decode_tma_status() { return tc::read_status(); }
