// Causal grouped-query attention of prompt portions over the paged cache on the 5th-generation tensor cores.
//
// One CTA owns up to 256 consecutive new tokens of one request for one query head, as two tiles of 128 rows, and walks
// the keys they may see in blocks of KB keys (128 for a head size of 64, 64 for 128).  320 threads:
//   warp 0      producer: TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the two Q tiles once, and per block of
//               the pages that hold its keys and values, one box per page, into rings of three stages each;
//   warp 1      MMA: one lane issues tcgen05.mma (cta_group::1, kind::f16, M=128):  S = Q K^T  (A and B K-major, N=KB)
//               into tensor memory, and  O_block = P V  (A = P K-major from shared memory, B = V MN-major exactly as the
//               cache stores it: keys x head dim, N = head dim);
//   warps 2..5  softmax of tile 0, warps 6..9 of tile 1: one thread per row.  tcgen05.ld of the row of S, masks, running
//               maximum and sum in float32, P as bfloat16 into swizzled shared memory, then tcgen05.ld of O_block,
//               which is added into the row's float32 accumulator in registers scaled by exp(old max - new max).
// The two tiles alternate on the tensor cores: while one tile's rows are in the softmax, the other's products run.
// Rows are [token, head*D] of the rotated queries (prefixserve/model/llama.py:113-116 of PrefixServe computes the same
// attention with a library kernel, prefixserve/model/attention.py:58-104); keys and values come from the pages named
// by the request's block table; query at position p sees keys max(0, p-window+1) .. p.
//
// Every wait on an mbarrier is bounded (tcgen05.cuh).  If one runs out, all warps of the CTA stop, wait for copies in
// flight, free the tensor memory and return; the host reads a non-zero status word.
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int TILE_M = 128;
constexpr int TILES = 2;
constexpr int ROWS_PER_CTA = TILE_M * TILES;
constexpr int THREADS = 32 * (2 + 4 * TILES);
constexpr int STAGES = 3;
constexpr int TMEM_COLS = 512;
constexpr float LOG2E_F = 1.4426950408889634f;

template <int D>
struct Shape {
  static constexpr int KB = D == 64 ? 128 : 64;           // keys per block
  static constexpr int DS = D / 64;                       // 64-element sub-tiles along the head dim
  static constexpr int Q_TILE_BYTES = TILE_M * D * 2;
  static constexpr int Q_SUB_BYTES = TILE_M * 128;        // one [128 x 64] sub-tile
  static constexpr int KV_STAGE_BYTES = KB * D * 2;
  static constexpr int KV_SUB_BYTES = KB * 128;           // one [KB x 64] sub-tile
  static constexpr int P_TILE_BYTES = TILE_M * KB * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILES * Q_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + STAGES * KV_STAGE_BYTES;
  static constexpr int P_OFF = V_OFF + STAGES * KV_STAGE_BYTES;
  static constexpr int BAR_OFF = P_OFF + TILES * P_TILE_BYTES;
  static constexpr int S_COL = 0;                         // S of tile t: columns [t*KB, +KB)
  static constexpr int O_COL = TILES * KB;                // O_block of tile t: columns [O_COL + t*D, +D)
  static_assert(O_COL + TILES * D <= TMEM_COLS, "tensor memory");
  static_assert(Q_TILE_BYTES % 1024 == 0 && KV_STAGE_BYTES % 1024 == 0 && P_TILE_BYTES % 1024 == 0, "swizzle atoms");
};

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  uint64_t s_full[TILES], p_ready[TILES], o_full[TILES];
  uint32_t tmem_base;
  uint32_t abort;
};

template <int D>
constexpr int smem_bytes() { return Shape<D>::BAR_OFF + 1024 /* alignment slack */ + (int)sizeof(Barriers); }

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// status codes: 1 producer, 2 MMA, 3 softmax
template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                 const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ item_start,
                                 const int32_t* __restrict__ kv_len, __nv_bfloat16* __restrict__ out, int num_items, int hq,
                                 int hkv, int page_shift, int window, float scale, int skip_single) {
  using Sh = Shape<D>;
  constexpr int KB = Sh::KB;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + Sh::BAR_OFF);
  volatile uint32_t* abort = &bars->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_trigger();
  // which request and which 256 rows of it?  (lengths are inputs of the step: readable before the wait)
  const int head = blockIdx.x;
  int item = -1, pair = 0, n = 0;
  {
    int left = blockIdx.y;  // block 0 takes the last (longest) rows of the last request
    for (int i = num_items - 1; i >= 0; --i) {
      const int ni = item_start[i + 1] - item_start[i];
      if (skip_single && ni == 1) continue;
      const int pairs = (ni + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
      if (left < pairs) { item = i; pair = pairs - 1 - left; n = ni; break; }
      left -= pairs;
    }
  }
  if (item < 0) return;  // uniform for the CTA, before anything is allocated

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int t = 0; t < TILES; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_ready[t], TILE_M);  // every softmax thread of the tile arrives
      mbar_init(&bars->o_full[t], 1);
    }
    bars->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc(&bars->tmem_base, TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int t0 = item_start[item];
  const int kvl = kv_len[item];
  const int first_pos = kvl - n;                      // position of the request's first new token
  const int row0 = pair * ROWS_PER_CTA;               // first of this CTA's rows among the new tokens
  const int rows_here = min(ROWS_PER_CTA, n - row0);
  const int ntiles = rows_here > TILE_M ? 2 : 1;
  int p_first[TILES], p_last[TILES], bend[TILES];
#pragma unroll
  for (int t = 0; t < TILES; ++t) {
    p_first[t] = first_pos + row0 + TILE_M * t;
    p_last[t] = first_pos + min(n, row0 + TILE_M * (t + 1)) - 1;
    bend[t] = p_last[t] / KB;
  }
  const int lo_key = (window > 0 && p_first[0] - window + 1 > 0) ? p_first[0] - window + 1 : 0;
  const int b0 = lo_key / KB;
  const int nblk = bend[ntiles - 1] - b0 + 1;
  const int kvh = head / (hq / hkv);

  pdl_wait();  // queries and this step's keys and values are the preceding kernel's output

  if (warp == 0) {
    // ---------------------------------------------------------------------------------------------- producer
    const int page = 1 << page_shift;
    const int pages_per_block = KB >> page_shift;
    const int last_page = (kvl - 1) >> page_shift;
    const int32_t* pages = table + (size_t)item * table_width;
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, (uint32_t)(ntiles * Sh::Q_TILE_BYTES));
      for (int t = 0; t < ntiles; ++t)
#pragma unroll
        for (int j = 0; j < Sh::DS; ++j)
          tma_load_2d(smem + Sh::Q_OFF + t * Sh::Q_TILE_BYTES + j * Sh::Q_SUB_BYTES, &map_q, head * D + 64 * j,
                      t0 + row0 + TILE_M * t, &bars->q_full);
    }
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int i = 0; ok && i < nblk; ++i) {
      const int b = b0 + i;
      int row_k = 0;
      if (lane < pages_per_block) {
        // pages past the request's last one hold nothing it may see; the last page is loaded in their place so that
        // what the masked columns multiply is finite
        const int pid = __ldg(pages + min(b * pages_per_block + lane, last_page));
        row_k = ((pid * 2) * hkv + kvh) * page;
      }
      const int row_v = row_k + hkv * page;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        uint64_t* empty = which ? &bars->v_empty[stage] : &bars->k_empty[stage];
        uint64_t* full = which ? &bars->v_full[stage] : &bars->k_full[stage];
        ok = mbar_wait(empty, phase ^ 1, abort, 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(full, (uint32_t)Sh::KV_STAGE_BYTES);
        __syncwarp();
        if (lane < pages_per_block) {
          unsigned char* dst = smem + (which ? Sh::V_OFF : Sh::K_OFF) + stage * Sh::KV_STAGE_BYTES + lane * page * 128;
#pragma unroll
          for (int j = 0; j < Sh::DS; ++j) tma_load_2d(dst + j * Sh::KV_SUB_BYTES, &map_kv, 64 * j, which ? row_v : row_k, full);
        }
      }
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------------------------------------------- MMA
    // All lanes follow the barriers; lane 0 issues.  The others only work on the block that holds the request's last
    // key: value rows behind it were never written by this request, and 0 x (whatever an earlier owner of the page
    // left there) must be 0, so those rows are cleared in shared memory before P V runs.
    const bool issuer = lane == 0;
    constexpr uint32_t IDESC_S = instr_desc(TILE_M, KB, false);
    constexpr uint32_t IDESC_O = instr_desc(TILE_M, D, true);
    const uint32_t q_addr = smem_u32(smem + Sh::Q_OFF), k_addr = smem_u32(smem + Sh::K_OFF);
    const uint32_t v_addr = smem_u32(smem + Sh::V_OFF), p_addr = smem_u32(smem + Sh::P_OFF);
    auto issue_s = [&](int t, uint32_t ks) {
      const uint32_t a = q_addr + t * Sh::Q_TILE_BYTES, bk = k_addr + ks * Sh::KV_STAGE_BYTES;
#pragma unroll
      for (int j = 0; j < Sh::DS; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_f16(tmem_base + Sh::S_COL + t * KB, smem_desc(a + j * Sh::Q_SUB_BYTES + k * 32),
                  smem_desc(bk + j * Sh::KV_SUB_BYTES + k * 32), IDESC_S, (j | k) != 0);
    };
    auto issue_pv = [&](int t, uint32_t vs) {
      const uint32_t a = p_addr + t * Sh::P_TILE_BYTES, bv = v_addr + vs * Sh::KV_STAGE_BYTES;
#pragma unroll
      for (int kk = 0; kk < KB / 16; ++kk)
        mma_f16(tmem_base + Sh::O_COL + t * D, smem_desc(a + (kk >> 2) * Sh::Q_SUB_BYTES + (kk & 3) * 32),
                smem_desc_mn(bv + kk * 2048, Sh::KV_SUB_BYTES), IDESC_O, kk != 0);
    };
    uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
    bool ok = mbar_wait(&bars->q_full, 0, abort, 2) && mbar_wait(&bars->k_full[0], 0, abort, 2);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      fence_after();
      if (issuer) {
        for (int t = 0; t < ntiles; ++t) {
          issue_s(t, 0);
          mma_commit(&bars->s_full[t]);
        }
        mma_commit(&bars->k_empty[0]);
      }
      ks = 1;
    }
    for (int i = 0; ok && i < nblk; ++i) {
      const int b = b0 + i;
      const bool next = i + 1 < nblk;
      ok = mbar_wait(&bars->v_full[vs], vph, abort, 2);
      if (ok && next) ok = mbar_wait(&bars->k_full[ks], kph, abort, 2);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int written = kvl - b * KB;  // rows of this block that hold the request's values
      if (written < KB) {
        unsigned char* stage = smem + Sh::V_OFF + vs * Sh::KV_STAGE_BYTES;
        const int first = written > 0 ? written : 0;
        for (int idx = first * 8 * Sh::DS + lane; idx < KB * 8 * Sh::DS; idx += 32) {
          const int row = idx / (8 * Sh::DS), rest = idx % (8 * Sh::DS);
          *reinterpret_cast<uint4*>(stage + (rest >> 3) * Sh::KV_SUB_BYTES + row * 128 + (rest & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_async_smem();
        __syncwarp();
      }
      fence_after();
      for (int t = 0; t < ntiles; ++t) {
        if (b > bend[t]) continue;
        ok = mbar_wait(&bars->p_ready[t], i & 1, abort, 2);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after();
        if (issuer) {
          issue_pv(t, vs);
          mma_commit(&bars->o_full[t]);
          if (next && b + 1 <= bend[t]) {
            issue_s(t, ks);
            mma_commit(&bars->s_full[t]);
          }
        }
      }
      if (!ok) break;
      if (issuer) mma_commit(&bars->v_empty[vs]);
      if (++vs == STAGES) { vs = 0; vph ^= 1; }
      if (next) {
        if (issuer) mma_commit(&bars->k_empty[ks]);
        if (++ks == STAGES) { ks = 0; kph ^= 1; }
      }
    }
  } else {
    // ----------------------------------------------------------------------------------------------- softmax
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;  // a warp may only touch tensor-memory lanes [32*(warp%4), +32)
    const int r = quarter * 32 + lane;
    if (t < ntiles) {
      const int row = row0 + TILE_M * t + r;             // among the request's new tokens
      const bool valid = row < n;
      const int pr = valid ? first_pos + row : -1;       // an absent row sees nothing
      const int lo_r = window > 0 ? pr - window + 1 : 0;
      const bool partial = row0 + TILE_M * (t + 1) > n;
      const float c = scale * LOG2E_F;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const uint32_t s_addr = lane_addr + Sh::S_COL + t * KB, o_addr = lane_addr + Sh::O_COL + t * D;
      unsigned char* p_row = smem + Sh::P_OFF + t * Sh::P_TILE_BYTES + r * 128;
      float o[D];
#pragma unroll
      for (int d = 0; d < D; ++d) o[d] = 0.f;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      const int my_blocks = bend[t] - b0 + 1;
      for (int i = 0; i < my_blocks; ++i) {
        const int key0 = (b0 + i) * KB;
        ok = mbar_wait(&bars->s_full[t], i & 1, abort, 3);
        if (!ok) break;
        fence_after();
        const bool need_mask = partial || key0 + KB - 1 > p_first[t] || (window > 0 && key0 < p_last[t] - window + 1);
        // pass 1: the row's maximum over this block
        float mx = -INFINITY;
#pragma unroll 1
        for (int cc = 0; cc < KB / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(s_addr + cc * 32, v);
          tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int key = key0 + cc * 32 + e;
              if (key <= pr && key >= lo_r) mx = fmaxf(mx, __uint_as_float(v[e]));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(v[e]), __uint_as_float(v[e + 1])));
          }
        }
        const float m_new = fmaxf(m_run, mx);
        const float m_ref = m_new == -INFINITY ? 0.f : m_new;   // a row that has seen nothing yet
        const float alpha = ex2((m_run - m_ref) * c);           // 0 while m_run is -inf
        const float mc = m_ref * c;
        // pass 2: P = exp(S - max) as bfloat16 into the swizzled operand tile, and its sum
        float sum = 0.f;
#pragma unroll 1
        for (int cc = 0; cc < KB / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(s_addr + cc * 32, v);
          tmem_ld_wait();
          float p[32];
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int key = key0 + cc * 32 + e;
              p[e] = (key <= pr && key >= lo_r) ? ex2(fmaf(__uint_as_float(v[e]), c, -mc)) : 0.f;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) p[e] = ex2(fmaf(__uint_as_float(v[e]), c, -mc));
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) sum += p[e];
          // keys [cc*32, +32) of the block: sub-tile (cc*32)/64, 16-byte chunks (cc*32 % 64)/8 .. +4 of the 128-byte row
          unsigned char* sub = p_row + ((cc * 32) >> 6) * Sh::Q_SUB_BYTES;
          const int chunk0 = ((cc * 32) & 63) >> 3;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 packed = make_uint4(pack2(p[q4 * 8 + 0], p[q4 * 8 + 1]), pack2(p[q4 * 8 + 2], p[q4 * 8 + 3]),
                                            pack2(p[q4 * 8 + 4], p[q4 * 8 + 5]), pack2(p[q4 * 8 + 6], p[q4 * 8 + 7]));
            *reinterpret_cast<uint4*>(sub + (((chunk0 + q4) ^ (r & 7)) << 4)) = packed;
          }
        }
        l_run = l_run * alpha + sum;
        m_run = m_new;
        fence_async_smem();   // P is read by the tensor cores
        fence_before();       // S has been read
        mbar_arrive(&bars->p_ready[t]);
        // O_block = P V of this block, added into the row's accumulator
        ok = mbar_wait(&bars->o_full[t], i & 1, abort, 3);
        if (!ok) break;
        fence_after();
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(o_addr + cc * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[cc * 32 + e] = fmaf(o[cc * 32 + e], alpha, __uint_as_float(v[e]));
        }
        fence_before();
      }
      if (ok && valid) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = out + ((size_t)(t0 + row) * hq + head) * D;
#pragma unroll
        for (int d = 0; d < D; d += 8)
          *reinterpret_cast<uint4*>(dst + d) = make_uint4(pack2(o[d] * inv, o[d + 1] * inv), pack2(o[d + 2] * inv, o[d + 3] * inv),
                                                          pack2(o[d + 4] * inv, o[d + 5] * inv), pack2(o[d + 6] * inv, o[d + 7] * inv));
      }
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

template <int D>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_kv, const void* table, int table_width, const void* item_start,
           const void* kv_len, void* out, int num_items, int num_pairs, int hq, int hkv, int page_shift, int window,
           float scale, int skip_single, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
    if (e != cudaSuccess) PSB_REFUSE("attention_prefill_tcgen05: cannot reserve %d bytes of shared memory: %s", smem_bytes<D>(), cudaGetErrorString(e));
    configured = true;
  }
  psb_launch(attention_prefill_tcgen05_kernel<D>, dim3(hq, num_pairs), dim3(THREADS), (size_t)smem_bytes<D>(), stream, map_q, map_kv,
             (const int32_t*)table, table_width, (const int32_t*)item_start, (const int32_t*)kv_len, (__nv_bfloat16*)out,
             num_items, hq, hkv, page_shift, window, scale, skip_single);
  return 0;
}

}  // namespace

// 1 if the kernel takes the head size and page size, else 0.
PSB_API int psb_attention_prefill_tcgen05_supported(int D, int page_size) {
  if (D != 64 && D != 128) return 0;
  const int kb = D == 64 ? 128 : 64;
  return page_size >= 8 && page_size <= kb && (page_size & (page_size - 1)) == 0 ? 1 : 0;
}

// rows (new tokens of one request, for one head) one CTA owns
PSB_API int psb_attention_prefill_tcgen05_rows_per_cta() { return ROWS_PER_CTA; }

// q [T, hq*D] and out [T, hq*D] bfloat16; kv [num_pages, 2, hkv, page_size, D] bfloat16; table [num_items, table_width]
// int32; item_start [num_items+1], kv_len [num_items] int32 on the device.  num_pairs: the sum over the requests this
// kernel owns (all, or those with more than one new token when skip_single) of ceil(new tokens / 256).
PSB_API int psb_attention_prefill_tcgen05(const void* q, const void* kv, const void* table, int table_width, const void* item_start,
                                          const void* kv_len, void* out, int num_items, int num_pairs, int T, int hq, int hkv,
                                          int D, int page_size, long long num_pages, int window, float scale, int skip_single,
                                          cudaStream_t stream) {
  if (!psb_attention_prefill_tcgen05_supported(D, page_size))
    PSB_REFUSE("attention_prefill_tcgen05: head size %d with pages of %d is not built (64 or 128; pages a power of two, 8..keys per block)", D, page_size);
  if (hq < 1 || hkv < 1 || hq % hkv) PSB_REFUSE("attention_prefill_tcgen05: %d query heads over %d key heads", hq, hkv);
  if (window < 0 || table_width < 1 || T < 1 || num_pages < 1) PSB_REFUSE("attention_prefill_tcgen05: bad sizes (window=%d table_width=%d T=%d)", window, table_width, T);
  if (num_items <= 0 || num_pairs <= 0) return 0;
  if (num_pairs > 65535) PSB_REFUSE("attention_prefill_tcgen05: %d row groups in one step (at most 65535)", num_pairs);
  const long long kv_rows = num_pages * 2 * hkv * page_size;
  if (kv_rows > 0x7fffffffLL) PSB_REFUSE("attention_prefill_tcgen05: the cache entry has %lld rows, beyond a TMA coordinate", kv_rows);
  if (((uintptr_t)q | (uintptr_t)kv | (uintptr_t)out) & 15) PSB_REFUSE("attention_prefill_tcgen05: operands must be 16-byte aligned");
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap map_q, map_kv;
  int r = make_map_bf16(&map_q, q, (uint64_t)T, (uint64_t)hq * D, (uint64_t)hq * D, TILE_M);
  if (r == 0) r = make_map_bf16(&map_kv, kv, (uint64_t)kv_rows, (uint64_t)D, (uint64_t)D, page_size);
  if (r == -1) PSB_REFUSE("attention_prefill_tcgen05: the driver does not export cuTensorMapEncodeTiled");
  if (r != 0) PSB_REFUSE("attention_prefill_tcgen05: cuTensorMapEncodeTiled failed with code %d", r);
  int rc;
  if (D == 64) rc = launch<64>(map_q, map_kv, table, table_width, item_start, kv_len, out, num_items, num_pairs, hq, hkv, page_shift, window, scale, skip_single, stream);
  else rc = launch<128>(map_q, map_kv, table, table_width, item_start, kv_len, out, num_items, num_pairs, hq, hkv, page_shift, window, scale, skip_single, stream);
  if (rc) return rc;
  PSB_LAUNCH_CHECK("attention_prefill_tcgen05");
  return 0;
}

// 0 while no bounded wait of this kernel has ever run out on the current device; reading it synchronises with the device.
PSB_API int psb_attention_tcgen05_status() { return tc::read_status(); }
