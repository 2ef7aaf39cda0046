// Causal grouped-query attention of prompt portions over the paged cache on the 5th-generation tensor cores.
//
// One CTA owns up to 256 consecutive new tokens of one request for one query head, as two tiles of 128 rows (or, when the
// step has too few such groups to give every SM one, up to 128 tokens as a single tile), and walks
// the keys they may see in blocks of KB keys (128 for a head size of 64, 64 for 128).  352 threads:
//   warp 0      producer: TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the two Q tiles once, and per block of
//               the pages that hold its keys and values, one box per page, into a ring of four or five stages (one
//               mbarrier per stage takes both, so the MMA warp waits once per block);
//   warp 1      (and, with 64 keys a block, warp 10 for S) MMA: one lane issues tcgen05.mma (cta_group::1, kind::f16, M=128):  S = Q K^T  (A and B K-major, N=KB)
//               into tensor memory, and  O += P V  (A = P from tensor memory, B = V MN-major exactly as the
//               cache stores it: keys x head dim, N = head dim).  S goes into three (128 keys a block) or four (64)
//               buffers in turn, so it is computed while the softmax of the blocks before it still runs.  This warp
//               sets the kernel's pace: what it waits on and issues per block and tile takes about as long as a
//               softmax warp's work on the block;
//   warps 2..5  softmax of tile 0, warps 6..9 of tile 1: one thread per row.  tcgen05.ld of the row of S, masks,
//               maximum and sum in float32 (three-input maxima and arithmetic on register pairs: the loop is bound by
//               the instructions it issues), P as bfloat16 into tensor memory over the scores it came from.  O
//               accumulates in tensor memory over the blocks; the row's reference maximum only follows the true one
//               when that has grown by more than 2^8, and only then is the row of O rescaled (tcgen05.ld, multiply,
//               tcgen05.st), which is rare.
// The two tiles alternate on the tensor cores: while one tile's rows are in the softmax, the other's products run.
// A step with few such CTAs and long cached prefixes (a prompt portion of a few hundred tokens) may also cut the keys
// into ranges: CTA (head, rows, range) then walks its share of the blocks and leaves an unnormalised partial result
// (float32 output, reference exponent, sum) per row, which attention_prefill_merge_kernel combines.
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
constexpr int SOFTMAX_WARPS = 4;                     // per tile: one thread per row, a warp per quarter of tensor-memory lanes
constexpr int S_WARP = 2 + SOFTMAX_WARPS * TILES;         // the warp that issues S = Q K^T (warp 1 issues O += P V)
constexpr int THREADS = 32 * (3 + SOFTMAX_WARPS * TILES);  // producer, two MMA warps, softmax
constexpr int MAX_STAGES = 5, MAX_S_BUFS = 4;
constexpr int TMEM_COLS = 512;
constexpr float LOG2E_F = 1.4426950408889634f;

template <int D>
struct Shape {
  static constexpr int KB = D == 64 ? 128 : 64;           // keys per block
  // S buffers, used in turn by the tiles' blocks: as many as tensor memory has room for beside the two output tiles.
  // With four, each of two tiles has two of its own and its next scores never wait for the other tile's softmax.
  static constexpr int S_BUFS = (TMEM_COLS - TILES * D) / KB >= 4 ? 4 : 3;
  // blocks of keys and values in shared memory at a time: S of one tile alone runs S_BUFS blocks ahead of its P V
  static constexpr int STAGES = S_BUFS + 1;
  static constexpr bool TWO_ISSUERS = KB == 64;           // S and P V issued by two warps (see the MMA warps)
  static constexpr int DS = D / 64;                       // 64-element sub-tiles along the head dim
  static constexpr int Q_TILE_BYTES = TILE_M * D * 2;
  static constexpr int Q_SUB_BYTES = TILE_M * 128;        // one [128 x 64] sub-tile
  static constexpr int KV_STAGE_BYTES = KB * D * 2;
  static constexpr int KV_SUB_BYTES = KB * 128;           // one [KB x 64] sub-tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILES * Q_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + STAGES * KV_STAGE_BYTES;
  static constexpr int BAR_OFF = V_OFF + STAGES * KV_STAGE_BYTES;
  static constexpr int S_COL = 0;                         // S buffer j: columns [j*KB, +KB)
  static constexpr int O_COL = S_BUFS * KB;               // O of tile t: columns [O_COL + t*D, +D)
  static_assert(O_COL + TILES * D <= TMEM_COLS && S_BUFS <= MAX_S_BUFS && STAGES <= MAX_STAGES, "tensor memory");
  static_assert(Q_TILE_BYTES % 1024 == 0 && KV_STAGE_BYTES % 1024 == 0, "swizzle atoms");
};

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[MAX_STAGES], kv_empty[MAX_STAGES];  // a block's keys and values arrive on one barrier
  uint64_t s_full[MAX_S_BUFS], p_used[MAX_S_BUFS], p_ready[TILES], o_full[TILES];
  uint32_t tmem_base;
  uint32_t abort;
};

template <int D>
constexpr int smem_bytes() { return Shape<D>::BAR_OFF + 1024 /* alignment slack */ + (int)sizeof(Barriers); }

// The softmax loops are bound by how many instructions they issue; sm_100 has float32 arithmetic on register pairs
// (one instruction, two results, each rounded as the scalar instruction would) and a maximum of three.
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void halves_of(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

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
                                 int hkv, int page_shift, int window, float scale, int skip_single, int rows_per_cta,
                                 int kv_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
  using Sh = Shape<D>;
  constexpr int KB = Sh::KB, NB = Sh::S_BUFS, STAGES = Sh::STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + Sh::BAR_OFF);
  volatile uint32_t* abort = &bars->abort;
  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;  // the warp's role is the same for all its lanes

  pdl_trigger();
  // which request and which 256 rows of it?  (lengths are inputs of the step: readable before the wait)
  const int head = blockIdx.x;
  int item = -1, pair = 0, n = 0;
  {
    int left = blockIdx.y;  // block 0 takes the last (longest) rows of the last request
    for (int i = num_items - 1; i >= 0; --i) {
      const int ni = item_start[i + 1] - item_start[i];
      if (skip_single && ni == 1) continue;
      const int pairs = (ni + rows_per_cta - 1) / rows_per_cta;
      if (left < pairs) { item = i; pair = pairs - 1 - left; n = ni; break; }
      left -= pairs;
    }
  }
  if (item < 0) return;  // uniform for the CTA, before anything is allocated

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int j = 0; j < NB; ++j) {
      mbar_init(&bars->s_full[j], 1);
      mbar_init(&bars->p_used[j], 1);
    }
    for (int t = 0; t < TILES; ++t) {
      mbar_init(&bars->p_ready[t], SOFTMAX_WARPS);  // one arrival per softmax warp of the tile (arrivals on one barrier serialise)
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
  const int row0 = pair * rows_per_cta;               // first of this CTA's rows among the new tokens
  const int rows_here = min(rows_per_cta, n - row0);
  const int ntiles = rows_here > TILE_M ? 2 : 1;
  int p_first[TILES], p_last[TILES], bend[TILES];
#pragma unroll
  for (int t = 0; t < TILES; ++t) {
    p_first[t] = first_pos + row0 + TILE_M * t;
    p_last[t] = first_pos + min(n, row0 + TILE_M * (t + 1)) - 1;
    bend[t] = p_last[t] / KB;
  }
  const int lo_key = (window > 0 && p_first[0] - window + 1 > 0) ? p_first[0] - window + 1 : 0;
  // the blocks this CTA's rows may see, and the share of them that is this CTA's key range (all of them without ranges)
  const int b_lo = lo_key / KB;
  const int per_range = (bend[ntiles - 1] - b_lo + kv_splits) / kv_splits;
  const int b0 = b_lo + (int)blockIdx.z * per_range;
#pragma unroll
  for (int t = 0; t < TILES; ++t) bend[t] = min(bend[t], b0 + per_range - 1);
  const int nblk = max(0, bend[ntiles - 1] - b0 + 1);
  const int kvh = head / (hq / hkv);
  // The tiles' blocks in the order their S is computed: (0,0) (1,0) (0,1) (1,1) ... while tile 0 still has blocks (n0 of
  // them), then tile 1's remaining ones.  The e-th of them uses S buffer e % NB, so S of a block is computed while the
  // softmax of the two blocks before it is still running.
  const int n0 = max(0, bend[0] - b0 + 1);   // a range may hold nothing that tile 0's (earlier) rows can see
  const int total = ntiles == 2 ? n0 + nblk : n0;
  auto seq_of = [&](int t, int i) { return ntiles == 1 ? i : (i < n0 ? 2 * i + t : n0 + i); };

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
      ok = mbar_wait(&bars->kv_empty[stage], phase ^ 1, abort, 1);  // P V of the block that used this stage has finished
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&bars->kv_full[stage], 2u * (uint32_t)Sh::KV_STAGE_BYTES);
      }
      __syncwarp();
      if (lane < pages_per_block) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          unsigned char* dst = smem + (which ? Sh::V_OFF : Sh::K_OFF) + stage * Sh::KV_STAGE_BYTES + lane * page * 128;
#pragma unroll
          for (int j = 0; j < Sh::DS; ++j)
            tma_load_2d(dst + j * Sh::KV_SUB_BYTES, &map_kv, 64 * j, which ? row_v : row_k, &bars->kv_full[stage]);
        }
      }
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1 || warp == S_WARP) {
    // --------------------------------------------------------------------------------------------------- MMA
    // With 64 keys a block (heads of 128) two warps issue the tensor-core instructions, S = Q K^T from one and
    // O += P V from the other: what one warp waits on and issues for both, per block and tile, took longer than a
    // softmax warp's work on the block and set the kernel's pace (8,192 tokens: 724 -> 568 us).  With 128 keys a block
    // the softmax takes twice as long per block and one warp keeps up; two were 5 % slower there (431 -> 452 us).
    // S of event e + NB takes the buffer that holds P of event e: one warp issues it behind that P V; with two, the S
    // warp waits until the P V has completed (p_used).  A block's keys are no longer needed once P V of its last tile
    // has been issued, because that follows the block's S of every tile through s_full, the softmax and p_ready.
    // All lanes follow the barriers; an elected lane issues each instruction (tcgen05.cuh says why).  All of them work
    // on the block that holds the request's last key: value rows behind it were never written by this request, and
    // 0 x (whatever an earlier owner of the page left there) must be 0, so those rows are cleared in shared memory
    // before P V runs.
    constexpr uint32_t IDESC_S = instr_desc(TILE_M, KB, false);
    constexpr uint32_t IDESC_O = instr_desc(TILE_M, D, true);
    // descriptors: low words (address field in 16-byte units, leading byte offset) of the operands' first tiles; the high
    // word is the same for all of them
    const uint64_t d_q = smem_desc(smem_u32(smem + Sh::Q_OFF)), d_k = smem_desc(smem_u32(smem + Sh::K_OFF));
    const uint64_t d_v = smem_desc_mn(smem_u32(smem + Sh::V_OFF), Sh::KV_SUB_BYTES);
    const uint32_t hi = (uint32_t)(d_q >> 32);  // stride byte offset, version, swizzle: equal in all three
    const uint32_t q_lo = (uint32_t)d_q, k_lo = (uint32_t)d_k, v_lo = (uint32_t)d_v;
    auto issue_s = [&](int t, uint32_t ks, int buf) {
      const uint32_t a = q_lo + t * (Sh::Q_TILE_BYTES >> 4), bk = k_lo + ks * (Sh::KV_STAGE_BYTES >> 4);
      const uint32_t dst = tmem_base + Sh::S_COL + buf * KB;
#pragma unroll
      for (int j = 0; j < Sh::DS; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_f16_split(dst, a + ((j * Sh::Q_SUB_BYTES + k * 32) >> 4), hi, bk + ((j * Sh::KV_SUB_BYTES + k * 32) >> 4), hi, IDESC_S,
                        (j | k) != 0);
    };
    // P of a block lies in the S buffer it was computed from: the 32 keys [32c, +32) of the block as 16 columns of two
    // bfloat16 at columns [32c, +16) (see the softmax warps); one MMA takes 16 keys, 8 columns
    auto issue_pv = [&](int t, uint32_t vs, int buf, int accumulate) {
      const uint32_t bv = v_lo + vs * (Sh::KV_STAGE_BYTES >> 4);
      const uint32_t dst = tmem_base + Sh::O_COL + t * D, src = tmem_base + Sh::S_COL + buf * KB;
#pragma unroll
      for (int kk = 0; kk < KB / 16; ++kk)
        mma_f16_tmem_a(dst, src + (kk >> 1) * 32 + (kk & 1) * 8, bv + ((kk * 2048) >> 4), hi, IDESC_O, (accumulate | kk) != 0);
    };
    // blocks (from b0) whose keys and values this warp has waited for (they arrive together), and blocks whose values
    // it has looked at
    int kv_seen = 0, v_seen = 0;
    auto tile_of = [&](int e) { return ntiles == 1 ? 0 : (e < 2 * n0 ? (e & 1) : 1); };
    auto block_of = [&](int e) { return ntiles == 1 ? e : (e < 2 * n0 ? (e >> 1) : e - n0); };
    auto block_ready = [&](int i) {  // waits (once) for every block up to i
      while (kv_seen <= i) {
        bool got = mbar_wait(&bars->kv_full[kv_seen % STAGES], (kv_seen / STAGES) & 1, abort, 2);
        got = __all_sync(0xffffffffu, got);
        if (!got) return false;
        ++kv_seen;
      }
      return true;
    };
    auto values_ready = [&](int i) {  // every block up to i: arrived, and the rows behind the request's last key cleared
      while (v_seen <= i) {
        if (!block_ready(v_seen)) return false;  // as a rule no wait: S of this block has been issued long ago
        const int written = kvl - (b0 + v_seen) * KB;  // rows of this block that hold the request's values
        if (written < KB) {
          unsigned char* stage = smem + Sh::V_OFF + (v_seen % STAGES) * Sh::KV_STAGE_BYTES;
          const int first = written > 0 ? written : 0;
          for (int idx = first * 8 * Sh::DS + lane; idx < KB * 8 * Sh::DS; idx += 32) {
            const int row = idx / (8 * Sh::DS), rest = idx % (8 * Sh::DS);
            *reinterpret_cast<uint4*>(stage + (rest >> 3) * Sh::KV_SUB_BYTES + row * 128 + (rest & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_async_smem();
          __syncwarp();
        }
        ++v_seen;
      }
      return true;
    };
    if constexpr (!Sh::TWO_ISSUERS) {
      if (warp == 1) {  // one warp issues both products, S of event e + NB behind P V of event e
        bool ok = mbar_wait(&bars->q_full, 0, abort, 2);
        ok = __all_sync(0xffffffffu, ok);
        for (int e = 0; ok && e < NB && e < total; ++e) {
          ok = block_ready(block_of(e));
          if (ok && elect_one()) {
            issue_s(tile_of(e), block_of(e) % STAGES, e % NB);
            mma_commit(&bars->s_full[e % NB]);
          }
          __syncwarp();
        }
        for (int e = 0; ok && e < total; ++e) {
          const int t = tile_of(e), i = block_of(e);
          ok = values_ready(i);
          const bool ahead = e + NB < total;  // S of the block NB steps on (it takes this block's buffer) goes out together with this P V
          if (ok && ahead) ok = block_ready(block_of(e + NB));
          if (!ok) break;
          ok = mbar_wait(&bars->p_ready[t], i & 1, abort, 2);  // P of this block is written (over its S)
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          fence_after();
          if (elect_one()) {
            issue_pv(t, i % STAGES, e % NB, i);
            mma_commit(&bars->o_full[t]);
            if (t == ntiles - 1) mma_commit(&bars->kv_empty[i % STAGES]);  // the last tile to use this block
            if (ahead) {
              issue_s(tile_of(e + NB), block_of(e + NB) % STAGES, e % NB);
              mma_commit(&bars->s_full[e % NB]);
            }
          }
          __syncwarp();
        }
      }
    } else if (warp == S_WARP) {
      bool ok = mbar_wait(&bars->q_full, 0, abort, 2);
      ok = __all_sync(0xffffffffu, ok);
      for (int e = 0; ok && e < total; ++e) {
        if (e >= NB) {  // P V of the event that had this buffer has read its P
          ok = mbar_wait(&bars->p_used[e % NB], ((e / NB) - 1) & 1, abort, 2);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          fence_after();
        }
        ok = block_ready(block_of(e));
        if (!ok) break;
        if (elect_one()) {
          issue_s(tile_of(e), block_of(e) % STAGES, e % NB);
          mma_commit(&bars->s_full[e % NB]);
        }
        __syncwarp();
      }
    } else {
      bool ok = true;
      for (int e = 0; ok && e < total; ++e) {
        const int t = tile_of(e), i = block_of(e);
        ok = values_ready(i);
        if (!ok) break;
        ok = mbar_wait(&bars->p_ready[t], i & 1, abort, 2);  // P of this block is written (over its S)
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after();
        if (elect_one()) {
          issue_pv(t, i % STAGES, e % NB, i);
          mma_commit(&bars->o_full[t]);
          mma_commit(&bars->p_used[e % NB]);
          if (t == ntiles - 1) mma_commit(&bars->kv_empty[i % STAGES]);  // the last tile to use this block
        }
        __syncwarp();
      }
    }
  } else {
    // ----------------------------------------------------------------------------------------------- softmax
    // One thread per row: it reads the row's scores of a block from tensor memory, finds the maximum, writes the
    // probabilities over the scores and keeps the row's running maximum and sum; nothing is shared between threads.
    // Measured per head size: with 128 keys a block the scores alone are 128 registers of the 168 a thread may have
    // (three warps on a scheduler), and arithmetic on register pairs, which wants them aligned, costs more in spills
    // than it saves in instructions; with 64 keys a block there is room and it pays.
    constexpr bool PAIRS = D == 128;
    const int sw = warp - 2;  // 0 .. SOFTMAX_WARPS * TILES - 1
    const int t = sw / SOFTMAX_WARPS;
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
      const uint32_t o_addr = lane_addr + Sh::O_COL + t * D;
      // m_run is the maximum the row's exponentials refer to.  It follows the true maximum only when that has grown by
      // more than 2^8 (in the exponent), so that the accumulator in tensor memory is rescaled rarely; sums and
      // products use the same reference, and the quotient at the end does not depend on it.
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      const int my_blocks = max(0, bend[t] - b0 + 1);
      // The row's scores of a block, 32 keys a chunk, stay in registers from the maximum to the exponentials.  They are
      // asked for as early as they can be: a block's scores are computed blocks ahead, so as a rule the loads of
      // block i+1 go out as soon as the exponentials of block i have let go of the registers, and arrive while this
      // thread waits for its stores and hands block i over.
      constexpr int NCH = KB / 32;
      float sv[NCH][32];
      auto load_scores = [&](int e) {
        fence_after();
        const uint32_t s_addr = lane_addr + Sh::S_COL + (e % NB) * KB;
#pragma unroll
        for (int cc = 0; cc < NCH; ++cc) tmem_ld32(s_addr + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[cc][0]));
      };
      auto request_scores = [&](int i) {  // false: a wait gave up
        const int e = seq_of(t, i);
        bool got = mbar_wait(&bars->s_full[e % NB], (e / NB) & 1, abort, 3);
        got = __all_sync(0xffffffffu, got);
        if (!got) return false;
        load_scores(e);
        return true;
      };
      auto request_scores_if_there = [&](int i) {  // asks for them only if they are computed already (the whole warp agrees)
        const int e = seq_of(t, i);
        if (!__all_sync(0xffffffffu, mbar_test_wait(&bars->s_full[e % NB], (e / NB) & 1))) return false;
        load_scores(e);
        return true;
      };
      if (my_blocks > 0) ok = request_scores(0);
      for (int i = 0; ok && i < my_blocks; ++i) {
        const int key0 = (b0 + i) * KB;
        const int e = seq_of(t, i);
        const uint32_t s_addr = lane_addr + Sh::S_COL + (e % NB) * KB;
        const bool need_mask = partial || key0 + KB - 1 > p_first[t] || (window > 0 && key0 < p_last[t] - window + 1);
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        tmem_ld_wait();
#pragma unroll
        for (int cc = 0; cc < NCH; ++cc) {
          float(&x)[32] = sv[cc];
          if (need_mask) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int key = key0 + cc * 32 + k;
              if (key > pr || key < lo_r) x[k] = -INFINITY;
            }
          }
#pragma unroll
          for (int k = 0; k < 32; k += 8) {
            mx0 = max3(mx0, x[k], x[k + 1]); mx1 = max3(mx1, x[k + 2], x[k + 3]);
            mx2 = max3(mx2, x[k + 4], x[k + 5]); mx3 = max3(mx3, x[k + 6], x[k + 7]);
          }
        }
        const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const bool grow = (m_new - m_run) * c > 8.f;  // false while the row has seen nothing (-inf - -inf)
        // Each phase of o_full (P V of this tile's block i-1 has finished) is waited for exactly once, during block i:
        // a parity wait can only tell the phase in progress from the one before it.  If O has to be rescaled, before
        // that.  Otherwise, with 128 keys a block, ahead of the exponentials too: P V of the block before has completed
        // by then as a rule, and nothing stands between this block's last store and its hand-over (8,192 tokens: 440 ->
        // 432 us); with 64 keys a block it often has not, and the wait comes at the end of the block (727 against 734).
        constexpr bool WAIT_EARLY = KB == 128;
        bool waited = i == 0;
        const bool any_grow = __any_sync(0xffffffffu, grow);
        if (i > 0 && (WAIT_EARLY || any_grow)) {
          ok = mbar_wait(&bars->o_full[t], (i - 1) & 1, abort, 3);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          waited = true;
        }
        if (any_grow) {
          // tensor-memory loads and stores are warp-wide: every lane takes part, with a factor of 1 where nothing grew
          const float alpha = grow ? ex2((m_run - m_new) * c) : 1.f;  // 0 from -inf
          if (grow) { m_run = m_new; l_run *= alpha; }
          if (i > 0) {
            fence_after();
#pragma unroll 1
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t v[32];
              tmem_ld32(o_addr + cc * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
              tmem_st32(o_addr + cc * 32, v);
            }
            tmem_st_wait();
          }
        }
        const float mc = (m_run == -INFINITY ? 0.f : m_run) * c;
        // P as bfloat16 over the S it came from: keys [32c, +32) of the block become 16 columns at the start of the 32
        // columns their scores occupied (the chunk is in registers by then, and nobody else reads those columns)
        const uint64_t c_pair = pair_of(c, c), mc_pair = pair_of(-mc, -mc);
        uint64_t sum_pair = pair_of(0.f, 0.f);  // even and odd keys add up apart
        float sum0 = 0.f, sum1 = 0.f;
        auto emit = [&](int cc, const float(&x)[32]) {
          uint32_t packed[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float p0, p1;                                        // masked entries are -inf: 0
            if constexpr (PAIRS) {
              float x0, x1;
              halves_of(fma_pair(pair_of(x[k], x[k + 1]), c_pair, mc_pair), x0, x1);
              p0 = ex2(x0), p1 = ex2(x1);
              sum_pair = add_pair(sum_pair, pair_of(p0, p1));
            } else {
              p0 = ex2(fmaf(x[k], c, -mc)), p1 = ex2(fmaf(x[k + 1], c, -mc));
              sum0 += p0;
              sum1 += p1;
            }
            packed[k >> 1] = pack2(p0, p1);
          }
          tmem_st16(s_addr + cc * 32, packed);
        };
#pragma unroll
        for (int cc = 0; cc < NCH; ++cc) emit(cc, sv[cc]);
        // The registers are free again: the next block's scores may start on their way, if they exist.  If they do
        // not, this block is handed over first: the other tile's next scores, and through them this tile's, are
        // computed behind this block's P V, and a warp that waited here would hold all of that up.
        const bool asked = i + 1 < my_blocks && request_scores_if_there(i + 1);
        tmem_st_wait();
        if constexpr (PAIRS) halves_of(sum_pair, sum0, sum1);
        l_run += sum0 + sum1;
        if (!waited) {
          ok = mbar_wait(&bars->o_full[t], (i - 1) & 1, abort, 3);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        fence_before();       // P written, O rescaled
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[t]);
        if (i + 1 < my_blocks && !asked) {
          ok = request_scores(i + 1);
          if (!ok) break;
        }
      }
      // the quotient
      if (ok && my_blocks > 0) {
        ok = mbar_wait(&bars->o_full[t], (my_blocks - 1) & 1, abort, 3);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok && kv_splits > 1) {
        // one key range of several: the row's unnormalised output with the exponent it refers to and its sum
        fence_after();
        const size_t slot = ((size_t)(t0 + row) * hq + head) * kv_splits + blockIdx.z;
        if (valid) {
          part_ml[slot * 2] = (my_blocks > 0 && m_run != -INFINITY) ? m_run * c : -INFINITY;
          part_ml[slot * 2 + 1] = my_blocks > 0 ? l_run : 0.f;
        }
        if (my_blocks > 0) {
          float* dst = part_o + slot * D;
#pragma unroll 1
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t v[32];
            tmem_ld32(o_addr + cc * 32, v);
            tmem_ld_wait();
            if (valid) {
#pragma unroll
              for (int k = 0; k < 32; k += 4)
                *reinterpret_cast<float4*>(dst + cc * 32 + k) = make_float4(__uint_as_float(v[k]), __uint_as_float(v[k + 1]),
                                                                            __uint_as_float(v[k + 2]), __uint_as_float(v[k + 3]));
            }
          }
        }
        fence_before();
      } else if (ok) {
        fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = out + ((size_t)(t0 + row) * hq + head) * D;
#pragma unroll 1
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(o_addr + cc * 32, v);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int k = 0; k < 32; k += 8)
              *reinterpret_cast<uint4*>(dst + cc * 32 + k) =
                  make_uint4(pack2(__uint_as_float(v[k]) * inv, __uint_as_float(v[k + 1]) * inv),
                             pack2(__uint_as_float(v[k + 2]) * inv, __uint_as_float(v[k + 3]) * inv),
                             pack2(__uint_as_float(v[k + 4]) * inv, __uint_as_float(v[k + 5]) * inv),
                             pack2(__uint_as_float(v[k + 6]) * inv, __uint_as_float(v[k + 7]) * inv));
          }
        }
        fence_before();
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

// One warp per (token, head): combines the key ranges' partial results.  out = sum_s w_s O_s / sum_s w_s l_s with
// w_s = 2^(e_s - max e); a range that saw nothing (sum 0) has weight 0 and its output is not read.
template <int D>
__global__ void attention_prefill_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                               const int32_t* __restrict__ token_item, const int32_t* __restrict__ item_start,
                                               __nv_bfloat16* __restrict__ out, int T, int hq, int kv_splits, int skip_single) {
  pdl_trigger();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int row = unit / hq, head = unit - row * hq;
  int n = 0;
  if (row < T) {
    const int item = token_item[row];
    n = item_start[item + 1] - item_start[item];
  }
  pdl_wait();
  if (row >= T || (skip_single && n == 1)) return;  // a single token's row belongs to the decode kernel
  const size_t base = ((size_t)row * hq + head) * kv_splits;
  const float e = lane < kv_splits ? part_ml[(base + lane) * 2] : -INFINITY;
  const float l = lane < kv_splits ? part_ml[(base + lane) * 2 + 1] : 0.f;
  const float top = warp_max(e);
  float w = (l > 0.f && e != -INFINITY) ? ex2(e - top) : 0.f;
  const float total = warp_sum(w * l);
  const float inv = total > 0.f ? 1.f / total : 0.f;
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < kv_splits; ++s) {
    const float ws = __shfl_sync(0xffffffffu, w, s);
    if (ws == 0.f) continue;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] = fmaf(ws, part_o[(base + s) * D + lane + 32 * i], acc[i]);
  }
  __nv_bfloat16* dst = out + ((size_t)row * hq + head) * D;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(acc[i] * inv);
}

template <int D>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_kv, const void* table, int table_width, const void* item_start,
           const void* kv_len, void* out, int num_items, int num_pairs, int hq, int hkv, int page_shift, int window,
           float scale, int skip_single, int rows_per_cta, int kv_splits, void* part_o, void* part_ml, const void* token_item,
           int T, cudaStream_t stream) {
  static PsbPerDevice configured; 
  if (!configured.get()) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
    if (e != cudaSuccess) PSB_REFUSE("attention_prefill_tcgen05: cannot reserve %d bytes of shared memory: %s", smem_bytes<D>(), cudaGetErrorString(e));
    configured.set(); 
  }
  psb_launch(attention_prefill_tcgen05_kernel<D>, dim3(hq, num_pairs, kv_splits), dim3(THREADS), (size_t)smem_bytes<D>(), stream, map_q, map_kv,
             (const int32_t*)table, table_width, (const int32_t*)item_start, (const int32_t*)kv_len, (__nv_bfloat16*)out,
             num_items, hq, hkv, page_shift, window, scale, skip_single, rows_per_cta, kv_splits, (float*)part_o, (float*)part_ml);
  if (kv_splits > 1) {
    const long long units = (long long)T * hq;
    psb_launch(attention_prefill_merge_kernel<D>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, (const float*)part_o,
               (const float*)part_ml, (const int32_t*)token_item, (const int32_t*)item_start, (__nv_bfloat16*)out, T, hq, kv_splits,
               skip_single);
  }
  return 0;
}

}  // namespace

// 1 if the kernel takes the head size and page size, else 0.
PSB_API int psb_attention_prefill_tcgen05_supported(int D, int page_size) {
  if (D != 64 && D != 128) return 0;
  const int kb = D == 64 ? 128 : 64;
  return page_size >= 8 && page_size <= kb && (page_size & (page_size - 1)) == 0 ? 1 : 0;
}

// rows (new tokens of one request, for one head) one CTA owns at most; a launch may ask for half of that
PSB_API int psb_attention_prefill_tcgen05_rows_per_cta() { return ROWS_PER_CTA; }

// q [T, hq*D] and out [T, hq*D] bfloat16; kv [num_pages, 2, hkv, page_size, D] bfloat16; table [num_items, table_width]
// int32; item_start [num_items+1], kv_len [num_items] int32 on the device.  rows_per_cta: 256 or 128.  num_pairs: the sum
// over the requests this kernel owns (all, or those with more than one new token when skip_single) of
// ceil(new tokens / rows_per_cta).  kv_splits > 1: the keys are cut into that many ranges; part_o (float32
// [T, hq, kv_splits, D]) and part_ml ([T, hq, kv_splits, 2]) take the ranges' partial results, token_item ([T] int32)
// tells the merge which request a row belongs to.
PSB_API int psb_attention_prefill_tcgen05(const void* q, const void* kv, const void* table, int table_width, const void* item_start,
                                          const void* kv_len, void* out, int num_items, int num_pairs, int T, int hq, int hkv,
                                          int D, int page_size, long long num_pages, int window, float scale, int skip_single,
                                          int rows_per_cta, int kv_splits, void* part_o, void* part_ml, const void* token_item,
                                          cudaStream_t stream) {
  if (kv_splits < 1 || kv_splits > 32 || (kv_splits > 1 && (!part_o || !part_ml || !token_item)))
    PSB_REFUSE("attention_prefill_tcgen05: %d key ranges (1 to 32), or their scratch is missing", kv_splits);
  if (rows_per_cta != ROWS_PER_CTA && rows_per_cta != TILE_M) PSB_REFUSE("attention_prefill_tcgen05: a CTA owns %d or %d rows, not %d", ROWS_PER_CTA, TILE_M, rows_per_cta);
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
  if (D == 64) rc = launch<64>(map_q, map_kv, table, table_width, item_start, kv_len, out, num_items, num_pairs, hq, hkv, page_shift, window, scale, skip_single, rows_per_cta, kv_splits, part_o, part_ml, token_item, T, stream);
  else rc = launch<128>(map_q, map_kv, table, table_width, item_start, kv_len, out, num_items, num_pairs, hq, hkv, page_shift, window, scale, skip_single, rows_per_cta, kv_splits, part_o, part_ml, token_item, T, stream);
  if (rc) return rc;
  PSB_LAUNCH_CHECK("attention_prefill_tcgen05");
  return 0;
}

// 0 while no bounded wait of this kernel has ever run out on the current device; reading it synchronises with the device.
PSB_API int psb_attention_tcgen05_status() { return tc::read_status(); }
