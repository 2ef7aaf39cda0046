// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// float32 accumulation, float32 online softmax), for prefill portions and for
// decode.  Keys and values go from global memory straight into MMA operand
// registers with 16-byte loads: no shared-memory staging.  That works because a
// dot product does not care about the order of its terms:
//  * QK^T: lane (g, t) of a quad-row loads 8 consecutive head dims of key g; the
//    query fragment is loaded with the same permutation of head dims.
//  * PV: lane (g, t) loads, for tokens {2t, 2t+1, 2t+8, 2t+9} of a 16-key tile, the
//    D/8 consecutive head dims starting at g*D/8; output column n of d-tile j is
//    then head dim n*D/8 + j, so each lane ends up owning D/4 consecutive dims.
// A warp therefore reads whole 64..256-byte runs of each key/value row, coalesced.
//
// Rows of the score matrix are (token, query head in the group) pairs of ONE
// key/value head, so keys and values are read once per group of query heads.
//
// Two kernels:
//  * prefill: a CTA owns 128 rows of one item (4 warps x 32 rows) and walks the keys
//    they may see (causal, optional window) in blocks of 64 shared through a ring
//    in shared memory;
//  * decode: a CTA owns one (item, key/value head, key range); its 4 warps take
//    16-key tiles in turn and merge at the end; key ranges of one item are merged
//    by a second small kernel (split-KV).  Only items that bring exactly one token.
//
// Math as in the generic kernel (prefixserve/model/attention.py:68-121 of
// PrefixServe): scores * scale, key j visible to position p iff j <= p (and
// j > p - window), softmax in float32, probabilities rounded to bfloat16 before
// the PV product (as the reference's probs.to(dtype), :119).
//
// Cache layout of one entry: [num_pages, 2, hkv, page_size, D], page_size a multiple of 16.
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 2^x by the hardware approximation (ex2.approx: relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// One 16-key tile in operand order.
template <int D>
struct KVTile {
  uint4 k[2][D / 32];  // [key half (keys g and g+8)][chunk of 32 head dims]
  uint4 v[4][D / 64];  // [token slot 2t, 2t+1, 2t+8, 2t+9][16-byte piece of this lane's D/8 dims]
};

// kp/vp point at key 0 of the tile for this key/value head; rows are D apart.
// Keys at index >= valid (counted from the tile's first key) are read as zeros.
template <int D>
__device__ __forceinline__ void load_tile(KVTile<D>& tile, const __nv_bfloat16* kp, const __nv_bfloat16* vp, int valid,
                                          int g, int t) {
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int key = half * 8 + g;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) tile.k[half][c] = key < valid ? ldg16(kp + key * D + c * 32 + t * 8) : zero;
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int key = 2 * t + (s & 1) + (s >> 1) * 8;
#pragma unroll
    for (int c = 0; c < D / 64; ++c) tile.v[s][c] = key < valid ? ldg16(vp + key * D + g * (D / 8) + c * 8) : zero;
  }
}

// Query fragments of one 16-row tile, permuted like the keys.  row0/row1: pointers to the rows g and g+8 (or null).
template <int D>
__device__ __forceinline__ void load_q(uint32_t (&qa)[D / 16][4], const __nv_bfloat16* row0, const __nv_bfloat16* row1, int t) {
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    const uint4 x = row0 ? ldg16(row0 + c * 32 + t * 8) : zero;
    const uint4 z = row1 ? ldg16(row1 + c * 32 + t * 8) : zero;
    qa[2 * c][0] = x.x; qa[2 * c][1] = z.x; qa[2 * c][2] = x.y; qa[2 * c][3] = z.y;
    qa[2 * c + 1][0] = x.z; qa[2 * c + 1][1] = z.z; qa[2 * c + 1][2] = x.w; qa[2 * c + 1][3] = z.w;
  }
}

// Running softmax state of the two rows (g, g+8) this lane sees of a 16-row tile.
template <int D>
struct RowState {
  float m[2];          // running maximum, in the scaled log2 domain
  float l[2];          // this lane's part of the running sum
  float o[D / 8][4];   // output accumulators, d-tile j: {row g: n=2t, 2t+1; row g+8: n=2t, 2t+1}
  __device__ __forceinline__ void init() {
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  }
};

// Scores of 16 rows x 16 keys; s[half][0..1] row g, s[half][2..3] row g+8; key = half*8 + 2t + (i&1).
template <int D>
__device__ __forceinline__ void scores(float (&s)[2][4], const uint32_t (&qa)[D / 16][4], const KVTile<D>& tile) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    s[half][0] = s[half][1] = s[half][2] = s[half][3] = 0.f;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      mma_bf16(s[half], qa[2 * c], tile.k[half][c].x, tile.k[half][c].y);
      mma_bf16(s[half], qa[2 * c + 1], tile.k[half][c].z, tile.k[half][c].w);
    }
  }
}

// Folds one tile's (already masked: -inf where hidden) scores into the running state and accumulates P.V.
// upper: rows 8..15 of the tile exist (false for the single token of a group of at most 8 query heads: they are padding).
template <int D>
__device__ __forceinline__ void fold(RowState<D>& st, float (&s)[2][4], const KVTile<D>& tile, float sl2, bool upper = true) {
  float p[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (r == 1 && !upper) continue;
    float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m[r], mx * sl2);
    const float m_safe = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen nothing yet
    const float alpha = fast_exp2(st.m[r] - m_safe);
    st.m[r] = m_new;
    float sum = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float e = fast_exp2(fmaf(s[half][2 * r + i], sl2, -m_safe));
        p[half][2 * r + i] = e;
        sum += e;
      }
    st.l[r] = st.l[r] * alpha + sum;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      st.o[j][2 * r] *= alpha;
      st.o[j][2 * r + 1] *= alpha;
    }
  }
  uint32_t pa[4];
  pa[0] = pack_bf16(p[0][0], p[0][1]);
  pa[1] = pack_bf16(p[0][2], p[0][3]);
  pa[2] = pack_bf16(p[1][0], p[1][1]);
  pa[3] = pack_bf16(p[1][2], p[1][3]);
  const uint32_t* v0 = reinterpret_cast<const uint32_t*>(&tile.v[0][0]);
  const uint32_t* v1 = reinterpret_cast<const uint32_t*>(&tile.v[1][0]);
  const uint32_t* v2 = reinterpret_cast<const uint32_t*>(&tile.v[2][0]);
  const uint32_t* v3 = reinterpret_cast<const uint32_t*>(&tile.v[3][0]);
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
    const uint32_t b0 = __byte_perm(v0[j >> 1], v1[j >> 1], sel);
    const uint32_t b1 = __byte_perm(v2[j >> 1], v3[j >> 1], sel);
    mma_bf16(st.o[j], pa, b0, b1);
  }
}

// Hides keys the row may not see.  key0: absolute position of the tile's first key; pos[r]/lo[r]: the row's own
// position and its lowest visible key.
__device__ __forceinline__ void mask_tile(float (&s)[2][4], int key0, int t, const int (&pos)[2], const int (&lo)[2]) {
#pragma unroll
  for (int half = 0; half < 2; ++half)
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int key = key0 + half * 8 + 2 * t + i;
        if (key > pos[r] || key < lo[r]) s[half][2 * r + i] = -INFINITY;
      }
}

// ---------------------------------------------------------------------------------------------- decode
// grid (splits, hkv, items).  Partial results (float32): part_o[item][head][split][D], part_ml[item][head][split][2].
//
// Each lane streams the 16-byte pieces it will need (the same ones load_tile reads) through a ring of its own in
// shared memory with cp.async: slot = ((warp*STAGES + stage)*PIECES + piece)*32 + lane.  A lane only ever touches
// its own slots, so the ring needs no barrier, only cp.async group counting, and it keeps STAGES-1 tiles per warp in
// flight without holding them in registers.
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int D>
struct DecodeShape {
  static constexpr int PIECES = 2 * (D / 32) + 4 * (D / 64);  // 16-byte pieces per lane per tile
  static constexpr int STAGES = 3;
  static constexpr int STAGE_BYTES = PIECES * 32 * 16;
  static constexpr int RING_BYTES = WARPS * STAGES * STAGE_BYTES;
  static constexpr int MERGE_BYTES = WARPS * 16 * (D + 4 + 2) * 4;
  static constexpr int SMEM_BYTES = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
};

__device__ __forceinline__ void cp16_cg(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp16_cg_zfill(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// --------------------------------------------------------------------------------------------- prefill
// A CTA owns 64*MT rows ((token, head-in-group) pairs of one key/value head of one item); its 4 warps own 16*MT rows
// each.  Keys are walked in blocks of 64 (four 16-key tiles): warp w brings tile w of every block into a ring in
// shared memory with cp.async, laid out piece-by-piece exactly as lanes will read them ((tile*PIECES + piece)*32 +
// lane), so every warp reads every tile without bank conflicts and each key/value is fetched once per CTA.  Scores
// of a whole block are held in registers and folded into the running softmax once per block.
template <int D>
struct PrefillShape {
  static constexpr int PIECES = 2 * (D / 32) + 4 * (D / 64);
  static constexpr int STAGES = 3;
  static constexpr int TILE_BYTES = PIECES * 32 * 16;
  static constexpr int STAGE_BYTES = WARPS * TILE_BYTES;  // one 64-key block
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES;
};

template <int D, int MT>
__global__ void __launch_bounds__(WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                         const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ item_start,
                         const int32_t* __restrict__ kv_len, __nv_bfloat16* __restrict__ out, int num_items, int hq, int hkv,
                         int page_shift, int window, float scale, int skip_single) {
  using Shape = PrefillShape<D>;
  constexpr int STAGES = Shape::STAGES, PIECES = Shape::PIECES, KP = 2 * (D / 32);
  constexpr int ROWS = WARPS * 16 * MT;  // rows per CTA
  constexpr int BLOCK = WARPS * 16;      // keys per block
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  const int G = hq / hkv;
  const int h = blockIdx.y;
  // which item and which of its row tiles is this CTA?  (lengths are inputs of the step: readable before the wait)
  int item = -1, tile = 0, n = 0;
  {
    int left = blockIdx.x;  // block 0 takes the last (longest) row tile of the last item
    for (int i = num_items - 1; i >= 0; --i) {
      const int ni = item_start[i + 1] - item_start[i];
      if (skip_single && ni == 1) continue;
      const int tiles = (ni * G + ROWS - 1) / ROWS;
      if (left < tiles) { item = i; tile = tiles - 1 - left; n = ni; break; }
      left -= tiles;
    }
  }
  pdl_wait();
  if (item < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int t0 = item_start[item];
  const int kvl = kv_len[item];
  const int first_pos = kvl - n;  // position of the item's first new token
  const int32_t* pages = table + (size_t)item * table_width;
  const float sl2 = scale * LOG2E;
  const int page_size = 1 << page_shift;
  const size_t page_elems = (size_t)2 * hkv * page_size * D;
  const __nv_bfloat16* kv_head = kv + (size_t)h * page_size * D;
  const int v_off = hkv * page_size * D;
  const int rows = n * G;

  // ---- this warp's rows
  const int r_base = tile * ROWS + warp * 16 * MT;
  uint32_t qa[MT][D / 16][4];
  int pos[MT][2], lo[MT][2], tok[MT][2], head[MT][2];
  int w_max_pos = -1, w_min_pos = 0x7fffffff, w_min_lo = 0x7fffffff, w_max_lo = 0;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const __nv_bfloat16* rp[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r_base + mt * 16 + g + 8 * r;
      if (row < rows) {
        tok[mt][r] = row / G;
        head[mt][r] = h * G + row % G;
        pos[mt][r] = first_pos + tok[mt][r];
        lo[mt][r] = (window > 0 && pos[mt][r] - window + 1 > 0) ? pos[mt][r] - window + 1 : 0;
        rp[r] = q + ((size_t)(t0 + tok[mt][r]) * hq + head[mt][r]) * D;
        w_max_pos = max(w_max_pos, pos[mt][r]);
        w_min_pos = min(w_min_pos, pos[mt][r]);
        w_min_lo = min(w_min_lo, lo[mt][r]);
        w_max_lo = max(w_max_lo, lo[mt][r]);
      } else {
        tok[mt][r] = -1; head[mt][r] = 0; pos[mt][r] = -1; lo[mt][r] = 0x7fffffff;
        rp[r] = nullptr;
      }
    }
    load_q<D>(qa[mt], rp[0], rp[1], t);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    w_max_pos = max(w_max_pos, __shfl_xor_sync(0xffffffffu, w_max_pos, o));
    w_min_pos = min(w_min_pos, __shfl_xor_sync(0xffffffffu, w_min_pos, o));
    w_min_lo = min(w_min_lo, __shfl_xor_sync(0xffffffffu, w_min_lo, o));
    w_max_lo = max(w_max_lo, __shfl_xor_sync(0xffffffffu, w_max_lo, o));
  }
  // ---- the CTA's key range: rows of the tile are consecutive, so its first and last row bound everything
  const int first_row = tile * ROWS, last_row = min(rows, first_row + ROWS) - 1;
  const int cta_max_pos = first_pos + last_row / G;
  const int cta_first_pos = first_pos + first_row / G;
  const int cta_min_lo = (window > 0 && cta_first_pos - window + 1 > 0) ? cta_first_pos - window + 1 : 0;
  const int k_first = cta_min_lo & ~(BLOCK - 1);
  const int n_blocks = (cta_max_pos - k_first) / BLOCK + 1;

  // ---- ring: warp w copies tile w of each block
  int off[PIECES], key_of[PIECES];
  {
    int piece = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int c = 0; c < D / 32; ++c, ++piece) {
        key_of[piece] = half * 8 + g;
        off[piece] = key_of[piece] * D + c * 32 + t * 8;
      }
#pragma unroll
    for (int sl = 0; sl < 4; ++sl)
#pragma unroll
      for (int c = 0; c < D / 64; ++c, ++piece) {
        key_of[piece] = 2 * t + (sl & 1) + (sl >> 1) * 8;
        off[piece] = v_off + key_of[piece] * D + g * (D / 8) + c * 8;
      }
  }
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t my_slot0 = smem0 + warp * Shape::TILE_BYTES + lane * 16;  // where this lane writes (stage 0)
  const uint32_t rd0 = smem0 + lane * 16;                                   // where this lane reads (stage 0, tile 0)
  auto fetch_pages = [&](int first_block) {  // page ids of this warp's tile in blocks first_block + lane
    const int key = k_first + (first_block + lane) * BLOCK + warp * 16;
    return (first_block + lane < n_blocks && key <= cta_max_pos) ? pages[key >> page_shift] : 0;
  };
  int page_ids = fetch_pages(0);
  int issued = 0, issue_stage = 0;
  auto issue = [&]() {
    if ((issued & 31) == 0 && issued > 0) page_ids = fetch_pages(issued);
    const int page = __shfl_sync(0xffffffffu, page_ids, issued & 31);
    const int key0 = k_first + issued * BLOCK + warp * 16;
    const uint32_t slot = my_slot0 + issue_stage * Shape::STAGE_BYTES;
    int valid = min(kvl, cta_max_pos + 1) - key0;  // keys of this tile anybody in the CTA may see
    const __nv_bfloat16* base = kv_head + (size_t)page * page_elems + (size_t)(key0 & (page_size - 1)) * D;
    if (valid >= 16) {
#pragma unroll
      for (int i = 0; i < PIECES; ++i) cp16_cg(slot + i * 512, base + off[i]);
    } else {  // keys nobody may see (or that do not exist) are filled with zeros, never read from memory
#pragma unroll
      for (int i = 0; i < PIECES; ++i) {
        const bool ok = key_of[i] < valid;
        cp16_cg_zfill(slot + i * 512, ok ? base + off[i] : kv, ok ? 16 : 0);
      }
    }
    ++issued;
    if (++issue_stage == STAGES) issue_stage = 0;
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (issued < n_blocks) issue();
    cp_async_commit();
  }

  RowState<D> st[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) st[mt].init();
  const bool warp_live = r_base < rows;

  int read_stage = 0;
  for (int b = 0; b < n_blocks; ++b) {
    cp_async_wait<STAGES - 2>();  // this thread's copies of block b have landed
    __syncthreads();              // ... and everybody's; and everybody is done with block b-1
    if (issued < n_blocks) issue();  // block b + STAGES - 1 goes where block b - 1 was
    cp_async_commit();
    const int key_b = k_first + b * BLOCK;
    const uint32_t rd = rd0 + read_stage * Shape::STAGE_BYTES;
    if (++read_stage == STAGES) read_stage = 0;
    if (!warp_live || key_b > w_max_pos || key_b + BLOCK <= w_min_lo) continue;  // nothing here for this warp's rows

    float s[MT][2 * WARPS][4];
#pragma unroll
    for (int tl = 0; tl < WARPS; ++tl) {
      uint4 kf[KP];
#pragma unroll
      for (int j = 0; j < KP; ++j) kf[j] = lds16(rd + tl * Shape::TILE_BYTES + j * 512);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float(&acc)[4] = s[mt][2 * tl + half];
          acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            const uint4 kk = kf[half * (D / 32) + c];
            mma_bf16(acc, qa[mt][2 * c], kk.x, kk.y);
            mma_bf16(acc, qa[mt][2 * c + 1], kk.z, kk.w);
          }
        }
    }
    const bool needs_mask = key_b + BLOCK - 1 > w_min_pos || key_b < w_max_lo;
    uint32_t pa[MT][WARPS][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (needs_mask) {
#pragma unroll
        for (int nt = 0; nt < 2 * WARPS; ++nt)
#pragma unroll
          for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int key = key_b + nt * 8 + 2 * t + i;
              if (key > pos[mt][r] || key < lo[mt][r]) s[mt][nt][2 * r + i] = -INFINITY;
            }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2 * WARPS; ++nt) mx = fmaxf(mx, fmaxf(s[mt][nt][2 * r], s[mt][nt][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st[mt].m[r], mx * sl2);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2(st[mt].m[r] - m_safe);
        st[mt].m[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2 * WARPS; ++nt)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float e = fast_exp2(fmaf(s[mt][nt][2 * r + i], sl2, -m_safe));
            s[mt][nt][2 * r + i] = e;
            sum += e;
          }
        st[mt].l[r] = st[mt].l[r] * alpha + sum;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          st[mt].o[j][2 * r] *= alpha;
          st[mt].o[j][2 * r + 1] *= alpha;
        }
      }
#pragma unroll
      for (int tl = 0; tl < WARPS; ++tl) {
        pa[mt][tl][0] = pack_bf16(s[mt][2 * tl][0], s[mt][2 * tl][1]);
        pa[mt][tl][1] = pack_bf16(s[mt][2 * tl][2], s[mt][2 * tl][3]);
        pa[mt][tl][2] = pack_bf16(s[mt][2 * tl + 1][0], s[mt][2 * tl + 1][1]);
        pa[mt][tl][3] = pack_bf16(s[mt][2 * tl + 1][2], s[mt][2 * tl + 1][3]);
      }
    }
#pragma unroll
    for (int tl = 0; tl < WARPS; ++tl) {
      uint4 vf[PIECES - KP];
#pragma unroll
      for (int j = 0; j < PIECES - KP; ++j) vf[j] = lds16(rd + tl * Shape::TILE_BYTES + (KP + j) * 512);
      const uint32_t* v0 = reinterpret_cast<const uint32_t*>(&vf[0 * (D / 64)]);
      const uint32_t* v1 = reinterpret_cast<const uint32_t*>(&vf[1 * (D / 64)]);
      const uint32_t* v2 = reinterpret_cast<const uint32_t*>(&vf[2 * (D / 64)]);
      const uint32_t* v3 = reinterpret_cast<const uint32_t*>(&vf[3 * (D / 64)]);
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(v0[j >> 1], v1[j >> 1], sel);
        const uint32_t b1 = __byte_perm(v2[j >> 1], v3[j >> 1], sel);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) mma_bf16(st[mt].o[j], pa[mt][tl], b0, b1);
      }
    }
  }
  cp_async_wait<0>();
  if (!warp_live) return;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = st[mt].l[r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (tok[mt][r] < 0) continue;
      const float inv = 1.f / l;
      __nv_bfloat16* orow = out + ((size_t)(t0 + tok[mt][r]) * hq + head[mt][r]) * D;
      // this lane owns dims [2t*D/8, (2t+2)*D/8): accumulator column 2t is the first half, 2t+1 the second
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        *reinterpret_cast<uint32_t*>(orow + (2 * t) * (D / 8) + j) =
            pack_bf16(st[mt].o[j][2 * r] * inv, st[mt].o[j + 1][2 * r] * inv);
        *reinterpret_cast<uint32_t*>(orow + (2 * t + 1) * (D / 8) + j) =
            pack_bf16(st[mt].o[j][2 * r + 1] * inv, st[mt].o[j + 1][2 * r + 1] * inv);
      }
    }
}

// all_single: every item of the step brings one token (then item i's token is row i and item_start need not be read).
template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                        const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ item_start,
                        const int32_t* __restrict__ kv_len, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int hq, int hkv, int page_shift, int window, float scale, int chunk,
                        int max_splits, int all_single) {
  using Shape = DecodeShape<D>;
  constexpr int STAGES = Shape::STAGES, PIECES = Shape::PIECES, KP = 2 * (D / 32);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // Lengths and page tables are inputs of the step: they may be read before the preceding kernel has finished.
  pdl_trigger();
  const int item = blockIdx.z, h = blockIdx.y, split = blockIdx.x;
  int t0 = item;
  bool mine = true;
  if (!all_single) {
    t0 = item_start[item];
    mine = item_start[item + 1] - t0 == 1;  // otherwise not a decode item: the prefill kernel has it
  }
  const int G = hq / hkv;
  const int kvl = kv_len[item];
  const int p = kvl - 1;
  const int lo_key = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int k_begin = (lo_key & ~15) + split * chunk;
  if (!mine || k_begin >= kvl) {  // the merge kernel knows how many splits this item has
    pdl_wait();
    return;
  }
  const int k_end = min(k_begin + chunk, kvl);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int32_t* pages = table + (size_t)item * table_width;
  const float sl2 = scale * LOG2E;
  const int page_size = 1 << page_shift;
  const size_t page_elems = (size_t)2 * hkv * page_size * D;
  const __nv_bfloat16* kv_head = kv + (size_t)h * page_size * D;
  const int v_off = hkv * page_size * D;

  // element offsets of this lane's pieces from the first key of a tile, and the key each piece belongs to
  int off[PIECES], key_of[PIECES];
  {
    int piece = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int c = 0; c < D / 32; ++c, ++piece) {
        key_of[piece] = half * 8 + g;
        off[piece] = key_of[piece] * D + c * 32 + t * 8;
      }
#pragma unroll
    for (int sl = 0; sl < 4; ++sl)
#pragma unroll
      for (int c = 0; c < D / 64; ++c, ++piece) {
        key_of[piece] = 2 * t + (sl & 1) + (sl >> 1) * 8;
        off[piece] = v_off + key_of[piece] * D + g * (D / 8) + c * 8;
      }
  }

  // this warp's tiles: first keys k_begin + (warp + WARPS*i) * 16
  const int first = k_begin + warp * 16;
  const int n_tiles = first < k_end ? (k_end - first + WARPS * 16 - 1) / (WARPS * 16) : 0;
  const uint32_t ring0 = (uint32_t)__cvta_generic_to_shared(smem_raw) + (uint32_t)warp * STAGES * Shape::STAGE_BYTES + lane * 16;
  // Page ids are fetched 32 tiles at a time, one per lane, and handed out by shuffle: a load in the issue path
  // would stall the warp for a full memory latency on every tile.
  auto fetch_pages = [&](int first_tile) {
    const int i = first_tile + lane;
    return i < n_tiles ? pages[(first + i * WARPS * 16) >> page_shift] : 0;
  };
  int page_ids = fetch_pages(0);
  int issue_key = first, issued = 0, issue_stage = 0;
  auto issue = [&]() {
    if ((issued & 31) == 0 && issued > 0) page_ids = fetch_pages(issued);
    const int page = __shfl_sync(0xffffffffu, page_ids, issued & 31);
    const __nv_bfloat16* base = kv_head + (size_t)page * page_elems + (size_t)(issue_key & (page_size - 1)) * D;
    const uint32_t slot = ring0 + issue_stage * Shape::STAGE_BYTES;
    const int valid = kvl - issue_key;
    if (valid >= 16) {
#pragma unroll
      for (int i = 0; i < PIECES; ++i) cp16_cg(slot + i * 512, base + off[i]);
    } else {  // the last tile: keys that do not exist yet are read as zeros
#pragma unroll
      for (int i = 0; i < PIECES; ++i) {
        const bool ok = key_of[i] < valid;
        cp16_cg_zfill(slot + i * 512, ok ? base + off[i] : base, ok ? 16 : 0);
      }
    }
    issue_key += WARPS * 16;
    ++issued;
    if (++issue_stage == STAGES) issue_stage = 0;
  };
  // Keys and values of earlier steps do not change during this step, so their tiles may be requested before the
  // preceding kernel (which writes this step's key and value at position p, and the queries) has finished.
  int primed = 0;
  for (; primed < STAGES - 1 && issued < n_tiles && issue_key + 15 < p; ++primed) {
    issue();
    cp_async_commit();
  }
  pdl_wait();  // from here on: the queries, and the tile that holds position p
  for (; primed < STAGES - 1; ++primed) {
    if (issued < n_tiles) issue();
    cp_async_commit();
  }

  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* r0 = g < G ? q + ((size_t)t0 * hq + h * G + g) * D : nullptr;
    const __nv_bfloat16* r1 = g + 8 < G ? q + ((size_t)t0 * hq + h * G + g + 8) * D : nullptr;
    load_q<D>(qa, r0, r1, t);
  }
  RowState<D> st;
  st.init();
  const int pos[2] = {p, p};
  const int lo[2] = {lo_key, lo_key};

  int read_stage = 0, key0 = first;
  for (int i = 0; i < n_tiles; ++i, key0 += WARPS * 16) {
    if (issued < n_tiles) issue();
    cp_async_commit();
    cp_async_wait<STAGES - 1>();  // everything but the newest STAGES-1 groups has landed: tile i is there
    KVTile<D> cur;
    {
      const uint32_t slot = ring0 + read_stage * Shape::STAGE_BYTES;
      uint4* kp = &cur.k[0][0];
      uint4* vp = &cur.v[0][0];
#pragma unroll
      for (int j = 0; j < KP; ++j) kp[j] = lds16(slot + j * 512);
#pragma unroll
      for (int j = 0; j < PIECES - KP; ++j) vp[j] = lds16(slot + (KP + j) * 512);
      if (++read_stage == STAGES) read_stage = 0;
    }
    float s[2][4];
    scores<D>(s, qa, cur);
    if (key0 + 15 > p || key0 < lo_key) mask_tile(s, key0, t, pos, lo);
    fold<D>(st, s, cur, sl2, G > 8);
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the same memory now carries the merge

  float(*sh_m)[16] = reinterpret_cast<float(*)[16]>(smem_raw);
  float(*sh_l)[16] = reinterpret_cast<float(*)[16]>(smem_raw + WARPS * 16 * 4);
  float(*sh_o)[16][D + 4] = reinterpret_cast<float(*)[16][D + 4]>(smem_raw + 2 * WARPS * 16 * 4);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = st.l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = g + 8 * r;
    if (row < G) {
      if (t == 0) { sh_m[warp][row] = st.m[r]; sh_l[warp][row] = l; }
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        sh_o[warp][row][(2 * t) * (D / 8) + j] = st.o[j][2 * r];
        sh_o[warp][row][(2 * t + 1) * (D / 8) + j] = st.o[j][2 * r + 1];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
    const int row = idx / D, d = idx - row * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sh_m[w][row]);
    const float m_safe = m == -INFINITY ? 0.f : m;
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float a = fast_exp2(sh_m[w][row] - m_safe);
      l += a * sh_l[w][row];
      o += a * sh_o[w][row][d];
    }
    const int head = h * G + row;
    if (max_splits == 1) {
      out[((size_t)t0 * hq + head) * D + d] = __float2bfloat16_rn(o / l);
    } else {
      const size_t slot = ((size_t)item * hq + head) * max_splits + split;
      part_o[slot * D + d] = o;
      if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
    }
  }
}

// grid (hq, items), MW warps: combines the key ranges of one (item, head).  Every warp finds the maximum over all
// ranges for itself (a few 8-byte loads a lane); the ranges are then shared out in contiguous runs, a warp adds up its
// run's weighted partial outputs (lanes over the head dims, eight ranges' loads in flight at a time), and the warps'
// sums are joined in warp order through shared memory.  One warp (MW = 1) is right for a handful of ranges; dozens of
// them (one request with tens of thousands of keys) are nothing but load latency in a single warp.
template <int D, int MW>
__global__ void __launch_bounds__(32 * MW)
attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                       const int32_t* __restrict__ item_start, const int32_t* __restrict__ kv_len,
                       __nv_bfloat16* __restrict__ out, int hq, int window, int chunk, int max_splits, int all_single) {
  __shared__ float sum_o[MW][D];
  __shared__ float sum_l[MW];
  pdl_trigger();
  const int item = blockIdx.y, head = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int t0 = item;
  bool mine = true;
  if (!all_single) {
    t0 = item_start[item];
    mine = item_start[item + 1] - t0 == 1;
  }
  const int kvl = kv_len[item];
  pdl_wait();
  if (!mine) return;
  const int p = kvl - 1;
  const int lo_key = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  // never more ranges than the launch provided scratch for (the host sizes them from the longest span it expects)
  const int splits = min((kvl - (lo_key & ~15) + chunk - 1) / chunk, max_splits);
  const size_t base = ((size_t)item * hq + head) * max_splits;
  const int per = (splits + MW - 1) / MW;
  const int s_lo = min(warp * per, splits), s_hi = min(s_lo + per, splits);
  // This warp's first eight partial outputs are asked for together with the maxima: where they lie does not depend
  // on the weights, and this kernel is nothing but the latency of its loads.
  float first[D / 32][8];
#pragma unroll
  for (int i = 0; i < D / 32; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) first[i][j] = s_lo + j < s_hi ? part_o[(base + s_lo + j) * D + lane + 32 * i] : 0.f;
  float m = -INFINITY;
  for (int s = lane; s < splits; s += 32) m = fmaxf(m, part_ml[(base + s) * 2]);
  m = warp_max(m);
  const float m_safe = m == -INFINITY ? 0.f : m;
  // The run in blocks of 32 ranges: a lane works out one range's weight, then the partial outputs are added up eight
  // ranges at a time, the next eight's loads on their way while these are used.
  float o[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) o[i] = 0.f;
  float l = 0.f;
  for (int blk = s_lo; blk < s_hi; blk += 32) {
    float a = 0.f;
    if (blk + lane < s_hi) {
      a = fast_exp2(part_ml[(base + blk + lane) * 2] - m_safe);
      l += a * part_ml[(base + blk + lane) * 2 + 1];
    }
    const int blk_hi = min(blk + 32, s_hi);
    for (int s0 = blk; s0 < blk_hi; s0 += 8) {
      float next[D / 32][8];
      const int n0 = s0 + 8;
      if (n0 < s_hi) {
#pragma unroll
        for (int i = 0; i < D / 32; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) next[i][j] = n0 + j < s_hi ? part_o[(base + n0 + j) * D + lane + 32 * i] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float w = __shfl_sync(0xffffffffu, a, (s0 - blk + j) & 31);
#pragma unroll
        for (int i = 0; i < D / 32; ++i) o[i] = fmaf(s0 + j < blk_hi ? w : 0.f, first[i][j], o[i]);
      }
      if (n0 < s_hi) {
#pragma unroll
        for (int i = 0; i < D / 32; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) first[i][j] = next[i][j];
      }
    }
  }
  l = warp_sum(l);
  if (MW > 1) {
#pragma unroll
    for (int i = 0; i < D / 32; ++i) sum_o[warp][lane + 32 * i] = o[i];
    if (lane == 0) sum_l[warp] = l;
    __syncthreads();
    if (warp != 0) return;
    l = 0.f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) o[i] = 0.f;
#pragma unroll
    for (int w = 0; w < MW; ++w) {
      l += sum_l[w];
#pragma unroll
      for (int i = 0; i < D / 32; ++i) o[i] += sum_o[w][lane + 32 * i];
    }
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < D / 32; ++i)
    out[((size_t)t0 * hq + head) * D + lane + 32 * i] = __float2bfloat16_rn(o[i] * inv);
}

// The merge with one warp up to eight ranges (one round of loads), four warps beyond.
template <int D>
void launch_merge(const float* part_o, const float* part_ml, const int32_t* item_start, const int32_t* kv_len, __nv_bfloat16* out,
                  int num_items, int hq, int window, int chunk, int max_splits, int all_single, cudaStream_t stream) {
  if (max_splits <= 8)
    psb_launch(attention_merge_kernel<D, 1>, dim3(hq, num_items), dim3(32), 0, stream, part_o, part_ml, item_start, kv_len, out, hq,
               window, chunk, max_splits, all_single);
  else
    psb_launch(attention_merge_kernel<D, 4>, dim3(hq, num_items), dim3(128), 0, stream, part_o, part_ml, item_start, kv_len, out, hq,
               window, chunk, max_splits, all_single);
}

int check_common(const char* who, int hq, int hkv, int D, int page_size, int table_width, int window) {
  if (hq < 1 || hkv < 1 || hq % hkv) PSB_REFUSE("%s: %d query heads cannot share %d key/value heads", who, hq, hkv);
  if (D != 64 && D != 128) PSB_REFUSE("%s: head size %d is not built for the tensor-core path (64 or 128)", who, D);
  if (page_size < 16 || page_size % 16) PSB_REFUSE("%s: page size %d is not a multiple of 16", who, page_size);
  if (table_width < 1 || window < 0) PSB_REFUSE("%s: bad table width %d or window %d", who, table_width, window);
  return 0;
}

}  // namespace

PSB_API int psb_attention_prefill_bf16(const void* q, const void* kv, const void* table, int table_width,
                                       const void* item_start, const void* kv_len, void* out, int num_items, int num_tiles,
                                       int hq, int hkv, int D, int page_size, int window, float scale, int skip_single,
                                       cudaStream_t stream) {
  if (int rc = check_common("attention_prefill", hq, hkv, D, page_size, table_width, window)) return rc;
  if (num_items < 0 || num_tiles < 0) PSB_REFUSE("attention_prefill: negative sizes");
  if (num_items == 0 || num_tiles == 0) return 0;
  if (hkv > 65535) PSB_REFUSE("attention_prefill: too many key/value heads");
  if (page_size & (page_size - 1)) PSB_REFUSE("attention_prefill: page size %d is not a power of two", page_size);
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  dim3 grid(num_tiles, hkv);
#define PSB_PREFILL(DD, MT)                                                                                          \
  do {                                                                                                               \
    static PsbPerDevice configured;  /* more than 48 KB of dynamic shared memory has to be asked for once */           \
    if (!configured.get()) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DD, MT>,                                         \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, PrefillShape<DD>::SMEM_BYTES); \
      if (e != cudaSuccess) PSB_REFUSE("attention_prefill: cannot reserve shared memory: %s", cudaGetErrorString(e)); \
      configured.set();                                                                                              \
    }                                                                                                                \
    psb_launch(attention_prefill_kernel<DD, MT>, grid, dim3(WARPS * 32), (size_t)PrefillShape<DD>::SMEM_BYTES, stream, \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv, (const int32_t*)table, table_width,                       \
        (const int32_t*)item_start, (const int32_t*)kv_len, (__nv_bfloat16*)out, num_items, hq, hkv, page_shift,     \
        window, scale, skip_single);                                                                                 \
  } while (0)
  if (D == 64) PSB_PREFILL(64, 2); else PSB_PREFILL(128, 1);
#undef PSB_PREFILL
  PSB_LAUNCH_CHECK("attention_prefill");
  return 0;
}

// rows of (token, head-in-group) pairs one CTA of the prefill kernel owns, by head size
PSB_API int psb_attention_prefill_rows_per_cta(int D) { return D == 64 ? WARPS * 16 * 2 : WARPS * 16; }

PSB_API int psb_attention_decode_bf16(const void* q, const void* kv, const void* table, int table_width,
                                      const void* item_start, const void* kv_len, void* out, void* part_o, void* part_ml,
                                      int num_items, int hq, int hkv, int D, int page_size, int window, float scale, int chunk,
                                      int max_splits, int all_single, cudaStream_t stream) {
  if (int rc = check_common("attention_decode", hq, hkv, D, page_size, table_width, window)) return rc;
  if (hq / hkv > 16) PSB_REFUSE("attention_decode: groups of more than 16 query heads are not built");
  // a range is walked in tiles of 16 keys that its warps take in turn: it may end after any whole tile
  if (chunk < WARPS * 16 || chunk % 16) PSB_REFUSE("attention_decode: key range %d is shorter than %d or no multiple of 16", chunk, WARPS * 16);
  if (max_splits < 1 || max_splits > 1024 || (max_splits > 1 && (!part_o || !part_ml)))
    PSB_REFUSE("attention_decode: %d key ranges (at most 1024), or their scratch is missing", max_splits);
  if (page_size & (page_size - 1)) PSB_REFUSE("attention_decode: page size %d is not a power of two", page_size);
  if (num_items <= 0) return 0;
  if (num_items > 65535 || hkv > 65535) PSB_REFUSE("attention_decode: batch too large");
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  dim3 grid(max_splits, hkv, num_items);
#define PSB_DECODE(DD)                                                                                               \
  do {                                                                                                               \
    static PsbPerDevice configured;  /* more than 48 KB of dynamic shared memory has to be asked for once */           \
    if (!configured.get()) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           DecodeShape<DD>::SMEM_BYTES);                                             \
      if (e != cudaSuccess) PSB_REFUSE("attention_decode: cannot reserve shared memory: %s", cudaGetErrorString(e)); \
      configured.set();                                                                                              \
    }                                                                                                                \
    psb_launch(attention_decode_kernel<DD>, grid, dim3(WARPS * 32), (size_t)DecodeShape<DD>::SMEM_BYTES, stream, \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv, (const int32_t*)table, table_width, (const int32_t*)item_start, \
        (const int32_t*)kv_len, (__nv_bfloat16*)out, (float*)part_o, (float*)part_ml, hq, hkv, page_shift, window, scale, \
        chunk, max_splits, all_single);                                                                              \
    if (max_splits > 1)                                                                                              \
      launch_merge<DD>((const float*)part_o, (const float*)part_ml, (const int32_t*)item_start, (const int32_t*)kv_len, \
                       (__nv_bfloat16*)out, num_items, hq, window, chunk, max_splits, all_single, stream);             \
  } while (0)
  if (D == 64) PSB_DECODE(64); else PSB_DECODE(128);
#undef PSB_DECODE
  PSB_LAUNCH_CHECK("attention_decode");
  return 0;
}

// The merge alone, for a decode kernel that lives in another file (attention_decode_tma.cu) and leaves its partial
// results in the same layout.
PSB_API int psb_attention_decode_merge_bf16(const void* part_o, const void* part_ml, const void* item_start, const void* kv_len,
                                            void* out, int num_items, int hq, int D, int window, int chunk, int max_splits,
                                            int all_single, cudaStream_t stream) {
  if (D != 64 && D != 128) PSB_REFUSE("attention_merge: head size %d is not built", D);
  if (max_splits < 2 || max_splits > 1024 || !part_o || !part_ml) PSB_REFUSE("attention_merge: %d key ranges, or their scratch is missing", max_splits);
  if (num_items <= 0) return 0;
  if (num_items > 65535) PSB_REFUSE("attention_merge: batch too large");
  if (D == 64)
    launch_merge<64>((const float*)part_o, (const float*)part_ml, (const int32_t*)item_start, (const int32_t*)kv_len,
                     (__nv_bfloat16*)out, num_items, hq, window, chunk, max_splits, all_single, stream);
  else
    launch_merge<128>((const float*)part_o, (const float*)part_ml, (const int32_t*)item_start, (const int32_t*)kv_len,
                      (__nv_bfloat16*)out, num_items, hq, window, chunk, max_splits, all_single, stream);
  PSB_LAUNCH_CHECK("attention_merge");
  return 0;
}

// ---- the same, with the scratch inside the library (see no_alloc.h: for callers that cannot allocate) -----------
#include "no_alloc.h"

namespace {
// Partial results of the key ranges.  File scope, so the memory exists from the moment the library is loaded on a
// device until the process ends.  In host code this name is only a handle for cudaGetSymbolAddress, never a pointer.
static __device__ __align__(256) float g_decode_scratch[PSB_STATIC_SCRATCH_FLOATS];
constexpr int MAX_DEVICES = 64;
float* g_decode_scratch_addr[MAX_DEVICES] = {};  // device address of the array, per device, looked up on first use
}  // namespace

PSB_API int psb_attention_decode_bf16_static(const void* q, const void* kv, const void* table, int table_width,
                                             const void* item_start, const void* kv_len, void* out, int num_items, int hq,
                                             int hkv, int D, int page_size, int window, float scale, int chunk,
                                             int max_splits, int all_single, cudaStream_t stream) {
  if (num_items < 0 || hq < 1 || D < 1 || max_splits < 1) PSB_REFUSE("attention_decode_static: bad sizes");
  const unsigned long long ranges = (unsigned long long)num_items * hq * max_splits;
  const unsigned long long need = ranges * (unsigned long long)(D + 2);
  if (need > PSB_STATIC_SCRATCH_FLOATS)
    PSB_REFUSE("attention_decode_static: %d items x %d heads x %d key ranges x (%d + 2) floats = %llu exceed the built-in "
               "scratch of %u floats; use fewer key ranges or the entry point that takes a scratch buffer",
               num_items, hq, max_splits, D, need, (unsigned)PSB_STATIC_SCRATCH_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) PSB_REFUSE("attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (device < 0 || device >= MAX_DEVICES) PSB_REFUSE("attention_decode_static: device index %d is out of range", device);
  if (g_decode_scratch_addr[device] == nullptr) {
    // once per device, with that device current; not inside a stream capture
    float* addr = nullptr;
    e = cudaGetSymbolAddress((void**)&addr, g_decode_scratch);
    if (e != cudaSuccess || addr == nullptr)
      PSB_REFUSE("attention_decode_static: cannot find the built-in scratch on device %d: %s", device, cudaGetErrorString(e));
    g_decode_scratch_addr[device] = addr;
  }
  float* part_o = g_decode_scratch_addr[device];
  float* part_ml = part_o + ranges * (unsigned long long)D;
  return psb_attention_decode_bf16(q, kv, table, table_width, item_start, kv_len, out, part_o, part_ml, num_items, hq, hkv, D,
                                   page_size, window, scale, chunk, max_splits, all_single, stream);
}
