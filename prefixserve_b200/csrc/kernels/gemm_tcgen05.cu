// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores, for many rows (prefill).
//
// Persistent, warp-specialised CTAs (one per SM), 192 threads, output tiles of 128 rows by BN columns (256, 192 or
// 128: the widest that still gives every SM a tile; a few hundred rows against a narrow matrix take the narrow ones):
//   warp 0      producer: one lane issues TMA loads (cp.async.bulk.tensor.2d) of a 128x64 tile of A and two
//               (BN/2)x64 tiles of W per stage into 128-byte-swizzled shared memory; completion by mbarrier
//               transaction bytes;
//   warp 1      MMA: an elected lane issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN, K=16; four per stage)
//               with shared-memory matrix descriptors; accumulators are float32 in tensor memory (two buffers 256
//               columns apart, so the epilogue of one tile overlaps the main loop of the next); tcgen05.commit hands
//               stages back to the producer and finished accumulators to the epilogue;
//   warps 2..5  epilogue: tcgen05.ld (32 lanes x 32 columns per instruction) -> registers -> bfloat16 -> global.
// The two W tiles of a stage are rows [n0, n0+BN/2) and [n1, n1+BN/2): for a plain product n1 = n0 + BN/2; for the
// gated feed-forward n0 indexes the gate rows and n1 the matching up rows, and the epilogue writes
// silu(gate) * up, so the [T, 2I] intermediate never exists (prefixserve/model/llama.py:120-121 of PrefixServe;
// F.linear at :113, :117).  For the projection of an attention layer the epilogue does the rotary kernel's job
// (rope.cu) on the sums and stores queries, keys and values where they belong (llama.py:113-116 and
// prefixserve/model/attention.py:105-106 of PrefixServe), so the [T, (hq + 2 hkv) D] matrix never exists either.
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

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;              // two accumulator buffers, 256 float32 columns apart
constexpr int ACC_STRIDE = 256;
constexpr int MAX_STAGES = 6;

// The output tile is 128 rows by BN columns: 256 where that fills the SMs evenly, 192 where it does not (a product of
// 192 tiles of 256 columns takes 148 CTAs two rounds, as 256 tiles of 192 columns two rounds of three quarters the size),
// 240 for plain products that 256 would cut into a few tiles less than there are SMs (2,048 rows by 2,048 columns:
// 128 tiles of 256 leave 20 SMs idle, 144 tiles of 240 do the same work in one round of 15/16 the length).
template <int BN>
struct Tile {
  static_assert(BN == 256 || BN == 240 || BN == 192 || BN == 128, "tile widths built");
  static constexpr int HALF = BN / 2;                  // rows of W per TMA load
  static constexpr int B_BYTES = BN * BK * 2;          // 32 to 16 KB, a multiple of 1,024 (the swizzle's period)
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN >= 240 ? 4 : (BN == 192 ? 5 : 6);
  static_assert(B_BYTES % 1024 == 0 && (HALF * BK * 2) % 1024 == 0, "operand tiles start on the swizzle's period");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
  static_assert(STAGES <= MAX_STAGES && SMEM_BYTES <= 227 * 1024, "beyond a CTA's shared memory");
};

// shared memory: [stages][A | B] (1024-byte aligned), then barriers and the tensor-memory address
struct Barriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};
static_assert(sizeof(Barriers) <= 256, "room kept for the barriers");

// status word: 0 ok; otherwise which wait gave up (1 producer, 2 mma, 3 epilogue, 4 mma/acc)
using namespace tc;

// mode: 0 plain (C[M, N], tile columns [n0, n0+BN/2) and [n0+BN/2, n0+BN)); 1 gated (C[M, I], W = [gate; up], tile
// columns [n0, n0+128) of the gate and the same of the up rows); 2 the projection of an attention layer (columns as in
// 0; the epilogue rotates queries and keys and stores queries, keys and values where RopeArgs says, C is not used).
enum : int { MODE_PLAIN = 0, MODE_GATED = 1, MODE_ROPE = 2, MODE_GATED_GELU = 3 };  // gated: SiLU, or the tanh form of GELU

// One thread's row of a 128 x BN tile of sums, for the projection of an attention layer: 16 columns are 8 pairs of one
// head (first-half elements, then the ones they are rotated with), so the job of the rotary kernel is done on the sums
// while they are in registers.  Each value is first rounded to bfloat16, which is what a separate projection would have
// stored for the rotary kernel to read.  HB > 0: a head is HB blocks of 16 columns and the caller holds the angles of
// the row's position in registers (cs, sn); HB == 0: any head size, angles fetched block by block.
template <int BN, int HB>
__device__ __forceinline__ void rope_store_row(uint32_t taddr, int row, int M, int n0, int N_out, const RopeArgs& rope, int pos,
                                               int page, const float (&cs)[HB > 0 ? HB : 1][8],
                                               const float (&sn)[HB > 0 ? HB : 1][8]) {
  static_assert(HB % 2 == 0 && BN % (16 * (HB > 0 ? HB : 1)) == 0, "tiles must start at a head's first column");
  constexpr int SPAN = HB > 0 ? 16 * HB : 32;  // columns per round: one head, or one load from tensor memory
  const int D = rope.D, q_cols = rope.hq * D, k_cols = rope.hkv * D;
  const int safe = pos < 0 ? 0 : (pos >= rope.max_positions ? rope.max_positions - 1 : pos);
  const bool page_ok = page >= 0 && page < rope.num_pages;  // the host checks tables before launch; a bad id is skipped
  const size_t in_page = (size_t)(pos & ((1 << rope.page_shift) - 1)) * D;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += SPAN) {
#pragma unroll
    for (int cc = 0; cc < SPAN; cc += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c0 + cc, v);
      tmem_ld_wait();
      if (row >= M) continue;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int col = n0 + c0 + cc + 16 * b;
        if (col >= N_out) continue;
        float lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          lo[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[16 * b + j])));
          hi[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[16 * b + 8 + j])));
        }
        __nv_bfloat16* dst = nullptr;
        if (col < q_cols + k_cols) {
          const int within = col < q_cols ? col : col - q_cols;
          const int head = within / D;
          const int blk = HB > 0 ? cc / 16 + b : (within - head * D) >> 4;
          if (rope.cos_t) {
            if constexpr (HB > 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float a, r;
                rotate_pair(lo[j], hi[j], cs[cc / 16 + b][j], sn[cc / 16 + b][j], a, r);
                lo[j] = a; hi[j] = r;
              }
            } else {
              const float4* cp = reinterpret_cast<const float4*>(rope.cos_t + (size_t)safe * (D >> 1) + blk * 8);
              const float4* sp = reinterpret_cast<const float4*>(rope.sin_t + (size_t)safe * (D >> 1) + blk * 8);
              const float4 c0v = __ldg(cp), c1v = __ldg(cp + 1), s0v = __ldg(sp), s1v = __ldg(sp + 1);
              const float cv[8] = {c0v.x, c0v.y, c0v.z, c0v.w, c1v.x, c1v.y, c1v.z, c1v.w};
              const float sv[8] = {s0v.x, s0v.y, s0v.z, s0v.w, s1v.x, s1v.y, s1v.z, s1v.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float a, r;
                rotate_pair(lo[j], hi[j], cv[j], sv[j], a, r);
                lo[j] = a; hi[j] = r;
              }
            }
          }
          if (col < q_cols) dst = rope.q_out + ((size_t)row * rope.hq + head) * D + blk * 16;
          else if (page_ok) dst = rope.kv + ((((size_t)page * 2) * rope.hkv + head) << rope.page_shift) * D + in_page + blk * 16;
        } else {
          const int within = col - q_cols - k_cols;
          const int head = within / D, d0 = within - head * D;
          if (page_ok) dst = rope.kv + ((((size_t)page * 2 + 1) * rope.hkv + head) << rope.page_shift) * D + in_page + d0;
        }
        if (dst) {
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(pack2(lo[0], lo[1]), pack2(lo[2], lo[3]), pack2(lo[4], lo[5]), pack2(lo[6], lo[7]));
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(pack2(hi[0], hi[1]), pack2(hi[2], hi[3]), pack2(hi[4], hi[5]), pack2(hi[6], hi[7]));
        }
      }
    }
  }
}

// BN: see Tile.  HB: see rope_store_row (0 unless mode is MODE_ROPE and the head size is 16 * HB).
template <int BN, int HB>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    __nv_bfloat16* __restrict__ C, int M, int N_out, int K, int ldc, int up_offset, int mode,
                    const RopeArgs rope) {
  using T = Tile<BN>;
  constexpr int BN_HALF = T::HALF, STAGES = T::STAGES, STAGE_BYTES = T::STAGE_BYTES;
  constexpr uint32_t INSTR_DESC = instr_desc(BM, BN, false);  // M=128, N=BN, both operands K-major
  const bool gated = mode == MODE_GATED || mode == MODE_GATED_GELU;
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
        const uint32_t acc = tmem_base + buf * ACC_STRIDE;
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
      const int row = m0 + quarter * 32 + lane;
      int pos = 0, page = -1;
      float cs[HB > 0 ? HB : 1][8], sn[HB > 0 ? HB : 1][8];  // HB > 0: the angles of this row's position, all of a head's pairs
      if (mode == MODE_ROPE && row < M) {  // this row's token: where it stands and which page takes it (inputs of the step)
        pos = rope.positions[row];
        page = rope.table[(size_t)rope.token_item[row] * rope.table_width + (pos >> rope.page_shift)];
        if (HB > 0 && rope.cos_t) {
          const int safe = pos < 0 ? 0 : (pos >= rope.max_positions ? rope.max_positions - 1 : pos);
          const float4* cp = reinterpret_cast<const float4*>(rope.cos_t + (size_t)safe * (rope.D >> 1));
          const float4* sp = reinterpret_cast<const float4*>(rope.sin_t + (size_t)safe * (rope.D >> 1));
#pragma unroll
          for (int b = 0; b < (HB > 0 ? HB : 1); ++b) {
            const float4 c0 = __ldg(cp + 2 * b), c1 = __ldg(cp + 2 * b + 1), s0 = __ldg(sp + 2 * b), s1 = __ldg(sp + 2 * b + 1);
            cs[b][0] = c0.x; cs[b][1] = c0.y; cs[b][2] = c0.z; cs[b][3] = c0.w; cs[b][4] = c1.x; cs[b][5] = c1.y; cs[b][6] = c1.z; cs[b][7] = c1.w;
            sn[b][0] = s0.x; sn[b][1] = s0.y; sn[b][2] = s0.z; sn[b][3] = s0.w; sn[b][4] = s1.x; sn[b][5] = s1.y; sn[b][6] = s1.z; sn[b][7] = s1.w;
          }
        }
      }
      ok = mbar_wait(&bars->acc_full[buf], use & 1, abort, 3);
      if (!ok) break;
      fence_after();
      const uint32_t taddr = tmem_base + buf * ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
      __nv_bfloat16* crow = C + (size_t)row * ldc;
      if (mode == MODE_ROPE) {
        rope_store_row<BN, HB>(taddr, row, M, n0, N_out, rope, pos, page, cs, sn);
      } else if (gated) {
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
                packed[q] = mode == MODE_GATED ? pack2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1)
                                               : pack2(gate_act(g0, PSB_ACT_GELU_TANH) * u0, gate_act(g1, PSB_ACT_GELU_TANH) * u1);
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
          tmem_ld32(taddr + c, v);  // (a tile of 240 columns: the last load reads 16 columns beyond it, which nobody stores)
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (BN % 32 != 0 && c + j >= BN) break;
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

int g_forced_width = 0;  // 0: the launcher chooses the tile width; 128, 192 or 256: tests compare them

// The tile width for a product: the one that gets it done in the fewest, shortest rounds over the SMs.  A round of
// tiles costs its width in tensor-core time plus a fixed share (first loads, the epilogue of the last tile).  The gated
// form needs an even split into gate and up columns and heads of 128 held in registers need whole heads: no 192.
int choose_width(int M, int N_out, bool gated, bool rope, int D, int sms) {
  const int m_blocks = (M + BM - 1) / BM;
  int best = 256;
  long best_cost = -1;
  for (int bn : {256, 240, 192, 128}) {
    if (bn == 192 && (gated || (rope && D == 128))) continue;
    if (bn == 240 && (gated || rope)) continue;  // whole heads and even halves want a power of two or 192
    if (g_forced_width && bn != g_forced_width) continue;
    const int span = gated ? bn / 2 : bn;
    const long tiles = (long)m_blocks * ((N_out + span - 1) / span);
    const long cost = ((tiles + sms - 1) / sms) * (bn + 24);
    // from the widest down: a narrower tile has to pay for itself (240 against 256 is the same kernel but for the width)
    if (best_cost < 0 || (bn == 240 ? cost < best_cost : cost * 10 <= best_cost * 9)) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

int launch(const void* a, const void* w, void* c, int M, int w_rows, int N_out, int K, int up_offset, int mode, int sms,
           cudaStream_t stream, const RopeArgs& rope = RopeArgs{}) {
  const bool gated = mode == MODE_GATED || mode == MODE_GATED_GELU;
  if (M < 1 || N_out < 1 || K < 8 || K % 8) PSB_REFUSE("gemm_tcgen05: needs K a multiple of 8 (M=%d N=%d K=%d)", M, N_out, K);
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)c) & 15) PSB_REFUSE("gemm_tcgen05: operands must be 16-byte aligned");
  const int m_blocks = (M + BM - 1) / BM;
  const int bn = choose_width(M, N_out, gated, mode == MODE_ROPE, rope.D, sms);
  CUtensorMap map_a, map_w;
  if (int rc = make_map(&map_a, a, M, K, BM)) return rc;
  if (int rc = make_map(&map_w, w, w_rows, K, bn / 2)) return rc;
  const int n_span = gated ? bn / 2 : bn;
  const int tiles = m_blocks * ((N_out + n_span - 1) / n_span);
  const int grid = tiles < sms ? tiles : sms;
#define PSB_TCGEN05(BN, HB)                                                                                          \
  do {                                                                                                               \
    static PsbPerDevice configured;  /* more than 48 KB of dynamic shared memory has to be asked for once */           \
    if (!configured.get()) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, HB>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           Tile<BN>::SMEM_BYTES);                                                    \
      if (e != cudaSuccess) PSB_REFUSE("gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", Tile<BN>::SMEM_BYTES, cudaGetErrorString(e)); \
      configured.set();                                                                                              \
    }                                                                                                                \
    psb_launch(gemm_tcgen05_kernel<BN, HB>, dim3(grid), dim3(THREADS), (size_t)Tile<BN>::SMEM_BYTES, stream, map_a,   \
               map_w, (__nv_bfloat16*)c, M, N_out, K, N_out, up_offset, mode, rope);                                 \
  } while (0)
  // the usual head sizes keep a row's angles in registers; every other multiple of 16 fetches them block by block
  if (mode == MODE_ROPE && rope.D == 128) { if (bn == 128) PSB_TCGEN05(128, 8); else PSB_TCGEN05(256, 8); }
  else if (mode == MODE_ROPE && rope.D == 64) { if (bn == 128) PSB_TCGEN05(128, 4); else if (bn == 192) PSB_TCGEN05(192, 4); else PSB_TCGEN05(256, 4); }
  else if (bn == 128) PSB_TCGEN05(128, 0);
  else if (bn == 192) PSB_TCGEN05(192, 0);
  else if (bn == 240) PSB_TCGEN05(240, 0);
  else PSB_TCGEN05(256, 0);
#undef PSB_TCGEN05
  PSB_LAUNCH_CHECK("gemm_tcgen05");
  return 0;
}

}  // namespace

// C[M,N] = A[M,K] W[N,K]^T, all bfloat16 row-major, K % 8 == 0.  sms: CTAs to launch at most (the SM count).
PSB_API int psb_gemm_tcgen05(const void* a, const void* w, void* c, int M, int N, int K, int sms, cudaStream_t stream) {
  return launch(a, w, c, M, N, N, K, 0, MODE_PLAIN, sms, stream);
}

// act[M,I] = f(A Wg^T) * (A Wu^T) for W = [Wg; Wu] of shape [2I, K], f the activation named by its code (PsbAct).
PSB_API int psb_gemm_tcgen05_gated(const void* a, const void* w, void* act, int M, int I, int K, int sms, int activation,
                                   cudaStream_t stream) {
  if (!psb_activation_known(activation)) PSB_REFUSE("gemm_tcgen05_gated: activation code %d is not built", activation);
  return launch(a, w, act, M, 2 * I, I, K, I, activation == PSB_ACT_SILU ? MODE_GATED : MODE_GATED_GELU, sms, stream);
}

// The projection of an attention layer for many tokens: A W^T with W = [queries; keys; values] [(hq + 2 hkv) D, K] in the
// pair-interleaved row order described at RopeArgs (common.cuh); queries rotated into q_out [M, hq, D], keys rotated
// and values as they are stored at the tokens' positions in the pages: what psb_gemm_tcgen05 followed by
// psb_rope_append in its paired form would do, without the [M, (hq + 2 hkv) D] matrix in between.
PSB_API int psb_gemm_tcgen05_rope(const void* a, const void* w, int M, int K, int sms, const void* positions, const void* token_item,
                                  const void* table, int table_width, const void* cos_t, const void* sin_t, void* kv, void* q_out,
                                  int hq, int hkv, int D, int page_size, int num_pages, int max_positions, cudaStream_t stream) {
  if (hq < 1 || hkv < 1 || D < 16 || D % 16) PSB_REFUSE("gemm_tcgen05_rope: needs a head size that is a multiple of 16 (hq=%d hkv=%d D=%d)", hq, hkv, D);
  if (page_size < 1 || (page_size & (page_size - 1)) || num_pages < 1 || table_width < 1) PSB_REFUSE("gemm_tcgen05_rope: page size %d must be a power of two (pages=%d, width=%d)", page_size, num_pages, table_width);
  if (!positions || !token_item || !table || !kv || !q_out) PSB_REFUSE("gemm_tcgen05_rope: cache arguments missing");
  if ((cos_t == nullptr) != (sin_t == nullptr) || (cos_t && max_positions < 1)) PSB_REFUSE("gemm_tcgen05_rope: angle tables incomplete");
  if (((uintptr_t)kv | (uintptr_t)q_out | (uintptr_t)cos_t | (uintptr_t)sin_t) & 31) PSB_REFUSE("gemm_tcgen05_rope: cache, queries and angle tables must be 32-byte aligned");
  RopeArgs rope;
  rope.positions = (const int32_t*)positions; rope.token_item = (const int32_t*)token_item; rope.table = (const int32_t*)table;
  rope.cos_t = (const float*)cos_t; rope.sin_t = (const float*)sin_t; rope.kv = (__nv_bfloat16*)kv; rope.q_out = (__nv_bfloat16*)q_out;
  rope.table_width = table_width; rope.hq = hq; rope.hkv = hkv; rope.D = D; rope.num_pages = num_pages; rope.max_positions = max_positions;
  rope.page_shift = 0;
  while ((1 << rope.page_shift) < page_size) ++rope.page_shift;
  const int N = (hq + 2 * hkv) * D;
  return launch(a, w, q_out, M, N, N, K, 0, MODE_ROPE, sms, stream, rope);
}

// For tests: 128, 192, 240 or 256 makes every later product use that tile width where the shape allows it, 0 gives the
// choice back.
PSB_API int psb_gemm_tcgen05_tile_width(int width) {
  if (width != 0 && width != 128 && width != 192 && width != 240 && width != 256) PSB_REFUSE("gemm_tcgen05: tile widths are 128, 192, 240 and 256, not %d", width);
  g_forced_width = width;
  return 0;
}

// How many output tiles the kernel would cut a product into (kind: 0 plain [M, N], 1 gated [M, N] from 2N rows, 2 the
// projection that rotates, with heads of D).  The host sends products with too few tiles for the SMs elsewhere.
PSB_API int psb_gemm_tcgen05_tiles(int M, int N_out, int kind, int D, int sms) {
  if (M < 1 || N_out < 1 || sms < 1) return 0;
  const int bn = choose_width(M, N_out, kind == 1, kind == 2, D, sms);
  const int span = kind == 1 ? bn / 2 : bn;
  return ((M + BM - 1) / BM) * ((N_out + span - 1) / span);
}

// 0 while no bounded wait has ever run out on the current device; reading it synchronises with the device.
PSB_API int psb_tcgen05_status() {
  return tc::read_status();
}
