// Causal grouped-query attention over the paged cache, written for any head
// size, page size and head grouping, in float32 or bfloat16 storage with all
// arithmetic in float32.  One warp owns one (token, query head): it walks the
// visible keys in runs of 32 aligned to absolute positions, keeps a running
// maximum and sum (online softmax) and accumulates the output in registers.
// Because the runs are aligned to absolute key positions, the order of every
// sum depends only on the token's own position, not on how the prompt was cut
// or what else is in the batch.
//
// It serves the 32-bit path, prefill and decode, and any shape the faster
// kernels refuse.  Math: scores = q.k / sqrt(D) (scale passed in), key j is
// visible to the query at absolute position p when j <= p (and j > p - window
// if a window is set), softmax in float32, output = probs . v; query head h
// uses key/value head h / (hq / hkv)
// (prefixserve/model/attention.py:68-121; scale :75, mask :116-118).
//
// Cache layout of one entry: [num_pages, 2, hkv, page_size, D].
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T, typename TKV>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, const TKV* __restrict__ kv, const int32_t* __restrict__ table,
                         int table_width, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                         T* __restrict__ out, int T_tokens, int hq, int hkv, int D, int page_size, int window, float scale) {
  __shared__ float qs[WARPS][MAX_D];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * WARPS + warp;
  if (unit >= (long long)T_tokens * hq) return;
  const int t = (int)(unit / hq), h = (int)(unit - (long long)t * hq);
  const int g = h / (hq / hkv);
  const int p = positions[t];
  const int item = token_item[t];
  const int32_t* pages = table + (size_t)item * table_width;
  const T* qrow = q + ((size_t)t * hq + h) * D;
  for (int d = lane; d < D; d += 32) qs[warp][d] = to_float<T>(qrow[d]);
  __syncwarp();

  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const size_t head_stride = (size_t)page_size * D;          // one head inside a page
  const size_t page_elems = (size_t)2 * hkv * head_stride;
  const size_t v_off = (size_t)hkv * head_stride;

  float m = -FLT_MAX, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int base = lo & ~31; base <= p; base += 32) {
    const int key = base + lane;
    const bool live = key >= lo && key <= p;
    long long off = -1;  // element offset of this lane's key row
    float s = -FLT_MAX;
    if (live) {
      const int page = pages[key / page_size];
      off = (long long)((size_t)page * page_elems + (size_t)g * head_stride + (size_t)(key % page_size) * D);
      const TKV* krow = kv + off;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(qs[warp][d], to_float<TKV>(krow[d]), dot);
      s = dot * scale;
    }
    const float run_max = warp_max(s);
    const float m_new = fmaxf(m, run_max);
    const float alpha = expf(m - m_new);   // first run: exp(-huge) = 0
    const float pr = live ? expf(s - m_new) : 0.f;
    // what multiplies the values is rounded to the storage type first (nothing happens in float32), as the reference
    // rounds its probabilities (prefixserve/model/attention.py:119) and as the tensor-core kernels do; the sum is not
    const float pv = to_float<T>(from_float<T>(pr));
    l = l * alpha + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
    const int n_live = min(32, p - base + 1);
    for (int j = 0; j < n_live; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pv, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;  // before the window
      const TKV* vrow = kv + oj + v_off;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pj, to_float<TKV>(vrow[d]), acc[i]);
      }
    }
  }
  const float inv = 1.f / l;
  T* orow = out + ((size_t)t * hq + h) * D;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

PSB_API int psb_attention_generic(const void* q, int dtype, const void* kv, int kv_dtype, const void* table,
                                  int table_width, const void* positions, const void* token_item, void* out, int T,
                                  int hq, int hkv, int D, int page_size, int window, float scale, cudaStream_t stream) {
  if (T < 0 || hq < 1 || hkv < 1 || hq % hkv) PSB_REFUSE("attention: %d query heads cannot share %d key/value heads", hq, hkv);
  if (D < 1 || D > MAX_D) PSB_REFUSE("attention: head size %d is outside [1, %d]", D, MAX_D);
  if (page_size < 1 || table_width < 1) PSB_REFUSE("attention: bad paging (page_size=%d width=%d)", page_size, table_width);
  if (window < 0) PSB_REFUSE("attention: negative window");
  if (T == 0) return 0;
  const long long units = (long long)T * hq;
  const long long blocks = (units + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) PSB_REFUSE("attention: batch too large");
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_generic_kernel<T_, TKV>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
          (const T_*)q, (const TKV*)kv, (const int32_t*)table, table_width, (const int32_t*)positions,
          (const int32_t*)token_item, (T_*)out, T, hq, hkv, D, page_size, window, scale);
    });
  });
  PSB_LAUNCH_CHECK("attention_generic");
  return 0;
}
