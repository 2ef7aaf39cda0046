// Rotary position encoding fused with the append of new keys and values to
// the paged cache.
//
// Input is the fused projection output [T, (hq + 2*hkv) * D] (queries, then
// keys, then values).  Queries are rotated into q_out [T, hq, D]; keys are
// rotated and, with the values, stored at their absolute position in the
// request's pages, so attention afterwards reads everything from the cache.
// Rotation is the split-half form: with x = (x1, x2) the halves of a head,
//   out = (x1*cos - x2*sin, x2*cos + x1*sin)
// (prefixserve/model/llama.py:72-77), angles indexed by ABSOLUTE position
// (prefixserve/llama_engine.py:190-193); the tables are float32 and hold D/2
// angles per position.  Destination of token at position p: page
// table[item][p / page_size], slot p % page_size
// (prefixserve/model/attention.py:14-16, :95-106).
//
// Cache layout of one entry: [num_pages, 2, hkv, page_size, D].
//
// ``paired`` (head sizes that are multiples of 16): the elements of every query and key head arrive in the order the
// attention part gives its projection rows, 8 elements of the first half followed by the 8 they are rotated with
// (stored index 16b+j <-> natural index 8b+j, stored 16b+8+j <-> natural D/2+8b+j), and queries and keys leave in
// that same order: scores do not depend on the order of a head's elements as long as both sides share it.  Values
// are always in natural order.
//
// The general kernel also takes a rotation over the first ``rotary_dim`` elements of a head only (the rest pass
// through; the tables then hold rotary_dim/2 angles per position) and the interleaved pairing, in which element 2j
// turns with element 2j+1 instead of j with j + rotary_dim/2.  The vector kernel and the fused projections bake in
// the split-half pairing over the whole head; the host sends every other description here.
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void load8v(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8v<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8v<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h2[k]);
    o[2 * k] = f.x; o[2 * k + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8v(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8v<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8v<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) h2[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

template <typename T, typename TKV>
__global__ void rope_append_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                   const int32_t* __restrict__ token_item, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, const int32_t* __restrict__ table, int table_width,
                                   TKV* __restrict__ kv, T* __restrict__ q_out, int hq, int hkv, int D, int page_size,
                                   int num_pages, int max_positions, int rotate, int write_kv, int rotary_dim,
                                   int interleaved) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = rotary_dim >> 1;  // pairs per head; elements from rotary_dim on pass through
  const int pos = positions[t];
  const int heads_in = hq + 2 * hkv;
  const T* row = qkv + (size_t)t * heads_in * D;
  const int safe_pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
  const float* c = cos_t + (size_t)safe_pos * half;
  const float* s = sin_t + (size_t)safe_pos * half;

  TKV* kdst = nullptr;
  TKV* vdst = nullptr;
  if (write_kv) {
    const int item = token_item[t];
    const int page = table[(size_t)item * table_width + pos / page_size];
    // the host checks tables before launch; a bad id is skipped rather than written through
    if (page >= 0 && page < num_pages) {
      const size_t page_elems = (size_t)2 * hkv * page_size * D;
      kdst = kv + (size_t)page * page_elems + (size_t)(pos % page_size) * D;
      vdst = kdst + (size_t)hkv * page_size * D;
    }
  }
  // rotated heads: queries then keys
  const int rot_heads = write_kv ? hq + hkv : hq;
  for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
    const int head = idx / half, j = idx - head * half;
    const int e1 = interleaved ? 2 * j : j, e2 = interleaved ? 2 * j + 1 : j + half;  // the two elements of pair j
    const float x1 = to_float<T>(row[head * D + e1]);
    const float x2 = to_float<T>(row[head * D + e2]);
    float o1 = x1, o2 = x2;
    if (rotate) {
      const float cs = c[j], sn = s[j];
      rotate_pair(x1, x2, cs, sn, o1, o2);
    }
    if (head < hq) {
      T* q = q_out + ((size_t)t * hq + head) * D;
      q[e1] = from_float<T>(o1);
      q[e2] = from_float<T>(o2);
    } else if (kdst) {
      TKV* k = kdst + (size_t)(head - hq) * page_size * D;
      k[e1] = from_float<TKV>(o1);
      k[e2] = from_float<TKV>(o2);
    }
  }
  const int rest = D - rotary_dim;
  for (int idx = threadIdx.x; idx < rot_heads * rest; idx += blockDim.x) {
    const int head = idx / rest, e = rotary_dim + (idx - head * rest);
    const T x = row[head * D + e];
    if (head < hq) q_out[((size_t)t * hq + head) * D + e] = x;
    else if (kdst) kdst[(size_t)(head - hq) * page_size * D + e] = from_float<TKV>(to_float<T>(x));
  }
  if (vdst) {
    const T* vrow = row + (size_t)(hq + hkv) * D;
    for (int idx = threadIdx.x; idx < hkv * D; idx += blockDim.x) {
      const int head = idx / D, j = idx - head * D;
      vdst[(size_t)head * page_size * D + j] = from_float<TKV>(to_float<T>(vrow[idx]));
    }
  }
}

// Eight pairs per thread: 16/32-byte loads of both halves of a head and of the angle tables.  Needs (D/2) % 8 == 0.
template <typename T, typename TKV>
__global__ void rope_append_vec_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                       const int32_t* __restrict__ token_item, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, const int32_t* __restrict__ table, int table_width,
                                       TKV* __restrict__ kv, T* __restrict__ q_out, int hq, int hkv, int D, int page_size,
                                       int num_pages, int max_positions, int rotate, int write_kv, int paired) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = D >> 1;
  const int pos = positions[t];
  const int heads_in = hq + 2 * hkv;
  const T* row = qkv + (size_t)t * heads_in * D;
  const int safe_pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
  const float* c = cos_t + (size_t)safe_pos * half;
  const float* s = sin_t + (size_t)safe_pos * half;
  TKV* kdst = nullptr;
  TKV* vdst = nullptr;
  if (write_kv) {
    const int item = token_item[t];
    const int page = table[(size_t)item * table_width + pos / page_size];
    if (page >= 0 && page < num_pages) {
      const size_t page_elems = (size_t)2 * hkv * page_size * D;
      kdst = kv + (size_t)page * page_elems + (size_t)(pos % page_size) * D;
      vdst = kdst + (size_t)hkv * page_size * D;
    }
  }
  const int rot_heads = write_kv ? hq + hkv : hq;
  const int vec_per_head = half >> 3;
  for (int idx = threadIdx.x; idx < rot_heads * vec_per_head; idx += blockDim.x) {
    const int head = idx / vec_per_head, j = (idx - head * vec_per_head) << 3;  // j: first of 8 angles
    const int at1 = paired ? 2 * j : j, at2 = paired ? 2 * j + 8 : j + half;     // where the two runs of 8 elements lie
    float x1[8], x2[8], o1[8], o2[8];
    load8v<T>(row + head * D + at1, x1);
    load8v<T>(row + head * D + at2, x2);
    if (rotate) {
      float cs[8], sn[8];
      load8v<float>(c + j, cs);
      load8v<float>(s + j, sn);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        rotate_pair(x1[k], x2[k], cs[k], sn[k], o1[k], o2[k]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) { o1[k] = x1[k]; o2[k] = x2[k]; }
    }
    if (head < hq) {
      T* qo = q_out + ((size_t)t * hq + head) * D;
      store8v<T>(qo + at1, o1);
      store8v<T>(qo + at2, o2);
    } else if (kdst) {
      TKV* k = kdst + (size_t)(head - hq) * page_size * D;
      store8v<TKV>(k + at1, o1);
      store8v<TKV>(k + at2, o2);
    }
  }
  if (vdst) {
    const T* vrow = row + (size_t)(hq + hkv) * D;
    for (int idx = threadIdx.x; idx < hkv * (D >> 3); idx += blockDim.x) {
      const int head = idx / (D >> 3), j = (idx - head * (D >> 3)) << 3;
      float v[8];
      load8v<T>(vrow + head * D + j, v);
      store8v<TKV>(vdst + (size_t)head * page_size * D + j, v);
    }
  }
}

}  // namespace

PSB_API int psb_rope_append(const void* qkv, int dtype, const void* positions, const void* token_item, const void* cos_t,
                            const void* sin_t, const void* table, int table_width, void* kv, int kv_dtype, void* q_out,
                            int T, int hq, int hkv, int D, int page_size, int num_pages, int max_positions, int rotate,
                            int write_kv, int paired, int rotary_dim, int interleaved, cudaStream_t stream) {
  if (T < 0 || hq < 1 || hkv < 0 || D < 2 || (D & 1)) PSB_REFUSE("rope_append: bad sizes T=%d hq=%d hkv=%d D=%d", T, hq, hkv, D);
  if (rotary_dim < 2 || rotary_dim > D || (rotary_dim & 1)) PSB_REFUSE("rope_append: rotary_dim %d must be even and in [2, %d]", rotary_dim, D);
  const bool general = rotary_dim != D || interleaved;
  if (general && paired) PSB_REFUSE("rope_append: the paired element order is built for the split-half rotation of a whole head only");
  if (write_kv && (page_size < 1 || num_pages < 1 || table_width < 1 || !kv || !table || hkv < 1))
    PSB_REFUSE("rope_append: cache arguments missing (page_size=%d num_pages=%d width=%d)", page_size, num_pages, table_width);
  if (rotate && (!cos_t || !sin_t || max_positions < 1)) PSB_REFUSE("rope_append: angle tables missing");
  if (paired && D % 16) PSB_REFUSE("rope_append: the paired element order needs a head size that is a multiple of 16, not %d", D);
  if (T == 0) return 0;
  const int work = (hq + hkv) * (D / 2);
  if (D % 16 == 0 && !general) {  // every 8-element run is aligned: vector accesses
    const int threads = work / 8 >= 256 ? 256 : (work / 8 >= 128 ? 128 : 64);
    PSB_DISPATCH_DTYPE(dtype, T_, {
      PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
        psb_launch(rope_append_vec_kernel<T_, TKV>, dim3(T), dim3(threads), 0, stream,
            (const T_*)qkv, (const int32_t*)positions, (const int32_t*)token_item, (const float*)cos_t, (const float*)sin_t,
            (const int32_t*)table, table_width, (TKV*)kv, (T_*)q_out, hq, hkv, D, page_size, num_pages, max_positions, rotate,
            write_kv, paired);
      });
    });
    PSB_LAUNCH_CHECK("rope_append");
    return 0;
  }
  const int threads = work >= 1024 ? 256 : 128;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(rope_append_kernel<T_, TKV>, dim3(T), dim3(threads), 0, stream,
          (const T_*)qkv, (const int32_t*)positions, (const int32_t*)token_item, (const float*)cos_t, (const float*)sin_t,
          (const int32_t*)table, table_width, (TKV*)kv, (T_*)q_out, hq, hkv, D, page_size, num_pages, max_positions, rotate,
          write_kv, rotary_dim, interleaved);
    });
  });
  PSB_LAUNCH_CHECK("rope_append");
  return 0;
}
