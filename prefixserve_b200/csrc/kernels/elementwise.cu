// Row-wise kernels around the matrix products: embedding gather, residual add
// fused with RMSNorm, SiLU(gate)*up.  All arithmetic is float32; only loads
// and stores use the storage type.
//
// Formulas (PrefixServe prefixserve/model/llama.py): embedding :109, RMSNorm
// :63-69 (mean of squares, rsqrt(mean+eps), then times the gain), residual
// sums :117,:121, SiLU-gated product :121.
#include "common.cuh"

namespace {

template <typename TT>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const TT* __restrict__ table,
                                 float* __restrict__ out, int H, int V) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  // ids are validated on the host; clamp so that a bad one can never read outside the table
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const TT* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = to_float<TT>(row[j]);
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  // every thread adds the partials in the same order: the result does not depend on the batch
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += scratch[w];
  __syncthreads();
  return total;
}

// x[i] = gain * ((h[r] + delta[r]) * rsqrt(mean((h[r]+delta[r])^2) + eps));  r = rows ? rows[i] : i.
// With update_h the sum is stored back into h[r] (float32 residual stream).
template <typename TD, typename TX>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ gain,
                                   const int32_t* __restrict__ rows, TX* __restrict__ x, int H, float eps, int update_h) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (size_t)r * H;
  const TD* dr = delta ? delta + (size_t)r * H : nullptr;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = hr[j];
    if (dr) v += to_float<TD>(dr[j]);
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)H + eps);
  TX* xr = x + (size_t)i * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = hr[j];
    if (dr) v += to_float<TD>(dr[j]);
    if (update_h && dr) hr[j] = v;
    xr[j] = from_float<TX>(gain[j] * (v * inv));
  }
}

template <typename T, int ACT>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / (size_t)I;
  const int j = (int)(idx - t * (size_t)I);
  const float g = to_float<T>(gu[t * 2 * (size_t)I + j]);
  const float u = to_float<T>(gu[t * 2 * (size_t)I + I + j]);
  out[idx] = from_float<T>(gate_act(g, ACT) * u);
}

// Eight elements per thread (16-byte loads and stores).  Needs I % 8 == 0 and bfloat16.
template <int ACT>
__global__ void silu_mul_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I, size_t vecs) {
  pdl_trigger();
  pdl_wait();
  const int per_row = I >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += (size_t)gridDim.x * blockDim.x) {
    const size_t t = v / per_row;
    const int j = (int)(v - t * per_row) << 3;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * (size_t)I + j);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * (size_t)I + I + j);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(gate_act(g.x, ACT) * u.x, gate_act(g.y, ACT) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)I + j) = o4;
  }
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h2[k]);
    o[2 * k] = f.x; o[2 * k + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) h2[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Residual add + RMSNorm with the row held in registers: one pass over memory.  H % 8 == 0, H <= 8 * VPT * blockDim.
template <typename TD, typename TX, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ gain,
                                       const int32_t* __restrict__ rows, TX* __restrict__ x, int H, float eps, int update_h) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (size_t)r * H;
  const TD* dr = delta ? delta + (size_t)r * H : nullptr;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int j = (c * blockDim.x + threadIdx.x) * 8;
    if (j < H) {
      load8<float>(hr + j, v[c]);
      if (dr) {
        float d[8];
        load8<TD>(dr + j, d);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] += d[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[c][k] * v[c][k];
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)H + eps);
  TX* xr = x + (size_t)i * H;
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int j = (c * blockDim.x + threadIdx.x) * 8;
    if (j < H) {
      if (update_h && dr) store8<float>(hr + j, v[c]);
      float gg[8], y[8];
      load8<float>(gain + j, gg);
#pragma unroll
      for (int k = 0; k < 8; ++k) y[k] = gg[k] * (v[c][k] * inv);
      store8<TX>(xr + j, y);
    }
  }
}

}  // namespace

PSB_API int psb_embedding(const void* ids, const void* table, int table_dtype, void* out, int T, int H, int V,
                          cudaStream_t stream) {
  if (T < 0 || H < 1 || V < 1) PSB_REFUSE("embedding: bad sizes T=%d H=%d V=%d", T, H, V);
  if (T == 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  PSB_DISPATCH_DTYPE(table_dtype, TT, {
    psb_launch(embedding_kernel<TT>, dim3(T), dim3(threads), 0, stream, (const int32_t*)ids, (const TT*)table, (float*)out, H, V);
  });
  PSB_LAUNCH_CHECK("embedding");
  return 0;
}

PSB_API int psb_add_rmsnorm(void* h, const void* delta, int delta_dtype, const void* gain, const void* rows, void* x,
                            int x_dtype, int n_rows, int H, float eps, int update_h, cudaStream_t stream) {
  if (n_rows < 0 || H < 1) PSB_REFUSE("add_rmsnorm: bad sizes rows=%d H=%d", n_rows, H);
  if (!(eps > 0.f)) PSB_REFUSE("add_rmsnorm: eps must be positive");
  if (n_rows == 0) return 0;
  if (H % 8 == 0 && H <= 8 * 4 * 256) {  // the row fits in registers: single pass, 16/32-byte accesses
    const int threads = H <= 8 * 128 ? 128 : 256;
    const int vpt = (H / 8 + threads - 1) / threads;  // 1..4
    PSB_DISPATCH_DTYPE(delta_dtype, TD, {
      PSB_DISPATCH_DTYPE(x_dtype, TX, {
        auto launch = [&](auto kernel) {
          psb_launch(kernel, dim3(n_rows), dim3(threads), 0, stream, (float*)h, (const TD*)delta, (const float*)gain,
                     (const int32_t*)rows, (TX*)x, H, eps, update_h);
        };
        if (vpt == 1) launch(add_rmsnorm_vec_kernel<TD, TX, 1>);
        else if (vpt == 2) launch(add_rmsnorm_vec_kernel<TD, TX, 2>);
        else if (vpt == 3) launch(add_rmsnorm_vec_kernel<TD, TX, 3>);
        else launch(add_rmsnorm_vec_kernel<TD, TX, 4>);
      });
    });
    PSB_LAUNCH_CHECK("add_rmsnorm");
    return 0;
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  PSB_DISPATCH_DTYPE(delta_dtype, TD, {
    PSB_DISPATCH_DTYPE(x_dtype, TX, {
      psb_launch(add_rmsnorm_kernel<TD, TX>, dim3(n_rows), dim3(threads), 0, stream, (float*)h, (const TD*)delta, (const float*)gain,
                                                                 (const int32_t*)rows, (TX*)x, H, eps, update_h);
    });
  });
  PSB_LAUNCH_CHECK("add_rmsnorm");
  return 0;
}

// out[T, I] = f(gate_up[:, :I]) * gate_up[:, I:], f the activation named by its code (PsbAct), a template parameter
// of the kernels.
template <int ACT>
static int launch_act_mul(const void* gate_up, int dtype, void* out, int T, int I, cudaStream_t stream) {
  if (dtype == PSB_BF16 && I % 8 == 0) {
    const size_t vecs = (size_t)T * (I / 8);
    const size_t want = (vecs + 255) / 256;
    const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    psb_launch(silu_mul_vec_kernel<ACT>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I, vecs);
    PSB_LAUNCH_CHECK("act_mul");
    return 0;
  }
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const size_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffull) PSB_REFUSE("act_mul: too many elements");
  PSB_DISPATCH_DTYPE(dtype, T_, {
    psb_launch(silu_mul_kernel<T_, ACT>, dim3((unsigned)blocks), dim3(threads), 0, stream, (const T_*)gate_up, (T_*)out, I, total);
  });
  PSB_LAUNCH_CHECK("act_mul");
  return 0;
}

PSB_API int psb_silu_mul(const void* gate_up, int dtype, void* out, int T, int I, int activation, cudaStream_t stream) {
  if (T < 0 || I < 1) PSB_REFUSE("act_mul: bad sizes T=%d I=%d", T, I);
  if (T == 0) return 0;
  if (activation == PSB_ACT_SILU) return launch_act_mul<PSB_ACT_SILU>(gate_up, dtype, out, T, I, stream);
  if (activation == PSB_ACT_GELU_TANH) return launch_act_mul<PSB_ACT_GELU_TANH>(gate_up, dtype, out, T, I, stream);
  PSB_REFUSE("act_mul: activation code %d is not built", activation);
}

// h[T, H] (float32) += delta[T, H]: the residual sum on its own, for block arrangements in which no norm follows it.
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    h[i] += to_float<TD>(delta[i]);
}

PSB_API int psb_residual_add(void* h, const void* delta, int delta_dtype, long long total, cudaStream_t stream) {
  if (total < 0) PSB_REFUSE("residual_add: negative size");
  if (total == 0) return 0;
  const size_t want = ((size_t)total + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  PSB_DISPATCH_DTYPE(delta_dtype, TD, {
    psb_launch(residual_add_kernel<TD>, dim3(blocks), dim3(256), 0, stream, (float*)h, (const TD*)delta, (size_t)total);
  });
  PSB_LAUNCH_CHECK("residual_add");
  return 0;
}
