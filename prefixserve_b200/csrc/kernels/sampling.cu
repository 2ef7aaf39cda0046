// Token choice from float32 logits: one block per row.
//
// temperature == 0: arg max, the lowest index winning ties (the reference's
// only mode, torch.argmax at prefixserve/llama_engine.py:146).
// temperature > 0: sampling from softmax(logits / temperature) by the
// Gumbel-max rule, token = argmax_i(logits[i] / temperature + g_i) with
// g_i = -log(-log(u_i)) and u_i drawn from a counter-based generator keyed by
// (request seed, absolute position of the new token, i).  The draw therefore
// does not depend on what else is in the batch, on how the prompt was cut, or
// on a recomputation after preemption.
#include <cfloat>

#include "common.cuh"

namespace {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  return z ^ (z >> 31);
}

// uniform in (0, 1) with 24 random bits
__device__ __forceinline__ float uniform01(uint64_t seed, uint32_t position, uint32_t index) {
  const uint64_t a = mix64(seed + 0x9e3779b97f4a7c15ULL * ((uint64_t)position + 1));
  const uint64_t r = mix64(a ^ (0xd1b54a32d192ed03ULL * ((uint64_t)index + 1)));
  return ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// Stage 1: block (row, part) scans its slice of the row and leaves its winner in part_v/part_i.
// Stage 2 (parts == 1 and final != nullptr in one launch, or a second launch over the winners): same reduction.
// The row's temperature, seed and position come either from three arrays with one entry per row, or (records given)
// from the record of the row's request slot: int32 words {position, temperature bits, seed low, seed high, ...}.
__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                              const int64_t* __restrict__ seed, const int32_t* __restrict__ position,
                              const int32_t* __restrict__ records, const int32_t* __restrict__ row_slot, int record_words,
                              int32_t* __restrict__ out, float* __restrict__ part_v, int32_t* __restrict__ part_i, int V,
                              int parts) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, part = blockIdx.y;
  const float* x = logits + (size_t)row * V;
  const int32_t* rec = records ? records + (size_t)row_slot[row] * record_words : nullptr;
  const float tau = rec ? __int_as_float(rec[1]) : (temperature ? temperature[row] : 0.f);
  const int per = (V + parts - 1) / parts;
  const int lo = part * per, hi = min(V, lo + per);
  float bv = -FLT_MAX;
  int bi = 0x7fffffff;
  if (tau > 0.f) {
    const uint64_t sd = rec ? ((uint64_t)(uint32_t)rec[2] | ((uint64_t)(uint32_t)rec[3] << 32)) : (uint64_t)seed[row];
    const uint32_t pos = (uint32_t)(rec ? rec[0] : position[row]);
    const float inv_tau = 1.f / tau;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float u = uniform01(sd, pos, (uint32_t)i);
      const float v = x[i] * inv_tau - logf(-logf(u));
      if (v > bv) { bv = v; bi = i; }   // strided scan keeps the lowest index of equal values
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float v = x[i];
      if (v > bv) { bv = v; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarp = blockDim.x >> 5;
    bv = lane < nwarp ? best_v[lane] : -FLT_MAX;
    bi = lane < nwarp ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      if (parts == 1) {
        // a row of NaNs (or of -FLT_MAX) never beats the initial value: answer 0 rather than an invalid id
        out[row] = bi == 0x7fffffff ? 0 : bi;
      } else {
        part_v[row * parts + part] = bv;
        part_i[row * parts + part] = bi;
      }
    }
  }
}

// One warp per row picks the winner among the parts (lowest index among equal values).
__global__ void sample_finish_kernel(const float* __restrict__ part_v, const int32_t* __restrict__ part_i,
                                     int32_t* __restrict__ out, int parts) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  float bv = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int p = lane; p < parts; p += 32) {
    const float v = part_v[row * parts + p];
    const int i = part_i[row * parts + p];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

}  // namespace

// Rows of a large vocabulary are scanned by several blocks each; their winners go through ``scratch``
// (S * parts floats followed by S * parts int32; psb_sample_scratch_bytes tells how much).
PSB_API int psb_sample_parts(int S, int V) {
  if (V < 32768 || S < 1) return 1;
  int parts = 1184 / S;  // a few blocks per SM in total
  parts = parts < 1 ? 1 : (parts > 64 ? 64 : parts);
  return parts;
}

PSB_API long long psb_sample_scratch_bytes(int S, int V) { return (long long)S * psb_sample_parts(S, V) * 8; }

PSB_API int psb_sample(const void* logits, const void* temperature, const void* seed, const void* position, void* out,
                       void* scratch, int S, int V, cudaStream_t stream) {
  if (S < 0 || V < 1) PSB_REFUSE("sample: bad sizes S=%d V=%d", S, V);
  if (temperature && (!seed || !position)) PSB_REFUSE("sample: temperature given without seed and position");
  if (S == 0) return 0;
  const int parts = psb_sample_parts(S, V);
  if (parts > 1 && !scratch) PSB_REFUSE("sample: scratch for %d parts per row missing", parts);
  const int per = (V + parts - 1) / parts;
  const int threads = per >= 16384 ? 1024 : (per >= 1024 ? 256 : 64);
  float* part_v = (float*)scratch;
  int32_t* part_i = (int32_t*)(part_v + (size_t)S * parts);
  psb_launch(sample_kernel, dim3(S, parts), dim3(threads), 0, stream, (const float*)logits, (const float*)temperature, (const int64_t*)seed,
             (const int32_t*)position, (const int32_t*)nullptr, (const int32_t*)nullptr, 0, (int32_t*)out, part_v, part_i, V, parts);
  if (parts > 1) psb_launch(sample_finish_kernel, dim3(S), dim3(32), 0, stream, (const float*)part_v, (const int32_t*)part_i, (int32_t*)out, parts);
  PSB_LAUNCH_CHECK("sample");
  return 0;
}

// The same choice with every row's temperature, seed and position read from the record of its request slot
// (records: int32 [num_slots, record_words] on the device; row_slot: int32 [S]).  Nothing about the requests is
// built on the host for a step.
PSB_API int psb_sample_slots(const void* logits, const void* records, const void* row_slot, int record_words, void* out,
                             void* scratch, int S, int V, cudaStream_t stream) {
  if (S < 0 || V < 1) PSB_REFUSE("sample: bad sizes S=%d V=%d", S, V);
  if (!records || !row_slot || record_words < 4) PSB_REFUSE("sample: slot records of at least 4 words and one slot per row are needed");
  if (S == 0) return 0;
  const int parts = psb_sample_parts(S, V);
  if (parts > 1 && !scratch) PSB_REFUSE("sample: scratch for %d parts per row missing", parts);
  const int per = (V + parts - 1) / parts;
  const int threads = per >= 16384 ? 1024 : (per >= 1024 ? 256 : 64);
  float* part_v = (float*)scratch;
  int32_t* part_i = (int32_t*)(part_v + (size_t)S * parts);
  psb_launch(sample_kernel, dim3(S, parts), dim3(threads), 0, stream, (const float*)logits, (const float*)nullptr,
             (const int64_t*)nullptr, (const int32_t*)nullptr, (const int32_t*)records, (const int32_t*)row_slot, record_words,
             (int32_t*)out, part_v, part_i, V, parts);
  if (parts > 1) psb_launch(sample_finish_kernel, dim3(S), dim3(32), 0, stream, (const float*)part_v, (const int32_t*)part_i, (int32_t*)out, parts);
  PSB_LAUNCH_CHECK("sample");
  return 0;
}
