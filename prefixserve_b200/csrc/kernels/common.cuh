// Shared helpers for the sm_100a kernels: element types, error reporting, and
// the C ABI conventions.  Every entry point returns 0 on success; otherwise it
// has left a message for psb_last_error() and launched nothing (or the launch
// itself failed).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#define PSB_API extern "C" __attribute__((visibility("default")))

enum PsbDtype : int { PSB_F32 = 0, PSB_BF16 = 1 };

void psb_set_error(const char* fmt, ...);

#define PSB_REFUSE(...)          \
  do {                           \
    psb_set_error(__VA_ARGS__);  \
    return 1;                    \
  } while (0)

#define PSB_LAUNCH_CHECK(name)                                                   \
  do {                                                                           \
    cudaError_t e_ = cudaGetLastError();                                         \
    if (e_ != cudaSuccess) {                                                     \
      psb_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));      \
      return 2;                                                                  \
    }                                                                            \
  } while (0)

// ---- programmatic dependent launch ---------------------------------------------------------------------------
// A decode step is a chain of some hundred short kernels, each waiting for the one before.  Launched with the
// programmatic-serialization attribute, a kernel may start while its predecessor is still draining: everything
// before pdl_wait() (index arithmetic, loads of weights and of the step's read-only inputs) overlaps with the
// predecessor; nothing the predecessor writes is read, and nothing is written, before pdl_wait() returns (it
// returns once the whole predecessor grid has finished and its writes are visible).  Every thread executes
// pdl_wait() before it exits, so that "this grid finished" always implies "its predecessor finished".  Without the
// launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

extern int psb_pdl_enabled;  // set through psb_set_pdl()

template <typename Kernel, typename... Args>
inline cudaError_t psb_launch(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (psb_pdl_enabled) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// A function attribute (more than 48 KB of dynamic shared memory) has to be set once on every device that runs the
// kernel.  One of these per call site: get() is false until set() has been called with the same device current.
struct PsbPerDevice {
  static constexpr int kMaxDevices = 64;
  bool done[kMaxDevices] = {};
  static int current() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return -1;
    return d;
  }
  bool get() const {
    const int d = current();
    return d >= 0 && done[d];
  }
  void set() {
    const int d = current();
    if (d >= 0) done[d] = true;
  }
};

// (x1, x2) turned by the angle whose cosine and sine are given.  Written with explicit roundings, so that every
// kernel that rotates (the rotary kernels, the projection that rotates in its epilogue) rounds alike whatever the
// compiler would make of the plain expression around it.
__device__ __forceinline__ void rotate_pair(float x1, float x2, float cs, float sn, float& o1, float& o2) {
  o1 = __fmaf_rn(x1, cs, -__fmul_rn(x2, sn));
  o2 = __fmaf_rn(x2, cs, __fmul_rn(x1, sn));
}

// What a fused projection needs to finish the job of the rotary kernel (rope.cu) in its own epilogue: W is the
// [queries; keys; values] matrix with the rows of every query and key head reordered so that a 16-row tile holds
// 8 elements of the head's first half and the 8 elements they are rotated with (stored index 16b+j <-> natural
// index 8b+j, stored 16b+8+j <-> natural D/2+8b+j).  Queries go to q_out [M, hq, D] and keys to the cache in that
// stored order (a dot product does not care, as long as both sides agree); values in natural order.
struct RopeArgs {
  const int32_t* positions;   // [M] absolute position of each token
  const int32_t* token_item;  // [M] row of the page table
  const int32_t* table;       // [items, table_width] page ids
  const float* cos_t;         // [max_positions, D/2], null: no rotation
  const float* sin_t;
  __nv_bfloat16* kv;          // [num_pages, 2, hkv, page_size, D]
  __nv_bfloat16* q_out;       // [M, hq, D]
  int table_width, hq, hkv, D, page_shift, num_pages, max_positions;
};

// The activation of a gated feed-forward, act(gate) * up, by code: SiLU (prefixserve/model/llama.py:121 of
// PrefixServe, the only one that architecture uses) and the tanh form of GELU.  Every kernel that applies the
// activation takes the code; entry points refuse codes that are not listed here.
enum PsbAct : int { PSB_ACT_SILU = 0, PSB_ACT_GELU_TANH = 1 };
inline bool psb_activation_known(int code) { return code == PSB_ACT_SILU || code == PSB_ACT_GELU_TANH; }
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == PSB_ACT_GELU_TANH) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.f + expf(-g));
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Calls f.template operator()<T>() with T chosen by a PsbDtype code.
#define PSB_DISPATCH_DTYPE(code, T, ...)                       \
  if ((code) == PSB_F32) { using T = float; __VA_ARGS__ }      \
  else if ((code) == PSB_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else PSB_REFUSE("unknown dtype code %d", (int)(code))
