// Per-request state that stays on the device: slot records (position, sampling temperature, sampling seed) and one
// page table row per slot and cache group, all in one int32 array.  The host keeps a mirror and sends only the words
// that changed since the last step, as (index, value) pairs at the end of the step's single input copy; the first
// kernel here puts them in place.  The second turns the resident rows of the slots a step names into the dense
// [items, width] table the attention and append kernels read, and notes each slot's new position in its record, so
// a step that appends no page sends no table at all.
//
// The reference rebuilds and uploads its flattened page lists on every step
// (prefixserve/llama_engine.py:183-209 of PrefixServe).
#include "common.cuh"

namespace {

__global__ void scatter_words_kernel(int32_t* __restrict__ resident, const int32_t* __restrict__ pairs, int n, int limit) {
  pdl_trigger();
  pdl_wait();  // earlier steps may still read the words replaced here
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int at = pairs[2 * i];
  if (at >= 0 && at < limit) resident[at] = pairs[2 * i + 1];  // the host sends each index once: no two threads meet
}

// grid (items, ceil(width / blockDim)): out[i, j] = rows[slots[i], j] for j < width; block column 0 also writes
// records[slots[i]].position = kv_len[i].
__global__ void step_prepare_kernel(int32_t* __restrict__ records, int record_words, const int32_t* __restrict__ kv_len,
                                    const int32_t* __restrict__ slots, const int32_t* __restrict__ rows, int row_width,
                                    int32_t* __restrict__ out, int width, int num_slots) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int slot = slots[i];
  if (slot < 0 || slot >= num_slots) return;  // the host has checked; never index outside on a bad word
  if (records != nullptr && blockIdx.y == 0 && threadIdx.x == 0) records[(size_t)slot * record_words] = kv_len[i];
  if (rows == nullptr) return;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j < width) out[(size_t)i * width + j] = j < row_width ? rows[(size_t)slot * row_width + j] : -1;
}

}  // namespace

PSB_API int psb_scatter_words(void* resident, const void* pairs, int n, int limit, cudaStream_t stream) {
  if (n < 0 || limit < 0) PSB_REFUSE("scatter_words: bad sizes n=%d limit=%d", n, limit);
  if (n == 0) return 0;
  if (!resident || !pairs) PSB_REFUSE("scatter_words: null array");
  psb_launch(scatter_words_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, (int32_t*)resident, (const int32_t*)pairs, n, limit);
  PSB_LAUNCH_CHECK("scatter_words");
  return 0;
}

// records may be null (no position is noted); rows may be null (no table is made: width must be 0).
PSB_API int psb_step_prepare(void* records, int record_words, const void* kv_len, const void* slots, const void* rows,
                             int row_width, void* out, int width, int num_items, int num_slots, cudaStream_t stream) {
  if (num_items < 0 || width < 0 || row_width < 0 || num_slots < 1) PSB_REFUSE("step_prepare: bad sizes");
  if (num_items == 0) return 0;
  if (!slots) PSB_REFUSE("step_prepare: null slot array");
  if (records && (!kv_len || record_words < 1)) PSB_REFUSE("step_prepare: records without kv_len");
  if (rows ? (!out || width < 1) : width != 0) PSB_REFUSE("step_prepare: table and output do not match");
  const int threads = 128;
  const int cols = width > 0 ? (width + threads - 1) / threads : 1;
  psb_launch(step_prepare_kernel, dim3(num_items, cols), dim3(threads), 0, stream, (int32_t*)records, record_words,
             (const int32_t*)kv_len, (const int32_t*)slots, (const int32_t*)rows, row_width, (int32_t*)out, width, num_slots);
  PSB_LAUNCH_CHECK("step_prepare");
  return 0;
}
