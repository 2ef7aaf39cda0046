// Split-KV decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in PrefixServe; it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a serving loop that
// promised its host process a fixed device-memory footprint, a plugin called from inside someone
// else's stream capture (allocation is illegal while a stream is being captured), and plain C or
// C++ callers that have no caching allocator to hand scratch buffers out and do not want the
// device-wide synchronisation that cudaMalloc / cudaFree bring into a latency-critical step.
//
// psb_attention_decode_bf16 needs a scratch buffer for the partial results of the key ranges
// (float32 [items, heads, ranges, head_dim] plus two floats per (item, head, range)) and expects
// the caller to provide it.  psb_attention_decode_bf16_static takes the same inputs and outputs
// but keeps that scratch in a fixed array inside the library:
//
//   * Size: PSB_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that loads the library holds
//     this much until the process exits.  A call that would need more, i.e.
//     items * heads * max_splits * (head_dim + 2) > PSB_STATIC_SCRATCH_FLOATS, is refused with
//     status 1 and a message in psb_last_error(); nothing is launched.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current).  Make that first call outside of any stream capture; later calls
//     on the same device only launch kernels.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.
//   * All calls share the one array.  Nothing in it has to start at zero: every range that the
//     merge step reads was written by the same call just before.  But two calls that overlap on
//     the GPU (different streams, or graphs replayed concurrently) overwrite each other's
//     partial results: serialise them.
//
// Arguments and return value are those of psb_attention_decode_bf16 without part_o / part_ml.
#pragma once

#include <cuda_runtime.h>

#define PSB_STATIC_SCRATCH_FLOATS (1u << 20)

extern "C" int psb_attention_decode_bf16_static(const void* q, const void* kv, const void* table, int table_width,
                                                const void* item_start, const void* kv_len, void* out, int num_items, int hq,
                                                int hkv, int D, int page_size, int window, float scale, int chunk,
                                                int max_splits, int all_single, cudaStream_t stream);
