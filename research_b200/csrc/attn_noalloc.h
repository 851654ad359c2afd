// Allocation-free entry point for split-KV paged decode attention.
//
// This function has no counterpart in the reference project. It exists for callers that are
// not allowed to allocate device memory at the point where they need attention: code running
// inside a region where the CUDA allocator must not be touched (a latency-critical serving
// loop that has frozen its memory pool, a host process that embeds this library next to
// another runtime which owns all device memory, a plugin called from a context that forbids
// cudaMalloc). The regular entry point, rb_paged_decode, needs a caller-provided workspace
// for the per-split partial results whenever num_splits > 1; this variant keeps that
// workspace inside the library instead.
//
// Contract
//   * The partial results live in one file-scope device array of RB_DECODE_NOALLOC_MAX_FLOATS
//     floats (16 MiB). Every GPU that loads the library holds that array until the process
//     exits. A call with num_splits > 1 needs B * Hq * num_splits * (D + 2) floats; a call that
//     needs more is rejected with RB_NOALLOC_TOO_LARGE and nothing is launched. A call with
//     num_splits == 1 writes its output directly, uses none of the array and has no size limit.
//   * The first call on each device looks up the array's device address (with that device
//     current) and remembers it. Make that first call before starting any stream capture.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine. Inputs
//     and the output are still the caller's buffers.
//   * All calls on a device share the one array and it keeps whatever the previous call left
//     in it. The kernels overwrite every element they later read, so nothing needs clearing,
//     but two calls that overlap on the GPU (different streams, or graphs replayed
//     concurrently) would race on it: serialise them.
//   * Results are identical to rb_paged_decode with the same num_splits.
#pragma once
#include <cuda_runtime.h>

#define RB_DECODE_NOALLOC_MAX_FLOATS (4 * 1024 * 1024)
#define RB_NOALLOC_TOO_LARGE (-40)
#define RB_NOALLOC_SYMBOL_LOOKUP_FAILED (-41)

#ifdef __cplusplus
extern "C" {
#endif

// q [B,Hq,D] bf16; k_cache / v_cache [num_blocks,Hkv,16,D] bf16; block_tables [B,max_blocks] int32;
// seq_lens [B] int32; out [B,Hq,D] bf16; status: device int (0 = ok). Returns 0 on success.
int rb_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                            const int* seq_lens, void* out, int B, int Hq, int Hkv, int D, int max_blocks,
                            int num_blocks, int block_size, int num_splits, float scale, int* status,
                            cudaStream_t stream);

// Floats of the internal array a call with these sizes would use (for callers that want to check first).
long long rb_paged_decode_noalloc_required_floats(int B, int Hq, int D, int num_splits);

#ifdef __cplusplus
}
#endif
