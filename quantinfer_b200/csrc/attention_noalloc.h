// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (aiqubits/quantinfer keeps its
// attention scores in a host vector); it exists for this library's own embedders.
//
// Who needs it: code that runs where cudaMalloc is off limits. Examples are a host
// callback or plugin that is invoked while the application's memory pool is frozen, a
// process that has handed all device memory to its own arena and forbids further
// driver allocations, and real-time loops in which an allocation (which may
// synchronise the device) would break a latency bound. Such callers can still pass
// inputs and outputs they own, but they cannot provide or create the scratch space the
// split-key decode kernel needs for its partial results.
//
// qi_attention_decode_tma_static does the same work as qi_attention_decode_tma, with the
// partial results kept in a fixed array inside the library instead of a caller-provided
// workspace:
//
//   * The array is QI_DECODE_STATIC_SCRATCH_BYTES (16 MiB) of device memory, reserved on
//     every GPU that loads the library until the process exits.
//   * A call needs batch * nq * n_splits * (d + 2) floats; a call that needs more than the
//     array holds is refused with an error (nothing is launched).
//   * The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress) with that device current. Make this first call outside any
//     stream capture; later calls only launch kernels.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
//   * All calls on a device share the one array, and it keeps whatever the last call left
//     in it. Nothing in it has to start at zero (every slot that is read has been written
//     by the same call first), but two calls that run on the GPU at the same time, for
//     instance on two streams, overwrite each other's partial results: serialise them.
//
// Arguments and return value are those of qi_attention_decode_tma without ws_o / ws_ml.
// Two preconditions, the same for both entry points:
//
//   * kv_len, q_start and block_table must be complete in device memory when the kernel
//     starts. The kernel reads them, and requests its first key/value tiles, before it
//     waits for the kernel ahead of it in the stream. After a copy or an ordinary kernel
//     launch that is always so. If you produce these arrays with a kernel launched under
//     programmatic dependent launch, that kernel must not release its successors early
//     (no cudaTriggerProgrammaticLaunchCompletion / griddepcontrol.launch_dependents).
//   * n_splits * chunk must cover the longest kv_len: `chunk` is the most keys a range may
//     hold, which the launch's staging is sized for (a request's key tiles are dealt out
//     evenly over the ranges, whatever its length). For a longer request the kernel sets
//     bit 16 of *status, and the caller must treat the output as invalid.
#pragma once

#include <cuda_runtime.h>

#define QI_DECODE_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int qi_attention_decode_tma_static(const void* q, void* out, const void* k_pages, const void* v_pages,
                                   const int* block_table, int max_blocks, int page_size, int num_pages,
                                   const int* kv_len, const int* q_start, int batch, int nq, int nkv, int d,
                                   float scale, int window, int chunk, int n_splits, int* status,
                                   cudaStream_t stream);

// Bytes of the static array (QI_DECODE_STATIC_SCRATCH_BYTES), for callers that size their batches by it.
unsigned long long qi_attention_decode_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
