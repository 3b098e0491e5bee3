// Declaration of the one entry point of this library that never allocates.
//
// This entry point has no counterpart in the reference (Koas-W/Pico-vLLM), whose kernels are
// Triton functions that let PyTorch allocate their buffers.  It exists for callers that cannot
// allocate device memory at the time they call: code that runs inside a region where the CUDA
// allocator must not be entered (a real-time loop with a fixed memory plan, a host process whose
// memory pool is owned by another component, a callback in which cudaMalloc would synchronise
// the device), and that still wants split-key paged attention, the one kernel family here that
// needs scratch memory beyond its inputs and outputs.
//
// The scratch (per-split partial outputs, maxima and sums) lives in a fixed array inside the
// library: PICO_NOALLOC_SCRATCH_FLOATS float32 values = 8 MiB of device memory, held by every
// GPU that loads the library until the process exits.
#pragma once
#include <cuda_runtime.h>

#define PICO_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Paged causal attention with the key range of every token cut into n_splits parts, exactly as
// pico_paged_attention_generic computes it, but with the partial results kept in the library's
// own fixed scratch array instead of a buffer from the caller.
//
// The caller passes inputs and outputs only (same meaning as pico_paged_attention_generic):
//   q [T rows of q_row_stride], k_pages / v_pages [pages, nkv, page_size, hd], out [T, nh*hd],
//   tok_seg, positions [T] int32, block_table [segments, table_stride] int32, act_dtype 0 =
//   float32, 1 = bfloat16.
//
// Returns 0 when the kernels were launched.  Returns a negative code and writes a message into
// err (if err != NULL and err_len > 0) when the call is refused: -3 for a size the kernels do
// not take, -5 when n_splits > 1 and T * nh * n_splits * (hd + 2) exceeds
// PICO_NOALLOC_SCRATCH_FLOATS (with n_splits == 1 no scratch is used and any T is taken), -6 when
// the address of the scratch array could not be obtained.  A positive value is the cudaError_t
// of a failed launch.
//
// It calls no cudaMalloc, cudaFree or any allocating routine.  The first call on a device looks
// up the device address of the scratch array (cudaGetSymbolAddress, once per device, with that
// device current); make that first call before any stream capture begins.  Two host threads that make
// their first calls on a device at the same moment both look the address up and both store the same value.  All calls share the
// one array, which keeps what the last call left: nothing in it has to start at zero, because
// every call writes each partial result before its second kernel reads it, but two calls whose
// kernels overlap on the GPU (different streams, or different threads) race on it - keep calls
// on one stream, or order them with events.
int pico_paged_attention_noalloc(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                 void* out, const int* tok_seg, const int* positions, const int* block_table,
                                 int table_stride, int T, int nh, int nkv, int hd, int page_size, int window,
                                 float scale, int n_splits, int act_dtype, cudaStream_t stream, char* err,
                                 int err_len);

#ifdef __cplusplus
}
#endif
