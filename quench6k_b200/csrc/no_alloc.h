// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference (lkarlslund/quench6k); it is an addition of this
// library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a host program that
// has handed all of the GPU's memory to its own arena and wants no second allocator touching the
// device, a control loop with a latency bound (cudaMalloc and cudaFree may synchronise the
// device), and a plug-in that is only given pointers and a stream by its host application.  The
// regular q6k_argmax takes a scratch buffer from its caller, and the Python wrapper gets that
// buffer from torch's allocator; the function below needs neither.
//
// q6k_argmax_noalloc(logits, rows, vocab, out, stream) writes into out[r] the index of the largest
// value of row r of the FP32 matrix logits [rows, vocab] (ties: the lowest index; NaN counts as
// the smallest value), exactly as q6k_argmax does.  Its scratch (the per-slice winners of the
// first pass) lives in a fixed array in the library's device image:
//
//   * limits: rows <= Q6K_NOALLOC_MAX_ROWS (64) and vocab <= Q6K_NOALLOC_MAX_VOCAB (1,048,576);
//     larger requests are refused with an error, never truncated.  The array takes
//     2 * 64 * 128 * 4 bytes = 64 KiB on every GPU that loads the library, until the process ends.
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current) and keeps it; make that first call outside any stream capture.
//     Later calls only launch the two kernels.
//   * the function calls no cudaMalloc, cudaFree or other allocating routine.
//   * all calls on a device share the one array.  Nothing in it has to start at zero (every word
//     that the second pass reads was written by the first pass of the same call), but two calls
//     whose kernels overlap on the GPU (different streams, no ordering between them) race on it:
//     order such calls yourself.
//
// Returns 0, or non-zero after storing a message for q6k_last_error().
#pragma once
#include <cuda_runtime.h>

#define Q6K_NOALLOC_MAX_ROWS 64
#define Q6K_NOALLOC_MAX_VOCAB (1 << 20)

extern "C" int q6k_argmax_noalloc(const float* logits, int rows, int vocab, int* out, cudaStream_t stream);
