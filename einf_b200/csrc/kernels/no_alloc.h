// einf_argmax_no_alloc: the greedy-token kernel for callers that may not allocate.
//
// This entry point has no counterpart in mon3stera/einf; it exists for hosts that embed
// these kernels without PyTorch's allocator.  Two kinds of caller cannot call cudaMalloc:
// a program that handed all device memory to a pool of its own when it started, and a
// latency-critical loop that cannot afford the device-wide synchronisation that cudaMalloc
// and cudaFree bring with them.  For them the scratch of the two-step argmax (32 partial
// (value, index) pairs and one arrival counter per row) lives in a file-scope device array
// inside the sampling library instead of a buffer the caller would have to provide.
//
// Contract
//   * The caller passes logits (float, [rows, vocab], contiguous) and tokens (int, [rows]),
//     both on the device that is current when the call is made, and the stream to launch on.
//   * rows may be at most EINF_ARGMAX_NO_ALLOC_MAX_ROWS; more is refused with
//     EINF_NO_ALLOC_TOO_MANY_ROWS and nothing is launched.
//   * The call makes no cudaMalloc, cudaFree or other allocating call.  The first call on a
//     device looks up the device address of the scratch array (cudaGetSymbolAddress) and keeps
//     it; make that first call before any stream capture begins.
//   * All calls on one device share the one scratch array, and it keeps what the last call
//     left in it.  The counters are cleared on the stream at the start of every call.  Two calls
//     that overlap on the GPU (different streams, no ordering between them) race on it: order
//     them yourself.
//   * Every GPU that loads the library holds the array (about 66 KB) until the process exits.
//   * The result equals einf_argmax: tokens[r] is the first index of the largest logit of row r.
//
// Return value: 0, a negative EINF_NO_ALLOC_* code, or a positive cudaError_t.
// einf_argmax_no_alloc_strerror turns any of them into text.
#pragma once

#include <cuda_runtime.h>

#define EINF_ARGMAX_NO_ALLOC_MAX_ROWS 256
#define EINF_NO_ALLOC_TOO_MANY_ROWS (-1)
#define EINF_NO_ALLOC_BAD_ARGUMENT (-2)

#ifdef __cplusplus
extern "C" {
#endif

int einf_argmax_no_alloc(const float* logits, int* tokens, int rows, int vocab, cudaStream_t stream);
const char* einf_argmax_no_alloc_strerror(int code);

#ifdef __cplusplus
}
#endif
