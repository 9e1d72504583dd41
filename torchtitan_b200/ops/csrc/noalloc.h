// RMSNorm backward for callers that must not allocate.
//
// This entry point has no counterpart in the reference framework.  It exists for
// hosts that own all device memory themselves -- a serving process that reserved the
// whole GPU for its own pool at start-up, a custom call running inside another
// framework's runtime, a plug-in invoked from a host callback -- where cudaMalloc
// either fails (nothing is left outside their pool) or is forbidden because it
// synchronises the device and breaks their latency budget.
//
// The regular operator (torch.ops.tb200.rmsnorm_bwd) allocates a [groups, dim] fp32
// buffer of per-group weight-gradient partial sums.  Here that buffer is a
// file-scope device array inside the library, so the call allocates nothing: no
// cudaMalloc / cudaFree and no allocating library routine, torch's allocator included.
//
// Limits and rules
//  * dim <= TB200_NOALLOC_MAX_DIM and dim a multiple of the 16-byte vector width
//    (8 for bf16, 4 for fp32); larger rows are rejected with TB200_NOALLOC_E_TOO_LARGE.
//    The array holds TB200_NOALLOC_MAX_GROUPS * TB200_NOALLOC_MAX_DIM floats (5 MiB) and
//    every GPU that loads the library keeps it until the process exits.
//  * The first call on a device looks up the device address of the array
//    (cudaGetSymbolAddress, with that device current) and remembers it.  Make that
//    first call before any stream capture begins.
//  * All calls on one device share the array, which keeps whatever the previous call
//    left in it.  Nothing in it has to start at zero: every group overwrites its whole
//    row of partial sums before the reduction reads it.  Two calls that overlap on the
//    GPU (different streams) race on the array -- serialise them.
//  * Inputs and outputs are the caller's: dy, x, dx are [rows, dim] row-major in the
//    same dtype, weight is [dim] in that dtype, rstd is fp32 [rows] as produced by the
//    forward, dw receives fp32 [dim].  All pointers must be device pointers of the
//    current device; dy, x, weight and dx must be 16-byte aligned.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB200_NOALLOC_MAX_DIM 8192
#define TB200_NOALLOC_MAX_GROUPS 160

enum {
  TB200_NOALLOC_OK = 0,
  TB200_NOALLOC_E_TOO_LARGE = 1,    // dim beyond TB200_NOALLOC_MAX_DIM
  TB200_NOALLOC_E_BAD_SHAPE = 2,    // dim not a multiple of the vector width, rows < 0, bad dtype
  TB200_NOALLOC_E_BAD_POINTER = 3,  // null or misaligned pointer
  TB200_NOALLOC_E_CUDA = 4,         // a CUDA call failed; see tb200_noalloc_last_cuda_error()
};

// dtype: 0 = bfloat16, 1 = float32.  `stream` is a cudaStream_t.  Returns one of the codes above.
int tb200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* weight, const float* rstd, void* dx,
                              float* dw, int64_t rows, int dim, int dtype, void* stream);

// Human-readable text for a return code.
const char* tb200_noalloc_strerror(int code);

// cudaError_t of the most recent failing CUDA call made by this entry point (0 if none).
int tb200_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
