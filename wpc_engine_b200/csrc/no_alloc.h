// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference (jpytka666-jpg/wpc-engine), which has no GPU code
// at all; it exists for embedders of this library.
//
// Who cannot allocate: code that runs inside somebody else's memory plan.  Examples are a
// plug-in called from a host application that hands out all device memory itself and forbids
// cudaMalloc from foreign code, a real-time loop in which an allocation's unbounded latency
// (it may synchronise the whole device) is not acceptable, and a process whose memory pool
// was sized up front and is already spoken for.  The library's normal product x . W^T with
// few tokens splits the shared dimension over several CTAs and needs scratch memory for their
// partial sums and tickets; wpc_engine_b200/ops.py gets that scratch from torch's allocator.
// The function below is the same kernel with its scratch in a fixed array that is part of the
// library image, so nothing is allocated at any time: not by the call, not at set-up.
//
//   x   [tokens, K]   bfloat16, row stride ldx elements, 1 <= tokens <= 128
//   w   [features, K] bfloat16, row stride ldw elements
//   out [tokens, features], row stride ldc elements, out_dtype WPC_DTYPE_BF16 or WPC_DTYPE_F32
//   bias: float32 [features] or null;  splits: CTAs along K per tile, 0 lets the call choose
//
// The caller still owns and passes every input and output.  Rows must be 16-byte aligned
// (pointers, and ldx, ldw multiples of 8) because the operands travel by TMA.
//
// Limits: the scratch array is WPC_STATIC_SCRATCH_BYTES (4 MiB + 8 KiB) and every GPU that
// loads the library holds it until the process exits.  A call needs
// ceil(features / 128) * splits * bn * 128 floats of it, bn being 16, 32, 64 or 128 (the next
// of these at or above `tokens`), and at most WPC_STATIC_MAX_TILES tiles of 128 features; a
// call that needs more returns WPC_ERR_TOO_LARGE (1003) and launches nothing.  With splits = 0
// the call picks the largest split count that fits.
//
// Set-up: the first call on each device looks up the array's device address (once per device,
// with that device current) before it launches.  Make that first call outside any stream
// capture.  All calls share the one array, and it keeps what the last call left: the tickets
// are cleared on `stream` at the start of every call, the partial sums need no clearing because
// every slice is written before it is read.  Two calls that overlap on the GPU (different
// streams, or different host threads on different streams) race on the array; run them one
// after another on one stream.
//
// Returns 0, a cudaError_t value, or a WPC_ERR_* code of common.cuh.  `splits` below zero is a
// bad argument.
//
// Errors that only the GPU can see: every wait inside the kernel is bounded, and a kernel whose
// wait ran out leaves its output unwritten and records WPC_ERR_DEVICE_WAIT (1004) in a status
// word that lies in the same array.  wpc_linear_few_tokens_static_status waits for `stream`,
// copies that word of the current device to `*status_out` (0: every call since the last look
// went through) and clears it; it allocates nothing either.  A caller that cannot afford the
// wait after every call asks once per batch of calls: the word keeps the last error.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#define WPC_STATIC_SCRATCH_FLOATS (1u << 20)
#define WPC_STATIC_MAX_TILES 1024
#define WPC_STATIC_SCRATCH_BYTES (WPC_STATIC_SCRATCH_FLOATS * 4u + 8192u)

#ifdef __cplusplus
extern "C" {
#endif

int wpc_linear_few_tokens_static(const void* x, int ldx, int tokens, const void* w, int ldw, int features, int K,
                                 const float* bias, void* out, int out_dtype, int ldc, int splits,
                                 cudaStream_t stream);
int wpc_linear_few_tokens_static_status(int* status_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
