// A GEMM entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it exists because some hosts of
// this library cannot call cudaMalloc at the point where they need a GEMM - code running
// inside a CUDA-graph capture or a latency-critical serving loop where an allocation would
// synchronise the device, plugins that are handed a stream and buffers by another runtime
// and are forbidden to touch its memory pool, and processes whose memory budget was fixed
// at start-up.  The regular entry point (zb_gemm_bf16) takes its split-K scratch from a
// per-device allocation made on first use; this one keeps the scratch in a fixed array
// that is part of the library image.
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of the built-in scratch for partial tiles.  Every GPU that loads the library holds
// this much (plus 16 KiB of counters) from load until the process exits.
#define ZB_NOALLOC_SCRATCH_BYTES (16u << 20)

// Return codes (0 = launched).
#define ZB_NOALLOC_ERR_TOO_LARGE (-101)   // the problem needs more scratch than the built-in array holds
#define ZB_NOALLOC_ERR_SETUP (-102)       // cudaGetSymbolAddress / device query failed on first use
#define ZB_NOALLOC_ERR_BAD_ARG (-103)     // null pointer, non-positive size, or unsupported alignment

// out[M,N] = a[M,K] * w[N,K]^T (+ bias[N]) (+ residual[M,N]); bf16 inputs, fp32 accumulation,
// bf16 output (out_f32 == 0) or fp32 output (any non-zero out_f32).  Same kernel and same numerics as
// zb_gemm_bf16.  All pointers are device pointers owned by the caller; lda / ldw / ldo are in
// elements and must be multiples of 8; K must be a multiple of 8.  `residual`, `bias` and
// `status_out` may be null.  `status_out`, when given, points to 16 bytes of device memory
// that receive {code, kernel, where, detail} if a bounded wait inside the kernel runs out
// (it is zeroed at the start of the call); the call itself never synchronises.
//
// Nothing is allocated or freed: no cudaMalloc, no cudaFree, no library workspace.
//   * Scratch use depends on the shape.  Few-token shapes (M <= 64) of any N, K always fit.
//     Shapes that would need more than ZB_NOALLOC_SCRATCH_BYTES return
//     ZB_NOALLOC_ERR_TOO_LARGE and print one line to stderr; nothing is launched.
//   * The first call on a device resolves the address of the built-in array on that device
//     (cudaGetSymbolAddress with that device current).  The first call of each tile shape
//     (a function of M and N) on each device also sets that kernel's shared-memory attribute.
//     Make a first call of every shape you will use before starting any stream capture on
//     that device.
//   * Every call on a device uses the same array, and the array keeps what the previous call
//     left in it.  The call zeroes the part that must start at zero (tile counters) on
//     `stream` before launching.  Two calls whose kernels can overlap on the GPU (different
//     streams without an ordering between them) race on the array: order them.
int zb_gemm_bf16_noalloc(const void* a, const void* w, void* out, const void* residual,
                         const void* bias, int m, int n, int k, int lda, int ldw, int ldo,
                         int out_f32, void* status_out, void* stream);

#ifdef __cplusplus
}
#endif
