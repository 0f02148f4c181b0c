// Allocation-free entry point of the torchturbo_b200 CUDA library.
//
// This declaration has no counterpart in the reference project: it exists for hosts that cannot obtain device
// memory at call time.  Examples: a plain C or C++ program that links this library without PyTorch (so there is no
// caching allocator to hand out workspaces), a service that has given all remaining device memory to another pool,
// or a latency-sensitive loop in which cudaMalloc / cudaFree (which may synchronise the whole device) must never run.
//
// ttb_rmsnorm_bwd_noalloc computes the same result as ttb_rmsnorm_bwd (RMSNorm backward: dx and the fp32 weight
// gradient) but takes no workspace argument.  Its per-block partial sums of the weight gradient live in a
// file-scope __device__ array inside the library instead.
//
// Limits and rules
//   * H (row width) must be a multiple of 8 and at most TTB_NOALLOC_MAX_H; larger or misaligned H is rejected with
//     TTB_NOALLOC_ERR_SIZE and nothing is launched.  T (rows) is unlimited.
//   * The scratch array is TTB_NOALLOC_BLOCKS x TTB_NOALLOC_MAX_H floats (2 MiB).  Every GPU on which this library is
//     loaded holds that array until the process exits, whether or not this function is ever called.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current) and remembers it.  Make that first call before starting any stream capture on the device.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine; inputs and outputs are the caller's.
//   * All calls on a device share the one array and it keeps whatever the previous call left in it.  Nothing in it has
//     to start at zero: each call overwrites every element it later reads.  Two calls whose kernels may overlap on
//     the GPU (different streams, no ordering between them) race on the array and give wrong weight gradients;
//     order such calls (same stream, or an event between them).
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define TTB_NOALLOC_MAX_H 8192
#define TTB_NOALLOC_BLOCKS 64

/* Return codes.  The three error classes use disjoint ranges (a CUDA error code is always below 10000), so a code
 * names its class and, for the last three, the CUDA error: code - base. */
#define TTB_NOALLOC_OK 0
#define TTB_NOALLOC_ERR_SIZE 901            /* H not a multiple of 8, or H > TTB_NOALLOC_MAX_H, or T < 0 */
#define TTB_NOALLOC_ERR_LAUNCH_DX 100000    /* launch of the dx / partial-sum kernel failed; + CUDA error code */
#define TTB_NOALLOC_ERR_LAUNCH_DW 110000    /* launch of the weight-gradient column sum failed; + CUDA error code */
#define TTB_NOALLOC_ERR_SYMBOL 200000       /* cudaGetDevice / cudaGetSymbolAddress failed; + CUDA error code */

/* dy, x, w, dres_in (may be NULL), dx: bf16 device pointers, row-major [T, H] ([H] for w); rstd: fp32 [T];
 * dw_out: fp32 [H].  `stream` is a cudaStream_t.  Returns TTB_NOALLOC_OK or one of the codes above. */
int ttb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                            void* dx, float* dw_out, long long T, int H, int one_plus_w, void* stream);

/* Human-readable text for a return code of the function above (static storage, never NULL). */
const char* ttb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
