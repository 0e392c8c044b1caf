/* A split-K GEMM entry point that allocates nothing.
 *
 * This entry point has no counterpart in the reference project. It exists for callers that
 * are not allowed to allocate device memory at the moment they need the product: code running
 * inside a memory-planned region where every buffer was laid out up front (an inference engine
 * or a pipeline stage with a fixed arena), a host thread that must not touch the CUDA allocator
 * because another thread holds it, or a C / Rust / Go embedding that links this library without
 * PyTorch's caching allocator. The regular Python path (`ops.native.gemm(..., splits > 1)`)
 * takes its split-K partial-sum buffer from a torch tensor; here that scratch is a fixed array
 * that is part of the loaded library image.
 *
 *   out[M, N] (fp32) = A . B^T,  bf16 operands, fp32 accumulation, K split into `splits` parts
 *   whose partial sums meet in the built-in scratch and are then added in a fixed order.
 *
 * Operand layout is that of `GemmProblem` in gemm_sm100.cuh: `a_mn == 0` means A is stored
 * [M, K] with row stride `lda` elements, `a_mn == 1` means it is stored [K, M]; likewise B is
 * [N, K] or [K, N] with `ldb`. `out` has row stride `ldo` floats. All pointers are device
 * pointers owned by the caller; operand bases and row strides must be multiples of 16 bytes.
 *
 * Limit: splits * M * N * 4 bytes must not exceed KMOSS_NOALLOC_SCRATCH_BYTES (16 MiB). That
 * covers the adapter-gradient shapes this path serves (for example 3072 x 64 outputs with up to
 * 21 splits). Every GPU that loads the library holds these 16 MiB until the process exits.
 *
 * Set-up: the first call on each device looks up the device address of the scratch array (with
 * that device current) and configures the kernel's shared-memory limit. Make that first call
 * before starting any CUDA stream capture; later calls only launch kernels.
 *
 * Sharing: all calls on a device use the same scratch. It keeps the previous call's partial
 * sums; nothing in it has to start at zero because every partial sum that is read is written
 * first by the same call. Two calls that overlap in time on one GPU (different streams) race
 * on the scratch and produce wrong results: keep calls on one stream or order them with events.
 *
 * Returns 0 on success, a negative KMOSS_NOALLOC_* code for a rejected argument (a message
 * naming the problem goes to stderr), or a positive cudaError_t value from a CUDA call.
 * The function calls no cudaMalloc, cudaFree or any other allocating routine.
 */
#pragma once

#include <cuda_runtime.h>

#define KMOSS_NOALLOC_SCRATCH_BYTES (16u << 20)
#define KMOSS_NOALLOC_ERR_TOO_LARGE (-1)   /* splits * M * N * 4 exceeds the scratch */
#define KMOSS_NOALLOC_ERR_ARGUMENT (-2)    /* null pointer, non-positive size, splits < 2 or > 64 */
#define KMOSS_NOALLOC_ERR_DEVICE (-3)      /* no current device or device index out of range */

#ifdef __cplusplus
extern "C" {
#endif

int kmoss_gemm_splitk_noalloc(const void* a, const void* b, float* out, int M, int N, int K, long lda, long ldb, long ldo,
                              int a_mn, int b_mn, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
