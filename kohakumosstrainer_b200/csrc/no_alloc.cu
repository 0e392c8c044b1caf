// Split-K GEMM without any allocation: the partial-sum scratch is a file-scope device array.
// See no_alloc.h for who needs this and for the contract.

#include "no_alloc.h"

#include <stdio.h>

#include "gemm_sm100.cuh"

namespace {

// The scratch lives in the library image: one copy per GPU that loads the library.
static __device__ __align__(256) unsigned char g_noalloc_scratch[KMOSS_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// Device address of the scratch per device. In host code `g_noalloc_scratch` is only a handle for
// the symbol, not a device address, so the address is looked up once per device.
float* g_scratch_ptr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" int kmoss_gemm_splitk_noalloc(const void* a, const void* b, float* out, int M, int N, int K, long lda, long ldb,
                                         long ldo, int a_mn, int b_mn, int splits, cudaStream_t stream) {
  if (a == nullptr || b == nullptr || out == nullptr || M <= 0 || N <= 0 || K <= 0 || splits < 2 || splits > 64) {
    fprintf(stderr, "kmoss_gemm_splitk_noalloc: bad argument (pointers must be non-null, M, N, K > 0, 2 <= splits <= 64)\n");
    return KMOSS_NOALLOC_ERR_ARGUMENT;
  }
  const size_t need = kmoss::gemm_workspace_bytes(M, N, splits);
  if (need > (size_t)KMOSS_NOALLOC_SCRATCH_BYTES) {
    fprintf(stderr, "kmoss_gemm_splitk_noalloc: splits * M * N * 4 = %zu bytes exceeds the built-in scratch of %u bytes\n",
            need, (unsigned)KMOSS_NOALLOC_SCRATCH_BYTES);
    return KMOSS_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) {
    fprintf(stderr, "kmoss_gemm_splitk_noalloc: device index %d out of range\n", dev);
    return KMOSS_NOALLOC_ERR_DEVICE;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    // first call on this device (it is current): resolve the symbol to its device address
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "kmoss_gemm_splitk_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return (int)e;
    }
    g_scratch_ptr[dev] = reinterpret_cast<float*>(ptr);
  }
  kmoss::GemmProblem g{};
  g.M = M; g.N = N; g.K = K;
  g.A = a; g.B = b; g.lda = lda; g.ldb = ldb;
  g.a_dtype = kmoss::GEMM_BF16; g.b_dtype = kmoss::GEMM_BF16;
  g.a_mn = a_mn ? 1 : 0; g.b_mn = b_mn ? 1 : 0;
  g.epilogue = kmoss::EPI_LINEAR;
  g.out = out; g.ldo = ldo; g.out_dtype = kmoss::OUT_F32;
  g.alpha = 1.f; g.beta = 0.f;
  g.splits = splits;
  g.workspace = g_scratch_ptr[dev];
  e = kmoss::gemm_launch(g, stream);
  return (int)e;
}
