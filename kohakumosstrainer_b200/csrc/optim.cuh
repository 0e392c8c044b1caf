// Host-visible interface of the optimiser kernels (see optim.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kmoss {

// One tensor of a parameter group. dtype codes: 0 = fp32, 1 = bf16.
struct OptTensor {
  void* param;
  const void* grad;
  float* exp_avg;
  float* exp_avg_sq;
  float* master;   // fp32 master copy (nullable: the parameter itself is the master)
  float* ema;      // fp32 EMA copy (nullable)
  long n;
  float lr_mul;
  float weight_decay;
  int param_dtype;
  int grad_dtype;
  int decay_to_one;
  int mode;        // writeback of a bf16 parameter without master: 0 nearest, 1 stochastic rounding, 2 Kahan (uses comp)
  void* comp;      // Kahan compensation, same dtype as the parameter (nullable)
  // 8-bit states (nullable; when set, exp_avg / exp_avg_sq are unused): blockwise (256) sqrt-companded codes of the
  // first moment (int8) and of r = sqrt(second moment) (uint8), with one fp32 absmax per block
  signed char* mq;
  unsigned char* rq;
  float* ms;
  float* rs;
};

struct AdamWHyper {
  float lr, beta1, beta2, eps;
  float inv_bc1;        // 1 / (1 - beta1^t)
  float inv_sqrt_bc2;   // 1 / sqrt(1 - beta2^t)
  float ema_decay;
  unsigned seed;        // stochastic rounding: hashed with the element index, changes every step
  const float* grad_scale;  // device scalar multiplied into every gradient (clip coefficient), nullable
  const int* skip;          // device flag: non-zero skips the whole step, nullable
};

int opt_chunk_elems();
// plain: every tensor of the table has fp32 states and nearest writeback (no 8-bit codes, no compensation buffer)
cudaError_t adamw_multi(const OptTensor* tensors, const int2* chunks, int n_chunks, const AdamWHyper& h, bool plain, cudaStream_t s);
// partial: [n_chunks] fp32 scratch; out[0] = norm, out[1] = clip coefficient, out[2] = sum of squares
cudaError_t grad_norm_multi(const OptTensor* tensors, const int2* chunks, int n_chunks, float* partial, int* nonfinite,
                            float max_norm, float* out, cudaStream_t s);
cudaError_t ema_multi(const OptTensor* tensors, const int2* chunks, int n_chunks, float decay, const int* skip, cudaStream_t s);

}  // namespace kmoss
