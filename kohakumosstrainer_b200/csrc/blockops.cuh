// Host-visible interface of the block-op kernels (see blockops.cu). All activations are
// bf16, row-major; modulation vectors are fp32 `[B, dim]` views with a row stride
// (`mod_stride`, 6 * dim for a slice of the shared `[B, 6, dim]` modulation); `seg` maps a
// row to its sample. Launchers enqueue on `stream` and allocate nothing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kmoss {

struct NormModArgs {
  const __nv_bfloat16* x; long ldx;
  const void* w; int w_f32;           // [dim] nullable; bf16 or fp32
  const float* shift; const float* scale; long mod_stride;  // nullable
  const int* seg;                     // nullable (with shift / scale)
  float eps;
  __nv_bfloat16* y; long ldy;
  float* rstd;                        // [rows] nullable
  uint8_t* yq; long ldq;              // optional e4m3 copy of y, scaled by *q_scale
  const float* q_scale;
  float* amax;                        // optional running max |y| (must start >= 0)
  int rows, dim;
};

struct NormModBwdArgs {
  const __nv_bfloat16* dy; long lddy;
  const __nv_bfloat16* x; long ldx;
  const void* w; int w_f32;
  const float* scale; long mod_stride;
  const int* seg;
  const float* rstd;
  __nv_bfloat16* dx; long lddx;
  const __nv_bfloat16* dres; long lddres; float dres_scale;  // optional: dx += dres_scale * dres
  int rows, dim;
};

struct SegSumArgs {
  const __nv_bfloat16* a; long lda;
  const __nv_bfloat16* b; long ldb;
  const void* w; int w_f32;
  const float* rstd;
  const int* cu;       // [batch + 1] row offsets of the (sorted) segments
  float* out; long ldo;
  int batch, dim, mode;
  float* partial;      // [split, batch, dim] scratch: a segment's rows are summed in `split` slices, then the slices in order
  int split;
};
constexpr int SEG_SUM_SPLIT = 32;

struct QkRopeArgs {
  const __nv_bfloat16* x; long ldx;   // [rows, heads * 128]
  const void* w; int w_f32;           // [128]
  const float* rope;                  // [rows, 128] cos | sin
  float eps;
  __nv_bfloat16* y; long ldy;
  float* rstd;                        // [rows, heads] nullable
  int rows, heads;
};

struct QkRopeBwdArgs {
  const __nv_bfloat16* y; long ldy;   // forward OUTPUT
  const __nv_bfloat16* dy; long lddy;
  const void* w; int w_f32;
  const float* rope;
  const float* rstd;
  __nv_bfloat16* dx; long lddx;
  float* dw_rows;                     // [rows, heads, 128] nullable
  int rows, heads;
};

struct TokenMseArgs {
  const void* pred; int pred_f32;     // [rows, dim] bf16 or fp32
  const float* target;                // [rows, dim] fp32
  const int* seg;
  const float* weight;                // [B] nullable
  const float* mask;                  // [rows] nullable
  int rows, dim;
};

cudaError_t rms_norm_mod_fwd(const NormModArgs& a, cudaStream_t s);
cudaError_t rms_norm_mod_bwd(const NormModBwdArgs& a, cudaStream_t s);
cudaError_t norm_weight_grad(const NormModBwdArgs& a, float* partial, int chunks, cudaStream_t s);
cudaError_t seg_sum(const SegSumArgs& a, cudaStream_t s);
cudaError_t rope_table(const float* pos, const float* bands, float* table, int rows, int axes, int n_bands, cudaStream_t s);
cudaError_t qk_norm_rope_fwd(const QkRopeArgs& a, cudaStream_t s);
cudaError_t qk_norm_rope_bwd(const QkRopeBwdArgs& a, cudaStream_t s);
cudaError_t situ_fwd(const void* up, const void* gate, long ld_in, void* out, long ld_out, int rows, int f, cudaStream_t s);
cudaError_t situ_bwd(const void* da, long ld_da, const void* up, const void* gate, long ld_in, void* dup, void* dgate,
                     long ld_out, int rows, int f, cudaStream_t s);
cudaError_t gated_residual(const void* x, const void* o, const float* gate, long gate_stride, const int* seg, float r,
                           void* out, int rows, int dim, cudaStream_t s);
cudaError_t seg_scale(const void* x, const float* vec, long vec_stride, const int* seg, void* out, int rows, int dim,
                      cudaStream_t s);
// Producers of an output gradient that also write its per-row e5m2 copy and scales ([2, rows] = {dequant, quant}).
bool situ_bwd_quant_supported(int f);
cudaError_t situ_bwd_quant(const void* da, long ld_da, const void* up, const void* gate, long ld_in, void* dup, void* dgate,
                           long ld_out, void* q, long ldq, float* row_scale, int rows, int f, cudaStream_t s);
bool seg_scale_quant_supported(int dim);
cudaError_t seg_scale_quant(const void* x, const float* vec, long vec_stride, const int* seg, void* out, void* q, float* row_scale,
                            int rows, int dim, cudaStream_t s);
int token_mse_blocks(int rows);
cudaError_t token_mse_fwd(const TokenMseArgs& a, float* partial, float* loss, cudaStream_t s);
cudaError_t token_mse_bwd(const TokenMseArgs& a, const float* dloss, void* dpred, cudaStream_t s);
cudaError_t fp8_amax(const void* x, long n, float* amax, cudaStream_t s);
cudaError_t fp8_scale_from_amax(const float* amax, float fmax, float* scale_out, cudaStream_t s);
cudaError_t fp8_cast(const void* x, long n, const float* qscale, void* q, int e5m2, cudaStream_t s);
// row_scale: fp32 [rows] dequant scales, or [2, rows] = {dequant, quant} with `with_inverse`
cudaError_t fp8_cast_rows(const void* x, long ldx, int rows, int dim, void* q, long ldq, float* row_scale, bool e5m2,
                          bool with_inverse, cudaStream_t s);

}  // namespace kmoss
