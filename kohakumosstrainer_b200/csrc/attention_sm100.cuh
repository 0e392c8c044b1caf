// Host-visible interface of the varlen attention kernels (see attention_sm100.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kmoss {

// Packed q, k, v, o: [N, H, 128] bf16; a token row is `ld*` elements apart, heads are 128
// apart. `tiles` is an int32 [T, 4] device table built on the host from the segment lengths:
// {first query row of the tile, segment start row, segment end row, unused}. Attention is
// full (non-causal) inside a segment. `lse` is fp32 [H, N]: log2-domain log-sum-exp of the
// scaled scores (scale * log2(e) folded in), which the backward kernels consume.
struct AttnArgs {
  const void* q; const void* k; const void* v;
  void* o;
  long ldq, ldk, ldv, ldo;
  float* lse;
  const int* tiles;
  int n_tiles;
  int n_rows;     // N
  int heads;
  float scale;    // softmax scale (Dh^-0.5)
  int* status;
};

struct AttnBwdArgs {
  const void* q; const void* k; const void* v; const void* o; const void* dout;
  long ldq, ldk, ldv, ldo, lddo;
  void* dq; void* dk; void* dv;
  long lddq, lddk, lddv;
  const float* lse;
  float* delta;        // fp32 [H, N] scratch: rowsum(dO * O)
  const int* tiles;    // 128-row tiles of each segment (query tiles for dQ, key tiles for dK / dV)
  int n_tiles;
  int n_rows;
  int heads;
  float scale;
  int* status;
  // nullable probe [2, timeline_iters, 8] (dQ kernel rows, then dK / dV rows): block (0, 0) records %clock64 per loop iteration:
  // element-wise warp 2 {loop top, operands ready, loaded from tensor memory, computed, staging free, stored}, MMA thread {6: products of
  // the next tile issued, 7: accumulation issued}. Slots past `timeline_iters` iterations are not written.
  unsigned long long* timeline;
  int timeline_iters;
};

// Install (or clear, with nullptr) the probe buffer used by the next backward launches.
void attention_set_timeline(unsigned long long* buf, int iters);

cudaError_t attention_fwd(const AttnArgs& a, cudaStream_t s);
cudaError_t attention_bwd(const AttnBwdArgs& a, cudaStream_t s);

}  // namespace kmoss
