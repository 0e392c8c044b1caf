// Host-visible interface of the peer-memory collectives (see comm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kmoss {

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_BLOCKS = 64;
constexpr size_t AR_ONE_SHOT_BYTES = 256 * 1024;
// uint32 words of flag memory each rank must provide: [2 phases][AR_MAX_BLOCKS][AR_MAX_WORLD]
constexpr int AR_FLAG_WORDS = 2 * AR_MAX_BLOCKS * AR_MAX_WORLD;

struct AllReduceArgs {
  void* ptrs[AR_MAX_WORLD];       // every rank's mapping of the bucket (index = rank)
  uint32_t* flags[AR_MAX_WORLD];  // every rank's flag words (zero-initialised once)
  void* mc_ptr;                   // NVLS multicast mapping of the bucket, or nullptr for peer loads / stores
  size_t n_vec;                   // bucket size in 16-byte vectors
  int rank, world;
  int dtype;                      // 0 = fp32, 1 = bf16
  float scale;                    // multiplied into the sum (1 / world for an average)
  uint32_t epoch;                 // strictly increasing per launch on this flag memory, starts at 1
  int* status;
};

int allreduce_max_blocks();
cudaError_t allreduce_launch(const AllReduceArgs& a, int blocks, cudaStream_t s);
cudaError_t bounded_wait_probe(const uint32_t* flag, uint32_t expect, uint64_t limit_ns, int* status, cudaStream_t s);

}  // namespace kmoss
