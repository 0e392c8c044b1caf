// Packed variable-length attention for sm_100a (head_dim 128, bf16, full attention inside a
// segment), forward and backward, on tcgen05 tensor cores with accumulators in tensor memory.
//
// Forward, per CTA = one 128-query tile of one (segment, head):
//   warp 0     TMA producer: Q once, then K / V tiles of 64 keys through a 2-stage ring
//   warp 1     MMA issuer:   S = Q K^T (128 x 64, fp32 in TMEM, double-buffered) and
//                            O += P V  (128 x 128, fp32 in TMEM); P is read from shared memory
//   warps 2-5  softmax:      one thread per query row reads its S row from TMEM, keeps the
//                            running max / sum in registers, writes P (bf16, 128-byte swizzled)
//                            and rescales O in TMEM only when the max grew by more than 2^8
// Two CTAs share an SM (256 TMEM columns and ~112 KB of shared memory each), so one CTA's
// softmax overlaps the other's MMAs. Scores are kept in the log2 domain (scale * log2 e folded
// in); `lse = m + log2 l` per (head, row) is saved for backward.
//
// The reference covers this op with Triton kernels (`src/kohakumoss_kernels/backends/triton/
// attention/_kernels.py:40-367`) and, on Blackwell, binds cuDNN's SDPA per segment instead
// (`docs/performance/training-b300.md:69-77`).

#include "attention_sm100.cuh"

#include "common.cuh"
#include "tma_host.cuh"

namespace kmoss {

namespace {

constexpr int DH = 128;
constexpr int BM = 128;        // query rows per CTA
constexpr int BN = 64;         // keys per iteration
constexpr int FWD_THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units: P stays below 2^8

// shared memory map (bytes, from a 1024-aligned base)
constexpr int SM_Q = 0;                       // 2 k-blocks x [128 rows][128 B]
constexpr int SM_KV = 32768;                  // 2 stages x (K 16 KB + V 16 KB)
constexpr int SM_P = SM_KV + 2 * 32768;       // [128 rows][128 B]
constexpr int SM_BAR = SM_P + 16384;
constexpr int FWD_SMEM = SM_BAR + 256;

// TMEM columns
constexpr uint32_t TM_S = 0;     // two S buffers of 64 columns
constexpr uint32_t TM_O = 128;   // 128 columns
constexpr uint32_t TM_COLS = 256;

__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const AttnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BAR);
  const uint32_t bar0 = smem_u32(bars);
  // barriers: 0 q_full | 1,2 k_full | 3,4 v_full | 5,6 kv_empty | 7,8 s_full | 9 p_full | 10 o_done
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int q0 = a.tiles[4 * tile + 0], seg_start = a.tiles[4 * tile + 1], seg_end = a.tiles[4 * tile + 2];
  const int n_kv = (seg_end - seg_start + BN - 1) / BN;

  if (threadIdx.x == 0) {
    if ((sbase & 1023u) != 0) report_status(a.status, STATUS_BAD_ARGUMENT, 900, (int)(sbase & 1023u));
    for (int i = 0; i < 11; ++i) mbar_init(bar(i), i == 9 ? 4 : 1);
    *abort_flag = (sbase & 1023u) != 0 ? 1 : 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one() && !*abort_flag) {
      mbar_expect_tx(bar(0), 32768);
      tma_load_2d(sbase + SM_Q, &map_q, bar(0), head * DH, q0);
      tma_load_2d(sbase + SM_Q + 16384, &map_q, bar(0), head * DH + 64, q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar(5 + st), ((j >> 1) & 1) ^ 1, abort_flag, a.status, 500 + st)) break;
        const uint32_t kdst = sbase + SM_KV + st * 32768, vdst = kdst + 16384;
        const int row = seg_start + j * BN;
        mbar_expect_tx(bar(1 + st), 16384);
        tma_load_2d(kdst, &map_k, bar(1 + st), head * DH, row);
        tma_load_2d(kdst + 8192, &map_k, bar(1 + st), head * DH + 64, row);
        mbar_expect_tx(bar(3 + st), 16384);
        tma_load_2d(vdst, &map_v, bar(3 + st), head * DH, row);
        tma_load_2d(vdst + 8192, &map_v, bar(3 + st), head * DH + 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && !*abort_flag) {
      constexpr uint32_t idesc_s = umma_idesc(1, 1, 0, 0, BM, BN);
      constexpr uint32_t idesc_o = umma_idesc(1, 1, 0, 1, BM, DH);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t kaddr = sbase + SM_KV + st * 32768;
        const uint32_t d = tmem + TM_S + (uint32_t)(st * BN);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t qd = umma_smem_desc(sbase + SM_Q + kb * 16384, 16, 1024);
          const uint64_t kd = umma_smem_desc(kaddr + kb * 8192, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16_ss(d, qd + 2 * k, kd + 2 * k, idesc_s, (kb | k) != 0);
        }
        tc_commit(bar(7 + st));
      };
      bool ok = mbar_wait(bar(0), 0, abort_flag, a.status, 600);
      ok = ok && mbar_wait(bar(1), 0, abort_flag, a.status, 601);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait(bar(1 + ((j + 1) & 1)), ((j + 1) >> 1) & 1, abort_flag, a.status, 602)) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(bar(9), j & 1, abort_flag, a.status, 603)) break;
        if (!mbar_wait(bar(3 + st), (j >> 1) & 1, abort_flag, a.status, 604)) break;
        tc_fence_after();
        const uint64_t pd = umma_smem_desc(sbase + SM_P, 16, 1024);
        const uint64_t vd = umma_smem_desc(sbase + SM_KV + st * 32768 + 16384, 8192, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_f16_ss(tmem + TM_O, pd + 2 * k, vd + 128 * k, idesc_o, (j | k) != 0);
        tc_commit(bar(5 + st));  // K / V stage free
        tc_commit(bar(10));      // O updated, P buffer free
      }
    }
  } else {
    // ----------------------------------- softmax ------------------------------------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // row inside the tile
    const int row = q0 + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sc = a.scale * LOG2E;
    float m_used = -INFINITY, l = 0.f;
    bool ok = !*abort_flag;
    for (int j = 0; ok && j < n_kv; ++j) {
      const int st = j & 1;
      if (!mbar_wait(bar(7 + st), (j >> 1) & 1, abort_flag, a.status, 700 + st)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[64];
      {
        uint32_t lo[32], hi[32];
        tmem_ld_32x32(tmem + lane_base + TM_S + st * BN, lo);
        tmem_ld_32x32(tmem + lane_base + TM_S + st * BN + 32, hi);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sr[i] = lo[i]; sr[32 + i] = hi[i]; }
      }
      const int valid = min(BN, seg_end - (seg_start + j * BN));
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        float v = __uint_as_float(sr[i]) * sc;
        v = i < valid ? v : -INFINITY;
        sr[i] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      float alpha = 1.f;
      const bool grow = mx > m_used + RESCALE_THRESHOLD;
      const bool any_grow = __any_sync(0xffffffffu, grow) && j > 0;
      if (grow) {
        alpha = exp2f(m_used - mx);  // 0 on the first tile (m_used = -inf)
        m_used = mx;
      }
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = exp2f(__uint_as_float(sr[2 * i]) - m_used);
        const float p1 = exp2f(__uint_as_float(sr[2 * i + 1]) - m_used);
        sum += p0 + p1;
        pk[i] = pack_bf16(p0, p1);
      }
      l = l * alpha + sum;
      if (j > 0) {
        // previous P V must be complete: the P buffer is reused and O may be rescaled
        if (!mbar_wait(bar(10), (j - 1) & 1, abort_flag, a.status, 710)) { ok = false; break; }
        tc_fence_after();
        if (any_grow) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem + lane_base + TM_O + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem + lane_base + TM_O + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      // P row -> shared memory, 16-byte chunks XOR-swizzled by (row & 7)
      uint8_t* prow = smem + SM_P + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 w = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(9));
    }
    if (ok && n_kv > 0 && mbar_wait(bar(10), (n_kv - 1) & 1, abort_flag, a.status, 720)) {
      tc_fence_after();
      const float inv = 1.f / l;
      const bool store = row < seg_end;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(a.o) + (size_t)(store ? row : 0) * a.ldo + head * DH;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem + lane_base + TM_O + c * 32, o);
        tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = w;
          }
        }
      }
      if (store && a.lse != nullptr) a.lse[(size_t)head * a.n_rows + row] = m_used + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, TM_COLS);
  }
}

}  // namespace

cudaError_t attention_fwd(const AttnArgs& a, cudaStream_t s) {
  if (a.n_tiles <= 0 || a.heads <= 0) return cudaSuccess;
  CUtensorMap mq, mk, mv;
  const uint64_t cols = (uint64_t)a.heads * DH;
  bool ok = tma_map_bf16_sw128(&mq, a.q, a.n_rows, cols, a.ldq, BM);
  ok &= tma_map_bf16_sw128(&mk, a.k, a.n_rows, cols, a.ldk, BN);
  ok &= tma_map_bf16_sw128(&mv, a.v, a.n_rows, cols, a.ldv, BN);
  if (!ok) return cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid(a.n_tiles, a.heads);
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, s>>>(mq, mk, mv, a);
  return cudaGetLastError();
}

}  // namespace kmoss
