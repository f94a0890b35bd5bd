// One-tile GEMMs through exactly the operand forms the attention kernels rely on, so that
// the test-suite can check the TMA swizzle / UMMA descriptor / tensor-memory layout
// conventions in isolation.
//   mode 0: D(128x128) = A(128x64) * B(128x64)^T     A, B from shared memory, K-contiguous
//   mode 1: D(128x64)  = A(128x128) * B(128x64)      A bf16 from tensor memory, B from shared
//                                                     memory read N-contiguous
//   mode 2: mode 0 plus one more k-step, A[:, :16] * B[:, :16]^T, from unswizzled (rows x 16)
//           side operands written by the threads (the form the dK/dV kernel's row constants take)
//   mode 3: no copy, no MMA: every thread waits, with the short limit `wait_limit_cycles`, on a barrier
//           that nothing will ever arrive at.  The wait must run out, the first thread to notice raises
//           the CTA's abort flag, the others leave at their next look at it, the CTA reports
//           kStatusWaitTimeout, frees its tensor memory and returns normally -- the give-up path every
//           kernel of the library shares, exercised without leaving anything waiting on the GPU.
#pragma once
#include "attn_common.cuh"

namespace b200attn {

struct SelftestSmem {
  alignas(1024) uint8_t a[kTileBytes];
  alignas(1024) uint8_t b[kTileBytes];
  alignas(128) uint8_t a2[kOnesTileBytes];
  alignas(128) uint8_t b2[kOnesTileBytes];
  alignas(8) uint64_t bar_load;
  uint64_t bar_mma;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(128)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, int mode,
                     const __nv_bfloat16* a_global, const __nv_bfloat16* b_global, float* d, int* status,
                     long long wait_limit_cycles) {
  extern __shared__ uint8_t smem_raw[];
  SelftestSmem* sm = reinterpret_cast<SelftestSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t bar_load = smem_u32(&sm->bar_load), bar_mma = smem_u32(&sm->bar_mma);
  volatile int* abort_flag = &sm->abort_flag;
  constexpr uint32_t kCols = 256;  // D: [0,128)   A (mode 1): [128,192)

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t lane_addr = uint32_t(warp * 32) << 16;

  if (mode == 3) {
    const bool done = warp_all(mbar_wait_limit(bar_mma, 0, abort_flag, wait_limit_cycles));
    if (!done && tid == 0 && status != nullptr) atomicOr(status, kStatusWaitTimeout);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
      __syncwarp();
      tmem_dealloc(tmem, kCols);
    }
    return;
  }

  if (tid == 0) {
    if (mode != 1) {
      mbar_arrive_expect_tx(bar_load, 2 * kTileBytes);
      tma_load_4d(smem_u32(sm->a), &tm_a, bar_load, 0, 0, 0, 0);
    } else {
      mbar_arrive_expect_tx(bar_load, kTileBytes);
    }
    tma_load_4d(smem_u32(sm->b), &tm_b, bar_load, 0, 0, 0, 0);
  }
  if (mode == 1) {  // thread r puts row r of A (128 bf16 = 64 words) into tensor memory
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a_global + tid * 128);
    uint32_t w[32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int c = 0; c < 32; ++c) w[c] = src[half * 32 + c];
      tmem_st32(tmem + 128 + lane_addr + half * 32, w);
    }
    tmem_wait_st();
  }
  if (mode == 2) {  // thread r puts the first 16 elements of row r of A and of B into the side tiles
    const uint4* ra = reinterpret_cast<const uint4*>(a_global + tid * 64);
    const uint4* rb = reinterpret_cast<const uint4*>(b_global + tid * 64);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      *reinterpret_cast<uint4*>(sm->a2 + ones_offset(tid, half)) = ra[half];
      *reinterpret_cast<uint4*>(sm->b2 + ones_offset(tid, half)) = rb[half];
    }
    fence_proxy_async_smem();   // written with ordinary stores, read by the tensor core
  }
  bool ok = warp_all(mbar_wait(bar_load, 0, abort_flag));
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (ok && tid == 0) {
    if (mode != 1) {
      const uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
      const uint64_t da = desc_kmajor(smem_u32(sm->a)), db = desc_kmajor(smem_u32(sm->b));
      for (int kk = 0; kk < 4; ++kk) umma_ss(tmem, da + kk * kDescKStepKMajor, db + kk * kDescKStepKMajor, idesc, kk > 0);
      if (mode == 2) umma_ss(tmem, desc_ones(smem_u32(sm->a2)), desc_ones(smem_u32(sm->b2)), idesc, 1);
    } else {
      const uint32_t idesc = make_idesc_bf16(128, 64, 0, 1);
      const uint64_t db = desc_mnmajor(smem_u32(sm->b));
      for (int kk = 0; kk < 8; ++kk) umma_ts(tmem, tmem + 128 + kk * 8, db + kk * kDescKStepMNMajor, idesc, kk > 0);
    }
    umma_commit(bar_mma);
  }
  __syncwarp();
  ok = ok && warp_all(mbar_wait(bar_mma, 0, abort_flag));
  if (ok) {
    tc_fence_after_sync();
    const int n = mode != 1 ? 128 : 64;
    uint32_t r[32];
    for (int c = 0; c < n / 32; ++c) {
      tmem_ld32(tmem + lane_addr + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 32; ++e) d[tid * n + c * 32 + e] = __uint_as_float(r[e]);
    }
  } else if (tid == 0 && status != nullptr) {
    atomicOr(status, kStatusWaitTimeout);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, kCols);
  }
}

}  // namespace b200attn
