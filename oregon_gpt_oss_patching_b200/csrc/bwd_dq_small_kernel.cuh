// dQ kernel for short key ranges (sliding-window layers), sm_100a.
//
// Same arithmetic as attn_bwd_dq_kernel (see bwd_dq_kernel.cuh), laid out for two CTAs per SM:
// with a 128-key window a query tile sees at most 255 keys, so a CTA has only a handful of
// steps and its prologue (barrier and tensor-memory set-up, first TMA round trip, copying Q and
// dO into tensor memory) and epilogue are as long as the steps themselves.  Half the footprint
// -- 256 threads, 256 tensor-memory columns, 64 KB of shared memory -- lets a second CTA run
// under those phases.  Keys are streamed in 64-key blocks; one compute warpgroup (one thread per
// query row) handles every step; S/dP live in a single tensor-memory buffer.
#pragma once
#include "attn_common.cuh"
#include "bwd_dkdv_kernel.cuh"  // kBlk, kBlkBytes
#include "bwd_dq_kernel.cuh"    // dq_compute_chunk

namespace b200attn {

constexpr int kDqsStages = 4;
constexpr int kDqsThreads = 256;
constexpr int kDqsTmemCols = 256;
// tensor-memory columns: S/dS [0,64)  dP [64,128)  Q bf16 [128,160)  dO bf16 [160,192)  dQ [192,256)

struct DqsSmem {
  alignas(1024) uint8_t k[kDqsStages][kBlkBytes];
  alignas(1024) uint8_t v[kDqsStages][kBlkBytes];
  alignas(8) uint64_t bar_q;               // Q and dO copied into tensor memory (128 arrivals)
  uint64_t bar_in_full[kDqsStages];        // K and V block of a stage landed
  uint64_t bar_s_full;                     // S and dP ready         (tcgen05.commit)
  uint64_t bar_p_full;                     // dS written             (128 arrivals)
  uint64_t bar_acc;                        // every MMA retired: dQ final
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;
};

// Half a step (32 key columns) for one query row: dS (bf16) from S/dP, adds sum_j P*dP to pdp.
template <bool kMask>
__device__ __forceinline__ void dqs_compute_half(const uint32_t (&rs)[32], const uint32_t (&rp)[32], float scale_log2,
                                                 float nl2, float delta, int i, int j0, int window, int len,
                                                 uint32_t (&pk)[16], float& pdp) {
  // The 32-key chunk is classified for the whole warp: visible to all 32 rows (no masking work), to
  // none (dS = 0 without a single exponential -- half the chunks of a sliding-window layer), or mixed.
  const uint32_t bits = kMask ? visible_keys32(i, j0, window, len) : 0xffffffffu;
  const float2 scale2 = make_float2(scale_log2, scale_log2), nl22 = make_float2(nl2, nl2);
  const float2 neg_delta2 = make_float2(-delta, -delta);
  float2 acc = make_float2(0.f, 0.f);
  if (kMask && __all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
    for (int k = 0; k < 16; ++k) pk[k] = 0u;
  } else if (!kMask || __all_sync(0xffffffffu, bits == 0xffffffffu)) {
    dq_compute_chunk<false>(rs, rp, scale2, nl22, neg_delta2, bits, pk, acc);
  } else {
    dq_compute_chunk<true>(rs, rp, scale2, nl22, neg_delta2, bits, pk, acc);
  }
  pdp += acc.x + acc.y;
}

__global__ void __launch_bounds__(kDqsThreads, 2)
attn_bwd_dq_small_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                         const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DqsSmem* sm = reinterpret_cast<DqsSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / a.group;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * kTile;
  const int len = seq_len(a, b);

  // eight sink-gradient partial slots per query tile; this kernel fills four, zeroes four
  float* ds_partial = a.dsinks_partial + (((long long)h * a.B + b) * (a.S_pad / kTile) + qt) * 8;
  if (q0 >= len) {  // padding only: dQ rows are zero, no sink gradient
    if (tid < kComputeThreads && q0 + tid < a.S) zero_row(a.dq.row(b, h, q0 + tid));
    if (tid < 8) ds_partial[tid] = 0.f;
    return;
  }

  const int hi = min(q0 + kTile - 1, len - 1);              // last visible key
  const int lo = a.window ? max(0, q0 - a.window + 1) : 0;  // first visible key
  const int kb_first = lo / kBlk;
  const int n_steps = hi / kBlk - kb_first + 1;
  const float* nlse_base = a.delta + (long long)a.B * a.Hq * a.S_pad;  // second half of the delta scratch

  // issue this thread's global loads before the set-up barrier so that they overlap it
  const int i = q0 + (tid & 127);  // this thread's query position (compute warps)
  uint4 q_row[8], do_row[8];
  float nl2 = 0.f, delta = 0.f;
  if (warp < 4) {
    const long long row_off = ((long long)(b * a.Hq + h)) * a.S_pad + i;
    nl2 = nlse_base[row_off];   // -LSE * log2(e)
    delta = a.delta[row_off];
    if (i < a.S) {
      const uint4* qr = reinterpret_cast<const uint4*>(a.q.row(b, h, i));
      const uint4* dr = reinterpret_cast<const uint4*>(a.d_o.row(b, h, i));
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        q_row[c] = qr[c];
        do_row[c] = dr[c];
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) q_row[c] = do_row[c] = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  const uint32_t bar_q = smem_u32(&sm->bar_q), bar_acc = smem_u32(&sm->bar_acc), bar_s_full = smem_u32(&sm->bar_s_full),
                 bar_p_full = smem_u32(&sm->bar_p_full);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_q, kComputeThreads);
    for (int s = 0; s < kDqsStages; ++s) mbar_init(smem_u32(&sm->bar_in_full[s]), 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, kComputeThreads);
    mbar_init(bar_acc, 1);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDqsTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 64, tmem_q = tmem + 128, tmem_do = tmem + 160, tmem_dq = tmem + 192;

  if (warp == 5) {
    // ------------------------------------ TMA loader ------------------------------------
    // at most kDqsStages steps are supported per launch of this kernel (the host checks), so
    // every block has its own stage and no stage is ever refilled
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      for (int it = 0; it < n_steps; ++it) {
        const int kv0 = (kb_first + it) * kBlk;
        const uint32_t bar = smem_u32(&sm->bar_in_full[it]);
        mbar_arrive_expect_tx(bar, 2 * kBlkBytes);
        tma_load_4d(smem_u32(sm->k[it]), &tm_k, bar, 0, kv0, g, b);
        tma_load_4d(smem_u32(sm->v[it]), &tm_v, bar, 0, kv0, g, b);
        *reinterpret_cast<volatile int*>(&sm->loads_issued) = it + 1;
      }
    }
    __syncwarp();
  } else if (warp == 4) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kBlk, 0, 0);     // A in TMEM, B K-contiguous, N = 64
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      tc_fence_after_sync();
      for (int it = 0; ok && it < n_steps; ++it) {
        if (!(ok = mbar_wait(smem_u32(&sm->bar_in_full[it]), 0, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[it]));
        const uint64_t v_desc = desc_kmajor(smem_u32(sm->v[it]));
        // S/dP of this step go behind the previous step's dQ MMAs in the pipe, which read dS from the same columns
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ts(tmem_s, tmem_q + kk * 8, k_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ts(tmem_dp, tmem_do + kk * 8, v_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
        umma_commit(bar_s_full);
        if (!(ok = mbar_wait(bar_p_full, it & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k[it]));
#pragma unroll
        for (int kk = 0; kk < kBlk / 16; ++kk)
          umma_ts(tmem_dq, tmem_s + kk * 8, kt_desc + kk * kDescKStepMNMajor, idesc_back, (it > 0 || kk > 0) ? 1u : 0u);
      }
      if (ok) umma_commit(bar_acc);
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp < 4) {
    // ------------------------------------- compute --------------------------------------
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;
    float pdp = 0.f;  // sum_j P_ij dP_ij
    bool ok = true;

    {  // this thread's rows of Q and dO into tensor memory as bf16
      uint32_t w[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) { w[4 * c] = q_row[c].x; w[4 * c + 1] = q_row[c].y; w[4 * c + 2] = q_row[c].z; w[4 * c + 3] = q_row[c].w; }
      tmem_st32(tmem_q + lane_addr, w);
#pragma unroll
      for (int c = 0; c < 8; ++c) { w[4 * c] = do_row[c].x; w[4 * c + 1] = do_row[c].y; w[4 * c + 2] = do_row[c].z; w[4 * c + 3] = do_row[c].w; }
      tmem_st32(tmem_do + lane_addr, w);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_q);
    }

    for (int it = 0; it < n_steps; ++it) {
      const int kv0 = (kb_first + it) * kBlk;
      const bool need_mask = (kv0 + kBlk - 1 > q0) || (a.window != 0 && kv0 <= q0 + kTile - 1 - a.window) || (q0 + kTile > len);
      if (!(ok = warp_all(mbar_wait(bar_s_full, it & 1, abort_flag)))) break;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32], pk[16];
        tmem_ld32(tmem_s + lane_addr + c * 32, rs);
        tmem_ld32(tmem_dp + lane_addr + c * 32, rp);
        tmem_wait_ld();
        if (need_mask) dqs_compute_half<true>(rs, rp, a.scale_log2, nl2, delta, i, kv0 + c * 32, a.window, len, pk, pdp);
        else dqs_compute_half<false>(rs, rp, a.scale_log2, nl2, delta, i, kv0 + c * 32, a.window, len, pk, pdp);
        tmem_st16(tmem_s + lane_addr + c * 16, pk);  // dS over S columns this thread has consumed
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p_full);
    }

    if (ok) ok = warp_all(mbar_wait(bar_acc, 0, abort_flag));
    if (ok) {
      // sink gradient of this warp's 32 rows (fixed-order shuffle tree); the other four slots are zero
      float dsk = (i < len) ? -fast_exp2(fmaf(a.sinks[h], kLog2e, nl2)) * pdp : 0.f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dsk += __shfl_xor_sync(0xffffffffu, dsk, off);
      if (lane == 0) {
        ds_partial[warp] = dsk;
        ds_partial[4 + warp] = 0.f;
      }
      tc_fence_after_sync();
      uint32_t r0[32], r1[32];
      tmem_ld32(tmem_dq + lane_addr, r0);
      tmem_ld32(tmem_dq + lane_addr + 32, r1);
      tmem_wait_ld();
      if (i < a.S) {
        __nv_bfloat16* dst = a.dq.row(b, h, i);
        const float sc = (i < len) ? a.scale : 0.f;
#pragma unroll
        for (int c = 0; c < 32; c += 8)
          store_bf16x8(dst + c, pack_bf16(__uint_as_float(r0[c]) * sc, __uint_as_float(r0[c + 1]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 2]) * sc, __uint_as_float(r0[c + 3]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 4]) * sc, __uint_as_float(r0[c + 5]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 6]) * sc, __uint_as_float(r0[c + 7]) * sc));
#pragma unroll
        for (int c = 0; c < 32; c += 8)
          store_bf16x8(dst + 32 + c, pack_bf16(__uint_as_float(r1[c]) * sc, __uint_as_float(r1[c + 1]) * sc),
                       pack_bf16(__uint_as_float(r1[c + 2]) * sc, __uint_as_float(r1[c + 3]) * sc),
                       pack_bf16(__uint_as_float(r1[c + 4]) * sc, __uint_as_float(r1[c + 5]) * sc),
                       pack_bf16(__uint_as_float(r1[c + 6]) * sc, __uint_as_float(r1[c + 7]) * sc));
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, kDqsTmemCols);
  }
  if (sm->abort_flag && tid == 5 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued;
    for (int it = 0; it < issued; ++it) mbar_wait_drain(smem_u32(&sm->bar_in_full[it]), 0);
  }
}

}  // namespace b200attn
