// dQ kernel for sm_100a.
//
// One CTA = one 128-row query tile of one query head of one sequence; it loops over the
// key tiles that tile can see.  Per key tile, on tcgen05 with accumulators in tensor memory:
//     S  = Q K^T          dP = dO V^T
// then with one thread per query row
//     P  = 2^(S*scale*log2e - LSE*log2e)      dS = P * (dP - delta)
// dS goes back to tensor memory as bf16 and is the A operand of
//     dQ += dS K          (accumulated in tensor memory over all key tiles)
// and the epilogue stores dQ * scale.  This is the dq part of the reference's `_attn_bwd`
// (attention_kernel.py:190-199, :206-207, :214-217).
//
// The same pass yields the sink gradient.  Because the softmax row (sink column included)
// sums to one,  sum_j P_ij dP_ij  equals delta_i exactly, so each thread also accumulates that
// sum in fp32 from the recomputed P and dP -- it does not inherit the bf16 rounding of the
// stored O that delta = rowsum(dO*O) carries -- and the CTA writes, per warp,
//     - sum_i exp(sink - LSE_i) * (sum_j P_ij dP_ij)
// to the dSinks scratch (the reference's per-tile term, attention_kernel.py:173-175).
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kDqStages = 2;
constexpr int kDqTmemCols = 512;  // S / dS: [0,128)   dP: [128,256)   dQ: [256,320)

struct DqSmem {
  alignas(1024) uint8_t q[kTileBytes];
  alignas(1024) uint8_t d_o[kTileBytes];
  alignas(1024) uint8_t k[kDqStages][kTileBytes];
  alignas(1024) uint8_t v[kDqStages][kTileBytes];
  alignas(8) uint64_t bar_q;   // Q and dO landed
  uint64_t bar_kv[kDqStages];  // K and V of a stage landed
  uint64_t bar_s;              // S and dP ready
  uint64_t bar_p;              // dS written by 128 threads
  uint64_t bar_o;              // dQ MMA of a tile finished (stage + S/dP columns reusable)
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem* sm = reinterpret_cast<DqSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / a.group;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * kTile;
  const int len = seq_len(a, b);

  float* ds_partial = a.dsinks_partial + (((long long)h * a.B + b) * (a.S_pad / kTile) + qt) * 4;
  if (q0 >= len) {  // padding only: dQ rows are zero, no sink gradient
    if (tid < kComputeThreads && q0 + tid < a.S) zero_row(a.dq.row(b, h, q0 + tid));
    if (tid < 4) ds_partial[tid] = 0.f;
    return;
  }

  const int hi = min(q0 + kTile - 1, len - 1);
  const int lo = a.window ? max(0, q0 - a.window + 1) : 0;
  const int t_first = lo / kTile;
  const int nt = hi / kTile - t_first + 1;

  const uint32_t bar_q = smem_u32(&sm->bar_q), bar_s = smem_u32(&sm->bar_s), bar_p = smem_u32(&sm->bar_p),
                 bar_o = smem_u32(&sm->bar_o);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kDqStages; ++s) mbar_init(smem_u32(&sm->bar_kv[s]), 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kComputeThreads);
    mbar_init(bar_o, 1);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDqTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dq = tmem + 256;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      prefetch_tmap(&tm_do);
      mbar_arrive_expect_tx(bar_q, 2 * kTileBytes);
      tma_load_4d(smem_u32(sm->q), &tm_q, bar_q, 0, q0, h, b);
      tma_load_4d(smem_u32(sm->d_o), &tm_do, bar_q, 0, q0, h, b);
      const int pre = nt < kDqStages ? nt : kDqStages;
      for (int s = 0; s < pre; ++s) {
        const int kv0 = (t_first + s) * kTile;
        mbar_arrive_expect_tx(smem_u32(&sm->bar_kv[s]), 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->k[s]), &tm_k, smem_u32(&sm->bar_kv[s]), 0, kv0, g, b);
        tma_load_4d(smem_u32(sm->v[s]), &tm_v, smem_u32(&sm->bar_kv[s]), 0, kv0, g, b);
      }
      const uint32_t idesc_nt = make_idesc_bf16(kTile, kTile, 0, 0);      // A, B both K-contiguous
      const uint32_t idesc_dq = make_idesc_bf16(kTile, kHeadDim, 0, 1);   // A in TMEM, B = K read N-contiguous
      const uint64_t q_desc = desc_kmajor(smem_u32(sm->q));
      const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o));
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      int issued = pre, waited = 0;
      for (int t = 0; ok && t < nt; ++t) {
        const int s = t % kDqStages;
        const uint32_t ph = (t / kDqStages) & 1;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_kv[s]), ph, abort_flag))) break;
        waited = t + 1;
        tc_fence_after_sync();
        const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[s]));
        const uint64_t v_desc = desc_kmajor(smem_u32(sm->v[s]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_s, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_nt, kk > 0);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_dp, do_desc + kk * kDescKStepKMajor, v_desc + kk * kDescKStepKMajor, idesc_nt, kk > 0);
        umma_commit(bar_s);
        if (!(ok = mbar_wait(bar_p, t & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k[s]));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(tmem_dq, tmem_s + kk * 8, kt_desc + kk * kDescKStepMNMajor, idesc_dq, (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar_o);
        if (t + kDqStages < nt) {
          if (!(ok = mbar_wait(bar_o, t & 1, abort_flag))) break;
          const int kv0 = (t_first + t + kDqStages) * kTile;
          mbar_arrive_expect_tx(smem_u32(&sm->bar_kv[s]), 2 * kTileBytes);
          tma_load_4d(smem_u32(sm->k[s]), &tm_k, smem_u32(&sm->bar_kv[s]), 0, kv0, g, b);
          tma_load_4d(smem_u32(sm->v[s]), &tm_v, smem_u32(&sm->bar_kv[s]), 0, kv0, g, b);
          ++issued;
        }
      }
      if (!ok) {
        report_abort(a);
        mbar_wait_drain(bar_q, 0);
        for (int t = waited; t < issued; ++t)
          mbar_wait_drain(smem_u32(&sm->bar_kv[t % kDqStages]), (t / kDqStages) & 1);
      }
    }
    __syncwarp();
  } else {
    const int i = q0 + tid;
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;
    const long long row_off = ((long long)(b * a.Hq + h)) * a.S_pad + i;
    const float neg_lse2 = -a.lse[row_off] * kLog2e;
    const float delta = a.delta[row_off];
    float pdp = 0.f;  // sum_j P_ij dP_ij in fp32
    bool ok = true;
    uint32_t rs[32], rp[32];

    for (int t = 0; t < nt; ++t) {
      const int kv0 = (t_first + t) * kTile;
      const bool need_mask = tile_needs_mask(q0, kv0, a.window, len);
      if (!(ok = warp_all(mbar_wait(bar_s, t & 1, abort_flag)))) break;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(tmem_s + lane_addr + c * 32, rs);
        tmem_ld32(tmem_dp + lane_addr + c * 32, rp);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(rs[e]), a.scale_log2, neg_lse2));
          float p1 = fast_exp2(fmaf(__uint_as_float(rs[e + 1]), a.scale_log2, neg_lse2));
          if (need_mask) {
            if (!visible(i, kv0 + c * 32 + e, a.window, len)) p0 = 0.f;
            if (!visible(i, kv0 + c * 32 + e + 1, a.window, len)) p1 = 0.f;
          }
          pdp = fmaf(p0, __uint_as_float(rp[e]), pdp);
          pdp = fmaf(p1, __uint_as_float(rp[e + 1]), pdp);
          const float ds0 = p0 * (__uint_as_float(rp[e]) - delta);
          const float ds1 = p1 * (__uint_as_float(rp[e + 1]) - delta);
          pk[e >> 1] = pack_bf16(ds0, ds1);
        }
        // dS chunk c overwrites columns [16c, 16c+16) of S, which this thread has consumed
        tmem_st16(tmem_s + lane_addr + c * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
    }

    if (ok) ok = warp_all(mbar_wait(bar_o, (nt - 1) & 1, abort_flag));
    if (ok) {
      // sink gradient of this warp's 32 rows (fixed-order shuffle tree)
      float dsk = (i < len) ? -fast_exp2(fmaf(a.sinks[h], kLog2e, neg_lse2)) * pdp : 0.f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dsk += __shfl_xor_sync(0xffffffffu, dsk, off);
      if (lane == 0) ds_partial[warp] = dsk;
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
    tmem_dealloc(tmem, kDqTmemCols);
  }
}

}  // namespace b200attn
