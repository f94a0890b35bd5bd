// dQ kernel for sm_100a.
//
// One CTA = one 128-row query tile of one query head of one sequence; it streams the 128-key
// tiles that query tile can see.  Per item (one key tile), on tcgen05 with accumulators in
// tensor memory:
//     S  = Q K^T          dP = dO V^T                          (N = 128)
// then with one thread per query row
//     P  = 2^(S*scale*log2e - LSE*log2e)      dS = P * (dP - delta)
// dS goes to tensor memory as bf16 and is the A operand of
//     dQ += dS K          (N = 64, accumulated in tensor memory over all key tiles)
// and the epilogue stores dQ * scale.  This is the dq part of the reference's `_attn_bwd`
// (attention_kernel.py:190-199, :206-207, :214-217).
//
// The same pass yields the sink gradient.  Because the softmax row (sink column included)
// sums to one,  sum_j P_ij dP_ij  equals delta_i exactly, so each thread also accumulates that
// sum in fp32 from the recomputed P and dP -- it does not inherit the bf16 rounding of the
// stored O that delta = rowsum(dO*O) carries -- and the CTA writes, per warp,
//     - sum_i exp(sink - LSE_i) * (sum_j P_ij dP_ij)
// to the dSinks scratch (the reference's per-tile term, attention_kernel.py:173-175).
//
// Q and dO (the A operands of S and dP for the CTA's whole life) are copied once into tensor
// memory as bf16, so those MMAs read only the K/V tile from shared memory.  Pipeline as in the
// dK/dV kernel: warp 9 streams K/V tiles through a 4-stage TMA ring, warp 8 issues the S/dP MMAs
// and warp 10 the dQ MMAs, the two compute warpgroups split the 128 key columns of an
// item, pull their half of S/dP into registers and release those columns at once (the tensor
// core computes the next item's S/dP under this item's exponentials), and write dS to its own
// columns once the previous item's dQ MMAs have left them.  Every wait is bounded.
#pragma once
#include "attn_common.cuh"
#include "bwd_dkdv_kernel.cuh"  // setmaxnreg helpers

namespace b200attn {

constexpr int kDqStages = 4;
constexpr int kDqThreads = 384;
constexpr int kDqTmemCols = 512;
// tensor-memory columns: S [0,128)  dP [128,256)  dS bf16 [256,320) and [448,512) (two buffers)  Q bf16 [320,352)
//                        dO bf16 [352,384)  dQ [384,448)

struct DqSmem {
  alignas(1024) uint8_t k[kDqStages][kTileBytes];
  alignas(1024) uint8_t v[kDqStages][kTileBytes];
  alignas(8) uint64_t bar_q;               // Q and dO copied into tensor memory (256 arrivals)
  uint64_t bar_in_full[kDqStages];         // K and V tile of a stage landed
  uint64_t bar_in_empty[kDqStages];        // the dQ MMAs reading a stage retired
  uint64_t bar_s_full;                     // S and dP ready                 (tcgen05.commit)
  uint64_t bar_s_free;                     // S and dP are in registers      (256 arrivals)
  uint64_t bar_p_full[2];                  // a dS buffer written            (256 arrivals); one barrier per buffer,
                                           // so that the writers can never complete two phases unobserved
  uint64_t bar_p_free[2];                  // the dQ MMAs have read a dS buffer   (tcgen05.commit)
  uint64_t bar_acc;                        // every MMA retired: dQ final
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;
};

// dS (bf16 pairs) of 32 key columns for one query row from S/dP in registers; adds P*dP to acc.
// Two elements per instruction (packed fp32 pairs): the special-function unit, not the issue
// slots, should be what the row waits for -- the MMA-issuing warps live on the slots left over.
template <bool kSelect>
__device__ __forceinline__ void dq_compute_chunk(const uint32_t (&rs)[32], const uint32_t (&rp)[32], float2 scale2, float2 nl22,
                                                 float2 neg_delta2, uint32_t bits, uint32_t (&pk)[16], float2& acc) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    const float2 x = __ffma2_rn(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), scale2, nl22);
    float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
    if (kSelect) {  // selects, not branches
      p.x = (bits >> e) & 1u ? p.x : 0.f;
      p.y = (bits >> (e + 1)) & 1u ? p.y : 0.f;
    }
    const float2 dp = make_float2(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1]));
    acc = __ffma2_rn(p, dp, acc);
    const float2 ds = __fmul2_rn(p, __fadd2_rn(dp, neg_delta2));
    pk[e >> 1] = pack_bf16(ds.x, ds.y);
  }
}

// dS of 64 key columns for one query row; adds sum_j P*dP to pdp.
template <bool kMask>
__device__ __forceinline__ void dq_compute(const uint32_t (&rs)[2][32], const uint32_t (&rp)[2][32], float scale_log2,
                                           float nl2, float delta, int i, int j0, int window, int len,
                                           uint32_t (&pk)[2][16], float& pdp) {
  float2 acc = make_float2(0.f, 0.f);
  const float2 scale2 = make_float2(scale_log2, scale_log2), nl22 = make_float2(nl2, nl2);
  const float2 neg_delta2 = make_float2(-delta, -delta);
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const uint32_t bits = kMask ? visible_keys32(i, j0 + c * 32, window, len) : 0xffffffffu;
    dq_compute_chunk<kMask>(rs[c], rp[c], scale2, nl22, neg_delta2, bits, pk[c], acc);
  }
  pdp += acc.x + acc.y;
}

__global__ void __launch_bounds__(kDqThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem* sm = reinterpret_cast<DqSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / a.group;
  const int qt = gridDim.x - 1 - blockIdx.x;  // long (late) tiles first
  const int q0 = qt * kTile;
  const int len = seq_len(a, b);

  // eight per-warp sink-gradient partials per query tile
  float* ds_partial = a.dsinks_partial + (((long long)h * a.B + b) * (a.S_pad / kTile) + qt) * 8;
  if (q0 >= len) {  // padding only: dQ rows are zero, no sink gradient
    if (tid < kComputeThreads && q0 + tid < a.S) zero_row(a.dq.row(b, h, q0 + tid));
    if (tid < 8) ds_partial[tid] = 0.f;
    return;
  }

  const int hi = min(q0 + kTile - 1, len - 1);              // last visible key
  const int lo = a.window ? max(0, q0 - a.window + 1) : 0;  // first visible key
  const int kt_first = lo / kTile;
  const int n_items = hi / kTile - kt_first + 1;
  const float* nlse_base = a.delta + (long long)a.B * a.Hq * a.S_pad;  // second half of the delta scratch

  const uint32_t bar_q = smem_u32(&sm->bar_q), bar_acc = smem_u32(&sm->bar_acc), bar_s_full = smem_u32(&sm->bar_s_full),
                 bar_s_free = smem_u32(&sm->bar_s_free);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_q, 2 * kComputeThreads);
    for (int s = 0; s < kDqStages; ++s) {
      mbar_init(smem_u32(&sm->bar_in_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_in_empty[s]), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, 2 * kComputeThreads);
    for (int q = 0; q < 2; ++q) {
      mbar_init(smem_u32(&sm->bar_p_full[q]), 2 * kComputeThreads);
      mbar_init(smem_u32(&sm->bar_p_free[q]), 1);
    }
    mbar_init(bar_acc, 1);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDqTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_ds = tmem + 256, tmem_ds1 = tmem + 448, tmem_q = tmem + 320, tmem_do = tmem + 352,
                 tmem_dq = tmem + 384;

  if (warp >= 8) {
  setmaxnreg_dec_72();
  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      for (int it = 0; it < n_items; ++it) {
        const int s = it % kDqStages;
        if (it >= kDqStages && !mbar_wait(smem_u32(&sm->bar_in_empty[s]), ((it / kDqStages) - 1) & 1, abort_flag)) {
          report_abort(a);
          break;
        }
        const int kv0 = (kt_first + it) * kTile;
        const uint32_t bar = smem_u32(&sm->bar_in_full[s]);
        mbar_arrive_expect_tx(bar, 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, kv0, g, b);
        tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, kv0, g, b);
        *reinterpret_cast<volatile int*>(&sm->loads_issued) = it + 1;
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------- MMA issuer, S and dP (front) -------------------------
    // tcgen05.mma issue is synchronous with the tensor pipe, and an issuing warp gets few issue
    // slots next to busy compute warps: front and back MMAs have an issuing warp each, on different
    // SM sub-partitions, so that neither waits behind the other's issue.
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kTile, 0, 0);    // A in TMEM, B K-contiguous, N = 128
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      for (int it = 0; ok && it < n_items; ++it) {
        // the stage has landed and the previous item's S/dP are in registers
        const int s = it % kDqStages;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_in_full[s]), (it / kDqStages) & 1, abort_flag))) break;
        if (it > 0 && !(ok = mbar_wait(bar_s_free, (it - 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[s]));
        const uint64_t v_desc = desc_kmajor(smem_u32(sm->v[s]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ts(tmem_s, tmem_q + kk * 8, k_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ts(tmem_dp, tmem_do + kk * 8, v_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
        umma_commit(bar_s_full);
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------ MMA issuer, dQ (back) ------------------------------
    if (lane == 0) {
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      bool ok = true;
      for (int it = 0; ok && it < n_items; ++it) {
        if (!(ok = mbar_wait(smem_u32(&sm->bar_p_full[it & 1]), (it >> 1) & 1, abort_flag))) break;   // dS of the item has been written
        tc_fence_after_sync();
        const int s = it % kDqStages;
        const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k[s]));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(tmem_dq, ((it & 1) ? tmem_ds1 : tmem_ds) + kk * 8, kt_desc + kk * kDescKStepMNMajor, idesc_back, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&sm->bar_p_free[it & 1]));   // the dS buffer is reusable once these retire
        umma_commit(smem_u32(&sm->bar_in_empty[s]));  // and so is the K/V stage (its S/dP MMAs retired before dS was written)
        if (it == n_items - 1) umma_commit(bar_acc);
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216();
  {
    // ------------------------------------- compute --------------------------------------
    const int wg = warp >> 2;             // which 64 key columns of every item
    const int r = tid & 127;
    const int i = q0 + r;                 // this thread's query position
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    const long long row_off = ((long long)(b * a.Hq + h)) * a.S_pad + i;
    const float nl2 = nlse_base[row_off];  // -LSE * log2(e)
    const float delta = a.delta[row_off];
    float pdp = 0.f;                       // this warpgroup's share of sum_j P_ij dP_ij
    bool ok = true;

    {  // copy this thread's row of Q (warpgroup 0) or dO (warpgroup 1) into tensor memory as bf16
      uint32_t w[32];
      if (i < a.S) {
        const uint4* row = reinterpret_cast<const uint4*>(wg == 0 ? a.q.row(b, h, i) : a.d_o.row(b, h, i));
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 x = row[c];
          w[4 * c] = x.x; w[4 * c + 1] = x.y; w[4 * c + 2] = x.z; w[4 * c + 3] = x.w;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) w[c] = 0u;
      }
      tmem_st32((wg == 0 ? tmem_q : tmem_do) + lane_addr, w);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_q);
    }

    bool s_ready = false;
    for (int it = 0; it < n_items; ++it) {
      const int j0 = (kt_first + it) * kTile + wg * 64;  // first key column of this thread
      const bool need_mask = (j0 + 63 > q0) || (a.window != 0 && j0 <= q0 + kTile - 1 - a.window) || (q0 + kTile > len);
      // (the phase was already tested at the end of the previous item, under its stores: a barrier
      // test costs ~100 cycles even when the phase is complete)
      if (!warp_all(s_ready) && !(ok = warp_all(mbar_wait(bar_s_full, it & 1, abort_flag)))) break;
      tc_fence_after_sync();
      uint32_t rs[2][32], rp[2][32];
      tmem_ld32(tmem_s + lane_addr + wg * 64, rs[0]);
      tmem_ld32(tmem_dp + lane_addr + wg * 64, rp[0]);
      tmem_ld32(tmem_s + lane_addr + wg * 64 + 32, rs[1]);
      tmem_ld32(tmem_dp + lane_addr + wg * 64 + 32, rp[1]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bar_s_free);  // S/dP columns may be overwritten by the next item
      // the dQ MMAs of the item before the previous one have long left this dS buffer: ask now, the
      // answer arrives under the exponentials
      const uint32_t bar_pf = smem_u32(&sm->bar_p_free[it & 1]);
      const bool p_free = it < 2 || mbar_test_wait(bar_pf, ((it >> 1) - 1) & 1);
      uint32_t pk[2][16];
      if (need_mask) dq_compute<true>(rs, rp, a.scale_log2, nl2, delta, i, j0, a.window, len, pk, pdp);
      else dq_compute<false>(rs, rp, a.scale_log2, nl2, delta, i, j0, a.window, len, pk, pdp);
      // the dQ MMAs of the item before the previous one must have left this dS buffer (asked above)
      if (!warp_all(p_free) && !(ok = warp_all(mbar_wait(bar_pf, ((it >> 1) - 1) & 1, abort_flag)))) break;
      tc_fence_after_sync();
      const uint32_t ds = ((it & 1) ? tmem_ds1 : tmem_ds) + lane_addr + wg * 32;
      tmem_st16(ds, pk[0]);
      tmem_st16(ds + 16, pk[1]);
      s_ready = it + 1 < n_items && mbar_test_wait(bar_s_full, (it + 1) & 1);   // answered under the stores
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->bar_p_full[it & 1]));
    }

    if (ok) ok = warp_all(mbar_wait(bar_acc, 0, abort_flag));
    if (ok) {
      // sink gradient of this warp's 32 rows for this warpgroup's key columns (fixed-order shuffle tree)
      float dsk = (i < len) ? -fast_exp2(fmaf(a.sinks[h], kLog2e, nl2)) * pdp : 0.f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dsk += __shfl_xor_sync(0xffffffffu, dsk, off);
      if (lane == 0) ds_partial[warp] = dsk;
      // warpgroup 0 stores dQ columns 0-31, warpgroup 1 columns 32-63
      tc_fence_after_sync();
      uint32_t r0[32];
      tmem_ld32(tmem_dq + lane_addr + wg * 32, r0);
      tmem_wait_ld();
      if (i < a.S) {
        __nv_bfloat16* dst = a.dq.row(b, h, i) + wg * 32;
        const float sc = (i < len) ? a.scale : 0.f;
#pragma unroll
        for (int c = 0; c < 32; c += 8)
          store_bf16x8(dst + c, pack_bf16(__uint_as_float(r0[c]) * sc, __uint_as_float(r0[c + 1]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 2]) * sc, __uint_as_float(r0[c + 3]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 4]) * sc, __uint_as_float(r0[c + 5]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 6]) * sc, __uint_as_float(r0[c + 7]) * sc));
      }
    }
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kDqTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued;
    for (int it = max(0, issued - kDqStages); it < issued; ++it)
      mbar_wait_drain(smem_u32(&sm->bar_in_full[it % kDqStages]), (it / kDqStages) & 1);
  }
}

}  // namespace b200attn
