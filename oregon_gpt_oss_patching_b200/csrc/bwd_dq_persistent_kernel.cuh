// Persistent dQ kernel for sm_100a, for layers whose query tiles see only a few key tiles
// (narrow sliding windows).
//
// Same arithmetic as the dQ kernel for long items (bwd_dq_kernel.cuh): per 128-key tile
//     S = Q K^T,  dP = dO V^T  (N = 128);   P = 2^(S*scale*log2e - LSE*log2e),  dS = P * (dP - delta);
//     dQ += dS K  (N = 64);   sum_j P*dP per row for the sink gradient.
// With two key tiles per query tile a CTA per work item spends most of its life filling and
// draining its pipeline, so here the grid is one CTA per SM and every CTA walks the work items
// (query tile, head, batch) in snake order; barriers, tensor memory and the TMA rings are set up
// once and run on across item boundaries:
//   * warp 9 streams Q/dO (double-buffered) and K/V tiles (3-stage ring) by TMA and runs ahead;
//   * warp 8 issues the S/dP MMAs (operands from shared memory), warp 10 the dQ MMAs;
//   * dS and dQ are double-buffered in tensor memory, so the dQ MMAs of an item never wait for the
//     previous item's epilogue, and the compute warpgroups run that epilogue (read dQ, scale, store,
//     sink-gradient partial) after the first key tile of the NEXT item, when the MMAs it has to wait
//     for have long retired.
// Every wait is bounded.
#pragma once
#include "attn_common.cuh"
#include "bwd_dkdv_kernel.cuh"  // setmaxnreg helpers
#include "bwd_dq_kernel.cuh"    // dq_compute_chunk

namespace b200attn {

constexpr int kDqpStages = 3;
constexpr int kDqpThreads = 384;
constexpr int kDqpTmemCols = 512;
// tensor-memory columns: S [0,128)  dP [128,256)  dS bf16, two buffers [256,320) [320,384)  dQ, two buffers [384,448) [448,512)

struct DqpSmem {
  alignas(1024) uint8_t q[2][kTileBytes];     // [buffer]: the next work item's Q and dO land while this one runs
  alignas(1024) uint8_t d_o[2][kTileBytes];
  alignas(1024) uint8_t k[kDqpStages][kTileBytes];
  alignas(1024) uint8_t v[kDqpStages][kTileBytes];
  alignas(8) uint64_t bar_q_full[2];       // Q and dO of a buffer landed
  uint64_t bar_q_empty[2];                 // the S/dP MMAs reading a buffer retired  (tcgen05.commit)
  uint64_t bar_in_full[kDqpStages];        // K and V tile of a stage landed
  uint64_t bar_in_empty[kDqpStages];       // the dQ MMAs reading a stage retired     (tcgen05.commit)
  uint64_t bar_s_full;                     // S and dP ready                 (tcgen05.commit)
  uint64_t bar_s_free;                     // S and dP are in registers      (256 arrivals)
  uint64_t bar_p_full[2];                  // a dS buffer written            (256 arrivals); one barrier per buffer,
                                           // so that the writers can never complete two phases unobserved
  uint64_t bar_p_free[2];                  // the dQ MMAs have read a dS buffer       (tcgen05.commit)
  uint64_t bar_dq_full[2];                 // every MMA into a dQ buffer retired      (tcgen05.commit)
  uint64_t bar_dq_free[2];                 // a dQ buffer read by the epilogue        (256 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;                        // K/V tile loads issued so far (for the abort drain)
  int q_loads_issued;                      // Q/dO loads (work items) issued so far
};

struct DqpItem {
  int b, h, g, qt, q0, len, kt_first, nt;   // nt = visible key tiles; 0 = the tile is padding only
};
struct DqpDivs {   // divisors of the item decode, prepared once per thread
  FastDiv per_qt, hq, group;
};
__device__ __forceinline__ DqpItem dqp_item(const KernelArgs& a, int id, const DqpDivs& dv) {
  DqpItem it;
  int q_idx, rem, g_rem;
  fast_divmod(id, dv.per_qt, q_idx, rem);
  it.qt = a.S_pad / kTile - 1 - q_idx;   // long (late) query tiles first; neighbouring ids share K/V in L2
  fast_divmod(rem, dv.hq, it.b, it.h);
  fast_divmod(it.h, dv.group, it.g, g_rem);
  it.q0 = it.qt * kTile;
  it.len = seq_len(a, it.b);
  if (it.q0 >= it.len) {
    it.kt_first = 0;
    it.nt = 0;
  } else {
    const int hi = min(it.q0 + kTile - 1, it.len - 1);              // last visible key
    const int lo = a.window ? max(0, it.q0 - a.window + 1) : 0;     // first visible key
    it.kt_first = lo / kTile;
    it.nt = hi / kTile - it.kt_first + 1;
  }
  return it;
}
// Work item of this CTA's round k: rounds alternate direction, so that with items sorted by
// decreasing length every CTA gets nearly the same total.
__device__ __forceinline__ int dqp_item_id(int k) {
  const int c = (k & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  return k * (int)gridDim.x + c;
}
// first round at or after `k` whose work item exists and has key tiles; false if none
__device__ __forceinline__ bool dqp_next_item(const KernelArgs& a, int& k, int n_items, int n_rounds, const DqpDivs& dv,
                                              DqpItem& it) {
  for (; k < n_rounds; ++k) {
    const int id = dqp_item_id(k);
    if (id >= n_items) continue;
    it = dqp_item(a, id, dv);
    if (it.nt > 0) return true;
  }
  return false;
}

__global__ void __launch_bounds__(kDqpThreads, 1)
attn_bwd_dq_persistent_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                              const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                              const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DqpSmem* sm = reinterpret_cast<DqpSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_items = (a.S_pad / kTile) * a.B * a.Hq;
  const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  const DqpDivs dv{make_fastdiv(a.B * a.Hq), make_fastdiv(a.Hq), make_fastdiv(a.group)};
  const float* nlse_base = a.delta + (long long)a.B * a.Hq * a.S_pad;  // plane 1 of the delta scratch

  const uint32_t bar_s_full = smem_u32(&sm->bar_s_full), bar_s_free = smem_u32(&sm->bar_s_free);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int q = 0; q < 2; ++q) {
      mbar_init(smem_u32(&sm->bar_q_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_q_empty[q]), 1);
      mbar_init(smem_u32(&sm->bar_p_full[q]), 2 * kComputeThreads);
      mbar_init(smem_u32(&sm->bar_p_free[q]), 1);
      mbar_init(smem_u32(&sm->bar_dq_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_dq_free[q]), 2 * kComputeThreads);
    }
    for (int s = 0; s < kDqpStages; ++s) {
      mbar_init(smem_u32(&sm->bar_in_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_in_empty[s]), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, 2 * kComputeThreads);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    sm->q_loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDqpTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_ds = tmem + 256, tmem_dq = tmem + 384;

  if (warp >= 8) {
  setmaxnreg_dec_72();
  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      int kq = 0;   // work items with key tiles so far (Q/dO buffer = kq & 1)
      int T = 0;    // key tiles so far (stage = T % kDqpStages)
      bool ok = true;
      DqpItem it;
      for (int k = 0; ok && dqp_next_item(a, k, n_items, n_rounds, dv, it); ++k, ++kq) {
        const int qb = kq & 1;
        if (kq >= 2 && !(ok = mbar_wait(smem_u32(&sm->bar_q_empty[qb]), ((kq >> 1) - 1) & 1, abort_flag))) break;
        const uint32_t bar_q = smem_u32(&sm->bar_q_full[qb]);
        mbar_arrive_expect_tx(bar_q, 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->q[qb]), &tm_q, bar_q, 0, it.q0, it.h, it.b);       // rows past the end arrive as zeros
        tma_load_4d(smem_u32(sm->d_o[qb]), &tm_do, bar_q, 0, it.q0, it.h, it.b);
        *reinterpret_cast<volatile int*>(&sm->q_loads_issued) = kq + 1;
        for (int t = 0; t < it.nt; ++t, ++T) {
          const int s = T % kDqpStages;
          if (T >= kDqpStages && !(ok = mbar_wait(smem_u32(&sm->bar_in_empty[s]), ((T / kDqpStages) - 1) & 1, abort_flag))) break;
          const int kv0 = (it.kt_first + t) * kTile;
          const uint32_t bar = smem_u32(&sm->bar_in_full[s]);
          mbar_arrive_expect_tx(bar, 2 * kTileBytes);
          tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, kv0, it.g, it.b);
          tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, kv0, it.g, it.b);
          *reinterpret_cast<volatile int*>(&sm->loads_issued) = T + 1;
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------- MMA issuer, S and dP (front) -------------------------
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kTile, 0, 0);    // A, B both K-contiguous, N = 128
      int kq = 0, T = 0;
      bool ok = true;
      DqpItem it;
      for (int k = 0; ok && dqp_next_item(a, k, n_items, n_rounds, dv, it); ++k, ++kq) {
        const int qb = kq & 1;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_q_full[qb]), (kq >> 1) & 1, abort_flag))) break;
        const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[qb]));
        const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o[qb]));
        for (int t = 0; t < it.nt; ++t, ++T) {
          // the stage has landed and the previous tile's S/dP are in registers
          const int s = T % kDqpStages;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_in_full[s]), (T / kDqpStages) & 1, abort_flag))) break;
          if (T > 0 && !(ok = mbar_wait(bar_s_free, (T - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[s]));
          const uint64_t v_desc = desc_kmajor(smem_u32(sm->v[s]));
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_s, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_dp, do_desc + kk * kDescKStepKMajor, v_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
          umma_commit(bar_s_full);
          if (t == it.nt - 1) umma_commit(smem_u32(&sm->bar_q_empty[qb]));   // Q/dO buffer free once these retire
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------ MMA issuer, dQ (back) ------------------------------
    if (lane == 0) {
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      int kq = 0, T = 0;
      bool ok = true;
      DqpItem it;
      for (int k = 0; ok && dqp_next_item(a, k, n_items, n_rounds, dv, it); ++k, ++kq) {
        const uint32_t dq = tmem_dq + (kq & 1) * 64;
        for (int t = 0; t < it.nt; ++t, ++T) {
          if (!(ok = mbar_wait(smem_u32(&sm->bar_p_full[T & 1]), (T >> 1) & 1, abort_flag))) break;   // dS of the tile written
          // the first dQ MMA of an item overwrites its dQ buffer: the epilogue of the item before the
          // previous one must have read it
          if (t == 0 && kq >= 2 && !(ok = mbar_wait(smem_u32(&sm->bar_dq_free[kq & 1]), ((kq >> 1) - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const int s = T % kDqpStages;
          const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k[s]));
          const uint32_t ds = tmem_ds + (T & 1) * 64;
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ts(dq, ds + kk * 8, kt_desc + kk * kDescKStepMNMajor, idesc_back, (t > 0 || kk > 0) ? 1u : 0u);
          umma_commit(smem_u32(&sm->bar_p_free[T & 1]));   // the dS buffer is reusable once these retire
          umma_commit(smem_u32(&sm->bar_in_empty[s]));     // and so is the K/V stage (its S/dP MMAs retired before dS was written)
          if (t == it.nt - 1) umma_commit(smem_u32(&sm->bar_dq_full[kq & 1]));
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216();
  {
    // ------------------------------------- compute --------------------------------------
    const int wg = warp >> 2;             // which 64 key columns of every tile
    const int r = tid & 127;
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
    int kq = 0, T = 0;
    bool ok = true;

    // next round at or after k with key tiles; padding-only items met on the way get their outputs here
    auto scan = [&](int& k, DqpItem& it) -> bool {
      for (; k < n_rounds; ++k) {
        const int id = dqp_item_id(k);
        if (id >= n_items) continue;
        it = dqp_item(a, id, dv);
        if (it.nt > 0) return true;
        if (tid < kComputeThreads && it.q0 + tid < a.S) zero_row(a.dq.row(it.b, it.h, it.q0 + tid));   // dQ rows are zero,
        if (tid < 8) a.dsinks_partial[(((long long)it.h * a.B + it.b) * (a.S_pad / kTile) + it.qt) * 8 + tid] = 0.f;  // no sink gradient
      }
      return false;
    };

    // The epilogue of a work item runs after the first key tile of the next one (see the file comment).
    bool pending = false;
    int p_b = 0, p_h = 0, p_qt = 0, p_len = 0, p_kq = 0;
    float p_nl2 = 0.f, p_pdp = 0.f;
    auto epilogue = [&]() -> bool {
      if (!warp_all(mbar_wait(smem_u32(&sm->bar_dq_full[p_kq & 1]), (p_kq >> 1) & 1, abort_flag))) return false;
      // warpgroup 0 stores dQ columns 0-31, warpgroup 1 columns 32-63
      tc_fence_after_sync();
      uint32_t r0[32];
      tmem_ld32(tmem_dq + (p_kq & 1) * 64 + lane_addr + wg * 32, r0);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->bar_dq_free[p_kq & 1]));   // the item after the next may overwrite this dQ buffer
      const int i = p_qt * kTile + r;
      // sink gradient of this warp's 32 rows for this warpgroup's key columns (fixed-order shuffle tree)
      float dsk = (i < p_len) ? -fast_exp2(fmaf(a.sinks[p_h], kLog2e, p_nl2)) * p_pdp : 0.f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dsk += __shfl_xor_sync(0xffffffffu, dsk, off);
      if (lane == 0) a.dsinks_partial[(((long long)p_h * a.B + p_b) * (a.S_pad / kTile) + p_qt) * 8 + warp] = dsk;
      if (i < a.S) {
        __nv_bfloat16* dst = a.dq.row(p_b, p_h, i) + wg * 32;
        const float sc = (i < p_len) ? a.scale : 0.f;
#pragma unroll
        for (int c = 0; c < 32; c += 8)
          store_bf16x8(dst + c, pack_bf16(__uint_as_float(r0[c]) * sc, __uint_as_float(r0[c + 1]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 2]) * sc, __uint_as_float(r0[c + 3]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 4]) * sc, __uint_as_float(r0[c + 5]) * sc),
                       pack_bf16(__uint_as_float(r0[c + 6]) * sc, __uint_as_float(r0[c + 7]) * sc));
      }
      return true;
    };

    DqpItem cur, nxt;
    int k = 0;
    bool have = scan(k, cur);
    float nl2 = 0.f, delta = 0.f;   // -LSE * log2(e) and delta of this thread's row
    if (have) {
      const long long row_off = ((long long)(cur.b * a.Hq + cur.h)) * a.S_pad + cur.q0 + r;
      nl2 = nlse_base[row_off];
      delta = a.delta[row_off];
    }
    while (ok && have) {
      int k_n = k + 1;
      const bool have_n = scan(k_n, nxt);
      float nl2_n = 0.f, delta_n = 0.f;   // the next item's row constants: in flight under this item's work
      if (have_n) {
        const long long row_off = ((long long)(nxt.b * a.Hq + nxt.h)) * a.S_pad + nxt.q0 + r;
        nl2_n = nlse_base[row_off];
        delta_n = a.delta[row_off];
      }
      const int i = cur.q0 + r;           // this thread's query position
      const float2 nl22 = make_float2(nl2, nl2), neg_delta2 = make_float2(-delta, -delta);
      float2 acc = make_float2(0.f, 0.f);   // this warpgroup's share of sum_j P_ij dP_ij, two lanes

      for (int t = 0; t < cur.nt; ++t, ++T) {
        const int j0 = (cur.kt_first + t) * kTile + wg * 64;  // first key column of this thread
        const bool need_mask = (j0 + 63 > cur.q0) || (a.window != 0 && j0 <= cur.q0 + kTile - 1 - a.window) || (cur.q0 + kTile > cur.len);
        if (!(ok = warp_all(mbar_wait(bar_s_full, T & 1, abort_flag)))) break;
        tc_fence_after_sync();
        uint32_t rs[2][32], rp[2][32];
        tmem_ld32(tmem_s + lane_addr + wg * 64, rs[0]);
        tmem_ld32(tmem_dp + lane_addr + wg * 64, rp[0]);
        tmem_ld32(tmem_s + lane_addr + wg * 64 + 32, rs[1]);
        tmem_ld32(tmem_dp + lane_addr + wg * 64 + 32, rp[1]);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(bar_s_free);  // S/dP columns may be overwritten by the next tile
        uint32_t pk[2][16];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          // every 32-key chunk is classified for the whole warp: visible to all rows, to none (dS = 0
          // without a single exponential -- half the chunks of a window-128 layer), or mixed
          const uint32_t bits = need_mask ? visible_keys32(i, j0 + c * 32, a.window, cur.len) : 0xffffffffu;
          if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[c][e] = 0u;
          } else if (__all_sync(0xffffffffu, bits == 0xffffffffu)) {
            dq_compute_chunk<false>(rs[c], rp[c], scale2, nl22, neg_delta2, bits, pk[c], acc);
          } else {
            dq_compute_chunk<true>(rs[c], rp[c], scale2, nl22, neg_delta2, bits, pk[c], acc);
          }
        }
        // the dQ MMAs of the tile before the previous one must have left this dS buffer (long done)
        if (T >= 2 && !(ok = warp_all(mbar_wait(smem_u32(&sm->bar_p_free[T & 1]), ((T >> 1) - 1) & 1, abort_flag)))) break;
        tc_fence_after_sync();
        const uint32_t ds = tmem_ds + (T & 1) * 64 + lane_addr + wg * 32;
        tmem_st16(ds, pk[0]);
        tmem_st16(ds + 16, pk[1]);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(smem_u32(&sm->bar_p_full[T & 1]));
        if (pending) {   // (only at t == 0) the previous item's epilogue, its MMAs long retired
          if (!(ok = epilogue())) break;
          pending = false;
        }
      }
      if (!ok) break;
      pending = true;
      p_b = cur.b; p_h = cur.h; p_qt = cur.qt; p_len = cur.len; p_kq = kq;
      p_nl2 = nl2;
      p_pdp = acc.x + acc.y;
      cur = nxt;
      k = k_n;
      have = have_n;
      nl2 = nl2_n;
      delta = delta_n;
      ++kq;
    }
    if (ok && pending) ok = epilogue();
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kDqpTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued, q_issued = sm->q_loads_issued;
    for (int k = max(0, q_issued - 2); k < q_issued; ++k) mbar_wait_drain(smem_u32(&sm->bar_q_full[k & 1]), (k >> 1) & 1);
    for (int it = max(0, issued - kDqpStages); it < issued; ++it)
      mbar_wait_drain(smem_u32(&sm->bar_in_full[it % kDqpStages]), (it / kDqpStages) & 1);
  }
}

}  // namespace b200attn
