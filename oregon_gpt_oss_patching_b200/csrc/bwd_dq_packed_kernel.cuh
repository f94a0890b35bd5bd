// dQ kernel for narrow sliding windows (window <= 128) with a group of 8 query heads per KV head, for
// sm_100a: the GPT-OSS sliding-window layer.  Same tile as the packed forward kernel
// (fwd_packed_kernel.cuh): the 128 accumulator rows are the 8 query heads of a KV group x 16 consecutive
// positions, which see the 144 keys [q0-128, q0+16), so per tile
//     S  = Q K^T,  dP = dO V^T          (M=128, N=144, K=64)   one product each, no second key tile
//     P  = 2^(S*scale*log2e - LSE*log2e),  dS = P * (dP - delta)   (128 of the 144 columns are visible per row)
//     dQ = dS K                          (M=128, N=64, K=144)
// (attention_kernel.py:190-199, :206-207, :214-217 of the reference) and sum_j P dP per row for the sink
// gradient (:173-175), as in bwd_dq_kernel.cuh.
//
// A work item is 32 consecutive positions of one (batch, KV group) = two tiles ("units") that share one
// staged block of K and V rows [q0-128, q0+32).  Persistent, one CTA per SM; consecutive CTAs take
// consecutive position blocks, so neighbouring K/V windows meet in L2.  Pipeline over units:
//   * warp 9 streams Q/dO tiles (double-buffered, one 4-D TMA box {d 64, positions 16, heads 8} each) and
//     K/V blocks (3-stage ring) and runs ahead;
//   * warp 8 issues the S/dP MMAs of unit u+1 as soon as the compute threads hold S/dP of unit u in registers;
//   * the two compute warpgroups split the 144 key columns (72 each), write dS (bf16) to tensor memory;
//   * warp 10 issues the dQ MMAs into one of two dQ accumulators, so they never wait for an epilogue;
//   * the epilogue of unit u (read dQ, scale, sink-gradient partial) runs after the compute of unit u+1, when
//     its MMAs have long retired; dQ rows leave through shared memory and one TMA store (warp 11), because a
//     thread's row is 128 contiguous bytes far from its neighbour's and plain stores of that shape keep the
//     load/store unit busy longer than the arithmetic takes.
// Every wait is bounded.
#pragma once
#include "attn_common.cuh"
#include "bwd_dq_kernel.cuh"        // dq_compute_chunk
#include "fwd_packed_kernel.cuh"    // tile constants, item decode, row masks

namespace b200attn {

constexpr int kDqPkThreads = 384;
constexpr int kDqPkTmemCols = 512;
constexpr int kDqPkHalf = kPkKeys / 2;   // 72 key columns per compute warpgroup
// tensor-memory columns: S [0,144)  dP [144,288)  dS bf16 [288,360)  dQ, two buffers [384,448) [448,512)
constexpr uint32_t kDqPkColDp = 144, kDqPkColDs = 288, kDqPkColDq = 384;
constexpr int kDqPkPartialsPerTile = 16;   // sink-gradient partials per (head, 128 positions): 8 units x 2 warpgroups

struct DqPkSmem {
  alignas(1024) uint8_t q[2][kTileBytes];          // [buffer]: the next unit's Q and dO land while this one runs
  alignas(1024) uint8_t d_o[2][kTileBytes];
  alignas(1024) uint8_t k[kPkStages][kPkKvBytes];
  alignas(1024) uint8_t v[kPkStages][kPkKvBytes];
  alignas(1024) uint8_t out[kTileBytes];           // dQ rows on their way out (TMA store)
  alignas(8) uint64_t bar_q_full[2];       // Q and dO of a buffer landed
  uint64_t bar_q_empty[2];                 // the S/dP MMAs reading a buffer retired          (tcgen05.commit)
  uint64_t bar_kv_full[kPkStages];         // K and V block of an item landed
  uint64_t bar_kv_empty[kPkStages];        // every MMA on a stage retired                     (tcgen05.commit)
  uint64_t bar_s_full;                     // S and dP ready                                   (tcgen05.commit)
  uint64_t bar_s_free;                     // S and dP are in registers                        (256 arrivals)
  uint64_t bar_p_full;                     // dS written                                       (256 arrivals)
  uint64_t bar_p_free;                     // the dQ MMAs have read dS                         (tcgen05.commit)
  uint64_t bar_dq_full[2];                 // the dQ MMAs into a buffer retired                (tcgen05.commit)
  uint64_t bar_dq_free[2];                 // a dQ buffer read by the epilogue                 (256 arrivals)
  uint64_t bar_out_full;                   // dQ rows are in shared memory                     (256 arrivals)
  uint64_t bar_out_free;                   // the TMA store has read them                      (1 arrival)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;                        // items whose K/V loads have been issued (for the abort drain)
  int q_loads_issued;                      // units whose Q/dO loads have been issued
};

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}

// dS of 8 key columns (the tail of a warpgroup's 72) for one query row; adds P*dP to acc.  Always with selects.
__device__ __forceinline__ void dq_compute_chunk8(const uint32_t (&rs)[8], const uint32_t (&rp)[8], float2 scale2, float2 nl22,
                                                  float2 neg_delta2, uint32_t bits, uint32_t (&pk)[4], float2& acc) {
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    const float2 x = __ffma2_rn(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), scale2, nl22);
    float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
    p.x = (bits >> e) & 1u ? p.x : 0.f;
    p.y = (bits >> (e + 1)) & 1u ? p.y : 0.f;
    const float2 dp = make_float2(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1]));
    acc = __ffma2_rn(p, dp, acc);
    const float2 ds = __fmul2_rn(p, __fadd2_rn(dp, neg_delta2));
    pk[e >> 1] = pack_bf16(ds.x, ds.y);
  }
}

__global__ void __launch_bounds__(kDqPkThreads, 1)
attn_bwd_dq_packed_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                          const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          const __grid_constant__ CUtensorMap tm_dq, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DqPkSmem* sm = reinterpret_cast<DqPkSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const PkDivs dv = pk_divs(a);
  const int n_items = dv.n_chunks * a.B * a.Hkv;
  const float* nlse_base = a.delta + (long long)a.B * a.Hq * a.S_pad;  // plane 1 of the delta scratch
  const int units_per_head = a.B * (a.S_pad / kPkPos);                  // sink-gradient partial slots: [head][batch][unit][warpgroup]

  const uint32_t bar_s_full = smem_u32(&sm->bar_s_full), bar_s_free = smem_u32(&sm->bar_s_free),
                 bar_p_full = smem_u32(&sm->bar_p_full), bar_p_free = smem_u32(&sm->bar_p_free),
                 bar_out_full = smem_u32(&sm->bar_out_full), bar_out_free = smem_u32(&sm->bar_out_free);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int q = 0; q < 2; ++q) {
      mbar_init(smem_u32(&sm->bar_q_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_q_empty[q]), 1);
      mbar_init(smem_u32(&sm->bar_dq_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_dq_free[q]), 2 * kComputeThreads);
    }
    for (int s = 0; s < kPkStages; ++s) {
      mbar_init(smem_u32(&sm->bar_kv_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_kv_empty[s]), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, 2 * kComputeThreads);
    mbar_init(bar_p_full, 2 * kComputeThreads);
    mbar_init(bar_p_free, 1);
    mbar_init(bar_out_full, 2 * kComputeThreads);
    mbar_init(bar_out_free, 1);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    sm->q_loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDqPkTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + kDqPkColDp, tmem_ds = tmem + kDqPkColDs, tmem_dq = tmem + kDqPkColDq;

  if (warp >= 8) {
  setmaxnreg_dec_72();
  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      bool ok = true;
      PkItem it;
      int n = 0;   // active items so far (K/V stage = n % kPkStages; units 2n, 2n+1; Q/dO buffer = unit & 1)
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        const int s = n % kPkStages;
        for (int x = 0; x < 2 && ok; ++x) {
          const int u = 2 * n + x, qb = x;
          if (u >= 2 && !(ok = mbar_wait(smem_u32(&sm->bar_q_empty[qb]), ((u >> 1) - 1) & 1, abort_flag))) break;
          const uint32_t bar_q = smem_u32(&sm->bar_q_full[qb]);
          mbar_arrive_expect_tx(bar_q, 2 * kTileBytes);
          tma_load_4d(smem_u32(sm->q[qb]), &tm_q, bar_q, 0, it.q0 + x * kPkPos, it.g * kPkHeads, it.b);      // rows past the end arrive as zeros
          tma_load_4d(smem_u32(sm->d_o[qb]), &tm_do, bar_q, 0, it.q0 + x * kPkPos, it.g * kPkHeads, it.b);
          *reinterpret_cast<volatile int*>(&sm->q_loads_issued) = u + 1;
          if (x == 0) {
            if (n >= kPkStages && !(ok = mbar_wait(smem_u32(&sm->bar_kv_empty[s]), ((n / kPkStages) - 1) & 1, abort_flag))) break;
            const uint32_t bar = smem_u32(&sm->bar_kv_full[s]);
            mbar_arrive_expect_tx(bar, 2 * kPkKvBytes);
            tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, it.q0 - kPkMaxWindow, it.g, it.b);               // keys before the sequence: zeros
            tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, it.q0 - kPkMaxWindow, it.g, it.b);
            *reinterpret_cast<volatile int*>(&sm->loads_issued) = n + 1;
          }
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 11) {
    // ------------------------------------ TMA stores of dQ ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_dq);
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        for (int x = 0; x < 2; ++x) {
          const int u = 2 * n + x;
          if (!(ok = mbar_wait(bar_out_full, u & 1, abort_flag))) break;
          tma_store_4d(&tm_dq, smem_u32(sm->out), 0, it.q0 + x * kPkPos, it.g * kPkHeads, it.b);   // rows past the end are clipped
          tma_store_commit();
          tma_store_wait_read();                       // shared memory has been read: the next unit's rows may land
          mbar_arrive(bar_out_free);
        }
      }
      tma_store_wait_all();
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------- MMA issuer, S and dP (front) -------------------------
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kPkKeys, 0, 0);    // A, B both K-contiguous, N = 144
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        const int s = n % kPkStages;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_kv_full[s]), (n / kPkStages) & 1, abort_flag))) break;
        for (int x = 0; x < 2; ++x) {
          const int u = 2 * n + x, qb = x;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_q_full[qb]), (u >> 1) & 1, abort_flag))) break;
          if (u > 0 && !(ok = mbar_wait(bar_s_free, (u - 1) & 1, abort_flag))) break;   // the previous unit's S/dP are in registers
          tc_fence_after_sync();
          const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[qb]));
          const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o[qb]));
          const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[s]) + x * kPkSubOffsetBytes);
          const uint64_t v_desc = desc_kmajor(smem_u32(sm->v[s]) + x * kPkSubOffsetBytes);
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_s, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_dp, do_desc + kk * kDescKStepKMajor, v_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
          umma_commit(bar_s_full);
          umma_commit(smem_u32(&sm->bar_q_empty[qb]));   // Q/dO buffer free once these retire
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------ MMA issuer, dQ (back) ------------------------------
    if (lane == 0) {
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        const int s = n % kPkStages;
        for (int x = 0; x < 2; ++x) {
          const int u = 2 * n + x;
          if (!(ok = mbar_wait(bar_p_full, u & 1, abort_flag))) break;   // dS of the unit written
          // the dQ buffer is overwritten: the epilogue of the unit before the previous one must have read it
          if (u >= 2 && !(ok = mbar_wait(smem_u32(&sm->bar_dq_free[u & 1]), ((u >> 1) - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k[s]) + x * kPkSubOffsetBytes);
          const uint32_t dq = tmem_dq + (u & 1) * 64;
#pragma unroll
          for (int kk = 0; kk < kPkKeys / 16; ++kk)
            umma_ts(dq, tmem_ds + kk * 8, kt_desc + kk * kDescKStepMNMajor, idesc_back, kk > 0 ? 1u : 0u);
          umma_commit(bar_p_free);                          // dS is reusable once these retire
          umma_commit(smem_u32(&sm->bar_dq_full[u & 1]));
          if (x == 1) umma_commit(smem_u32(&sm->bar_kv_empty[s]));   // and so is the K/V stage (its S/dP MMAs retired before dS was written)
        }
        if (!ok) break;
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216();
  {
    // ------------------------------------- compute --------------------------------------
    const int wg = warp >> 2;             // which 72 key columns of every unit
    const int r = tid & 127;
    const int hl = r >> 4, sp = r & 15;   // head within the group, position within the unit
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
    const int c0 = wg * kDqPkHalf;        // first key column of this thread
    uint8_t* const out_row = sm->out + r * 128;
    int u = 0;                            // units so far
    bool ok = true;

    // row constants of a unit: -LSE * log2(e) and delta of this thread's row
    auto row_off_of = [&](const PkItem& it, int x) -> long long {
      return ((long long)(it.b * a.Hq + it.g * kPkHeads + hl)) * a.S_pad + it.q0 + x * kPkPos + sp;
    };

    // The epilogue of a unit runs after the compute of the next one (see the file comment).
    bool pending = false;
    int p_b = 0, p_h = 0, p_i = 0, p_len = 0, p_u = 0;
    float p_nl2 = 0.f, p_pdp = 0.f;
    auto epilogue = [&]() -> bool {
      if (!warp_all(mbar_wait(smem_u32(&sm->bar_dq_full[p_u & 1]), (p_u >> 1) & 1, abort_flag))) return false;
      // warpgroup 0 takes dQ columns 0-31, warpgroup 1 columns 32-63
      tc_fence_after_sync();
      uint32_t r0[32];
      tmem_ld32(tmem_dq + (p_u & 1) * 64 + lane_addr + wg * 32, r0);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->bar_dq_free[p_u & 1]));   // the unit after the next may overwrite this dQ buffer
      // sink gradient of this warp's two heads (16 rows each) for this warpgroup's key columns: fixed-order tree
      float dsk = (p_i < p_len) ? -fast_exp2(fmaf(a.sinks[p_h], kLog2e, p_nl2)) * p_pdp : 0.f;
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) dsk += __shfl_xor_sync(0xffffffffu, dsk, off);
      if (sp == 0)
        a.dsinks_partial[((long long)p_h * units_per_head + (long long)p_b * (a.S_pad / kPkPos) + (p_i >> 4)) * 2 + wg] = dsk;
      // the row goes to shared memory in the layout the TMA store expects (16-byte chunk c of row r at chunk
      // position c ^ (r % 8)); the store of the previous unit must have read the buffer
      if (p_u >= 1 && !warp_all(mbar_wait(bar_out_free, (p_u - 1) & 1, abort_flag))) return false;
      const float sc = (p_i < p_len) ? a.scale : 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(out_row + (((wg * 4 + c) ^ (r & 7)) << 4)) =
            make_uint4(pack_bf16(__uint_as_float(r0[c * 8]) * sc, __uint_as_float(r0[c * 8 + 1]) * sc),
                       pack_bf16(__uint_as_float(r0[c * 8 + 2]) * sc, __uint_as_float(r0[c * 8 + 3]) * sc),
                       pack_bf16(__uint_as_float(r0[c * 8 + 4]) * sc, __uint_as_float(r0[c * 8 + 5]) * sc),
                       pack_bf16(__uint_as_float(r0[c * 8 + 6]) * sc, __uint_as_float(r0[c * 8 + 7]) * sc));
      fence_proxy_async_smem();   // written with ordinary stores, read by the TMA engine
      mbar_arrive(bar_out_full);
      return true;
    };

    // next item at or after round k with real rows; padding-only items met on the way get their outputs here
    auto scan = [&](int& k, PkItem& it) -> bool {
      for (;; ++k) {
        const int id = k * (int)gridDim.x + (int)blockIdx.x;
        if (id >= n_items) return false;
        it = pk_item(a, id, dv);
        if (it.q0 < it.len) return true;
        const int h = it.g * kPkHeads + hl;
        for (int x = 0; x < 2; ++x) {
          const int i = it.q0 + x * kPkPos + sp;
          if (wg == 0 && i < a.S) zero_row(a.dq.row(it.b, h, i));   // dQ rows are zero,
          if (sp == 0) a.dsinks_partial[((long long)h * units_per_head + (long long)it.b * (a.S_pad / kPkPos) + (i >> 4)) * 2 + wg] = 0.f;  // no sink gradient
        }
      }
    };

    PkItem cur, nxt;
    int k = 0;
    bool have = scan(k, cur);
    float nl2[2] = {0.f, 0.f}, delta[2] = {0.f, 0.f};   // per unit of the current item
    if (have) {
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const long long ro = row_off_of(cur, x);
        nl2[x] = nlse_base[ro];
        delta[x] = a.delta[ro];
      }
    }
    while (ok && have) {
      int k_n = k + 1;
      const bool have_n = scan(k_n, nxt);
      float nl2_n[2] = {0.f, 0.f}, delta_n[2] = {0.f, 0.f};   // the next item's row constants: in flight under this item's work
      if (have_n) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const long long ro = row_off_of(nxt, x);
          nl2_n[x] = nlse_base[ro];
          delta_n[x] = a.delta[ro];
        }
      }
#pragma unroll
      for (int x = 0; x < 2; ++x, ++u) {
        const int i = cur.q0 + x * kPkPos + sp;           // this thread's query position
        const int kb = cur.q0 + x * kPkPos - kPkMaxWindow;   // key of column 0
        const PkRowMask rm = pk_row_mask(sp, kb, a.window, cur.len);
        const float2 nl22 = make_float2(nl2[x], nl2[x]), neg_delta2 = make_float2(-delta[x], -delta[x]);
        float2 acc = make_float2(0.f, 0.f);   // this warpgroup's share of sum_j P_ij dP_ij, two lanes

        if (!(ok = warp_all(mbar_wait(bar_s_full, u & 1, abort_flag)))) break;
        tc_fence_after_sync();
        uint32_t rs[2][32], rp[2][32], rs8[8], rp8[8];
        tmem_ld32(tmem_s + lane_addr + c0, rs[0]);
        tmem_ld32(tmem_dp + lane_addr + c0, rp[0]);
        tmem_ld32(tmem_s + lane_addr + c0 + 32, rs[1]);
        tmem_ld32(tmem_dp + lane_addr + c0 + 32, rp[1]);
        tmem_ld8(tmem_s + lane_addr + c0 + 64, rs8);
        tmem_ld8(tmem_dp + lane_addr + c0 + 64, rp8);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(bar_s_free);  // S/dP columns may be overwritten by the next unit
        uint32_t pk[2][16], pk8[4];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          // every 32-key chunk is classified for the whole warp: visible to all rows, to none, or mixed
          const uint32_t bits = range_bits(rm.lo - (c0 + c * 32), rm.hi - (c0 + c * 32));
          if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[c][e] = 0u;
          } else if (__all_sync(0xffffffffu, bits == 0xffffffffu)) {
            dq_compute_chunk<false>(rs[c], rp[c], scale2, nl22, neg_delta2, bits, pk[c], acc);
          } else {
            dq_compute_chunk<true>(rs[c], rp[c], scale2, nl22, neg_delta2, bits, pk[c], acc);
          }
        }
        dq_compute_chunk8(rs8, rp8, scale2, nl22, neg_delta2, range_bits(rm.lo - (c0 + 64), rm.hi - (c0 + 64)), pk8, acc);
        // the dQ MMAs of the previous unit must have left dS (long done: they ran under this unit's exponentials)
        if (u >= 1 && !(ok = warp_all(mbar_wait(bar_p_free, (u - 1) & 1, abort_flag)))) break;
        tc_fence_after_sync();
        const uint32_t ds = tmem_ds + lane_addr + wg * (kDqPkHalf / 2);
        tmem_st16(ds, pk[0]);
        tmem_st16(ds + 16, pk[1]);
        tmem_st4(ds + 32, pk8);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar_p_full);
        if (pending) {   // the previous unit's epilogue, its MMAs long retired
          if (!(ok = epilogue())) break;
        }
        pending = true;
        p_b = cur.b; p_h = cur.g * kPkHeads + hl; p_i = i; p_len = cur.len; p_u = u;
        p_nl2 = nl2[x];
        p_pdp = acc.x + acc.y;
      }
      if (!ok) break;
      cur = nxt;
      k = k_n;
      have = have_n;
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        nl2[x] = nl2_n[x];
        delta[x] = delta_n[x];
      }
    }
    if (ok && pending) ok = epilogue();
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kDqPkTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued, q_issued = sm->q_loads_issued;
    for (int uu = max(0, q_issued - 2); uu < q_issued; ++uu) mbar_wait_drain(smem_u32(&sm->bar_q_full[uu & 1]), (uu >> 1) & 1);
    for (int n = max(0, issued - kPkStages); n < issued; ++n)
      mbar_wait_drain(smem_u32(&sm->bar_kv_full[n % kPkStages]), (n / kPkStages) & 1);
  }
}

}  // namespace b200attn
