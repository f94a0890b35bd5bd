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
// consecutive position blocks, so neighbouring K/V windows meet in L2.
//
// What shapes the pipeline: with the arithmetic and the MMAs knocked out the first version still took 2800
// cycles per unit -- the compute warps' own chain of barrier waits, tensor-memory loads and stores, epilogue
// and bookkeeping, each step a 50-300 cycle latency that nothing hides (the two compute warpgroups work on the
// same unit in lockstep) -- against 1600 for the arithmetic itself.  So the compute warps do nothing but
//   load S/dP (72 columns each) -> exponentials and dS -> store dS,
// and everything else runs beside them:
//   * warp 13 streams Q/dO tiles (double-buffered, one 4-D TMA box {d 64, positions 16, heads 8} each) and
//     K/V blocks (3-stage ring) and runs ahead;
//   * warp 12 issues the S/dP MMAs of unit u+1 as soon as the compute threads hold S/dP of unit u in registers;
//   * dS is double-buffered in tensor memory and stored chunk by chunk as it is computed, so the compute
//     threads never wait for the dQ MMAs of the unit before; warp 14 issues those MMAs;
//   * a third warpgroup (warps 8-11) runs every epilogue: reads dQ, scales, stages the rows in shared memory
//     for one TMA store (warp 15) -- a thread's row is 128 contiguous bytes far from its neighbour's and plain
//     stores of that shape keep the load/store unit busy longer than the arithmetic takes -- and reduces the
//     sink-gradient partial from the per-row sums the compute threads hand over through shared memory.
// 512 threads; registers after setmaxnreg: compute 2 x 128 x 200, epilogue 128 x 56, the rest 128 x 56
// (= 512 x 128, the pool the CTA is launched with).  Barrier phases that are certainly complete are asked about
// early (a test costs 100-300 cycles of latency even then) and only waited for if not.  Every wait is bounded.
#pragma once
#include "attn_common.cuh"
#include "bwd_dq_kernel.cuh"        // dq_compute_chunk
#include "fwd_packed_kernel.cuh"    // tile constants, item decode, row masks

namespace b200attn {

constexpr int kDqPkThreads = 512;
constexpr int kDqPkTmemCols = 512;
constexpr int kDqPkHalf = kPkKeys / 2;   // 72 key columns per compute warpgroup
// tensor-memory columns: S [0,144)  dP [144,288)  dS bf16, two buffers [288,360) [368,440)  dQ [448,512)
constexpr uint32_t kDqPkColDp = 144, kDqPkColDs = 288, kDqPkColDsStride = 80, kDqPkColDq = 448;
constexpr int kDqPkPartialsPerTile = 8;   // sink-gradient partials per (head, 128 positions): one per unit

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
  uint64_t bar_p_full[2];                  // a dS buffer written                              (256 arrivals); one barrier per buffer,
                                           // so that the writers can never complete two phases unobserved
  uint64_t bar_p_free[2];                  // the dQ MMAs have read a dS buffer                (tcgen05.commit)
  uint64_t bar_dq_full;                    // the dQ MMAs of a unit retired                    (tcgen05.commit)
  uint64_t bar_dq_free;                    // dQ read by the epilogue                          (128 arrivals)
  uint64_t bar_acc_full;                   // the rows' sink-gradient terms are in shared memory (256 arrivals)
  uint64_t bar_out_full;                   // dQ rows are in shared memory (and the sink terms read) (128 arrivals)
  uint64_t bar_out_free;                   // the TMA store has read them                      (1 arrival)
  float acc[2][kTile];                     // [compute warpgroup][row]: -exp(sink - LSE) * sum_j P dP over its columns
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

// dS (bf16 pairs) of N key columns for one query row from S/dP in registers, stored to N/2 tensor-memory
// columns at `tmem_ds`; adds sum P*dP to acc.  Masked columns get S = -inf first (P = 0, dS = 0; dP is finite),
// which is skipped when the whole warp sees all N columns; nothing at all is computed when it sees none.
template <int N>
__device__ __forceinline__ void dqpk_chunk(uint32_t (&rs)[N], const uint32_t (&rp)[N], uint32_t bits, float2 scale2, float2 nl22,
                                           float2 neg_delta2, float2& acc, uint32_t tmem_ds) {
  constexpr uint32_t kAll = N == 32 ? 0xffffffffu : ((1u << N) - 1u);
  bits &= kAll;
  uint32_t pk[N / 2];
  if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
    for (int e = 0; e < N / 2; ++e) pk[e] = 0u;
  } else {
    if (!__all_sync(0xffffffffu, bits == kAll)) {
#pragma unroll
      for (int e = 0; e < N; ++e) rs[e] = (bits >> e) & 1u ? rs[e] : 0xff800000u;   // -inf
    }
#pragma unroll
    for (int e = 0; e < N; e += 2) {
      const float2 x = __ffma2_rn(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), scale2, nl22);
      const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
      const float2 dp = make_float2(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1]));
      acc = __ffma2_rn(p, dp, acc);
      const float2 ds = __fmul2_rn(p, __fadd2_rn(dp, neg_delta2));
      pk[e >> 1] = pack_bf16(ds.x, ds.y);
    }
  }
  if constexpr (N == 16) tmem_st8(tmem_ds, pk);
  else tmem_st4(tmem_ds, pk);
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
  const int units_per_head = a.B * (a.S_pad / kPkPos);                  // sink-gradient partial slots: [head][batch][unit]

  const uint32_t bar_s_full = smem_u32(&sm->bar_s_full), bar_s_free = smem_u32(&sm->bar_s_free),
                 bar_dq_full = smem_u32(&sm->bar_dq_full), bar_dq_free = smem_u32(&sm->bar_dq_free),
                 bar_acc_full = smem_u32(&sm->bar_acc_full), bar_out_full = smem_u32(&sm->bar_out_full),
                 bar_out_free = smem_u32(&sm->bar_out_free);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int q = 0; q < 2; ++q) {
      mbar_init(smem_u32(&sm->bar_q_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_q_empty[q]), 1);
      mbar_init(smem_u32(&sm->bar_p_full[q]), 2 * kComputeThreads);
      mbar_init(smem_u32(&sm->bar_p_free[q]), 1);
    }
    for (int s = 0; s < kPkStages; ++s) {
      mbar_init(smem_u32(&sm->bar_kv_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_kv_empty[s]), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, 2 * kComputeThreads);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_free, kComputeThreads);
    mbar_init(bar_acc_full, 2 * kComputeThreads);
    mbar_init(bar_out_full, kComputeThreads);
    mbar_init(bar_out_free, 1);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    sm->q_loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 12) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDqPkTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + kDqPkColDp, tmem_ds = tmem + kDqPkColDs, tmem_dq = tmem + kDqPkColDq;

  if (warp >= 12) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 13) {
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
#pragma unroll 1
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
  } else if (warp == 15) {
    // ------------------------------------ TMA stores of dQ ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_dq);
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
#pragma unroll 1
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
  } else if (warp == 12) {
    // ------------------------- MMA issuer, S and dP (front) -------------------------
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kPkKeys, 0, 0);    // A, B both K-contiguous, N = 144
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        const int s = n % kPkStages;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_kv_full[s]), (n / kPkStages) & 1, abort_flag))) break;
#pragma unroll 1
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
  } else {
    // ------------------------------ MMA issuer, dQ (back) ------------------------------
    if (lane == 0) {
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        const int s = n % kPkStages;
#pragma unroll 1
        for (int x = 0; x < 2; ++x) {
          const int u = 2 * n + x;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_p_full[u & 1]), (u >> 1) & 1, abort_flag))) break;   // dS of the unit written
          if (u >= 1 && !(ok = mbar_wait(bar_dq_free, (u - 1) & 1, abort_flag))) break;               // dQ of the unit before read
          tc_fence_after_sync();
          const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k[s]) + x * kPkSubOffsetBytes);
          const uint32_t ds = tmem_ds + (u & 1) * kDqPkColDsStride;
#pragma unroll
          for (int kk = 0; kk < kPkKeys / 16; ++kk)
            umma_ts(tmem_dq, ds + kk * 8, kt_desc + kk * kDescKStepMNMajor, idesc_back, kk > 0 ? 1u : 0u);
          umma_commit(smem_u32(&sm->bar_p_free[u & 1]));    // the dS buffer is reusable once these retire
          umma_commit(bar_dq_full);
          if (x == 1) umma_commit(smem_u32(&sm->bar_kv_empty[s]));   // and so is the K/V stage (its S/dP MMAs retired before dS was written)
        }
        if (!ok) break;
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  {
    // ------------------------------------- epilogues --------------------------------------
    const int r = tid & 127;
    const int hl = r >> 4, sp = r & 15;   // head within the group, position within the unit
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    uint8_t* const out_row = sm->out + r * 128;
    bool ok = true;
    PkItem it;
    int n = 0;
    for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
#pragma unroll 1
      for (int x = 0; x < 2; ++x) {
        const int u = 2 * n + x;
        const int i = it.q0 + x * kPkPos + sp;
        const int h = it.g * kPkHeads + hl;
        // sink gradient of this warp's two heads (16 rows each): the two compute warpgroups' terms, fixed-order tree
        if (!(ok = warp_all(mbar_wait(bar_acc_full, u & 1, abort_flag)))) break;
        float dsk = sm->acc[0][r] + sm->acc[1][r];
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) dsk += __shfl_xor_sync(0xffffffffu, dsk, off);
        if (sp == 0) a.dsinks_partial[(long long)h * units_per_head + (long long)it.b * (a.S_pad / kPkPos) + (i >> 4)] = dsk;
        if (!(ok = warp_all(mbar_wait(bar_dq_full, u & 1, abort_flag)))) break;
        tc_fence_after_sync();
        // the store of the previous unit must have read the staging buffer
        if (u >= 1 && !(ok = warp_all(mbar_wait(bar_out_free, (u - 1) & 1, abort_flag)))) break;
        const float sc = (i < it.len) ? a.scale : 0.f;
        // the row goes to shared memory in the layout the TMA store expects: 16-byte chunk c of row r at chunk
        // position c ^ (r % 8); 32 columns at a time (this warpgroup lives on few registers)
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t r0[32];
          tmem_ld32(tmem_dq + lane_addr + half * 32, r0);
          tmem_wait_ld();
          if (half == 1) {
            tc_fence_before_sync();
            mbar_arrive(bar_dq_free);   // the next unit's dQ MMAs may overwrite dQ
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(out_row + (((half * 4 + c) ^ (r & 7)) << 4)) =
                make_uint4(pack_bf16(__uint_as_float(r0[c * 8]) * sc, __uint_as_float(r0[c * 8 + 1]) * sc),
                           pack_bf16(__uint_as_float(r0[c * 8 + 2]) * sc, __uint_as_float(r0[c * 8 + 3]) * sc),
                           pack_bf16(__uint_as_float(r0[c * 8 + 4]) * sc, __uint_as_float(r0[c * 8 + 5]) * sc),
                           pack_bf16(__uint_as_float(r0[c * 8 + 6]) * sc, __uint_as_float(r0[c * 8 + 7]) * sc));
        }
        fence_proxy_async_smem();   // written with ordinary stores, read by the TMA engine
        mbar_arrive(bar_out_full);
      }
    }
    if (!ok && r == 0) report_abort(a);
  }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
  {
    // ------------------------------------- compute --------------------------------------
    const int wg = warp >> 2;             // which 72 key columns of every unit
    const int r = tid & 127;
    const int hl = r >> 4, sp = r & 15;   // head within the group, position within the unit
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
    const int c0 = wg * kDqPkHalf;        // first key column of this thread
    int u = 0;                            // units so far
    int g_cur = -1;
    float sink2 = 0.f;                    // this thread's head's sink logit * log2(e), for the group at hand
    bool s_ready = false;
    bool ok = true;

    // row constants of a unit: -LSE * log2(e) and delta of this thread's row
    auto row_off_of = [&](const PkItem& it, int x) -> long long {
      return ((long long)(it.b * a.Hq + it.g * kPkHeads + hl)) * a.S_pad + it.q0 + x * kPkPos + sp;
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
          if (wg == 0 && sp == 0) a.dsinks_partial[(long long)h * units_per_head + (long long)it.b * (a.S_pad / kPkPos) + (i >> 4)] = 0.f;  // no sink gradient
        }
      }
    };

    // one flat loop over units (unit u = item u/2, half u%2), not unrolled: see the note at the chunk loop
    PkItem cur;
    int k = 0;
    bool have = scan(k, cur);
    int x = 0;                            // which half of the current item
    float nl2 = 0.f, delta = 0.f;         // -LSE * log2(e) and delta of this thread's row of the current unit
    if (have) {
      const long long ro = row_off_of(cur, 0);
      nl2 = nlse_base[ro];
      delta = a.delta[ro];
    }
#pragma unroll 1
    for (; have; ++u) {
      if (cur.g != g_cur) {   // (consecutive items nearly always belong to the same group)
        g_cur = cur.g;
        sink2 = a.sinks[cur.g * kPkHeads + hl] * kLog2e;
      }
      const int i = cur.q0 + x * kPkPos + sp;              // this thread's query position
      const int kb = cur.q0 + x * kPkPos - kPkMaxWindow;   // key of column 0
      const int len = cur.len;
      const PkRowMask rm = pk_row_mask(sp, kb, a.window, len);
      const float2 nl22 = make_float2(nl2, nl2), neg_delta2 = make_float2(-delta, -delta);
      float2 acc = make_float2(0.f, 0.f);   // this warpgroup's share of sum_j P_ij dP_ij, two lanes
      // the unit after this one: the item's other half, or the first half of the next item with real rows
      PkItem nxt = cur;
      bool have_n = true;
      if (x == 1) {
        ++k;
        have_n = scan(k, nxt);
      }
      const int x_n = x ^ 1;

      // barrier phases needed further down and certainly complete by then: ask now, the answers arrive under
      // the loads.  The dS buffer was read by the dQ MMAs of the unit before the previous one; the epilogue of
      // the previous unit has read the sink terms (one slot: the producer may not get two phases ahead).
      const uint32_t bar_pf = smem_u32(&sm->bar_p_free[u & 1]);
      const bool p_free = u < 2 || mbar_test_wait(bar_pf, ((u >> 1) - 1) & 1);
      const bool acc_free = u == 0 || mbar_test_wait(bar_out_full, (u - 1) & 1);
      if (!warp_all(s_ready) && !(ok = warp_all(mbar_wait(bar_s_full, u & 1, abort_flag)))) break;
      tc_fence_after_sync();
      if (!warp_all(p_free) && !(ok = warp_all(mbar_wait(bar_pf, ((u >> 1) - 1) & 1, abort_flag)))) break;
      tc_fence_after_sync();
      // the next unit's row constants: a whole unit of arithmetic before their first use
      float nl2_n = 0.f, delta_n = 0.f;
      if (have_n) {
        const long long ro = row_off_of(nxt, x_n);
        nl2_n = nlse_base[ro];
        delta_n = a.delta[ro];
      }
      // This warpgroup's 72 columns, streamed from tensor memory 16 at a time (the next 16 in flight under
      // this chunk's exponentials) by a ROLLED loop: the unrolled form is ~20 KB of straight-line code per
      // unit and had the warps waiting for instruction fetch most of the time.
      const uint32_t s_row = tmem_s + lane_addr + c0, dp_row = tmem_dp + lane_addr + c0;
      const uint32_t ds = tmem_ds + (u & 1) * kDqPkColDsStride + lane_addr + wg * (kDqPkHalf / 2);
      {
        uint32_t sa[16], pa[16], sb[16], pb[16], s8[8], p8[8];
        tmem_ld16(s_row, sa);
        tmem_ld16(dp_row, pa);
#pragma unroll 1
        for (int cc = 0; cc < 4; cc += 2) {
          tmem_wait_ld();
          tmem_ld16(s_row + (cc + 1) * 16, sb);
          tmem_ld16(dp_row + (cc + 1) * 16, pb);
          dqpk_chunk<16>(sa, pa, range_bits(rm.lo - (c0 + cc * 16), rm.hi - (c0 + cc * 16)), scale2, nl22, neg_delta2, acc, ds + cc * 8);
          tmem_wait_ld();
          if (cc == 0) {
            tmem_ld16(s_row + 32, sa);
            tmem_ld16(dp_row + 32, pa);
          } else {
            tmem_ld8(s_row + 64, s8);
            tmem_ld8(dp_row + 64, p8);
          }
          dqpk_chunk<16>(sb, pb, range_bits(rm.lo - (c0 + (cc + 1) * 16), rm.hi - (c0 + (cc + 1) * 16)), scale2, nl22, neg_delta2, acc,
                         ds + (cc + 1) * 8);
        }
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(bar_s_free);  // all of S/dP is in registers or used: the next unit's may be computed
        dqpk_chunk<8>(s8, p8, range_bits(rm.lo - (c0 + 64), rm.hi - (c0 + 64)), scale2, nl22, neg_delta2, acc, ds + 32);
      }
      s_ready = mbar_test_wait(bar_s_full, (u + 1) & 1);   // the next unit's S/dP: asked under the stores
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->bar_p_full[u & 1]));
      // this row's term of the sink gradient for the epilogue warpgroup
      if (!warp_all(acc_free) && !(ok = warp_all(mbar_wait(bar_out_full, (u - 1) & 1, abort_flag)))) break;
      sm->acc[wg][r] = (i < len) ? -fast_exp2(sink2 + nl2) * (acc.x + acc.y) : 0.f;
      mbar_arrive(bar_acc_full);
      cur = nxt;
      x = x_n;
      have = have_n;
      nl2 = nl2_n;
      delta = delta_n;
    }
    if (!ok && tid == 0) report_abort(a);
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) {
    __syncwarp();
    tmem_dealloc(tmem, kDqPkTmemCols);
  }
  if (sm->abort_flag && tid == 13 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    report_abort(a);
    const int issued = sm->loads_issued, q_issued = sm->q_loads_issued;
    for (int uu = max(0, q_issued - 2); uu < q_issued; ++uu) mbar_wait_drain(smem_u32(&sm->bar_q_full[uu & 1]), (uu >> 1) & 1);
    for (int n = max(0, issued - kPkStages); n < issued; ++n)
      mbar_wait_drain(smem_u32(&sm->bar_kv_full[n % kPkStages]), (n / kPkStages) & 1);
  }
}

}  // namespace b200attn
