// dK/dV kernel for sm_100a.
//
// One CTA owns one 128-key tile of one KV head of one sequence and keeps dK and dV for it in
// tensor memory while it streams, for each of the G query heads of the group, the 64-row query
// blocks that can see the key tile.  Per step (one head, one query block), transposed so that
// keys are the accumulator rows:
//     S^T  = K Q^T            dP^T = V dO^T                 (tcgen05, fp32 in TMEM, N = 64)
//     P^T  = 2^(S^T*scale*log2e - LSE*log2e)    dS^T = P^T * (dP^T - delta)   (1 thread / key)
//     dV  += P^T dO           dK  += dS^T Q                 (A operand = bf16 in TMEM)
// The epilogue stores dV and dK * scale once.  No atomics: every dK/dV element has one owner
// and is accumulated in fp32 (the reference adds bf16 partial tiles into global memory with
// atomics, attention_kernel.py:201-212).
//
// K and V (the A operands of S^T and dP^T for the CTA's whole life) are copied once into
// tensor memory as bf16, so those MMAs read only the 64-row Q/dO block from shared memory --
// with both operands in shared memory a 128x64x16 MMA is bound by shared-memory bandwidth.
//
// Pipeline: warp 9 streams Q/dO blocks (+ the LSE and delta rows) through a 4-stage TMA ring;
// warp 8 issues every MMA from a first-ready service loop; S^T/dP^T live in two rotating
// tensor-memory buffers so that the tensor core computes step t+1 while the compute warps are
// still busy with step t; two compute warpgroups (warps 0-3 and 4-7) take the steps
// alternately.  Every wait is bounded.
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kBlk = 64;                               // query rows per step
constexpr int kBlkBytes = kBlk * kHeadDim * 2;         // 8 KB
constexpr int kDkvStages = 4;
constexpr int kDkvBufs = 2;
constexpr int kDkvThreads = 384;
constexpr int kDkvTmemCols = 512;
// tensor-memory columns: buffer b: S^T/P^T [128b, 128b+64)  dP^T/dS^T [128b+64, 128b+128);
// K bf16 [256,288)  V bf16 [288,320)  dV [320,384)  dK [384,448)

struct DkvSmem {
  alignas(1024) uint8_t q[kDkvStages][kBlkBytes];
  alignas(1024) uint8_t d_o[kDkvStages][kBlkBytes];
  alignas(16) float nlse[kDkvStages][kBlk];   // -LSE * log2(e) of the block's query rows
  alignas(16) float delta[kDkvStages][kBlk];
  alignas(8) uint64_t bar_kv;                 // K and V copied into tensor memory (256 arrivals)
  uint64_t bar_in_full[kDkvStages];           // Q, dO, nlse, delta of a stage landed
  uint64_t bar_in_empty[kDkvStages];          // the MMAs reading a stage retired
  uint64_t bar_s_full[kDkvBufs];              // S^T and dP^T of a buffer ready
  uint64_t bar_p_full[kDkvBufs];              // P^T and dS^T written (128 arrivals)
  uint64_t bar_acc;                           // every MMA retired: dK/dV final
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;
};

constexpr uint32_t kDkvStageBytes = 2 * kBlkBytes + 2 * kBlk * sizeof(float);

struct DkvStep {  // which (head, query block) a step works on
  int h, q0;
};
__device__ __forceinline__ DkvStep dkv_step(int it, int nq, int qb_first, int g, int group) {
  return DkvStep{g * group + it / nq, (qb_first + it % nq) * kBlk};
}

// One step for one key row: reads the 64 S^T and dP^T values of the row, writes P^T and dS^T
// (bf16) back over the columns it has consumed.
template <bool kMask>
__device__ __forceinline__ void dkv_compute_step(uint32_t buf, const float* nlse, const float* delta, float scale_log2,
                                                 int q0, int j, int window, int len) {
  uint32_t rs[2][32], rp[2][32];
  tmem_ld32(buf, rs[0]);
  tmem_ld32(buf + 64, rp[0]);
  tmem_ld32(buf + 32, rs[1]);
  tmem_ld32(buf + 96, rp[1]);
  tmem_wait_ld();
  const float4* nl4 = reinterpret_cast<const float4*>(nlse);
  const float4* de4 = reinterpret_cast<const float4*>(delta);
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t pp[16], pd[16];
    const uint32_t bits = kMask ? visible_queries32(j, q0 + c * 32, window, len) : 0xffffffffu;
#pragma unroll
    for (int e4 = 0; e4 < 8; ++e4) {
      const float4 L = nl4[c * 8 + e4];
      const float4 D = de4[c * 8 + e4];
      const float lv[4] = {L.x, L.y, L.z, L.w};
      const float dl[4] = {D.x, D.y, D.z, D.w};
      float p[4], ds[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e4 * 4 + u;
        p[u] = fast_exp2(fmaf(__uint_as_float(rs[c][e]), scale_log2, lv[u]));
        if (kMask) p[u] = (bits >> e) & 1u ? p[u] : 0.f;  // select, not a branch
        ds[u] = p[u] * (__uint_as_float(rp[c][e]) - dl[u]);
      }
      pp[e4 * 2] = pack_bf16(p[0], p[1]);
      pp[e4 * 2 + 1] = pack_bf16(p[2], p[3]);
      pd[e4 * 2] = pack_bf16(ds[0], ds[1]);
      pd[e4 * 2 + 1] = pack_bf16(ds[2], ds[3]);
    }
    tmem_st16(buf + c * 16, pp);        // P^T over consumed S^T columns
    tmem_st16(buf + 64 + c * 16, pd);   // dS^T over consumed dP^T columns
  }
}

__global__ void __launch_bounds__(kDkvThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DkvSmem* sm = reinterpret_cast<DkvSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int g = blockIdx.y;
  const int kt = blockIdx.x;  // early key tiles are seen by the most query rows: first
  const int kv0 = kt * kTile;
  const int len = seq_len(a, b);

  if (kv0 >= len) {  // padding only
    if (tid < kComputeThreads && kv0 + tid < a.S) {
      zero_row(a.dk.row(b, g, kv0 + tid));
      zero_row(a.dv.row(b, g, kv0 + tid));
    }
    return;
  }

  const int j_max = min(kv0 + kTile - 1, len - 1);
  const int i_max = a.window ? min(len - 1, j_max + a.window - 1) : len - 1;  // last query row that sees the tile
  const int qb_first = kv0 / kBlk;
  const int nq = i_max / kBlk - qb_first + 1;  // query blocks per head
  const int n_steps = nq * a.group;
  const float* nlse_base = a.delta + (long long)a.B * a.Hq * a.S_pad;  // second half of the delta scratch

  const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_acc = smem_u32(&sm->bar_acc);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_kv, 2 * kComputeThreads);
    for (int s = 0; s < kDkvStages; ++s) {
      mbar_init(smem_u32(&sm->bar_in_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_in_empty[s]), 1);
    }
    for (int s = 0; s < kDkvBufs; ++s) {
      mbar_init(smem_u32(&sm->bar_s_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_p_full[s]), kComputeThreads);
    }
    mbar_init(bar_acc, 1);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDkvTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_k = tmem + 256, tmem_v = tmem + 288, tmem_dv = tmem + 320, tmem_dk = tmem + 384;

  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      for (int it = 0; it < n_steps; ++it) {
        const int s = it % kDkvStages;
        if (it >= kDkvStages && !mbar_wait(smem_u32(&sm->bar_in_empty[s]), ((it / kDkvStages) - 1) & 1, abort_flag)) {
          report_abort(a);
          break;
        }
        const DkvStep st = dkv_step(it, nq, qb_first, g, a.group);
        const uint32_t bar = smem_u32(&sm->bar_in_full[s]);
        const long long row_off = ((long long)(b * a.Hq + st.h)) * a.S_pad + st.q0;
        mbar_arrive_expect_tx(bar, kDkvStageBytes);
        tma_load_4d(smem_u32(sm->q[s]), &tm_q, bar, 0, st.q0, st.h, b);
        tma_load_4d(smem_u32(sm->d_o[s]), &tm_do, bar, 0, st.q0, st.h, b);
        bulk_load_1d(smem_u32(sm->nlse[s]), nlse_base + row_off, kBlk * sizeof(float), bar);
        bulk_load_1d(smem_u32(sm->delta[s]), a.delta + row_off, kBlk * sizeof(float), bar);
        *reinterpret_cast<volatile int*>(&sm->loads_issued) = it + 1;
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kBlk, 0, 0);     // A in TMEM, B K-contiguous, N = 64
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      bool ok = mbar_wait(bar_kv, 0, abort_flag);
      tc_fence_after_sync();
      int front = 0, back = 0;  // next step whose S^T/dP^T resp. dV/dK MMAs are to be issued
      long long t_idle0 = 0;
      uint32_t idle = 0;
      while (ok && back < n_steps) {
        bool progressed = false;
        if (back < front && mbar_try_wait(smem_u32(&sm->bar_p_full[back % kDkvBufs]), (back / kDkvBufs) & 1)) {
          tc_fence_after_sync();
          const int s = back % kDkvStages;
          const uint32_t buf = tmem + (back % kDkvBufs) * 128;
          const uint64_t dot_desc = desc_mnmajor(smem_u32(sm->d_o[s]));
          const uint64_t qt_desc = desc_mnmajor(smem_u32(sm->q[s]));
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk)
            umma_ts(tmem_dv, buf + kk * 8, dot_desc + kk * kDescKStepMNMajor, idesc_back, (back > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk)
            umma_ts(tmem_dk, buf + 64 + kk * 8, qt_desc + kk * kDescKStepMNMajor, idesc_back, (back > 0 || kk > 0) ? 1u : 0u);
          umma_commit(smem_u32(&sm->bar_in_empty[s]));  // the stage (and the buffer) are free once these retire
          if (back == n_steps - 1) umma_commit(bar_acc);
          ++back;
          progressed = true;
        }
        if (front < n_steps && front < back + kDkvBufs &&
            mbar_try_wait(smem_u32(&sm->bar_in_full[front % kDkvStages]), (front / kDkvStages) & 1)) {
          tc_fence_after_sync();
          const int s = front % kDkvStages;
          const uint32_t buf = tmem + (front % kDkvBufs) * 128;
          const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[s]));
          const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o[s]));
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ts(buf, tmem_k + kk * 8, q_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ts(buf + 64, tmem_v + kk * 8, do_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
          umma_commit(smem_u32(&sm->bar_s_full[front % kDkvBufs]));
          ++front;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if ((++idle & 1023u) == 0u) {  // bounded: give up after ~2 s without progress
          if (idle == 1024u) t_idle0 = clock64();
          if (*abort_flag || clock64() - t_idle0 > kWaitLimitCycles) {
            sm->abort_flag = 1;
            ok = false;
          }
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------- compute --------------------------------------
    const int wg = warp >> 2;             // takes steps wg, wg+2, ...
    const int j = kv0 + (tid & 127);      // this thread's key position
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    bool ok = true;

    {  // copy this thread's row of K (warpgroup 0) or V (warpgroup 1) into tensor memory as bf16
      const StridedPtr& src = wg == 0 ? a.k : a.v;
      uint32_t w[32];
      if (j < a.S) {
        const uint4* row = reinterpret_cast<const uint4*>(src.row(b, g, j));
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 x = row[c];
          w[4 * c] = x.x; w[4 * c + 1] = x.y; w[4 * c + 2] = x.z; w[4 * c + 3] = x.w;
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) w[c] = 0u;
      }
      tmem_st32((wg == 0 ? tmem_k : tmem_v) + lane_addr, w);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_kv);
    }

    for (int it = wg; it < n_steps; it += 2) {
      const int s = it % kDkvStages;
      const int bi = it % kDkvBufs;
      const int q0 = dkv_step(it, nq, qb_first, g, a.group).q0;
      const bool need_mask = (kv0 + kTile - 1 > q0) || (a.window != 0 && kv0 <= q0 + kBlk - 1 - a.window) || (q0 + kBlk > len);
      // nlse/delta of this stage are read with plain loads below: observe their barrier directly
      if (!(ok = warp_all(mbar_wait(smem_u32(&sm->bar_in_full[s]), (it / kDkvStages) & 1, abort_flag)))) break;
      if (!(ok = warp_all(mbar_wait(smem_u32(&sm->bar_s_full[bi]), (it / kDkvBufs) & 1, abort_flag)))) break;
      tc_fence_after_sync();
      const uint32_t buf = tmem + bi * 128 + lane_addr;
      if (need_mask) dkv_compute_step<true>(buf, sm->nlse[s], sm->delta[s], a.scale_log2, q0, j, a.window, len);
      else dkv_compute_step<false>(buf, sm->nlse[s], sm->delta[s], a.scale_log2, q0, j, a.window, len);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm->bar_p_full[bi]));
    }

    if (ok) ok = warp_all(mbar_wait(bar_acc, 0, abort_flag));
    if (ok) {
      // warpgroup 0 stores dV, warpgroup 1 stores dK * scale
      tc_fence_after_sync();
      const uint32_t src = (wg == 0 ? tmem_dv : tmem_dk) + lane_addr;
      const float sc = wg == 0 ? 1.f : a.scale;
      uint32_t r0[32], r1[32];
      tmem_ld32(src, r0);
      tmem_ld32(src + 32, r1);
      tmem_wait_ld();
      if (j < a.S) {
        __nv_bfloat16* dst = wg == 0 ? a.dv.row(b, g, j) : a.dk.row(b, g, j);
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
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kDkvTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued;
    for (int it = max(0, issued - kDkvStages); it < issued; ++it)
      mbar_wait_drain(smem_u32(&sm->bar_in_full[it % kDkvStages]), (it / kDkvStages) & 1);
  }
}

}  // namespace b200attn
