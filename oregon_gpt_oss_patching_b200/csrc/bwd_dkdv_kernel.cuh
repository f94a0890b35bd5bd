// dK/dV kernel for sm_100a.
//
// One CTA owns one 128-key tile of one KV head of one sequence and keeps dK and dV for it
// in tensor memory while it loops over the G query heads of the group and, for each, the
// query tiles that can see the key tile.  Per (head, query tile), transposed so that keys
// are the accumulator rows:
//     S^T  = K Q^T            dP^T = V dO^T                 (tcgen05, fp32 in TMEM)
//     P^T  = 2^(S^T*scale*log2e - LSE*log2e)    dS^T = P^T * (dP^T - delta)   (1 thread / key)
//     dV  += P^T dO           dK  += dS^T Q                 (A operand from TMEM, bf16)
// The epilogue stores dV and dK * scale once.  No atomics: every dK/dV element has one owner
// and is accumulated in fp32 (the reference adds bf16 partial tiles into global memory with
// atomics, attention_kernel.py:201-212).
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kDkvStages = 2;
constexpr int kDkvTmemCols = 512;  // S^T/P^T: [0,128)  dP^T/dS^T: [128,256)  dV: [256,320)  dK: [320,384)

struct DkvSmem {
  alignas(1024) uint8_t k[kTileBytes];
  alignas(1024) uint8_t v[kTileBytes];
  alignas(1024) uint8_t q[kDkvStages][kTileBytes];
  alignas(1024) uint8_t d_o[kDkvStages][kTileBytes];
  alignas(16) float lse[kDkvStages][kTile];
  alignas(16) float delta[kDkvStages][kTile];
  alignas(8) uint64_t bar_kv;    // K and V landed
  uint64_t bar_in[kDkvStages];   // Q, dO, lse, delta of a stage landed
  uint64_t bar_s;                // S^T and dP^T ready
  uint64_t bar_p;                // P^T and dS^T written by 128 threads
  uint64_t bar_o;                // dV/dK MMAs of an iteration finished
  uint32_t tmem_base;
  int abort_flag;
};

constexpr uint32_t kDkvStageBytes = 2 * kTileBytes + 2 * kTile * sizeof(float);

__device__ __forceinline__ void dkv_issue_stage(DkvSmem* sm, int s, const CUtensorMap* tm_q, const CUtensorMap* tm_do,
                                                const KernelArgs& a, int b, int h, int q0) {
  const uint32_t bar = smem_u32(&sm->bar_in[s]);
  const long long row_off = ((long long)(b * a.Hq + h)) * a.S_pad + q0;
  mbar_arrive_expect_tx(bar, kDkvStageBytes);
  tma_load_4d(smem_u32(sm->q[s]), tm_q, bar, 0, q0, h, b);
  tma_load_4d(smem_u32(sm->d_o[s]), tm_do, bar, 0, q0, h, b);
  bulk_load_1d(smem_u32(sm->lse[s]), a.lse + row_off, kTile * sizeof(float), bar);
  bulk_load_1d(smem_u32(sm->delta[s]), a.delta + row_off, kTile * sizeof(float), bar);
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DkvSmem* sm = reinterpret_cast<DkvSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int g = blockIdx.y;
  const int kt = blockIdx.x;  // early key tiles are seen by the most query tiles: first
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
  const int i_max = a.window ? min(len - 1, j_max + a.window - 1) : len - 1;
  const int m_first = kt;
  const int nq = i_max / kTile - m_first + 1;   // query tiles per head
  const int n_iter = nq * a.group;

  const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_s = smem_u32(&sm->bar_s), bar_p = smem_u32(&sm->bar_p),
                 bar_o = smem_u32(&sm->bar_o);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < kDkvStages; ++s) mbar_init(smem_u32(&sm->bar_in[s]), 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kComputeThreads);
    mbar_init(bar_o, 1);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kDkvTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dv = tmem + 256, tmem_dk = tmem + 320;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      prefetch_tmap(&tm_do);
      mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
      tma_load_4d(smem_u32(sm->k), &tm_k, bar_kv, 0, kv0, g, b);
      tma_load_4d(smem_u32(sm->v), &tm_v, bar_kv, 0, kv0, g, b);
      const int pre = n_iter < kDkvStages ? n_iter : kDkvStages;
      for (int it = 0; it < pre; ++it)
        dkv_issue_stage(sm, it, &tm_q, &tm_do, a, b, g * a.group + it / nq, (m_first + it % nq) * kTile);
      const uint32_t idesc_nt = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_acc = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      const uint64_t k_desc = desc_kmajor(smem_u32(sm->k));
      const uint64_t v_desc = desc_kmajor(smem_u32(sm->v));
      bool ok = mbar_wait(bar_kv, 0, abort_flag);
      int issued = pre, waited = 0;
      for (int it = 0; ok && it < n_iter; ++it) {
        const int s = it % kDkvStages;
        const uint32_t ph = (it / kDkvStages) & 1;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_in[s]), ph, abort_flag))) break;
        waited = it + 1;
        tc_fence_after_sync();
        const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[s]));
        const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o[s]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_s, k_desc + kk * kDescKStepKMajor, q_desc + kk * kDescKStepKMajor, idesc_nt, kk > 0);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_dp, v_desc + kk * kDescKStepKMajor, do_desc + kk * kDescKStepKMajor, idesc_nt, kk > 0);
        umma_commit(bar_s);
        if (!(ok = mbar_wait(bar_p, it & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t dot_desc = desc_mnmajor(smem_u32(sm->d_o[s]));
        const uint64_t qt_desc = desc_mnmajor(smem_u32(sm->q[s]));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(tmem_dv, tmem_s + kk * 8, dot_desc + kk * kDescKStepMNMajor, idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(tmem_dk, tmem_dp + kk * 8, qt_desc + kk * kDescKStepMNMajor, idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar_o);
        if (it + kDkvStages < n_iter) {
          if (!(ok = mbar_wait(bar_o, it & 1, abort_flag))) break;
          const int nx = it + kDkvStages;
          dkv_issue_stage(sm, s, &tm_q, &tm_do, a, b, g * a.group + nx / nq, (m_first + nx % nq) * kTile);
          ++issued;
        }
      }
      if (!ok) {
        report_abort(a);
        mbar_wait_drain(bar_kv, 0);
        for (int it = waited; it < issued; ++it)
          mbar_wait_drain(smem_u32(&sm->bar_in[it % kDkvStages]), (it / kDkvStages) & 1);
      }
    }
    __syncwarp();
  } else {
    const int j = kv0 + tid;  // this thread's key position
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;
    bool ok = true;
    uint32_t rs[32], rp[32];

    for (int it = 0; it < n_iter; ++it) {
      const int s = it % kDkvStages;
      const int q0 = (m_first + it % nq) * kTile;
      const bool need_mask = tile_needs_mask(q0, kv0, a.window, len);
      // lse/delta of this stage are read with plain loads below: observe their barrier directly
      if (!(ok = warp_all(mbar_wait(smem_u32(&sm->bar_in[s]), (it / kDkvStages) & 1, abort_flag)))) break;
      if (!(ok = warp_all(mbar_wait(bar_s, it & 1, abort_flag)))) break;
      tc_fence_after_sync();
      const float4* lse4 = reinterpret_cast<const float4*>(sm->lse[s]);
      const float4* del4 = reinterpret_cast<const float4*>(sm->delta[s]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(tmem_s + lane_addr + c * 32, rs);
        tmem_ld32(tmem_dp + lane_addr + c * 32, rp);
        tmem_wait_ld();
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 L = lse4[c * 8 + e4];
          const float4 D = del4[c * 8 + e4];
          const float lv[4] = {L.x, L.y, L.z, L.w};
          const float dv_[4] = {D.x, D.y, D.z, D.w};
          float p[4], ds[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 * 4 + u;
            p[u] = fast_exp2(fmaf(__uint_as_float(rs[e]), a.scale_log2, -lv[u] * kLog2e));
            if (need_mask && !visible(q0 + c * 32 + e, j, a.window, len)) p[u] = 0.f;
            ds[u] = p[u] * (__uint_as_float(rp[e]) - dv_[u]);
          }
          pp[e4 * 2] = pack_bf16(p[0], p[1]);
          pp[e4 * 2 + 1] = pack_bf16(p[2], p[3]);
          pd[e4 * 2] = pack_bf16(ds[0], ds[1]);
          pd[e4 * 2 + 1] = pack_bf16(ds[2], ds[3]);
        }
        tmem_st16(tmem_s + lane_addr + c * 16, pp);   // P^T over consumed S^T columns
        tmem_st16(tmem_dp + lane_addr + c * 16, pd);  // dS^T over consumed dP^T columns
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
    }

    if (ok) ok = warp_all(mbar_wait(bar_o, (n_iter - 1) & 1, abort_flag));
    if (ok) {
      tc_fence_after_sync();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tmem_dv : tmem_dk;
        const float sc = which == 0 ? 1.f : a.scale;
        tmem_ld32(src + lane_addr, rs);
        tmem_ld32(src + lane_addr + 32, rp);
        tmem_wait_ld();
        if (j < a.S) {
          __nv_bfloat16* dst = which == 0 ? a.dv.row(b, g, j) : a.dk.row(b, g, j);
#pragma unroll
          for (int c = 0; c < 32; c += 8)
            store_bf16x8(dst + c, pack_bf16(__uint_as_float(rs[c]) * sc, __uint_as_float(rs[c + 1]) * sc),
                         pack_bf16(__uint_as_float(rs[c + 2]) * sc, __uint_as_float(rs[c + 3]) * sc),
                         pack_bf16(__uint_as_float(rs[c + 4]) * sc, __uint_as_float(rs[c + 5]) * sc),
                         pack_bf16(__uint_as_float(rs[c + 6]) * sc, __uint_as_float(rs[c + 7]) * sc));
#pragma unroll
          for (int c = 0; c < 32; c += 8)
            store_bf16x8(dst + 32 + c, pack_bf16(__uint_as_float(rp[c]) * sc, __uint_as_float(rp[c + 1]) * sc),
                         pack_bf16(__uint_as_float(rp[c + 2]) * sc, __uint_as_float(rp[c + 3]) * sc),
                         pack_bf16(__uint_as_float(rp[c + 4]) * sc, __uint_as_float(rp[c + 5]) * sc),
                         pack_bf16(__uint_as_float(rp[c + 6]) * sc, __uint_as_float(rp[c + 7]) * sc));
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, kDkvTmemCols);
  }
}

}  // namespace b200attn
