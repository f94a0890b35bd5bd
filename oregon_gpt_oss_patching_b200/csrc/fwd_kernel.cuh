// Forward attention kernel for sm_100a.
//
// One CTA = one 128-row query tile of one query head of one sequence.  Per visible
// 128-key tile:  S = Q K^T on tcgen05 (operands staged by TMA, accumulator in tensor
// memory), online softmax in registers with one thread per row (running max starts at the
// head's sink logit, the sink joins the denominator in the epilogue), P written back to
// tensor memory as bf16 and used as the A operand of  O_tile = P V.  Key tiles that are
// entirely masked (above the diagonal, left of the window, past the sequence end) are
// never loaded.  Computes what the reference's `_attn_fwd` does
// (attention_kernel.py:11-100), in the log2 domain.
//
// Warps 0-3: softmax + output accumulation (thread r owns row r = TMEM lane r).
// Warp 4, lane 0: TMA producer and MMA issuer.
// Two CTAs fit per SM (256 TMEM columns, 80 KB shared memory each), so one CTA's tensor
// work overlaps the other's softmax.
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kFwdStages = 2;
constexpr int kFwdTmemCols = 256;  // S: [0,128)  P: [128,192)  O tile: [192,256)

struct FwdSmem {
  alignas(1024) uint8_t q[kTileBytes];
  alignas(1024) uint8_t k[kFwdStages][kTileBytes];
  alignas(1024) uint8_t v[kFwdStages][kTileBytes];
  alignas(8) uint64_t bar_q;
  uint64_t bar_k[kFwdStages];
  uint64_t bar_v[kFwdStages];
  uint64_t bar_s;  // S ready in TMEM            (tcgen05.commit)
  uint64_t bar_p;  // P written by 128 threads   (count 128)
  uint64_t bar_o;  // O tile ready in TMEM       (tcgen05.commit)
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem* sm = reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / a.group;
  const int qt = gridDim.x - 1 - blockIdx.x;  // long (late) tiles first
  const int q0 = qt * kTile;
  const int len = seq_len(a, b);
  float* lse_row = a.lse + ((long long)(b * a.Hq + h)) * a.S_pad + q0;

  if (q0 >= len) {  // tile is padding only: define its output, no tensor work
    if (tid < kComputeThreads) {
      if (q0 + tid < a.S) zero_row(a.o.row(b, h, q0 + tid));
      lse_row[tid] = 0.f;
    }
    return;
  }

  const int hi = min(q0 + kTile - 1, len - 1);                         // last visible key
  const int lo = a.window ? max(0, q0 - a.window + 1) : 0;             // first visible key
  const int t_first = lo / kTile;
  const int nt = hi / kTile - t_first + 1;

  const uint32_t bar_q = smem_u32(&sm->bar_q), bar_s = smem_u32(&sm->bar_s), bar_p = smem_u32(&sm->bar_p),
                 bar_o = smem_u32(&sm->bar_o);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(smem_u32(&sm->bar_k[s]), 1);
      mbar_init(smem_u32(&sm->bar_v[s]), 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kComputeThreads);
    mbar_init(bar_o, 1);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_p = tmem + 128, tmem_o = tmem + 192;

  if (warp == 4) {
    // ------------------------------ producer + MMA issuer ------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(bar_q, kTileBytes);
      tma_load_4d(smem_u32(sm->q), &tm_q, bar_q, 0, q0, h, b);
      const int pre = nt < kFwdStages ? nt : kFwdStages;
      for (int s = 0; s < pre; ++s) {
        const int kv0 = (t_first + s) * kTile;
        mbar_arrive_expect_tx(smem_u32(&sm->bar_k[s]), kTileBytes);
        tma_load_4d(smem_u32(sm->k[s]), &tm_k, smem_u32(&sm->bar_k[s]), 0, kv0, g, b);
        mbar_arrive_expect_tx(smem_u32(&sm->bar_v[s]), kTileBytes);
        tma_load_4d(smem_u32(sm->v[s]), &tm_v, smem_u32(&sm->bar_v[s]), 0, kv0, g, b);
      }
      const uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      const uint64_t dq_desc = desc_kmajor(smem_u32(sm->q));
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      int issued = pre, k_waited = 0, v_waited = 0;  // K/V tile loads issued / seen complete
      for (int t = 0; ok && t < nt; ++t) {
        const int s = t % kFwdStages;
        const uint32_t ph = (t / kFwdStages) & 1;
        // S = Q K^T
        if (!(ok = mbar_wait(smem_u32(&sm->bar_k[s]), ph, abort_flag))) break;
        k_waited = t + 1;
        tc_fence_after_sync();
        const uint64_t dk_desc = desc_kmajor(smem_u32(sm->k[s]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_s, dq_desc + kk * kDescKStepKMajor, dk_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
        umma_commit(bar_s);
        // O_tile = P V   (P from tensor memory)
        if (!(ok = mbar_wait(smem_u32(&sm->bar_v[s]), ph, abort_flag))) break;
        v_waited = t + 1;
        if (!(ok = mbar_wait(bar_p, t & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t dv_desc = desc_mnmajor(smem_u32(sm->v[s]));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(tmem_o, tmem_p + kk * 8, dv_desc + kk * kDescKStepMNMajor, idesc_pv, kk > 0);
        umma_commit(bar_o);
        // refill this stage once the tensor core is done with it
        if (t + kFwdStages < nt) {
          if (!(ok = mbar_wait(bar_o, t & 1, abort_flag))) break;
          const int kv0 = (t_first + t + kFwdStages) * kTile;
          mbar_arrive_expect_tx(smem_u32(&sm->bar_k[s]), kTileBytes);
          tma_load_4d(smem_u32(sm->k[s]), &tm_k, smem_u32(&sm->bar_k[s]), 0, kv0, g, b);
          mbar_arrive_expect_tx(smem_u32(&sm->bar_v[s]), kTileBytes);
          tma_load_4d(smem_u32(sm->v[s]), &tm_v, smem_u32(&sm->bar_v[s]), 0, kv0, g, b);
          ++issued;
        }
      }
      if (!ok) {
        report_abort(a);
        // give copies that are still in flight a bounded chance to land before the CTA exits
        for (int t = k_waited; t < issued; ++t)
          mbar_wait_drain(smem_u32(&sm->bar_k[t % kFwdStages]), (t / kFwdStages) & 1);
        for (int t = v_waited; t < issued; ++t)
          mbar_wait_drain(smem_u32(&sm->bar_v[t % kFwdStages]), (t / kFwdStages) & 1);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax ------------------------------------
    const int i = q0 + tid;                               // this thread's query position
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;  // this warp's TMEM lane quarter
    const float sink2 = a.sinks[h] * kLog2e;
    float m = sink2;   // running max (log2 domain), starts at the sink logit
    float l = 0.f;     // running denominator without the sink
    float acc[kHeadDim];
#pragma unroll
    for (int c = 0; c < kHeadDim; ++c) acc[c] = 0.f;
    bool ok = true;
    uint32_t r[32];

    for (int t = 0; t < nt; ++t) {
      const int kv0 = (t_first + t) * kTile;
      const bool need_mask = tile_needs_mask(q0, kv0, a.window, len);
      if (!(ok = warp_all(mbar_wait(bar_s, t & 1, abort_flag)))) break;
      tc_fence_after_sync();
      // pass 1: row maximum of the visible logits
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(tmem_s + lane_addr + c * 32, r);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (visible(i, kv0 + c * 32 + e, a.window, len)) mx = fmaxf(mx, __uint_as_float(r[e]));
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
        }
      }
      const float m_new = fmaxf(m, mx * a.scale_log2);
      const float alpha = fast_exp2(m - m_new);
      // pass 2: p = 2^(s*scale - m), row sum, P -> TMEM as bf16
      float rowsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld32(tmem_s + lane_addr + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(r[e]), a.scale_log2, -m_new));
          float p1 = fast_exp2(fmaf(__uint_as_float(r[e + 1]), a.scale_log2, -m_new));
          if (need_mask) {
            if (!visible(i, kv0 + c * 32 + e, a.window, len)) p0 = 0.f;
            if (!visible(i, kv0 + c * 32 + e + 1, a.window, len)) p1 = 0.f;
          }
          rowsum += p0 + p1;
          pk[e >> 1] = pack_bf16(p0, p1);
        }
        tmem_st16(tmem_p + lane_addr + c * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
      l = l * alpha + rowsum;
      m = m_new;
      // O += P V
      if (!(ok = warp_all(mbar_wait(bar_o, t & 1, abort_flag)))) break;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld32(tmem_o + lane_addr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[c * 32 + e] = fmaf(acc[c * 32 + e], alpha, __uint_as_float(r[e]));
      }
      tc_fence_before_sync();
    }

    if (ok) {
      const float z = l + fast_exp2(sink2 - m);   // the sink joins the denominator only
      const float inv = 1.f / z;
      if (i < a.S) {
        __nv_bfloat16* dst = a.o.row(b, h, i);
#pragma unroll
        for (int c = 0; c < kHeadDim; c += 8)
          store_bf16x8(dst + c, pack_bf16(acc[c] * inv, acc[c + 1] * inv), pack_bf16(acc[c + 2] * inv, acc[c + 3] * inv),
                       pack_bf16(acc[c + 4] * inv, acc[c + 5] * inv), pack_bf16(acc[c + 6] * inv, acc[c + 7] * inv));
      }
      lse_row[tid] = (i < len) ? (m + log2f(z)) * kLn2 : 0.f;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
}

}  // namespace b200attn
