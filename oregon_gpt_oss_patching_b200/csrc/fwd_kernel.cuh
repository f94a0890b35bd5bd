// Forward attention kernel for sm_100a.
//
// One CTA = one 128-row query tile of TWO query heads of the same KV group (tile A and tile
// B), so that every K/V tile staged in shared memory by TMA feeds two heads; the other heads
// of the group run in neighbouring CTAs and find the same K/V tiles in L2.  (With an odd group
// size only tile A is active.)  Per visible 128-key tile and per query tile:
//     S = Q K^T                      tcgen05.mma, fp32 accumulator in tensor memory
//     P = 2^(S*scale*log2e - m)      one thread per row, online softmax in registers
//     O_tile = P V                   tcgen05.mma with P (bf16) as the A operand from tensor memory
//     acc = acc * alpha + O_tile     in registers
// The running maximum m starts at the head's sink logit; the sink joins the denominator in the
// epilogue and carries no value.  Computes what the reference's `_attn_fwd` does
// (attention_kernel.py:11-100), in the log2 domain.  Key tiles that are entirely masked (above
// the diagonal, left of the window, past the sequence end) are never loaded.
//
// Warp roles: warps 0-3 softmax of tile A, warps 4-7 softmax of tile B (thread r owns row r =
// TMEM lane r), warp 8 lane 0 issues every MMA, warp 9 lane 0 issues every TMA load.  While one
// tile's threads run their softmax the tensor core works for the other tile.
//
// A softmax thread holds its whole 128-column row of S in registers (one burst of tensor-memory
// loads per tile), so the row maximum, the exponentials and the row sum are computed without a
// second read.  The register file is re-partitioned with setmaxnreg: the two softmax warpgroups
// take 224 registers per thread, the warpgroup holding the MMA and TMA warps keeps 56
// (2*128*224 + 128*56 = 384*168, the pool the CTA is launched with).
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kFwdStages = 3;
constexpr int kFwdThreads = 384;  // 3 warpgroups: softmax A, softmax B, {MMA warp, TMA warp, 2 idle warps}
constexpr int kFwdTmemCols = 512;
// tensor-memory columns: S_A [0,128) S_B [128,256) P_A [256,320) P_B [320,384) O_A [384,448) O_B [448,512)

struct FwdSmem {
  alignas(1024) uint8_t q[2][kTileBytes];
  alignas(1024) uint8_t k[kFwdStages][kTileBytes];
  alignas(1024) uint8_t v[kFwdStages][kTileBytes];
  alignas(8) uint64_t bar_q;
  uint64_t bar_kv_full[kFwdStages];
  uint64_t bar_kv_empty[kFwdStages];
  uint64_t bar_s_full[2];   // S of tile X ready            (tcgen05.commit)
  uint64_t bar_p_full[2];   // P of tile X written          (128 arrivals)
  uint64_t bar_o_full[2];   // O_tile of tile X ready       (tcgen05.commit)
  uint64_t bar_o_empty[2];  // O_tile of tile X consumed    (128 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;         // K/V tile loads the loader has issued so far (for the abort drain)
};

// acc = acc * alpha + O_tile for the 64 output columns of this thread's row
__device__ __forceinline__ void fwd_accumulate(float (&acc)[kHeadDim], uint32_t tmem_o_row, float alpha) {
  uint32_t r0[32], r1[32];
  tmem_ld32(tmem_o_row, r0);
  tmem_ld32(tmem_o_row + 32, r1);
  tmem_wait_ld();
  if (alpha == 1.f) {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      acc[e] += __uint_as_float(r0[e]);
      acc[32 + e] += __uint_as_float(r1[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      acc[e] = fmaf(acc[e], alpha, __uint_as_float(r0[e]));
      acc[32 + e] = fmaf(acc[32 + e], alpha, __uint_as_float(r1[e]));
    }
  }
}

// Softmax of one 128-column row held in registers: returns the new running maximum, writes
// P (bf16) to tensor memory and adds the row sum.
template <bool kMask>
__device__ __forceinline__ float fwd_softmax_row(uint32_t tmem_s_row, uint32_t tmem_p_row, float scale_log2, float m,
                                                 int i, int kv0, int window, int len, float& rowsum) {
  uint32_t s[4][32];
#pragma unroll
  for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s_row + c * 32, s[c]);
  tmem_wait_ld();
  if (kMask) {  // branch-free: one visibility bit mask per 32 keys, then selects
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t bits = visible_keys32(i, kv0 + c * 32, window, len);
#pragma unroll
      for (int e = 0; e < 32; ++e) s[c][e] = (bits >> e) & 1u ? s[c][e] : 0xff800000u;  // -inf
    }
  }
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int e = 0; e < 32; ++e) mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(s[c][e]));
  const float m_new = fmaxf(m, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2);
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t pk[16];
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
      const float p0 = fast_exp2(fmaf(__uint_as_float(s[c][e]), scale_log2, -m_new));
      const float p1 = fast_exp2(fmaf(__uint_as_float(s[c][e + 1]), scale_log2, -m_new));
      sum[(e >> 1) & 3] += p0 + p1;
      pk[e >> 1] = pack_bf16(p0, p1);
    }
    tmem_st16(tmem_p_row + c * 16, pk);
  }
  rowsum = (sum[0] + sum[1]) + (sum[2] + sum[3]);
  return m_new;
}

__device__ __forceinline__ void setmaxnreg_inc_224() { asm volatile("setmaxnreg.inc.sync.aligned.u32 224;"); }
__device__ __forceinline__ void setmaxnreg_dec_56() { asm volatile("setmaxnreg.dec.sync.aligned.u32 56;"); }

__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem* sm = reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int n_act = (a.group % 2 == 0) ? 2 : 1;   // query heads (tiles) handled by this CTA
  const int h0 = blockIdx.y * n_act;
  const int g = h0 / a.group;
  const int qt = gridDim.x - 1 - blockIdx.x;      // long (late) tiles first
  const int q0 = qt * kTile;
  const int len = seq_len(a, b);

  if (q0 >= len) {  // tile is padding only: define its output, no tensor work
    if (tid < n_act * kComputeThreads) {
      const int x = tid >> 7, r = tid & 127;
      if (q0 + r < a.S) zero_row(a.o.row(b, h0 + x, q0 + r));
      a.lse[((long long)(b * a.Hq + h0 + x)) * a.S_pad + q0 + r] = 0.f;
    }
    return;
  }

  const int hi = min(q0 + kTile - 1, len - 1);              // last visible key
  const int lo = a.window ? max(0, q0 - a.window + 1) : 0;  // first visible key
  const int t_first = lo / kTile;
  const int nt = hi / kTile - t_first + 1;

  const uint32_t bar_q = smem_u32(&sm->bar_q);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(smem_u32(&sm->bar_kv_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_kv_empty[s]), 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&sm->bar_s_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_p_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_o_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_o_empty[x]), kComputeThreads);
    }
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;

  if (warp >= 8) {
  setmaxnreg_dec_56();

  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(bar_q, n_act * kTileBytes);
      for (int x = 0; x < n_act; ++x) tma_load_4d(smem_u32(sm->q[x]), &tm_q, bar_q, 0, q0, h0 + x, b);
      for (int t = 0; t < nt; ++t) {
        const int s = t % kFwdStages;
        if (t >= kFwdStages && !mbar_wait(smem_u32(&sm->bar_kv_empty[s]), ((t / kFwdStages) - 1) & 1, abort_flag)) {
          report_abort(a);
          break;
        }
        const int kv0 = (t_first + t) * kTile;
        const uint32_t bar = smem_u32(&sm->bar_kv_full[s]);
        mbar_arrive_expect_tx(bar, 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, kv0, g, b);
        tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, kv0, g, b);
        *reinterpret_cast<volatile int*>(&sm->loads_issued) = t + 1;
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      uint64_t q_desc[2];
      for (int x = 0; x < 2; ++x) q_desc[x] = desc_kmajor(smem_u32(sm->q[x]));
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      if (ok) ok = mbar_wait(smem_u32(&sm->bar_kv_full[0]), 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[0]));
        for (int x = 0; x < n_act; ++x) {
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem + x * 128, q_desc[x] + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
          umma_commit(smem_u32(&sm->bar_s_full[x]));
        }
      }
      // Serve whichever tile has its P ready first, so that the two softmax warpgroups fall into
      // anti-phase (one computes while the tensor core works for the other) instead of lockstep.
      int next_t[2] = {0, n_act == 2 ? 0 : nt};   // next key tile whose P V is to be issued, per tile
      long long t_idle0 = 0;
      uint32_t idle = 0;
      while (ok && (next_t[0] < nt || next_t[1] < nt)) {
        bool progressed = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int t = next_t[x];
          if (t >= nt) continue;
          if (!mbar_test_wait(smem_u32(&sm->bar_p_full[x]), t & 1)) continue;
          if (t >= 1 && !mbar_test_wait(smem_u32(&sm->bar_o_empty[x]), (t - 1) & 1)) continue;
          const int sn = (t + 1) % kFwdStages;
          if (t + 1 < nt && !mbar_test_wait(smem_u32(&sm->bar_kv_full[sn]), ((t + 1) / kFwdStages) & 1)) continue;
          tc_fence_after_sync();
          const int s = t % kFwdStages;
          const uint64_t v_desc = desc_mnmajor(smem_u32(sm->v[s]));
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ts(tmem + 384 + x * 64, tmem + 256 + x * 64 + kk * 8, v_desc + kk * kDescKStepMNMajor, idesc_pv, kk > 0);
          umma_commit(smem_u32(&sm->bar_o_full[x]));
          // S of the next key tile goes behind P V in the pipe: when it is ready, P has been read
          // and the softmax threads may overwrite the P columns.
          if (t + 1 < nt) {
            const uint64_t kn_desc = desc_kmajor(smem_u32(sm->k[sn]));
#pragma unroll
            for (int kk = 0; kk < kHeadDim / 16; ++kk)
              umma_ss(tmem + x * 128, q_desc[x] + kk * kDescKStepKMajor, kn_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
            umma_commit(smem_u32(&sm->bar_s_full[x]));
          }
          next_t[x] = t + 1;
          // K[s], V[s] are free once both tiles' MMAs on them retire
          if (next_t[x ^ 1] > t) umma_commit(smem_u32(&sm->bar_kv_empty[s]));
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if ((++idle & 1023u) == 0u) {   // bounded: give up after ~2 s without progress
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
  }
  } else {
  setmaxnreg_inc_224();
  if (warp < 4 * n_act) {
    // -------------------------------------- softmax --------------------------------------
    const int x = warp >> 2;                                      // tile A or B
    const int h = h0 + x;
    const int r = tid & 127;
    const int i = q0 + r;                                         // this thread's query position
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;   // this warp's TMEM lane quarter
    const uint32_t tmem_s_row = tmem + x * 128 + lane_addr;
    const uint32_t tmem_p_row = tmem + 256 + x * 64 + lane_addr;
    const uint32_t tmem_o_row = tmem + 384 + x * 64 + lane_addr;
    const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_p = smem_u32(&sm->bar_p_full[x]),
                   bar_o = smem_u32(&sm->bar_o_full[x]), bar_oe = smem_u32(&sm->bar_o_empty[x]);
    const float sink2 = a.sinks[h] * kLog2e;
    float m = sink2;         // reference maximum of the exponents (log2 domain), starts at the sink logit
    float l = 0.f;           // running denominator without the sink, relative to m
    float alpha = 1.f;       // rescale factor of the latest key tile
    float acc[kHeadDim];
#pragma unroll
    for (int c = 0; c < kHeadDim; ++c) acc[c] = 0.f;
    bool ok = true;

    for (int t = 0; t < nt; ++t) {
      const int kv0 = (t_first + t) * kTile;
      const bool need_mask = tile_needs_mask(q0, kv0, a.window, len);
      if (!(ok = warp_all(mbar_wait(bar_s, t & 1, abort_flag)))) break;
      if (t > 0) {
        // P V of the previous key tile retired before this S did: fold it in first
        if (!(ok = warp_all(mbar_wait(bar_o, (t - 1) & 1, abort_flag)))) break;
        tc_fence_after_sync();
        fwd_accumulate(acc, tmem_o_row, alpha);
        tc_fence_before_sync();
        mbar_arrive(bar_oe);
      }
      tc_fence_after_sync();
      float rowsum;
      const float m_new = need_mask
          ? fwd_softmax_row<true>(tmem_s_row, tmem_p_row, a.scale_log2, m, i, kv0, a.window, len, rowsum)
          : fwd_softmax_row<false>(tmem_s_row, tmem_p_row, a.scale_log2, m, i, kv0, a.window, len, rowsum);
      alpha = fast_exp2(m - m_new);
      m = m_new;
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
      l = l * alpha + rowsum;
    }
    if (ok) ok = warp_all(mbar_wait(bar_o, (nt - 1) & 1, abort_flag));
    if (ok) {
      tc_fence_after_sync();
      fwd_accumulate(acc, tmem_o_row, alpha);
      const float z = l + fast_exp2(sink2 - m);   // the sink joins the denominator only
      const float inv = 1.f / z;
      if (i < a.S) {
        __nv_bfloat16* dst = a.o.row(b, h, i);
#pragma unroll
        for (int c = 0; c < kHeadDim; c += 8)
          store_bf16x8(dst + c, pack_bf16(acc[c] * inv, acc[c + 1] * inv), pack_bf16(acc[c + 2] * inv, acc[c + 3] * inv),
                       pack_bf16(acc[c + 4] * inv, acc[c + 5] * inv), pack_bf16(acc[c + 6] * inv, acc[c + 7] * inv));
      }
      a.lse[((long long)(b * a.Hq + h)) * a.S_pad + i] = (i < len) ? (m + log2f(z)) * kLn2 : 0.f;
    }
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued;
    mbar_wait_drain(bar_q, 0);
    for (int t = max(0, issued - kFwdStages); t < issued; ++t)
      mbar_wait_drain(smem_u32(&sm->bar_kv_full[t % kFwdStages]), (t / kFwdStages) & 1);
  }
}

}  // namespace b200attn
