// Forward kernel for short key ranges (sliding-window layers), sm_100a.
//
// Same arithmetic as attn_fwd_kernel (see fwd_kernel.cuh), laid out for two CTAs per SM: with a
// 128-key window a query tile sees at most two key tiles, so a CTA's life is dominated by its
// prologue (set-up, first TMA round trip), the S -> softmax -> P V dependency chain of those two
// tiles and its epilogue, none of which one CTA can overlap with anything.  Half the footprint
// -- one query head, 256 threads, 256 tensor-memory columns, 80 KB of shared memory -- lets a
// second CTA fill those gaps.  Both key tiles get their own shared-memory stage (no ring).
#pragma once
#include "attn_common.cuh"
#include "attn_common.cuh"

namespace b200attn {

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


constexpr int kFwdsStages = 2;      // = the most key tiles a launch of this kernel may need per query tile
constexpr int kFwdsThreads = 256;
constexpr int kFwdsTmemCols = 256;  // S [0,128)  P bf16 [128,192)  O tile [192,256)

struct FwdsSmem {
  alignas(1024) uint8_t q[kTileBytes];
  alignas(1024) uint8_t k[kFwdsStages][kTileBytes];
  alignas(1024) uint8_t v[kFwdsStages][kTileBytes];
  alignas(8) uint64_t bar_q;
  uint64_t bar_kv_full[kFwdsStages];
  uint64_t bar_s_full;   // S ready            (tcgen05.commit)
  uint64_t bar_p_full;   // P written          (128 arrivals)
  uint64_t bar_o_full;   // O tile ready       (tcgen05.commit)
  uint64_t bar_o_empty;  // O tile consumed    (128 arrivals)
  uint32_t tmem_base;
  int abort_flag;
};

// Softmax of one 128-column row in two 64-column halves (64 registers live): a first sweep for
// the row maximum, a second one that re-reads S, exponentiates and writes P.
template <bool kMask>
__device__ __forceinline__ float fwds_softmax_row(uint32_t tmem_s_row, uint32_t tmem_p_row, float scale_log2, float m,
                                                  int i, int kv0, int window, int len, float& rowsum) {
  uint32_t s[2][32];
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    tmem_ld32(tmem_s_row + half * 64, s[0]);
    tmem_ld32(tmem_s_row + half * 64 + 32, s[1]);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint32_t bits = kMask ? visible_keys32(i, kv0 + half * 64 + c * 32, window, len) : 0xffffffffu;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float x = __uint_as_float(s[c][e]);
        mx[e & 3] = fmaxf(mx[e & 3], kMask ? ((bits >> e) & 1u ? x : -INFINITY) : x);
      }
    }
  }
  const float m_new = fmaxf(m, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2);
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    tmem_ld32(tmem_s_row + half * 64, s[0]);
    tmem_ld32(tmem_s_row + half * 64 + 32, s[1]);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint32_t bits = kMask ? visible_keys32(i, kv0 + half * 64 + c * 32, window, len) : 0xffffffffu;
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float p0 = fast_exp2(fmaf(__uint_as_float(s[c][e]), scale_log2, -m_new));
        float p1 = fast_exp2(fmaf(__uint_as_float(s[c][e + 1]), scale_log2, -m_new));
        if (kMask) {  // selects, not branches
          p0 = (bits >> e) & 1u ? p0 : 0.f;
          p1 = (bits >> (e + 1)) & 1u ? p1 : 0.f;
        }
        sum[(e >> 1) & 3] += p0 + p1;
        pk[e >> 1] = pack_bf16(p0, p1);
      }
      tmem_st16(tmem_p_row + half * 32 + c * 16, pk);
    }
  }
  rowsum = (sum[0] + sum[1]) + (sum[2] + sum[3]);
  return m_new;
}

__device__ __forceinline__ void setmaxnreg_inc_192() { asm volatile("setmaxnreg.inc.sync.aligned.u32 192;"); }
__device__ __forceinline__ void setmaxnreg_dec_64() { asm volatile("setmaxnreg.dec.sync.aligned.u32 64;"); }

__global__ void __launch_bounds__(kFwdsThreads, 2)
attn_fwd_small_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdsSmem* sm = reinterpret_cast<FwdsSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int h = blockIdx.y;
  const int g = h / a.group;
  const int qt = gridDim.x - 1 - blockIdx.x;
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

  const int hi = min(q0 + kTile - 1, len - 1);              // last visible key
  const int lo = a.window ? max(0, q0 - a.window + 1) : 0;  // first visible key
  const int t_first = lo / kTile;
  const int nt = hi / kTile - t_first + 1;                  // <= kFwdsStages (the host checks the window)

  const uint32_t bar_q = smem_u32(&sm->bar_q), bar_s = smem_u32(&sm->bar_s_full), bar_p = smem_u32(&sm->bar_p_full),
                 bar_o = smem_u32(&sm->bar_o_full), bar_oe = smem_u32(&sm->bar_o_empty);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kFwdsStages; ++s) mbar_init(smem_u32(&sm->bar_kv_full[s]), 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kComputeThreads);
    mbar_init(bar_o, 1);
    mbar_init(bar_oe, kComputeThreads);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdsTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;

  if (warp >= 4) {
  setmaxnreg_dec_64();
  if (warp == 5) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(bar_q, kTileBytes);
      tma_load_4d(smem_u32(sm->q), &tm_q, bar_q, 0, q0, h, b);
      for (int t = 0; t < nt; ++t) {
        const int kv0 = (t_first + t) * kTile;
        const uint32_t bar = smem_u32(&sm->bar_kv_full[t]);
        mbar_arrive_expect_tx(bar, 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->k[t]), &tm_k, bar, 0, kv0, g, b);
        tma_load_4d(smem_u32(sm->v[t]), &tm_v, bar, 0, kv0, g, b);
      }
    }
    __syncwarp();
  } else if (warp == 4) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      const uint64_t q_desc = desc_kmajor(smem_u32(sm->q));
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      for (int t = 0; ok && t < nt; ++t) {
        // S(t): the tile's K/V have landed; when t > 0 it goes behind P V of the previous tile in the pipe
        if (!(ok = mbar_wait(smem_u32(&sm->bar_kv_full[t]), 0, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[t]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
        umma_commit(bar_s);
        if (!(ok = mbar_wait(bar_p, t & 1, abort_flag))) break;
        if (t >= 1 && !(ok = mbar_wait(bar_oe, (t - 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t v_desc = desc_mnmajor(smem_u32(sm->v[t]));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(tmem + 192, tmem + 128 + kk * 8, v_desc + kk * kDescKStepMNMajor, idesc_pv, kk > 0);
        umma_commit(bar_o);
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_192();
  {
    // -------------------------------------- softmax --------------------------------------
    const int i = q0 + tid;                               // this thread's query position
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;  // this warp's TMEM lane quarter
    const uint32_t tmem_s_row = tmem + lane_addr, tmem_p_row = tmem + 128 + lane_addr, tmem_o_row = tmem + 192 + lane_addr;
    const float sink2 = a.sinks[h] * kLog2e;
    float m = sink2;    // running maximum (log2 domain), starts at the sink logit
    float l = 0.f;      // running denominator without the sink, relative to m
    float alpha = 1.f;  // rescale factor of the latest key tile
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
          ? fwds_softmax_row<true>(tmem_s_row, tmem_p_row, a.scale_log2, m, i, kv0, a.window, len, rowsum)
          : fwds_softmax_row<false>(tmem_s_row, tmem_p_row, a.scale_log2, m, i, kv0, a.window, len, rowsum);
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
      lse_row[tid] = (i < len) ? (m + log2f(z)) * kLn2 : 0.f;
    }
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, kFwdsTmemCols);
  }
  if (sm->abort_flag && tid == 5 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    mbar_wait_drain(bar_q, 0);
    for (int t = 0; t < nt; ++t) mbar_wait_drain(smem_u32(&sm->bar_kv_full[t]), 0);
  }
}

}  // namespace b200attn
