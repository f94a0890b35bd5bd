// Forward attention kernel for sm_100a.
//
// One work item = one 128-row query tile of TWO query heads of the same KV group (tile A and tile
// B), so that every K/V tile staged in shared memory by TMA feeds two heads; the other heads
// of the group run in neighbouring CTAs and find the same K/V tiles in L2.  (With an odd group
// size only tile A is active.)  Per visible 128-key tile and per query tile:
//     S = Q K^T                      tcgen05.mma, fp32 accumulator in tensor memory
//     P = 2^(S*scale*log2e - m)      one thread per row, online softmax in registers
//     O += P V                       tcgen05.mma with P (bf16) as the A operand from tensor memory,
//                                    accumulating in tensor memory
// The reference maximum m of a row starts at the head's sink logit and is only raised when the
// row maximum has grown by more than 2^8 (the exponentials stay far inside the fp32/bf16 range and
// the final normalisation uses the same m, so the result does not depend on when m is raised);
// raising it rescales the row of O in tensor memory, which is rare after the first key tiles.
// The sink joins the denominator in the epilogue and carries no value.  Computes what the reference's `_attn_fwd` does
// (attention_kernel.py:11-100), in the log2 domain.  Key tiles that are entirely masked (above
// the diagonal, left of the window, past the sequence end) are never loaded.
//
// Warp roles: warps 0-3 softmax of tile A, warps 4-7 softmax of tile B (thread r owns row r =
// TMEM lane r), warp 8 lane 0 issues tile A's MMAs, warp 10 lane 0 tile B's, warp 9 lane 0 every TMA load.  S of the
// next key tile is issued as soon as the softmax threads have pulled the current S into registers,
// so it is computed underneath the exponentials; P V follows when P is written.
//
// A softmax thread holds its whole 128-column row of S in registers (one burst of tensor-memory
// loads per tile), so the row maximum, the exponentials and the row sum are computed without a
// second read.  The register file is re-partitioned with setmaxnreg: the two softmax warpgroups
// take 216 registers per thread, the warpgroup holding the MMA and TMA warps keeps 72
// (2*128*216 + 128*72 = 384*168, the pool the CTA is launched with).
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kFwdStages = 4;
constexpr int kFwdThreads = 384;  // 3 warpgroups: softmax A, softmax B, {MMA warp A, TMA warp, MMA warp B, idle warp}
constexpr int kFwdTmemCols = 512;
// tensor-memory columns: S_A [0,128) S_B [128,256) P_A [256,320) P_B [320,384) O_A [384,448) O_B [448,512)

// shared memory of the persistent kernel
struct FwdSmem {
  alignas(1024) uint8_t q[2][2][kTileBytes];   // [buffer][query tile A/B]: the next work item's Q lands while this one runs
  alignas(1024) uint8_t k[kFwdStages][kTileBytes];
  alignas(1024) uint8_t v[kFwdStages][kTileBytes];
  alignas(8) uint64_t bar_q_full[2];   // Q of a buffer landed
  uint64_t bar_q_empty[2];             // every S MMA reading a Q buffer retired   (tcgen05.commit per tile)
  uint64_t bar_kv_full[kFwdStages];
  uint64_t bar_kv_empty[kFwdStages];
  uint64_t bar_s_full[2];   // S of tile X ready                    (tcgen05.commit)
  uint64_t bar_s_empty[2];  // S of tile X copied into registers    (128 arrivals)
  uint64_t bar_p_full[2];   // P of tile X written                  (128 arrivals)
  uint64_t bar_o_full[2];   // P V of tile X retired: P free, O current (tcgen05.commit)
  uint64_t bar_o_free[2];   // O of tile X read by the epilogue     (128 arrivals)
  uint64_t bar_exp[2];      // tile X may run its exponentials       (128 arrivals of the other tile)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;         // K/V tile loads the loader has issued so far (for the abort drain)
  int q_loads_issued;       // Q loads (work items) issued so far
};

// shared memory of the one-item-per-CTA kernel
struct FwdOneSmem {
  alignas(1024) uint8_t q[2][kTileBytes];
  alignas(1024) uint8_t k[kFwdStages][kTileBytes];
  alignas(1024) uint8_t v[kFwdStages][kTileBytes];
  alignas(8) uint64_t bar_q;
  uint64_t bar_kv_full[kFwdStages];
  uint64_t bar_kv_empty[kFwdStages];
  uint64_t bar_s_full[2];   // S of tile X ready                    (tcgen05.commit)
  uint64_t bar_s_empty[2];  // S of tile X copied into registers    (128 arrivals)
  uint64_t bar_p_full[2];   // P of tile X written                  (128 arrivals)
  uint64_t bar_o_full[2];   // P V of tile X retired: P free, O current (tcgen05.commit)
  uint64_t bar_exp[2];      // tile X may run its exponentials       (128 arrivals of the other tile)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;         // K/V tile loads the loader has issued so far (for the abort drain)
};

// O_row *= alpha for the 64 output columns of this thread's row, in tensor memory
__device__ __forceinline__ void fwd_rescale_o(uint32_t tmem_o_row, float alpha) {
  uint32_t r0[32], r1[32];
  tmem_ld32(tmem_o_row, r0);
  tmem_ld32(tmem_o_row + 32, r1);
  tmem_wait_ld();
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    r0[e] = __float_as_uint(__uint_as_float(r0[e]) * alpha);
    r1[e] = __float_as_uint(__uint_as_float(r1[e]) * alpha);
  }
  tmem_st32(tmem_o_row, r0);
  tmem_st32(tmem_o_row + 32, r1);
  tmem_wait_st();
}

// Largest growth of the row maximum (log2 domain) tolerated before the reference maximum is raised.
constexpr float kFwdRescaleThreshold = 8.f;

struct FwdRowState {
  float m;   // reference maximum of the exponents (log2 domain)
  float l;   // running denominator without the sink, relative to m
};

__device__ __forceinline__ float fwd_row_max(const uint32_t (&s)[4][32]) {
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int e = 0; e < 32; e += 2)
      mx[(e >> 1) & 3] = fmax3(mx[(e >> 1) & 3], __uint_as_float(s[c][e]), __uint_as_float(s[c][e + 1]));
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// How a 32-key chunk looks to the 32 rows of this warp: the same answer in every lane, so branches on
// it are warp-uniform.  On the diagonal and at the window's edge most chunks are either visible to
// all 32 rows (no masking work) or to none (no exponentials at all: P = 0).
enum : int { kChunkNone = 0, kChunkAll = 1, kChunkSome = 2 };
__device__ __forceinline__ int fwd_chunk_kind(uint32_t bits) {
  if (__all_sync(0xffffffffu, bits == 0u)) return kChunkNone;
  if (__all_sync(0xffffffffu, bits == 0xffffffffu)) return kChunkAll;
  return kChunkSome;
}
__device__ __forceinline__ void fwd_mask_bits(uint32_t (&sc)[32], uint32_t bits) {
#pragma unroll
  for (int e = 0; e < 32; ++e) sc[e] = (bits >> e) & 1u ? sc[e] : 0xff800000u;  // -inf
}

// P = 2^(S*scale*log2e - m_ref) of one 32-key chunk of a row: packed to bf16, row sum and (when
// kWithMax) row maximum of S accumulated.  Exponentials, sum, packing and maximum are interleaved
// element by element (packed fp32 pairs where the hardware has them), so that the special-function
// unit, the bottleneck, is fed all the time instead of idling during a separate maximum pass.
template <bool kWithMax>
__device__ __forceinline__ void fwd_exp_chunk(const uint32_t (&sc)[32], float2 scale2, float2 neg_m2, uint32_t (&pk)[16],
                                              float2 (&sum)[4], float (&mx)[4]) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    const float s0 = __uint_as_float(sc[e]), s1 = __uint_as_float(sc[e + 1]);
    const float2 x = __ffma2_rn(make_float2(s0, s1), scale2, neg_m2);
    const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
    sum[(e >> 1) & 3] = __fadd2_rn(sum[(e >> 1) & 3], p);
    pk[e >> 1] = pack_bf16(p.x, p.y);
    if (kWithMax) mx[(e >> 1) & 3] = fmax3(mx[(e >> 1) & 3], s0, s1);
  }
}

__device__ __forceinline__ float fwd_sum4(const float2 (&sum)[4]) {
  return ((sum[0].x + sum[0].y) + (sum[1].x + sum[1].y)) + ((sum[2].x + sum[2].y) + (sum[3].x + sum[3].y));
}

// One key tile of one 128-column row: pulls S into registers (and releases the S columns), writes
// P as bf16 to tensor memory and adds the row sum.  After the first key tile the exponentials are
// taken against the current reference maximum right away, 32 keys at a time while the next 32
// scores are on their way from tensor memory, with the row maximum computed alongside; only when
// the row maximum turns out to exceed the reference by more than the threshold (rare) is the
// reference raised: the row of O in tensor memory and this tile's P (already bf16) are multiplied
// by 2^(old - new).  P is stored only after the whole row is done, when P V of the previous key tile
// has certainly left the P columns, so the softmax threads never stand waiting for the tensor core.  `t` is the
// key-tile counter of this query tile (kClassify: 32-key chunks no row of the warp can see are skipped
// -- worth it where most tiles are partly masked, i.e. in sliding-window layers), `prev_parity` the phase of bar_o that the previous key tile's
// P V completes.  Returns false when a bounded wait was abandoned.
template <bool kMask, bool kClassify>
__device__ __forceinline__ bool fwd_softmax_tile(FwdRowState& st, int t, uint32_t tmem_s_row, uint32_t tmem_p_row,
                                                 uint32_t tmem_o_row, uint32_t bar_s_empty, uint32_t bar_o,
                                                 uint32_t prev_parity, uint32_t bar_exp_mine, uint32_t exp_parity, uint32_t bar_exp_other,
                                                 float scale_log2, int i, int kv0, int window, int len,
                                                 volatile int* abort_flag) {
  uint32_t s[4][32];
  const float2 scale2 = make_float2(scale_log2, scale_log2);
  float2 sum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  if (t == 0) {
    // nothing accumulated yet: take the whole row, adopt its maximum (the reference starts at the
    // sink logit), then the exponentials
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s_row + c * 32, s[c]);
    tmem_wait_ld();
    tc_fence_before_sync();
    mbar_arrive(bar_s_empty);   // the tensor core may overwrite S with the next key tile's scores
    int kind[4] = {kChunkAll, kChunkAll, kChunkAll, kChunkAll};
    if (kMask) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t bits = visible_keys32(i, kv0 + c * 32, window, len);
        kind[c] = kClassify ? fwd_chunk_kind(bits) : kChunkSome;
        if (kind[c] != kChunkAll) fwd_mask_bits(s[c], bits);   // (a chunk nobody sees becomes -inf: out of the maximum)
      }
    }
    st.m = fmaxf(st.m, fwd_row_max(s) * scale_log2);
    const float2 neg_m2 = make_float2(-st.m, -st.m);
    if (bar_exp_mine != 0u && !warp_all(mbar_wait(bar_exp_mine, exp_parity, abort_flag))) return false;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[16];
      if (c == 1 && bar_exp_other != 0u) mbar_arrive(bar_exp_other);
      if (kMask && kClassify && kind[c] == kChunkNone) {
#pragma unroll
        for (int k = 0; k < 16; ++k) pk[k] = 0u;
      } else {
        fwd_exp_chunk<false>(s[c], scale2, neg_m2, pk, sum, mx);
      }
      tmem_st16(tmem_p_row + c * 16, pk);
    }
  } else {
    const float2 neg_m2 = make_float2(-st.m, -st.m);
    uint32_t pk[4][16];
    tmem_ld32(tmem_s_row, s[0]);
    tmem_wait_ld();
    // The exponentials of the two query tiles take turns (bar_exp_mine == 0: single tile, no turns):
    // the special-function unit is the bottleneck, and a tile that has it to itself finishes its row
    // while the other tile stores P, waits for its next S and loads it, instead of both tiles
    // crawling through the exponentials in lockstep and then both leaving the unit idle.
    if (bar_exp_mine != 0u && !warp_all(mbar_wait(bar_exp_mine, exp_parity, abort_flag))) return false;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (c < 3) tmem_ld32(tmem_s_row + (c + 1) * 32, s[c + 1]);   // in flight under this chunk's exponentials
      if (c == 1 && bar_exp_other != 0u) mbar_arrive(bar_exp_other);   // hand over after the first chunk: the other tile wakes, loads and
                                                                         // classifies under this tile's remaining three (measured against 0, 2 and 3)
      int kind = kChunkAll;
      if (kMask) {
        const uint32_t bits = visible_keys32(i, kv0 + c * 32, window, len);
        kind = kClassify ? fwd_chunk_kind(bits) : kChunkSome;
        if (kind == kChunkSome) fwd_mask_bits(s[c], bits);
      }
      if (kMask && kClassify && kind == kChunkNone) {
#pragma unroll
        for (int k = 0; k < 16; ++k) pk[c][k] = 0u;
      } else {
        fwd_exp_chunk<true>(s[c], scale2, neg_m2, pk[c], sum, mx);
      }
      if (c < 3) tmem_wait_ld();
      if (c == 2) {
        tc_fence_before_sync();
        mbar_arrive(bar_s_empty);   // the whole row is in registers: S of the next key tile may be computed
      }
    }
    const float m_row = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
    // P V of the previous key tile has long retired by now: the P columns are free and O is current
    if (!warp_all(mbar_wait(bar_o, prev_parity, abort_flag))) return false;
    tc_fence_after_sync();
    // Raising m is a warp-wide decision (the tensor-memory accesses of the rescale are warp-collective).
    if (__any_sync(0xffffffffu, m_row - st.m > kFwdRescaleThreshold)) {
      const float m_new = fmaxf(st.m, m_row);
      const float alpha = fast_exp2(st.m - m_new);
      st.m = m_new;
      st.l = (st.l + fwd_sum4(sum)) * alpha;
#pragma unroll
      for (int k = 0; k < 4; ++k) sum[k] = make_float2(0.f, 0.f);
      fwd_rescale_o(tmem_o_row, alpha);
      const uint32_t alpha2 = pack_bf16(alpha, alpha);
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < 16; ++k) pk[c][k] = mul_bf16x2(pk[c][k], alpha2);   // P of this tile, moved to the new reference
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_st16(tmem_p_row + c * 16, pk[c]);
  }
  st.l += fwd_sum4(sum);
  return true;
}

__device__ __forceinline__ void setmaxnreg_inc_216_fwd() { asm volatile("setmaxnreg.inc.sync.aligned.u32 216;"); }
__device__ __forceinline__ void setmaxnreg_dec_72_fwd() { asm volatile("setmaxnreg.dec.sync.aligned.u32 72;"); }

// One CTA = one work item (long items: the hardware's CTA scheduler balances the SMs, and the
// constant per-CTA addresses keep the MMA-issuing threads' instruction count lowest).
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdOneSmem* sm = reinterpret_cast<FwdOneSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

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
      mbar_init(smem_u32(&sm->bar_kv_empty[s]), n_act);   // one tcgen05.commit per active query tile
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&sm->bar_s_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_s_empty[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_p_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_o_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_exp[x]), kComputeThreads);
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
  setmaxnreg_dec_72_fwd();

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
  } else if (warp == 8 || warp == 10) {
    // ----------------------- MMA issuer of tile A (warp 8) / tile B (warp 10) -----------------------
    // One issuing thread per query tile, on different SM sub-partitions: tcgen05.mma issue is
    // synchronous with the tensor pipe and an issuing warp gets few issue slots next to busy softmax
    // warps, so one thread for both tiles would serialise the two tiles' chains.
    const int x = (warp - 8) >> 1;
    if (lane == 0 && x < n_act) {
      const uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[x]));
      const uint32_t tmem_s = tmem + x * 128, tmem_p = tmem + 256 + x * 64, tmem_o = tmem + 384 + x * 64;
      const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_se = smem_u32(&sm->bar_s_empty[x]),
                     bar_p = smem_u32(&sm->bar_p_full[x]), bar_o = smem_u32(&sm->bar_o_full[x]);
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      for (int t = -1; ok && t < nt; ++t) {
        // S of key tile t+1: as soon as the softmax threads have emptied the S columns (copied S of
        // tile t into registers), so that it is computed underneath their exponentials
        if (t + 1 < nt) {
          const int sn = (t + 1) % kFwdStages;
          if (t >= 0 && !(ok = mbar_wait(bar_se, t & 1, abort_flag))) break;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_kv_full[sn]), ((t + 1) / kFwdStages) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[sn]));
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_s, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
          umma_commit(bar_s);
        }
        // O += P V of key tile t: as soon as P is written
        if (t >= 0) {
          if (!(ok = mbar_wait(bar_p, t & 1, abort_flag))) break;
          tc_fence_after_sync();
          const int s = t % kFwdStages;
          const uint64_t v_desc = desc_mnmajor(smem_u32(sm->v[s]));
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ts(tmem_o, tmem_p + kk * 8, v_desc + kk * kDescKStepMNMajor, idesc_pv, t > 0 || kk > 0);
          umma_commit(bar_o);
          umma_commit(smem_u32(&sm->bar_kv_empty[s]));   // K[s], V[s] are free once every tile's MMAs on them retire
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216_fwd();
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
    const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_se = smem_u32(&sm->bar_s_empty[x]),
                   bar_p = smem_u32(&sm->bar_p_full[x]), bar_o = smem_u32(&sm->bar_o_full[x]);
    const float sink2 = a.sinks[h] * kLog2e;
    FwdRowState st{sink2, 0.f};   // the reference maximum starts at the sink logit
    const uint32_t bar_exp_mine = n_act == 2 ? smem_u32(&sm->bar_exp[x]) : 0u;
    const uint32_t bar_exp_other = n_act == 2 ? smem_u32(&sm->bar_exp[x ^ 1]) : 0u;
    bool ok = true;

    for (int t = 0; t < nt; ++t) {
      const int kv0 = (t_first + t) * kTile;
      const bool need_mask = tile_needs_mask(q0, kv0, a.window, len);
      if (!(ok = warp_all(mbar_wait(bar_s, t & 1, abort_flag)))) break;
      tc_fence_after_sync();
      // tile A goes first: its first wait (parity 1 of a fresh barrier) passes at once
      const uint32_t exp_parity = (x == 0) ? ((t & 1) ^ 1) : (t & 1);
      ok = need_mask
          ? fwd_softmax_tile<true, false>(st, t, tmem_s_row, tmem_p_row, tmem_o_row, bar_se, bar_o, (t - 1) & 1, bar_exp_mine, exp_parity,
                                   bar_exp_other, a.scale_log2, i, kv0, a.window, len, abort_flag)
          : fwd_softmax_tile<false, false>(st, t, tmem_s_row, tmem_p_row, tmem_o_row, bar_se, bar_o, (t - 1) & 1, bar_exp_mine, exp_parity,
                                    bar_exp_other, a.scale_log2, i, kv0, a.window, len, abort_flag);
      if (!ok) break;
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
    }
    if (ok) ok = warp_all(mbar_wait(bar_o, (nt - 1) & 1, abort_flag));
    if (ok) {
      tc_fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld32(tmem_o_row, o0);
      tmem_ld32(tmem_o_row + 32, o1);
      tmem_wait_ld();
      const float z = st.l + fast_exp2(sink2 - st.m);   // the sink joins the denominator only
      const float inv = 1.f / z;
      if (i < a.S) {
        __nv_bfloat16* dst = a.o.row(b, h, i);
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          store_bf16x8(dst + c, pack_bf16(__uint_as_float(o0[c]) * inv, __uint_as_float(o0[c + 1]) * inv),
                       pack_bf16(__uint_as_float(o0[c + 2]) * inv, __uint_as_float(o0[c + 3]) * inv),
                       pack_bf16(__uint_as_float(o0[c + 4]) * inv, __uint_as_float(o0[c + 5]) * inv),
                       pack_bf16(__uint_as_float(o0[c + 6]) * inv, __uint_as_float(o0[c + 7]) * inv));
          store_bf16x8(dst + 32 + c, pack_bf16(__uint_as_float(o1[c]) * inv, __uint_as_float(o1[c + 1]) * inv),
                       pack_bf16(__uint_as_float(o1[c + 2]) * inv, __uint_as_float(o1[c + 3]) * inv),
                       pack_bf16(__uint_as_float(o1[c + 4]) * inv, __uint_as_float(o1[c + 5]) * inv),
                       pack_bf16(__uint_as_float(o1[c + 6]) * inv, __uint_as_float(o1[c + 7]) * inv));
        }
      }
      a.lse[((long long)(b * a.Hq + h)) * a.S_pad + i] = (i < len) ? (st.m + log2f(z)) * kLn2 : 0.f;
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


// One unit of work: one 128-row query tile of n_act (1 or 2) query heads of one KV group.
struct FwdItem {
  int b, h0, g, q0, len, t_first, nt;   // nt = visible key tiles; 0 = the tile is padding only
};
// the divisors of the item decode, prepared once per thread
struct FwdItemDivs {
  FastDiv per_qt, n_hp, group;
  int n_act;
};
__device__ __forceinline__ FwdItemDivs fwd_item_divs(const KernelArgs& a, int n_act) {
  const int n_hp = a.Hq / n_act;
  return FwdItemDivs{make_fastdiv(a.B * n_hp), make_fastdiv(n_hp), make_fastdiv(a.group), n_act};
}
__device__ __forceinline__ FwdItem fwd_item(const KernelArgs& a, int id, const FwdItemDivs& dv) {
  int q_idx, rem, hp;
  FwdItem it;
  fast_divmod(id, dv.per_qt, q_idx, rem);
  const int qt = a.S_pad / kTile - 1 - q_idx;   // long (late) query tiles first; neighbouring ids share K/V in L2
  fast_divmod(rem, dv.n_hp, it.b, hp);
  it.h0 = hp * dv.n_act;
  int g_rem;
  fast_divmod(it.h0, dv.group, it.g, g_rem);
  it.q0 = qt * kTile;
  it.len = seq_len(a, it.b);
  if (it.q0 >= it.len) {
    it.t_first = 0;
    it.nt = 0;
  } else {
    const int hi = min(it.q0 + kTile - 1, it.len - 1);               // last visible key
    const int lo = a.window ? max(0, it.q0 - a.window + 1) : 0;      // first visible key
    it.t_first = lo / kTile;
    it.nt = hi / kTile - it.t_first + 1;
  }
  return it;
}
// Work item of this CTA's round k: rounds alternate direction (0, 1, .., G-1, then G-1, .., 0), so
// that with items sorted by decreasing length every CTA gets nearly the same total.
__device__ __forceinline__ int fwd_item_id(int k) {
  const int c = (k & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  return k * (int)gridDim.x + c;
}
// first round at or after `k` whose work item exists and has key tiles; false if none
__device__ __forceinline__ bool fwd_next_item(const KernelArgs& a, int& k, int n_items, int n_rounds, const FwdItemDivs& dv, FwdItem& it) {
  for (; k < n_rounds; ++k) {
    const int id = fwd_item_id(k);
    if (id >= n_items) continue;
    it = fwd_item(a, id, dv);
    if (it.nt > 0) return true;
  }
  return false;
}

// Persistent: the grid is one CTA per SM and every CTA walks the work items id = blockIdx.x,
// blockIdx.x + gridDim.x, ...  Barriers, tensor memory and the TMA rings are set up once; the loader
// runs ahead across item boundaries (Q is double-buffered), and S of an item's first key tile is
// issued before P V of the previous item's last one, so the per-item set-up and first-load latency
// that dominate short (sliding-window) items are hidden behind the previous item's work.
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_persistent_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem* sm = reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_act = (a.group % 2 == 0) ? 2 : 1;   // query heads (tiles) handled per work item
  const int n_items = (a.S_pad / kTile) * a.B * (a.Hq / n_act);
  const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  const FwdItemDivs dv = fwd_item_divs(a, n_act);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int q = 0; q < 2; ++q) {
      mbar_init(smem_u32(&sm->bar_q_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_q_empty[q]), n_act);    // one tcgen05.commit per active query tile
    }
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(smem_u32(&sm->bar_kv_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_kv_empty[s]), n_act);   // one tcgen05.commit per active query tile
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&sm->bar_s_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_s_empty[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_p_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_o_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_o_free[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_exp[x]), kComputeThreads);
    }
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    sm->q_loads_issued = 0;
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
  setmaxnreg_dec_72_fwd();

  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      int kq = 0;   // work items with key tiles so far (Q buffer = kq & 1)
      int T = 0;    // key tiles so far (stage = T % kFwdStages)
      bool ok = true;
      FwdItem it;
      for (int k = 0; ok && fwd_next_item(a, k, n_items, n_rounds, dv, it); ++k, ++kq) {
        const int qb = kq & 1;
        if (kq >= 2 && !(ok = mbar_wait(smem_u32(&sm->bar_q_empty[qb]), ((kq >> 1) - 1) & 1, abort_flag))) break;
        const uint32_t bar_q = smem_u32(&sm->bar_q_full[qb]);
        mbar_arrive_expect_tx(bar_q, n_act * kTileBytes);
        for (int x = 0; x < n_act; ++x) tma_load_4d(smem_u32(sm->q[qb][x]), &tm_q, bar_q, 0, it.q0, it.h0 + x, it.b);
        *reinterpret_cast<volatile int*>(&sm->q_loads_issued) = kq + 1;
        for (int t = 0; t < it.nt; ++t, ++T) {
          const int s = T % kFwdStages;
          if (T >= kFwdStages && !(ok = mbar_wait(smem_u32(&sm->bar_kv_empty[s]), ((T / kFwdStages) - 1) & 1, abort_flag))) break;
          const int kv0 = (it.t_first + t) * kTile;
          const uint32_t bar = smem_u32(&sm->bar_kv_full[s]);
          mbar_arrive_expect_tx(bar, 2 * kTileBytes);
          tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, kv0, it.g, it.b);
          tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, kv0, it.g, it.b);
          *reinterpret_cast<volatile int*>(&sm->loads_issued) = T + 1;
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 8 || warp == 10) {
    // ----------------------- MMA issuer of tile A (warp 8) / tile B (warp 10) -----------------------
    // One issuing thread per query tile, on different SM sub-partitions: tcgen05.mma issue is
    // synchronous with the tensor pipe and an issuing warp gets few issue slots next to busy softmax
    // warps, so one thread for both tiles would serialise the two tiles' chains.
    const int x = (warp - 8) >> 1;
    if (lane == 0 && x < n_act) {
      const uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      const uint32_t tmem_s = tmem + x * 128, tmem_p = tmem + 256 + x * 64, tmem_o = tmem + 384 + x * 64;
      const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_se = smem_u32(&sm->bar_s_empty[x]),
                     bar_p = smem_u32(&sm->bar_p_full[x]), bar_o = smem_u32(&sm->bar_o_full[x]),
                     bar_of = smem_u32(&sm->bar_o_free[x]);
      // Two cursors walk the same sequence of (work item, key tile): one for the S MMAs, one, a key
      // tile behind, for the P V MMAs.  Order of issue: S(first); then S(next), P V(this), S(next), ...
      // so that S of a key tile -- of the next work item, at an item's end -- is computed underneath the
      // exponentials of the tile before it.  (Plain locals, no helper closures: this thread gets few
      // issue slots and every extra instruction lengthens the chains that wait for it.)
      FwdItem it_s, it_p;
      int k_s = 0, k_p = 0;      // round of the cursor's work item
      int kq_s = 0, kq_p = 0;    // work items with key tiles before the cursor's (Q buffer = kq & 1)
      int t_s = 0, t_p = 0;      // key tile within the work item
      int Ts = 0, Tp = 0;        // key tiles issued so far (K/V stage = T % kFwdStages)
      bool have_s = fwd_next_item(a, k_s, n_items, n_rounds, dv, it_s);
      bool have_p = have_s;
      it_p = it_s;
      k_p = k_s;
      bool ok = true;
      bool first = true;
      while (ok && have_p) {
        if (have_s) {
          // S of key tile t_s: Q landed (first tile), the softmax threads have emptied the S columns
          // (copied the previous S into registers), K landed
          const int qb = kq_s & 1, s = Ts % kFwdStages;
          if (t_s == 0 && !(ok = mbar_wait(smem_u32(&sm->bar_q_full[qb]), (kq_s >> 1) & 1, abort_flag))) break;
          if (Ts >= 1 && !(ok = mbar_wait(bar_se, (Ts - 1) & 1, abort_flag))) break;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_kv_full[s]), (Ts / kFwdStages) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[qb][x]));
          const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[s]));
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_s, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
          umma_commit(bar_s);
          ++Ts;
          if (++t_s == it_s.nt) {
            umma_commit(smem_u32(&sm->bar_q_empty[qb]));   // Q is free once every tile's S MMAs retire
            t_s = 0;
            ++kq_s;
            ++k_s;
            have_s = fwd_next_item(a, k_s, n_items, n_rounds, dv, it_s);
          }
        }
        if (first) {   // the very first S has no P V to go with
          first = false;
          continue;
        }
        {
          // O (+)= P V of key tile t_p: P written; the first P V of an item overwrites O, so the previous
          // item's epilogue must have read it
          if (!(ok = mbar_wait(bar_p, Tp & 1, abort_flag))) break;
          if (t_p == 0 && kq_p >= 1 && !(ok = mbar_wait(bar_of, (kq_p - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const int s = Tp % kFwdStages;
          const uint64_t v_desc = desc_mnmajor(smem_u32(sm->v[s]));
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ts(tmem_o, tmem_p + kk * 8, v_desc + kk * kDescKStepMNMajor, idesc_pv, t_p > 0 || kk > 0);
          umma_commit(bar_o);
          umma_commit(smem_u32(&sm->bar_kv_empty[s]));   // K[s], V[s] are free once every tile's MMAs on them retire
          ++Tp;
          if (++t_p == it_p.nt) {
            t_p = 0;
            ++kq_p;
            ++k_p;
            have_p = fwd_next_item(a, k_p, n_items, n_rounds, dv, it_p);
          }
        }
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216_fwd();
  {
    // -------------------------------------- softmax --------------------------------------
    const int x = warp >> 2;                                      // tile A or B
    const int r = tid & 127;
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;   // this warp's TMEM lane quarter
    const uint32_t tmem_s_row = tmem + x * 128 + lane_addr;
    const uint32_t tmem_p_row = tmem + 256 + x * 64 + lane_addr;
    const uint32_t tmem_o_row = tmem + 384 + x * 64 + lane_addr;
    const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_se = smem_u32(&sm->bar_s_empty[x]),
                   bar_p = smem_u32(&sm->bar_p_full[x]), bar_o = smem_u32(&sm->bar_o_full[x]),
                   bar_of = smem_u32(&sm->bar_o_free[x]);
    const uint32_t bar_exp_mine = n_act == 2 ? smem_u32(&sm->bar_exp[x]) : 0u;
    const uint32_t bar_exp_other = n_act == 2 ? smem_u32(&sm->bar_exp[x ^ 1]) : 0u;
    int T = 0;   // key tiles so far
    bool ok = true;

    for (int k = 0; ok && k < n_rounds; ++k) {
      const int id = fwd_item_id(k);
      if (id >= n_items || x >= n_act) continue;
      const FwdItem it = fwd_item(a, id, dv);
      const float sink = a.sinks[it.h0 + x];
      const int h = it.h0 + x;
      const int i = it.q0 + r;                                    // this thread's query position
      float* lse_out = a.lse + ((long long)(it.b * a.Hq + h)) * a.S_pad + i;
      if (it.nt == 0) {  // tile is padding only: define its output, no tensor work
        if (i < a.S) zero_row(a.o.row(it.b, h, i));
        *lse_out = 0.f;
        continue;
      }
      const float sink2 = sink * kLog2e;
      FwdRowState st{sink2, 0.f};   // the reference maximum starts at the sink logit

      for (int t = 0; t < it.nt; ++t, ++T) {
        const int kv0 = (it.t_first + t) * kTile;
        const bool need_mask = tile_needs_mask(it.q0, kv0, a.window, it.len);
        if (!(ok = warp_all(mbar_wait(bar_s, T & 1, abort_flag)))) break;
        tc_fence_after_sync();
        // tile A goes first: its first wait (parity 1 of a fresh barrier) passes at once
        const uint32_t exp_parity = (x == 0) ? ((T & 1) ^ 1) : (T & 1);
        ok = need_mask
            ? fwd_softmax_tile<true, true>(st, t, tmem_s_row, tmem_p_row, tmem_o_row, bar_se, bar_o, (T - 1) & 1, bar_exp_mine,
                                     exp_parity, bar_exp_other, a.scale_log2, i, kv0, a.window, it.len, abort_flag)
            : fwd_softmax_tile<false, true>(st, t, tmem_s_row, tmem_p_row, tmem_o_row, bar_se, bar_o, (T - 1) & 1, bar_exp_mine,
                                      exp_parity, bar_exp_other, a.scale_log2, i, kv0, a.window, it.len, abort_flag);
        if (!ok) break;
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar_p);
      }
      if (!ok) break;
      if (!(ok = warp_all(mbar_wait(bar_o, (T - 1) & 1, abort_flag)))) break;
      tc_fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld32(tmem_o_row, o0);
      tmem_ld32(tmem_o_row + 32, o1);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bar_of);   // the next item's first P V may overwrite O
      const float z = st.l + fast_exp2(sink2 - st.m);   // the sink joins the denominator only
      const float inv = 1.f / z;
      if (i < a.S) {
        __nv_bfloat16* dst = a.o.row(it.b, h, i);
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          store_bf16x8(dst + c, pack_bf16(__uint_as_float(o0[c]) * inv, __uint_as_float(o0[c + 1]) * inv),
                       pack_bf16(__uint_as_float(o0[c + 2]) * inv, __uint_as_float(o0[c + 3]) * inv),
                       pack_bf16(__uint_as_float(o0[c + 4]) * inv, __uint_as_float(o0[c + 5]) * inv),
                       pack_bf16(__uint_as_float(o0[c + 6]) * inv, __uint_as_float(o0[c + 7]) * inv));
          store_bf16x8(dst + 32 + c, pack_bf16(__uint_as_float(o1[c]) * inv, __uint_as_float(o1[c + 1]) * inv),
                       pack_bf16(__uint_as_float(o1[c + 2]) * inv, __uint_as_float(o1[c + 3]) * inv),
                       pack_bf16(__uint_as_float(o1[c + 4]) * inv, __uint_as_float(o1[c + 5]) * inv),
                       pack_bf16(__uint_as_float(o1[c + 6]) * inv, __uint_as_float(o1[c + 7]) * inv));
        }
      }
      *lse_out = (i < it.len) ? (st.m + log2f(z)) * kLn2 : 0.f;
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
    const int issued = sm->loads_issued, q_issued = sm->q_loads_issued;
    for (int k = max(0, q_issued - 2); k < q_issued; ++k) mbar_wait_drain(smem_u32(&sm->bar_q_full[k & 1]), (k >> 1) & 1);
    for (int t = max(0, issued - kFwdStages); t < issued; ++t)
      mbar_wait_drain(smem_u32(&sm->bar_kv_full[t % kFwdStages]), (t / kFwdStages) & 1);
  }
}

}  // namespace b200attn
