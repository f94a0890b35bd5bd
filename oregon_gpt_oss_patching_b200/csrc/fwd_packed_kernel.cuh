// Forward attention kernel for narrow sliding windows (window <= 128) with a group of 8 query heads per
// KV head, for sm_100a: the GPT-OSS sliding-window layer.
//
// The 128 accumulator rows of a tile are the 8 QUERY HEADS of one KV group x 16 consecutive positions
// (row r = head*16 + position), not 128 positions of one head.  Such a tile sees the keys
// [q0-128, q0+16): one S = Q K^T product with N = 144 covers every visible key of every row (128 of the
// 144 columns are visible to each row, against 128 of 256 when a 128-position tile meets two 128-key
// tiles), there is no second key tile and therefore no online-softmax rescaling at all, and all eight
// heads of the group share the one staged K/V tile.  One 4-D TMA box {d 64, positions 16, heads 8, batch 1}
// lands the Q tile with the 128-byte swizzle intact (rows of 128 bytes, 8 rows per swizzle atom), and the
// same box shape takes the O tile back.
//
// A work item is 32 consecutive positions of one (batch, KV group): sub-tile A = the first 16 positions,
// sub-tile B = the next 16; both read one staged block of K and of V rows [q0-128, q0+32) (160 rows), each
// at its own 16-row offset (two swizzle atoms, so the UMMA descriptors just start 2 KB later).  Per
// sub-tile:
//     S = Q K^T  (M=128, N=144, K=64)   tcgen05.mma, fp32 in tensor memory
//     P = 2^(S*scale*log2e - m)         one thread per row; m = the head's sink logit (any m gives the same
//                                       result as long as nothing overflows; a row whose sum does overflow --
//                                       logits ~100 above the sink -- is redone with m = its true maximum),
//                                       so the common path needs no pass for the row maximum
//     O = P V    (M=128, N=64, K=144)   P as bf16 A operand from tensor memory
//     O / (sum P + 2^(sink - m)),  LSE = m + log(...)       (attention_kernel.py:53-98 of the reference)
//
// What shapes the code (counters of earlier versions: ~1 of the 2-3 busy warps per scheduler always stalled on
// "no instruction", the special-function unit 25 % busy, removing the exponentials altogether -4 %):
//   * Instruction fetch.  A fully unrolled 144-column row is ~25 KB of straight-line code executed once per
//     item; with two or three such roles per scheduler the instruction cache holds none of it and every phase
//     runs at a quarter of its issue rate.  So the row is a ROLLED loop over 32-column chunks streamed from
//     tensor memory (load chunk c+1, exponentials of chunk c, store 16 packed columns of P): a few hundred
//     instructions that stay hot (16-column chunks pay the pipeline's fill and drain nine times a row and
//     were half as fast).
//   * MMA issue.  A separate issuing warp next to busy compute warps gets few issue slots, and every
//     hand-over costs a barrier round trip (~400 cycles from "P written" to "P V issued" + ~800 to issue).
//     Here thread 0 of each softmax warpgroup issues its sub-tile's MMAs itself, right after the warpgroup's
//     P is complete: P V of this item, then S of the next item behind it (the pipe runs them in order).
//   * Output.  A thread's O row is 128 contiguous bytes 8 KB from its neighbour's; as plain stores that costs
//     3000 cycles of the load/store unit per item.  Rows go to shared memory and leave with one TMA store per
//     sub-tile, issued by an otherwise idle warp.
// The two sub-tiles run freely side by side (two warps per scheduler in their exponentials together get 13 %
// more out of the special-function unit than one after the other: 2700 against 2 x 1530 cycles for a pair of
// rows in isolation, so turn-taking costs more than it saves here) and share ONE O accumulator, which they
// use strictly in turn.
//
// Persistent: one CTA per SM walks the items (consecutive CTAs take consecutive position blocks of the same
// (batch, group), so neighbouring K/V windows meet in L2); Q is double-buffered and K/V go through a 3-stage
// TMA ring that runs ahead across items.  384 threads: warps 0-3 / 4-7 softmax + MMA issue + epilogue of
// sub-tile A / B, warp 9 lane 0 every TMA load, warp 11 lane 0 every TMA store.  Every wait is bounded.
#pragma once
#include "attn_common.cuh"
#include "fwd_kernel.cuh"   // exponential helpers, setmaxnreg helpers

namespace b200attn {

constexpr int kPkPos = 16;                       // positions per sub-tile
constexpr int kPkHeads = 8;                      // query heads per sub-tile = the KV group size this kernel serves
constexpr int kPkItemPos = 2 * kPkPos;           // positions per work item (two sub-tiles)
constexpr int kPkMaxWindow = 128;
constexpr int kPkKeys = kPkMaxWindow + kPkPos;   // 144 key columns per sub-tile
constexpr int kPkChunks = kPkKeys / 16;          // 9 chunks of 16 columns
constexpr int kPkKvRows = kPkMaxWindow + kPkItemPos;   // 160 staged K (and V) rows per item
constexpr int kPkKvBytes = kPkKvRows * kHeadDim * 2;   // 20 KB
constexpr int kPkSubOffsetBytes = kPkPos * kHeadDim * 2;   // sub-tile B's keys start 16 rows = 2 KB into the block
constexpr int kPkStages = 3;
constexpr int kFwdPkThreads = 384;
constexpr int kFwdPkTmemCols = 512;
// tensor-memory columns: S_A [0,144)  S_B [144,288)  P_A [288,360)  P_B [368,440)  O (shared, used in turn) [448,512)
constexpr uint32_t kFwdPkColS = 144, kFwdPkColP = 288, kFwdPkColPStride = 80, kFwdPkColO = 448;

struct FwdPkSmem {
  alignas(1024) uint8_t q[2][2][kTileBytes];        // [buffer][sub-tile]: the next item's Q lands while this one runs
  alignas(1024) uint8_t k[kPkStages][kPkKvBytes];
  alignas(1024) uint8_t v[kPkStages][kPkKvBytes];
  alignas(1024) uint8_t o[2][kTileBytes];           // [sub-tile]: O rows on their way out (TMA store)
  alignas(8) uint64_t bar_q_full[2];      // Q of a buffer landed
  uint64_t bar_q_empty[2];                // both sub-tiles' S MMAs reading a Q buffer retired    (2 x tcgen05.commit)
  uint64_t bar_kv_full[kPkStages];
  uint64_t bar_kv_empty[kPkStages];       // both sub-tiles' MMAs on a stage retired              (2 x tcgen05.commit)
  uint64_t bar_s_full[2];                 // S of sub-tile X ready                                (tcgen05.commit)
  uint64_t bar_p_full[2];                 // P of sub-tile X written                              (128 arrivals)
  uint64_t bar_pv_done[2];                // P V of sub-tile X retired: O current, P free         (tcgen05.commit)
  uint64_t bar_o_free;                    // O read by an epilogue; phase u = 2 * item + sub-tile (128 arrivals)
  uint64_t bar_ost_full[2];               // O rows of sub-tile X are in shared memory            (128 arrivals)
  uint64_t bar_ost_free[2];               // the TMA store has read them                          (1 arrival)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;                       // items whose loads the loader has issued (for the abort drain)
};

struct PkItem {
  int b, g, q0, len;   // q0: first position of the item; the item is padding only when q0 >= len
};
struct PkDivs {
  FastDiv chunks, hkv;
  int n_chunks;
};
__device__ __forceinline__ PkDivs pk_divs(const KernelArgs& a) {
  const int n_chunks = a.S_pad / kPkItemPos;
  return PkDivs{make_fastdiv(n_chunks), make_fastdiv(a.Hkv), n_chunks};
}
__device__ __forceinline__ PkItem pk_item(const KernelArgs& a, int id, const PkDivs& dv) {
  int bg, c;
  PkItem it;
  fast_divmod(id, dv.chunks, bg, c);
  fast_divmod(bg, dv.hkv, it.b, it.g);
  it.q0 = c * kPkItemPos;
  it.len = seq_len(a, it.b);
  return it;
}
// first item at or after round k of this CTA that has real rows; false if none
__device__ __forceinline__ bool pk_next_item(const KernelArgs& a, int& k, int n_items, const PkDivs& dv, PkItem& it) {
  for (;; ++k) {
    const int id = k * (int)gridDim.x + (int)blockIdx.x;
    if (id >= n_items) return false;
    it = pk_item(a, id, dv);
    if (it.q0 < it.len) return true;
  }
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}

// Visibility of the key columns of a packed sub-tile for one row.  Column c of the sub-tile is key kb + c with
// kb = (first position of the sub-tile) - 128; the row's position is kb + 128 + sp.  Visible columns are
// lo .. hi:  key <= position, key > position - window, key >= 0; nothing when the row is padding.
struct PkRowMask {
  int lo, hi;
};
__device__ __forceinline__ PkRowMask pk_row_mask(int sp, int kb, int window, int len) {
  PkRowMask m;
  m.lo = max(kPkMaxWindow + 1 + sp - window, -kb);
  m.hi = (kb + kPkMaxWindow + sp < len) ? kPkMaxWindow + sp : -1;
  return m;
}

__device__ __forceinline__ float pk_max16(const uint32_t (&s)[16]) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int e = 0; e < 16; e += 2) mx[(e >> 1) & 1] = fmax3(mx[(e >> 1) & 1], __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
  return fmaxf(mx[0], mx[1]);
}
__device__ __forceinline__ float pk_max32(const uint32_t (&s)[32]) {
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int e = 0; e < 32; e += 2) mx[(e >> 1) & 3] = fmax3(mx[(e >> 1) & 3], __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}
__device__ __forceinline__ void pk_exp16(const uint32_t (&sc)[16], float2 scale2, float2 neg_m2, uint32_t (&pk)[8], float2 (&sum)[4]) {
#pragma unroll
  for (int e = 0; e < 16; e += 2) {
    const float2 x = __ffma2_rn(make_float2(__uint_as_float(sc[e]), __uint_as_float(sc[e + 1])), scale2, neg_m2);
    const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
    sum[(e >> 1) & 3] = __fadd2_rn(sum[(e >> 1) & 3], p);
    pk[e >> 1] = pack_bf16(p.x, p.y);
  }
}

// One 16-column chunk of a row: P = 2^(S*scale*log2e - m) for the columns whose bit is set, 0 for the others,
// packed to bf16 and stored to 8 tensor-memory columns; the row sum grows by the chunk's.  The mask work is
// skipped when the whole warp sees all 16 columns, the exponentials when it sees none.
__device__ __forceinline__ void pk_softmax_chunk16(uint32_t (&sc)[16], uint32_t bits, float2 scale2, float2 neg_m2,
                                                   float2 (&sum)[4], uint32_t tmem_p) {
  uint32_t pk[8];
  if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
    for (int e = 0; e < 8; ++e) pk[e] = 0u;
  } else {
    if (!__all_sync(0xffffffffu, bits == 0xffffu)) {
#pragma unroll
      for (int e = 0; e < 16; ++e) sc[e] = (bits >> e) & 1u ? sc[e] : 0xff800000u;   // -inf
    }
    pk_exp16(sc, scale2, neg_m2, pk, sum);
  }
  tmem_st8(tmem_p, pk);
}
// The same for a 32-column chunk (16 packed columns of P).
__device__ __forceinline__ void pk_softmax_chunk32(uint32_t (&sc)[32], uint32_t bits, float2 scale2, float2 neg_m2,
                                                   float2 (&sum)[4], uint32_t tmem_p) {
  uint32_t pk[16];
  const int kind = fwd_chunk_kind(bits);
  if (kind == kChunkNone) {
#pragma unroll
    for (int e = 0; e < 16; ++e) pk[e] = 0u;
  } else {
    if (kind == kChunkSome) fwd_mask_bits(sc, bits);
    float unused_mx[4];
    fwd_exp_chunk<false>(sc, scale2, neg_m2, pk, sum, unused_mx);
  }
  tmem_st16(tmem_p, pk);
}
// Maximum of the visible columns of a 16-column chunk.
__device__ __forceinline__ float pk_masked_max16(const uint32_t (&sc)[16], uint32_t bits) {
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < 16; e += 2)
    mx = fmax3(mx, (bits >> e) & 1u ? __uint_as_float(sc[e]) : -INFINITY, (bits >> (e + 1)) & 1u ? __uint_as_float(sc[e + 1]) : -INFINITY);
  return mx;
}

__global__ void __launch_bounds__(kFwdPkThreads, 1)
attn_fwd_packed_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                       const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdPkSmem* sm = reinterpret_cast<FwdPkSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const PkDivs dv = pk_divs(a);
  const int n_items = dv.n_chunks * a.B * a.Hkv;
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int q = 0; q < 2; ++q) {
      mbar_init(smem_u32(&sm->bar_q_full[q]), 1);
      mbar_init(smem_u32(&sm->bar_q_empty[q]), 2);
    }
    for (int s = 0; s < kPkStages; ++s) {
      mbar_init(smem_u32(&sm->bar_kv_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_kv_empty[s]), 2);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&sm->bar_s_full[x]), 1);
      mbar_init(smem_u32(&sm->bar_p_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_pv_done[x]), 1);
      mbar_init(smem_u32(&sm->bar_ost_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_ost_free[x]), 1);
    }
    mbar_init(smem_u32(&sm->bar_o_free), kComputeThreads);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdPkTmemCols);
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
      bool ok = true;
      PkItem it;
      int n = 0;   // active items so far (Q buffer = n & 1, K/V stage = n % kPkStages)
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        const int qb = n & 1, s = n % kPkStages;
        if (n >= 2 && !(ok = mbar_wait(smem_u32(&sm->bar_q_empty[qb]), ((n >> 1) - 1) & 1, abort_flag))) break;
        const uint32_t bar_q = smem_u32(&sm->bar_q_full[qb]);
        mbar_arrive_expect_tx(bar_q, 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->q[qb][0]), &tm_q, bar_q, 0, it.q0, it.g * kPkHeads, it.b);            // rows past the end arrive as zeros
        tma_load_4d(smem_u32(sm->q[qb][1]), &tm_q, bar_q, 0, it.q0 + kPkPos, it.g * kPkHeads, it.b);
        if (n >= kPkStages && !(ok = mbar_wait(smem_u32(&sm->bar_kv_empty[s]), ((n / kPkStages) - 1) & 1, abort_flag))) break;
        const uint32_t bar = smem_u32(&sm->bar_kv_full[s]);
        mbar_arrive_expect_tx(bar, 2 * kPkKvBytes);
        tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, it.q0 - kPkMaxWindow, it.g, it.b);             // keys before the sequence: zeros
        tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, it.q0 - kPkMaxWindow, it.g, it.b);
        *reinterpret_cast<volatile int*>(&sm->loads_issued) = n + 1;
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else if (warp == 11) {
    // ------------------------------------ TMA stores of O ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_o);
      bool ok = true;
      PkItem it;
      int n = 0;
      for (int k = 0; ok && pk_next_item(a, k, n_items, dv, it); ++k, ++n) {
        for (int x = 0; x < 2; ++x) {
          if (!(ok = mbar_wait(smem_u32(&sm->bar_ost_full[x]), n & 1, abort_flag))) break;
          tma_store_4d(&tm_o, smem_u32(sm->o[x]), 0, it.q0 + x * kPkPos, it.g * kPkHeads, it.b);   // rows past the end are clipped
          tma_store_commit();
          tma_store_wait_read();                       // shared memory has been read: the rows of the next item may land
          mbar_arrive(smem_u32(&sm->bar_ost_free[x]));
        }
      }
      tma_store_wait_all();
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216_fwd();
  {
    // ------------------------- softmax, MMA issue and epilogue of one sub-tile -------------------------
    const int x = warp >> 2;                                      // sub-tile A or B
    const int r = tid & 127;
    const int hl = r >> 4, sp = r & 15;                           // head within the group, position within the sub-tile
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;   // this warp's TMEM lane quarter
    const uint32_t tmem_s = tmem + x * kFwdPkColS, tmem_p = tmem + kFwdPkColP + x * kFwdPkColPStride, tmem_o = tmem + kFwdPkColO;
    const uint32_t tmem_s_row = tmem_s + lane_addr, tmem_p_row = tmem_p + lane_addr, tmem_o_row = tmem_o + lane_addr;
    const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_p = smem_u32(&sm->bar_p_full[x]),
                   bar_pv = smem_u32(&sm->bar_pv_done[x]), bar_of = smem_u32(&sm->bar_o_free),
                   bar_ostf = smem_u32(&sm->bar_ost_full[x]), bar_oste = smem_u32(&sm->bar_ost_free[x]);
    const uint32_t idesc_qk = make_idesc_bf16(kTile, kPkKeys, 0, 0);
    const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
    const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
    uint8_t* const o_row_smem = sm->o[x] + r * 128;               // this thread's row of the outgoing O tile
    int n = 0;   // active items so far
    int g_cur = -1;
    float sink2 = 0.f;
    bool ok = true;

    // S of item n of this sub-tile (issued by thread 0 of the warpgroup): Q and K landed.  S of item n-1 has been
    // read by every thread of the warpgroup (they had written P of item n-1 before this is called).
    auto issue_s = [&](int n_) -> bool {
      const int qb = n_ & 1, s = n_ % kPkStages;
      if (!mbar_wait(smem_u32(&sm->bar_q_full[qb]), (n_ >> 1) & 1, abort_flag)) return false;
      if (!mbar_wait(smem_u32(&sm->bar_kv_full[s]), (n_ / kPkStages) & 1, abort_flag)) return false;
      tc_fence_after_sync();
      const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[qb][x]));
      const uint64_t k_desc = desc_kmajor(smem_u32(sm->k[s]) + x * kPkSubOffsetBytes);
#pragma unroll
      for (int kk = 0; kk < kHeadDim / 16; ++kk)
        umma_ss(tmem_s, q_desc + kk * kDescKStepKMajor, k_desc + kk * kDescKStepKMajor, idesc_qk, kk > 0);
      umma_commit(bar_s);
      umma_commit(smem_u32(&sm->bar_q_empty[qb]));   // Q is free once both sub-tiles' S MMAs retire
      return true;
    };

    int k = 0;
    PkItem it;
    // padding-only items met on the way get their outputs defined here (no tensor work)
    auto scan = [&](int& k_, PkItem& it_) -> bool {
      for (;; ++k_) {
        const int id = k_ * (int)gridDim.x + (int)blockIdx.x;
        if (id >= n_items) return false;
        it_ = pk_item(a, id, dv);
        if (it_.q0 < it_.len) return true;
        const int h = it_.g * kPkHeads + hl, i = it_.q0 + x * kPkPos + sp;
        if (i < a.S) zero_row(a.o.row(it_.b, h, i));
        a.lse[((long long)(it_.b * a.Hq + h)) * a.S_pad + i] = 0.f;
      }
    };
    bool have = scan(k, it);
    if (have && r == 0) {
      if (!issue_s(0)) *abort_flag = 1;
    }
    __syncwarp();

#pragma unroll 1
    while (have) {
      const int h = it.g * kPkHeads + hl;
      const int i = it.q0 + x * kPkPos + sp;                      // this thread's query position
      float* lse_out = a.lse + ((long long)(it.b * a.Hq + h)) * a.S_pad + i;
      const int len = it.len, s_stage = n % kPkStages;
      if (it.g != g_cur) {   // (consecutive items nearly always belong to the same group)
        g_cur = it.g;
        sink2 = a.sinks[h] * kLog2e;
      }
      const int kb = it.q0 + x * kPkPos - kPkMaxWindow;           // key of column 0
      const PkRowMask rm = pk_row_mask(sp, kb, a.window, len);
      // the next item (its first use is thread 0's S issue, but every thread walks the same sequence)
      ++k;
      have = scan(k, it);

      if (!(ok = warp_all(mbar_wait(bar_s, n & 1, abort_flag)))) break;
      tc_fence_after_sync();
      // (P V of this sub-tile's previous item retired before its epilogue ran: the P columns are free)
      float m = sink2;
      float l;
#pragma unroll 1
      for (int pass = 0;; ++pass) {
        const float2 neg_m2 = make_float2(-m, -m);
        float2 sum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        // 32 columns per step (two steps per trip round the loop, the next step's scores in flight under this
        // step's exponentials), the last 16 columns after the loop
        uint32_t sa[32], sb[32], st[16];
        tmem_ld32(tmem_s_row, sa);
#pragma unroll 1
        for (int c = 0; c < 4; c += 2) {
          tmem_wait_ld();
          tmem_ld32(tmem_s_row + (c + 1) * 32, sb);
          pk_softmax_chunk32(sa, range_bits(rm.lo - c * 32, rm.hi - c * 32), scale2, neg_m2, sum, tmem_p_row + c * 16);
          tmem_wait_ld();
          if (c == 0) tmem_ld32(tmem_s_row + 64, sa); else tmem_ld16(tmem_s_row + 128, st);
          pk_softmax_chunk32(sb, range_bits(rm.lo - (c + 1) * 32, rm.hi - (c + 1) * 32), scale2, neg_m2, sum, tmem_p_row + (c + 1) * 16);
        }
        tmem_wait_ld();
        pk_softmax_chunk16(st, range_bits(rm.lo - 128, rm.hi - 128) & 0xffffu, scale2, neg_m2, sum, tmem_p_row + 64);
        l = fwd_sum4(sum);
        // Scores ~100 (log2 domain) above the sink logit overflow against m = sink: such rows (next to none on
        // real data; a warp-wide decision) are redone with their true maximum.  S is still in tensor memory.
        if (pass == 1 || !__any_sync(0xffffffffu, !(l < 1.0e30f))) break;
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < kPkChunks; ++c) {
          tmem_ld16(tmem_s_row + c * 16, st);
          tmem_wait_ld();
          mx = fmaxf(mx, pk_masked_max16(st, range_bits(rm.lo - c * 16, rm.hi - c * 16) & 0xffffu));
        }
        m = fmaxf(sink2, mx * a.scale_log2);   // (a padding row sees nothing: mx = -inf, m = the sink)
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);

      if (r == 0) {
        // ---- thread 0: O = P V of this item, then S of the next item behind it ----
        bool go = mbar_wait(bar_p, n & 1, abort_flag);                  // the whole warpgroup's P is written
        const int u = 2 * n + x;
        if (go && u >= 1) go = mbar_wait(bar_of, (u - 1) & 1, abort_flag);   // O's previous contents (the other sub-tile's) read
        if (go) {
          tc_fence_after_sync();
          const uint64_t v_desc = desc_mnmajor(smem_u32(sm->v[s_stage]) + x * kPkSubOffsetBytes);
#pragma unroll
          for (int kk = 0; kk < kPkKeys / 16; ++kk)
            umma_ts(tmem_o, tmem_p + kk * 8, v_desc + kk * kDescKStepMNMajor, idesc_pv, kk > 0);
          umma_commit(bar_pv);
          umma_commit(smem_u32(&sm->bar_kv_empty[s_stage]));   // K[s], V[s] are free once both sub-tiles' MMAs on them retire
          if (have) go = issue_s(n + 1);
        }
        if (!go) *abort_flag = 1;
      }
      __syncwarp();
      const float z = l + fast_exp2(sink2 - m);   // the sink joins the denominator only
      const float inv = 1.f / z;

      // ---- epilogue: O rows to shared memory in the layout the TMA store expects (16-byte chunk c of row r at
      // chunk position c ^ (r % 8)); the store of this sub-tile's previous item must have read the buffer ----
      const bool st_free = n == 0 || mbar_test_wait(bar_oste, (n - 1) & 1);   // asked early, answered under the wait below
      if (!(ok = warp_all(mbar_wait(bar_pv, n & 1, abort_flag)))) break;
      tc_fence_after_sync();
      if (!warp_all(st_free) && !(ok = warp_all(mbar_wait(bar_oste, (n - 1) & 1, abort_flag)))) break;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t o0[32];
        tmem_ld32(tmem_o_row + half * 32, o0);
        tmem_wait_ld();
        if (half == 1) {
          tc_fence_before_sync();
          mbar_arrive(bar_of);   // all of O is in registers or shared memory: the other sub-tile's P V may overwrite it
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(o_row_smem + (((half * 4 + c) ^ (r & 7)) << 4)) =
              make_uint4(pack_bf16(__uint_as_float(o0[c * 8]) * inv, __uint_as_float(o0[c * 8 + 1]) * inv),
                         pack_bf16(__uint_as_float(o0[c * 8 + 2]) * inv, __uint_as_float(o0[c * 8 + 3]) * inv),
                         pack_bf16(__uint_as_float(o0[c * 8 + 4]) * inv, __uint_as_float(o0[c * 8 + 5]) * inv),
                         pack_bf16(__uint_as_float(o0[c * 8 + 6]) * inv, __uint_as_float(o0[c * 8 + 7]) * inv));
      }
      fence_proxy_async_smem();   // written with ordinary stores, read by the TMA engine
      mbar_arrive(bar_ostf);
      *lse_out = (i < len) ? (m + log2f(z)) * kLn2 : 0.f;
      ++n;
    }
    if (!ok && r == 0) report_abort(a);
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kFwdPkTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    report_abort(a);
    const int issued = sm->loads_issued;
    for (int n = max(0, issued - 2); n < issued; ++n) mbar_wait_drain(smem_u32(&sm->bar_q_full[n & 1]), (n >> 1) & 1);
    for (int n = max(0, issued - kPkStages); n < issued; ++n)
      mbar_wait_drain(smem_u32(&sm->bar_kv_full[n % kPkStages]), (n / kPkStages) & 1);
  }
}

}  // namespace b200attn
