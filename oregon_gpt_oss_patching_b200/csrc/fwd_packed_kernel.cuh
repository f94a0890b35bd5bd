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
//     P = 2^(S*scale*log2e - m)         one thread per row, all 144 scores in registers; m = the head's sink
//                                       logit (any m gives the same result as long as nothing overflows; a row
//                                       whose sum does overflow -- logits ~100 above the sink -- is redone with
//                                       m = its true maximum), so the common path needs no row-maximum pass
//     O = P V    (M=128, N=64, K=144)   P as bf16 A operand from tensor memory
//     O / (sum P + 2^(sink - m)),  LSE = m + log(...)       (attention_kernel.py:53-98 of the reference)
// The exponentials are the bottleneck of this layer (144 per row against 276 + 441 tensor-pipe cycles per
// sub-tile), so the two sub-tiles take turns at them: while one runs them the other's MMAs, loads, stores
// and epilogue proceed.  S of a sub-tile's next item is issued as soon as its S is in registers (S and P have
// columns of their own); the two sub-tiles share ONE O accumulator, which they use strictly in turn.
// O rows leave through shared memory and one TMA store per sub-tile, issued by an otherwise idle warp: a
// thread's row is 128 contiguous bytes 8 KB from its neighbour's, and as plain stores those cost 3000
// cycles of the load/store unit per item -- more than everything else together.
//
// Persistent: one CTA per SM walks the items (consecutive CTAs take consecutive position blocks of the same
// (batch, group), so neighbouring K/V windows meet in L2); Q is double-buffered and K/V go through a 3-stage
// TMA ring that runs ahead across items.  Warp roles: warps 0-3 / 4-7 softmax of sub-tile A / B, warp 8 / 10
// lane 0 issue A's / B's MMAs, warp 9 lane 0 every TMA load, warp 11 lane 0 every TMA store.  Every wait is
// bounded.
#pragma once
#include "attn_common.cuh"
#include "fwd_kernel.cuh"   // exponential helpers, setmaxnreg helpers

namespace b200attn {

constexpr int kPkPos = 16;                       // positions per sub-tile
constexpr int kPkHeads = 8;                      // query heads per sub-tile = the KV group size this kernel serves
constexpr int kPkItemPos = 2 * kPkPos;           // positions per work item (two sub-tiles)
constexpr int kPkMaxWindow = 128;
constexpr int kPkKeys = kPkMaxWindow + kPkPos;   // 144 key columns per sub-tile
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
  uint64_t bar_s_empty[2];                // S of sub-tile X copied into registers                (128 arrivals)
  uint64_t bar_p_full[2];                 // P of sub-tile X written                              (128 arrivals)
  uint64_t bar_pv_done[2];                // P V of sub-tile X retired: O current, P free         (tcgen05.commit)
  uint64_t bar_o_free;                    // O read by an epilogue; phase u = 2 * item + sub-tile (128 arrivals)
  uint64_t bar_ost_full[2];               // O rows of sub-tile X are in shared memory            (128 arrivals)
  uint64_t bar_ost_free[2];               // the TMA store has read them                          (1 arrival)
  uint64_t bar_exp[2];                    // sub-tile X may run its exponentials                  (128 arrivals of the other)
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
      mbar_init(smem_u32(&sm->bar_s_empty[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_p_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_pv_done[x]), 1);
      mbar_init(smem_u32(&sm->bar_ost_full[x]), kComputeThreads);
      mbar_init(smem_u32(&sm->bar_ost_free[x]), 1);
      mbar_init(smem_u32(&sm->bar_exp[x]), kComputeThreads);
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
  } else if (warp == 8 || warp == 10) {
    // -------------------- MMA issuer of sub-tile A (warp 8) / sub-tile B (warp 10) --------------------
    const int x = (warp - 8) >> 1;
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(kTile, kPkKeys, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(kTile, kHeadDim, 0, 1);
      const uint32_t tmem_s = tmem + x * kFwdPkColS, tmem_p = tmem + kFwdPkColP + x * kFwdPkColPStride, tmem_o = tmem + kFwdPkColO;
      const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_se = smem_u32(&sm->bar_s_empty[x]),
                     bar_p = smem_u32(&sm->bar_p_full[x]), bar_pv = smem_u32(&sm->bar_pv_done[x]),
                     bar_of = smem_u32(&sm->bar_o_free);
      bool ok = true;
      PkItem it;
      int k = 0;
      bool have = pk_next_item(a, k, n_items, dv, it);
      // S of item n: Q and K landed, and the softmax threads hold S of item n-1 in registers
      auto issue_s = [&](int n) -> bool {
        const int qb = n & 1, s = n % kPkStages;
        if (n >= 1 && !mbar_wait(bar_se, (n - 1) & 1, abort_flag)) return false;
        if (!mbar_wait(smem_u32(&sm->bar_q_full[qb]), (n >> 1) & 1, abort_flag)) return false;
        if (!mbar_wait(smem_u32(&sm->bar_kv_full[s]), (n / kPkStages) & 1, abort_flag)) return false;
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
      if (have) ok = issue_s(0);
      for (int n = 0; ok && have; ++n) {
        ++k;
        have = pk_next_item(a, k, n_items, dv, it);
        // S of the next item first: it only waits for this item's S to be in registers, so it is computed
        // underneath this item's exponentials
        if (have && !(ok = issue_s(n + 1))) break;
        // O = P V of item n: P written, and O's previous contents (the other sub-tile's, use u-1) read
        if (!(ok = mbar_wait(bar_p, n & 1, abort_flag))) break;
        const int u = 2 * n + x;
        if (u >= 1 && !(ok = mbar_wait(bar_of, (u - 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        const int s = n % kPkStages;
        const uint64_t v_desc = desc_mnmajor(smem_u32(sm->v[s]) + x * kPkSubOffsetBytes);
#pragma unroll
        for (int kk = 0; kk < kPkKeys / 16; ++kk)
          umma_ts(tmem_o, tmem_p + kk * 8, v_desc + kk * kDescKStepMNMajor, idesc_pv, kk > 0);
        umma_commit(bar_pv);
        umma_commit(smem_u32(&sm->bar_kv_empty[s]));   // K[s], V[s] are free once both sub-tiles' MMAs on them retire
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216_fwd();
  {
    // -------------------------------------- softmax --------------------------------------
    const int x = warp >> 2;                                      // sub-tile A or B
    const int r = tid & 127;
    const int hl = r >> 4, sp = r & 15;                           // head within the group, position within the sub-tile
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;   // this warp's TMEM lane quarter
    const uint32_t tmem_s_row = tmem + x * kFwdPkColS + lane_addr;
    const uint32_t tmem_p_row = tmem + kFwdPkColP + x * kFwdPkColPStride + lane_addr;
    const uint32_t tmem_o_row = tmem + kFwdPkColO + lane_addr;
    const uint32_t bar_s = smem_u32(&sm->bar_s_full[x]), bar_se = smem_u32(&sm->bar_s_empty[x]),
                   bar_p = smem_u32(&sm->bar_p_full[x]), bar_pv = smem_u32(&sm->bar_pv_done[x]),
                   bar_of = smem_u32(&sm->bar_o_free), bar_ostf = smem_u32(&sm->bar_ost_full[x]),
                   bar_oste = smem_u32(&sm->bar_ost_free[x]);
    const uint32_t bar_exp_mine = smem_u32(&sm->bar_exp[x]), bar_exp_other = smem_u32(&sm->bar_exp[x ^ 1]);
    const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
    uint8_t* const o_row_smem = sm->o[x] + r * 128;               // this thread's row of the outgoing O tile
    int n = 0;   // active items so far
    int g_cur = -1;
    float sink2 = 0.f;
    bool ok = true;

    for (int k = 0;; ++k) {
      const int id = k * (int)gridDim.x + (int)blockIdx.x;
      if (id >= n_items) break;
      const PkItem it = pk_item(a, id, dv);
      const int h = it.g * kPkHeads + hl;
      const int i = it.q0 + x * kPkPos + sp;                      // this thread's query position
      float* lse_out = a.lse + ((long long)(it.b * a.Hq + h)) * a.S_pad + i;
      if (it.q0 >= it.len) {  // the item is padding only: define its output, no tensor work
        if (i < a.S) zero_row(a.o.row(it.b, h, i));
        *lse_out = 0.f;
        continue;
      }
      if (it.g != g_cur) {   // (consecutive items nearly always belong to the same group)
        g_cur = it.g;
        sink2 = a.sinks[h] * kLog2e;
      }
      const int kb = it.q0 + x * kPkPos - kPkMaxWindow;           // key of column 0
      const PkRowMask rm = pk_row_mask(sp, kb, a.window, it.len);

      if (!(ok = warp_all(mbar_wait(bar_s, n & 1, abort_flag)))) break;
      tc_fence_after_sync();
      uint32_t s[4][32], s4[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s_row + c * 32, s[c]);
      tmem_ld16(tmem_s_row + 128, s4);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bar_se);   // the tensor core may overwrite S with the next item's scores
      // masks: a chunk all 32 rows of the warp see needs no work, one nobody sees no exponentials
      int kind[5];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t bits = range_bits(rm.lo - c * 32, rm.hi - c * 32);
        kind[c] = fwd_chunk_kind(bits);
        if (kind[c] == kChunkSome) fwd_mask_bits(s[c], bits);
      }
      {
        const uint32_t bits = range_bits(rm.lo - 128, rm.hi - 128) & 0xffffu;   // 16 columns
        kind[4] = __all_sync(0xffffffffu, bits == 0u) ? kChunkNone : (__all_sync(0xffffffffu, bits == 0xffffu) ? kChunkAll : kChunkSome);
        if (kind[4] == kChunkSome) {
#pragma unroll
          for (int e = 0; e < 16; ++e) s4[e] = (bits >> e) & 1u ? s4[e] : 0xff800000u;
        }
      }
      // the two sub-tiles take turns at the exponentials; sub-tile A goes first (its first wait, parity 1 of a
      // fresh barrier, passes at once)
      const uint32_t exp_parity = (x == 0) ? ((n & 1) ^ 1) : (n & 1);
      if (!(ok = warp_all(mbar_wait(bar_exp_mine, exp_parity, abort_flag)))) break;
      // P V of this sub-tile's previous item retired before its epilogue ran: the P columns are free
      float m = sink2;
      float l;
      {
        const float2 neg_m2 = make_float2(-m, -m);
        float2 sum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        float unused_mx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
          if (c == 3) mbar_arrive(bar_exp_other);   // hand over early: covers the other side's wake-up latency
          if (kind[c] == kChunkNone) {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = 0u;
          } else {
            fwd_exp_chunk<false>(s[c], scale2, neg_m2, pk, sum, unused_mx);
          }
          tmem_st16(tmem_p_row + c * 16, pk);
        }
        uint32_t pk[8];
        if (kind[4] == kChunkNone) {
#pragma unroll
          for (int e = 0; e < 8; ++e) pk[e] = 0u;
        } else {
          pk_exp16(s4, scale2, neg_m2, pk, sum);
        }
        tmem_st8(tmem_p_row + 64, pk);
        l = fwd_sum4(sum);
      }
      // Scores far above the sink logit (about 100 in the log2 domain) overflow against m = sink: redo such rows
      // with their true maximum.  A warp-wide decision, taken by next to no warp on real data.
      if (__any_sync(0xffffffffu, !(l < 1.0e30f))) {
        float mx = -INFINITY;   // over the chunks somebody sees; masked scores in them are -inf already
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (kind[c] != kChunkNone) mx = fmaxf(mx, pk_max32(s[c]));
        if (kind[4] != kChunkNone) mx = fmaxf(mx, pk_max16(s4));
        m = fmaxf(sink2, mx * a.scale_log2);   // (a padding row sees nothing: mx = -inf, m = the sink)
        const float2 neg_m2 = make_float2(-m, -m);
        float2 sum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        float unused_mx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
          if (kind[c] == kChunkNone) {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = 0u;
          } else {
            fwd_exp_chunk<false>(s[c], scale2, neg_m2, pk, sum, unused_mx);
          }
          tmem_st16(tmem_p_row + c * 16, pk);
        }
        uint32_t pk[8];
        if (kind[4] == kChunkNone) {
#pragma unroll
          for (int e = 0; e < 8; ++e) pk[e] = 0u;
        } else {
          pk_exp16(s4, scale2, neg_m2, pk, sum);
        }
        tmem_st8(tmem_p_row + 64, pk);
        l = fwd_sum4(sum);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
      const float z = l + fast_exp2(sink2 - m);   // the sink joins the denominator only
      const float inv = 1.f / z;

      if (!(ok = warp_all(mbar_wait(bar_pv, n & 1, abort_flag)))) break;
      tc_fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld32(tmem_o_row, o0);
      tmem_ld32(tmem_o_row + 32, o1);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bar_of);   // the other sub-tile's P V may overwrite O
      // the row goes to shared memory in the layout the TMA store expects (16-byte chunk c of row r at chunk
      // position c ^ (r % 8)); the store of this sub-tile's previous item must have read the buffer
      if (n >= 1 && !(ok = warp_all(mbar_wait(bar_oste, (n - 1) & 1, abort_flag)))) break;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4*>(o_row_smem + ((c ^ (r & 7)) << 4)) =
            make_uint4(pack_bf16(__uint_as_float(o0[c * 8]) * inv, __uint_as_float(o0[c * 8 + 1]) * inv),
                       pack_bf16(__uint_as_float(o0[c * 8 + 2]) * inv, __uint_as_float(o0[c * 8 + 3]) * inv),
                       pack_bf16(__uint_as_float(o0[c * 8 + 4]) * inv, __uint_as_float(o0[c * 8 + 5]) * inv),
                       pack_bf16(__uint_as_float(o0[c * 8 + 6]) * inv, __uint_as_float(o0[c * 8 + 7]) * inv));
        *reinterpret_cast<uint4*>(o_row_smem + (((c + 4) ^ (r & 7)) << 4)) =
            make_uint4(pack_bf16(__uint_as_float(o1[c * 8]) * inv, __uint_as_float(o1[c * 8 + 1]) * inv),
                       pack_bf16(__uint_as_float(o1[c * 8 + 2]) * inv, __uint_as_float(o1[c * 8 + 3]) * inv),
                       pack_bf16(__uint_as_float(o1[c * 8 + 4]) * inv, __uint_as_float(o1[c * 8 + 5]) * inv),
                       pack_bf16(__uint_as_float(o1[c * 8 + 6]) * inv, __uint_as_float(o1[c * 8 + 7]) * inv));
      }
      fence_proxy_async_smem();   // written with ordinary stores, read by the TMA engine
      mbar_arrive(bar_ostf);
      *lse_out = (i < it.len) ? (m + log2f(z)) * kLn2 : 0.f;
      ++n;
    }
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
    const int issued = sm->loads_issued;
    for (int n = max(0, issued - 2); n < issued; ++n) mbar_wait_drain(smem_u32(&sm->bar_q_full[n & 1]), (n >> 1) & 1);
    for (int n = max(0, issued - kPkStages); n < issued; ++n)
      mbar_wait_drain(smem_u32(&sm->bar_kv_full[n % kPkStages]), (n / kPkStages) & 1);
  }
}

}  // namespace b200attn
