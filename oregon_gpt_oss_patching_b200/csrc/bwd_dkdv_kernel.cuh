// dK/dV kernel for sm_100a.
//
// One CTA owns one 128-key tile of one KV head of one sequence and keeps dK and dV for it in
// tensor memory while it streams, for each of the G query heads of the group, the 128-row query
// tiles that can see the key tile.  Per item (one head, one query tile), transposed so that keys
// are the accumulator rows:
//     S'^T = K Q^T - LSE/scale        dP'^T = V dO^T - delta      (tcgen05, fp32 in TMEM, N = 128)
//     P^T  = 2^(S'^T*scale*log2e)     dS^T = P^T * dP'^T          (1 thread / key)
//     dV  += P^T dO           dK  += dS^T Q                 (A operand = bf16 in TMEM, N = 64)
// The per-query-row constants -LSE/scale and -delta are added by the tensor core: one more k-step
// whose B operand is a (128 queries x 16) side tile, written by the preprocess kernel, holding each
// constant as three bf16 terms (24 mantissa bits), and whose A operand is a constant tile of ones in
// the matching columns.  Taken in the compute step instead they are per-COLUMN constants there and
// cost every thread 32 shared-memory loads per item -- next to the exponentials the most expensive
// part of the step.  The epilogue stores dV and dK * scale once.  No atomics: every dK/dV element has one owner
// and is accumulated in fp32 (the reference adds bf16 partial tiles into global memory with
// atomics, attention_kernel.py:201-212).
//
// Pipeline.  Warp 9 streams Q/dO tiles (+ the side tile) through a 4-stage TMA ring.
// Warp 8 issues the S^T/dP^T MMAs and warp 10 the dV/dK MMAs.  The two compute warpgroups split
// the 128 query columns of an item (warps 0-3: columns 0-63, warps 4-7: columns 64-127), pull
// their half of S^T/dP^T into registers and release those columns at once, so the tensor core
// computes S^T/dP^T of the next item while the exponentials of this one are still running;
// P^T/dS^T go to their own columns, which the dV/dK MMAs of the previous item must have left
// first.  Every wait is bounded.
#pragma once
#include "attn_common.cuh"

namespace b200attn {

constexpr int kDkvStages = 4;
constexpr int kDkvThreads = 384;
constexpr int kDkvTmemCols = 512;
// tensor-memory columns: S^T [0,128)  dP^T [128,256)  P^T bf16 [256,320)  dS^T bf16 [320,384)  dV [384,448)  dK [448,512)

struct DkvSmem {
  alignas(1024) uint8_t k[kTileBytes];
  alignas(1024) uint8_t v[kTileBytes];
  alignas(1024) uint8_t q[kDkvStages][kTileBytes];
  alignas(1024) uint8_t d_o[kDkvStages][kTileBytes];
  alignas(128) uint8_t side[kDkvStages][kSideTileBytes + kSidePadBytes];  // per item: (-LSE/scale, -delta) of its query rows, 3 bf16 terms each
  alignas(128) uint8_t ones_k[kOnesTileBytes];            // ones in the columns of the -LSE/scale terms
  alignas(128) uint8_t ones_v[kOnesTileBytes];            // ones in the columns of the -delta terms
  alignas(1024) uint8_t out[2][kTileBytes];               // dV and dK rows on their way out (TMA store)
  alignas(8) uint64_t bar_kv;                 // K and V landed
  uint64_t bar_in_full[kDkvStages];           // Q, dO and the side tile of a stage landed
  uint64_t bar_in_empty[kDkvStages];          // the dV/dK MMAs reading a stage retired
  uint64_t bar_s_full;                        // S^T and dP^T ready                  (tcgen05.commit)
  uint64_t bar_s_free;                        // S^T and dP^T are in registers       (256 arrivals)
  uint64_t bar_p_full;                        // P^T and dS^T written                (256 arrivals)
  uint64_t bar_p_free;                        // the dV/dK MMAs have read P^T, dS^T  (tcgen05.commit)
  uint64_t bar_acc;                           // every MMA retired: dK/dV final
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;
};

constexpr uint32_t kDkvStageBytes = 2 * kTileBytes + kSideTileBytes;


// P^T and dS^T (bf16 pairs) of 32 query columns for one key row, from S^T/dP^T in registers.
// Two elements per instruction (packed fp32 pairs): the special-function unit, not the issue
// slots, should be what the row waits for -- the MMA-issuing warps live on the slots left over.
template <bool kSelect>
__device__ __forceinline__ void dkv_compute_chunk(const uint32_t (&rs)[32], const uint32_t (&rp)[32], float2 scale2,
                                                  uint32_t bits, uint32_t (&pp)[16], uint32_t (&pd)[16]) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    const float2 x = __fmul2_rn(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), scale2);
    float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
    if (kSelect) {  // selects, not branches
      p.x = (bits >> e) & 1u ? p.x : 0.f;
      p.y = (bits >> (e + 1)) & 1u ? p.y : 0.f;
    }
    const float2 ds = __fmul2_rn(p, make_float2(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1])));   // P * (dP - delta)
    pp[e >> 1] = pack_bf16(p.x, p.y);
    pd[e >> 1] = pack_bf16(ds.x, ds.y);
  }
}

// P^T and dS^T of 64 query columns for one key row.  With kClassify, on partly masked tiles (kMask)
// every 32-query chunk is classified for the whole warp: visible to all 32 key rows (no masking
// work), to none (zeros without a single exponential -- half the chunks of a sliding-window layer),
// or mixed; it pays where most tiles are partly masked and costs a little where few are.
template <bool kMask, bool kClassify>
__device__ __forceinline__ void dkv_compute(const uint32_t (&rs)[2][32], const uint32_t (&rp)[2][32], float scale_log2,
                                            int i0, int j, int window, int len, uint32_t (&pp)[2][16],
                                            uint32_t (&pd)[2][16]) {
  const float2 scale2 = make_float2(scale_log2, scale_log2);
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    if (kMask && kClassify) {
      const uint32_t bits = visible_queries32(j, i0 + c * 32, window, len);
      if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          pp[c][k] = 0u;
          pd[c][k] = 0u;
        }
      } else if (__all_sync(0xffffffffu, bits == 0xffffffffu)) {
        dkv_compute_chunk<false>(rs[c], rp[c], scale2, bits, pp[c], pd[c]);
      } else {
        dkv_compute_chunk<true>(rs[c], rp[c], scale2, bits, pp[c], pd[c]);
      }
    } else {
      const uint32_t bits = kMask ? visible_queries32(j, i0 + c * 32, window, len) : 0xffffffffu;
      dkv_compute_chunk<kMask>(rs[c], rp[c], scale2, bits, pp[c], pd[c]);
    }
  }
}

__device__ __forceinline__ void setmaxnreg_inc_216() { asm volatile("setmaxnreg.inc.sync.aligned.u32 216;"); }
__device__ __forceinline__ void setmaxnreg_dec_72() { asm volatile("setmaxnreg.dec.sync.aligned.u32 72;"); }

template <bool kClassify>
__global__ void __launch_bounds__(kDkvThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
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
  const int qt_first = kt;
  const int nq = i_max / kTile - qt_first + 1;  // query tiles per head
  const int n_items = nq * a.group;
  // side tiles of the preprocess kernel: planes 2..5 of the delta scratch, 16 bytes per query row
  const uint8_t* side_base = reinterpret_cast<const uint8_t*>(a.delta + 2ll * a.B * a.Hq * a.S_pad);

  const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_acc = smem_u32(&sm->bar_acc), bar_s_full = smem_u32(&sm->bar_s_full),
                 bar_s_free = smem_u32(&sm->bar_s_free), bar_p_full = smem_u32(&sm->bar_p_full),
                 bar_p_free = smem_u32(&sm->bar_p_free);
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < kDkvStages; ++s) {
      mbar_init(smem_u32(&sm->bar_in_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_in_empty[s]), 2);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, 2 * kComputeThreads);
    mbar_init(bar_p_full, 2 * kComputeThreads);
    mbar_init(bar_p_free, 2);
    mbar_init(bar_acc, 2);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (tid < kTile) {
    // constant A operands of the extra k-step: ones in columns 0-2 resp. 4-6 of row `tid`
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(sm->ones_k + ones_offset(tid, 0)) = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
    *reinterpret_cast<uint4*>(sm->ones_v + ones_offset(tid, 0)) = make_uint4(0u, 0u, 0x3f803f80u, 0x00003f80u);
    *reinterpret_cast<uint4*>(sm->ones_k + ones_offset(tid, 1)) = zero;
    *reinterpret_cast<uint4*>(sm->ones_v + ones_offset(tid, 1)) = zero;
    if (tid < kDkvStages * (kSidePadBytes / 16))   // the pads behind the side tiles: read as the last row group's second half
      *reinterpret_cast<uint4*>(sm->side[tid / (kSidePadBytes / 16)] + kSideTileBytes + (tid % (kSidePadBytes / 16)) * 16) = zero;
    fence_proxy_async_smem();   // written with ordinary stores, read by the tensor core
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
  const uint32_t tmem_st = tmem, tmem_dpt = tmem + 128, tmem_pt = tmem + 256, tmem_dst = tmem + 320, tmem_dv = tmem + 384,
                 tmem_dk = tmem + 448;

  if (warp >= 8) {
  setmaxnreg_dec_72();
  if (warp == 9) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      prefetch_tmap(&tm_do);
      mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
      tma_load_4d(smem_u32(sm->k), &tm_k, bar_kv, 0, kv0, g, b);
      tma_load_4d(smem_u32(sm->v), &tm_v, bar_kv, 0, kv0, g, b);
      // items run over a head's query tiles, then the next head of the group (running counters: the
      // hardware's division sequence would queue behind the exponentials on the special-function unit)
      int h = g * a.group, qi = 0;
      for (int it = 0; it < n_items; ++it) {
        const int s = it % kDkvStages;
        if (it >= kDkvStages && !mbar_wait(smem_u32(&sm->bar_in_empty[s]), ((it / kDkvStages) - 1) & 1, abort_flag)) {
          report_abort(a);
          break;
        }
        const int item_q0 = (qt_first + qi) * kTile;
        const uint32_t bar = smem_u32(&sm->bar_in_full[s]);
        const long long row_off = ((long long)(b * a.Hq + h)) * a.S_pad + item_q0;
        mbar_arrive_expect_tx(bar, kDkvStageBytes);
        tma_load_4d(smem_u32(sm->q[s]), &tm_q, bar, 0, item_q0, h, b);
        tma_load_4d(smem_u32(sm->d_o[s]), &tm_do, bar, 0, item_q0, h, b);
        bulk_load_1d(smem_u32(sm->side[s]), side_base + row_off * kSideRowBytes, kSideTileBytes, bar);
        *reinterpret_cast<volatile int*>(&sm->loads_issued) = it + 1;
        if (++qi == nq) {
          qi = 0;
          ++h;
        }
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------ MMA issuer, S^T and dP^T (front) ------------------------
    // tcgen05.mma issue is synchronous with the tensor pipe, and an issuing warp gets few issue
    // slots next to busy compute warps: front and back MMAs have an issuing warp each, on different
    // SM sub-partitions, so that neither waits behind the other's issue.
    if (lane == 0) {
      const uint32_t idesc_front = make_idesc_bf16(kTile, kTile, 0, 0);    // A, B both K-contiguous, N = 128
      const uint64_t k_desc = desc_kmajor(smem_u32(sm->k));
      const uint64_t v_desc = desc_kmajor(smem_u32(sm->v));
      const uint64_t ones_k_desc = desc_ones(smem_u32(sm->ones_k)), ones_v_desc = desc_ones(smem_u32(sm->ones_v));
      bool ok = mbar_wait(bar_kv, 0, abort_flag);
      for (int it = 0; ok && it < n_items; ++it) {
        // the stage has landed and the previous item's S^T/dP^T are in registers
        const int s = it % kDkvStages;
        if (!(ok = mbar_wait(smem_u32(&sm->bar_in_full[s]), (it / kDkvStages) & 1, abort_flag))) break;
        if (it > 0 && !(ok = mbar_wait(bar_s_free, (it - 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[s]));
        const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o[s]));
        const uint64_t side_desc = desc_side(smem_u32(sm->side[s]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_st, k_desc + kk * kDescKStepKMajor, q_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
        umma_ss(tmem_st, ones_k_desc, side_desc, idesc_front, 1);    // - LSE/scale per query column
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          umma_ss(tmem_dpt, v_desc + kk * kDescKStepKMajor, do_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
        umma_ss(tmem_dpt, ones_v_desc, side_desc, idesc_front, 1);   // - delta per query column
        umma_commit(bar_s_full);
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  } else {
    // ------------- MMA issuers, dV (warp 10) and dK (warp 11), on two SM sub-partitions -------------
    // An issuing thread gets few issue slots next to the compute warps of its sub-partition; the two
    // products are independent, so each has a thread of its own.  Every barrier they release counts two commits.
    if (lane == 0) {
      const uint32_t idesc_back = make_idesc_bf16(kTile, kHeadDim, 0, 1);  // A in TMEM, B read N-contiguous
      const bool is_dv = warp == 10;
      const uint32_t acc = is_dv ? tmem_dv : tmem_dk, src = is_dv ? tmem_pt : tmem_dst;
      bool ok = true;
      for (int it = 0; ok && it < n_items; ++it) {
        if (!(ok = mbar_wait(bar_p_full, it & 1, abort_flag))) break;   // P^T/dS^T of the item have been written
        tc_fence_after_sync();
        const int s = it % kDkvStages;
        const uint64_t b_desc = desc_mnmajor(smem_u32(is_dv ? sm->d_o[s] : sm->q[s]));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          umma_ts(acc, src + kk * 8, b_desc + kk * kDescKStepMNMajor, idesc_back, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar_p_free);                      // P^T/dS^T columns reusable once these retire
        umma_commit(smem_u32(&sm->bar_in_empty[s]));  // and so is the Q/dO stage (its S^T/dP^T MMAs retired before P^T was written)
        if (it == n_items - 1) umma_commit(bar_acc);
      }
      if (!ok) report_abort(a);
    }
    __syncwarp();
  }
  } else {
  setmaxnreg_inc_216();
  {
    // ------------------------------------- compute --------------------------------------
    const int wg = warp >> 2;             // which 64 query columns of every item
    const int j = kv0 + (tid & 127);      // this thread's key position
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    bool ok = true;

    int qi = 0;   // query tile of the item within its head (items run over the head's tiles, then the next head)
    for (int it = 0; it < n_items; ++it, qi = (qi + 1 == nq) ? 0 : qi + 1) {
      const int i0 = (qt_first + qi) * kTile + wg * 64;  // first query column of this thread
      const bool need_mask = (kv0 + kTile - 1 > i0) || (a.window != 0 && kv0 <= i0 + 63 - a.window) || (i0 + 64 > len);
      if (!(ok = warp_all(mbar_wait(bar_s_full, it & 1, abort_flag)))) break;
      tc_fence_after_sync();
      uint32_t rs[2][32], rp[2][32];
      tmem_ld32(tmem_st + lane_addr + wg * 64, rs[0]);
      tmem_ld32(tmem_dpt + lane_addr + wg * 64, rp[0]);
      tmem_ld32(tmem_st + lane_addr + wg * 64 + 32, rs[1]);
      tmem_ld32(tmem_dpt + lane_addr + wg * 64 + 32, rp[1]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bar_s_free);  // S^T/dP^T columns may be overwritten by the next item
      uint32_t pp[2][16], pd[2][16];
      if (need_mask) dkv_compute<true, kClassify>(rs, rp, a.scale_log2, i0, j, a.window, len, pp, pd);
      else dkv_compute<false, kClassify>(rs, rp, a.scale_log2, i0, j, a.window, len, pp, pd);
      // the dV/dK MMAs of the previous item must have left the P^T/dS^T columns
      if (it > 0 && !(ok = warp_all(mbar_wait(bar_p_free, (it - 1) & 1, abort_flag)))) break;
      tc_fence_after_sync();
      tmem_st16(tmem_pt + lane_addr + wg * 32, pp[0]);
      tmem_st16(tmem_pt + lane_addr + wg * 32 + 16, pp[1]);
      tmem_st16(tmem_dst + lane_addr + wg * 32, pd[0]);
      tmem_st16(tmem_dst + lane_addr + wg * 32 + 16, pd[1]);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p_full);
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
      // The rows leave through shared memory and one TMA store per tensor (issued after the CTA-wide barrier
      // below): a thread's row is 128 contiguous bytes far from its neighbour's, and as plain stores the two tiles
      // took 4500 cycles of the load/store unit, a tenth of the CTA's life.  16-byte chunk c of row r goes to
      // chunk position c ^ (r % 8), the layout the tensor map's 128-byte swizzle expects.
      uint8_t* const out_row = sm->out[wg] + (tid & 127) * 128;
      const int rr = tid & 7;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4*>(out_row + ((c ^ rr) << 4)) =
            make_uint4(pack_bf16(__uint_as_float(r0[c * 8]) * sc, __uint_as_float(r0[c * 8 + 1]) * sc),
                       pack_bf16(__uint_as_float(r0[c * 8 + 2]) * sc, __uint_as_float(r0[c * 8 + 3]) * sc),
                       pack_bf16(__uint_as_float(r0[c * 8 + 4]) * sc, __uint_as_float(r0[c * 8 + 5]) * sc),
                       pack_bf16(__uint_as_float(r0[c * 8 + 6]) * sc, __uint_as_float(r0[c * 8 + 7]) * sc));
        *reinterpret_cast<uint4*>(out_row + (((c + 4) ^ rr) << 4)) =
            make_uint4(pack_bf16(__uint_as_float(r1[c * 8]) * sc, __uint_as_float(r1[c * 8 + 1]) * sc),
                       pack_bf16(__uint_as_float(r1[c * 8 + 2]) * sc, __uint_as_float(r1[c * 8 + 3]) * sc),
                       pack_bf16(__uint_as_float(r1[c * 8 + 4]) * sc, __uint_as_float(r1[c * 8 + 5]) * sc),
                       pack_bf16(__uint_as_float(r1[c * 8 + 6]) * sc, __uint_as_float(r1[c * 8 + 7]) * sc));
      }
      fence_proxy_async_smem();   // written with ordinary stores, read by the TMA engine
    }
    if (!ok) sm->abort_flag = 1;   // (already set by whoever gave up; keeps the stores below from running on a partial tile)
  }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && !sm->abort_flag) {   // rows past the end of the tensor are clipped by the store
    tma_store_4d(&tm_dv, smem_u32(sm->out[0]), 0, kv0, g, b);
    tma_store_4d(&tm_dk, smem_u32(sm->out[1]), 0, kv0, g, b);
    tma_store_commit();
    tma_store_wait_all();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kDkvTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued;
    mbar_wait_drain(bar_kv, 0);
    for (int it = max(0, issued - kDkvStages); it < issued; ++it)
      mbar_wait_drain(smem_u32(&sm->bar_in_full[it % kDkvStages]), (it / kDkvStages) & 1);
  }
}

}  // namespace b200attn
