// One backward kernel for narrow sliding-window layers (window <= 128): dK, dV and dQ from one pass.
//
// Same work decomposition as the dK/dV kernel: one CTA owns one 128-key tile of one KV head of one
// sequence, keeps dK and dV for it in tensor memory and streams, for each of the G query heads of the
// group, the (at most two) 128-row query tiles that can see the key tile.  Per item, keys being the
// accumulator rows:
//     S'^T = K Q^T - LSE/scale        dP'^T = V dO^T - delta      (tcgen05, fp32 in TMEM, N = 128)
//     P^T  = 2^(S'^T*scale*log2e)     dS^T = P^T * dP'^T          (1 thread / key)
//     dV  += P^T dO   (A = P^T, bf16 in TMEM)       dK += dS^T Q   (A = dS^T in shared memory, K-contiguous)
// and, what the separate dQ kernel otherwise recomputes S, dP and every exponential for,
//     dQ_item = dS K     (A = the same dS^T tile read M-contiguous: rows are its K dimension; N = 64)
// A query tile is seen by exactly two key tiles when the window is at most 128 (its own and the one
// before), so every dQ element is the sum of at most two items' contributions.  Each item's tile is
// rounded to bf16, staged in shared memory and ADDED to dQ in global memory by the TMA engine
// (cp.reduce.async.bulk.tensor .add); dQ must hold zeros when the kernel starts (the preprocess
// kernel clears it).  With two terms the sum does not depend on which arrives first, so the result is
// still bit-reproducible -- that is why the kernel refuses wider windows, where a dQ element would get
// three or more terms in arbitrary order.
//
// The per-query-row constants enter through one more k-step against the preprocess kernel's side
// tiles, as in the dK/dV kernel.
//
// Sink gradient.  With w_i = 2^(sink_h*log2e - LSE_i*log2e) (the sink's probability in row i) and
// c_i = sum_j P_ij dP_ij, dsink_h = -sum_i w_i c_i (attention_kernel.py:173-175 of the reference).  Here
// keys, not queries, are the rows a thread owns, so c_i is never in one place; but
// sum_j dS_ij = c_i - delta_i (1 - w_i), hence
//     dsink_h = -( sum_ij w_i dS_ij  +  sum_i w_i (1 - w_i) delta_i ).
// The second sum is the preprocess kernel's; the first is accumulated here from the fp32 dS values, each
// thread over its key row with w_i read from shared memory (the preprocess kernel leaves w in the plane
// the other dQ kernels use for -LSE*log2e), then per warp -- eight partials per (head, key tile).  The
// rounding error of delta (O is only known in bf16) cancels between the two sums, so the result is as
// exact as with c_i computed directly.
//
// Warps 0-7: compute (two warpgroups, 64 query columns each).  Warp 8: S^T/dP^T issuer (and tensor-
// memory owner), 9: TMA loads, 10: dV/dK issuer, 11: dQ issuer (an issuing thread gets few issue slots next to
// the compute warps of its SM sub-partition: with two threads the 24 MMAs behind an item leave sooner; with
// three -- dV, dK, dQ each on its own -- the kernel was slower again), 12-15: dQ epilogue
// (tensor memory -> bf16 -> shared memory -> TMA reduction).  Every wait is bounded.
#pragma once
#include "attn_common.cuh"
#include "bwd_dkdv_kernel.cuh"

namespace b200attn {

constexpr int kFwStages = 3;
constexpr int kFwThreads = 512;
constexpr int kFwTmemCols = 512;
constexpr int kFwMaxWindow = 128;
// tensor-memory columns: S^T [0,128)  dP^T [128,256)  P^T bf16 [256,320)  dQ [320,384)  dV [384,448)  dK [448,512)

struct FwSmem {
  alignas(1024) uint8_t k[kTileBytes];
  alignas(1024) uint8_t v[kTileBytes];
  alignas(1024) uint8_t q[kFwStages][kTileBytes];     // q[0] / d_o[0] double as the staging tiles of dV / dK at the end
  alignas(1024) uint8_t d_o[kFwStages][kTileBytes];
  alignas(1024) uint8_t ds[2][kTileBytes];            // dS^T (keys x queries): panel p = query columns 64p..64p+63
  alignas(1024) uint8_t dq_out[kTileBytes];           // an item's dQ rows on their way out
  alignas(128) uint8_t side[kFwStages][kSideTileBytes + kSidePadBytes];
  alignas(128) uint8_t ones_k[kOnesTileBytes];
  alignas(128) uint8_t ones_v[kOnesTileBytes];
  alignas(16) float w[kFwStages][kTile];                // sink probability of an item's query rows
  alignas(8) uint64_t bar_kv;
  uint64_t bar_in_full[kFwStages];
  uint64_t bar_in_empty[kFwStages];
  uint64_t bar_s_full;        // S^T and dP^T ready                         (tcgen05.commit)
  uint64_t bar_s_free;        // S^T and dP^T are in registers              (256 arrivals)
  uint64_t bar_p_full;        // P^T (tensor memory) and dS^T (shared) written (256 arrivals)
  uint64_t bar_p_free;        // the dV/dK and the dQ MMAs have read them    (2 x tcgen05.commit)
  uint64_t bar_dq_full;       // an item's dQ is complete                    (tcgen05.commit)
  uint64_t bar_dq_free;       // ... and has been read out of tensor memory  (128 arrivals)
  uint64_t bar_acc;           // every MMA retired: dK/dV final
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;
};

constexpr uint32_t kFwStageBytes = 2 * kTileBytes + kSideTileBytes + kTile * 4;
constexpr int kFwSinkPartials = 9;   // per (head, batch, 128 positions): slot 0 the preprocess kernel's term, 1..8 one per compute warp

// P^T and dS^T (bf16 pairs) of 32 query columns for one key row, as dkv_compute_chunk, plus this row's share of
// sum_i w_i dS_ij (two lanes) with w of the 32 columns read from shared memory (the same address for the whole warp).
template <bool kSelect>
__device__ __forceinline__ void fw_compute_chunk(const uint32_t (&rs)[32], const uint32_t (&rp)[32], float2 scale2,
                                                 uint32_t bits, const float* w, float2& acc, uint32_t (&pp)[16],
                                                 uint32_t (&pd)[16]) {
#pragma unroll
  for (int e4 = 0; e4 < 32; e4 += 4) {
    const float4 w4 = *reinterpret_cast<const float4*>(w + e4);
#pragma unroll
    for (int e = e4; e < e4 + 4; e += 2) {
      const float2 x = __fmul2_rn(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), scale2);
      float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
      if (kSelect) {  // selects, not branches
        p.x = (bits >> e) & 1u ? p.x : 0.f;
        p.y = (bits >> (e + 1)) & 1u ? p.y : 0.f;
      }
      const float2 ds = __fmul2_rn(p, make_float2(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1])));   // P * (dP - delta)
      acc = __ffma2_rn(ds, e == e4 ? make_float2(w4.x, w4.y) : make_float2(w4.z, w4.w), acc);
      pp[e >> 1] = pack_bf16(p.x, p.y);
      pd[e >> 1] = pack_bf16(ds.x, ds.y);
    }
  }
}

// One (128 x 64) bf16 tile from shared memory ADDED to the tensor in global memory by the TMA engine.
__device__ __forceinline__ void tma_reduce_add_4d(const void* tmap, uint32_t src_smem, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(tmap), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Barrier 1 among the 128 threads of the dQ epilogue warpgroup, returning the OR of their predicates.
__device__ __forceinline__ bool epi_barrier_or(bool pred) {
  uint32_t any;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(any)
      : "r"((uint32_t)pred)
      : "memory");
  return any != 0;
}

__global__ void __launch_bounds__(kFwThreads, 1)
attn_bwd_window_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                             const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                             const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                             const __grid_constant__ CUtensorMap tm_dq, const KernelArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwSmem* sm = reinterpret_cast<FwSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int g = blockIdx.y;
  const int kt = blockIdx.x;
  const int kv0 = kt * kTile;
  const int len = seq_len(a, b);

  if (kv0 >= len) {  // padding only (dQ of these rows was cleared with the rest)
    if (tid < kComputeThreads && kv0 + tid < a.S) {
      zero_row(a.dk.row(b, g, kv0 + tid));
      zero_row(a.dv.row(b, g, kv0 + tid));
    }
    if (tid < 8 * a.group) {   // no sink gradient from here
      const int h = g * a.group + (tid >> 3);
      a.dsinks_partial[(((long long)h * a.B + b) * (a.S_pad / kTile) + kt) * kFwSinkPartials + 1 + (tid & 7)] = 0.f;
    }
    return;
  }

  const int j_max = min(kv0 + kTile - 1, len - 1);
  const int i_max = min(len - 1, j_max + a.window - 1);   // last query row that sees the tile
  const int qt_first = kt;
  const int nq = i_max / kTile - qt_first + 1;            // query tiles per head: one or two
  const int n_items = nq * a.group;
  const uint8_t* side_base = reinterpret_cast<const uint8_t*>(a.delta + 2ll * a.B * a.Hq * a.S_pad);
  const float* w_base = a.delta + 1ll * a.B * a.Hq * a.S_pad;   // plane 1: the sink's probability per query row

  const uint32_t bar_kv = smem_u32(&sm->bar_kv), bar_acc = smem_u32(&sm->bar_acc), bar_s_full = smem_u32(&sm->bar_s_full),
                 bar_s_free = smem_u32(&sm->bar_s_free), bar_p_full = smem_u32(&sm->bar_p_full),
                 bar_p_free = smem_u32(&sm->bar_p_free), bar_dq_full = smem_u32(&sm->bar_dq_full),
                 bar_dq_free = smem_u32(&sm->bar_dq_free);
  volatile int* abort_flag = &sm->abort_flag;

  // The loading thread sets up the barriers of its own copies and starts them at once: K, V and the first items'
  // tiles are on their way while the rest of the CTA is still being set up (tensor-memory allocation, constant
  // tiles).  It also owns the walk over the items: a head's query tiles, then the next head of the group.
  int ld_h = g * a.group, ld_qi = 0, ld_it = 0;
  auto issue_load = [&](int it) -> bool {
    const int s = it % kFwStages;
    if (it >= kFwStages && !mbar_wait(smem_u32(&sm->bar_in_empty[s]), ((it / kFwStages) - 1) & 1, abort_flag)) return false;
    const int item_q0 = (qt_first + ld_qi) * kTile;
    const uint32_t bar = smem_u32(&sm->bar_in_full[s]);
    const long long row_off = ((long long)(b * a.Hq + ld_h)) * a.S_pad + item_q0;
    mbar_arrive_expect_tx(bar, kFwStageBytes);
    tma_load_4d(smem_u32(sm->q[s]), &tm_q, bar, 0, item_q0, ld_h, b);
    tma_load_4d(smem_u32(sm->d_o[s]), &tm_do, bar, 0, item_q0, ld_h, b);
    bulk_load_1d(smem_u32(sm->side[s]), side_base + row_off * kSideRowBytes, kSideTileBytes, bar);
    bulk_load_1d(smem_u32(sm->w[s]), w_base + row_off, kTile * 4, bar);
    *reinterpret_cast<volatile int*>(&sm->loads_issued) = it + 1;
    if (++ld_qi == nq) {
      ld_qi = 0;
      ++ld_h;
    }
    return true;
  };
  if (tid == 9 * 32) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < kFwStages; ++s) {
      mbar_init(smem_u32(&sm->bar_in_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_in_empty[s]), 1);
    }
    sm->loads_issued = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_do);
    mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
    tma_load_4d(smem_u32(sm->k), &tm_k, bar_kv, 0, kv0, g, b);
    tma_load_4d(smem_u32(sm->v), &tm_v, bar_kv, 0, kv0, g, b);
    for (; ld_it < min(kFwStages, n_items); ++ld_it) issue_load(ld_it);   // (the first ring-full waits for nothing)
  }
  if (tid == 0) {
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, 2 * kComputeThreads);
    mbar_init(bar_p_full, 2 * kComputeThreads);
    mbar_init(bar_p_free, 2);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_free, kComputeThreads);
    mbar_init(bar_acc, 1);
    sm->abort_flag = 0;
    fence_mbar_init();
  }
  if (tid < kTile) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(sm->ones_k + ones_offset(tid, 0)) = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
    *reinterpret_cast<uint4*>(sm->ones_v + ones_offset(tid, 0)) = make_uint4(0u, 0u, 0x3f803f80u, 0x00003f80u);
    *reinterpret_cast<uint4*>(sm->ones_k + ones_offset(tid, 1)) = zero;
    *reinterpret_cast<uint4*>(sm->ones_v + ones_offset(tid, 1)) = zero;
    if (tid < kFwStages * (kSidePadBytes / 16))   // the pads behind the side tiles: read as the last row group's second half
      *reinterpret_cast<uint4*>(sm->side[tid / (kSidePadBytes / 16)] + kSideTileBytes + (tid % (kSidePadBytes / 16)) * 16) = zero;
    fence_proxy_async_smem();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kFwTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_st = tmem, tmem_dpt = tmem + 128, tmem_pt = tmem + 256, tmem_dq = tmem + 320, tmem_dv = tmem + 384,
                 tmem_dk = tmem + 448;

  if (warp >= 8 && warp < 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 9) {
      // ------------------------------------ TMA loader ------------------------------------
      if (lane == 0) {   // (K, V and the first items were requested before the CTA-wide barrier)
        bool ok = true;
        for (int it = ld_it; ok && it < n_items; ++it) ok = issue_load(it);
        if (!ok) report_abort(a);
      }
      __syncwarp();
    } else if (warp == 8) {
      // ------------------------ MMA issuer, S^T and dP^T (front) ------------------------
      if (lane == 0) {
        const uint32_t idesc_front = make_idesc_bf16(kTile, kTile, 0, 0);
        const uint64_t k_desc = desc_kmajor(smem_u32(sm->k));
        const uint64_t v_desc = desc_kmajor(smem_u32(sm->v));
        const uint64_t ones_k_desc = desc_ones(smem_u32(sm->ones_k)), ones_v_desc = desc_ones(smem_u32(sm->ones_v));
        bool ok = mbar_wait(bar_kv, 0, abort_flag);
        for (int it = 0; ok && it < n_items; ++it) {
          const int s = it % kFwStages;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_in_full[s]), (it / kFwStages) & 1, abort_flag))) break;
          if (it > 0 && !(ok = mbar_wait(bar_s_free, (it - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t q_desc = desc_kmajor(smem_u32(sm->q[s]));
          const uint64_t do_desc = desc_kmajor(smem_u32(sm->d_o[s]));
          const uint64_t side_desc = desc_side(smem_u32(sm->side[s]));
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_st, k_desc + kk * kDescKStepKMajor, q_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
          umma_ss(tmem_st, ones_k_desc, side_desc, idesc_front, 1);
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            umma_ss(tmem_dpt, v_desc + kk * kDescKStepKMajor, do_desc + kk * kDescKStepKMajor, idesc_front, kk > 0);
          umma_ss(tmem_dpt, ones_v_desc, side_desc, idesc_front, 1);
          umma_commit(bar_s_full);
        }
        if (!ok) report_abort(a);
      }
      __syncwarp();
    } else if (warp == 10) {
      // ------------------------------ MMA issuer, dV and dK ------------------------------
      if (lane == 0) {
        const uint32_t idesc_dv = make_idesc_bf16(kTile, kHeadDim, 0, 1);   // A in TMEM, B read N-contiguous
        const uint32_t idesc_dk = make_idesc_bf16(kTile, kHeadDim, 0, 1);   // A = dS^T K-contiguous, B = Q read N-contiguous
        const uint32_t ds_base = smem_u32(sm->ds[0]);
        bool ok = true;
        for (int it = 0; ok && it < n_items; ++it) {
          if (!(ok = mbar_wait(bar_p_full, it & 1, abort_flag))) break;
          tc_fence_after_sync();
          const int s = it % kFwStages;
          const uint64_t dot_desc = desc_mnmajor(smem_u32(sm->d_o[s]));
          const uint64_t qt_desc = desc_mnmajor(smem_u32(sm->q[s]));
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ts(tmem_dv, tmem_pt + kk * 8, dot_desc + kk * kDescKStepMNMajor, idesc_dv, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)   // k-step kk = queries 16kk..16kk+15: panel kk/4, 32 bytes per step inside it
            umma_ss(tmem_dk, desc_kmajor(ds_base + (kk >> 2) * kTileBytes) + (kk & 3) * kDescKStepKMajor,
                    qt_desc + kk * kDescKStepMNMajor, idesc_dk, (it > 0 || kk > 0) ? 1u : 0u);
          umma_commit(bar_p_free);
          umma_commit(smem_u32(&sm->bar_in_empty[s]));
          if (it == n_items - 1) umma_commit(bar_acc);
        }
        if (!ok) report_abort(a);
      }
      __syncwarp();
    } else {
      // --------------------------------- MMA issuer, dQ ---------------------------------
      if (lane == 0) {
        const uint32_t idesc_dq = make_idesc_bf16(kTile, kHeadDim, 1, 1);   // A = dS^T read M-contiguous, B = K read N-contiguous
        // dS^T with queries as the M dimension: two 64-query panels kTileBytes apart, 8-key groups 1024 B apart
        const uint64_t ds_mn_desc = make_smem_desc_sw128(smem_u32(sm->ds[0]), kTileBytes, 1024);
        const uint64_t kt_desc = desc_mnmajor(smem_u32(sm->k));
        bool ok = mbar_wait(bar_kv, 0, abort_flag);
        for (int it = 0; ok && it < n_items; ++it) {
          if (!(ok = mbar_wait(bar_p_full, it & 1, abort_flag))) break;
          // the previous item's dQ must have left tensor memory
          if (it > 0 && !(ok = mbar_wait(bar_dq_free, (it - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)   // k-step kk = keys 16kk..16kk+15
            umma_ss(tmem_dq, ds_mn_desc + kk * kDescKStepMNMajor, kt_desc + kk * kDescKStepMNMajor, idesc_dq, kk > 0 ? 1u : 0u);
          umma_commit(bar_p_free);
          umma_commit(bar_dq_full);
        }
        if (!ok) report_abort(a);
      }
      __syncwarp();
    }
  } else if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    {
      // ------------------------------------ dQ epilogue ------------------------------------
      const int r = tid & 127;               // query row of the item's tile = tensor-memory lane
      const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
      bool ok = true;
      int h = g * a.group, qi = 0;
      if (r == 0) prefetch_tmap(&tm_dq);
      for (int it = 0; it < n_items; ++it) {
        ok = mbar_wait(bar_dq_full, it & 1, abort_flag);
        tc_fence_after_sync();
        // the previous item's reduction (issued by thread 0 of this warpgroup) must have read the staging tile
        if (r == 0) tma_store_wait_read();
        // one answer for the whole warpgroup (a thread that left alone would strand the others at the next barrier)
        if (epi_barrier_or(!ok || *abort_flag != 0)) {
          ok = false;
          break;
        }
        uint8_t* const out_row = sm->dq_out + r * 128;
        const float sc = a.scale;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t r0[32];
          tmem_ld32(tmem_dq + lane_addr + half * 32, r0);
          tmem_wait_ld();
          if (half == 1) {
            tc_fence_before_sync();
            mbar_arrive(bar_dq_free);   // the next item's dQ MMAs may overwrite the accumulator
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(out_row + (((half * 4 + c) ^ (r & 7)) << 4)) =
                make_uint4(pack_bf16(__uint_as_float(r0[c * 8]) * sc, __uint_as_float(r0[c * 8 + 1]) * sc),
                           pack_bf16(__uint_as_float(r0[c * 8 + 2]) * sc, __uint_as_float(r0[c * 8 + 3]) * sc),
                           pack_bf16(__uint_as_float(r0[c * 8 + 4]) * sc, __uint_as_float(r0[c * 8 + 5]) * sc),
                           pack_bf16(__uint_as_float(r0[c * 8 + 6]) * sc, __uint_as_float(r0[c * 8 + 7]) * sc));
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (r == 0) {
          tma_reduce_add_4d(&tm_dq, smem_u32(sm->dq_out), 0, (qt_first + qi) * kTile, h, b);   // rows past the end are clipped
          tma_store_commit();
        }
        if (++qi == nq) {
          qi = 0;
          ++h;
        }
      }
      if (r == 0) tma_store_wait_all();
      if (!ok && r == 0) report_abort(a);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
    {
      // ------------------------------------- compute --------------------------------------
      const int wg = warp >> 2;             // which 64 query columns of every item
      const int jl = tid & 127;             // this thread's key row
      const int j = kv0 + jl;
      const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
      bool ok = true;
      float2 sink_acc = make_float2(0.f, 0.f);   // sum_i w_i dS_ij over this thread's key and the current head's items
      int h = g * a.group;

      int qi = 0;
      for (int it = 0; it < n_items; ++it, qi = (qi + 1 == nq) ? 0 : qi + 1) {
        const int i0 = (qt_first + qi) * kTile + wg * 64;  // first query column of this thread
        const float* w = sm->w[it % kFwStages] + wg * 64;
        if (!(ok = warp_all(mbar_wait(bar_s_full, it & 1, abort_flag)))) break;
        tc_fence_after_sync();
        // The thread's 64 columns in two chunks of 32 by a ROLLED loop (one copy of the arithmetic in the
        // instruction cache, 64 instead of 128 score registers alive).  Every chunk is classified for the whole
        // warp: visible to nobody (zeros, no exponential -- half the chunks of these layers), to everybody (no
        // masking work), or mixed.
        uint32_t pp[2][16], pd[2][16];
        const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t rs[32], rp[32], tp[16], td[16];
          tmem_ld32(tmem_st + lane_addr + wg * 64 + c * 32, rs);
          tmem_ld32(tmem_dpt + lane_addr + wg * 64 + c * 32, rp);
          tmem_wait_ld();
          if (c == 1) {   // S^T/dP^T are out of tensor memory: the next item's may be computed
            tc_fence_before_sync();
            mbar_arrive(bar_s_free);
          }
          const uint32_t bits = visible_queries32(j, i0 + c * 32, a.window, len);
          if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              tp[k] = 0u;
              td[k] = 0u;
            }
          } else if (__all_sync(0xffffffffu, bits == 0xffffffffu)) {
            fw_compute_chunk<false>(rs, rp, scale2, bits, w + c * 32, sink_acc, tp, td);
          } else {
            fw_compute_chunk<true>(rs, rp, scale2, bits, w + c * 32, sink_acc, tp, td);
          }
#pragma unroll
          for (int k = 0; k < 16; ++k) {   // (the loop is rolled, so the chunk index cannot select the registers)
            if (c == 0) {
              pp[0][k] = tp[k];
              pd[0][k] = td[k];
            } else {
              pp[1][k] = tp[k];
              pd[1][k] = td[k];
            }
          }
        }
        if (qi + 1 == nq) {   // the head's last item: this warp's partial, lanes added in a fixed order
          float t = sink_acc.x + sink_acc.y;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
          if (lane == 0)
            a.dsinks_partial[(((long long)h * a.B + b) * (a.S_pad / kTile) + kt) * kFwSinkPartials + 1 + warp] = -t;
          sink_acc = make_float2(0.f, 0.f);
          ++h;
        }
        // the MMAs of the previous item must have read P^T and dS^T
        if (it > 0 && !(ok = warp_all(mbar_wait(bar_p_free, (it - 1) & 1, abort_flag)))) break;
        tc_fence_after_sync();
        tmem_st16(tmem_pt + lane_addr + wg * 32, pp[0]);
        tmem_st16(tmem_pt + lane_addr + wg * 32 + 16, pp[1]);
        uint8_t* const ds_row = sm->ds[wg] + jl * 128;
        // dS^T row of this key: 64 queries = one 128-byte row of the warpgroup's panel, 16-byte chunk c at c ^ (row % 8)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(ds_row + ((c ^ (jl & 7)) << 4)) =
              make_uint4(pd[c >> 2][(c & 3) * 4], pd[c >> 2][(c & 3) * 4 + 1], pd[c >> 2][(c & 3) * 4 + 2], pd[c >> 2][(c & 3) * 4 + 3]);
        fence_proxy_async_smem();   // read by the tensor core
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar_p_full);
      }

      if (ok) ok = warp_all(mbar_wait(bar_acc, 0, abort_flag));
      if (ok) {
        // warpgroup 0 stores dV, warpgroup 1 stores dK * scale, through the (now idle) first Q / dO stage
        tc_fence_after_sync();
        const uint32_t src = (wg == 0 ? tmem_dv : tmem_dk) + lane_addr;
        const float sc = wg == 0 ? 1.f : a.scale;
        uint32_t r0[32], r1[32];
        tmem_ld32(src, r0);
        tmem_ld32(src + 32, r1);
        tmem_wait_ld();
        uint8_t* const out_row = (wg == 0 ? sm->q[0] : sm->d_o[0]) + jl * 128;
        const int rr = jl & 7;
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
        fence_proxy_async_smem();
      }
      if (!ok) sm->abort_flag = 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && !sm->abort_flag) {   // rows past the end of the tensor are clipped by the store
    tma_store_4d(&tm_dv, smem_u32(sm->q[0]), 0, kv0, g, b);
    tma_store_4d(&tm_dk, smem_u32(sm->d_o[0]), 0, kv0, g, b);
    tma_store_commit();
    tma_store_wait_all();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, kFwTmemCols);
  }
  if (sm->abort_flag && tid == 9 * 32) {
    const int issued = sm->loads_issued;
    mbar_wait_drain(bar_kv, 0);
    for (int it = max(0, issued - kFwStages); it < issued; ++it)
      mbar_wait_drain(smem_u32(&sm->bar_in_full[it % kFwStages]), (it / kFwStages) & 1);
  }
}

}  // namespace b200attn
