// Grouped bf16 GEMM for the GPT-OSS mixture-of-experts block on sm_100a (tcgen05 + TMA).
//
// Replaces the per-expert Python loop of Hugging Face's GptOssExperts.forward
// (transformers/models/gpt_oss/modeling_gpt_oss.py:90-114: `current_state @ gate_up_proj[e] + bias`,
// `gated_output @ down_proj[e] + bias`) and the three matrix products autograd derives from each of them.
// Token rows are sorted by expert into one buffer in which every expert's segment starts at a multiple of
// 128 rows (padding rows hold zeros); `offsets` (device, num_groups + 1 entries) gives the segment bounds, so
// nothing about the routing has to be known on the host.
//
//   mode 0 (rows grouped):  D[r, :] = A[r, :] . B_g (+ bias_g)     for the rows r of group g
//        A (rows x K) K-contiguous.  B_g either (K x N) N-contiguous -- the forward products, weights as
//        stored -- or (N x K) K-contiguous -- the input-gradient products, the same weights read transposed.
//   mode 1 (inner dimension grouped):  D_g = A[rows of g, :]^T . B[rows of g, :]
//        the weight-gradient products: A (rows x M) and B (rows x N) are both read "transposed" by the tensor
//        core (M/N-contiguous operands), rows of the group are the inner dimension.
//
// One CTA computes a 256 x 192 tile of D as two M = 128 tcgen05.mma chains that share every staged B tile
// (fp32 accumulators in tensor memory, columns [0,192) and [256,448)); 192 divides both 2880 and 5760, so no
// column tile of the GPT-OSS sizes is ragged.  Operands arrive by TMA with the 128-byte swizzle through a
// 3-stage ring (56 KB per stage: 64 inner elements of 256 + 192 rows).  A 256-row tile never crosses a group
// boundary: a group with an odd number of 128-row blocks ends in a half tile (one chain, half the A bytes).
// Persistent: CTA c takes tiles c, c + gridDim.x, ...; consecutive tiles share the A rows (mode 0) and walk the
// columns of one expert's weights, so an expert's weights are read from HBM once and then hit in L2.
//
// Warp 0 lane 0: every TMA load (two or three operations per inner block: an M/N-contiguous operand whose width
// is a multiple of 64 is described to the engine as (64, rows, width / 64), so one box lands all its 64-element
// panels).  Warp 1 lane 0: every MMA (warp 1 owns the tensor memory).  Warps 4-7 / 8-11: epilogue of
// accumulator rows 0-127 / 128-255 in two phases: tensor memory -> (+ bias) -> packed bf16 in registers, which
// releases the accumulators to the next tile's MMAs; then registers -> shared memory (swizzled 128 x 64 tile) ->
// one TMA store per 64 columns; rows or columns past the end of D are clipped by the store.  The first GEMM of the
// block also writes the gated activation of its (gate, up) column pairs from the same registers (`glu_out`), so that
// H needs no pass of its own.  Every wait is bounded.
#pragma once
#include <cuda.h>

#include "moe_aux_kernels.cuh"
#include "sm100_ptx.cuh"

namespace b200moe {

using namespace b200attn;

constexpr int kBM = 256, kBN = 192, kBK = 64;
constexpr int kHalfM = 128;
constexpr int kGemmStages = 3;
constexpr int kGemmThreads = 384;
constexpr int kHalfABytes = kHalfM * kBK * 2;   // 16 KB: 128 rows x 64 inner elements
constexpr int kABytes = 2 * kHalfABytes;
constexpr int kBBytes = kBN * kBK * 2;          // 24 KB
constexpr int kPanelBytes = 64 * kBK * 2;       // 8 KB: 64 inner rows x 64 M/N elements (M/N-contiguous operands)
constexpr int kOutBytes = 128 * 64 * 2;         // 16 KB staging tile per epilogue warpgroup
constexpr int kMaxGroups = 256;
constexpr uint32_t kAccCols = 256;              // column distance of the two accumulators
constexpr int kGemmTmemCols = 512;

struct GemmSmem {
  alignas(1024) uint8_t a[kGemmStages][kABytes];
  alignas(1024) uint8_t b[kGemmStages][kBBytes];
  alignas(1024) uint8_t out[2][kOutBytes];
  alignas(8) uint64_t bar_full[kGemmStages];
  uint64_t bar_empty[kGemmStages];
  uint64_t bar_acc_full;    // a tile's MMAs retired                     (tcgen05.commit)
  uint64_t bar_acc_empty;   // ... and both accumulators have been read  (256 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  int loads_issued;
  int tile_prefix[kMaxGroups + 1];   // mode 0: 256-row tiles before group g
  int row_off[kMaxGroups + 1];       // the group offsets, read once
};

struct GemmArgs {
  int mode;           // 0: rows grouped, 1: inner dimension grouped
  int a_mn, b_mn;     // operand forms: 0 = inner dimension contiguous, 1 = M/N contiguous
  int a_merged, b_merged;   // an M/N-contiguous operand whose panels of a block arrive in one TMA box (width % 64 == 0)
  int num_groups;
  int M, N, K;        // mode 0: N output columns, K inner (M unused: rows come from offsets); mode 1: M x N per group (K unused)
  const int* offsets; // (num_groups + 1) row offsets of the groups, multiples of 128
  const __nv_bfloat16* bias;   // (num_groups, N) or nullptr
  __nv_bfloat16* glu_out;      // mode 0 only, or nullptr: (rows x N/2), the gated activation of D's (gate, up) column pairs
  int* status;
};

// One tile of work.
struct GemmTile {
  int g;         // group
  int row0;      // mode 0: first row of A and D; mode 1: first row (of M) of D_g
  int halves;    // 1 or 2 accumulators of 128 rows in use
  int n0;        // first output column
  int k_row0;    // mode 1: first row of the group (inner dimension origin)
  int k_blocks;  // inner blocks of 64
};

// Named barrier `id` among 128 threads, returning the OR of their predicates.
__device__ __forceinline__ bool wg_barrier_or(int id, bool pred) {
  uint32_t any;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 q, %2, 0;\n\t"
      "bar.red.or.pred p, %1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(any)
      : "r"(id), "r"((uint32_t)pred)
      : "memory");
  return any != 0;
}

// Walks the tiles of one CTA in order.  All roles construct the same sequence.
struct TileWalker {
  const GemmArgs& a;
  const GemmSmem* sm;
  int n_tiles_n, m_tiles, total, id, g;
  __device__ TileWalker(const GemmArgs& a_, const GemmSmem* sm_) : a(a_), sm(sm_), id((int)blockIdx.x), g(0) {
    n_tiles_n = (a.N + kBN - 1) / kBN;
    m_tiles = (a.M + kBM - 1) / kBM;
    total = a.mode == 0 ? sm->tile_prefix[a.num_groups] * n_tiles_n : a.num_groups * m_tiles * n_tiles_n;
  }
  __device__ bool next(GemmTile& t) {
    if (id >= total) return false;
    if (a.mode == 0) {
      const int st = id / n_tiles_n;
      while (sm->tile_prefix[g + 1] <= st) ++g;   // tile ids only grow: the cursor never moves back
      const int local = st - sm->tile_prefix[g];
      const int rows = sm->row_off[g + 1] - sm->row_off[g] - local * kBM;
      t.g = g;
      t.row0 = sm->row_off[g] + local * kBM;
      t.halves = rows > kHalfM ? 2 : 1;
      t.n0 = (id - st * n_tiles_n) * kBN;
      t.k_row0 = 0;
      t.k_blocks = (a.K + kBK - 1) / kBK;
    } else {
      const int per_group = m_tiles * n_tiles_n;
      t.g = id / per_group;
      const int rem = id - t.g * per_group;
      const int mt = rem / n_tiles_n;
      t.row0 = mt * kBM;
      t.halves = a.M - t.row0 > kHalfM ? 2 : 1;
      t.n0 = (rem - mt * n_tiles_n) * kBN;
      t.k_row0 = sm->row_off[t.g];
      t.k_blocks = (sm->row_off[t.g + 1] - sm->row_off[t.g]) / kBK;
    }
    id += (int)gridDim.x;
    return true;
  }
};

__global__ void __launch_bounds__(kGemmThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_full,
                        const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_d, const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmem* sm = reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile int* abort_flag = &sm->abort_flag;
  const uint32_t bar_acc_full = smem_u32(&sm->bar_acc_full), bar_acc_empty = smem_u32(&sm->bar_acc_empty);

  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(smem_u32(&sm->bar_full[s]), 1);
      mbar_init(smem_u32(&sm->bar_empty[s]), 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 256);
    sm->abort_flag = 0;
    sm->loads_issued = 0;
    fence_mbar_init();
  }
  if (warp == 2) {
    // group offsets and, for mode 0, the number of 256-row tiles before each group
    for (int g = lane; g <= a.num_groups; g += 32) sm->row_off[g] = a.offsets[g];
    __syncwarp();
    if (lane == 0) {
      int acc = 0;
      for (int g = 0; g < a.num_groups; ++g) {
        sm->tile_prefix[g] = acc;
        acc += (sm->row_off[g + 1] - sm->row_off[g] + kBM - 1) / kBM;
      }
      sm->tile_prefix[a.num_groups] = acc;
    }
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&sm->tmem_base), kGemmTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;

  // Registers move from the warpgroup of the single-thread roles to the two epilogue warpgroups, which hold a
  // whole packed accumulator row (96 registers) while they store it: 128 * 72 + 2 * 128 * 216 = 384 * 168.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 0) {
    // ------------------------------------ TMA loader ------------------------------------
    if (lane == 0) {
      prefetch_tmap(&tm_a);
      prefetch_tmap(&tm_a_full);
      prefetch_tmap(&tm_b);
      // As few TMA operations per block as the layouts allow (the engine's issue rate, not its bandwidth, is what a
      // block of seven 8 KB boxes ran into): M/N-contiguous operands whose width is a multiple of 64 are described
      // to the engine as (64, rows, width/64) so that ONE box {64, 64 inner rows, panels} lands all the 64-element
      // panels of a block, each panel a contiguous 8 KB tile as the MMA descriptors expect.
      TileWalker w(a, sm);
      GemmTile t;
      int it = 0;
      bool ok = true;
      while (ok && w.next(t)) {
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          const int s = it % kGemmStages;
          if (it >= kGemmStages && !(ok = mbar_wait(smem_u32(&sm->bar_empty[s]), ((it / kGemmStages) - 1) & 1, abort_flag))) break;
          const uint32_t bar = smem_u32(&sm->bar_full[s]);
          const uint32_t sa = smem_u32(sm->a[s]), sb = smem_u32(sm->b[s]);
          const int k0 = kb * kBK;
          const int a_bytes = (a.a_merged ? 2 : t.halves) * kHalfABytes;   // a merged box always carries both halves
          mbar_arrive_expect_tx(bar, a_bytes + kBBytes);
          if (a.mode == 0) {
            // A: rows x K, K contiguous: one box for both accumulator halves
            if (t.halves == 2) tma_load_4d(sa, &tm_a_full, bar, k0, t.row0, 0, 0);   // (64 x 256-row) box
            else tma_load_4d(sa, &tm_a, bar, k0, t.row0, 0, 0);                       // half tile: (64 x 128-row) box
            if (!a.b_mn) {
              tma_load_4d(sb, &tm_b, bar, k0, t.n0, t.g, 0);                       // B_g: N x K, K contiguous: one (64 x 192-row) box
            } else if (a.b_merged) {
              tma_load_4d(sb, &tm_b, bar, 0, k0, t.n0 >> 6, t.g);                  // B_g: K x N, N contiguous: three panels in one box
            } else {
              for (int p = 0; p < kBN / 64; ++p) tma_load_4d(sb + p * kPanelBytes, &tm_b, bar, t.n0 + p * 64, k0, t.g, 0);
            }
          } else {
            // both operands rows x (M | N), read with the group's rows as the inner dimension
            const int r0 = t.k_row0 + k0;
            if (a.a_merged) {
              tma_load_4d(sa, &tm_a, bar, 0, r0, t.row0 >> 6, 0);                  // four panels (panels past M arrive as zeros)
            } else {
              for (int p = 0; p < 2 * t.halves; ++p) tma_load_4d(sa + p * kPanelBytes, &tm_a, bar, t.row0 + p * 64, r0, 0, 0);
            }
            if (a.b_merged) {
              tma_load_4d(sb, &tm_b, bar, 0, r0, t.n0 >> 6, 0);
            } else {
              for (int p = 0; p < kBN / 64; ++p) tma_load_4d(sb + p * kPanelBytes, &tm_b, bar, t.n0 + p * 64, r0, 0, 0);
            }
          }
          *reinterpret_cast<volatile int*>(&sm->loads_issued) = it + 1;
        }
      }
      if (!ok && a.status != nullptr) atomicOr(a.status, 1);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kHalfM, kBN, a.a_mn, a.b_mn);
      // descriptor forms: inner-contiguous tiles are rows of 128 B in 1024-byte swizzle atoms (16 inner elements
      // = 32 B along the row); M/N-contiguous tiles are 64-element panels 8 KB apart (16 inner rows = 2048 B)
      const uint32_t a_lbo = a.a_mn ? kPanelBytes : 16, b_lbo = a.b_mn ? kPanelBytes : 16;
      const uint32_t a_step = a.a_mn ? (2048 >> 4) : (32 >> 4), b_step = a.b_mn ? (2048 >> 4) : (32 >> 4);
      TileWalker w(a, sm);
      GemmTile t;
      int it = 0, n_done = 0;
      bool ok = true;
      while (ok && w.next(t)) {
        if (n_done >= 1 && !(ok = mbar_wait(bar_acc_empty, (n_done - 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          const int s = it % kGemmStages;
          if (!(ok = mbar_wait(smem_u32(&sm->bar_full[s]), (it / kGemmStages) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t a0 = make_smem_desc_sw128(smem_u32(sm->a[s]), a_lbo, 1024);
          const uint64_t a1 = make_smem_desc_sw128(smem_u32(sm->a[s]) + kHalfABytes, a_lbo, 1024);
          const uint64_t b0 = make_smem_desc_sw128(smem_u32(sm->b[s]), b_lbo, 1024);
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks) {
            const uint32_t acc = (kb > 0 || ks > 0) ? 1u : 0u;
            umma_ss(tmem, a0 + ks * a_step, b0 + ks * b_step, idesc, acc);
            if (t.halves == 2) umma_ss(tmem + kAccCols, a1 + ks * a_step, b0 + ks * b_step, idesc, acc);
          }
          umma_commit(smem_u32(&sm->bar_empty[s]));
        }
        if (!ok) break;
        umma_commit(bar_acc_full);
        ++n_done;
      }
      if (!ok && a.status != nullptr) atomicOr(a.status, 1);
    }
    __syncwarp();
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ------------------------------------- epilogue -------------------------------------
    const int wg = (warp - 4) >> 2;                               // accumulator half
    const int r = (warp & 3) * 32 + lane;                         // row of the half = tensor-memory lane
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tmem_row = tmem + wg * kAccCols + lane_addr;
    uint8_t* const out_row = sm->out[wg] + r * 128;
    const bool leader = (tid & 127) == 0;
    if (leader) prefetch_tmap(&tm_d);
    TileWalker w(a, sm);
    GemmTile t;
    int n_done = 0;
    bool ok = true;
    while (w.next(t)) {
      // one answer per warp (the tensor-memory loads below are warp-collective), and one per warpgroup at the
      // named barriers: nobody leaves the loop alone
      bool failed = !warp_all(mbar_wait(bar_acc_full, n_done & 1, abort_flag));
      ++n_done;
      tc_fence_after_sync();
      if (wg >= t.halves) {
        // this half of the tile does not exist: nothing to read
        if (wg_barrier_or(1 + wg, failed)) { ok = false; break; }
        mbar_arrive(bar_acc_empty);
        continue;
      }
      const int n_chunks = min(kBN / 64, (a.N - t.n0 + 63) / 64);
      // Phase 1, on the critical path of the next tile: the accumulator leaves tensor memory (+ bias, packed to
      // bf16: 32 registers per 64 columns) and the MMAs of the next tile are released.  Phase 2, under those MMAs:
      // the packed rows go through the staging tile to global memory.
      uint32_t pk[kBN / 64][32];
#pragma unroll
      for (int c = 0; c < kBN / 64; ++c) {
        if (c < n_chunks) {
          uint32_t v0[32], v1[32];
          if (t.k_blocks > 0 && !failed) {
            tmem_ld32(tmem_row + c * 64, v0);
            tmem_ld32(tmem_row + c * 64 + 32, v1);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v0[e] = v1[e] = 0u;   // a group without rows: D_g = 0
          }
          if (a.bias != nullptr) {
            const __nv_bfloat16* bias = a.bias + (long long)t.g * a.N + t.n0 + c * 64;
            const int valid = a.N - (t.n0 + c * 64);
            if (valid >= 64) {   // (N is a multiple of 8 and the chunk starts at a multiple of 64: 16-byte aligned)
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(bias) + q);
                const uint4 b1 = __ldg(reinterpret_cast<const uint4*>(bias) + 4 + q);
                const uint32_t w0[4] = {b0.x, b0.y, b0.z, b0.w}, w1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {   // a bf16 is the upper half of the fp32 with the same value
                  v0[q * 8 + 2 * e] = __float_as_uint(__uint_as_float(v0[q * 8 + 2 * e]) + __uint_as_float(w0[e] << 16));
                  v0[q * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(v0[q * 8 + 2 * e + 1]) + __uint_as_float(w0[e] & 0xffff0000u));
                  v1[q * 8 + 2 * e] = __float_as_uint(__uint_as_float(v1[q * 8 + 2 * e]) + __uint_as_float(w1[e] << 16));
                  v1[q * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(v1[q * 8 + 2 * e + 1]) + __uint_as_float(w1[e] & 0xffff0000u));
                }
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                if (e < valid) v0[e] = __float_as_uint(__uint_as_float(v0[e]) + __bfloat162float(bias[e]));
                if (e + 32 < valid) v1[e] = __float_as_uint(__uint_as_float(v1[e]) + __bfloat162float(bias[e + 32]));
              }
            }
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            pk[c][e] = pack_bf16(__uint_as_float(v0[2 * e]), __uint_as_float(v0[2 * e + 1]));
            pk[c][16 + e] = pack_bf16(__uint_as_float(v1[2 * e]), __uint_as_float(v1[2 * e + 1]));
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar_acc_empty);   // the accumulators are in registers: the next tile's MMAs may start
#pragma unroll
      for (int c = 0; c < kBN / 64; ++c) {
        if (c < n_chunks) {
          if (a.glu_out != nullptr) {
            // the gated activation of this row's 32 (gate, up) pairs, from the bf16 values D holds: 64 bytes per row,
            // written straight from registers (under the next tile's MMAs)
            const int pairs_valid = (a.N - (t.n0 + c * 64)) >> 1;
            __nv_bfloat16* dst = a.glu_out + (long long)(t.row0 + wg * kHalfM + r) * (a.N >> 1) + ((t.n0 + c * 64) >> 1);
            if (pairs_valid >= 32) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                reinterpret_cast<uint4*>(dst)[q] =
                    make_uint4(pack2(glu_value(pk[c][q * 8]), glu_value(pk[c][q * 8 + 1])), pack2(glu_value(pk[c][q * 8 + 2]), glu_value(pk[c][q * 8 + 3])),
                               pack2(glu_value(pk[c][q * 8 + 4]), glu_value(pk[c][q * 8 + 5])), pack2(glu_value(pk[c][q * 8 + 6]), glu_value(pk[c][q * 8 + 7])));
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (e < pairs_valid) dst[e] = __float2bfloat16_rn(glu_value(pk[c][e]));
            }
          }
          // the previous store of this warpgroup must have read the staging tile
          if (leader) tma_store_wait_read();
          if (wg_barrier_or(1 + wg, failed)) { failed = true; break; }
#pragma unroll
          for (int q = 0; q < 8; ++q)   // 16-byte chunk q of row r sits at chunk position q ^ (r % 8)
            *reinterpret_cast<uint4*>(out_row + ((q ^ (r & 7)) << 4)) =
                make_uint4(pk[c][q * 4], pk[c][q * 4 + 1], pk[c][q * 4 + 2], pk[c][q * 4 + 3]);
          fence_proxy_async_smem();   // written with ordinary stores, read by the TMA engine
          wg_barrier_or(1 + wg, false);
          if (leader) {
            tma_store_4d(&tm_d, smem_u32(sm->out[wg]), t.n0 + c * 64, t.row0 + wg * kHalfM, a.mode == 0 ? 0 : t.g, 0);
            tma_store_commit();
          }
        }
      }
      if (failed) { ok = false; break; }
    }
    if (leader) tma_store_wait_all();
    if (!ok) {
      sm->abort_flag = 1;
      if (leader && a.status != nullptr) atomicOr(a.status, 1);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, kGemmTmemCols);
  }
  if (sm->abort_flag && tid == 0) {
    // abandoned: give copies still in flight a bounded chance to land before shared memory goes away
    const int issued = sm->loads_issued;
    for (int it = max(0, issued - kGemmStages); it < issued; ++it)
      mbar_wait_drain(smem_u32(&sm->bar_full[it % kGemmStages]), (it / kGemmStages) & 1);
  }
}

}  // namespace b200moe
