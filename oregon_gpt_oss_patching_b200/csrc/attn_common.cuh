// Shared definitions of the attention kernels: tile constants, kernel argument block,
// visibility rule, and the UMMA descriptors of the three operand forms they use.
#pragma once
#include <cuda.h>

#include "sm100_ptx.cuh"

namespace b200attn {

constexpr int kTile = 128;                     // query rows / keys per tile
constexpr int kHeadDim = 64;                   // head_dim (one 128-byte swizzle row of bf16)
constexpr int kTileBytes = kTile * kHeadDim * 2;  // 16 KB: one (128 x 64) bf16 tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

constexpr int kComputeThreads = 128;           // warps 0-3: one thread per tile row / TMEM lane
constexpr int kThreads = kComputeThreads + 32; // warp 4: TMA producer + MMA issuer (lane 0)

constexpr int kStatusWaitTimeout = 1;          // OR-ed into *status when a bounded wait gave up

struct StridedPtr {  // bf16 (B,H,S,d) view, element strides, d stride 1
  __nv_bfloat16* ptr;
  long long sb, sh, ss;
  __device__ __forceinline__ __nv_bfloat16* row(int b, int h, int s) const {
    return ptr + b * sb + h * sh + (long long)s * ss;
  }
};

struct KernelArgs {
  int B, Hq, Hkv, S, S_pad, group;  // group = Hq / Hkv
  int window;                       // 0 = full causal
  float scale;                      // logits multiplier
  float scale_log2;                 // scale * log2(e)
  const int* seqlens;               // (B) or nullptr
  const float* sinks;               // (Hq)
  int* status;                      // may be nullptr
  float* lse;                       // (B,Hq,S_pad), natural log
  float* delta;                     // (B,Hq,S_pad)
  float* dsinks;                    // (Hq)
  float* dsinks_partial;            // (Hq, B * S_pad/128 * partials_per_tile)
  int partials_per_tile;            // sink-gradient partials written per (head, 128 positions) by the kernel that makes them
  int fused_bwd;                    // 1: narrow window, one kernel makes dK, dV and dQ; the preprocess kernel clears dQ
                                    //    and writes the sink-gradient partials
  StridedPtr o, d_o, dq, dk, dv;    // tensors touched with plain loads/stores
  StridedPtr q, k, v;
};

__device__ __forceinline__ int seq_len(const KernelArgs& a, int b) {
  if (a.seqlens == nullptr) return a.S;
  int L = a.seqlens[b];
  return L < 0 ? 0 : (L > a.S ? a.S : L);
}

// key j visible to query i (both already known to be < len where that matters)
__device__ __forceinline__ bool visible(int i, int j, int window, int len) {
  return (j <= i) && (window == 0 || j > i - window) && (i < len);
}

// Bit e (0..31) set iff lo <= e <= hi.  Branch-free; any lo/hi is allowed (empty when lo > hi).
__device__ __forceinline__ uint32_t range_bits(int lo, int hi) {
  const int hc = min(max(hi, -1), 31), lc = min(max(lo, 0), 32);
  const uint32_t m_hi = hc < 0 ? 0u : (0xffffffffu >> (31 - hc));
  const uint32_t m_lo = lc > 31 ? 0u : (0xffffffffu << lc);
  return m_hi & m_lo;
}
// Visibility of the 32 keys j0 .. j0+31 for query i, as a bit mask (bit e <-> key j0+e):
// j <= i, j > i - window (when window > 0), i < len.
__device__ __forceinline__ uint32_t visible_keys32(int i, int j0, int window, int len) {
  const int hi = i < len ? i - j0 : -1;
  const int lo = window ? i - window + 1 - j0 : 0;
  return range_bits(lo, hi);
}
// Visibility of the 32 queries i0 .. i0+31 for key j (bit e <-> query i0+e):
// i >= j, i < j + window (when window > 0), i < len.
__device__ __forceinline__ uint32_t visible_queries32(int j, int i0, int window, int len) {
  const int last = window ? min(j + window - 1, len - 1) : len - 1;
  return range_bits(j - i0, last - i0);
}

// Does a (query tile at q0, key tile at kv0) pair contain any masked (i, j)?
__device__ __forceinline__ bool tile_needs_mask(int q0, int kv0, int window, int len) {
  return (kv0 + kTile - 1 > q0) || (window != 0 && kv0 <= q0 + kTile - 1 - window) || (q0 + kTile > len);
}

// ---- UMMA operand descriptors --------------------------------------------------------
// All shared-memory operand tiles are (128 rows x 64 bf16) written by TMA with the 128-byte
// swizzle.  Read with rows as M/N and columns as K ("K-major"), one MMA K-step of 16 is 32
// bytes along the row.  Read with rows as K and columns as M/N ("MN-major", 64 = exactly one
// swizzle atom wide), one K-step of 16 is 16 rows = 2048 bytes.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t smem_addr) {
  return make_smem_desc_sw128(smem_addr, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t smem_addr) {
  return make_smem_desc_sw128(smem_addr, kTileBytes, 1024);
}
// The (rows x 16) bf16 operands of the extra k-step, K-contiguous, unswizzled, made of 8-row x 16-byte core
// matrices (128 contiguous bytes each).
//   "ones" tiles (A operand, constant): core matrix (row group rg, 8-column half kc) at rg*256 + kc*128,
//   element (r, c) at + (r%8)*16 + (c%8)*2; the second half (columns 8-15) is all zeros.
//   side tiles (B operand, from the preprocess kernel): only columns 0-7 exist, 16 bytes per row: row group rg
//   at rg*128.  The descriptor's K-neighbour offset equals the row-group offset, so the "second half" of a row
//   group reads the next row group's real (finite) values -- times the zeros of the A operand's second half.
//   The last row group reads 128 bytes past the tile: every shared-memory copy is followed by a 128-byte pad
//   that the kernel zeroes once.
constexpr int kOnesTileBytes = kTile * 16 * 2;   // 4 KB
constexpr int kSideTileBytes = kTile * 8 * 2;    // 2 KB: 16 bytes per query row
constexpr int kSidePadBytes = 128;
constexpr int kSideRowBytes = 16;
__device__ __forceinline__ uint64_t desc_ones(uint32_t smem_addr) { return make_smem_desc_noswizzle(smem_addr, 128, 256); }
__device__ __forceinline__ uint64_t desc_side(uint32_t smem_addr) { return make_smem_desc_noswizzle(smem_addr, 128, 128); }
__device__ __forceinline__ uint32_t ones_offset(int row, int half) { return (row >> 3) * 256 + half * 128 + (row & 7) * 16; }
__device__ __forceinline__ uint32_t side_offset(int row) { return (row >> 3) * 128 + (row & 7) * 16; }
constexpr uint32_t kDescKStepKMajor = 32 >> 4;     // +32 B per K-step, in 16-byte units
constexpr uint32_t kDescKStepMNMajor = 2048 >> 4;  // +2048 B per K-step

// Record a timed-out wait for the host.
__device__ __forceinline__ void report_abort(const KernelArgs& a) {
  if (a.status != nullptr) atomicOr(a.status, kStatusWaitTimeout);
}

// 16-byte vector store of 8 bf16 values given as 4 packed words
__device__ __forceinline__ void store_bf16x8(__nv_bfloat16* dst, uint32_t w0, uint32_t w1, uint32_t w2,
                                             uint32_t w3) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(w0, w1, w2, w3);
}

__device__ __forceinline__ void zero_row(__nv_bfloat16* dst) {
#pragma unroll
  for (int c = 0; c < kHeadDim; c += 8) store_bf16x8(dst + c, 0u, 0u, 0u, 0u);
}

// Division by a number fixed for the kernel's life without the hardware's division sequence, whose
// reciprocal and conversion steps run on the special-function unit and queue up behind the
// exponentials: quotient estimate by a multiply-high with floor((2^32-1)/d), at most one too small.
struct FastDiv {
  uint32_t d, m;
};
__device__ __forceinline__ FastDiv make_fastdiv(uint32_t d) { return FastDiv{d, 0xffffffffu / d}; }
__device__ __forceinline__ void fast_divmod(uint32_t n, const FastDiv& f, int& q, int& r) {
  uint32_t qq = __umulhi(n, f.m);
  uint32_t rr = n - qq * f.d;
  if (rr >= f.d) {
    ++qq;
    rr -= f.d;
  }
  q = (int)qq;
  r = (int)rr;
}

}  // namespace b200attn
