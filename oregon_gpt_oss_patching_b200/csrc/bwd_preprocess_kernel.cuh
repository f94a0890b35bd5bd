// Memory-bound backward helpers.
//
// attn_bwd_preprocess_kernel:  delta[b,h,i] = sum_c dO[b,h,i,c] * O[b,h,i,c]  in fp32 (the
// reference's `_attn_bwd_precompute_D`, attention_kernel.py:102-120); the second half of the
// scratch receives -LSE*log2(e), the exponent offset the dQ kernels add per query row, and planes
// 2..5 the dK/dV kernel's side tiles: per 128 query rows the first eight columns of a (128 x 16) bf16
// MMA operand in the unswizzled core-matrix layout (see side_offset), 16 bytes per row: row i holds
// -LSE_i/scale in columns 0-2 and -delta_i in columns 4-6, each as three bf16 terms (hi, mid, lo: 24
// mantissa bits).
//
// With a.fused_bwd (narrow windows, where one kernel makes dK, dV and dQ and adds its dQ tiles into
// global memory) the kernel also clears its 128 rows of dQ, leaves w_i = 2^(sink_h*log2e - LSE_i*log2e)
// (the sink's probability in row i; 0 for padding rows) in the second plane instead of -LSE*log2(e), and
// writes its part of the sink gradient, -sum_i w_i (1 - w_i) delta_i (the backward kernel adds the rest).
//
// attn_bwd_dsinks_kernel:  dsinks[h] = sum of head h's partials written by the dQ kernel (or, see
// above, by the preprocess kernel), in a fixed order with a warp-shuffle tree, so the result is bit-reproducible (the
// reference adds its per-tile terms with relaxed atomics, attention_kernel.py:176).
#pragma once
#include "attn_common.cuh"

namespace b200attn {

__device__ __forceinline__ float dot8_bf16(uint4 x, uint4 y) {
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&x);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&y);
  float s = 0.f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 fa = __bfloat1622float2(a[t]);
    const float2 fb = __bfloat1622float2(b[t]);
    s = fmaf(fa.x, fb.x, s);
    s = fmaf(fa.y, fb.y, s);
  }
  return s;
}

// v as three bf16 terms: w0 = (hi, mid), w1 = (lo, 0)
__device__ __forceinline__ void split_bf16x3(float v, uint32_t& w0, uint32_t& w1) {
  const __nv_bfloat16 hi = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(hi);
  const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
  const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
  w0 = uint32_t(__bfloat16_as_ushort(hi)) | (uint32_t(__bfloat16_as_ushort(mid)) << 16);
  w1 = uint32_t(__bfloat16_as_ushort(lo));
}

// grid (S_pad/128, Hq, B), 128 threads.  Eight lanes share a row (16 bytes of O and of dO
// each), so a warp covers 4 rows per step and 32 rows in 8 steps.
__global__ void __launch_bounds__(128) attn_bwd_preprocess_kernel(const KernelArgs a) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int len = seq_len(a, b);
  const int sub = lane >> 3;       // row within the step
  const int part = lane & 7;       // 16-byte slice of the row
  const long long row_base = ((long long)(b * a.Hq + h)) * a.S_pad + (long long)tile * kTile;
  const long long nlse_off = (long long)a.B * a.Hq * a.S_pad;  // plane 1 of the scratch: -LSE*log2(e)
  uint8_t* side_base = reinterpret_cast<uint8_t*>(a.delta + 2 * nlse_off);   // planes 2..5: side tiles, 16 bytes per row
  const float inv_scale = 1.f / a.scale;

  // the CTA's side tile is put together in shared memory and leaves with coalesced 16-byte stores
  __shared__ uint4 side_tile[kSideTileBytes / 16];

  if (a.fused_bwd) {   // dQ is accumulated into: clear this tile's rows (16 bytes per thread and step, coalesced)
    for (int idx = tid; idx < kTile * 8; idx += 128) {
      const int i = tile * kTile + (idx >> 3);
      if (i < a.S) *reinterpret_cast<uint4*>(a.dq.row(b, h, i) + (idx & 7) * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  const float sink2 = a.fused_bwd ? a.sinks[h] * kLog2e : 0.f;
  float sink_term = 0.f;   // this thread's rows' share of -sum 2^(sink - LSE) * delta

  uint4 xo[8], xd[8];
#pragma unroll
  for (int step = 0; step < 8; ++step) {
    const int i = tile * kTile + warp * 32 + step * 4 + sub;
    if (i < len) {
      xo[step] = *reinterpret_cast<const uint4*>(a.o.row(b, h, i) + part * 8);
      xd[step] = *reinterpret_cast<const uint4*>(a.d_o.row(b, h, i) + part * 8);
    } else {
      xo[step] = make_uint4(0, 0, 0, 0);
      xd[step] = make_uint4(0, 0, 0, 0);
    }
  }
#pragma unroll
  for (int step = 0; step < 8; ++step) {
    float s = dot8_bf16(xo[step], xd[step]);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    const int r = warp * 32 + step * 4 + sub;
    if (part == 0) {
      const float lse = a.lse[row_base + r];
      a.delta[row_base + r] = s;  // zero for padding rows
      const float w = (a.fused_bwd && tile * kTile + r < len) ? fast_exp2(sink2 - lse * kLog2e) : 0.f;
      a.delta[nlse_off + row_base + r] = a.fused_bwd ? w : -lse * kLog2e;
      uint32_t u0, u1, d0, d1;
      split_bf16x3(-lse * inv_scale, u0, u1);
      split_bf16x3(-s, d0, d1);
      side_tile[side_offset(r) >> 4] = make_uint4(u0, u1, d0, d1);   // r is the row within the tile
      sink_term -= w * (1.f - w) * s;
    }
  }
  __shared__ float warp_term[4];
  if (a.fused_bwd) {   // fixed-order tree: lanes, then the four warps
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sink_term += __shfl_xor_sync(0xffffffffu, sink_term, off);
    if (lane == 0) warp_term[warp] = sink_term;
  }
  __syncthreads();
  if (a.fused_bwd && tid == 0)
    a.dsinks_partial[(((long long)h * a.B + b) * (a.S_pad / kTile) + tile) * a.partials_per_tile] =
        (warp_term[0] + warp_term[1]) + (warp_term[2] + warp_term[3]);
  uint4* dst = reinterpret_cast<uint4*>(side_base + row_base * kSideRowBytes);   // this CTA's 128 rows
  dst[tid] = side_tile[tid];
}

// grid (Hq), 256 threads
__global__ void __launch_bounds__(256) attn_bwd_dsinks_kernel(const KernelArgs a) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x;
  const int n = a.B * (a.S_pad / kTile) * a.partials_per_tile;  // the dQ kernel's partials per query tile
  const float* src = a.dsinks_partial + (long long)h * n;
  float s = 0.f;
  for (int idx = tid; idx < n; idx += 256) s += src[idx];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  __shared__ float warp_sum[8];
  if (lane == 0) warp_sum[warp] = s;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += warp_sum[w];
    a.dsinks[h] = t;
  }
}

}  // namespace b200attn
