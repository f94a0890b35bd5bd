// The memory-bound steps around the grouped GEMMs of the mixture-of-experts block: moving token rows into
// and out of the expert-sorted buffer, the gated activation and its derivative, and the bias gradients.
// They stand in for the indexing and elementwise tensor operations of GptOssExperts.forward
// (transformers/models/gpt_oss/modeling_gpt_oss.py:76-82 `_apply_gate`, :104 `hidden_states[token_idx]`,
// :108-109 `out * routing_weights[...]`, `index_add_`) and for what autograd derives from them.  Every sum is
// taken in a fixed order in fp32 (the index_add_ of the original accumulates bf16 values with atomics).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

constexpr float kGluAlpha = 1.702f;   // GptOssExperts.alpha
constexpr float kGluLimit = 7.0f;     // GptOssExperts.limit

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// out[r, :] = src[row_src[r], :] * (row_scale ? row_scale[r] : 1)   when row_src[r] >= 0, zeros otherwise.
// One thread moves 16 bytes; `cols` is a multiple of 8.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ row_src,
                                       const float* __restrict__ row_scale, __nv_bfloat16* __restrict__ out,
                                       int rows, int cols) {
  const int vec_per_row = cols >> 3;
  const long long total = (long long)rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row), c = (int)(i - (long long)r * vec_per_row);
    const int s = row_src[r];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (s >= 0) {
      v = __ldg(reinterpret_cast<const uint4*>(src + (long long)s * cols) + c);
      if (row_scale != nullptr) {
        const float w = row_scale[r];
        v.x = pack2(bf16_lo(v.x) * w, bf16_hi(v.x) * w);
        v.y = pack2(bf16_lo(v.y) * w, bf16_hi(v.y) * w);
        v.z = pack2(bf16_lo(v.z) * w, bf16_hi(v.z) * w);
        v.w = pack2(bf16_lo(v.w) * w, bf16_hi(v.w) * w);
      }
    }
    reinterpret_cast<uint4*>(out + (long long)r * cols)[c] = v;
  }
}

// out[t, :] = sum_{j < top_k} (weights ? weights[t, j] : 1) * y[pos[t, j], :]   (fp32 sum, j ascending)
__global__ void moe_combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                        const float* __restrict__ weights, __nv_bfloat16* __restrict__ out,
                                        int tokens, int top_k, int cols) {
  const int vec_per_row = cols >> 3;
  const long long total = (long long)tokens * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row), c = (int)(i - (long long)t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int r = pos[t * top_k + j];
      const float w = weights != nullptr ? weights[t * top_k + j] : 1.f;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + (long long)r * cols) + c);
      acc[0] = fmaf(w, bf16_lo(v.x), acc[0]); acc[1] = fmaf(w, bf16_hi(v.x), acc[1]);
      acc[2] = fmaf(w, bf16_lo(v.y), acc[2]); acc[3] = fmaf(w, bf16_hi(v.y), acc[3]);
      acc[4] = fmaf(w, bf16_lo(v.z), acc[4]); acc[5] = fmaf(w, bf16_hi(v.z), acc[5]);
      acc[6] = fmaf(w, bf16_lo(v.w), acc[6]); acc[7] = fmaf(w, bf16_hi(v.w), acc[7]);
    }
    reinterpret_cast<uint4*>(out + (long long)t * cols)[c] =
        make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7]));
  }
}

// dots[t, j] = sum_c g[t, c] * y[pos[t, j], c]: the gradient of the routing weight of (token t, choice j).
// One warp per (t, j); lanes stride the row 16 bytes at a time, partials added by a shuffle tree (fixed order).
__global__ void moe_row_dot_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ y,
                                   const int* __restrict__ pos, float* __restrict__ dots, int pairs, int top_k, int cols) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int p = blockIdx.x * warps_per_block + (threadIdx.x >> 5); p < pairs; p += gridDim.x * warps_per_block) {
    const int t = p / top_k;
    const uint4* gr = reinterpret_cast<const uint4*>(g + (long long)t * cols);
    const uint4* yr = reinterpret_cast<const uint4*>(y + (long long)pos[p] * cols);
    float acc = 0.f;
    for (int c = lane; c < (cols >> 3); c += 32) {
      const uint4 a = __ldg(gr + c), b = __ldg(yr + c);
      acc = fmaf(bf16_lo(a.x), bf16_lo(b.x), acc); acc = fmaf(bf16_hi(a.x), bf16_hi(b.x), acc);
      acc = fmaf(bf16_lo(a.y), bf16_lo(b.y), acc); acc = fmaf(bf16_hi(a.y), bf16_hi(b.y), acc);
      acc = fmaf(bf16_lo(a.z), bf16_lo(b.z), acc); acc = fmaf(bf16_hi(a.z), bf16_hi(b.z), acc);
      acc = fmaf(bf16_lo(a.w), bf16_lo(b.w), acc); acc = fmaf(bf16_hi(a.w), bf16_hi(b.w), acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) dots[p] = acc;
  }
}

// The gated activation on interleaved (gate, up) column pairs (modeling_gpt_oss.py:76-82):
//   gate = min(g, limit), up = clamp(u, -limit, limit), h = (up + 1) * gate * sigmoid(alpha * gate).
struct GluParts {
  float gate, up, sig;
};
__device__ __forceinline__ GluParts glu_parts(float g, float u) {
  GluParts p;
  p.gate = fminf(g, kGluLimit);
  p.up = fminf(fmaxf(u, -kGluLimit), kGluLimit);
  p.sig = 1.f / (1.f + __expf(-kGluAlpha * p.gate));
  return p;
}
__device__ __forceinline__ float glu_value(uint32_t gate_up) {
  const GluParts p = glu_parts(bf16_lo(gate_up), bf16_hi(gate_up));
  return (p.up + 1.f) * p.gate * p.sig;
}

// h[r, c] = glu(y1[r, 2c], y1[r, 2c + 1]); y1 has 2 * cols_h columns.  One thread: 16 input -> 8 output columns.
__global__ void moe_glu_kernel(const __nv_bfloat16* __restrict__ y1, __nv_bfloat16* __restrict__ h, long long rows, int cols_h) {
  const int vec_per_row = cols_h >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(y1) + 2 * i;   // (rows are 2 * cols_h wide: vector 2i, 2i+1 of the flat array)
    const uint4 a = __ldg(src), b = __ldg(src + 1);
    reinterpret_cast<uint4*>(h)[i] = make_uint4(pack2(glu_value(a.x), glu_value(a.y)), pack2(glu_value(a.z), glu_value(a.w)),
                                                pack2(glu_value(b.x), glu_value(b.y)), pack2(glu_value(b.z), glu_value(b.w)));
  }
}

// dy1[r, 2c], dy1[r, 2c + 1] from dh[r, c] and y1 (clamps pass the gradient inside their closed range, as torch.clamp does).
__device__ __forceinline__ uint32_t glu_grad(uint32_t gate_up, float dh) {
  const float g = bf16_lo(gate_up), u = bf16_hi(gate_up);
  const GluParts p = glu_parts(g, u);
  const float glu = p.gate * p.sig;
  const float d_gate = g <= kGluLimit ? dh * (p.up + 1.f) * (p.sig + kGluAlpha * glu * (1.f - p.sig)) : 0.f;
  const float d_up = (u >= -kGluLimit && u <= kGluLimit) ? dh * glu : 0.f;
  return pack2(d_gate, d_up);
}
__global__ void moe_glu_bwd_kernel(const __nv_bfloat16* __restrict__ y1, const __nv_bfloat16* __restrict__ dh,
                                   __nv_bfloat16* __restrict__ dy1, long long rows, int cols_h) {
  const int vec_per_row = cols_h >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(y1) + 2 * i;
    const uint4 a = __ldg(src), b = __ldg(src + 1);
    const uint4 d = __ldg(reinterpret_cast<const uint4*>(dh) + i);
    uint4* dst = reinterpret_cast<uint4*>(dy1) + 2 * i;
    dst[0] = make_uint4(glu_grad(a.x, bf16_lo(d.x)), glu_grad(a.y, bf16_hi(d.x)), glu_grad(a.z, bf16_lo(d.y)), glu_grad(a.w, bf16_hi(d.y)));
    dst[1] = make_uint4(glu_grad(b.x, bf16_lo(d.z)), glu_grad(b.y, bf16_hi(d.z)), glu_grad(b.z, bf16_lo(d.w)), glu_grad(b.w, bf16_hi(d.w)));
  }
}

// db[g, c] = sum over the rows r of group g of dy[r, c], in fp32, in an order fixed by the launch shape alone.
// Block = (group, 128 columns), 256 threads as 16 column lanes x 16 row lanes: a thread owns 8 columns (one 16-byte
// load per row) and sums rows r0 + y, r0 + y + 16, ...; the sixteen partials of a column are then added in row-lane
// order.  (128 columns per block rather than 256: twice the blocks and loads in flight for the 2880-column case.)
constexpr int kBiasGradRowLanes = 16;
constexpr int kBiasGradColLanes = 16;
__global__ void __launch_bounds__(kBiasGradRowLanes * kBiasGradColLanes)
moe_bias_grad_kernel(const __nv_bfloat16* __restrict__ dy, const int* __restrict__ offsets,
                     __nv_bfloat16* __restrict__ db, int cols) {
  __shared__ float part[kBiasGradRowLanes][kBiasGradColLanes][9];   // (padded against bank conflicts)
  const int g = blockIdx.y;
  const int x = threadIdx.x % kBiasGradColLanes, y = threadIdx.x / kBiasGradColLanes;
  const int c0 = (blockIdx.x * kBiasGradColLanes + x) * 8;
  const int r0 = offsets[g], r1 = offsets[g + 1];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < cols) {
    const uint4* col = reinterpret_cast<const uint4*>(dy + c0);
    const long long stride = cols >> 3;
#pragma unroll 4
    for (int r = r0 + y; r < r1; r += kBiasGradRowLanes) {
      const uint4 v = __ldg(col + r * stride);
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) part[y][x][e] = acc[e];
  __syncthreads();
  if (y == 0 && c0 < cols) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      s[e] = part[0][x][e];
#pragma unroll
      for (int k = 1; k < kBiasGradRowLanes; ++k) s[e] += part[k][x][e];
    }
    *reinterpret_cast<uint4*>(db + (long long)g * cols + c0) =
        make_uint4(pack2(s[0], s[1]), pack2(s[2], s[3]), pack2(s[4], s[5]), pack2(s[6], s[7]));
  }
}

// Routing bookkeeping in one launch of one CTA: the (token, choice) pairs sorted by expert (stable: inside an expert
// the pairs keep their order), every expert's segment starting at a multiple of 128 rows.  Stands in for the
// `one_hot` / `nonzero` / `torch.where` bookkeeping of GptOssExperts.forward (modeling_gpt_oss.py:86-103), which
// synchronises with the host once per expert.  Warp w owns the contiguous pairs [w * chunk, (w + 1) * chunk) and
// walks them 32 at a time (coalesced loads, the next batch's in flight under this one's bookkeeping):
//   1. count: the lanes of a batch that share an expert find each other (`match.any`), the lowest of them adds
//      their number to the warp's counter of that expert (shared memory, one column per warp);
//   2. one warp per expert turns the 32 counts into exclusive prefix sums (the warp's first row inside the
//      expert's segment) and the expert's total;
//   3. thread 0 lays the segments out (totals rounded up to 128);
//   4. the same walk again: a pair's row is segment start + the warp's running count + the number of lower lanes
//      of the batch with the same expert; row_token / row_weight are written at that row and the row into pos.
// row_token and row_weight must hold -1 / 0 for the padding rows before the launch (the entry point clears them).
constexpr int kRouteThreads = 1024;
constexpr int kRouteWarps = kRouteThreads / 32;
constexpr int kRouteAlign = 128;
constexpr int kRouteMaxGroups = 256;
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const long long* __restrict__ indices, const float* __restrict__ weights, int pairs, int top_k, int num_groups,
                 int* __restrict__ offsets, int* __restrict__ row_token, int* __restrict__ pos, float* __restrict__ row_weight) {
  __shared__ int cnt[kRouteMaxGroups][kRouteWarps + 1];   // counts, then first rows inside the segment (+1: no bank conflicts in step 2)
  __shared__ int seg_start[kRouteMaxGroups + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = ((pairs + kRouteWarps - 1) / kRouteWarps + 31) / 32 * 32;   // whole batches per warp
  const int p0 = min(warp * chunk, pairs), p1 = min(p0 + chunk, pairs);
  for (int i = tid; i < num_groups * (kRouteWarps + 1); i += kRouteThreads) (&cnt[0][0])[i] = 0;
  __syncthreads();
  // an index out of range is no expert's pair: it gets no row
  auto expert_of = [&](int p) -> int {
    if (p >= p1) return -1;
    const int e = (int)indices[p];
    return (unsigned)e < (unsigned)num_groups ? e : -1;
  };
  int e_next = expert_of(p0 + lane);
  for (int p = p0; p < p1; p += 32) {
    const int e = e_next;
    e_next = expert_of(p + 32 + lane);
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && lane == __ffs(same) - 1) cnt[e][warp] += __popc(same);
    __syncwarp();   // the next batch's leader of this expert may be another lane
  }
  __syncthreads();
  for (int e = warp; e < num_groups; e += kRouteWarps) {
    const int c = cnt[e][lane];
    int incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += up;
    }
    cnt[e][lane] = incl - c;
    if (lane == 31) seg_start[e + 1] = incl;   // the expert's total, for now
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    seg_start[0] = 0;
    offsets[0] = 0;
    for (int e = 0; e < num_groups; ++e) {
      acc += (seg_start[e + 1] + kRouteAlign - 1) / kRouteAlign * kRouteAlign;
      seg_start[e + 1] = acc;
      offsets[e + 1] = acc;
    }
  }
  __syncthreads();
  e_next = expert_of(p0 + lane);
  float w_next = p0 + lane < p1 ? weights[p0 + lane] : 0.f;
  for (int p = p0; p < p1; p += 32) {
    const int e = e_next;
    const float w = w_next;
    e_next = expert_of(p + 32 + lane);
    w_next = p + 32 + lane < p1 ? weights[p + 32 + lane] : 0.f;
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    if (e >= 0) {
      const int row = seg_start[e] + cnt[e][warp] + __popc(same & ((1u << lane) - 1u));
      row_token[row] = (p + lane) / top_k;
      row_weight[row] = w;
      pos[p + lane] = row;
    } else if (p + lane < p1) {
      pos[p + lane] = 0;
    }
    __syncwarp();
    if (e >= 0 && lane == __ffs(same) - 1) cnt[e][warp] += __popc(same);
    __syncwarp();
  }
}

}  // namespace b200moe
