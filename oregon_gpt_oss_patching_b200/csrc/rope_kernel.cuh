// Rotary position embedding of the GPT-OSS attention layer as one pass (the step right before the
// attention kernels): the half-split rotation of Hugging Face's `_apply_rotary_emb`
// (transformers/models/gpt_oss/modeling_gpt_oss.py:226-234),
//     out[..., :32] = x[..., :32] * cos - x[..., 32:] * sin
//     out[..., 32:] = x[..., 32:] * cos + x[..., :32] * sin
// on a (batch, head, position, 64) view with arbitrary outer strides, so the projection's (B, S, H, d) output
// is read where it lies and the result is written in the layout the attention kernels take in place.
// `sin_sign` = -1 applies the inverse rotation, which is the gradient of the forward one.  The original runs
// the expression as seven elementwise tensor operations per tensor (two chunks, four products, a sum, a
// difference, a concatenation), each a pass over memory, and rounds every intermediate to bf16; here every
// element is read once and written once and the arithmetic is fp32 with one rounding.
//
// One thread rotates 8 element pairs: 16 bytes of the first half with the matching 16 bytes of the second.
#pragma once
#include "attn_common.cuh"

namespace b200attn {

struct RopeArgs {
  StridedPtr x, out;                 // (B, H, S, 64) views
  const __nv_bfloat16* cos;          // (B, S, 32), element strides below (a batch stride of 0 shares one table)
  const __nv_bfloat16* sin;
  long long cs_b, cs_s;
  int B, H, S;
  float sin_sign;
};

__global__ void rope_kernel(const RopeArgs a) {
  const long long total = (long long)a.B * a.H * a.S * 4;   // 4 threads per row
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i & 3);
    long long row = i >> 2;
    // heads fastest: neighbouring threads touch neighbouring memory when the tensor is stored (B, S, H, d)
    const int h = (int)(row % a.H);
    row /= a.H;
    const int s = (int)(row % a.S);
    const int b = (int)(row / a.S);
    const __nv_bfloat16* src = a.x.row(b, h, s);
    const uint4 lo = *reinterpret_cast<const uint4*>(src + v * 8);
    const uint4 hi = *reinterpret_cast<const uint4*>(src + 32 + v * 8);
    const long long t = b * a.cs_b + s * a.cs_s + v * 8;
    const uint4 c4 = __ldg(reinterpret_cast<const uint4*>(a.cos + t));
    const uint4 s4 = __ldg(reinterpret_cast<const uint4*>(a.sin + t));
    const uint32_t xl[4] = {lo.x, lo.y, lo.z, lo.w}, xh[4] = {hi.x, hi.y, hi.z, hi.w};
    const uint32_t cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float l0 = __uint_as_float(xl[e] << 16), l1 = __uint_as_float(xl[e] & 0xffff0000u);
      const float h0 = __uint_as_float(xh[e] << 16), h1 = __uint_as_float(xh[e] & 0xffff0000u);
      const float c0 = __uint_as_float(cc[e] << 16), c1 = __uint_as_float(cc[e] & 0xffff0000u);
      const float s0 = a.sin_sign * __uint_as_float(ss[e] << 16), s1 = a.sin_sign * __uint_as_float(ss[e] & 0xffff0000u);
      ol[e] = pack_bf16(fmaf(l0, c0, -h0 * s0), fmaf(l1, c1, -h1 * s1));
      oh[e] = pack_bf16(fmaf(h0, c0, l0 * s0), fmaf(h1, c1, l1 * s1));
    }
    __nv_bfloat16* dst = a.out.row(b, h, s);
    *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    *reinterpret_cast<uint4*>(dst + 32 + v * 8) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
}

}  // namespace b200attn
