// C ABI of the mixture-of-experts entry points (declared in include/b200moe.h): argument validation,
// TMA tensor maps, kernel launches.  No device memory is allocated here and nothing synchronises.
#include "../../include/b200moe.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include "host_common.cuh"
#include "moe_gemm_kernel.cuh"   // (includes moe_aux_kernels.cuh)

namespace {

using namespace b200moe;
using namespace b200attn::host;

// 4-D bf16 maps with the 128-byte swizzle; the inner box extent is always 64 elements.
int encode4(CUtensorMap* map, const void* ptr, const cuuint64_t (&dims)[4], const cuuint64_t (&strides)[3], const cuuint32_t (&box)[4]) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return B200ATTN_ECUDA;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200ATTN_OK : B200ATTN_ETENSORMAP;
}
// (groups, rows, inner) row-major seen as (inner, rows, groups, 1): boxes of 64 inner elements x box_rows rows.
int make_map_rows(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t groups, uint32_t box_rows) {
  const cuuint64_t dims[4] = {inner, rows, groups, 1};
  const cuuint64_t strides[3] = {inner * 2, inner * rows * 2, inner * rows * groups * 2};
  const cuuint32_t box[4] = {64, box_rows, 1, 1};
  return encode4(map, ptr, dims, strides, box);
}
// The same matrix with a width that is a multiple of 64, seen as (64, rows, width / 64, groups): one box of
// (64, 64 rows, panels) lands `panels` neighbouring 64-column panels, each as a contiguous (64 rows x 128 B) tile.
int make_map_panels(CUtensorMap* map, const void* ptr, uint64_t width, uint64_t rows, uint64_t groups, uint32_t panels) {
  const cuuint64_t dims[4] = {64, rows, width / 64, groups};
  const cuuint64_t strides[3] = {width * 2, 128, width * rows * 2};
  const cuuint32_t box[4] = {64, 64, panels, 1};
  return encode4(map, ptr, dims, strides, box);
}

int sm_count(int device) {
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) return 148;
  return n;
}

int elementwise_grid(long long work_items, int block, int device) {
  const long long want = (work_items + block - 1) / block;
  const long long cap = (long long)sm_count(device) * 16;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

int check_matrix(const void* p, int64_t cols) {
  if (p == nullptr) return B200ATTN_EINVAL;
  if (!aligned16(p) || cols % 8 != 0) return B200ATTN_EALIGN;
  return B200ATTN_OK;
}

}  // namespace

extern "C" {

size_t b200moe_sizeof_gemm_params(void) { return sizeof(b200moe_gemm_params); }

int b200moe_grouped_gemm(const b200moe_gemm_params* p) {
  if (p == nullptr || p->offsets == nullptr || p->a == nullptr || p->b == nullptr || p->d == nullptr) return B200ATTN_EINVAL;
  if (p->op < B200MOE_ROWS_NN || p->op > B200MOE_INNER_TN) return B200ATTN_EINVAL;
  if (p->num_groups <= 0 || p->num_groups > B200MOE_MAX_GROUPS || p->rows <= 0 || p->rows % B200MOE_ROW_ALIGN != 0) return B200ATTN_ESHAPE;
  const bool inner = p->op == B200MOE_INNER_TN;
  if (p->N <= 0 || (inner ? p->M <= 0 : p->K <= 0)) return B200ATTN_EINVAL;
  if (p->N % 8 != 0 || (inner ? p->M % 8 != 0 : p->K % 8 != 0)) return B200ATTN_EALIGN;
  if (!aligned16(p->a) || !aligned16(p->b) || !aligned16(p->d) || (p->bias != nullptr && !aligned16(p->bias))) return B200ATTN_EALIGN;
  if (inner && p->bias != nullptr) return B200ATTN_EINVAL;
  if (p->glu_out != nullptr && (p->op != B200MOE_ROWS_NN || p->N % 16 != 0 || !aligned16(p->glu_out))) return B200ATTN_EINVAL;
  int rc = check_device(p->device);
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;

  GemmArgs a{};
  a.mode = inner ? 1 : 0;
  a.num_groups = p->num_groups;
  a.M = inner ? p->M : 0;
  a.N = p->N;
  a.K = inner ? 0 : p->K;
  a.offsets = p->offsets;
  a.bias = static_cast<const __nv_bfloat16*>(p->bias);
  a.glu_out = static_cast<__nv_bfloat16*>(p->glu_out);
  a.status = p->status;
  CUtensorMap ta, ta_full, tb, td;
  long long max_tiles;
  const long long n_tiles = (p->N + kBN - 1) / kBN;
  if (!inner) {
    a.a_mn = 0;
    a.b_mn = p->op == B200MOE_ROWS_NN ? 1 : 0;
    a.b_merged = (a.b_mn && p->N % 64 == 0) ? 1 : 0;
    if ((rc = make_map_rows(&ta, p->a, p->K, p->rows, 1, kHalfM))) return rc;                    // (64 inner x 128 rows) boxes: half tiles
    if ((rc = make_map_rows(&ta_full, p->a, p->K, p->rows, 1, kBM))) return rc;                  // (64 inner x 256 rows) boxes: full tiles
    if (a.b_merged) {
      if ((rc = make_map_panels(&tb, p->b, p->N, p->K, p->num_groups, kBN / 64))) return rc;     // three (64 columns x 64 inner rows) panels per box
    } else if (a.b_mn) {
      if ((rc = make_map_rows(&tb, p->b, p->N, p->K, p->num_groups, 64))) return rc;             // one panel per box
    } else {
      if ((rc = make_map_rows(&tb, p->b, p->K, p->N, p->num_groups, kBN))) return rc;            // (64 inner x 192 rows) boxes
    }
    if ((rc = make_map_rows(&td, p->d, p->N, p->rows, 1, kHalfM))) return rc;
    max_tiles = ((long long)p->rows / kHalfM + p->num_groups) * n_tiles;   // an upper bound; the kernel counts the real ones
  } else {
    a.a_mn = 1;
    a.b_mn = 1;
    a.a_merged = p->M % 64 == 0 ? 1 : 0;
    a.b_merged = p->N % 64 == 0 ? 1 : 0;
    if ((rc = a.a_merged ? make_map_panels(&ta, p->a, p->M, p->rows, 1, kBM / 64) : make_map_rows(&ta, p->a, p->M, p->rows, 1, 64))) return rc;
    if ((rc = a.b_merged ? make_map_panels(&tb, p->b, p->N, p->rows, 1, kBN / 64) : make_map_rows(&tb, p->b, p->N, p->rows, 1, 64))) return rc;
    if ((rc = make_map_rows(&td, p->d, p->N, p->M, p->num_groups, kHalfM))) return rc;
    ta_full = ta;
    max_tiles = (long long)p->num_groups * ((p->M + kBM - 1) / kBM) * n_tiles;
  }
  const size_t smem = sizeof(GemmSmem) + 1024;
  if ((rc = set_smem<moe_grouped_gemm_kernel>(smem))) return rc;
  if (p->max_ctas < 0) return B200ATTN_EINVAL;
  long long sms = sm_count(p->device);
  if (p->max_ctas > 0 && p->max_ctas < sms) sms = p->max_ctas;
  const int grid = (int)(max_tiles < sms ? max_tiles : sms);
  moe_grouped_gemm_kernel<<<grid, kGemmThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(ta, ta_full, tb, td, a);
  return launch_status();
}

int b200moe_gather_rows(const void* src, const int32_t* row_src, const float* row_scale, void* out, int32_t rows,
                        int32_t cols, int32_t device, void* stream) {
  if (row_src == nullptr || rows <= 0 || cols <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_matrix(src, cols)) || (rc = check_matrix(out, cols)) || (rc = check_device(device))) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const int grid = elementwise_grid((long long)rows * (cols / 8), 256, device);
  moe_gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), row_src, row_scale, static_cast<__nv_bfloat16*>(out), rows, cols);
  return launch_status();
}

int b200moe_combine_rows(const void* y, const int32_t* pos, const float* weights, void* out, int32_t tokens,
                         int32_t top_k, int32_t cols, int32_t device, void* stream) {
  if (pos == nullptr || tokens <= 0 || top_k <= 0 || cols <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_matrix(y, cols)) || (rc = check_matrix(out, cols)) || (rc = check_device(device))) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const int grid = elementwise_grid((long long)tokens * (cols / 8), 256, device);
  moe_combine_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), pos, weights, static_cast<__nv_bfloat16*>(out), tokens, top_k, cols);
  return launch_status();
}

int b200moe_row_dot(const void* g, const void* y, const int32_t* pos, float* dots, int32_t tokens, int32_t top_k,
                    int32_t cols, int32_t device, void* stream) {
  if (pos == nullptr || dots == nullptr || tokens <= 0 || top_k <= 0 || cols <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_matrix(g, cols)) || (rc = check_matrix(y, cols)) || (rc = check_device(device))) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const int pairs = tokens * top_k;
  const int grid = elementwise_grid((long long)pairs * 32, 256, device);
  moe_row_dot_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(y), pos, dots, pairs, top_k, cols);
  return launch_status();
}

int b200moe_glu(const void* y1, void* h, int64_t rows, int32_t cols_h, int32_t device, void* stream) {
  if (rows <= 0 || cols_h <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_matrix(y1, 2 * (int64_t)cols_h)) || (rc = check_matrix(h, cols_h)) || (rc = check_device(device))) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const int grid = elementwise_grid(rows * (cols_h / 8), 256, device);
  moe_glu_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(y1),
                                                                       static_cast<__nv_bfloat16*>(h), rows, cols_h);
  return launch_status();
}

int b200moe_glu_bwd(const void* y1, const void* dh, void* dy1, int64_t rows, int32_t cols_h, int32_t device,
                    void* stream) {
  if (rows <= 0 || cols_h <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_matrix(y1, 2 * (int64_t)cols_h)) || (rc = check_matrix(dy1, 2 * (int64_t)cols_h)) ||
      (rc = check_matrix(dh, cols_h)) || (rc = check_device(device)))
    return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const int grid = elementwise_grid(rows * (cols_h / 8), 256, device);
  moe_glu_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y1), static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(dy1), rows, cols_h);
  return launch_status();
}

int b200moe_bias_grad(const void* dy, const int32_t* offsets, void* db, int32_t num_groups, int32_t cols,
                      int32_t device, void* stream) {
  if (offsets == nullptr || num_groups <= 0 || cols <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_matrix(dy, cols)) || (rc = check_matrix(db, cols)) || (rc = check_device(device))) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const int cols_per_block = kBiasGradColLanes * 8;
  const dim3 grid((cols + cols_per_block - 1) / cols_per_block, num_groups);
  moe_bias_grad_kernel<<<grid, kBiasGradRowLanes * kBiasGradColLanes, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(dy), offsets,
                                                                             static_cast<__nv_bfloat16*>(db), cols);
  return launch_status();
}

int b200moe_route(const int64_t* indices, const float* weights, int32_t tokens, int32_t top_k, int32_t num_groups, int32_t rows,
                  int32_t* offsets, int32_t* row_token, int32_t* pos, float* row_weight, int32_t device, void* stream) {
  if (indices == nullptr || weights == nullptr || offsets == nullptr || row_token == nullptr || pos == nullptr || row_weight == nullptr)
    return B200ATTN_EINVAL;
  if (tokens <= 0 || top_k <= 0 || num_groups <= 0 || num_groups > kRouteMaxGroups) return B200ATTN_ESHAPE;
  const long long pairs = (long long)tokens * top_k;
  // room for any routing: every group may waste up to 127 rows
  if (rows % B200MOE_ROW_ALIGN != 0 || rows < pairs + (long long)num_groups * (B200MOE_ROW_ALIGN - 1) || pairs > (1ll << 30))
    return B200ATTN_ESHAPE;
  int rc = check_device(device);
  if (rc) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(row_token, 0xff, (size_t)rows * sizeof(int32_t), st) != cudaSuccess ||      // -1: padding row
      cudaMemsetAsync(row_weight, 0, (size_t)rows * sizeof(float), st) != cudaSuccess)
    return B200ATTN_ECUDA;
  moe_route_kernel<<<1, kRouteThreads, 0, st>>>(reinterpret_cast<const long long*>(indices), weights, (int)pairs, top_k, num_groups,
                                                   offsets, row_token, pos, row_weight);
  return launch_status();
}

}  // extern "C"
