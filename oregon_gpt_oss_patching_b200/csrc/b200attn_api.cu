// C ABI of the library (declared in include/b200attn.h): argument validation, TMA tensor
// maps, kernel launches.  No device memory is allocated here and nothing synchronises.
#include "../../include/b200attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "attn_common.cuh"
#include "host_common.cuh"
#include "bwd_dkdv_kernel.cuh"
#include "bwd_dq_kernel.cuh"
#include "bwd_dq_persistent_kernel.cuh"
#include "bwd_preprocess_kernel.cuh"
#include "bwd_window_fused_kernel.cuh"
#include "fwd_kernel.cuh"
#include "fwd_packed_kernel.cuh"
#include "rope_kernel.cuh"
#include "umma_selftest.cuh"

namespace {

using namespace b200attn;
using namespace b200attn::host;

// A dimension of extent 1 may carry any stride; give it a harmless one.
int64_t usable_stride(int64_t stride, int64_t extent, int64_t fallback) { return extent == 1 ? fallback : stride; }

int check_tensor(const b200attn_tensor& t, int B, int H, int S) {
  if (t.ptr == nullptr) return B200ATTN_EINVAL;
  if (!aligned16(t.ptr)) return B200ATTN_EALIGN;
  const int64_t ss = usable_stride(t.stride_s, S, kHeadDim), sh = usable_stride(t.stride_h, H, kHeadDim),
                sb = usable_stride(t.stride_b, B, kHeadDim);
  if (ss % 8 || sh % 8 || sb % 8 || ss < kHeadDim || sh <= 0 || sb <= 0) return B200ATTN_EALIGN;
  return B200ATTN_OK;
}

// 4-D bf16 map (d, S, H, B) with a (64 x rows x heads) box and the 128-byte swizzle.
int make_map(CUtensorMap* map, const b200attn_tensor& t, int B, int H, int S, int box_rows, int box_heads = 1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return B200ATTN_ECUDA;
  const int64_t ss = usable_stride(t.stride_s, S, kHeadDim), sh = usable_stride(t.stride_h, H, (int64_t)S * ss),
                sb = usable_stride(t.stride_b, B, (int64_t)S * ss);
  cuuint64_t dims[4] = {(cuuint64_t)kHeadDim, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {(cuuint32_t)kHeadDim, (cuuint32_t)box_rows, (cuuint32_t)box_heads, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200ATTN_OK : B200ATTN_ETENSORMAP;
}

StridedPtr strided(const b200attn_tensor& t) {
  return StridedPtr{static_cast<__nv_bfloat16*>(t.ptr), (long long)t.stride_b, (long long)t.stride_h, (long long)t.stride_s};
}

enum Need { kNeedFwd = 1, kNeedBwdIn = 2, kNeedDelta = 4, kNeedPartial = 8, kNeedDq = 16, kNeedDkv = 32, kNeedDsinks = 64 };

int validate(const b200attn_params* p, int need) {
  if (p == nullptr) return B200ATTN_EINVAL;
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->S <= 0 || !(p->scale > 0.f)) return B200ATTN_EINVAL;
  if (p->d != kHeadDim) return B200ATTN_EHEADDIM;
  if (p->Hq % p->Hkv != 0 || p->window < 0 || p->S > (1 << 24) || p->B > 65535 || p->Hq > 65535) return B200ATTN_ESHAPE;
  if (p->sinks == nullptr || p->lse == nullptr) return B200ATTN_EINVAL;
  if (!aligned16(p->lse)) return B200ATTN_EALIGN;
  int rc;
  if ((rc = check_tensor(p->q, p->B, p->Hq, p->S))) return rc;
  if ((rc = check_tensor(p->k, p->B, p->Hkv, p->S))) return rc;
  if ((rc = check_tensor(p->v, p->B, p->Hkv, p->S))) return rc;
  if (need & (kNeedFwd | kNeedBwdIn))
    if ((rc = check_tensor(p->o, p->B, p->Hq, p->S))) return rc;
  if (need & kNeedBwdIn)
    if ((rc = check_tensor(p->d_o, p->B, p->Hq, p->S))) return rc;
  if (need & kNeedDelta) {
    if (p->delta == nullptr) return B200ATTN_ESCRATCH;
    if (!aligned16(p->delta)) return B200ATTN_EALIGN;
  }
  if ((need & kNeedPartial) && p->dsinks_partial == nullptr) return B200ATTN_ESCRATCH;
  if ((need & kNeedDsinks) && p->dsinks == nullptr) return B200ATTN_EINVAL;
  if (need & kNeedDq)
    if ((rc = check_tensor(p->dq, p->B, p->Hq, p->S))) return rc;
  if (need & kNeedDkv) {
    if ((rc = check_tensor(p->dk, p->B, p->Hkv, p->S))) return rc;
    if ((rc = check_tensor(p->dv, p->B, p->Hkv, p->S))) return rc;
  }
  return check_device(p->device);
}

bool packed_window_layer(const b200attn_params* p);
bool fused_window_bwd(const b200attn_params* p);

KernelArgs make_args(const b200attn_params* p) {
  KernelArgs a{};
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.S = p->S;
  a.S_pad = (int)b200attn_padded_len(p->S);
  a.group = p->Hq / p->Hkv;
  a.window = p->window;
  a.scale = p->scale;
  a.scale_log2 = p->scale * kLog2e;
  a.seqlens = p->seqlens;
  a.sinks = p->sinks;
  a.status = p->status;
  a.lse = p->lse;
  a.delta = p->delta;
  a.dsinks = p->dsinks;
  a.dsinks_partial = p->dsinks_partial;
  a.fused_bwd = fused_window_bwd(p) ? 1 : 0;
  a.partials_per_tile = a.fused_bwd ? kFwSinkPartials : 8;
  a.o = strided(p->o); a.d_o = strided(p->d_o); a.dq = strided(p->dq); a.dk = strided(p->dk); a.dv = strided(p->dv);
  a.q = strided(p->q); a.k = strided(p->k); a.v = strided(p->v);
  return a;
}

// Layers the head-packed kernels serve: a causal window of at most 128 keys with 8 query heads per KV head.
bool packed_window_layer(const b200attn_params* p) {
  return p->window > 0 && p->window <= kPkMaxWindow && p->Hq / p->Hkv == kPkHeads;
}

// Layers whose backward is one kernel: a query tile is seen by at most two key tiles, so the kernel's dQ
// contributions can be added in global memory without the result depending on their order.
bool fused_window_bwd(const b200attn_params* p) { return p->window > 0 && p->window <= kFwMaxWindow; }



}  // namespace

extern "C" {

int b200attn_version(void) { return B200ATTN_VERSION; }

size_t b200attn_sizeof_params(void) { return sizeof(b200attn_params); }

const char* b200attn_strerror(int code) {
  switch (code) {
    case B200ATTN_OK: return "success";
    case B200ATTN_EINVAL: return "invalid argument (NULL pointer, non-positive size or scale)";
    case B200ATTN_ESHAPE: return "unsupported shape (Hq % Hkv != 0, negative window, or size out of range)";
    case B200ATTN_EHEADDIM: return "unsupported head_dim (only 64)";
    case B200ATTN_EALIGN: return "pointer not 16-byte aligned or stride not a multiple of 8 elements";
    case B200ATTN_EDEVICE: return "device is not an sm_100 (compute capability 10.x) GPU";
    case B200ATTN_ECUDA: return "a CUDA runtime or driver call failed";
    case B200ATTN_ETENSORMAP: return "the driver rejected a TMA tensor map";
    case B200ATTN_ESCRATCH: return "scratch buffer missing";
    case B200ATTN_ETOOLARGE: return "problem exceeds the fixed scratch of b200attn_bwd_static_scratch (B*Hq*S_pad > B200ATTN_STATIC_MAX_ROWS)";
    default: return "unknown b200attn error code";
  }
}

int64_t b200attn_padded_len(int64_t S) { return (S + B200ATTN_ROW_TILE - 1) / B200ATTN_ROW_TILE * B200ATTN_ROW_TILE; }

int64_t b200attn_dsinks_scratch_floats(const b200attn_params* p) {
  if (p == nullptr) return 0;
  return (int64_t)p->Hq * p->B * (b200attn_padded_len(p->S) / B200ATTN_ROW_TILE) * 9;
}

int b200attn_fwd(const b200attn_params* p) {
  int rc = validate(p, kNeedFwd);
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;
  CUtensorMap tq, tk, tv;
  const KernelArgs a = make_args(p);
  if (packed_window_layer(p)) {
    // the GPT-OSS sliding-window layer: tiles of 8 heads x 16 positions, one 144-key product per tile
    if ((rc = make_map(&tq, p->q, p->B, p->Hq, p->S, kPkPos, kPkHeads))) return rc;
    if ((rc = make_map(&tk, p->k, p->B, p->Hkv, p->S, kPkKvRows))) return rc;
    if ((rc = make_map(&tv, p->v, p->B, p->Hkv, p->S, kPkKvRows))) return rc;
    CUtensorMap to;
    if ((rc = make_map(&to, p->o, p->B, p->Hq, p->S, kPkPos, kPkHeads))) return rc;
    const size_t smem = sizeof(FwdPkSmem) + 1024;
    if ((rc = set_smem<attn_fwd_packed_kernel>(smem))) return rc;
    int n_sm = 0;
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, p->device) != cudaSuccess || n_sm <= 0) return B200ATTN_ECUDA;
    const long long n_items = (long long)(a.S_pad / kPkItemPos) * p->B * p->Hkv;
    const unsigned grid = (unsigned)(n_items < n_sm ? n_items : n_sm);
    attn_fwd_packed_kernel<<<grid, kFwdPkThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tq, tk, tv, to, a);
    return launch_status();
  }
  if ((rc = make_map(&tq, p->q, p->B, p->Hq, p->S, kTile))) return rc;
  if ((rc = make_map(&tk, p->k, p->B, p->Hkv, p->S, kTile))) return rc;
  if ((rc = make_map(&tv, p->v, p->B, p->Hkv, p->S, kTile))) return rc;
  const int heads_per_item = (a.group % 2 == 0) ? 2 : 1;  // two heads of a KV group share staged K/V tiles
  if (p->window > 0 && p->window <= 32 * kTile) {
    // short work items (measured cross-over near 4096 keys): the persistent kernel, one CTA per SM
    // walking the items, hides the per-item set-up and first-load latency that dominate them
    const size_t smem = sizeof(FwdSmem) + 1024;
    if ((rc = set_smem<attn_fwd_persistent_kernel>(smem))) return rc;
    int n_sm = 0;
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, p->device) != cudaSuccess || n_sm <= 0) return B200ATTN_ECUDA;
    const long long n_items = (long long)(a.S_pad / kTile) * p->B * (p->Hq / heads_per_item);
    const unsigned grid = (unsigned)(n_items < n_sm ? n_items : n_sm);
    attn_fwd_persistent_kernel<<<grid, kFwdThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tq, tk, tv, a);
    return launch_status();
  }
  const size_t smem = sizeof(FwdOneSmem) + 1024;
  if ((rc = set_smem<attn_fwd_kernel>(smem))) return rc;
  dim3 grid(a.S_pad / kTile, p->Hq / heads_per_item, p->B);
  attn_fwd_kernel<<<grid, kFwdThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tq, tk, tv, a);
  return launch_status();
}

int b200attn_bwd_dq_is_fused(const b200attn_params* p) { return (p != nullptr && fused_window_bwd(p)) ? 1 : 0; }

int b200attn_bwd_preprocess(const b200attn_params* p) {
  if (p == nullptr) return B200ATTN_EINVAL;
  int rc = validate(p, kNeedBwdIn | kNeedDelta | (fused_window_bwd(p) ? (kNeedDq | kNeedPartial) : 0));
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const KernelArgs a = make_args(p);
  dim3 grid(a.S_pad / kTile, p->Hq, p->B);
  attn_bwd_preprocess_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(p->stream)>>>(a);
  return launch_status();
}

int b200attn_bwd_dsinks(const b200attn_params* p) {
  int rc = validate(p, kNeedPartial | kNeedDsinks);
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;
  const KernelArgs a = make_args(p);
  attn_bwd_dsinks_kernel<<<p->Hq, 256, 0, static_cast<cudaStream_t>(p->stream)>>>(a);
  return launch_status();
}

int b200attn_bwd_dkdv(const b200attn_params* p) {
  if (p == nullptr) return B200ATTN_EINVAL;
  int rc = validate(p, kNeedBwdIn | kNeedDelta | kNeedDkv | (fused_window_bwd(p) ? kNeedDq : 0));
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;
  CUtensorMap tq, tk, tv, tdo;
  if ((rc = make_map(&tq, p->q, p->B, p->Hq, p->S, kTile))) return rc;
  if ((rc = make_map(&tk, p->k, p->B, p->Hkv, p->S, kTile))) return rc;
  if ((rc = make_map(&tv, p->v, p->B, p->Hkv, p->S, kTile))) return rc;
  if ((rc = make_map(&tdo, p->d_o, p->B, p->Hq, p->S, kTile))) return rc;
  CUtensorMap tdk, tdv;   // the tiles leave with one TMA store each
  if ((rc = make_map(&tdk, p->dk, p->B, p->Hkv, p->S, kTile))) return rc;
  if ((rc = make_map(&tdv, p->dv, p->B, p->Hkv, p->S, kTile))) return rc;
  const KernelArgs a = make_args(p);
  dim3 grid(a.S_pad / kTile, p->Hkv, p->B);
  if (fused_window_bwd(p)) {
    // narrow window: dQ comes out of the same pass (added into the rows the preprocess kernel cleared)
    CUtensorMap tdq;
    if ((rc = make_map(&tdq, p->dq, p->B, p->Hq, p->S, kTile))) return rc;
    const size_t fsmem = sizeof(FwSmem) + 1024;
    if ((rc = set_smem<attn_bwd_window_fused_kernel>(fsmem))) return rc;
    attn_bwd_window_fused_kernel<<<grid, kFwThreads, fsmem, static_cast<cudaStream_t>(p->stream)>>>(tq, tk, tv, tdo, tdk, tdv, tdq, a);
    return launch_status();
  }
  const size_t smem = sizeof(DkvSmem) + 1024;
  if (p->window > 0 && p->window <= 2 * kTile) {
    // narrow window: most tiles are partly masked, skipping the chunks nobody sees pays
    if ((rc = set_smem<attn_bwd_dkdv_kernel<true>>(smem))) return rc;
    attn_bwd_dkdv_kernel<true><<<grid, kDkvThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tq, tk, tv, tdo, tdk, tdv, a);
  } else {
    if ((rc = set_smem<attn_bwd_dkdv_kernel<false>>(smem))) return rc;
    attn_bwd_dkdv_kernel<false><<<grid, kDkvThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tq, tk, tv, tdo, tdk, tdv, a);
  }
  return launch_status();
}

int b200attn_bwd_dq(const b200attn_params* p) {
  int rc = validate(p, kNeedBwdIn | kNeedDelta | kNeedDq | kNeedPartial);
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;
  if (fused_window_bwd(p)) return B200ATTN_OK;   // the dK/dV stage made dQ as well
  CUtensorMap tk, tv;
  const KernelArgs a = make_args(p);
  dim3 grid(a.S_pad / kTile, p->Hq, p->B);
  if (p->window > 0 && p->window <= 8 * kTile) {
    // short work items (at most nine key tiles per query tile; measured cross-over between 1024 and 2048
    // keys): the persistent kernel, one CTA per SM walking the items
    CUtensorMap tq, tdo;
    if ((rc = make_map(&tq, p->q, p->B, p->Hq, p->S, kTile))) return rc;
    if ((rc = make_map(&tdo, p->d_o, p->B, p->Hq, p->S, kTile))) return rc;
    if ((rc = make_map(&tk, p->k, p->B, p->Hkv, p->S, kTile))) return rc;
    if ((rc = make_map(&tv, p->v, p->B, p->Hkv, p->S, kTile))) return rc;
    const size_t smem = sizeof(DqpSmem) + 1024;
    if ((rc = set_smem<attn_bwd_dq_persistent_kernel>(smem))) return rc;
    int n_sm = 0;
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, p->device) != cudaSuccess || n_sm <= 0) return B200ATTN_ECUDA;
    const long long n_items = (long long)(a.S_pad / kTile) * p->B * p->Hq;
    const unsigned pgrid = (unsigned)(n_items < n_sm ? n_items : n_sm);
    attn_bwd_dq_persistent_kernel<<<pgrid, kDqpThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tq, tdo, tk, tv, a);
    return launch_status();
  }
  if ((rc = make_map(&tk, p->k, p->B, p->Hkv, p->S, kTile))) return rc;
  if ((rc = make_map(&tv, p->v, p->B, p->Hkv, p->S, kTile))) return rc;
  const size_t smem = sizeof(DqSmem) + 1024;
  if ((rc = set_smem<attn_bwd_dq_kernel>(smem))) return rc;
  attn_bwd_dq_kernel<<<grid, kDqThreads, smem, static_cast<cudaStream_t>(p->stream)>>>(tk, tv, a);
  return launch_status();
}

int b200attn_bwd(const b200attn_params* p) {
  int rc = validate(p, kNeedBwdIn | kNeedDelta | kNeedPartial | kNeedDsinks | kNeedDq | kNeedDkv);
  if (rc) return rc;
  if ((rc = b200attn_bwd_preprocess(p))) return rc;
  if ((rc = b200attn_bwd_dkdv(p))) return rc;
  if ((rc = b200attn_bwd_dq(p))) return rc;
  return b200attn_bwd_dsinks(p);
}

// ---- backward without caller-provided scratch ------------------------------------------------
// Fixed device-resident scratch for b200attn_bwd_static_scratch.  Every GPU that loads the
// library holds these ~6.4 MB until the process exits.
constexpr int64_t kStaticMaxRows = B200ATTN_STATIC_MAX_ROWS;
static __device__ __align__(256) float g_static_delta[B200ATTN_DELTA_PLANES * kStaticMaxRows];   // delta | -lse*log2(e) | side tiles
static __device__ __align__(256) float g_static_dsinks_partial[kStaticMaxRows / 128 * 9];  // up to 9 partials per 128 rows

namespace {
std::mutex g_static_mutex;
float* g_static_delta_ptr[kMaxDevices] = {};
float* g_static_partial_ptr[kMaxDevices] = {};

// The arrays' names are host-side stand-ins, not device addresses: resolve them once per device,
// with that device current.
int static_scratch_for(int device, float** delta, float** partial) {
  if (device < 0 || device >= kMaxDevices) return B200ATTN_EDEVICE;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_delta_ptr[device] == nullptr) {
    void* d = nullptr;
    void* s = nullptr;
    if (cudaGetSymbolAddress(&d, g_static_delta) != cudaSuccess) return B200ATTN_ECUDA;
    if (cudaGetSymbolAddress(&s, g_static_dsinks_partial) != cudaSuccess) return B200ATTN_ECUDA;
    g_static_delta_ptr[device] = static_cast<float*>(d);
    g_static_partial_ptr[device] = static_cast<float*>(s);
  }
  *delta = g_static_delta_ptr[device];
  *partial = g_static_partial_ptr[device];
  return B200ATTN_OK;
}
}  // namespace

int b200attn_bwd_static_scratch(const b200attn_params* p) {
  if (p == nullptr) return B200ATTN_EINVAL;
  if (p->B <= 0 || p->Hq <= 0 || p->S <= 0) return B200ATTN_EINVAL;
  const int64_t rows = (int64_t)p->B * p->Hq * b200attn_padded_len(p->S);
  if (rows > kStaticMaxRows) return B200ATTN_ETOOLARGE;
  int rc = check_device(p->device);
  if (rc) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return B200ATTN_ECUDA;
  b200attn_params q = *p;
  if ((rc = static_scratch_for(p->device, &q.delta, &q.dsinks_partial))) return rc;
  return b200attn_bwd(&q);
}

int b200attn_umma_selftest(int mode, const void* a, const void* b, float* d, int32_t* status, int device, void* stream) {
  if (a == nullptr || b == nullptr || d == nullptr || (mode < 0 || mode > 2)) return B200ATTN_EINVAL;
  if (!aligned16(a) || !aligned16(b)) return B200ATTN_EALIGN;
  int rc = check_device(device);
  if (rc) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  CUtensorMap ta, tb;
  // modes 0, 2: A is (128 x 64), B is (128 x 64).  mode 1: A is read with plain loads, B is (128 x 64).
  b200attn_tensor tb_view{const_cast<void*>(b), 128 * 64, 128 * 64, 64};
  b200attn_tensor ta_view{const_cast<void*>(mode != 1 ? a : b), 128 * 64, 128 * 64, 64};
  if ((rc = make_map(&ta, ta_view, 1, 1, 128, kTile))) return rc;
  if ((rc = make_map(&tb, tb_view, 1, 1, 128, kTile))) return rc;
  const size_t smem = sizeof(SelftestSmem) + 1024;
  if ((rc = set_smem<umma_selftest_kernel>(smem))) return rc;
  umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(ta, tb, mode, static_cast<const __nv_bfloat16*>(a),
                                                                                       static_cast<const __nv_bfloat16*>(b), d, status, 0);
  return launch_status();
}

int b200attn_wait_selftest(int64_t wait_limit_cycles, int32_t* status, int device, void* stream) {
  if (status == nullptr || wait_limit_cycles <= 0 || wait_limit_cycles > 100000000ll) return B200ATTN_EINVAL;
  int rc = check_device(device);
  if (rc) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  CUtensorMap unused{};   // the waiting mode touches no tensor map
  const size_t smem = sizeof(SelftestSmem) + 1024;
  if ((rc = set_smem<umma_selftest_kernel>(smem))) return rc;
  umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(unused, unused, 3, nullptr, nullptr, nullptr, status,
                                                                            (long long)wait_limit_cycles);
  return launch_status();
}

int b200attn_rope(const b200attn_tensor* x, const b200attn_tensor* out, const void* cos_table, const void* sin_table,
                  int64_t table_stride_b, int64_t table_stride_s, int32_t B, int32_t H, int32_t S, int32_t inverse,
                  int32_t device, void* stream) {
  if (x == nullptr || out == nullptr || cos_table == nullptr || sin_table == nullptr || B <= 0 || H <= 0 || S <= 0) return B200ATTN_EINVAL;
  int rc;
  if ((rc = check_tensor(*x, B, H, S)) || (rc = check_tensor(*out, B, H, S))) return rc;
  if (!aligned16(cos_table) || !aligned16(sin_table) || table_stride_b % 8 || table_stride_s % 8 || table_stride_s < kHeadDim / 2)
    return B200ATTN_EALIGN;
  if ((rc = check_device(device))) return rc;
  DeviceGuard guard(device);
  if (!guard.ok) return B200ATTN_ECUDA;
  RopeArgs a{};
  a.x = strided(*x);
  a.out = strided(*out);
  a.cos = static_cast<const __nv_bfloat16*>(cos_table);
  a.sin = static_cast<const __nv_bfloat16*>(sin_table);
  a.cs_b = table_stride_b;
  a.cs_s = table_stride_s;
  a.B = B; a.H = H; a.S = S;
  a.sin_sign = inverse ? -1.f : 1.f;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const long long threads = (long long)B * H * S * 4;
  const long long want = (threads + 255) / 256, cap = (long long)sms * 16;
  rope_kernel<<<(int)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return launch_status();
}

}  // extern "C"
