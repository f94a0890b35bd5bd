/*
 * b200attn -- C ABI of the B200 (sm_100a) GPT-OSS attention forward/backward library.
 *
 * The reference project has no native interface: its device code is three Triton kernels
 * launched from Python (attention_kernel.py:244-262, :305-313, :316-339).  Each entry point
 * below stands in for one of those launch sites (or for the host code around it) and is
 * what a host-language binding for this path would bind.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless said otherwise.  The library allocates no
 *     device memory and keeps none after a call returns; all buffers belong to the caller
 *     (as in the reference, where they are torch tensors: attention_kernel.py:241-242,
 *     :295-298).
 *   - Calls only enqueue work on `stream` of `device`; they never synchronise.
 *   - Return value: 0 on success, a negative B200ATTN_E* code otherwise.  Nothing throws,
 *     exits or traps.  `status`, when not NULL, is a device int32 the kernels OR a non-zero
 *     code into if a bounded device-side wait gave up (it is never written on success); the
 *     caller zeroes it and reads it back after synchronising.
 *   - Tensors are bf16 4-D views (batch, head, position, head_dim) described by element
 *     strides; the head_dim stride must be 1, pointers 16-byte aligned and the other strides
 *     multiples of 8 elements -- the constraints the reference inherits from its TMA tensor
 *     descriptors (attention_kernel.py:245-251).  Any permutation of the outer three
 *     dimensions is therefore accepted: (B,H,S,d) as the attention module passes q/k/v, or
 *     (B,S,H,d) as it expects the output (attention_kernel.py:272).
 *   - Masking: key j is visible to query i of sequence b iff j <= i, j > i - window (when
 *     window > 0) and j < seqlens[b]; rows i >= seqlens[b] are padding (o = 0, no gradient).
 *     The reference ignores padding (attention_kernel.py:348-358); seqlens == NULL gives
 *     exactly its behaviour.  Padding rows of q, k, v and dO are still read (they share tiles
 *     with real rows) and enter the tensor-core products with a zero weight, so they must hold
 *     FINITE values: anything finite leaves every result bit-identical, Inf/NaN there do not.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_VERSION 1
#define B200ATTN_ROW_TILE 128 /* lse/delta rows are padded to a multiple of this */
#define B200ATTN_DELTA_PLANES 6 /* the delta scratch holds this many fp32-sized values per (b, h, padded row) */

enum {
  B200ATTN_OK = 0,
  B200ATTN_EINVAL = -1,      /* NULL params / pointer, non-positive size          */
  B200ATTN_ESHAPE = -2,      /* Hq % Hkv != 0, window < 0, S too large            */
  B200ATTN_EHEADDIM = -3,    /* head_dim other than 64                            */
  B200ATTN_EALIGN = -4,      /* pointer not 16-byte aligned / stride not % 8      */
  B200ATTN_EDEVICE = -5,     /* device is not compute capability 10.x             */
  B200ATTN_ECUDA = -6,       /* a CUDA runtime/driver call failed                 */
  B200ATTN_ETENSORMAP = -7,  /* the driver rejected a TMA tensor map              */
  B200ATTN_ESCRATCH = -8,    /* scratch buffer missing or too small               */
  B200ATTN_ETOOLARGE = -9    /* larger than b200attn_bwd_static_scratch can take  */
};

/* Bits of the `status` word.  Kernels only ever OR bits in.
 *   B200ATTN_STATUS_WAIT_TIMEOUT   a bounded device-side wait (on a TMA copy or a tensor-core
 *                                  completion) ran out; the CTA gave up, freed its tensor memory
 *                                  and returned, results of that call are undefined.
 *   B200ATTN_STATUS_NONPREFIX_MASK not set by the library itself: the Python binding ORs it in
 *                                  when a padding mask is not right-padded (a real token after a
 *                                  padding token), which `seqlens` cannot express. */
#define B200ATTN_STATUS_WAIT_TIMEOUT 1
#define B200ATTN_STATUS_NONPREFIX_MASK 2

/* Largest B * Hq * b200attn_padded_len(S) that b200attn_bwd_static_scratch accepts. */
#define B200ATTN_STATIC_MAX_ROWS (1 << 18)

/* bf16 tensor view (batch, head, position, head_dim); strides in ELEMENTS, head_dim stride 1 */
typedef struct b200attn_tensor {
  void* ptr;
  int64_t stride_b;
  int64_t stride_h;
  int64_t stride_s;
} b200attn_tensor;

typedef struct b200attn_params {
  /* problem size: q/o/dO/dq have Hq heads, k/v/dk/dv have Hkv heads, all have S positions */
  int32_t B, Hq, Hkv, S, d;
  int32_t window;          /* 0 = full causal, W > 0 = causal sliding window of W keys (incl. self) */
  float scale;             /* logits multiplier, 1/sqrt(d) for GPT-OSS */
  int32_t device;          /* CUDA device ordinal the pointers live on */
  void* stream;            /* cudaStream_t (0 = legacy default stream) */
  int32_t* status;         /* device int32, may be NULL */
  const int32_t* seqlens;  /* (B) valid lengths for right-padded batches, may be NULL */
  const float* sinks;      /* (Hq) fp32 per-head sink logits */

  b200attn_tensor q, k, v; /* inputs */
  b200attn_tensor o;       /* forward output; backward input */
  float* lse;              /* (B,Hq,S_pad) fp32, S_pad = b200attn_padded_len(S): natural-log
                              softmax denominator incl. the sink; forward output, backward input */

  /* backward only */
  b200attn_tensor d_o;        /* gradient of o */
  b200attn_tensor dq, dk, dv; /* outputs, fully overwritten (no pre-zeroing needed) */
  float* delta;               /* (B200ATTN_DELTA_PLANES,B,Hq,S_pad) fp32-sized scratch: [0] rowsum(dO*O),
                                 [1] -lse*log2(e) (the sink's probability per row where b200attn_bwd_dq_is_fused()),
                                 [2..5] MMA side operands of the dK/dV kernels (bf16) */
  float* dsinks;              /* (Hq) fp32 output, overwritten */
  float* dsinks_partial;      /* fp32 scratch of b200attn_dsinks_scratch_floats() elements */
} b200attn_params;

/* Library/ABI version (B200ATTN_VERSION the library was built with). */
int b200attn_version(void);

/* sizeof(b200attn_params) as the library was compiled, so that a binding written in another
 * language can verify its own mirror of the struct before the first call. */
size_t b200attn_sizeof_params(void);

/* Static description of a return code.  Never NULL. */
const char* b200attn_strerror(int code);

/* S rounded up to the row tile: the S_pad of lse/delta. */
int64_t b200attn_padded_len(int64_t S);

/* Number of floats `dsinks_partial` must hold for this problem. */
int64_t b200attn_dsinks_scratch_floats(const b200attn_params* p);

/*
 * Forward: o = softmax_with_sink(q k^T * scale + mask) v, lse.
 * Replaces the `_attn_fwd[grid](...)` launch and the pad / transpose copies around it
 * (attention_kernel.py:230-262, :272).  Reads q,k,v,sinks,seqlens; writes o, lse.
 */
int b200attn_fwd(const b200attn_params* p);

/*
 * Backward: dq, dk, dv, dsinks from q,k,v,o,lse,dO.  Enqueues the four stages below in the
 * order preprocess, dkdv, dq, dsinks.  Replaces attention_kernel.py:290-339 (dO transpose copy, zero-fills, the
 * `_attn_bwd_precompute_D` launch and the `_attn_bwd` launch).
 */
int b200attn_bwd(const b200attn_params* p);

/* Backward stages, exported separately so that each can be timed and tested alone.
 *
 * Layers with a sliding window of at most 128 keys (b200attn_bwd_dq_is_fused() == 1) have a shorter
 * backward: a query tile is seen by at most two key tiles there, so ONE kernel computes dK, dV and dQ
 * (S, dP and the exponentials once instead of twice) and adds its bf16 dQ tiles into global memory --
 * two terms per element, so the sum does not depend on their order and the result stays
 * bit-reproducible.  For such layers the preprocess stage also clears dq and writes the sink-gradient
 * partials (it needs dq and dsinks_partial), the dkdv stage runs that kernel (it needs dq, which must
 * still hold the zeros of the preprocess stage), and the dq stage returns at once. */
int b200attn_bwd_dq_is_fused(const b200attn_params* p);

/* delta[0] = rowsum(dO * O), delta[1] = -lse * log2(e), delta[2..5] = the same two per-row constants
 * as bf16 MMA operand tiles for the dK/dV kernel.  Replaces `_attn_bwd_precompute_D`
 * (attention_kernel.py:102-120).  Reads o, dO, lse; writes delta. */
int b200attn_bwd_preprocess(const b200attn_params* p);

/* dsinks[h] = sum of the partials the dq stage wrote (fixed order, warp-shuffle tree:
 * deterministic, unlike the reference's atomics at attention_kernel.py:176).  Must run after
 * b200attn_bwd_dq.  Reads dsinks_partial; writes dsinks. */
int b200attn_bwd_dsinks(const b200attn_params* p);

/* dk, dv: one CTA owns a 128-key tile of one KV head and loops over the query heads of the
 * group and the query tiles that see it; no atomics (the reference accumulates through
 * global atomics, attention_kernel.py:201-212).  Reads q,k,v,dO,lse,delta. */
int b200attn_bwd_dkdv(const b200attn_params* p);

/* dq: one CTA owns a 128-row query tile of one head (attention_kernel.py:214-217).  Also writes
 * the sink-gradient partials -sum_i exp(sink - lse_i) * sum_j P_ij dP_ij of its rows
 * (attention_kernel.py:173-175) to dsinks_partial (a fixed number per head and 128 positions, which depends
 * on the kernel variant the problem selects; b200attn_dsinks_scratch_floats covers every variant).  Reads q,k,v,dO,lse,delta,sinks. */
int b200attn_bwd_dq(const b200attn_params* p);

/*
 * Backward for callers that must not allocate.  This entry point has no counterpart in the
 * reference.  Some hosts of this library cannot call cudaMalloc at the moment they need a
 * backward pass: code running inside a memory-pool or arena that has already handed out all
 * device memory, real-time or signal-like contexts where an allocation's latency (or its
 * implicit synchronisation) is not acceptable, and bindings from runtimes that own the
 * allocator and do not let foreign code use it.  For them the two scratch buffers of
 * b200attn_bwd (`delta` and `dsinks_partial`, which are ignored here and may be NULL) live in
 * a fixed array inside the library's device image: about 6.4 MB that every GPU loading the
 * library holds until the process exits.  Inputs and outputs are still the caller's.
 *
 *   - Limit: B * Hq * b200attn_padded_len(S) <= B200ATTN_STATIC_MAX_ROWS (e.g. B=1, Hq=64,
 *     S=4096); anything larger returns B200ATTN_ETOOLARGE without launching.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress per array, with that device current, under a host mutex); make
 *     that first call outside any stream capture.  No call allocates or frees memory.
 *   - All calls on a device share the one array and it keeps the previous call's contents;
 *     every element that is read is overwritten first by the same call, so nothing needs
 *     clearing, but two calls whose kernels overlap on the GPU (different streams) race.
 *     Serialise them on one stream or with events.
 */
int b200attn_bwd_static_scratch(const b200attn_params* p);

/*
 * Rotary position embedding on a (batch, head, position, 64) view, one pass: out = rotate(x) with
 * the half-split rotation of the attention layer the reference patches (the `apply_rotary_pos_emb`
 * call in front of the patched function, transformers/models/gpt_oss/modeling_gpt_oss.py:226-242,
 * :318-319): out[..., :32] = x[..., :32] * cos - x[..., 32:] * sin, out[..., 32:] = x[..., 32:] * cos +
 * x[..., :32] * sin.  x and out may have any outer strides (the projection's (B,S,H,d) output is read
 * where it lies, the result lands in the layout b200attn_fwd takes in place) and may be the same
 * buffer.  cos_table / sin_table: bf16 (B, S, 32) with the given element strides (multiples of 8; a
 * batch stride of 0 shares one table).  inverse != 0 rotates the other way: the gradient of the
 * forward rotation, applied to dq / dk.
 */
int b200attn_rope(const b200attn_tensor* x, const b200attn_tensor* out, const void* cos_table, const void* sin_table,
                  int64_t table_stride_b, int64_t table_stride_s, int32_t B, int32_t H, int32_t S, int32_t inverse,
                  int32_t device, void* stream);

/*
 * Self-test of the tensor-core building blocks, used by the test-suite: D = A * B^T for one
 * 128 x N x K tile through TMA + tcgen05.  No counterpart in the reference.
 *   mode 0: A (128 x K) and B (N x K) both K-contiguous in shared memory, K = 64, N = 128
 *   mode 1: A from tensor memory (bf16), B given as (K x N) row-major, i.e. N-contiguous,
 *           K = 128, N = 64
 *   mode 2: mode 0 plus one more k-step, A[:, :16] * B[:, :16]^T, from unswizzled (rows x 16)
 *           side operands in shared memory
 * a, b: bf16 row-major matrices as described; d: fp32 (128 x N) row-major.
 */
int b200attn_umma_selftest(int mode, const void* a, const void* b, float* d, int32_t* status, int device,
                           void* stream);

/*
 * Self-test of the bounded waits, used by the test-suite.  No counterpart in the reference.
 * One CTA sets up as the attention kernels do (barriers, tensor memory), then every thread waits
 * on a barrier nothing arrives at, giving up after `wait_limit_cycles` SM cycles (1 ..
 * 100 000 000, i.e. at most ~50 ms): the kernel must OR B200ATTN_STATUS_WAIT_TIMEOUT into
 * *status, release its tensor memory and return normally.  Never leaves anything waiting.
 */
int b200attn_wait_selftest(int64_t wait_limit_cycles, int32_t* status, int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
