/*
 * b200moe -- C ABI of the B200 (sm_100a) GPT-OSS mixture-of-experts block: grouped GEMMs on the
 * tensor cores and the memory-bound steps around them.  Part of libb200attn.so.
 *
 * The reference project runs this block through Hugging Face's GptOssExperts.forward
 * (transformers/models/gpt_oss/modeling_gpt_oss.py:84-114), a Python loop over the experts that
 * gathers each expert's tokens, multiplies, applies the gated activation, multiplies again and
 * scatter-adds.  It has no native interface; each entry point below names the lines it replaces.
 *
 * Data layout.  The (token, choice) pairs are sorted by expert into one buffer of `rows` rows in
 * which every expert's segment starts at a multiple of 128 rows; rows between a segment's last
 * pair and the next multiple of 128 are padding and hold zeros.  `offsets` (DEVICE int32,
 * num_groups + 1 entries, multiples of 128, offsets[0] = 0) gives the segment bounds, so the host
 * never needs to know how many tokens an expert received.  All matrices are bf16, row-major, with
 * a column count that is a multiple of 8 and 16-byte aligned base pointers.
 *
 * Conventions as in b200attn.h: device pointers, no allocation, no synchronisation, calls only
 * enqueue work on `stream` of `device`; 0 on success or a negative B200ATTN_E* code
 * (b200attn_strerror explains it); `status`, when not NULL, is a device int32 into which a kernel
 * ORs B200ATTN_STATUS_WAIT_TIMEOUT if a bounded device-side wait gave up.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ROW_ALIGN 128 /* every group's segment starts at a multiple of this many rows */
#define B200MOE_MAX_GROUPS 256

enum {
  B200MOE_ROWS_NN = 0, /* D[r,:] = A[r,:] . B_g (+ bias_g);  B_g is (K x N), row-major              */
  B200MOE_ROWS_NT = 1, /* D[r,:] = A[r,:] . B_g^T;           B_g is (N x K), row-major              */
  B200MOE_INNER_TN = 2 /* D_g = A[rows of g,:]^T . B[rows of g,:];  A (rows x M), B (rows x N)       */
};

typedef struct b200moe_gemm_params {
  int32_t op;             /* one of B200MOE_ROWS_NN, B200MOE_ROWS_NT, B200MOE_INNER_TN                */
  int32_t num_groups;     /* experts                                                                   */
  int32_t rows;           /* rows of the sorted buffer (allocation size; only offsets[num_groups] used) */
  int32_t M, N, K;        /* ROWS_*: N columns of D, K inner (M ignored); INNER_TN: D_g is M x N (K ignored) */
  const int32_t* offsets; /* device, (num_groups + 1)                                                   */
  const void* a;          /* ROWS_*: (rows x K);  INNER_TN: (rows x M)                                  */
  const void* b;          /* ROWS_NN: (num_groups, K, N); ROWS_NT: (num_groups, N, K); INNER_TN: (rows x N) */
  const void* bias;       /* ROWS_* only: (num_groups, N) bf16 added to every row of the group, or NULL   */
  void* d;                /* ROWS_*: (rows x N);  INNER_TN: (num_groups, M, N), fully overwritten         */
  int32_t device;
  void* stream;           /* cudaStream_t */
  int32_t* status;        /* device int32, may be NULL */
  void* glu_out;          /* ROWS_NN only, or NULL: (rows x N/2) bf16 that receives b200moe_glu of D's rows from the
                             same launch (N a multiple of 16), so that the activation needs no pass of its own */
  int32_t max_ctas;       /* 0: one persistent CTA per SM.  > 0: at most this many, for callers that run another
                             kernel beside it (a collective's CTAs hold SMs, and a persistent CTA without an SM
                             waits for one to finish all of its tiles) */
} b200moe_gemm_params;

/* sizeof(b200moe_gemm_params) as compiled, for bindings that mirror the struct. */
size_t b200moe_sizeof_gemm_params(void);

/*
 * Grouped GEMM on tcgen05 (fp32 accumulation in tensor memory, bf16 in and out).
 *   ROWS_NN  replaces `current_state @ self.gate_up_proj[e] + self.gate_up_proj_bias[e]` and
 *            `gated_output @ self.down_proj[e] + self.down_proj_bias[e]` for all experts at once
 *            (modeling_gpt_oss.py:105, :107).
 *   ROWS_NT  the gradient of those products with respect to their left operand (dA = dD . W_e^T).
 *   INNER_TN the gradient with respect to the weights (dW_e = A_e^T . dD_e); an expert without
 *            rows gets zeros.
 * Rows of D that belong to no group (at or past offsets[num_groups]) are not written.
 */
int b200moe_grouped_gemm(const b200moe_gemm_params* p);

/*
 * Routing bookkeeping, one launch: sorts the tokens * top_k (token, choice) pairs by expert (stable: pairs of one
 * expert keep their order) into segments that start at multiples of B200MOE_ROW_ALIGN rows.  Replaces the
 * `one_hot` / `nonzero` / `torch.where` bookkeeping of GptOssExperts.forward (modeling_gpt_oss.py:86-103), which
 * synchronises with the host once per expert; nothing here does.
 *   indices     device int64 (tokens x top_k): the expert of each pair, 0 <= index < num_groups <= 256 (a pair with
 *               any other index belongs to no expert: it gets no row and pos = 0)
 *   weights     device fp32 (tokens x top_k): the routing weight of each pair
 *   rows        size of the sorted buffer: a multiple of 128, at least tokens*top_k + num_groups*127
 *   offsets     out, device int32 (num_groups + 1): segment bounds
 *   row_token   out, device int32 (rows): token of each sorted row, -1 for padding rows
 *   pos         out, device int32 (tokens x top_k): sorted row of each pair
 *   row_weight  out, device fp32 (rows): routing weight of each sorted row, 0 for padding rows
 */
int b200moe_route(const int64_t* indices, const float* weights, int32_t tokens, int32_t top_k, int32_t num_groups, int32_t rows,
                  int32_t* offsets, int32_t* row_token, int32_t* pos, float* row_weight, int32_t device, void* stream);

/*
 * out[r,:] = src[row_src[r],:] * (row_scale ? row_scale[r] : 1) for row_src[r] >= 0, zeros for
 * row_src[r] < 0 (padding rows).  Replaces `hidden_states[token_idx]` (modeling_gpt_oss.py:104);
 * with row_scale = the routing weight of each sorted row it is also the gradient of the weighted
 * scatter-add (:108-109) with respect to the expert outputs.  src: (n_src x cols), out: (rows x cols),
 * row_src: device int32 (rows), row_scale: device fp32 (rows) or NULL.
 */
int b200moe_gather_rows(const void* src, const int32_t* row_src, const float* row_scale, void* out, int32_t rows,
                        int32_t cols, int32_t device, void* stream);

/*
 * out[t,:] = sum_j (weights ? weights[t,j] : 1) * y[pos[t,j],:], j = 0 .. top_k-1 in that order, in
 * fp32.  Replaces `out * routing_weights[token_idx, top_k_pos, None]` and `next_states.index_add_`
 * (modeling_gpt_oss.py:108-109), whose bf16 atomics make the result depend on the order of arrival.
 * pos: device int32 (tokens x top_k) row of each (token, choice) in the sorted buffer; weights:
 * device fp32 (tokens x top_k) or NULL; y: (rows x cols); out: (tokens x cols).
 */
int b200moe_combine_rows(const void* y, const int32_t* pos, const float* weights, void* out, int32_t tokens,
                         int32_t top_k, int32_t cols, int32_t device, void* stream);

/*
 * dots[t,j] = <g[t,:], y[pos[t,j],:]> in fp32: the gradient of routing_weights[t,j] through
 * modeling_gpt_oss.py:108-109.  g: (tokens x cols), y: (rows x cols), dots: device fp32 (tokens x top_k).
 */
int b200moe_row_dot(const void* g, const void* y, const int32_t* pos, float* dots, int32_t tokens, int32_t top_k,
                    int32_t cols, int32_t device, void* stream);

/*
 * h[r,c] = (up + 1) * gate * sigmoid(1.702 * gate), gate = min(y1[r,2c], 7), up = clamp(y1[r,2c+1], -7, 7):
 * GptOssExperts._apply_gate (modeling_gpt_oss.py:76-82).  y1: (rows x 2*cols_h), h: (rows x cols_h).
 */
int b200moe_glu(const void* y1, void* h, int64_t rows, int32_t cols_h, int32_t device, void* stream);

/* dy1 from dh and y1: the derivative of b200moe_glu.  dh: (rows x cols_h); y1, dy1: (rows x 2*cols_h). */
int b200moe_glu_bwd(const void* y1, const void* dh, void* dy1, int64_t rows, int32_t cols_h, int32_t device,
                    void* stream);

/*
 * db[g,c] = sum of dy[r,c] over the rows r of group g, in fp32 in row order: the gradients of
 * gate_up_proj_bias and down_proj_bias (modeling_gpt_oss.py:105, :107).  dy: (rows x cols),
 * db: (num_groups x cols) bf16.
 */
int b200moe_bias_grad(const void* dy, const int32_t* offsets, void* db, int32_t num_groups, int32_t cols,
                      int32_t device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
