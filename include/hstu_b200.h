/*
 * C ABI of the B200 (sm_100a) HSTU jagged attention forward.
 *
 *   O = ( silu(alpha * (Q.K^T + attn_bias)) * silu_scale * M ) . V      per sequence, per head
 *
 * over variable-length sequences packed along the token axis by seq_offset.  The functions below are what the
 * reference's torch adapter binds for this operator through its two-phase "aclnn" C interface:
 *
 *   aclnnHstuJaggedForwardGetWorkspaceSize / aclnnHstuJaggedForward
 *     contract:  ascendc/attention/hstu_v1/hstu_forward_v1/docs/aclnn_hstu_forward.md:47-62,107-112
 *     call site: ascendc/attention/hstu_v1/torch_extension/hstu_jagged_plugin.cpp:63-65
 *     macro:     ascendc/common/torch_plugin/pytorch_npu_helper.hpp:625-677 (phase 1 sizes the workspace, the
 *                caller allocates it, phase 2 enqueues the kernel on the caller's stream)
 *
 * Rules of the boundary
 *   - plain C, no exceptions: every function returns 0 on success or a negative HSTU_E* code; the text of the last
 *     error of the calling thread is available from hstu_last_error().
 *   - the caller owns every buffer, including the workspace; the library allocates no device memory.  (The only
 *     device memory the library holds is the fixed scratch block of hstu_jagged_fwd_static, below, which is part of
 *     the library image: HSTU_STATIC_SCRATCH_BYTES per GPU, from load until the process exits.)
 *   - hstu_jagged_fwd is asynchronous on `stream`; it never synchronises and never reads device data on the host.
 *     The sequence offsets are device data, so per-call scheduling happens in a small device pre-pass.
 *   - there is no CPU implementation behind these entry points.
 */
#ifndef HSTU_B200_H_
#define HSTU_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define HSTU_API __attribute__((visibility("default")))
#else
#define HSTU_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element type of q/k/v/out/attn_bias/mask */
enum { HSTU_DTYPE_BF16 = 0, HSTU_DTYPE_FP16 = 1, HSTU_DTYPE_FP32 = 2 };

/* mask_type values of the reference (ascendc/attention/hstu_v1/torch_extension/hstu_common.h:36-39);
 * 1 (upper-triangular) is rejected there and here. */
enum { HSTU_MASK_TRIL = 0, HSTU_MASK_TRIU = 1, HSTU_MASK_NONE = 2, HSTU_MASK_CUSTOM = 3 };

/* flags */
enum {
  HSTU_FLAG_DETERMINISTIC = 1u << 0, /* accepted for schema compatibility; results are always deterministic */
  HSTU_FLAG_ALPHA_BEFORE_BIAS = 1u << 1, /* silu(alpha*QK^T + bias) instead of the reference's silu(alpha*(QK^T + bias)) */
  HSTU_FLAG_FORCE_GENERIC = 1u << 2 /* use the generic fp32-accumulate CUDA-core kernel even where the tensor-core one applies */
};

/* error codes (the reference's aclnn layer reports 161001 for null pointers and 161002 for invalid
 * parameters, aclnn_hstu_forward.md:109-112; these are their counterparts) */
enum {
  HSTU_OK = 0,
  HSTU_E_NULL = -1,      /* required pointer is null */
  HSTU_E_PARAM = -2,     /* shape / dtype / range check failed */
  HSTU_E_WORKSPACE = -3, /* workspace missing, misaligned or too small */
  HSTU_E_CUDA = -4,      /* CUDA runtime or driver call failed */
  HSTU_E_ARCH = -5,      /* device is not sm_100 */
  HSTU_E_SCRATCH_LIMIT = -6 /* hstu_jagged_fwd_static: the call needs more scratch than the built-in block holds */
};

/* bits of the device status word written by the pre-pass (read it with hstu_jagged_fwd_status) */
enum {
  HSTU_ST_BAD_OFFSETS = 1u << 0,   /* offsets not monotone */
  HSTU_ST_LEN_GT_MAX = 1u << 1,    /* a sequence is longer than max_seq_len (bias/mask rows would be overrun) */
  HSTU_ST_BAD_CTX_TARGET = 1u << 2,/* num_context + num_target exceeds the sequence length, or negative */
  HSTU_ST_BAD_PAGES = 1u << 3,     /* hstu_paged: a page table that does not describe len_k - num_target cached rows,
                                      or a page id outside the cache */
  HSTU_ST_PIPE_TIMEOUT = 1u << 8   /* a bounded wait inside the tensor-core kernel gave up */
};

typedef struct HstuJaggedArgs {
  uint32_t struct_bytes; /* sizeof(HstuJaggedArgs), checked */
  int32_t dtype;         /* HSTU_DTYPE_* */

  /* device pointers; q [total_q, heads_q, dim_qk], k [total_k, heads_k, dim_qk], v [total_k, heads_k, dim_v],
   * out [total_q, heads_q, dim_v]; all contiguous (hstu_jagged_plugin.cpp:35-37 makes them so) */
  const void* q;
  const void* k;
  const void* v;
  void* out;
  /* optional [B, heads_q, max_seq_len_q, max_seq_len_k]; bias_batch_stride == 0 broadcasts one
   * [heads_q, max_seq_len_q, max_seq_len_k] block over the batch (extension of the reference) */
  const void* attn_bias;
  int64_t bias_batch_stride; /* in elements */
  /* required iff mask_type == HSTU_MASK_CUSTOM: [B, heads_q, max_seq_len_q, max_seq_len_k], values multiply P */
  const void* mask;

  /* [batch + 1] exclusive prefix sums on the device, int32 or int64 (index_bytes = 4 or 8);
   * seq_offset_k == NULL means "same as seq_offset_q" (the .equal overload) */
  const void* seq_offset_q;
  const void* seq_offset_k;
  /* optional [batch], same integer width as the offsets; NULL means all zero */
  const void* num_context;
  const void* num_target;
  int32_t index_bytes;

  int32_t batch;
  int64_t total_q;
  int64_t total_k;
  int32_t heads_q;
  int32_t heads_k;
  int32_t dim_qk;
  int32_t dim_v;

  int32_t mask_type;      /* HSTU_MASK_* */
  int32_t max_seq_len_q;  /* [1, 20480] */
  int32_t max_seq_len_k;
  int32_t target_group_size;
  float silu_scale;       /* 0 => 1 / max_seq_len_q (hstu_jagged_plugin.cpp:61) */
  float alpha;
  uint32_t flags;         /* HSTU_FLAG_* */
  uint32_t reserved;
} HstuJaggedArgs;

/* Phase 1 (replaces aclnnHstuJaggedForwardGetWorkspaceSize): validates the arguments that can be checked
 * without touching device memory and returns the number of workspace bytes phase 2 needs (never 0). */
HSTU_API int hstu_jagged_fwd_get_workspace_size(const HstuJaggedArgs* args, uint64_t* workspace_bytes);

/* Phase 2 (replaces aclnnHstuJaggedForward): enqueue the forward on `stream` (a cudaStream_t; NULL = default
 * stream) of the current device.  `workspace` is device memory, 256-byte aligned, at least the size phase 1
 * returned, and must stay alive until the work completes. */
HSTU_API int hstu_jagged_fwd(const HstuJaggedArgs* args, void* workspace, uint64_t workspace_bytes, void* stream);

/* Size of the scratch block built into the library for hstu_jagged_fwd_static (1 MiB per GPU that loads the
 * library, held until the process exits).  It covers heads_q * (total_q / 256 + batch) <= 131040 work items. */
#define HSTU_STATIC_SCRATCH_BYTES (1u << 20)

/* The forward without any allocation, for callers that cannot give it a workspace: processes that froze their
 * device-memory budget after start-up, plugins whose host forbids allocation inside the enqueue callback, code
 * that cannot tolerate the device-wide synchronisation of cudaMalloc / cudaFree.  Same arguments, same kernels and
 * bit-identical results as hstu_jagged_fwd; the scheduler's scratch lives in a fixed block inside the library.
 * This entry point has no counterpart in the reference (its adapter always allocates the workspace tensor,
 * ascendc/common/torch_plugin/pytorch_npu_helper.hpp:650-656).
 *   - It calls no cudaMalloc, cudaFree or other allocating routine.
 *   - A call whose work list does not fit returns HSTU_E_SCRATCH_LIMIT (use hstu_jagged_fwd with a workspace).
 *   - The first call on each device looks up the block's device address (cudaGetSymbolAddress, that device
 *     current); make that first call during start-up, before any stream capture begins.
 *   - All calls on a device share the one block, which keeps what the previous call left in it.  Each call's
 *     pre-pass re-initialises everything it reads, so calls that run one after another (same stream, or ordered by
 *     events) are safe; two calls that overlap on the GPU race on the block and give undefined results.
 *   - The looked-up address is cached for the life of the process; it does not survive cudaDeviceReset.
 *   - Every error, HSTU_E_SCRATCH_LIMIT included, leaves its text in hstu_last_error(). */
HSTU_API int hstu_jagged_fwd_static(const HstuJaggedArgs* args, void* stream);

/* The device status word (HSTU_ST_* bits) of the last hstu_jagged_fwd_static call on the current device: its caller
 * holds no workspace pointer that hstu_jagged_fwd_status could take.  Waits for `stream`, allocates nothing.  No
 * counterpart in the reference. */
HSTU_API int hstu_jagged_fwd_static_status(void* stream, uint32_t* status);

/* ------------------------------------------------------------------------------------------------------- paged
 * The forward with the history keys / values in a paged KV cache: replaces the aclnnHstuPagedForward call of the
 * reference adapter (ascendc/attention/hstu_v1/torch_extension/hstu_paged_plugin.cpp:21-72, the EXEC_NPU_CMD at
 * :67-69; kernel hstu_forward_v1/op_kernel/atlas950/hstu_paged_forward_kernel.h).  Per sequence b the operator attends
 * over  K/V = [pages page_ids[page_offsets[b] .. page_offsets[b+1]) of kv_cache, the last cut to last_page_len[b]]
 * followed by the last num_target[b] rows of the sequence's segment of base.k / base.v, with the composite mask of
 * the jagged operator (num_target targets, each seeing the cache and itself).
 *   base            the jagged arguments: q, out [total_q, heads_q, dim]; k, v [total_q, heads_k, dim] (only their
 *                   target rows are read); seq_offset_q; seq_offset_k (REQUIRED: offsets of cached rows + targets per
 *                   sequence); num_target; mask / attn_bias / mask_type / lengths / scales as in the jagged call;
 *                   dim_qk == dim_v; base.total_k is ignored; num_context must be null (the reference passes zeros)
 *   kv_cache        [num_pages, 2, page_size, heads_k, dim], element type of q; index 0 = keys, 1 = values
 *   page_offsets    [batch + 1], page_ids [num_page_ids], last_page_len [batch]: device integers of the offsets' width
 *   seq_offset_t    [batch + 1] offsets of num_target; implied by num_target and not read (may be null)
 * Workspace (phase 1 sizes it): the forward's work list plus two staging tensors of
 * (num_page_ids * page_size + total_q + 128) rows into which one gather pass packs the keys and values; the
 * attention itself is then the jagged forward in its delta form on the same kernels.  batch <= 65535. */
typedef struct HstuPagedArgs {
  uint32_t struct_bytes;  /* sizeof(HstuPagedArgs) */
  int32_t page_size;
  HstuJaggedArgs base;
  const void* kv_cache;
  const void* page_offsets;
  const void* page_ids;
  const void* last_page_len;
  const void* seq_offset_t;
  int64_t num_pages;
  int64_t num_page_ids;
} HstuPagedArgs;
HSTU_API int hstu_paged_fwd_get_workspace_size(const HstuPagedArgs* args, uint64_t* workspace_bytes);
HSTU_API int hstu_paged_fwd(const HstuPagedArgs* args, void* workspace, uint64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------------- backward
 * Replaces the aclnnHstuJaggedBackward call of the reference adapter
 * (ascendc/attention/hstu_v1/torch_extension/hstu_jagged_plugin.cpp:69-138, the EXEC_NPU_CMD at :126-128):
 * gradients of the forward above with respect to q, k, v and attn_bias.
 *   dV = P^T dO,  dS = (dO V^T) * scale * alpha * sg * (1 + x - x sg),  dQ = dS K,  dK = dS^T Q,  d_bias = dS
 * with x = alpha (S + bias), sg = sigmoid(x) * M (hstu_backward_v1/op_kernel/vector_score.h:159-209); with grouped
 * heads dK / dV sum over the query heads of a group.  `fwd` holds the arguments of the forward call (`fwd.out` is
 * not read and may be null).  grad_bias is required exactly when fwd.attn_bias is given; EVERY element of it is
 * written (zeros outside each sequence's visible region), so the caller need not clear it.  attn_bias must be
 * per-sequence here (bias_batch_stride != 0 unless batch == 1). */
typedef struct HstuJaggedBwdArgs {
  uint32_t struct_bytes;  /* sizeof(HstuJaggedBwdArgs) */
  uint32_t reserved;
  HstuJaggedArgs fwd;
  const void* grad_out;   /* [total_q, heads_q, dim_v], same dtype as q */
  void* grad_q;           /* [total_q, heads_q, dim_qk] */
  void* grad_k;           /* [total_k, heads_k, dim_qk] */
  void* grad_v;           /* [total_k, heads_k, dim_v] */
  void* grad_bias;        /* [batch, heads_q, max_seq_len_q, max_seq_len_k] or null */
} HstuJaggedBwdArgs;

/* Phase 1 / phase 2 of the backward, same contract as the forward pair (workspace: device memory, 256-byte
 * aligned, alive until the work completes; asynchronous on `stream`).  The workspace holds the status word, the work
 * counters and the tile lists of the two passes (8 bytes per 128-row tile and head). */
HSTU_API int hstu_jagged_bwd_get_workspace_size(const HstuJaggedBwdArgs* args, uint64_t* workspace_bytes);
HSTU_API int hstu_jagged_bwd(const HstuJaggedBwdArgs* args, void* workspace, uint64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------------ ln_mul
 * The step that consumes the attention output in an HSTU layer: out = (LayerNorm(x) * gamma + beta) * u over the
 * rows of fp32 [rows, cols] matrices, eps = 1e-5 (fixed by the reference's host code, ln_mul/op_host/ln_mul.cpp:73).
 * Replaces the aclnnLnMul call of ascendc/activation/ln_mul/torch_extension/ln_mul_plugin.cpp:51.  x, u, out:
 * contiguous [rows, cols]; gamma, beta: [cols]; all fp32 device pointers.  Asynchronous on `stream`; no workspace. */
HSTU_API int ops_rec_ln_mul_f32(const void* x, const void* u, const void* gamma, const void* beta, void* out,
                                int64_t rows, int64_t cols, void* stream);

/* ---------------------------------------------------------------------------------------------- in_linear_silu
 * The step that produces the attention's inputs in an HSTU layer (forward): mixed = x . weight^T + bias;
 * linear_output = mixed (rounded to the input type); (user, value, query, key) = split(silu(linear_output)) along
 * the last dimension.  Replaces the aclnnInLinearSilu call of
 * ascendc/activation/in_linear_silu/torch_extension/in_linear_silu_plugin.cpp:91-93; shape rules of :36-66
 * (k in [16, 8192] and n in [64, 32768] multiples of 16, n a multiple of 4 k, four split sizes in [16, 8192] multiples
 * of 16 that add up to n).  x [m, k], weight [n, k]: bf16 or fp16, contiguous, 16-byte aligned; bias [n] fp32 or null;
 * outputs in the input type, contiguous, 16-byte aligned.  Asynchronous on `stream`; no workspace. */
typedef struct OpsRecInLinearSiluArgs {
  uint32_t struct_bytes;  /* sizeof(OpsRecInLinearSiluArgs) */
  int32_t dtype;          /* HSTU_DTYPE_BF16 or HSTU_DTYPE_FP16 */
  const void* x;
  const void* weight;
  const void* bias;
  void* user;             /* [m, split[0]] */
  void* value;            /* [m, split[1]] */
  void* query;            /* [m, split[2]] */
  void* key;              /* [m, split[3]] */
  void* linear_output;    /* [m, n] */
  int64_t m;
  int32_t n;
  int32_t k;
  int32_t split[4];
  /* optional device uint32, or NULL: HSTU_ST_PIPE_TIMEOUT is or-ed into it if a bounded wait inside the kernel gives up
   * (the tile concerned is then not stored).  The caller clears it; the library only ever sets bits. */
  void* status;
} OpsRecInLinearSiluArgs;
HSTU_API int ops_rec_in_linear_silu_fwd(const OpsRecInLinearSiluArgs* args, void* stream);

/* Its backward: replaces the aclnnInLinearSiluBackward call of
 * ascendc/activation/in_linear_silu/torch_extension/in_linear_silu_backward_plugin.cpp:147-149.  With
 * g = cat(user_grad, value_grad, query_grad, key_grad) and lo = linear_output (saved by the forward):
 *   dL = g * sigmoid(lo) * (1 + lo * (1 - sigmoid(lo)));  bias_grad = column sums of dL (fp32);
 *   x_grad = round(dL) . weight;  weight_grad = round(dL)^T . x        (fp32 accumulation, results in the input type)
 * Same shape rules as the forward; the gradients and linear_output are [m, split[i]] / [m, n] in the input type,
 * contiguous, 16-byte aligned; bias_grad is fp32 [n] or NULL.  Two-phase like the attention calls: phase 1 sizes the
 * workspace (device memory, 256-byte aligned: dL, its transpose, weight^T, x^T and the partial column sums), phase 2
 * enqueues on `stream`.  m <= 4 194 240. */
typedef struct OpsRecInLinearSiluBwdArgs {
  uint32_t struct_bytes;  /* sizeof(OpsRecInLinearSiluBwdArgs) */
  int32_t dtype;          /* HSTU_DTYPE_BF16 or HSTU_DTYPE_FP16 */
  const void* x;          /* [m, k] */
  const void* weight;     /* [n, k] */
  const void* user_grad;
  const void* value_grad;
  const void* query_grad;
  const void* key_grad;
  const void* linear_output; /* [m, n] */
  void* x_grad;           /* [m, k] */
  void* weight_grad;      /* [n, k] */
  void* bias_grad;        /* [n] fp32, or NULL */
  int64_t m;
  int32_t n;
  int32_t k;
  int32_t split[4];
  void* status;           /* optional device uint32, as in the forward */
} OpsRecInLinearSiluBwdArgs;
HSTU_API int ops_rec_in_linear_silu_bwd_get_workspace_size(const OpsRecInLinearSiluBwdArgs* args,
                                                           uint64_t* workspace_bytes);
HSTU_API int ops_rec_in_linear_silu_bwd(const OpsRecInLinearSiluBwdArgs* args, void* workspace,
                                        uint64_t workspace_bytes, void* stream);

/* Optional: wait for `stream` and fetch the device status word of the last launch that used `workspace`
 * (0 = inputs were consistent).  The reference reads out of bounds on such inputs without noticing. */
HSTU_API int hstu_jagged_fwd_status(const void* workspace, void* stream, uint32_t* status);

/* Which kernel phase 2 would run for these arguments: 1 = tcgen05 tensor-core kernel, 0 = generic kernel,
 * negative = error code. */
HSTU_API int hstu_jagged_fwd_kernel_kind(const HstuJaggedArgs* args);

/* Host-side run of the scheduling pre-pass on HOST copies of the offsets (the same ordering rule the device
 * pre-pass applies), for tests and tooling.  Writes up to `capacity` work items, each {sequence, head << 16 | q_pair} as two
 * uint32, returns the item count (or a negative error code) and the status bits. */
HSTU_API int64_t hstu_plan_host(const HstuJaggedArgs* args, const void* host_offset_q, const void* host_offset_k,
                       const void* host_num_context, const void* host_num_target, uint32_t* items,
                       int64_t capacity, uint32_t* status);

/* Text of the last error raised on the calling thread ("" if none). */
HSTU_API const char* hstu_last_error(void);

/* Library version, e.g. 100 = 0.1.0 */
HSTU_API int hstu_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HSTU_B200_H_ */
