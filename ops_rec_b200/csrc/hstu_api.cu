// C ABI of the library (declared in include/hstu_b200.h): argument validation, workspace sizing, kernel choice.
//
// The checks restate what the reference enforces on its way to the kernel:
//   torch adapter  ascendc/attention/hstu_v1/torch_extension/hstu_jagged_plugin.cpp:29-51, hstu_common.h:68-82
//   host tiling    ascendc/attention/hstu_v1/hstu_forward_v1/op_host/tiling_policy.cpp:68-93,
//                  tiling_policy_jagged.cpp:103-203 (head ratio, equal k/v token and head counts, dims)
// with two documented relaxations (batch may exceed 2048; attn_bias may be broadcast over the batch).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/hstu_b200_testing.h"
#include "hstu_common.cuh"

namespace hstu {
cudaError_t launch_generic(const KParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_prepass(const KParams& p, bool build_items, cudaStream_t stream);
cudaError_t launch_bwd_prepass(const KParams& p, cudaStream_t stream);
long long plan_host(const KParams& p, uint32_t* items, long long capacity, uint32_t* status);
bool tc_supported(const KParams& p, int dtype);
cudaError_t launch_tc(const KParams& p, int dtype, int num_sms, cudaStream_t stream);
cudaError_t launch_bwd_generic(const BwdParams& bp, int dtype, cudaStream_t stream);
bool bwd_tc_supported(const BwdParams& bp, int dtype);
cudaError_t launch_bwd_tc(const BwdParams& bp, int dtype, int num_sms, cudaStream_t stream);
cudaError_t launch_ln_mul(const float* x, const float* u, const float* gamma, const float* beta, float* out,
                          long long rows, int cols, float eps, int num_sms, cudaStream_t stream);
cudaError_t launch_in_linear_silu(const LinSiluParams& p, const void* x, const void* weight, int dtype,
                                  cudaStream_t stream);
uint64_t in_linear_silu_bwd_workspace(long long m, int n, int k);
cudaError_t launch_in_linear_silu_bwd(const LinSiluParams& shape, const void* x, const void* weight,
                                      const void* const grads[4], const void* lo, void* x_grad, void* weight_grad,
                                      float* bias_grad, void* workspace, int dtype, uint32_t* status,
                                      cudaStream_t stream);
cudaError_t launch_paged_gather(const KParams& p, const void* kv_cache, const void* k_in, const void* v_in,
                                void* k_out, void* v_out, long long capacity, long long num_pages,
                                long long num_page_ids, int esize, cudaStream_t stream);
}  // namespace hstu

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

constexpr int kMaxSeqLen = 20480;  // hstu_common.h:36
constexpr int kMaxHeads = 16;      // hstu_common.h:40
constexpr int kMaxDim = 512;       // hstu_common.h:45

int validate(const HstuJaggedArgs* a) {
  if (!a) return fail(HSTU_E_NULL, "args is null");
  if (a->struct_bytes != sizeof(HstuJaggedArgs))
    return fail(HSTU_E_PARAM, "struct_bytes is %u, this library expects %zu", a->struct_bytes, sizeof(HstuJaggedArgs));
  if (a->dtype != HSTU_DTYPE_BF16 && a->dtype != HSTU_DTYPE_FP16 && a->dtype != HSTU_DTYPE_FP32)
    return fail(HSTU_E_PARAM, "dtype must be bf16, fp16 or fp32 (fp8 inputs are not supported)");
  if (a->batch < 1) return fail(HSTU_E_PARAM, "seq_offset params error should have at least two element.");
  if (a->index_bytes != 4 && a->index_bytes != 8) return fail(HSTU_E_PARAM, "seq_offset must be int32 or int64");
  if (a->total_q < 0 || a->total_k < 0) return fail(HSTU_E_PARAM, "negative token count");
  if (a->heads_q < 1 || a->heads_q > kMaxHeads || a->heads_k < 1)
    return fail(HSTU_E_PARAM, "head count expect in [1, %d], but value is %d", kMaxHeads, a->heads_q);
  if (a->heads_q % a->heads_k != 0)
    return fail(HSTU_E_PARAM, "head_num_q (%d) must be divisible by head_num_k (%d)", a->heads_q, a->heads_k);
  if (a->dim_qk < 1 || a->dim_qk > kMaxDim) return fail(HSTU_E_PARAM, "q/k head dim expect in [1, 512], but value is %d", a->dim_qk);
  if (a->dim_v < 16 || a->dim_v > kMaxDim || a->dim_v % 16 != 0)
    return fail(HSTU_E_PARAM, "v head dim expect a multiple of 16 in [16, 512], but value is %d", a->dim_v);
  if (a->mask_type < HSTU_MASK_TRIL || a->mask_type > HSTU_MASK_CUSTOM)
    return fail(HSTU_E_PARAM, "maskType expect in [0, 3], but value is %d", a->mask_type);
  if (a->mask_type == HSTU_MASK_TRIU)
    return fail(HSTU_E_PARAM, "maskType current not support triu now, pls use custome mask");
  if (a->mask_type == HSTU_MASK_CUSTOM && !a->mask)
    return fail(HSTU_E_PARAM, "use custome mask must have valide mask tensor");
  if (a->max_seq_len_q < 1 || a->max_seq_len_q > kMaxSeqLen)
    return fail(HSTU_E_PARAM, "maxSeqLen expect in [1, 20480], but value is %d", a->max_seq_len_q);
  if (a->max_seq_len_k < 1 || a->max_seq_len_k > kMaxSeqLen)
    return fail(HSTU_E_PARAM, "maxSeqLenK expect in [1, 20480], but value is %d", a->max_seq_len_k);
  if (a->target_group_size < 0) return fail(HSTU_E_PARAM, "target_group_size must be >= 0");
  if (a->bias_batch_stride < 0) return fail(HSTU_E_PARAM, "bias_batch_stride must be >= 0");
  if (!(a->silu_scale == a->silu_scale) || !(a->alpha == a->alpha)) return fail(HSTU_E_PARAM, "silu_scale / alpha is NaN");
  return HSTU_OK;
}

int validate_pointers(const HstuJaggedArgs* a) {
  if (!a->seq_offset_q) return fail(HSTU_E_NULL, "seq_offset is null");
  if (a->total_q > 0 && (!a->q || !a->out)) return fail(HSTU_E_NULL, "q / out is null");
  if (a->total_k > 0 && (!a->k || !a->v)) return fail(HSTU_E_NULL, "k / v is null");
  return HSTU_OK;
}

hstu::KParams to_params(const HstuJaggedArgs* a, void* workspace, uint64_t workspace_bytes) {
  hstu::KParams p;
  memset(&p, 0, sizeof(p));
  p.q = a->q;
  p.k = a->k;
  p.v = a->v;
  p.out = a->out;
  p.bias = a->attn_bias;
  p.mask = a->mask_type == HSTU_MASK_CUSTOM ? a->mask : nullptr;
  p.offq = a->seq_offset_q;
  p.offk = a->seq_offset_k ? a->seq_offset_k : a->seq_offset_q;
  p.ctx = a->num_context;
  p.tgt = a->num_target;
  p.total_q = a->total_q;
  p.total_k = a->total_k;
  p.bias_bstride = a->bias_batch_stride;
  p.index_bytes = a->index_bytes;
  p.batch = a->batch;
  p.hq = a->heads_q;
  p.hk = a->heads_k;
  p.dqk = a->dim_qk;
  p.dv = a->dim_v;
  p.gqa_ratio = a->heads_q / a->heads_k;
  p.mask_type = a->mask_type;
  p.maxq = a->max_seq_len_q;
  p.maxk = a->max_seq_len_k;
  p.group = a->target_group_size;
  p.scale = a->silu_scale == 0.0f ? 1.0f / static_cast<float>(a->max_seq_len_q) : a->silu_scale;
  p.alpha = a->alpha;
  p.flags = a->flags;
  p.fwd_by_steps = static_cast<long long>(a->heads_q) * (a->total_q / hstu::kPairM) < hstu::kFewItems ? 1 : 0;
  if (workspace) {
    p.ws_header = static_cast<uint32_t*>(workspace);
    p.items = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + hstu::kWsHeaderBytes);
    p.item_capacity = workspace_bytes > hstu::kWsHeaderBytes
                          ? static_cast<long long>((workspace_bytes - hstu::kWsHeaderBytes) / 8)
                          : 0;
  }
  return p;
}

// Upper bound of the work-list length that needs no device data: every sequence adds at most one partial pair.
long long item_bound(const HstuJaggedArgs* a) {
  return static_cast<long long>(a->heads_q) * (a->total_q / hstu::kPairM + a->batch);
}

bool wants_tc(const HstuJaggedArgs* a, const hstu::KParams& p) {
  return !(a->flags & HSTU_FLAG_FORCE_GENERIC) && hstu::tc_supported(p, a->dtype);
}

struct DeviceInfo {
  int major = -1, sms = 0;
};
int device_info(DeviceInfo* out) {
  static thread_local int cached_dev = -1;
  static thread_local DeviceInfo cached;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev != cached_dev) {
    DeviceInfo d;
    e = cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail(HSTU_E_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    cached = d;
    cached_dev = dev;
  }
  *out = cached;
  return HSTU_OK;
}

}  // namespace

extern "C" {

// for the other translation units of the library (not exported)
int hstu_set_last_error(int code, const char* text) { return fail(code, "%s", text); }

int hstu_b200_version(void) { return 101; }

const char* hstu_last_error(void) { return g_err; }

int hstu_jagged_fwd_get_workspace_size(const HstuJaggedArgs* args, uint64_t* workspace_bytes) {
  g_err[0] = 0;
  if (!workspace_bytes) return fail(HSTU_E_NULL, "workspace_bytes is null");
  int rc = validate(args);
  if (rc) return rc;
  const hstu::KParams p = to_params(args, nullptr, 0);
  uint64_t bytes = hstu::kWsHeaderBytes;
  if (wants_tc(args, p)) bytes += static_cast<uint64_t>(item_bound(args)) * 8;
  *workspace_bytes = (bytes + 255) & ~static_cast<uint64_t>(255);
  return HSTU_OK;
}

int hstu_jagged_fwd_kernel_kind(const HstuJaggedArgs* args) {
  g_err[0] = 0;
  int rc = validate(args);
  if (rc) return rc;
  const hstu::KParams p = to_params(args, nullptr, 0);
  return wants_tc(args, p) ? 1 : 0;
}

// `paged` (hstu_paged only): parameters that carry the page table, for the pre-pass's consistency check.
static int jagged_fwd_impl(const HstuJaggedArgs* args, void* workspace, uint64_t workspace_bytes, void* stream_v,
                           const hstu::KParams* paged);

int hstu_jagged_fwd(const HstuJaggedArgs* args, void* workspace, uint64_t workspace_bytes, void* stream_v) {
  g_err[0] = 0;
  return jagged_fwd_impl(args, workspace, workspace_bytes, stream_v, nullptr);
}

static int jagged_fwd_impl(const HstuJaggedArgs* args, void* workspace, uint64_t workspace_bytes, void* stream_v,
                           const hstu::KParams* paged) {
  int rc = validate(args);
  if (rc) return rc;
  rc = validate_pointers(args);
  if (rc) return rc;
  uint64_t need = 0;
  rc = hstu_jagged_fwd_get_workspace_size(args, &need);
  if (rc) return rc;
  if (!workspace) return fail(HSTU_E_WORKSPACE, "workspace is null (%llu bytes needed)", (unsigned long long)need);
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(HSTU_E_WORKSPACE, "workspace must be 256-byte aligned");
  if (workspace_bytes < need)
    return fail(HSTU_E_WORKSPACE, "workspace has %llu bytes, %llu needed", (unsigned long long)workspace_bytes,
                (unsigned long long)need);
  DeviceInfo dev;
  rc = device_info(&dev);
  if (rc) return rc;
  if (dev.major != 10) return fail(HSTU_E_ARCH, "this library is built for sm_100a only; device has compute capability %d.x", dev.major);

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  hstu::KParams p = to_params(args, workspace, need);
  if (paged) {
    p.page_offsets = paged->page_offsets;
    p.page_ids = paged->page_ids;
    p.last_page_len = paged->last_page_len;
    p.page_size = paged->page_size;
    p.num_pages = paged->num_pages;
    p.num_page_ids = paged->num_page_ids;
    p.kv_cache = paged->kv_cache;
    p.paged_direct = paged->paged_direct;
  }
  const bool tc = wants_tc(args, p);
  cudaError_t e = hstu::launch_prepass(p, tc, stream);
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "pre-pass launch: %s", cudaGetErrorString(e));
  if (args->total_q == 0) return HSTU_OK;
  if (tc) {
    e = hstu::launch_tc(p, args->dtype, dev.sms, stream);
    if (e == cudaErrorNotSupported) return fail(HSTU_E_CUDA, "cuTensorMapEncodeTiled failed or is unavailable");
  } else {
    e = hstu::launch_generic(p, args->dtype, stream);
  }
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return HSTU_OK;
}

// --------------------------------------------------------------------------------------------------- paged
namespace {
struct PagedPlan {
  HstuJaggedArgs fwd;        // the jagged call on the staging tensors
  uint64_t fwd_bytes;        // its workspace
  uint64_t stage_bytes;      // one staging tensor (256-byte multiple)
  long long capacity;        // rows of a staging tensor
  int esize;
};

int plan_paged(const HstuPagedArgs* a, PagedPlan* pl) {
  if (!a) return fail(HSTU_E_NULL, "args is null");
  if (a->struct_bytes != sizeof(HstuPagedArgs))
    return fail(HSTU_E_PARAM, "struct_bytes is %u, this library expects %zu", a->struct_bytes, sizeof(HstuPagedArgs));
  int rc = validate(&a->base);
  if (rc) return rc;
  if (a->base.dim_qk != a->base.dim_v)
    return fail(HSTU_E_PARAM, "hstu_paged: keys and values share the cache layout, dim_qk (%d) must equal dim_v (%d)",
                a->base.dim_qk, a->base.dim_v);
  if (a->page_size < 1) return fail(HSTU_E_PARAM, "hstu_paged: page_size must be positive, but value is %d", a->page_size);
  if (a->num_pages < 1 || a->num_page_ids < 1) return fail(HSTU_E_PARAM, "kv_cache / page_ids must not be empty");
  if (a->base.batch > 65535) return fail(HSTU_E_PARAM, "hstu_paged: batch expect in [1, 65535], but value is %d", a->base.batch);
  if (a->base.num_context) return fail(HSTU_E_PARAM, "hstu_paged takes no num_context");
  if (a->base.num_target && a->base.target_group_size <= 0)
    return fail(HSTU_E_PARAM, "targetGroupSize must be greater than 0 when numTarget is defined");
  const __int128 cap = static_cast<__int128>(a->num_page_ids) * a->page_size + a->base.total_q + hstu::kTileN;
  if (cap > 0x7fffff00ll) return fail(HSTU_E_PARAM, "hstu_paged: page table too large (%lld page slots of %d rows)",
                                      (long long)a->num_page_ids, a->page_size);
  pl->capacity = static_cast<long long>(cap);
  pl->esize = a->base.dtype == HSTU_DTYPE_FP32 ? 4 : 2;
  pl->stage_bytes = (static_cast<uint64_t>(pl->capacity) * a->base.heads_k * a->base.dim_qk * pl->esize + 255) &
                    ~static_cast<uint64_t>(255);
  pl->fwd = a->base;
  pl->fwd.total_k = pl->capacity;
  pl->fwd.num_context = nullptr;
  // k / v are filled in by the caller of this plan once the workspace is known; a 256-byte aligned stand-in keeps
  // the kernel choice (which looks at alignment) the same in both phases
  pl->fwd.k = pl->fwd.v = reinterpret_cast<const void*>(static_cast<uintptr_t>(256));
  if (!pl->fwd.out) pl->fwd.out = reinterpret_cast<void*>(static_cast<uintptr_t>(256));
  if (!pl->fwd.q) pl->fwd.q = reinterpret_cast<const void*>(static_cast<uintptr_t>(256));
  return hstu_jagged_fwd_get_workspace_size(&pl->fwd, &pl->fwd_bytes);
}
}  // namespace

int hstu_paged_fwd_get_workspace_size(const HstuPagedArgs* args, uint64_t* workspace_bytes) {
  g_err[0] = 0;
  if (!workspace_bytes) return fail(HSTU_E_NULL, "workspace_bytes is null");
  PagedPlan pl;
  int rc = plan_paged(args, &pl);
  if (rc) return rc;
  *workspace_bytes = pl.fwd_bytes + 2 * pl.stage_bytes;
  return HSTU_OK;
}

int hstu_paged_fwd(const HstuPagedArgs* args, void* workspace, uint64_t workspace_bytes, void* stream_v) {
  g_err[0] = 0;
  PagedPlan pl;
  int rc = plan_paged(args, &pl);
  if (rc) return rc;
  const HstuJaggedArgs* b = &args->base;
  if (!b->seq_offset_q || !b->seq_offset_k) return fail(HSTU_E_NULL, "seq_offset / seq_offset_k is null");
  if (!args->kv_cache || !args->page_offsets || !args->page_ids || !args->last_page_len)
    return fail(HSTU_E_NULL, "kv_cache / page_offsets / page_ids / last_page_len is null");
  if (b->total_q > 0 && (!b->q || !b->out || !b->k || !b->v)) return fail(HSTU_E_NULL, "q / k / v / out is null");
  const uint64_t need = pl.fwd_bytes + 2 * pl.stage_bytes;
  if (!workspace) return fail(HSTU_E_WORKSPACE, "workspace is null (%llu bytes needed)", (unsigned long long)need);
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(HSTU_E_WORKSPACE, "workspace must be 256-byte aligned");
  if (workspace_bytes < need)
    return fail(HSTU_E_WORKSPACE, "workspace has %llu bytes, %llu needed", (unsigned long long)workspace_bytes,
                (unsigned long long)need);
  char* base = static_cast<char*>(workspace);
  void* k_stage = base + pl.fwd_bytes;
  void* v_stage = base + pl.fwd_bytes + pl.stage_bytes;
  pl.fwd.q = b->q;
  pl.fwd.out = b->out;
  pl.fwd.k = k_stage;
  pl.fwd.v = v_stage;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  hstu::KParams p = to_params(&pl.fwd, nullptr, 0);
  p.page_offsets = args->page_offsets;
  p.page_ids = args->page_ids;
  p.last_page_len = args->last_page_len;
  p.page_size = args->page_size;
  p.num_pages = args->num_pages;
  p.num_page_ids = args->num_page_ids;
  p.kv_cache = args->kv_cache;
  // whole 128-row pages go from the cache straight into the tensor-core kernel's K / V ring
  p.paged_direct = (args->page_size == hstu::kTileN && args->num_pages <= 0x7fffffll && wants_tc(&pl.fwd, p)) ? 1 : 0;
  const cudaError_t e = hstu::launch_paged_gather(p, args->kv_cache, b->k, b->v, k_stage, v_stage, pl.capacity,
                                                  args->num_pages, args->num_page_ids, pl.esize, stream);
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "gather launch: %s", cudaGetErrorString(e));
  return jagged_fwd_impl(&pl.fwd, workspace, pl.fwd_bytes, stream_v, &p);
}

// ------------------------------------------------------------------------------------------------ backward
static int validate_bwd(const HstuJaggedBwdArgs* a) {
  if (!a) return fail(HSTU_E_NULL, "args is null");
  if (a->struct_bytes != sizeof(HstuJaggedBwdArgs))
    return fail(HSTU_E_PARAM, "struct_bytes is %u, this library expects %zu", a->struct_bytes,
                sizeof(HstuJaggedBwdArgs));
  int rc = validate(&a->fwd);
  if (rc) return rc;
  if (a->fwd.attn_bias && a->fwd.bias_batch_stride == 0 && a->fwd.batch > 1)
    return fail(HSTU_E_PARAM, "the backward needs a per-sequence attn_bias (a bias shared by the batch has no "
                              "per-sequence gradient slot)");
  // grad_bias is a contiguous [batch, heads_q, max_seq_len_q, max_seq_len_k] tensor and is addressed like the
  // bias: a padded batch stride would put the gradients of one and the zeros of the other in different places
  const long long block = static_cast<long long>(a->fwd.heads_q) * a->fwd.max_seq_len_q * a->fwd.max_seq_len_k;
  if (a->fwd.attn_bias && a->fwd.bias_batch_stride != 0 && a->fwd.bias_batch_stride != block)
    return fail(HSTU_E_PARAM, "the backward needs a contiguous attn_bias: bias_batch_stride must be heads_q * "
                              "max_seq_len_q * max_seq_len_k (%lld), but value is %lld", block,
                (long long)a->fwd.bias_batch_stride);
  return HSTU_OK;
}

// Upper bounds of the backward's two tile lists that need no device data: every sequence adds at most one partial
// tile per head; with a grad_bias the dQ pass visits every q-tile slot (rows past a sequence's end must be zeroed).
static void bwd_list_bounds(const HstuJaggedArgs* f, long long* cap_q, long long* cap_k) {
  const long long slots_q = static_cast<long long>(f->batch) * ((f->max_seq_len_q + hstu::kTileM - 1) / hstu::kTileM);
  *cap_q = static_cast<long long>(f->heads_q) * (f->attn_bias ? slots_q : f->total_q / hstu::kTileM + f->batch);
  *cap_k = static_cast<long long>(f->heads_k) * (f->total_k / hstu::kTileN + f->batch);
}
static uint64_t bwd_workspace_bytes(const HstuJaggedArgs* f) {
  long long cap_q, cap_k;
  bwd_list_bounds(f, &cap_q, &cap_k);
  return hstu::kWsHeaderBytes + 8ull * static_cast<uint64_t>(cap_q + cap_k);
}

int hstu_jagged_bwd_get_workspace_size(const HstuJaggedBwdArgs* args, uint64_t* workspace_bytes) {
  g_err[0] = 0;
  if (!workspace_bytes) return fail(HSTU_E_NULL, "workspace_bytes is null");
  int rc = validate_bwd(args);
  if (rc) return rc;
  *workspace_bytes = bwd_workspace_bytes(&args->fwd);  // status word, work counters and the two tile lists
  return HSTU_OK;
}

int hstu_jagged_bwd(const HstuJaggedBwdArgs* args, void* workspace, uint64_t workspace_bytes, void* stream_v) {
  g_err[0] = 0;
  int rc = validate_bwd(args);
  if (rc) return rc;
  const HstuJaggedArgs* f = &args->fwd;
  if (!f->seq_offset_q) return fail(HSTU_E_NULL, "seq_offset is null");
  if (f->total_q > 0 && (!f->q || !args->grad_out || !args->grad_q)) return fail(HSTU_E_NULL, "q / grad / grad_q is null");
  if (f->total_k > 0 && (!f->k || !f->v || !args->grad_k || !args->grad_v))
    return fail(HSTU_E_NULL, "k / v / grad_k / grad_v is null");
  if (f->attn_bias && !args->grad_bias) return fail(HSTU_E_NULL, "grad_bias is null but attn_bias is given");
  const uint64_t ws_need = bwd_workspace_bytes(f);
  if (!workspace) return fail(HSTU_E_WORKSPACE, "workspace is null (%llu bytes needed)", (unsigned long long)ws_need);
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(HSTU_E_WORKSPACE, "workspace must be 256-byte aligned");
  if (workspace_bytes < ws_need)
    return fail(HSTU_E_WORKSPACE, "workspace has %llu bytes, %llu needed", (unsigned long long)workspace_bytes,
                (unsigned long long)ws_need);
  DeviceInfo dev;
  rc = device_info(&dev);
  if (rc) return rc;
  if (dev.major != 10) return fail(HSTU_E_ARCH, "this library is built for sm_100a only; device has compute capability %d.x", dev.major);

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  hstu::BwdParams bp;
  bp.f = to_params(f, workspace, ws_need);
  bp.dout = args->grad_out;
  bp.dq = args->grad_q;
  bp.dk = args->grad_k;
  bp.dv = args->grad_v;
  bp.dbias = f->attn_bias ? args->grad_bias : nullptr;
  // input consistency -> status word; for the tensor-core kernels also their two tile lists
  const bool tc = hstu::bwd_tc_supported(bp, f->dtype);
  if (tc) {
    bwd_list_bounds(f, &bp.f.bwd_cap_q, &bp.f.bwd_cap_k);
    bp.f.bwd_all_q_tiles = bp.dbias ? 1 : 0;
    // few tiles per CTA: the lists are ordered by step count (longest first); many: sequence by sequence (L2 reuse)
    bp.f.bwd_by_steps = static_cast<long long>(f->heads_q) * (f->total_q / hstu::kTileM) < hstu::kFewItems ? 1 : 0;
  }
  cudaError_t e = tc ? hstu::launch_bwd_prepass(bp.f, stream) : hstu::launch_prepass(bp.f, false, stream);
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "pre-pass launch: %s", cudaGetErrorString(e));
  if (f->total_q == 0 && bp.dbias) {
    // no query rows: no kernel visits grad_bias, and every element of it is promised to be written
    const size_t esize = f->dtype == HSTU_DTYPE_FP32 ? 4 : 2;
    const size_t bytes = static_cast<size_t>(f->batch) * f->heads_q * f->max_seq_len_q * f->max_seq_len_k * esize;
    e = cudaMemsetAsync(bp.dbias, 0, bytes, stream);
    if (e != cudaSuccess) return fail(HSTU_E_CUDA, "clearing grad_bias: %s", cudaGetErrorString(e));
    bp.dbias = nullptr;
    bp.f.bias = nullptr;   // (nothing reads the bias either)
  }
  if (f->total_q == 0 && f->total_k == 0) return HSTU_OK;
  if (tc) {
    e = hstu::launch_bwd_tc(bp, f->dtype, dev.sms, stream);
    if (e == cudaErrorNotSupported) return fail(HSTU_E_CUDA, "cuTensorMapEncodeTiled failed or is unavailable");
  } else {
    e = hstu::launch_bwd_generic(bp, f->dtype, stream);
  }
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return HSTU_OK;
}

// ---------------------------------------------------------------------------------------- in_linear_silu
int ops_rec_in_linear_silu_fwd(const OpsRecInLinearSiluArgs* a, void* stream_v) {
  g_err[0] = 0;
  if (!a) return fail(HSTU_E_NULL, "args is null");
  if (a->struct_bytes != sizeof(OpsRecInLinearSiluArgs))
    return fail(HSTU_E_PARAM, "struct_bytes is %u, this library expects %zu", a->struct_bytes, sizeof(OpsRecInLinearSiluArgs));
  if (a->dtype != HSTU_DTYPE_BF16 && a->dtype != HSTU_DTYPE_FP16)
    return fail(HSTU_E_PARAM, "in_linear_silu: x and weight must be bf16 or fp16");
  long long total = 0;
  for (int i = 0; i < 4; ++i) {
    if (a->split[i] < 16 || a->split[i] > 8192 || a->split[i] % 16 != 0)
      return fail(HSTU_E_PARAM, "uvqk dim must in range[16, 8192] and multiples of 16.");
    total += a->split[i];
  }
  if (a->k < 16 || a->k > 8192 || a->k % 16 != 0)
    return fail(HSTU_E_PARAM, "x dim[1] must in range[16, 8192] and multiples of 16.");
  if (a->n < 64 || a->n > 32768 || a->n % 16 != 0)
    return fail(HSTU_E_PARAM, "weight dim[0] must in range[64, 32768] and multiples of 16.");
  if (total != a->n) return fail(HSTU_E_PARAM, "weight_dim[0] must equal to sum(splitList).");
  if (a->n % (4 * a->k) != 0) return fail(HSTU_E_PARAM, "weight dim[0] must be a multiple of 4 x dim[1]");
  if (a->m < 0 || a->m > 0x7fffff00ll) return fail(HSTU_E_PARAM, "in_linear_silu: bad row count");
  if (a->m == 0) return HSTU_OK;
  if (!a->x || !a->weight || !a->user || !a->value || !a->query || !a->key || !a->linear_output)
    return fail(HSTU_E_NULL, "in_linear_silu: null pointer");
  const uintptr_t align = reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->weight) |
                          reinterpret_cast<uintptr_t>(a->bias) | reinterpret_cast<uintptr_t>(a->user) |
                          reinterpret_cast<uintptr_t>(a->value) | reinterpret_cast<uintptr_t>(a->query) |
                          reinterpret_cast<uintptr_t>(a->key) | reinterpret_cast<uintptr_t>(a->linear_output);
  if (align & 15u) return fail(HSTU_E_PARAM, "in_linear_silu: every tensor must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(a->status) & 3u) return fail(HSTU_E_PARAM, "in_linear_silu: status must be 4-byte aligned");
  DeviceInfo dev;
  int rc = device_info(&dev);
  if (rc) return rc;
  if (dev.major != 10) return fail(HSTU_E_ARCH, "this library is built for sm_100a only; device has compute capability %d.x", dev.major);
  hstu::LinSiluParams p;
  memset(&p, 0, sizeof(p));
  p.bias = static_cast<const float*>(a->bias);
  p.out[0] = a->user, p.out[1] = a->value, p.out[2] = a->query, p.out[3] = a->key;
  p.linear = a->linear_output;
  int at = 0;
  for (int i = 0; i < 4; ++i) {
    p.width[i] = a->split[i];
    p.start[i] = at;
    at += a->split[i];
  }
  p.start[4] = at;
  p.m = a->m;
  p.n = a->n;
  p.k = a->k;
  p.status = static_cast<uint32_t*>(a->status);
  const cudaError_t e = hstu::launch_in_linear_silu(p, a->x, a->weight, a->dtype, static_cast<cudaStream_t>(stream_v));
  if (e == cudaErrorNotSupported) return fail(HSTU_E_CUDA, "cuTensorMapEncodeTiled failed or is unavailable");
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "in_linear_silu launch: %s", cudaGetErrorString(e));
  return HSTU_OK;
}

static int validate_linsilu_bwd(const OpsRecInLinearSiluBwdArgs* a) {
  if (!a) return fail(HSTU_E_NULL, "args is null");
  if (a->struct_bytes != sizeof(OpsRecInLinearSiluBwdArgs))
    return fail(HSTU_E_PARAM, "struct_bytes is %u, this library expects %zu", a->struct_bytes,
                sizeof(OpsRecInLinearSiluBwdArgs));
  if (a->dtype != HSTU_DTYPE_BF16 && a->dtype != HSTU_DTYPE_FP16)
    return fail(HSTU_E_PARAM, "in_linear_silu_backward: tensors must be bf16 or fp16");
  long long total = 0;
  for (int i = 0; i < 4; ++i) {
    if (a->split[i] < 16 || a->split[i] > 8192 || a->split[i] % 16 != 0)
      return fail(HSTU_E_PARAM, "uvqk dim must in range[16, 8192] and multiples of 16.");
    total += a->split[i];
  }
  if (a->k < 16 || a->k > 8192 || a->k % 16 != 0)
    return fail(HSTU_E_PARAM, "x dim[1] must in range[16, 8192] and multiples of 16.");
  if (a->n < 64 || a->n > 32768 || a->n % 16 != 0)
    return fail(HSTU_E_PARAM, "weight dim[0] must in range[64, 32768] and multiples of 16.");
  if (total != a->n) return fail(HSTU_E_PARAM, "weight_dim[0] must equal to sum(split_list).");
  if (a->n % (4 * a->k) != 0) return fail(HSTU_E_PARAM, "weight dim[0] must be a multiple of 4 x dim[1]");
  if (a->m < 0 || a->m > 4194240ll) return fail(HSTU_E_PARAM, "in_linear_silu_backward: row count expect in [0, 4194240]");
  return HSTU_OK;
}

int ops_rec_in_linear_silu_bwd_get_workspace_size(const OpsRecInLinearSiluBwdArgs* a, uint64_t* workspace_bytes) {
  g_err[0] = 0;
  if (!workspace_bytes) return fail(HSTU_E_NULL, "workspace_bytes is null");
  int rc = validate_linsilu_bwd(a);
  if (rc) return rc;
  *workspace_bytes = hstu::in_linear_silu_bwd_workspace(a->m, a->n, a->k) + 256;
  return HSTU_OK;
}

int ops_rec_in_linear_silu_bwd(const OpsRecInLinearSiluBwdArgs* a, void* workspace, uint64_t workspace_bytes,
                               void* stream_v) {
  g_err[0] = 0;
  int rc = validate_linsilu_bwd(a);
  if (rc) return rc;
  if (a->m == 0) return HSTU_OK;
  if (!a->x || !a->weight || !a->user_grad || !a->value_grad || !a->query_grad || !a->key_grad || !a->linear_output ||
      !a->x_grad || !a->weight_grad)
    return fail(HSTU_E_NULL, "in_linear_silu_backward: null pointer");
  const uintptr_t align = reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->weight) |
                          reinterpret_cast<uintptr_t>(a->user_grad) | reinterpret_cast<uintptr_t>(a->value_grad) |
                          reinterpret_cast<uintptr_t>(a->query_grad) | reinterpret_cast<uintptr_t>(a->key_grad) |
                          reinterpret_cast<uintptr_t>(a->linear_output) | reinterpret_cast<uintptr_t>(a->x_grad) |
                          reinterpret_cast<uintptr_t>(a->weight_grad);
  if (align & 15u) return fail(HSTU_E_PARAM, "in_linear_silu_backward: every tensor must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(a->bias_grad) | reinterpret_cast<uintptr_t>(a->status)) & 3u)
    return fail(HSTU_E_PARAM, "in_linear_silu_backward: bias_grad / status must be 4-byte aligned");
  const uint64_t need = hstu::in_linear_silu_bwd_workspace(a->m, a->n, a->k) + 256;
  if (!workspace) return fail(HSTU_E_WORKSPACE, "workspace is null (%llu bytes needed)", (unsigned long long)need);
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(HSTU_E_WORKSPACE, "workspace must be 256-byte aligned");
  if (workspace_bytes < need)
    return fail(HSTU_E_WORKSPACE, "workspace has %llu bytes, %llu needed", (unsigned long long)workspace_bytes,
                (unsigned long long)need);
  DeviceInfo dev;
  rc = device_info(&dev);
  if (rc) return rc;
  if (dev.major != 10) return fail(HSTU_E_ARCH, "this library is built for sm_100a only; device has compute capability %d.x", dev.major);
  hstu::LinSiluParams p;
  memset(&p, 0, sizeof(p));
  int at = 0;
  for (int i = 0; i < 4; ++i) {
    p.width[i] = a->split[i];
    p.start[i] = at;
    at += a->split[i];
  }
  p.start[4] = at;
  p.m = a->m;
  p.n = a->n;
  p.k = a->k;
  const void* grads[4] = {a->user_grad, a->value_grad, a->query_grad, a->key_grad};
  const cudaError_t e = hstu::launch_in_linear_silu_bwd(
      p, a->x, a->weight, grads, a->linear_output, a->x_grad, a->weight_grad, static_cast<float*>(a->bias_grad),
      workspace, a->dtype, static_cast<uint32_t*>(a->status), static_cast<cudaStream_t>(stream_v));
  if (e == cudaErrorNotSupported) return fail(HSTU_E_CUDA, "cuTensorMapEncodeTiled failed or is unavailable");
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "in_linear_silu_backward launch: %s", cudaGetErrorString(e));
  return HSTU_OK;
}

// ------------------------------------------------------------------------------------------------ ln_mul
int ops_rec_ln_mul_f32(const void* x, const void* u, const void* gamma, const void* beta, void* out, int64_t rows,
                       int64_t cols, void* stream_v) {
  g_err[0] = 0;
  if (rows < 0 || cols < 0 || cols > 0x7fffffffll) return fail(HSTU_E_PARAM, "ln_mul: bad shape [%lld, %lld]", (long long)rows, (long long)cols);
  if (rows > 0 && cols > 0 && (!x || !u || !gamma || !beta || !out)) return fail(HSTU_E_NULL, "ln_mul: null pointer");
  DeviceInfo dev;
  int rc = device_info(&dev);
  if (rc) return rc;
  if (dev.major != 10) return fail(HSTU_E_ARCH, "this library is built for sm_100a only; device has compute capability %d.x", dev.major);
  const cudaError_t e = hstu::launch_ln_mul(static_cast<const float*>(x), static_cast<const float*>(u),
                                            static_cast<const float*>(gamma), static_cast<const float*>(beta),
                                            static_cast<float*>(out), rows, static_cast<int>(cols), 1e-5f, dev.sms,
                                            static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "ln_mul launch: %s", cudaGetErrorString(e));
  return HSTU_OK;
}

int hstu_jagged_fwd_status(const void* workspace, void* stream_v, uint32_t* status) {
  g_err[0] = 0;
  if (!workspace || !status) return fail(HSTU_E_NULL, "workspace / status is null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(HSTU_E_CUDA, "reading the status word: %s", cudaGetErrorString(e));
  return HSTU_OK;
}

int64_t hstu_plan_host(const HstuJaggedArgs* args, const void* host_offset_q, const void* host_offset_k,
                       const void* host_num_context, const void* host_num_target, uint32_t* items, int64_t capacity,
                       uint32_t* status) {
  g_err[0] = 0;
  int rc = validate(args);
  if (rc) return rc;
  if (!host_offset_q) return fail(HSTU_E_NULL, "host_offset_q is null");
  hstu::KParams p = to_params(args, nullptr, 0);
  p.offq = host_offset_q;
  p.offk = host_offset_k ? host_offset_k : host_offset_q;
  p.ctx = host_num_context;
  p.tgt = host_num_target;
  return hstu::plan_host(p, items, items ? capacity : 0, status);
}

// Host evaluation of the device mask predicate and tile classifier (identical code, compiled for the host),
// so that the CUDA-side mask logic can be checked against the reference's create_causal_mask without a GPU.
int hstu_debug_mask_host(int32_t len_q, int32_t len_k, int32_t num_context, int32_t num_target,
                         int32_t target_group_size, int32_t mask_type, uint8_t* out) {
  if (!out || len_q < 0 || len_k < 0) return HSTU_E_PARAM;
  hstu::SeqInfo s;
  s.q0 = s.k0 = 0;
  s.lq = len_q;
  s.lk = len_k;
  s.ctx = num_context;
  s.tgt = num_target;
  for (int i = 0; i < len_q; ++i) {
    const hstu::RowBounds rb = hstu::row_bounds(s, i, mask_type, target_group_size);
    for (int j = 0; j < len_k; ++j) out[static_cast<size_t>(i) * len_k + j] = hstu::allowed(rb, j) ? 1 : 0;
  }
  return HSTU_OK;
}

// For the q-tile of rows [r0, r0 + rows): number of K tiles of width bn to visit, and (bit t of full_bits,
// t < 64) whether K tile t is classified "no predicate needed".
int hstu_debug_tiles_host(int32_t len_q, int32_t len_k, int32_t num_context, int32_t num_target,
                          int32_t target_group_size, int32_t mask_type, int32_t r0, int32_t rows, int32_t bn,
                          uint64_t* full_bits) {
  hstu::SeqInfo s;
  s.q0 = s.k0 = 0;
  s.lq = len_q;
  s.lk = len_k;
  s.ctx = num_context;
  s.tgt = num_target;
  const int n = hstu::kv_tiles_for_rows(s, r0, rows, mask_type, bn);
  uint64_t bits = 0;
  for (int t = 0; t < n && t < 64; ++t)
    if (hstu::tile_is_full(s, r0, rows, t * bn, bn, mask_type, target_group_size)) bits |= 1ull << t;
  if (full_bits) *full_bits = bits;
  return n;
}

}  // extern "C"
