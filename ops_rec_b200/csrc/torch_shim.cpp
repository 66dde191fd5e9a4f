// torch operator registration for the HSTU jagged forward and backward, dispatching into the C ABI (include/hstu_b200.h).
//
// Schema strings, argument defaults and argument normalisation are those of the reference adapter
//   ascendc/attention/hstu_v1/torch_extension/hstu_jagged_plugin.cpp:22-67   (normalisation)
//   …/hstu_jagged_plugin.cpp:140-161                                         (equal / delta wrappers)
//   …/hstu_jagged_plugin.cpp:186-231                                         (schemas)
//   …/hstu_jagged_plugin.cpp:269-282                                         (Meta implementation)
// with the CUDA dispatch key in place of PrivateUse1.  As in the reference there is no C++ autograd key on
// the forward.  Differences, all documented for users: the output is not zero-filled first (no atomics are
// used, every row is written exactly once); batch may exceed 2048; attn_bias may be [H,S,S] or [1,H,S,S]
// (shared by all sequences); fp8 inputs are rejected.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include "hstu_b200.h"

namespace {

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kBFloat16: return HSTU_DTYPE_BF16;
    case at::kHalf: return HSTU_DTYPE_FP16;
    case at::kFloat: return HSTU_DTYPE_FP32;
    default: TORCH_CHECK(false, "hstu_jagged: dtype ", t, " is not supported (bf16, fp16, fp32)");
  }
}

// Every tensor whose address reaches a kernel must live on q's device: a CPU tensor, or one on another GPU, would be
// read through a raw pointer and fault on the device instead of failing here.
void check_same_device(const at::Tensor& t, const at::Tensor& q, const char* name) {
  TORCH_CHECK(t.device() == q.device(), "hstu_jagged: ", name, " is on ", t.device(), " but q is on ", q.device(),
              " (every tensor of a call must be on the same CUDA device)");
}

// The normalised arguments of one call: the C-ABI argument block plus the tensors that own what it points to.
struct Prepared {
  HstuJaggedArgs a;
  at::Tensor q, k, v, bias, cmask, ctx, tgt, off_q, off_k;
};

Prepared prepare(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                 const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias,
                 int64_t mask_type, int64_t max_seq_len_q, int64_t max_seq_len_k, double silu_scale,
                 const at::Tensor& seq_offset, const at::Tensor& seq_offset_k,
                 const c10::optional<at::Tensor>& num_context, const c10::optional<at::Tensor>& num_target,
                 const c10::optional<int64_t>& target_group_size, const c10::optional<double>& alpha,
                 bool deterministic) {
  TORCH_CHECK(q.dim() == 3, "The q should be 3D in jagged layout");
  TORCH_CHECK(k.dim() == 3 && v.dim() == 3, "The k and v should be 3D in jagged layout");
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda() && seq_offset.is_cuda(),
              "hstu_jagged: tensors must be CUDA tensors (there is no CPU implementation)");
  check_same_device(k, q, "k");
  check_same_device(v, q, "v");
  check_same_device(seq_offset, q, "seq_offset");
  check_same_device(seq_offset_k, q, "seq_offset_k");
  if (attn_bias.has_value() && attn_bias->defined()) check_same_device(*attn_bias, q, "attn_bias");
  if (mask.has_value() && mask->defined()) check_same_device(*mask, q, "mask");
  TORCH_CHECK(seq_offset.scalar_type() == at::kInt || seq_offset.scalar_type() == at::kLong,
              "seq_offset must be int32 or int64");
  Prepared pr;
  at::Tensor& off_q = pr.off_q;
  at::Tensor& off_k = pr.off_k;
  off_q = seq_offset.contiguous();
  off_k = seq_offset_k.to(off_q.scalar_type()).contiguous();
  TORCH_CHECK(off_q.size(0) >= 2, "acSeqOffset params error should have at least two element.");
  TORCH_CHECK(off_k.size(0) >= 2, "acSeqOffsetK params error should have at least two element.");
  TORCH_CHECK(off_k.size(0) == off_q.size(0), "seq_offset and seq_offset_k must have the same length");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(),
              "q, k and v must have the same dtype");
  TORCH_CHECK(k.size(0) == v.size(0) && k.size(1) == v.size(1), "k and v must agree in tokens and heads");
  TORCH_CHECK(k.size(2) == q.size(2), "q and k must have the same head dim");

  at::Tensor &dq = pr.q, &dk = pr.k, &dv = pr.v;
  dq = q.contiguous();
  dk = k.contiguous();
  dv = v.contiguous();
  const int64_t batch = off_q.size(0) - 1;

  HstuJaggedArgs& a = pr.a;
  memset(&a, 0, sizeof(a));
  a.struct_bytes = sizeof(a);
  a.dtype = dtype_code(q.scalar_type());
  a.q = dq.data_ptr();
  a.k = dk.data_ptr();
  a.v = dv.data_ptr();

  at::Tensor &bias = pr.bias, &cmask = pr.cmask, &ctx = pr.ctx, &tgt = pr.tgt;
  if (attn_bias.has_value() && attn_bias->defined()) {
    bias = attn_bias->to(q.scalar_type()).contiguous();
    TORCH_CHECK(bias.dim() == 4 || bias.dim() == 3, "attn_bias must be [B,H,Sq,Sk] (or [H,Sq,Sk] shared by the batch)");
    TORCH_CHECK(bias.size(-1) == max_seq_len_k && bias.size(-2) == max_seq_len_q && bias.size(-3) == q.size(1),
                "attn_bias must be [.., heads_q, max_seq_len, max_seq_len_k]");
    const bool shared = bias.dim() == 3 || bias.size(0) == 1;
    TORCH_CHECK(shared || bias.size(0) >= batch, "attn_bias batch dimension is smaller than the batch");
    a.attn_bias = bias.data_ptr();
    a.bias_batch_stride = shared ? 0 : bias.size(1) * bias.size(2) * bias.size(3);
  }
  if (mask.has_value() && mask->defined() && mask_type == HSTU_MASK_CUSTOM) {
    cmask = mask->to(q.scalar_type()).contiguous();
    TORCH_CHECK(cmask.dim() == 4 && cmask.size(0) >= batch && cmask.size(1) == q.size(1) &&
                    cmask.size(2) == max_seq_len_q && cmask.size(3) == max_seq_len_k,
                "mask must be [B, heads_q, max_seq_len, max_seq_len_k]");
    a.mask = cmask.data_ptr();
  }
  a.seq_offset_q = off_q.data_ptr();
  a.seq_offset_k = off_k.data_ptr();
  a.index_bytes = static_cast<int32_t>(off_q.element_size());
  if (num_context.has_value() && num_context->defined()) {
    ctx = num_context->to(off_q.device(), off_q.scalar_type()).contiguous();
    TORCH_CHECK(ctx.numel() >= batch, "num_context is shorter than the batch");
    a.num_context = ctx.data_ptr();
  }
  if (num_target.has_value() && num_target->defined()) {
    tgt = num_target->to(off_q.device(), off_q.scalar_type()).contiguous();
    TORCH_CHECK(tgt.numel() >= batch, "num_target is shorter than the batch");
    a.num_target = tgt.data_ptr();
  }
  a.batch = static_cast<int32_t>(batch);
  a.total_q = dq.size(0);
  a.total_k = dk.size(0);
  a.heads_q = static_cast<int32_t>(dq.size(1));
  a.heads_k = static_cast<int32_t>(dk.size(1));
  a.dim_qk = static_cast<int32_t>(dq.size(2));
  a.dim_v = static_cast<int32_t>(dv.size(2));
  a.mask_type = static_cast<int32_t>(mask_type);
  // range checks with the reference's messages happen inside the C ABI; keep int32 conversion safe here
  TORCH_CHECK(max_seq_len_q >= 1 && max_seq_len_q <= 20480, "maxSeqLen expect in [1, 20480], but value is ", max_seq_len_q);
  TORCH_CHECK(max_seq_len_k >= 1 && max_seq_len_k <= 20480, "maxSeqLenK expect in [1, 20480], but value is ", max_seq_len_k);
  a.max_seq_len_q = static_cast<int32_t>(max_seq_len_q);
  a.max_seq_len_k = static_cast<int32_t>(max_seq_len_k);
  a.target_group_size = static_cast<int32_t>(target_group_size.value_or(0));
  a.silu_scale = static_cast<float>(silu_scale);
  a.alpha = static_cast<float>(alpha.value_or(1.0));
  a.flags = deterministic ? HSTU_FLAG_DETERMINISTIC : 0u;
  if (mask_type == HSTU_MASK_CUSTOM && !a.mask) {
    // let the C ABI produce the reference's message
    a.mask = nullptr;
  }

  return pr;
}

at::Tensor forward_impl(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                        const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias,
                        int64_t mask_type, int64_t max_seq_len_q, int64_t max_seq_len_k, double silu_scale,
                        const at::Tensor& seq_offset, const at::Tensor& seq_offset_k,
                        const c10::optional<at::Tensor>& num_context, const c10::optional<at::Tensor>& num_target,
                        const c10::optional<int64_t>& target_group_size, const c10::optional<double>& alpha,
                        bool deterministic) {
  c10::cuda::CUDAGuard guard(q.device());
  Prepared pr = prepare(q, k, v, mask, attn_bias, mask_type, max_seq_len_q, max_seq_len_k, silu_scale, seq_offset,
                        seq_offset_k, num_context, num_target, target_group_size, alpha, deterministic);
  HstuJaggedArgs& a = pr.a;
  const at::Tensor& dq = pr.q;
  auto out = at::empty({pr.q.size(0), pr.q.size(1), pr.v.size(2)}, pr.q.options());
  a.out = out.data_ptr();

  uint64_t ws_bytes = 0;
  int rc = hstu_jagged_fwd_get_workspace_size(&a, &ws_bytes);
  TORCH_CHECK(rc == 0, "hstu_jagged: ", hstu_last_error());
  auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, dq.options().dtype(at::kByte));
  rc = hstu_jagged_fwd(&a, ws.data_ptr(), ws_bytes, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "hstu_jagged: ", hstu_last_error());
  return out;
}

at::Tensor hstu_jagged_equal(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                             const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias,
                             int64_t mask_type, int64_t max_seq_len, double silu_scale, const at::Tensor& seq_offset,
                             const c10::optional<at::Tensor>& num_context, const c10::optional<at::Tensor>& num_target,
                             c10::optional<int64_t> target_group_size, c10::optional<double> alpha, bool deterministic) {
  return forward_impl(q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len, silu_scale, seq_offset, seq_offset,
                      num_context, num_target, target_group_size, alpha, deterministic);
}

at::Tensor hstu_jagged_delta(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                             const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias,
                             int64_t mask_type, int64_t max_seq_len, int64_t max_seq_len_k, double silu_scale,
                             const at::Tensor& seq_offset, const at::Tensor& seq_offset_k,
                             const c10::optional<at::Tensor>& num_context, const c10::optional<at::Tensor>& num_target,
                             c10::optional<int64_t> target_group_size, c10::optional<double> alpha, bool deterministic) {
  return forward_impl(q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len_k, silu_scale, seq_offset,
                      seq_offset_k, num_context, num_target, target_group_size, alpha, deterministic);
}

// Backward: (dq, dk, dv, d_bias) through hstu_jagged_bwd.  Argument checks of the reference adapter
// (hstu_jagged_plugin.cpp:77-95); the fourth result is an undefined tensor without attn_bias, as there (:131-137).
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> backward_impl(
    const at::Tensor& grad, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
    const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias, int64_t mask_type,
    int64_t max_seq_len_q, int64_t max_seq_len_k, double silu_scale, const at::Tensor& seq_offset,
    const at::Tensor& seq_offset_k, const c10::optional<at::Tensor>& num_context,
    const c10::optional<at::Tensor>& num_target, const c10::optional<int64_t>& target_group_size,
    const c10::optional<double>& alpha) {
  const bool has_ctx = num_context.has_value() && num_context->defined();
  const bool has_tgt = num_target.has_value() && num_target->defined();
  if (has_ctx || has_tgt) {
    TORCH_CHECK(has_ctx, "numContext is required when numTarget or targetGroupSize is not None");
    TORCH_CHECK(has_tgt, "numTarget is required when numContext or targetGroupSize is not None");
    TORCH_CHECK(num_context->dim() == 1, "The numContext should be 1D in normal layout");
    TORCH_CHECK(num_target->dim() == 1, "The numTarget should be 1D in normal layout");
  }
  TORCH_CHECK(grad.dim() == 3 && grad.is_cuda() && grad.scalar_type() == q.scalar_type(),
              "grad must be a 3D CUDA tensor of q's dtype");
  check_same_device(grad, q, "grad");
  c10::cuda::CUDAGuard guard(q.device());
  Prepared pr = prepare(q, k, v, mask, attn_bias, mask_type, max_seq_len_q, max_seq_len_k, silu_scale, seq_offset,
                        seq_offset_k, num_context, num_target, target_group_size, alpha, false);
  TORCH_CHECK(grad.size(0) == pr.q.size(0) && grad.size(1) == pr.q.size(1) && grad.size(2) == pr.v.size(2),
              "grad must be [total_q, heads_q, dim_v]");
  auto g = grad.contiguous();
  HstuJaggedBwdArgs b;
  memset(&b, 0, sizeof(b));
  b.struct_bytes = sizeof(b);
  b.fwd = pr.a;
  auto gq = at::empty_like(pr.q), gk = at::empty_like(pr.k), gv = at::empty_like(pr.v);
  at::Tensor gbias;
  if (pr.bias.defined()) {
    TORCH_CHECK(pr.bias.dim() == 4, "the backward needs attn_bias as [B, heads_q, max_seq_len, max_seq_len_k]");
    // the kernels write every element of the first `batch` blocks; a bias with spare blocks gets them zeroed
    gbias = pr.bias.size(0) == pr.a.batch ? at::empty_like(pr.bias) : at::zeros_like(pr.bias);
    b.grad_bias = gbias.data_ptr();
  }
  b.grad_out = g.data_ptr();
  b.grad_q = gq.data_ptr();
  b.grad_k = gk.data_ptr();
  b.grad_v = gv.data_ptr();
  uint64_t ws_bytes = 0;
  int rc = hstu_jagged_bwd_get_workspace_size(&b, &ws_bytes);
  TORCH_CHECK(rc == 0, "hstu_jagged_backward: ", hstu_last_error());
  auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, pr.q.options().dtype(at::kByte));
  rc = hstu_jagged_bwd(&b, ws.data_ptr(), ws_bytes, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "hstu_jagged_backward: ", hstu_last_error());
  return std::make_tuple(gq, gk, gv, gbias);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> hstu_jagged_backward_equal(
    const at::Tensor& grad, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
    const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias, int64_t mask_type,
    int64_t max_seq_len, double silu_scale, const at::Tensor& seq_offset,
    const c10::optional<at::Tensor>& num_context, const c10::optional<at::Tensor>& num_target,
    c10::optional<int64_t> target_group_size, c10::optional<double> alpha) {
  return backward_impl(grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len, silu_scale, seq_offset,
                       seq_offset, num_context, num_target, target_group_size, alpha);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> hstu_jagged_backward_delta(
    const at::Tensor& grad, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
    const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias, int64_t mask_type,
    int64_t max_seq_len, int64_t max_seq_len_k, double silu_scale, const at::Tensor& seq_offset,
    const at::Tensor& seq_offset_k, const c10::optional<at::Tensor>& num_context,
    const c10::optional<at::Tensor>& num_target, c10::optional<int64_t> target_group_size,
    c10::optional<double> alpha) {
  return backward_impl(grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len_k, silu_scale, seq_offset,
                       seq_offset_k, num_context, num_target, target_group_size, alpha);
}

// Meta: gradients shaped like their inputs (hstu_jagged_plugin.cpp:284-310)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> backward_meta_out(
    const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& attn_bias) {
  auto m = [](const at::Tensor& t) { return at::empty_like(t, t.options().device(c10::kMeta)); };
  at::Tensor gb;
  if (attn_bias.has_value() && attn_bias->defined()) gb = m(*attn_bias);
  return std::make_tuple(m(q), m(k), m(v), gb);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> hstu_jagged_backward_equal_meta(
    const at::Tensor&, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
    const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>& attn_bias, int64_t, int64_t, double,
    const at::Tensor&, const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, c10::optional<int64_t>,
    c10::optional<double>) {
  return backward_meta_out(q, k, v, attn_bias);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> hstu_jagged_backward_delta_meta(
    const at::Tensor&, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
    const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>& attn_bias, int64_t, int64_t, int64_t, double,
    const at::Tensor&, const at::Tensor&, const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
    c10::optional<int64_t>, c10::optional<double>) {
  return backward_meta_out(q, k, v, attn_bias);
}

// ln_mul (ascendc/activation/ln_mul/torch_extension/ln_mul_plugin.cpp:28-55): same checks and messages, fp32 only.
at::Tensor ln_mul(const at::Tensor& x, const at::Tensor& u, const at::Tensor& gamma, const at::Tensor& beta) {
  for (const auto* t : {&x, &u, &gamma, &beta}) TORCH_CHECK(t->defined() && t->numel() > 0, "ln_mul: input tensor is empty");
  TORCH_CHECK(x.is_cuda() && u.is_cuda() && gamma.is_cuda() && beta.is_cuda() && u.device() == x.device() &&
                  gamma.device() == x.device() && beta.device() == x.device(),
              "ln_mul: all tensors must be on the same CUDA device");
  TORCH_CHECK(x.dim() == 2, "The x should be 2D");
  TORCH_CHECK(u.dim() == 2, "The u should be 2D");
  TORCH_CHECK(gamma.dim() == 1, "The gamma should be 1D");
  TORCH_CHECK(beta.dim() == 1, "The beta should be 1D");
  TORCH_CHECK(x.sizes() == u.sizes(), "x and u must have identical shape");
  TORCH_CHECK(gamma.size(0) == x.size(1) && beta.size(0) == x.size(1), "gamma and beta must have x.size(1) elements");
  TORCH_CHECK(x.scalar_type() == at::kFloat && u.scalar_type() == at::kFloat && gamma.scalar_type() == at::kFloat &&
                  beta.scalar_type() == at::kFloat,
              "ln_mul supports float32 only");
  c10::cuda::CUDAGuard guard(x.device());
  auto xc = x.contiguous(), uc = u.contiguous(), gc = gamma.contiguous(), bc = beta.contiguous();
  auto y = at::empty_like(xc);
  const int rc = ops_rec_ln_mul_f32(xc.data_ptr(), uc.data_ptr(), gc.data_ptr(), bc.data_ptr(), y.data_ptr(), xc.size(0),
                                    xc.size(1), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ln_mul: ", hstu_last_error());
  return y;
}

at::Tensor ln_mul_meta(const at::Tensor& x, const at::Tensor& u, const at::Tensor& gamma, const at::Tensor& beta) {
  TORCH_CHECK(x.dim() == 2, "x must be 2D");
  TORCH_CHECK(u.dim() == 2, "u must be 2D");
  TORCH_CHECK(gamma.dim() == 1, "gamma must be 1D");
  TORCH_CHECK(beta.dim() == 1, "beta must be 1D");
  TORCH_CHECK(x.sizes() == u.sizes(), "x and u must share the same shape");
  return at::empty_like(x, x.options());
}

// distance_in_linear_silu (in_linear_silu/torch_extension/in_linear_silu_plugin.cpp:36-98): forward only.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> in_linear_silu_fwd(
    const at::Tensor& x, const at::Tensor& weight, const at::Tensor& bias, at::IntArrayRef split) {
  TORCH_CHECK(x.defined() && x.numel() > 0, "x is empty");
  TORCH_CHECK(weight.defined() && weight.numel() > 0, "weight is empty");
  TORCH_CHECK(x.dim() == 2, "x must be 2D");
  TORCH_CHECK(weight.dim() == 2, "weight must be 2D");
  TORCH_CHECK(split.size() == 4, "splitList must have 4 elements.");
  TORCH_CHECK(x.is_cuda() && weight.is_cuda(), "in_linear_silu: tensors must be CUDA tensors");
  TORCH_CHECK(weight.device() == x.device() && (!bias.defined() || bias.device() == x.device()),
              "in_linear_silu: x, weight and bias must be on the same CUDA device");
  TORCH_CHECK(weight.scalar_type() == x.scalar_type(), "weight must have the dtype of x");
  TORCH_CHECK(weight.size(1) == x.size(1), "weight dim[1] must equal to x dim[1].");
  c10::cuda::CUDAGuard guard(x.device());
  auto xc = x.contiguous(), wc = weight.contiguous();
  at::Tensor bc;
  if (bias.defined()) {
    TORCH_CHECK(bias.dim() == 1 && bias.numel() > 0, "bias must be 1D and not empty");
    TORCH_CHECK(bias.size(0) == weight.size(0), "bias dim[0] must equal to weight dim[0].");
    bc = bias.to(at::kFloat).contiguous();
  }
  const int64_t m = xc.size(0), n = wc.size(0);
  OpsRecInLinearSiluArgs a;
  memset(&a, 0, sizeof(a));
  a.struct_bytes = sizeof(a);
  a.dtype = dtype_code(x.scalar_type());
  TORCH_CHECK(a.dtype != HSTU_DTYPE_FP32, "in_linear_silu: x and weight must be bf16 or fp16");
  at::Tensor outs[4];
  for (int i = 0; i < 4; ++i) {
    TORCH_CHECK(split[i] >= 16 && split[i] <= 8192 && split[i] % 16 == 0,
                "uvqk dim must in range[16, 8192] and multiples of 16.");
    outs[i] = at::empty({m, split[i]}, xc.options());
    a.split[i] = static_cast<int32_t>(split[i]);
  }
  auto lin = at::empty({m, n}, xc.options());
  a.x = xc.data_ptr();
  a.weight = wc.data_ptr();
  a.bias = bc.defined() ? bc.data_ptr() : nullptr;
  a.user = outs[0].data_ptr();
  a.value = outs[1].data_ptr();
  a.query = outs[2].data_ptr();
  a.key = outs[3].data_ptr();
  a.linear_output = lin.data_ptr();
  a.m = m;
  TORCH_CHECK(n <= 32768 && xc.size(1) <= 8192, "weight dim[0] must in range[64, 32768] and multiples of 16.");
  a.n = static_cast<int32_t>(n);
  a.k = static_cast<int32_t>(xc.size(1));
  const int rc = ops_rec_in_linear_silu_fwd(&a, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, hstu_last_error());
  return std::make_tuple(outs[0], outs[1], outs[2], outs[3], lin);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> in_linear_silu_fwd_meta(
    const at::Tensor& x, const at::Tensor& weight, const at::Tensor&, at::IntArrayRef split) {
  TORCH_CHECK(split.size() == 4, "splitList must have 4 elements.");
  const auto m = x.size(0);
  auto o = x.options();
  return std::make_tuple(at::empty({m, split[0]}, o), at::empty({m, split[1]}, o), at::empty({m, split[2]}, o),
                         at::empty({m, split[3]}, o), at::empty({m, weight.size(0)}, o));
}

// in_linear_silu_backward (ascendc/activation/in_linear_silu/torch_extension/in_linear_silu_backward_plugin.cpp:
// checks :41-103, implementation :118-152): (x_grad, weight_grad, bias_grad, undefined).  bias_grad is fp32 like the
// bias; x_grad / weight_grad come back in the input type.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> in_linear_silu_bwd(
    const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias, const at::Tensor& user_grad,
    const at::Tensor& value_grad, const at::Tensor& query_grad, const at::Tensor& key_grad,
    const at::Tensor& linear_output, at::IntArrayRef split) {
  TORCH_CHECK(x.defined() && x.numel() > 0, "x is empty");
  TORCH_CHECK(weight.defined() && weight.numel() > 0, "weight is empty");
  TORCH_CHECK(x.dim() == 2, "x must be 2D");
  TORCH_CHECK(weight.dim() == 2, "weight must be 2D");
  TORCH_CHECK(split.size() == 4, "split_list must have 4 elements.");
  TORCH_CHECK(x.is_cuda() && weight.is_cuda(), "in_linear_silu_backward: tensors must be CUDA tensors");
  TORCH_CHECK(weight.scalar_type() == x.scalar_type(), "weight must have the dtype of x");
  TORCH_CHECK(weight.size(1) == x.size(1), "weight dim[1] must equal to x dim[1].");
  const at::Tensor* gs[5] = {&user_grad, &value_grad, &query_grad, &key_grad, &linear_output};
  const char* names[5] = {"user_grad", "value_grad", "query_grad", "key_grad", "linear_output"};
  for (int i = 0; i < 5; ++i) {
    TORCH_CHECK(gs[i]->defined() && gs[i]->numel() > 0, names[i], " is empty");
    TORCH_CHECK(gs[i]->dim() == 2, names[i], " must be 2D");
    TORCH_CHECK(gs[i]->device() == x.device() && gs[i]->scalar_type() == x.scalar_type(), names[i],
                " must be on x's device and of x's dtype");
    TORCH_CHECK(gs[i]->size(0) == x.size(0),
                "user_grad, value_grad, query_grad, key_grad linear_output dim[0] must equal to x dim[0].");
    if (i < 4) TORCH_CHECK(gs[i]->size(1) == split[i], "user_grad, value_grad, query_grad, key_grad dim[1] must be equal to split_list.");
  }
  TORCH_CHECK(linear_output.size(1) == weight.size(0), "linear_output dim[1] must equal to weight dim[0].");
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias) {
    TORCH_CHECK(bias->dim() == 1 && bias->numel() > 0, "bias must be 1D and not empty");
    TORCH_CHECK(bias->size(0) == weight.size(0), "bias dim[0] must equal to weight dim[0].");
    TORCH_CHECK(bias->device() == x.device(), "bias must be on x's device");
  }
  c10::cuda::CUDAGuard guard(x.device());
  auto xc = x.contiguous(), wc = weight.contiguous();
  at::Tensor gc[5];
  for (int i = 0; i < 5; ++i) gc[i] = gs[i]->contiguous();
  auto x_grad = at::empty_like(xc), w_grad = at::empty_like(wc);
  at::Tensor b_grad;
  if (has_bias) b_grad = at::empty({wc.size(0)}, xc.options().dtype(at::kFloat));
  OpsRecInLinearSiluBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.struct_bytes = sizeof(a);
  a.dtype = dtype_code(x.scalar_type());
  TORCH_CHECK(a.dtype != HSTU_DTYPE_FP32, "in_linear_silu_backward: tensors must be bf16 or fp16");
  a.x = xc.data_ptr();
  a.weight = wc.data_ptr();
  a.user_grad = gc[0].data_ptr();
  a.value_grad = gc[1].data_ptr();
  a.query_grad = gc[2].data_ptr();
  a.key_grad = gc[3].data_ptr();
  a.linear_output = gc[4].data_ptr();
  a.x_grad = x_grad.data_ptr();
  a.weight_grad = w_grad.data_ptr();
  a.bias_grad = has_bias ? b_grad.data_ptr() : nullptr;
  a.m = xc.size(0);
  a.n = static_cast<int32_t>(wc.size(0));
  a.k = static_cast<int32_t>(xc.size(1));
  for (int i = 0; i < 4; ++i) a.split[i] = static_cast<int32_t>(split[i]);
  uint64_t ws_bytes = 0;
  int rc = ops_rec_in_linear_silu_bwd_get_workspace_size(&a, &ws_bytes);
  TORCH_CHECK(rc == 0, hstu_last_error());
  auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, xc.options().dtype(at::kByte));
  rc = ops_rec_in_linear_silu_bwd(&a, ws.data_ptr(), ws_bytes, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, hstu_last_error());
  if (has_bias && bias->scalar_type() != at::kFloat) b_grad = b_grad.to(bias->scalar_type());
  return std::make_tuple(x_grad, w_grad, b_grad, at::Tensor());
}

// (in_linear_silu_backward_plugin.cpp:105-116)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> in_linear_silu_bwd_meta(
    const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias, const at::Tensor&,
    const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&, at::IntArrayRef) {
  at::Tensor b_grad;
  if (bias.has_value() && bias->defined()) b_grad = at::empty_like(*bias);
  return std::make_tuple(at::empty_like(x), at::empty_like(weight), b_grad, at::Tensor());
}

// hstu_dense: [B, S, N, D] layout, every batch row one sequence of S tokens
// (ascendc/attention/hstu_v1/torch_extension/hstu_dense_plugin.cpp:19-40).  It is the jagged forward over equal
// lengths: the tensors are viewed as [B*S, N, D] and the offsets 0, S, 2S, ... are generated on the device.
at::Tensor hstu_dense(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                      const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias,
                      int64_t mask_type, int64_t max_seq_len, double silu_scale) {
  TORCH_CHECK(q.dim() == 4, "The q should be 4D in dense layout");
  TORCH_CHECK(k.dim() == 4 && v.dim() == 4, "The k and v should be 4D in dense layout");
  TORCH_CHECK(k.size(0) == q.size(0) && v.size(0) == q.size(0) && k.size(1) == v.size(1),
              "q, k and v must agree in batch, and k and v in sequence length");
  TORCH_CHECK(k.size(1) == q.size(1), "hstu_dense expects q and k of the same sequence length");
  const int64_t B = q.size(0), S = q.size(1);
  auto dq = q.contiguous().view({B * S, q.size(2), q.size(3)});
  auto dk = k.contiguous().view({B * S, k.size(2), k.size(3)});
  auto dv = v.contiguous().view({B * S, v.size(2), v.size(3)});
  auto off = at::arange(0, (B + 1) * S, S, q.options().dtype(at::kLong));
  // the reference takes max_seq_len only for the default silu_scale; the bias / mask row stride is S
  const double scale = silu_scale == 0.0 ? 1.0 / static_cast<double>(max_seq_len > 0 ? max_seq_len : S) : silu_scale;
  TORCH_CHECK(max_seq_len >= 1 && max_seq_len <= 20480, "maxSeqLen expect in [1, 20480], but value is ", max_seq_len);
  auto out = forward_impl(dq, dk, dv, mask, attn_bias, mask_type, S, S, scale, off, off, c10::nullopt, c10::nullopt,
                          0, 1.0, false);
  return out.view({B, S, q.size(2), v.size(3)});
}

at::Tensor hstu_dense_meta(const at::Tensor& q, const at::Tensor&, const at::Tensor&,
                           const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, int64_t, int64_t,
                           double) {
  TORCH_CHECK(q.dim() == 4, "The q should be 4D in dense layout");
  return at::empty_like(q, q.options().device(c10::kMeta));
}

// hstu_paged (ascendc/attention/hstu_v1/torch_extension/hstu_paged_plugin.cpp:21-72): the same checks and
// conversions - kv_cache / page_ids / last_page_len not empty, the page table and seq_offset_k / seq_offset_t
// converted to seq_offset's integer type, q 3-D, offsets of at least two entries, targetGroupSize > 0 with numTarget,
// silu_scale 0 -> 1 / max_seq_len, alpha None -> 1, no num_context (the reference passes zeros).
at::Tensor hstu_paged(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& kv_cache,
                      const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& attn_bias,
                      int64_t mask_type, int64_t max_seq_len, int64_t max_seq_len_k, double silu_scale,
                      const at::Tensor& seq_offset, const at::Tensor& seq_offset_k, const at::Tensor& seq_offset_t,
                      const at::Tensor& page_offsets, const at::Tensor& page_ids, const at::Tensor& last_page_len,
                      const at::Tensor& num_target, int64_t target_group_size, c10::optional<double> alpha,
                      bool deterministic) {
  TORCH_CHECK(kv_cache.defined() && kv_cache.numel() > 0, "kv_cache is empty");
  TORCH_CHECK(page_ids.defined() && page_ids.numel() > 0, "page_ids is empty");
  TORCH_CHECK(last_page_len.defined() && last_page_len.numel() > 0, "last_page_len is empty");
  TORCH_CHECK(q.dim() == 3, "The q should be 3D in jagged layout");
  TORCH_CHECK(seq_offset.defined() && seq_offset_k.defined() && page_offsets.defined(),
              "seq_offset, seq_offset_k and page_offsets are required");
  TORCH_CHECK(seq_offset_t.defined() ? seq_offset_t.size(0) >= 2 : true,
              "acSeqOffsetT params error should have at least two element.");
  TORCH_CHECK(!num_target.defined() || target_group_size > 0,
              "targetGroupSize must be greater than 0 when numTarget is defined");
  TORCH_CHECK(kv_cache.dim() == 5 && kv_cache.size(1) == 2 && kv_cache.size(3) == k.size(1) &&
                  kv_cache.size(4) == k.size(2) && kv_cache.scalar_type() == q.scalar_type(),
              "kv_cache must be [pages, 2, page_size, heads_k, dim] in q's dtype");
  TORCH_CHECK(k.size(0) == q.size(0), "k and v hold the same tokens as q (only their target rows are read)");
  c10::cuda::CUDAGuard guard(q.device());
  c10::optional<at::Tensor> tgt = num_target.defined() ? c10::optional<at::Tensor>(num_target) : c10::nullopt;
  Prepared pr = prepare(q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len_k, silu_scale, seq_offset,
                        seq_offset_k, c10::nullopt, tgt, target_group_size, alpha, deterministic);
  for (const auto* t : {&kv_cache, &page_offsets, &page_ids, &last_page_len}) check_same_device(*t, q, "a page-table tensor");
  const auto it = pr.off_q.scalar_type();
  auto cache = kv_cache.contiguous();
  auto po = page_offsets.to(it).contiguous(), pi = page_ids.to(it).contiguous(), ll = last_page_len.to(it).contiguous();
  TORCH_CHECK(po.numel() == pr.off_q.numel(), "page_offsets must have batch + 1 entries");
  TORCH_CHECK(ll.numel() >= pr.off_q.numel() - 1, "last_page_len is shorter than the batch");
  HstuPagedArgs a;
  memset(&a, 0, sizeof(a));
  a.struct_bytes = sizeof(a);
  a.page_size = static_cast<int32_t>(cache.size(2));
  a.base = pr.a;
  auto out = at::empty({pr.q.size(0), pr.q.size(1), pr.v.size(2)}, pr.q.options());
  a.base.out = out.data_ptr();
  a.kv_cache = cache.data_ptr();
  a.page_offsets = po.data_ptr();
  a.page_ids = pi.data_ptr();
  a.last_page_len = ll.data_ptr();
  a.num_pages = cache.size(0);
  a.num_page_ids = pi.numel();
  uint64_t ws_bytes = 0;
  int rc = hstu_paged_fwd_get_workspace_size(&a, &ws_bytes);
  TORCH_CHECK(rc == 0, "hstu_paged: ", hstu_last_error());
  auto ws = at::empty({static_cast<int64_t>(ws_bytes)}, pr.q.options().dtype(at::kByte));
  rc = hstu_paged_fwd(&a, ws.data_ptr(), ws_bytes, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "hstu_paged: ", hstu_last_error());
  return out;
}

// (hstu_paged_plugin.cpp:107-118)
at::Tensor hstu_paged_meta(const at::Tensor& q, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                           const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, int64_t, int64_t,
                           int64_t, double, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                           const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&, int64_t,
                           c10::optional<double>, bool) {
  TORCH_CHECK(q.dim() == 3, "The q should be 3D in jagged layout");
  return at::empty_like(q, q.options().device(c10::kMeta));
}

at::Tensor meta_out(const at::Tensor& q, const at::Tensor& v) {
  TORCH_CHECK(q.dim() == 3, "The q should be 3D in jagged layout");
  std::vector<c10::SymInt> shape = {q.sym_size(0), q.sym_size(1), v.sym_size(2)};
  return at::empty_symint(shape, q.options().device(c10::kMeta));
}

at::Tensor hstu_jagged_equal_meta(const at::Tensor& q, const at::Tensor&, const at::Tensor& v,
                                  const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, int64_t, int64_t,
                                  double, const at::Tensor&, const c10::optional<at::Tensor>&,
                                  const c10::optional<at::Tensor>&, c10::optional<int64_t>, c10::optional<double>, bool) {
  return meta_out(q, v);
}

at::Tensor hstu_jagged_delta_meta(const at::Tensor& q, const at::Tensor&, const at::Tensor& v,
                                  const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, int64_t, int64_t,
                                  int64_t, double, const at::Tensor&, const at::Tensor&,
                                  const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                  c10::optional<int64_t>, c10::optional<double>, bool) {
  return meta_out(q, v);
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(ops_rec, m) {
  m.def("hstu_jagged.equal(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, "
        "int mask_type=0, int max_seq_len=0, float silu_scale=0.0, Tensor seq_offset=None, "
        "Tensor? num_context=None, Tensor? num_target=None, int? target_group_size=0, float? alpha=1.0, "
        "bool deterministic=False) -> Tensor");
  m.def("hstu_jagged.delta(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, "
        "int mask_type=0, int max_seq_len=0, int max_seq_len_k=0, float silu_scale=0.0, Tensor seq_offset=None, "
        "Tensor seq_offset_k=None, Tensor? num_context=None, Tensor? num_target=None, int? target_group_size=0, "
        "float? alpha=1.0, bool deterministic=False) -> Tensor");
  m.def("hstu_jagged_backward.equal(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor? mask=None, "
        "Tensor? attn_bias=None, int mask_type=0, int max_seq_len=0, float silu_scale=0.0, Tensor seq_offset=None, "
        "Tensor? num_context=None, Tensor? num_target=None, int? target_group_size=0, float? alpha=1.0) "
        "-> (Tensor, Tensor, Tensor, Tensor)");
  m.def("hstu_jagged_backward.delta(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor? mask=None, "
        "Tensor? attn_bias=None, int mask_type=0, int max_seq_len=0, int max_seq_len_k=0, float silu_scale=0.0, "
        "Tensor seq_offset=None, Tensor seq_offset_k=None, Tensor? num_context=None, Tensor? num_target=None, "
        "int? target_group_size=0, float? alpha=1.0) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("ln_mul(Tensor x, Tensor u, Tensor gamma, Tensor beta) -> Tensor");
  m.def("distance_in_linear_silu(Tensor x, Tensor weight, Tensor bias, int[] attr_dict) -> "
        "(Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("hstu_dense(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, "
        "int max_seq_len=0, float silu_scale=0.0) -> Tensor");
  // in_linear_silu_backward_plugin.cpp:154-161
  m.def("in_linear_silu_backward(Tensor x, Tensor weight, Tensor ? bias,Tensor user_grad, Tensor value_grad, "
        "Tensor query_grad, Tensor key_grad,Tensor linear_output,int[] attr_dict) -> (Tensor, Tensor, Tensor, Tensor)");
  // hstu_paged_plugin.cpp:75-98
  m.def("hstu_paged(Tensor q, Tensor k, Tensor v, Tensor kv_cache=None, Tensor? mask=None, Tensor? attn_bias=None,"
        " int mask_type=0, int max_seq_len=0, int max_seq_len_k=0, float silu_scale=0.0, Tensor seq_offset=None,"
        " Tensor seq_offset_k=None, Tensor seq_offset_t=None, Tensor page_offsets=None, Tensor page_ids=None,"
        " Tensor last_page_len=None, Tensor num_target=None, int target_group_size=0, float? alpha=1.0,"
        " bool deterministic=False) -> Tensor");
}

TORCH_LIBRARY_IMPL(ops_rec, CUDA, m) {
  m.impl("hstu_jagged.equal", TORCH_FN(hstu_jagged_equal));
  m.impl("hstu_jagged.delta", TORCH_FN(hstu_jagged_delta));
  m.impl("hstu_jagged_backward.equal", TORCH_FN(hstu_jagged_backward_equal));
  m.impl("hstu_jagged_backward.delta", TORCH_FN(hstu_jagged_backward_delta));
  m.impl("ln_mul", TORCH_FN(ln_mul));
  m.impl("distance_in_linear_silu", TORCH_FN(in_linear_silu_fwd));
  m.impl("hstu_dense", TORCH_FN(hstu_dense));
  m.impl("hstu_paged", TORCH_FN(hstu_paged));
  m.impl("in_linear_silu_backward", TORCH_FN(in_linear_silu_bwd));
}

TORCH_LIBRARY_IMPL(ops_rec, Meta, m) {
  m.impl("hstu_jagged.equal", TORCH_FN(hstu_jagged_equal_meta));
  m.impl("hstu_jagged.delta", TORCH_FN(hstu_jagged_delta_meta));
  m.impl("hstu_jagged_backward.equal", TORCH_FN(hstu_jagged_backward_equal_meta));
  m.impl("hstu_jagged_backward.delta", TORCH_FN(hstu_jagged_backward_delta_meta));
  m.impl("ln_mul", TORCH_FN(ln_mul_meta));
  m.impl("distance_in_linear_silu", TORCH_FN(in_linear_silu_fwd_meta));
  m.impl("hstu_dense", TORCH_FN(hstu_dense_meta));
  m.impl("hstu_paged", TORCH_FN(hstu_paged_meta));
  m.impl("in_linear_silu_backward", TORCH_FN(in_linear_silu_bwd_meta));
}
