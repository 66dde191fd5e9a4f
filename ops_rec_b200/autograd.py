"""Autograd formulas of `hstu_jagged` (.equal and .delta), bound to the `hstu_jagged_backward` operator.

Same arrangement as the reference (ascendc/attention/hstu_v1/torch_extension/hstu_v1_autograd.py:143-330): the
forward has no C++ autograd key; `torch.library.register_autograd` attaches the backward operator as its formula on
the Autograd dispatch key, so eager and compiled training both just call the forward and `loss.backward()`.
Gradients flow to q, k, v and attn_bias; a mask that requires grad is rejected (the backward has no mask gradient).
"""
from __future__ import annotations

import torch

_EQUAL_DEFAULTS = (None, None, None, None, None, 0, 0, 0.0, None, None, None, 0, 1.0, False)
_DELTA_DEFAULTS = (None, None, None, None, None, 0, 0, 0, 0.0, None, None, None, None, 0, 1.0, False)

_registered = False
registration_errors = {}


def _unpack(inputs, defaults):
    """Inputs in schema order; slots a torch version did not pass take the schema's defaults."""
    vals = list(inputs)
    vals.extend(defaults[len(vals):])
    return tuple(vals[:len(defaults)])


def _reject_mask_grad(mask, name):
    if mask is not None and mask.requires_grad:
        raise NotImplementedError(f"{name}: mask is not differentiable (the backward has no mask gradient)")


def _equal_setup(ctx, inputs, output=None):
    (q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, num_context, num_target,
     target_group_size, alpha, _det) = _unpack(inputs, _EQUAL_DEFAULTS)
    _reject_mask_grad(mask, "hstu_jagged.equal")
    ctx.save_for_backward(q, k, v, mask, attn_bias, seq_offset, num_context, num_target)
    ctx.scalars = (mask_type, max_seq_len, silu_scale, target_group_size, alpha)
    ctx.nargs = len(inputs)


def _equal_backward(ctx, grad):
    q, k, v, mask, attn_bias, seq_offset, num_context, num_target = ctx.saved_tensors
    mask_type, max_seq_len, silu_scale, group, alpha = ctx.scalars
    dq, dk, dv, dbias = torch.ops.ops_rec.hstu_jagged_backward.equal(
        grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, num_context, num_target,
        group, alpha)
    grads = [dq, dk, dv, None, dbias if attn_bias is not None else None] + [None] * (len(_EQUAL_DEFAULTS) - 5)
    return tuple(grads[:ctx.nargs])


def _delta_setup(ctx, inputs, output=None):
    (q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len_k, silu_scale, seq_offset, seq_offset_k,
     num_context, num_target, target_group_size, alpha, _det) = _unpack(inputs, _DELTA_DEFAULTS)
    _reject_mask_grad(mask, "hstu_jagged.delta")
    ctx.save_for_backward(q, k, v, mask, attn_bias, seq_offset, seq_offset_k, num_context, num_target)
    ctx.scalars = (mask_type, max_seq_len, max_seq_len_k, silu_scale, target_group_size, alpha)
    ctx.nargs = len(inputs)


def _delta_backward(ctx, grad):
    q, k, v, mask, attn_bias, seq_offset, seq_offset_k, num_context, num_target = ctx.saved_tensors
    mask_type, max_seq_len, max_seq_len_k, silu_scale, group, alpha = ctx.scalars
    dq, dk, dv, dbias = torch.ops.ops_rec.hstu_jagged_backward.delta(
        grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, max_seq_len_k, silu_scale, seq_offset, seq_offset_k,
        num_context, num_target, group, alpha)
    grads = [dq, dk, dv, None, dbias if attn_bias is not None else None] + [None] * (len(_DELTA_DEFAULTS) - 5)
    return tuple(grads[:ctx.nargs])


# ----------------------------------------------------------------------------------------- in_linear_silu
# distance_in_linear_silu(x, weight, bias, attr_dict) -> (user, value, query, key, linear_output), bound to
# in_linear_silu_backward exactly as ascendc/activation/in_linear_silu/torch_extension/_autograd.py:37-85 does: the
# forward's linear_output is saved, its own incoming gradient is ignored (the backward operator applies the SiLU
# derivative itself).
def _linsilu_setup(ctx, inputs, output):
    x, weight, bias, attr_dict = inputs
    ctx.has_bias = bias is not None
    if ctx.has_bias:
        ctx.save_for_backward(x, weight, bias, output[-1])
    else:
        ctx.save_for_backward(x, weight, output[-1])
    ctx.attr_dict = list(attr_dict)


def _linsilu_backward(ctx, user_grad, value_grad, query_grad, key_grad, linear_output_grad):
    if ctx.has_bias:
        x, weight, bias, linear_output = ctx.saved_tensors
    else:
        x, weight, linear_output = ctx.saved_tensors
        bias = None
    x_grad, weight_grad, bias_grad, _ = torch.ops.ops_rec.in_linear_silu_backward(
        x, weight, bias, user_grad, value_grad, query_grad, key_grad, linear_output, ctx.attr_dict)
    return x_grad, weight_grad, bias_grad, None


def register_autograd():
    """Attach the formulas (idempotent).  A failure for one overload is recorded in `registration_errors` and does
    not stop the other, as in the reference's registration (hstu_v1_autograd.py:301-312)."""
    global _registered
    if _registered:
        return
    _registered = True
    for name, op, bwd, setup in (
            ("hstu_jagged.equal", torch.ops.ops_rec.hstu_jagged.equal, _equal_backward, _equal_setup),
            ("hstu_jagged.delta", torch.ops.ops_rec.hstu_jagged.delta, _delta_backward, _delta_setup),
            ("distance_in_linear_silu", torch.ops.ops_rec.distance_in_linear_silu.default, _linsilu_backward,
             _linsilu_setup)):
        try:
            torch.library.register_autograd(op, bwd, setup_context=setup)
        except Exception as e:  # noqa: BLE001 - differences between torch versions are recorded, not fatal
            registration_errors[name] = f"{type(e).__name__}: {e}"
