"""ctypes binding of the C ABI declared in include/hstu_b200.h.

This is the binding a Python caller without the torch operator registration would write; the parity tests use
it so that every GPU result they check went through the C entry points.  torch is used only for device memory
and the current stream.  Loading fails loudly when the shared library has not been built - there is no
fallback of any kind.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libhstu_b200.so")

DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
MASK_TRIL, MASK_TRIU, MASK_NONE, MASK_CUSTOM = 0, 1, 2, 3
FLAG_DETERMINISTIC, FLAG_ALPHA_BEFORE_BIAS, FLAG_FORCE_GENERIC = 1, 2, 4
ST_BAD_OFFSETS, ST_LEN_GT_MAX, ST_BAD_CTX_TARGET, ST_BAD_PAGES, ST_PIPE_TIMEOUT = 1, 2, 4, 8, 256

EXPORTS = (
    "hstu_jagged_fwd_get_workspace_size", "hstu_jagged_fwd", "hstu_jagged_fwd_status",
    "hstu_jagged_fwd_kernel_kind", "hstu_plan_host", "hstu_debug_mask_host", "hstu_debug_tiles_host",
    "hstu_last_error", "hstu_b200_version", "hstu_jagged_fwd_static", "hstu_jagged_fwd_static_status",
    "hstu_jagged_bwd_get_workspace_size", "hstu_jagged_bwd", "ops_rec_ln_mul_f32", "ops_rec_in_linear_silu_fwd",
    "hstu_paged_fwd_get_workspace_size", "hstu_paged_fwd",
    "ops_rec_in_linear_silu_bwd_get_workspace_size", "ops_rec_in_linear_silu_bwd",
)
STATIC_SCRATCH_BYTES = 1 << 20
E_SCRATCH_LIMIT = -6


class HstuJaggedArgs(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32), ("dtype", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("attn_bias", C.c_void_p), ("bias_batch_stride", C.c_int64), ("mask", C.c_void_p),
        ("seq_offset_q", C.c_void_p), ("seq_offset_k", C.c_void_p),
        ("num_context", C.c_void_p), ("num_target", C.c_void_p), ("index_bytes", C.c_int32),
        ("batch", C.c_int32), ("total_q", C.c_int64), ("total_k", C.c_int64),
        ("heads_q", C.c_int32), ("heads_k", C.c_int32), ("dim_qk", C.c_int32), ("dim_v", C.c_int32),
        ("mask_type", C.c_int32), ("max_seq_len_q", C.c_int32), ("max_seq_len_k", C.c_int32),
        ("target_group_size", C.c_int32), ("silu_scale", C.c_float), ("alpha", C.c_float),
        ("flags", C.c_uint32), ("reserved", C.c_uint32),
    ]


class HstuPagedArgs(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32), ("page_size", C.c_int32), ("base", HstuJaggedArgs),
        ("kv_cache", C.c_void_p), ("page_offsets", C.c_void_p), ("page_ids", C.c_void_p),
        ("last_page_len", C.c_void_p), ("seq_offset_t", C.c_void_p), ("num_pages", C.c_int64),
        ("num_page_ids", C.c_int64),
    ]


class HstuJaggedBwdArgs(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32), ("reserved", C.c_uint32), ("fwd", HstuJaggedArgs),
        ("grad_out", C.c_void_p), ("grad_q", C.c_void_p), ("grad_k", C.c_void_p), ("grad_v", C.c_void_p),
        ("grad_bias", C.c_void_p),
    ]


class OpsRecInLinearSiluArgs(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32), ("dtype", C.c_int32), ("x", C.c_void_p), ("weight", C.c_void_p),
        ("bias", C.c_void_p), ("user", C.c_void_p), ("value", C.c_void_p), ("query", C.c_void_p), ("key", C.c_void_p),
        ("linear_output", C.c_void_p), ("m", C.c_int64), ("n", C.c_int32), ("k", C.c_int32), ("split", C.c_int32 * 4),
        ("status", C.c_void_p),
    ]


class OpsRecInLinearSiluBwdArgs(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32), ("dtype", C.c_int32), ("x", C.c_void_p), ("weight", C.c_void_p),
        ("user_grad", C.c_void_p), ("value_grad", C.c_void_p), ("query_grad", C.c_void_p), ("key_grad", C.c_void_p),
        ("linear_output", C.c_void_p), ("x_grad", C.c_void_p), ("weight_grad", C.c_void_p), ("bias_grad", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int32), ("k", C.c_int32), ("split", C.c_int32 * 4), ("status", C.c_void_p),
    ]


class HstuError(RuntimeError):
    """A non-zero status from the C ABI (code in .code, text from hstu_last_error())."""

    def __init__(self, code, text):
        super().__init__(f"hstu_b200 error {code}: {text}")
        self.code = code


_lib = None


def load():
    """dlopen the library (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python ops_rec_b200/_build.py` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    A = C.POINTER(HstuJaggedArgs)
    lib.hstu_jagged_fwd_get_workspace_size.argtypes = [A, C.POINTER(C.c_uint64)]
    lib.hstu_jagged_fwd_get_workspace_size.restype = C.c_int
    lib.hstu_jagged_fwd.argtypes = [A, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.hstu_jagged_fwd.restype = C.c_int
    lib.hstu_jagged_fwd_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)]
    lib.hstu_jagged_fwd_status.restype = C.c_int
    lib.hstu_jagged_fwd_kernel_kind.argtypes = [A]
    lib.hstu_jagged_fwd_kernel_kind.restype = C.c_int
    lib.hstu_plan_host.argtypes = [A, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                   C.POINTER(C.c_uint32)]
    lib.hstu_plan_host.restype = C.c_int64
    lib.hstu_debug_mask_host.argtypes = [C.c_int32] * 6 + [C.c_void_p]
    lib.hstu_debug_mask_host.restype = C.c_int
    lib.hstu_debug_tiles_host.argtypes = [C.c_int32] * 9 + [C.POINTER(C.c_uint64)]
    lib.hstu_debug_tiles_host.restype = C.c_int
    lib.hstu_jagged_fwd_static.argtypes = [A, C.c_void_p]
    lib.hstu_jagged_fwd_static.restype = C.c_int
    lib.hstu_jagged_fwd_static_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
    lib.hstu_jagged_fwd_static_status.restype = C.c_int
    B = C.POINTER(HstuJaggedBwdArgs)
    lib.hstu_jagged_bwd_get_workspace_size.argtypes = [B, C.POINTER(C.c_uint64)]
    lib.hstu_jagged_bwd_get_workspace_size.restype = C.c_int
    lib.hstu_jagged_bwd.argtypes = [B, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.hstu_jagged_bwd.restype = C.c_int
    P = C.POINTER(HstuPagedArgs)
    lib.hstu_paged_fwd_get_workspace_size.argtypes = [P, C.POINTER(C.c_uint64)]
    lib.hstu_paged_fwd_get_workspace_size.restype = C.c_int
    lib.hstu_paged_fwd.argtypes = [P, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.hstu_paged_fwd.restype = C.c_int
    LB = C.POINTER(OpsRecInLinearSiluBwdArgs)
    lib.ops_rec_in_linear_silu_bwd_get_workspace_size.argtypes = [LB, C.POINTER(C.c_uint64)]
    lib.ops_rec_in_linear_silu_bwd_get_workspace_size.restype = C.c_int
    lib.ops_rec_in_linear_silu_bwd.argtypes = [LB, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.ops_rec_in_linear_silu_bwd.restype = C.c_int
    lib.ops_rec_ln_mul_f32.argtypes = [C.c_void_p] * 5 + [C.c_int64, C.c_int64, C.c_void_p]
    lib.ops_rec_ln_mul_f32.restype = C.c_int
    lib.ops_rec_in_linear_silu_fwd.argtypes = [C.POINTER(OpsRecInLinearSiluArgs), C.c_void_p]
    lib.ops_rec_in_linear_silu_fwd.restype = C.c_int
    lib.hstu_last_error.restype = C.c_char_p
    lib.hstu_b200_version.restype = C.c_int
    _lib = lib
    return lib


def check(rc):
    if rc < 0:
        raise HstuError(rc, load().hstu_last_error().decode())
    return rc


def _dtype_code(t):
    import torch
    code = {torch.bfloat16: DTYPE_BF16, torch.float16: DTYPE_FP16, torch.float32: DTYPE_FP32}.get(t)
    if code is None:
        raise HstuError(-2, f"dtype {t} is not supported (bf16, fp16, fp32 only; fp8 inputs are rejected)")
    return code


def make_args(q, k, v, out, seq_offset, *, seq_offset_k=None, mask=None, attn_bias=None, mask_type=0,
              max_seq_len=0, max_seq_len_k=None, silu_scale=0.0, num_context=None, num_target=None,
              target_group_size=0, alpha=1.0, flags=0, ptr=lambda t: t.data_ptr()):
    """Fill an HstuJaggedArgs from tensors (torch tensors by default; `ptr` extracts the address).
    Returns (args, keepalive) - keepalive holds converted temporaries that must outlive the launch."""
    for name, t in (("k", k), ("v", v), ("out", out), ("seq_offset", seq_offset), ("seq_offset_k", seq_offset_k),
                    ("mask", mask), ("attn_bias", attn_bias), ("num_context", num_context),
                    ("num_target", num_target)):
        # a pointer to another device (or to host memory) would fault inside the kernel instead of failing here
        if t is not None and hasattr(t, "device") and hasattr(q, "device") and t.device != q.device:
            raise ValueError(f"{name} is on {t.device} but q is on {q.device}")
    a = HstuJaggedArgs()
    a.struct_bytes = C.sizeof(HstuJaggedArgs)
    a.dtype = _dtype_code(q.dtype)
    keep = []
    a.q, a.k, a.v = ptr(q), ptr(k), ptr(v)
    a.out = ptr(out) if out is not None else None
    if attn_bias is not None:
        a.attn_bias = ptr(attn_bias)
        if attn_bias.dim() == 3 or attn_bias.shape[0] == 1:
            a.bias_batch_stride = 0
        else:
            a.bias_batch_stride = attn_bias.shape[-3] * attn_bias.shape[-2] * attn_bias.shape[-1]
    if mask is not None:
        a.mask = ptr(mask)
    a.seq_offset_q = ptr(seq_offset)
    a.seq_offset_k = ptr(seq_offset_k) if seq_offset_k is not None else None
    a.index_bytes = seq_offset.element_size()
    for name, t in (("num_context", num_context), ("num_target", num_target)):
        if t is not None:
            if t.dtype != seq_offset.dtype:
                t = t.to(seq_offset.dtype)
                keep.append(t)
            setattr(a, name, ptr(t))
    a.batch = seq_offset.shape[0] - 1
    a.total_q, a.total_k = q.shape[0], k.shape[0]
    a.heads_q, a.heads_k, a.dim_qk, a.dim_v = q.shape[1], k.shape[1], q.shape[2], v.shape[2]
    a.mask_type = int(mask_type)
    a.max_seq_len_q = int(max_seq_len)
    a.max_seq_len_k = int(max_seq_len_k if max_seq_len_k else max_seq_len)
    a.target_group_size = int(target_group_size or 0)
    a.silu_scale = float(silu_scale)
    a.alpha = float(1.0 if alpha is None else alpha)
    a.flags = int(flags)
    return a, keep


def workspace_size(args):
    n = C.c_uint64(0)
    check(load().hstu_jagged_fwd_get_workspace_size(C.byref(args), C.byref(n)))
    return n.value


def kernel_kind(args):
    return check(load().hstu_jagged_fwd_kernel_kind(C.byref(args)))


def hstu_jagged_forward(q, k, v, mask=None, attn_bias=None, mask_type=0, max_seq_len=0, silu_scale=0.0,
                        seq_offset=None, num_context=None, num_target=None, target_group_size=0, alpha=1.0,
                        deterministic=False, *, max_seq_len_k=None, seq_offset_k=None, flags=0,
                        return_status=False, out=None):
    """The operator through the C ABI on CUDA tensors (argument order of ops_rec::hstu_jagged.equal,
    ascendc/attention/hstu_v1/torch_extension/hstu_jagged_plugin.cpp:188-201; the keyword-only extras give the
    .delta overload).  Launches on torch's current stream; with return_status=True it also synchronises and
    returns the device status word."""
    import torch
    if q.dim() != 3:
        raise HstuError(-2, "The q should be 3D in jagged layout")
    if not q.is_cuda:
        raise HstuError(-2, "tensors must live on a CUDA device; there is no CPU implementation")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty(q.shape[0], q.shape[1], v.shape[2], dtype=q.dtype, device=q.device)
    if deterministic:
        flags |= FLAG_DETERMINISTIC
    args, keep = make_args(q, k, v, out, seq_offset, seq_offset_k=seq_offset_k, mask=mask, attn_bias=attn_bias,
                           mask_type=mask_type, max_seq_len=max_seq_len, max_seq_len_k=max_seq_len_k,
                           silu_scale=silu_scale, num_context=num_context, num_target=num_target,
                           target_group_size=target_group_size, alpha=alpha, flags=flags)
    nbytes = workspace_size(args)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        check(load().hstu_jagged_fwd(C.byref(args), ws.data_ptr(), nbytes, stream))
        if return_status:
            st = C.c_uint32(0)
            check(load().hstu_jagged_fwd_status(ws.data_ptr(), stream, C.byref(st)))
            return out, st.value
    del keep
    return out


def hstu_jagged_backward(grad, q, k, v, mask=None, attn_bias=None, mask_type=0, max_seq_len=0, max_seq_len_k=0,
                         silu_scale=0.0, seq_offset=None, seq_offset_k=None, num_context=None, num_target=None,
                         target_group_size=0, alpha=1.0, *, flags=0, return_status=False):
    """Gradients (dq, dk, dv, d_bias or None) through hstu_jagged_bwd on CUDA tensors; argument order of
    ops_rec::hstu_jagged_backward.delta (hstu_v1/torch_extension/hstu_jagged_plugin.cpp:237-252).  d_bias needs no
    clearing: the kernels write every element of it."""
    import torch
    if q.dim() != 3:
        raise HstuError(-2, "The q should be 3D in jagged layout")
    if not q.is_cuda:
        raise HstuError(-2, "tensors must live on a CUDA device; there is no CPU implementation")
    grad, q, k, v = grad.contiguous(), q.contiguous(), k.contiguous(), v.contiguous()
    if attn_bias is not None:
        attn_bias = attn_bias.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dbias = torch.empty_like(attn_bias) if attn_bias is not None else None
    fwd, keep = make_args(q, k, v, None, seq_offset, seq_offset_k=seq_offset_k, mask=mask, attn_bias=attn_bias,
                          mask_type=mask_type, max_seq_len=max_seq_len, max_seq_len_k=max_seq_len_k or None,
                          silu_scale=silu_scale, num_context=num_context, num_target=num_target,
                          target_group_size=target_group_size, alpha=alpha, flags=flags)
    a = HstuJaggedBwdArgs()
    a.struct_bytes = C.sizeof(HstuJaggedBwdArgs)
    a.fwd = fwd
    a.grad_out, a.grad_q, a.grad_k, a.grad_v = grad.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.grad_bias = dbias.data_ptr() if dbias is not None else None
    n = C.c_uint64(0)
    check(load().hstu_jagged_bwd_get_workspace_size(C.byref(a), C.byref(n)))
    ws = torch.empty(n.value, dtype=torch.uint8, device=q.device)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        check(load().hstu_jagged_bwd(C.byref(a), ws.data_ptr(), n.value, stream))
        if return_status:
            st = C.c_uint32(0)
            check(load().hstu_jagged_fwd_status(ws.data_ptr(), stream, C.byref(st)))
            return (dq, dk, dv, dbias), st.value
    del keep
    return dq, dk, dv, dbias


def hstu_paged_forward(q, k, v, kv_cache, mask=None, attn_bias=None, mask_type=0, max_seq_len=0, max_seq_len_k=0,
                       silu_scale=0.0, seq_offset=None, seq_offset_k=None, seq_offset_t=None, page_offsets=None,
                       page_ids=None, last_page_len=None, num_target=None, target_group_size=0, alpha=1.0, *,
                       flags=0, return_status=False, workspace_fill=None):
    """ops_rec::hstu_paged through hstu_paged_fwd on CUDA tensors (argument order of the reference schema,
    hstu_v1/torch_extension/hstu_paged_plugin.cpp:75-98).  The page-table tensors are converted to seq_offset's
    integer type like the reference adapter does (:33-35)."""
    import torch
    if q.dim() != 3:
        raise HstuError(-2, "The q should be 3D in jagged layout")
    if not q.is_cuda:
        raise HstuError(-2, "tensors must live on a CUDA device; there is no CPU implementation")
    q, k, v, kv_cache = q.contiguous(), k.contiguous(), v.contiguous(), kv_cache.contiguous()
    it = seq_offset.dtype
    conv = [t.to(it).contiguous() for t in (seq_offset_k, page_offsets, page_ids, last_page_len)]
    seq_offset_k, page_offsets, page_ids, last_page_len = conv
    for name, t in (("kv_cache", kv_cache), ("page_offsets", page_offsets), ("page_ids", page_ids),
                    ("last_page_len", last_page_len)):
        if t.device != q.device:
            raise ValueError(f"{name} is on {t.device} but q is on {q.device}")
    out = torch.empty(q.shape[0], q.shape[1], v.shape[2], dtype=q.dtype, device=q.device)
    base, keep = make_args(q, k, v, out, seq_offset, seq_offset_k=seq_offset_k, mask=mask, attn_bias=attn_bias,
                           mask_type=mask_type, max_seq_len=max_seq_len, max_seq_len_k=max_seq_len_k or None,
                           silu_scale=silu_scale, num_target=num_target, target_group_size=target_group_size,
                           alpha=alpha, flags=flags)
    a = HstuPagedArgs()
    a.struct_bytes = C.sizeof(HstuPagedArgs)
    a.page_size = kv_cache.shape[2]
    a.base = base
    a.kv_cache, a.page_offsets, a.page_ids = kv_cache.data_ptr(), page_offsets.data_ptr(), page_ids.data_ptr()
    a.last_page_len = last_page_len.data_ptr()
    a.seq_offset_t = seq_offset_t.data_ptr() if seq_offset_t is not None else None
    a.num_pages, a.num_page_ids = kv_cache.shape[0], page_ids.numel()
    n = C.c_uint64(0)
    check(load().hstu_paged_fwd_get_workspace_size(C.byref(a), C.byref(n)))
    # (workspace_fill: tests fill the workspace with a byte pattern first - nothing the call reads may be uninitialised)
    ws = torch.empty(n.value, dtype=torch.uint8, device=q.device)
    if workspace_fill is not None:
        ws.fill_(workspace_fill)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        check(load().hstu_paged_fwd(C.byref(a), ws.data_ptr(), n.value, stream))
        if return_status:
            st = C.c_uint32(0)
            check(load().hstu_jagged_fwd_status(ws.data_ptr(), stream, C.byref(st)))
            return out, st.value
    del keep, conv
    return out


def in_linear_silu(x, weight, bias, split):
    """(user, value, query, key, linear_output) through ops_rec_in_linear_silu_fwd on CUDA tensors (argument order of
    ops_rec::distance_in_linear_silu, in_linear_silu/torch_extension/in_linear_silu_plugin.cpp:70-98)."""
    import torch
    if x.dim() != 2 or weight.dim() != 2:
        raise HstuError(-2, "x and weight must be 2D")
    if not x.is_cuda:
        raise HstuError(-2, "tensors must live on a CUDA device; there is no CPU implementation")
    x, weight = x.contiguous(), weight.contiguous()
    bias = bias.float().contiguous() if bias is not None else None
    a = OpsRecInLinearSiluArgs()
    a.struct_bytes = C.sizeof(OpsRecInLinearSiluArgs)
    a.dtype = _dtype_code(x.dtype)
    m, k, n = x.shape[0], x.shape[1], weight.shape[0]
    if weight.shape[1] != k:
        raise HstuError(-2, "weight dim[1] must equal to x dim[1].")
    split = [int(v) for v in split]
    if len(split) != 4:
        raise HstuError(-2, "splitList must have 4 elements.")
    outs = [torch.empty(m, w, dtype=x.dtype, device=x.device) for w in split]
    lin = torch.empty(m, n, dtype=x.dtype, device=x.device)
    a.x, a.weight = x.data_ptr(), weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.user, a.value, a.query, a.key = (o.data_ptr() for o in outs)
    a.linear_output = lin.data_ptr()
    a.m, a.n, a.k = m, n, k
    for i in range(4):
        a.split[i] = split[i]
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        check(load().ops_rec_in_linear_silu_fwd(C.byref(a), stream))
    return (*outs, lin)


def in_linear_silu_backward(x, weight, bias, user_grad, value_grad, query_grad, key_grad, linear_output, split):
    """(x_grad, weight_grad, bias_grad or None) through ops_rec_in_linear_silu_bwd on CUDA tensors (argument order of
    ops_rec::in_linear_silu_backward).  bias only says whether bias_grad is wanted."""
    import torch
    ts = [t.contiguous() for t in (x, weight, user_grad, value_grad, query_grad, key_grad, linear_output)]
    x, weight = ts[0], ts[1]
    x_grad, w_grad = torch.empty_like(x), torch.empty_like(weight)
    b_grad = torch.empty(weight.shape[0], dtype=torch.float32, device=x.device) if bias is not None else None
    a = OpsRecInLinearSiluBwdArgs()
    a.struct_bytes = C.sizeof(OpsRecInLinearSiluBwdArgs)
    a.dtype = _dtype_code(x.dtype)
    a.x, a.weight = x.data_ptr(), weight.data_ptr()
    a.user_grad, a.value_grad, a.query_grad, a.key_grad = (t.data_ptr() for t in ts[2:6])
    a.linear_output = ts[6].data_ptr()
    a.x_grad, a.weight_grad = x_grad.data_ptr(), w_grad.data_ptr()
    a.bias_grad = b_grad.data_ptr() if b_grad is not None else None
    a.m, a.n, a.k = x.shape[0], weight.shape[0], x.shape[1]
    a.split = (C.c_int32 * 4)(*[int(s) for s in split])
    n = C.c_uint64(0)
    check(load().ops_rec_in_linear_silu_bwd_get_workspace_size(C.byref(a), C.byref(n)))
    ws = torch.empty(n.value, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(load().ops_rec_in_linear_silu_bwd(C.byref(a), ws.data_ptr(), n.value,
                                                torch.cuda.current_stream(x.device).cuda_stream))
    del ts
    return x_grad, w_grad, b_grad


def ln_mul(x, u, gamma, beta):
    """(LayerNorm(x) * gamma + beta) * u through ops_rec_ln_mul_f32 on fp32 CUDA tensors (argument order of
    ops_rec::ln_mul, ascendc/activation/ln_mul/torch_extension/ln_mul_plugin.cpp:28-55)."""
    import torch
    if x.dim() != 2 or u.dim() != 2:
        raise HstuError(-2, "The x should be 2D")
    if not x.is_cuda:
        raise HstuError(-2, "tensors must live on a CUDA device; there is no CPU implementation")
    if x.dtype != torch.float32:
        raise HstuError(-2, "ln_mul supports float32 only")
    x, u, gamma, beta = x.contiguous(), u.contiguous(), gamma.contiguous(), beta.contiguous()
    out = torch.empty_like(x)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        check(load().ops_rec_ln_mul_f32(x.data_ptr(), u.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                        x.shape[0], x.shape[1], stream))
    return out


def hstu_jagged_forward_static(q, k, v, out, mask=None, attn_bias=None, mask_type=0, max_seq_len=0, silu_scale=0.0,
                               seq_offset=None, num_context=None, num_target=None, target_group_size=0, alpha=1.0,
                               *, max_seq_len_k=None, seq_offset_k=None, flags=0, return_status=False):
    """The operator through hstu_jagged_fwd_static: no workspace, nothing allocated by the call.  `out` must be
    preallocated by the caller ([total_q, heads_q, dim_v], q's dtype); inputs must already be contiguous.
    Raises HstuError(E_SCRATCH_LIMIT) when the work list does not fit the library's built-in scratch block.
    With return_status the device status word is read back through hstu_jagged_fwd_static_status (this waits)."""
    import torch
    args, keep = make_args(q, k, v, out, seq_offset, seq_offset_k=seq_offset_k, mask=mask, attn_bias=attn_bias,
                           mask_type=mask_type, max_seq_len=max_seq_len, max_seq_len_k=max_seq_len_k,
                           silu_scale=silu_scale, num_context=num_context, num_target=num_target,
                           target_group_size=target_group_size, alpha=alpha, flags=flags)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        rc = load().hstu_jagged_fwd_static(C.byref(args), stream)
    check(rc)
    if return_status:
        st = C.c_uint32(0)
        with torch.cuda.device(q.device):
            check(load().hstu_jagged_fwd_static_status(stream, C.byref(st)))
        del keep
        return out, st.value
    del keep
    return out


def plan_host(seq_offset, heads_q, *, num_context=None, num_target=None, max_seq_len=20480, dim=128,
              dtype_code=DTYPE_BF16, mask_type=0, total_q=None, count_only=False):
    """Run the scheduler's ordering rule on host arrays; returns (items[n,2] uint32, status), or with count_only
    (number of items the offsets describe, status).  total_q defaults to the last offset."""
    off = np.ascontiguousarray(np.asarray(seq_offset, dtype=np.int64))
    a = HstuJaggedArgs()
    a.struct_bytes = C.sizeof(HstuJaggedArgs)
    a.dtype = dtype_code
    a.index_bytes = 8
    a.batch = len(off) - 1
    a.total_q = a.total_k = int(off[-1]) if total_q is None else int(total_q)
    a.heads_q = a.heads_k = heads_q
    a.dim_qk = a.dim_v = dim
    a.mask_type = mask_type
    a.max_seq_len_q = a.max_seq_len_k = max_seq_len
    a.alpha = 1.0
    ctx = np.ascontiguousarray(np.asarray(num_context, dtype=np.int64)) if num_context is not None else None
    tgt = np.ascontiguousarray(np.asarray(num_target, dtype=np.int64)) if num_target is not None else None
    cap = heads_q * (int(a.total_q) // 256 + a.batch) + 1
    items = np.zeros((cap, 2), dtype=np.uint32)
    st = C.c_uint32(0)
    n = check(load().hstu_plan_host(
        C.byref(a), off.ctypes.data, None, ctx.ctypes.data if ctx is not None else None,
        tgt.ctypes.data if tgt is not None else None, items.ctypes.data, cap, C.byref(st)))
    if count_only:
        return n, st.value
    return items[:min(n, cap)], st.value


def debug_mask(len_q, len_k, ctx, tgt, group, mask_type=0):
    out = np.zeros((len_q, len_k), dtype=np.uint8)
    check(load().hstu_debug_mask_host(len_q, len_k, ctx, tgt, group, mask_type, out.ctypes.data))
    return out.astype(bool)


def debug_tiles(len_q, len_k, ctx, tgt, group, mask_type, r0, rows, bn):
    bits = C.c_uint64(0)
    n = check(load().hstu_debug_tiles_host(len_q, len_k, ctx, tgt, group, mask_type, r0, rows, bn, C.byref(bits)))
    return n, bits.value
