"""Generate the golden fixtures in this directory by running the REFERENCE's own goldens.

Run once, in a container that has the reference tree (it is not needed at test time):

    python tests/golden/make_golden.py /path/to/ops-rec

Two reference goldens are executed on small seeded inputs and their outputs stored as .npz:

  * `get_golden_jagged` (numpy, fp32, per-sequence loop; no alpha) from
    ascendc/attention/hstu_v1/hstu_forward_v1/test/pytest/common.py:189-252 -- imported as a module with a
    stand-in for the `torch.npu` attribute it touches at import time (common.py:28);
  * `PytorchNative.kernel(...)._forward_impl` (torch, pads to dense; has alpha and rab) from
    ascendc/attention/hstu_v2/test/pytest/backend/pytorch_native_backend.py:48-86 -- loaded by file path under a
    synthetic package so the NPU-only sibling backends are never imported; its mask input is built with
    `create_causal_mask` of the same reference file set (common.py:128-137).

Every fixture stores the inputs too, so the tests need nothing but numpy/torch.  bf16 arrays are stored as
their uint16 bit patterns (key suffix `__bf16`).
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_reference(ref_root):
    v1 = os.path.join(ref_root, "ascendc/attention/hstu_v1/hstu_forward_v1/test/pytest")
    v2 = os.path.join(ref_root, "ascendc/attention/hstu_v2/test/pytest/backend")
    if not hasattr(torch, "npu"):
        torch.npu = types.SimpleNamespace(config=types.SimpleNamespace())
    spec = importlib.util.spec_from_file_location("ref_v1_common", os.path.join(v1, "common.py"))
    v1c = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(v1c)
    pkg = types.ModuleType("ref_v2_backend")
    pkg.__path__ = [v2]
    sys.modules["ref_v2_backend"] = pkg
    for name in ("common", "pytorch_native_backend"):
        spec = importlib.util.spec_from_file_location(f"ref_v2_backend.{name}", os.path.join(v2, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"ref_v2_backend.{name}"] = mod
        spec.loader.exec_module(mod)
    return v1c, sys.modules["ref_v2_backend.pytorch_native_backend"]


def _store(path, arrays):
    out = {}
    for key, val in arrays.items():
        if val is None:
            continue
        if isinstance(val, torch.Tensor):
            if val.dtype == torch.bfloat16:
                out[key + "__bf16"] = val.view(torch.int16).numpy().view(np.uint16)
                continue
            val = val.numpy()
        out[key] = np.asarray(val)
    np.savez_compressed(path, **out)


# name, B, Hq, Hk, Dqk, Dv, maxL, len range, dtype, alpha, rab, ctx, target, group, mask_type, delta
CASES = [
    # BASELINE config 1: B4 H2 d32 fp32, L ~ U[1,128] seed 0, alpha 1/32, causal, no rab
    dict(name="cfg1_fp32_causal", B=4, Hq=2, Hk=2, Dqk=32, Dv=32, maxL=128, lo=1, hi=128, dtype="fp32",
         alpha=1.0 / 32, rab=False, ctx=0, tgt=0, g=0, mask_type=0, numpy_rng_lengths=True),
    dict(name="fp32_rab_alpha", B=3, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=40, lo=1, hi=40, dtype="fp32",
         alpha=0.37, rab=True, ctx=0, tgt=0, g=0, mask_type=0),
    dict(name="fp32_target_g1", B=3, Hq=2, Hk=2, Dqk=16, Dv=32, maxL=70, lo=1, hi=30, dtype="fp32",
         alpha=1.0, rab=True, ctx=0, tgt=30, g=1, mask_type=0),
    dict(name="fp32_ctx_target_g3", B=4, Hq=4, Hk=2, Dqk=32, Dv=16, maxL=80, lo=1, hi=40, dtype="fp32",
         alpha=0.5, rab=False, ctx=6, tgt=30, g=3, mask_type=0),
    dict(name="fp32_ctx_only", B=2, Hq=2, Hk=1, Dqk=16, Dv=16, maxL=50, lo=1, hi=40, dtype="fp32",
         alpha=1.0, rab=True, ctx=6, tgt=0, g=1, mask_type=0),
    dict(name="fp32_target_g0", B=2, Hq=1, Hk=1, Dqk=16, Dv=16, maxL=50, lo=1, hi=30, dtype="fp32",
         alpha=1.0, rab=False, ctx=0, tgt=9, g=0, mask_type=0),
    dict(name="fp32_mask_none", B=3, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=33, lo=1, hi=33, dtype="fp32",
         alpha=0.25, rab=True, ctx=0, tgt=0, g=0, mask_type=2),
    dict(name="fp32_mask_custom", B=2, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=29, lo=1, hi=29, dtype="fp32",
         alpha=1.0, rab=False, ctx=0, tgt=0, g=0, mask_type=3),
    dict(name="fp32_delta", B=3, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=48, lo=1, hi=48, dtype="fp32",
         alpha=0.3, rab=True, ctx=0, tgt=0, g=0, mask_type=0, delta=True),
    dict(name="bf16_d128_rab_target", B=3, Hq=2, Hk=2, Dqk=128, Dv=128, maxL=300, lo=100, hi=260, dtype="bf16",
         alpha=1.0 / 128, rab=True, ctx=0, tgt=17, g=1, mask_type=0),
    dict(name="bf16_d64_gqa", B=4, Hq=4, Hk=2, Dqk=64, Dv=64, maxL=200, lo=1, hi=200, dtype="bf16",
         alpha=1.0 / 64, rab=False, ctx=0, tgt=0, g=0, mask_type=0),
]


def build_case(case, v1c, v2b):
    torch.manual_seed(1234 + len(case["name"]))
    rng = np.random.default_rng(0)
    B, Hq, Hk, Dqk, Dv, maxL = (case[k] for k in ("B", "Hq", "Hk", "Dqk", "Dv", "maxL"))
    dtype = torch.float32 if case["dtype"] == "fp32" else torch.bfloat16
    ctx, tgt, g = case["ctx"], case["tgt"], case["g"]
    base = rng.integers(case["lo"], case["hi"] + 1, B)
    len_k = base + (ctx + tgt if case["mask_type"] == 0 else 0)
    if case.get("delta"):
        len_q = np.maximum(1, len_k - rng.integers(0, 9, B))
    else:
        len_q = len_k.copy()
    assert len_k.max() <= maxL
    offq = np.concatenate([[0], np.cumsum(len_q)]).astype(np.int64)
    offk = np.concatenate([[0], np.cumsum(len_k)]).astype(np.int64)
    scale_in = 1.0 if case["dtype"] == "fp32" else 0.5
    q = (torch.randn(int(offq[-1]), Hq, Dqk) * scale_in).to(dtype)
    k = (torch.randn(int(offk[-1]), Hk, Dqk) * scale_in).to(dtype)
    v = (torch.randn(int(offk[-1]), Hk, Dv) * scale_in).to(dtype)
    rab = (torch.randn(B, Hq, maxL, maxL) * (1.0 if case["dtype"] == "fp32" else 0.1)).to(dtype) \
        if case["rab"] else None
    num_context = np.full(B, ctx, dtype=np.int64)
    num_target = np.full(B, tgt, dtype=np.int64)
    mask = None
    if case["mask_type"] == 3:
        mask = torch.randint(0, 2, (B, Hq, maxL, maxL)).to(dtype)

    # dense mask tensor the v2 golden multiplies by (reference semantics, reference code)
    dense_mask = None
    if case["mask_type"] == 0:
        dense_mask = torch.zeros(B, Hq, maxL, maxL)
        for b in range(B):
            lq, lk = int(len_q[b]), int(len_k[b])
            dense_mask[b, :, :lq, :lk] = v1c.create_causal_mask(lq, lk, ctx or None, tgt or None, g or None)
    elif case["mask_type"] == 3:
        dense_mask = mask.float()

    # golden A: v2 torch golden in fp32 (alpha, rab, mask) -- the fp32-accumulated reference
    kern = v2b.PytorchNative.kernel(case["alpha"], 0.0, rab is not None, maxL, maxL,
                                    torch.from_numpy(offq), torch.from_numpy(offk))
    with torch.enable_grad():
        out_v2_fp32 = kern._forward_impl(q.float().clone(), k.float().clone(), v.float().clone(),
                                         rab.float().clone() if rab is not None else None,
                                         dense_mask).detach()
    arrays = dict(q=q, k=k, v=v, rab=rab, mask=mask, seq_offset=offq, seq_offset_k=offk,
                  num_context=num_context, num_target=num_target,
                  meta=np.array([B, Hq, Hk, Dqk, Dv, maxL, ctx, tgt, g, case["mask_type"]], dtype=np.int64),
                  alpha=np.float64(case["alpha"]), out_v2_fp32=out_v2_fp32)
    # golden B: v2 torch golden in the input dtype (low-precision side of the double-reference rule)
    if dtype != torch.float32:
        kern2 = v2b.PytorchNative.kernel(case["alpha"], 0.0, rab is not None, maxL, maxL,
                                         torch.from_numpy(offq), torch.from_numpy(offk))
        with torch.enable_grad():
            arrays["out_v2_lowp"] = kern2._forward_impl(
                q.clone(), k.clone(), v.clone(), rab.clone() if rab is not None else None,
                dense_mask.to(dtype) if dense_mask is not None else None).detach()
    # golden C: v1 numpy golden (no alpha => only comparable when alpha == 1)
    if case["alpha"] == 1.0:
        out_v1 = v1c.get_golden_jagged(
            q.float().numpy(), k.float().numpy(), v.float().numpy(),
            mask=mask.float().numpy() if mask is not None else None,
            attn_bias=rab.float().numpy() if rab is not None else None,
            mask_type=case["mask_type"], max_seq_len=maxL, silu_scale=0.0, seq_offset=offq, seq_offset_k=offk,
            num_context=num_context if ctx else None, num_target=num_target if tgt else None,
            target_group_size=g)
        arrays["out_v1_numpy"] = out_v1
    return arrays


def _load_reference_backward(ref_root):
    """The reference's backward golden: TestHstuJaggedDemo.pytorch_hstu_mha (autograd through the padded dense
    forward) from ascendc/attention/hstu_v1/hstu_backward_v1/test/pytest/test_hstu_jagged_backward.py:160-223.
    The file imports the NPU packages at module level; empty stand-ins satisfy those imports, the golden itself is
    pure torch."""
    d = os.path.join(ref_root, "ascendc/attention/hstu_v1/hstu_backward_v1/test/pytest")
    for name in ("torch_npu", "ops_rec"):
        sys.modules.setdefault(name, types.ModuleType(name))
    # its helper module sets the NPU device at import time (test_common_utils.py:30-32)
    torch.npu = types.SimpleNamespace(config=types.SimpleNamespace(), set_device=lambda *_: None)
    sys.path.insert(0, d)
    try:
        spec = importlib.util.spec_from_file_location("ref_bwd_test", os.path.join(d, "test_hstu_jagged_backward.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        sys.path.remove(d)
    return mod


# name, B, Hq, Hk, Dqk, Dv, maxL, dtype, alpha, silu_scale, rab, ctx, tgt, g, mask_type, delta
BWD_CASES = [
    dict(name="bwd_fp32_causal", B=3, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=40, dtype="fp32", alpha=0.5, silu_scale=0.0,
         rab=False, ctx=0, tgt=0, g=0, mask_type=0),
    dict(name="bwd_fp32_rab_gqa_ctx_target", B=3, Hq=4, Hk=2, Dqk=24, Dv=16, maxL=70, dtype="fp32", alpha=0.37,
         silu_scale=1.0 / 256, rab=True, ctx=3, tgt=20, g=3, mask_type=0),
    dict(name="bwd_fp32_delta_rab", B=3, Hq=2, Hk=1, Dqk=16, Dv=32, maxL=48, dtype="fp32", alpha=0.5, silu_scale=0.0,
         rab=True, ctx=0, tgt=0, g=0, mask_type=0, delta=True),
    dict(name="bwd_fp32_mask_none", B=2, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=33, dtype="fp32", alpha=0.25,
         silu_scale=0.0, rab=True, ctx=0, tgt=0, g=0, mask_type=2),
    dict(name="bwd_fp32_mask_custom", B=2, Hq=2, Hk=2, Dqk=16, Dv=16, maxL=29, dtype="fp32", alpha=1.0,
         silu_scale=0.0, rab=True, ctx=0, tgt=0, g=0, mask_type=3),
    dict(name="bwd_bf16_d64_rab_target", B=3, Hq=2, Hk=2, Dqk=64, Dv=64, maxL=96, dtype="bf16", alpha=0.5,
         silu_scale=0.0, rab=True, ctx=0, tgt=9, g=1, mask_type=0),
]


def build_bwd_case(case, v1c, ref_bwd):
    torch.manual_seed(4321 + len(case["name"]))
    rng = np.random.default_rng(7)
    B, Hq, Hk, Dqk, Dv, maxL = (case[k] for k in ("B", "Hq", "Hk", "Dqk", "Dv", "maxL"))
    dtype = torch.float32 if case["dtype"] == "fp32" else torch.bfloat16
    ctx, tgt, g = case["ctx"], case["tgt"], case["g"]
    lo = 1 + ctx + tgt
    len_k = rng.integers(lo, maxL + 1, B)
    len_q = np.maximum(lo, len_k - rng.integers(0, 9, B)) if case.get("delta") else len_k.copy()
    offq = np.concatenate([[0], np.cumsum(len_q)]).astype(np.int64)
    offk = np.concatenate([[0], np.cumsum(len_k)]).astype(np.int64)
    # value ranges of the reference's own generator (jagged_data_gen, :58-63): uniform(-1, 1)
    grad = torch.empty(int(offq[-1]), Hq, Dv).uniform_(-1, 1).to(dtype)
    q = torch.empty(int(offq[-1]), Hq, Dqk).uniform_(-1, 1).to(dtype)
    k = torch.empty(int(offk[-1]), Hk, Dqk).uniform_(-1, 1).to(dtype)
    v = torch.empty(int(offk[-1]), Hk, Dv).uniform_(-1, 1).to(dtype)
    rab = torch.empty(B, Hq, maxL, maxL).uniform_(-1, 1).to(dtype)
    mask = torch.randint(0, 2, (B, Hq, maxL, maxL)).to(dtype) if case["mask_type"] == 3 else None
    dense_mask = None
    if case["mask_type"] == 0:
        dense_mask = torch.zeros(B, Hq, maxL, maxL)
        for b in range(B):
            lq, lk = int(len_q[b]), int(len_k[b])
            dense_mask[b, :, :lq, :lk] = v1c.create_causal_mask(lq, lk, ctx or None, tgt or None, g or None)
    elif case["mask_type"] == 3:
        dense_mask = mask.float()

    def golden(dt):
        m = dense_mask.to(dt) if dense_mask is not None else None
        res = ref_bwd.TestHstuJaggedDemo.pytorch_hstu_mha(
            maxL, case["alpha"], grad.to(dt), q.to(dt).clone(), k.to(dt).clone(), v.to(dt).clone(),
            torch.from_numpy(offq), torch.from_numpy(offk), m, rab.to(dt).clone(), case["rab"], case["silu_scale"])
        return [r.detach() if r is not None else None for r in res]

    dq32, dk32, dv32, db32 = golden(torch.float32)
    arrays = dict(grad=grad, q=q, k=k, v=v, rab=rab if case["rab"] else None, mask=mask, seq_offset=offq,
                  seq_offset_k=offk, num_context=np.full(B, ctx, dtype=np.int64),
                  num_target=np.full(B, tgt, dtype=np.int64),
                  meta=np.array([B, Hq, Hk, Dqk, Dv, maxL, ctx, tgt, g, case["mask_type"]], dtype=np.int64),
                  alpha=np.float64(case["alpha"]), silu_scale=np.float64(case["silu_scale"]),
                  dq_fp32=dq32, dk_fp32=dk32, dv_fp32=dv32, dbias_fp32=db32)
    if dtype != torch.float32:
        dql, dkl, dvl, dbl = golden(dtype)
        arrays.update(dq_lowp=dql, dk_lowp=dkl, dv_lowp=dvl, dbias_lowp=dbl)
    return arrays


def main_backward(ref_root, v1c):
    ref_bwd = _load_reference_backward(ref_root)
    for case in BWD_CASES:
        arrays = build_bwd_case(case, v1c, ref_bwd)
        path = os.path.join(HERE, case["name"] + ".npz")
        _store(path, arrays)
        print(f"{case['name']:28s} tokens_q={arrays['q'].shape[0]:5d} {os.path.getsize(path) / 1024:8.1f} KiB")


LNMUL_SHAPES = [(1, 1), (8, 64), (33, 100), (4, 1024), (2, 2048), (3, 4100), (1, 9000)]


def main_ln_mul(ref_root):
    """ln_mul fixtures from the reference's numpy golden, ascendc/activation/ln_mul/test/pytest/test_ln_mul.py:37-50
    (`get_golden`).  The test module imports the NPU package and touches torch.npu at import time; stand-ins
    satisfy that, the golden itself is pure numpy."""
    d = os.path.join(ref_root, "ascendc/activation/ln_mul/test/pytest")
    sys.modules.setdefault("ops_rec", types.ModuleType("ops_rec"))
    if not hasattr(torch, "npu"):
        torch.npu = types.SimpleNamespace(config=types.SimpleNamespace())
    spec = importlib.util.spec_from_file_location("ref_ln_mul_test", os.path.join(d, "test_ln_mul.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for a, r in LNMUL_SHAPES:
        rng = np.random.default_rng(1000 * a + r)
        x, u = rng.standard_normal((a, r), dtype=np.float32), rng.standard_normal((a, r), dtype=np.float32)
        gamma, beta = rng.standard_normal(r, dtype=np.float32), rng.standard_normal(r, dtype=np.float32)
        if r > 1:
            x[0] += 30.0   # a row with a large mean: the two-pass variance matters
        y = mod.get_golden(x, u, gamma, beta)
        path = os.path.join(HERE, f"lnmul_{a}x{r}.npz")
        np.savez_compressed(path, x=x, u=u, gamma=gamma, beta=beta, y=y)
        print(f"lnmul_{a}x{r:<6d} {os.path.getsize(path) / 1024:8.1f} KiB")


# m, n, k, dtype, split (None: the reference's uneven split of its diff-dim test)
LINSILU_CASES = [(100, 64, 16, "fp16", [16, 16, 16, 16]), (37, 256, 64, "bf16", None), (130, 512, 128, "bf16", None),
                 (64, 384, 96, "fp16", [96, 96, 96, 96])]


def main_in_linear_silu(ref_root):
    """in_linear_silu fixtures from the reference's torch golden, in_linear_silu_forward/test/pytest/
    test_in_linear_silu.py:36-50 (`get_user_value_query_key_tensors_uniattn`), with its input recipe (:93-97: integer
    x in [-100, 100], xavier-uniform weight, bias of ones).  Stand-ins satisfy the module-level NPU imports."""
    d = os.path.join(ref_root, "ascendc/activation/in_linear_silu/in_linear_silu_forward/test/pytest")
    sys.modules.setdefault("ops_rec", types.ModuleType("ops_rec"))
    if not hasattr(torch, "npu"):
        torch.npu = types.SimpleNamespace(config=types.SimpleNamespace())
    spec = importlib.util.spec_from_file_location("ref_in_linear_silu_test", os.path.join(d, "test_in_linear_silu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for m, n, k, dt, split in LINSILU_CASES:
        torch.manual_seed(m + n + k)
        dtype = torch.float16 if dt == "fp16" else torch.bfloat16
        q = n // 4
        split = split or [q - 16, q - 16, q + 16, q + 16]
        x = torch.randint(low=-100, high=101, size=(m, k)).to(dtype)
        w = torch.nn.init.xavier_uniform_(torch.empty(n, k)).to(dtype)
        bias = torch.ones(n, dtype=dtype)
        # the golden runs in fp32 on the 16-bit values and is rounded like an addmm in the input dtype
        outs = mod.get_user_value_query_key_tensors_uniattn(x, w, bias, split)
        arrays = dict(x=x, weight=w, bias=bias.float(), split=np.array(split, dtype=np.int64))
        for name, t in zip(("user", "value", "query", "key", "linear_output"), outs):
            arrays[name] = t
        path = os.path.join(HERE, f"linsilu_{m}x{n}x{k}_{dt}.npz")
        out = {}
        for key, val in arrays.items():
            if isinstance(val, torch.Tensor):
                if val.dtype == torch.bfloat16:
                    out[key + "__bf16"] = val.contiguous().view(torch.int16).numpy().view(np.uint16)
                    continue
                val = val.contiguous().numpy()
            out[key] = np.asarray(val)
        np.savez_compressed(path, **out)
        print(f"{os.path.basename(path):32s} {os.path.getsize(path) / 1024:8.1f} KiB")


def main_in_linear_silu_backward(ref_root):
    """in_linear_silu_backward fixtures: inputs from the reference test's `get_data` and the outputs of its two goldens,
    `ln_linear_silu_backward_golden_cpu` (fp32) and `ln_linear_silu_backward_npu` (16-bit intermediate), in
    in_linear_silu_backward/test/pytest/test_in_linear_silu_backward.py:125-195.  The module imports `ops_rec` and
    touches `torch.npu` at import time; both get empty stand-ins."""
    d = os.path.join(ref_root, "ascendc/activation/in_linear_silu/in_linear_silu_backward/test/pytest")
    torch.npu = types.SimpleNamespace(config=types.SimpleNamespace())
    sys.modules.setdefault("ops_rec", types.ModuleType("ops_rec"))
    spec = importlib.util.spec_from_file_location("ref_linsilu_bwd_test", os.path.join(d, "test_in_linear_silu_backward.py"))
    rb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rb)
    for name, m, dim, has_bias, dt, diff in (("linsilu_bwd_37x64x256_bf16", 37, (64, 256), True, torch.bfloat16, False),
                                             ("linsilu_bwd_130x128x512_fp16_diff", 130, (128, 512), True, torch.float16, True),
                                             ("linsilu_bwd_64x16x128_bf16_nobias", 64, (16, 128), False, torch.bfloat16, False)):
        torch.manual_seed(0)
        u, v, q, k, x, w, bias, lo, split = rb.get_data(m, dim[0], dim[1], has_bias, dt, diff)
        mixed = torch.cat((u, v, q, k), dim=-1)
        xg32, wg32, bg32 = rb.ln_linear_silu_backward_golden_cpu(mixed, x, w, bias, lo)
        xg16, wg16, bg16 = rb.ln_linear_silu_backward_npu(mixed, x, w, bias, lo, dt)
        as16 = (lambda t: t) if dt == torch.bfloat16 else (lambda t: t.float())   # fp16 is stored as fp32 (exact)
        arrays = dict(user_grad=as16(u), value_grad=as16(v), query_grad=as16(q), key_grad=as16(k), x=as16(x),
                      weight=as16(w), bias=bias, linear_output=as16(lo), split=np.array(split, dtype=np.int64),
                      is_fp16=np.int64(dt == torch.float16), x_grad_fp32=xg32, weight_grad_fp32=wg32, bias_grad_fp32=bg32,
                      x_grad_lowp=xg16.float(), weight_grad_lowp=wg16.float(), bias_grad_lowp=bg16)
        path = os.path.join(HERE, name + ".npz")
        _store(path, arrays)
        print(f"{name:36s} {os.path.getsize(path) / 1024:8.1f} KiB")


# name, B, heads (q, k), dim, max new history, max targets, page size, previous history in the cache, dtype, mask
PAGED_CASES = [
    dict(name="paged_fp32_p32", B=3, Hq=2, Hk=2, D=32, hist=100, cand=25, page=32, prev=False, dtype="fp32", mask_type=0),
    dict(name="paged_fp32_p128_prev", B=4, Hq=4, Hk=2, D=32, hist=200, cand=25, page=128, prev=True, dtype="fp32",
         mask_type=0),
    dict(name="paged_fp32_nocand", B=2, Hq=2, Hk=2, D=16, hist=100, cand=0, page=32, prev=True, dtype="fp32", mask_type=0),
    dict(name="paged_fp32_custom", B=2, Hq=2, Hk=1, D=16, hist=70, cand=9, page=32, prev=False, dtype="fp32", mask_type=3),
    dict(name="paged_bf16_p256", B=2, Hq=2, Hk=2, D=128, hist=200, cand=40, page=256, prev=True, dtype="bf16",
         mask_type=0),
    dict(name="paged_bf16_d64_p32", B=5, Hq=4, Hk=2, D=64, hist=200, cand=30, page=32, prev=False, dtype="bf16",
         mask_type=0),
]


def main_paged(ref_root, v1c):
    """hstu_paged fixtures.  Inputs come from the reference test's own generators and the expected outputs from its two
    goldens: the torch golden `_hstu_paged_kv_attention` (hstu_forward_v1/test/pytest/test_hstu_paged.py:203-277; has
    alpha, a cache longer than the new history, custom masks) for every case, and the numpy golden `get_golden_paged`
    (test/pytest/common.py:255-300; no alpha, cache length == history) where it applies.  test_hstu_paged.py imports
    `ops_rec` and asks `torch.npu` for a device at module / call level; both get stand-ins that run on the CPU."""
    d = os.path.join(ref_root, "ascendc/attention/hstu_v1/hstu_forward_v1/test/pytest")
    torch.npu = types.SimpleNamespace(config=types.SimpleNamespace(), current_device=lambda: "cpu",
                                      synchronize=lambda: None)
    sys.modules["common"] = v1c
    sys.modules.setdefault("ops_rec", types.ModuleType("ops_rec"))
    spec = importlib.util.spec_from_file_location("ref_paged_test", os.path.join(d, "test_hstu_paged.py"))
    rp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rp)
    for case in PAGED_CASES:
        torch.manual_seed(77 + len(case["name"]))
        dtype = torch.float32 if case["dtype"] == "fp32" else torch.bfloat16
        B, Hq, Hk, D, page = case["B"], case["Hq"], case["Hk"], case["D"], case["page"]
        # the input recipe of paged_hstu_attn_kernel (test_hstu_paged.py:373-412), with its own helper functions
        kv_data, new_hist, kv_len = rp.generate_kvdata_testcase(case["hist"], B, Hq, Hk, D, is_prev_hist=case["prev"])
        kv_data = kv_data.to(dtype)
        table, meta = rp.setup_kvcache_testcase(page, Hk, D, dtype, kv_data, kv_len, None)
        if case["cand"] > 0:
            cand = torch.randint(1, case["cand"] + 1, (B,), dtype=torch.int32)
        else:
            cand = torch.zeros((B,), dtype=torch.int32)
        seqlen = new_hist + cand
        off_q = rp.get_offsets_from_lengths(seqlen)
        off_k = rp.get_offsets_from_lengths(cand + kv_len)
        off_t = rp.get_offsets_from_lengths(cand)
        T = int(off_q[-1])
        q = torch.empty(T, Hq, D).uniform_(-1, 1).to(dtype)
        k = torch.empty(T, Hk, D).uniform_(-1, 1).to(dtype)
        v = torch.empty(T, Hk, D).uniform_(-1, 1).to(dtype)
        max_q, max_k = int(seqlen.max()), int((cand + kv_len).max())
        mask = rp.generate_attn_mask(B, Hq, max_q, max_k, dtype, seqlen, meta, page, cand, case["mask_type"])
        alpha = 1.0 / (D ** 0.5)
        page_ids = torch.tensor(meta[0], dtype=torch.int32)
        page_off = torch.tensor(meta[1], dtype=torch.int32)
        last_len = torch.tensor(meta[2], dtype=torch.int32)

        def golden(up):
            out = rp._hstu_paged_kv_attention(
                num_heads_q=Hq, num_heads_k=Hk, attention_dim=D, linear_dim=D, seqlen_q=max_q, seqlen_k=max_k,
                q=q, k=k, v=v, q_offsets=off_q, k_offsets=off_k, num_targets=cand, invalid_attn_mask=mask, upcast=up,
                kv_cache=table, page_offsets=page_off, page_ids=page_ids, last_page_lens=last_len, alpha=alpha)
            return out.view(-1, Hq, D)

        arrays = dict(q=q, k=k, v=v, kv_cache=table, mask=mask if case["mask_type"] == 3 else None,
                      seq_offset=off_q.to(torch.int64), seq_offset_k=off_k.to(torch.int64),
                      seq_offset_t=off_t.to(torch.int64), page_offsets=page_off, page_ids=page_ids,
                      last_page_len=last_len, num_target=cand.to(torch.int64), alpha=np.float64(alpha),
                      meta=np.array([B, Hq, Hk, D, page, max_q, max_k, case["mask_type"]], dtype=np.int64),
                      out_torch_fp32=golden(True).float())
        if dtype != torch.float32:
            arrays["out_torch_lowp"] = golden(False)
        if not case["prev"] and case["mask_type"] == 0 and Hq == Hk:
            # the numpy golden (equal head counts only): no alpha (scores enter SiLU as they are), explicit scale
            arrays["out_numpy_noalpha"] = v1c.get_golden_paged(
                q.float().numpy(), k.float().numpy(), v.float().numpy(), table.float().numpy(), off_q.numpy(),
                page_off.numpy(), page_ids.numpy(), last_len.numpy(), cand.numpy(), 1.0 / max_q)
        path = os.path.join(HERE, case["name"] + ".npz")
        _store(path, arrays)
        print(f"{case['name']:28s} {os.path.getsize(path) / 1024:8.1f} KiB")


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to the ops-rec tree> [backward | ln_mul | in_linear_silu | in_linear_silu_backward | paged]")
    ref_root = sys.argv[1]
    if len(sys.argv) > 2 and sys.argv[2] == "in_linear_silu_backward":
        main_in_linear_silu_backward(ref_root)
        return
    if len(sys.argv) > 2 and sys.argv[2] == "paged":            # only the hstu_paged fixtures
        v1c, _ = _load_reference(ref_root)
        main_paged(ref_root, v1c)
        return
    if len(sys.argv) > 2 and sys.argv[2] == "in_linear_silu":   # only the in_linear_silu fixtures
        main_in_linear_silu(ref_root)
        return
    if len(sys.argv) > 2 and sys.argv[2] == "ln_mul":   # only the ln_mul fixtures
        main_ln_mul(ref_root)
        return
    v1c, v2b = _load_reference(ref_root)
    if len(sys.argv) > 2 and sys.argv[2] == "backward":   # only the backward fixtures
        main_backward(ref_root, v1c)
        return
    main_backward(ref_root, v1c)
    main_ln_mul(ref_root)
    main_in_linear_silu(ref_root)
    main_in_linear_silu_backward(ref_root)
    main_paged(ref_root, v1c)
    for case in CASES:
        arrays = build_case(case, v1c, v2b)
        path = os.path.join(HERE, case["name"] + ".npz")
        _store(path, arrays)
        print(f"{case['name']:28s} tokens_q={arrays['q'].shape[0]:5d} {os.path.getsize(path) / 1024:8.1f} KiB")

    # dense layout (hstu_dense): the reference's numpy golden get_golden (common.py:160-186)
    for name, (B, S, N, D), bias_on, mask_type in [("dense_fp32_tril_bias", (2, 40, 2, 16), True, 0),
                                                    ("dense_fp32_none", (3, 17, 1, 32), False, 2),
                                                    ("dense_fp32_custom", (2, 33, 2, 16), True, 3)]:
        torch.manual_seed(99 + S)
        q, k, v = (torch.randn(B, S, N, D) for _ in range(3))
        bias = torch.randn(B, N, S, S) if bias_on else None
        mask = torch.randint(0, 2, (B, N, S, S)).float() if mask_type == 3 else None
        out = v1c.get_golden(q.numpy(), k.numpy(), v.numpy(), mask.numpy() if mask is not None else None,
                             bias.numpy() if bias is not None else None, mask_type, S, 1.0 / 256)
        path = os.path.join(HERE, name + ".npz")
        _store(path, dict(q=q, k=k, v=v, rab=bias, mask=mask, out_v1_numpy=out,
                          meta=np.array([B, S, N, D, mask_type], dtype=np.int64), silu_scale=np.float64(1.0 / 256)))
        print(f"{name:28s} {os.path.getsize(path) / 1024:8.1f} KiB")

    # mask-only fixtures: the reference's create_causal_mask over a grid incl. the boundary values its tests use
    grid = []
    masks = {}
    for (lq, lk) in [(1, 1), (7, 7), (33, 33), (64, 64), (65, 65), (40, 52), (129, 129)]:
        for c in (0, 1, 6, 31):
            for t in (0, 1, 5, 30):
                for g in (0, 1, 3):
                    if c + t > lq:
                        continue
                    m = v1c.create_causal_mask(lq, lk, c or None, t or None, g or None).numpy().astype(np.uint8)
                    key = f"m_{lq}_{lk}_{c}_{t}_{g}"
                    masks[key] = np.packbits(m, axis=None)
                    grid.append((lq, lk, c, t, g))
    masks["grid"] = np.array(grid, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "mask_grid.npz"), **masks)
    print("mask_grid", len(grid), "masks")


if __name__ == "__main__":
    main()
