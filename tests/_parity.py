"""Parity assertions shared by the GPU tests: CUDA result (through the C ABI) against the CPU oracle."""
from __future__ import annotations

import torch

from oracle import hstu_oracle as O
from ops_rec_b200 import cabi


def to_cuda(args):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in args.items()}


def run_cabi(args, **extra):
    """Operator through the C ABI on cuda:0; returns (out_cpu, status)."""
    out, status = cabi.hstu_jagged_forward(**to_cuda(args), **extra, return_status=True)
    torch.cuda.synchronize()
    return out.cpu(), status


def assert_parity(out, args, *, label=""):
    """bf16/fp16: rtol = atol = 1e-2 against the fp32-accumulated oracle, the reference's double-reference
    rule (x5) and its outlier-fraction criterion, plus an error bound relative to the output scale (the
    absolute tolerances alone are loose when outputs are small).  fp32: 1e-5."""
    dtype = args["q"].dtype
    ref32 = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32)
    assert out.shape == ref32.shape and out.dtype == dtype, label
    assert torch.isfinite(out.float()).all(), label
    scale = max(ref32.abs().max().item(), 1e-30)
    err = (out.float() - ref32).abs().max().item()
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref32, rtol=1e-5, atol=1e-5, msg=lambda m: f"{label}: {m}")
        assert err <= 2e-5 * scale, (label, err, scale)
        return
    lowp = O.hstu_jagged_forward(**args)  # P and O rounded to the input dtype, like the reference kernel
    torch.testing.assert_close(out.float(), ref32, rtol=1e-2, atol=1e-2, msg=lambda m: f"{label}: {m}")
    ok, detail = O.double_reference_ok(out, lowp, ref32, multiplier=5)
    assert ok, (label, detail)
    atol, ratio = (5e-3, 5e-3) if dtype == torch.bfloat16 else (1e-3, 1e-3)  # test_hstu_jagged.py:216-225
    assert O.outlier_fraction_ok(out, lowp, atol, ratio), label
    assert err <= (2e-2 if dtype == torch.bfloat16 else 4e-3) * scale, (label, err, scale)
