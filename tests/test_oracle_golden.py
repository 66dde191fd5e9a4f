"""The CPU oracle against the outputs of the reference's own goldens (tests/golden/*.npz).

Fixtures were produced by tests/golden/make_golden.py from
  hstu_v2/test/pytest/backend/pytorch_native_backend.py:48-86   (torch golden with alpha / rab / mask)
  hstu_forward_v1/test/pytest/common.py:118-137,189-252         (numpy golden, create_causal_mask)
"""
import numpy as np
import pytest
import torch

from oracle import hstu_oracle as O
from tests._util import GOLDEN_DIR, fixture_call_args, fixture_names, load_fixture


@pytest.mark.parametrize("name", fixture_names())
def test_oracle_matches_reference_goldens(name):
    fx = load_fixture(name)
    args = fixture_call_args(fx)
    got = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32)
    ref = fx["out_v2_fp32"]
    assert got.shape == ref.shape
    # fp32 tolerance of the build target (1e-5), relative to the output scale
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-6)
    if "out_v1_numpy" in fx:
        torch.testing.assert_close(got, fx["out_v1_numpy"].float(), rtol=1e-5, atol=1e-6)
    if "out_v2_lowp" in fx:
        # low precision: the oracle's rounded-P result must satisfy the reference's own acceptance rule
        low = O.hstu_jagged_forward(**args)
        ok, detail = O.double_reference_ok(low, fx["out_v2_lowp"], ref, multiplier=5)
        assert ok, detail
        torch.testing.assert_close(low.float(), ref, rtol=1e-2, atol=1e-2)


def test_fp64_oracle_agrees():
    fx = load_fixture("fp32_ctx_target_g3")
    args = fixture_call_args(fx)
    a = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32)
    b = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float64, compute_dtype=torch.float64)
    torch.testing.assert_close(a.double(), b, rtol=1e-5, atol=1e-7)


def test_mask_grid_matches_reference_create_causal_mask():
    raw = np.load(GOLDEN_DIR + "/mask_grid.npz")
    grid = raw["grid"]
    assert len(grid) > 200
    for lq, lk, c, t, g in grid.tolist():
        want = np.unpackbits(raw[f"m_{lq}_{lk}_{c}_{t}_{g}"])[: lq * lk].reshape(lq, lk).astype(bool)
        got = O.hstu_mask(lq, lk, c, t, g, 0)
        assert np.array_equal(got, want), (lq, lk, c, t, g)


def test_alpha_is_applied_after_the_bias():
    # the ordering every reference golden with alpha uses: silu(alpha * (QK^T + rab))
    fx = load_fixture("fp32_rab_alpha")
    args = fixture_call_args(fx)
    after = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32)
    before = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32, alpha_before_bias=True)
    torch.testing.assert_close(after, fx["out_v2_fp32"], rtol=1e-5, atol=1e-6)
    assert (before - fx["out_v2_fp32"]).abs().max() > 1e-3


def test_empty_and_padded_offsets():
    fx = load_fixture("cfg1_fp32_causal")
    args = fixture_call_args(fx)
    base = O.hstu_jagged_forward(**args)
    # trailing repeated offsets (the reference tests pad this way, test_hstu_jagged.py:58-61) change nothing
    off = args["seq_offset"]
    padded = torch.cat([off, off[-1:], off[-1:]])
    args2 = dict(args, seq_offset=padded, seq_offset_k=padded)
    torch.testing.assert_close(O.hstu_jagged_forward(**args2), base, rtol=0, atol=0)
    # an empty sequence in the middle
    mid = torch.cat([off[:2], off[1:]])
    args3 = dict(args, seq_offset=mid, seq_offset_k=mid)
    torch.testing.assert_close(O.hstu_jagged_forward(**args3), base, rtol=0, atol=0)


# ---------------------------------------------------------------------------------------------- backward
# Fixtures: outputs of the reference's autograd golden (hstu_backward_v1/test/pytest/test_hstu_jagged_backward.py
# :160-223, TestHstuJaggedDemo.pytorch_hstu_mha), produced by tests/golden/make_golden.py.
from tests._util import bwd_fixture_names  # noqa: E402


@pytest.mark.parametrize("name", bwd_fixture_names())
def test_backward_oracle_matches_reference_autograd_golden(name):
    fx = load_fixture(name)
    args = fixture_call_args(fx)
    got = O.hstu_jagged_backward(fx["grad"], **args, round_mid=False, out_dtype=torch.float32)
    for g, key in zip(got, ("dq_fp32", "dk_fp32", "dv_fp32", "dbias_fp32")):
        if key not in fx:
            assert g is None
            continue
        assert g.shape == fx[key].shape
        torch.testing.assert_close(g, fx[key], rtol=1e-5, atol=2e-6, msg=lambda m: f"{key}: {m}")
    if "dq_lowp" in fx:
        # low precision: the rounded-intermediate oracle passes the reference's own acceptance rule (x5)
        low = O.hstu_jagged_backward(fx["grad"], **args)
        for g, key in zip(low, ("dq", "dk", "dv", "dbias")):
            ok, detail = O.double_reference_ok(g, fx[key + "_lowp"], fx[key + "_fp32"], multiplier=5)
            assert ok, (key, detail)


def test_backward_oracle_is_the_gradient_of_the_forward_oracle():
    fx = load_fixture("bwd_fp32_rab_gqa_ctx_target")
    args = fixture_call_args(fx)
    leaves = {n: args[n].double().requires_grad_(True) for n in ("q", "k", "v", "attn_bias")}
    out = O.hstu_jagged_forward(**dict(args, **leaves), round_p=False, compute_dtype=torch.float64)
    want = torch.autograd.grad(out, list(leaves.values()), fx["grad"].double())
    got = O.hstu_jagged_backward(fx["grad"].double(), **dict(args, **{n: t.detach() for n, t in leaves.items()}),
                                 round_mid=False, compute_dtype=torch.float64)
    for w, g in zip(want, got):
        torch.testing.assert_close(g, w, rtol=1e-10, atol=1e-12)
