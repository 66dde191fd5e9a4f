"""in_linear_silu (forward): the oracle against the reference golden's outputs (CPU), the tensor-core kernel through the
C ABI and the torch operator against the oracle (GPU).  Input recipe, shapes and tolerances follow the reference test
in_linear_silu_forward/test/pytest/test_in_linear_silu.py:59-100 (fp16 1e-3, bf16 5e-3; integer x in [-100, 100],
xavier-uniform weight, bias of ones; n a multiple of 4 k)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import in_linear_silu_oracle as IO
from tests._util import GOLDEN_DIR, load_fixture

FIXTURES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "linsilu_*.npz"))
                  if "linsilu_bwd_" not in p)
NAMES = ("user", "value", "query", "key", "linear_output")
TOL = {torch.float16: 1e-3, torch.bfloat16: 5e-3}


def _close(got, want, dtype, label):
    # the reference's criterion (compare_result, test_in_linear_silu.py:59-70), plus one unit in the last place of
    # the 16-bit format for values that sit on a rounding boundary
    tol = TOL[dtype]
    g, w = got.float(), want.float()
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    bad = (g - w).abs() > tol + tol * w.abs() + ulp * w.abs()
    assert not bad.any(), (label, int(bad.sum()), float((g - w).abs().max()))


def _case(m, n, k, dtype, split=None, seed=0, bias=True):
    gen = torch.Generator().manual_seed(seed + m + n + k)
    q = n // 4
    split = split or ([q] * 4 if q < 32 else [q - 16, q - 16, q + 16, q + 16])
    x = torch.randint(-100, 101, (m, k), generator=gen).to(dtype)
    bound = (6.0 / (n + k)) ** 0.5
    w = ((torch.rand(n, k, generator=gen) * 2 - 1) * bound).to(dtype)
    b = torch.ones(n) if bias else None
    return x, w, b, split


@pytest.mark.parametrize("name", FIXTURES)
def test_oracle_matches_the_reference_golden(name):
    fx = load_fixture(name)
    split = [int(v) for v in fx["split"]]
    got = IO.in_linear_silu(fx["x"], fx["weight"], fx["bias"], split)
    for g, key in zip(got, NAMES):
        assert g.shape == fx[key].shape and g.dtype == fx[key].dtype
        _close(g, fx[key], g.dtype, f"{name} {key}")


def test_fixture_set_is_complete():
    assert len(FIXTURES) == 4


def _gpu(x, w, b, split):
    from ops_rec_b200 import cabi
    outs = cabi.in_linear_silu(x.cuda(), w.cuda(), b.cuda() if b is not None else None, split)
    torch.cuda.synchronize()
    return [o.cpu() for o in outs]


@pytest.mark.gpu
@pytest.mark.parametrize("name", FIXTURES)
def test_gpu_against_the_reference_golden(name):
    fx = load_fixture(name)
    split = [int(v) for v in fx["split"]]
    got = _gpu(fx["x"], fx["weight"], fx["bias"], split)
    for g, key in zip(got, NAMES):
        _close(g, fx[key], g.dtype, f"{name} {key}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(1, 64, 16), (100, 64, 16), (127, 128, 32), (128, 256, 64), (129, 512, 128),
                                   (300, 1024, 256), (1000, 2048, 512), (257, 4096, 1024), (64, 320, 80)])
def test_gpu_grid_against_the_oracle(m, n, k, dtype):
    x, w, b, split = _case(m, n, k, dtype)
    got = _gpu(x, w, b, split)
    want = IO.in_linear_silu(x, w, b, split)
    for g, t, name in zip(got, want, NAMES):
        assert g.shape == t.shape and g.dtype == dtype
        _close(g, t, dtype, f"{m}x{n}x{k} {name}")
    # against the unrounded fp64 result: within the rounding of the 16-bit output
    exact = IO.in_linear_silu(x, w, b, split, exact=True)
    for g, t, name in zip(got, exact, NAMES):
        rel = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
        assert ((g.double() - t).abs() <= 2 * rel * t.abs() + 1e-2).all(), name


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,split", [
    (300, 256, 16, [16, 48, 80, 112]),        # split boundaries at odd multiples of 16: inside a 32-column store chunk
    (10300, 1024, 64, None),                  # 41 x 4 = 164 tiles on 148 persistent CTAs: some walk two tiles
    (40000, 512, 128, [64, 64, 192, 192]),    # 157 x 2 = 314 tiles: every CTA walks two or three
])
def test_gpu_persistent_tiles_and_split_boundaries(m, n, k, split):
    x, w, b, split = _case(m, n, k, torch.bfloat16, split=split, seed=5)
    got = _gpu(x, w, b, split)
    want = IO.in_linear_silu(x, w, b, split)
    for g, t, name in zip(got, want, NAMES):
        assert g.shape == t.shape
        _close(g, t, torch.bfloat16, f"{m}x{n}x{k} {name}")


@pytest.mark.gpu
def test_gpu_no_bias_even_split_torch_operator_and_errors():
    import ops_rec_b200 as ops_rec
    from ops_rec_b200 import cabi
    x, w, b, split = _case(200, 512, 128, torch.bfloat16, split=[128, 128, 128, 128], bias=False)
    got = _gpu(x, w, None, split)
    want = IO.in_linear_silu(x, w, None, split)
    for g, t, name in zip(got, want, NAMES):
        _close(g, t, torch.bfloat16, name)
    op = ops_rec.ascendc.activation.distance_in_linear_silu
    x, w, b, split = _case(77, 256, 64, torch.float16)
    res = op(x.cuda(), w.cuda(), b.cuda(), split)
    for g, t, name in zip(res, IO.in_linear_silu(x, w, b, split), NAMES):
        _close(g.cpu(), t, torch.float16, name)
    with pytest.raises(RuntimeError, match="sum"):
        op(x.cuda(), w.cuda(), b.cuda(), [64, 64, 64, 16])
    with pytest.raises(RuntimeError, match="multiple of 4"):
        op(x.cuda(), w[:128].cuda(), b[:128].cuda(), [32, 32, 32, 32])
    with pytest.raises(cabi.HstuError, match="uvqk dim"):
        cabi.in_linear_silu(x.cuda(), w.cuda(), b.cuda(), [8, 120, 64, 64])
