"""ln_mul: the oracle against the reference golden's outputs (CPU), the CUDA kernels through the C ABI and the torch
operator against the oracle (GPU).  Shapes and tolerances follow the reference test
ascendc/activation/ln_mul/test/pytest/test_ln_mul.py:53-70 (a, r in powers of two up to 2048; rtol = atol = 1e-4)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import ln_mul_oracle as LO
from tests._util import GOLDEN_DIR

FIXTURES = sorted(glob.glob(os.path.join(GOLDEN_DIR, "lnmul_*.npz")))


def _inputs(a, r, seed=0):
    rng = np.random.default_rng(seed + 7919 * a + r)
    return (rng.standard_normal((a, r), dtype=np.float32), rng.standard_normal((a, r), dtype=np.float32),
            rng.standard_normal(r, dtype=np.float32), rng.standard_normal(r, dtype=np.float32))


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[:-4] for p in FIXTURES])
def test_oracle_matches_the_reference_golden(path):
    fx = np.load(path)
    got = LO.ln_mul(fx["x"], fx["u"], fx["gamma"], fx["beta"])
    assert got.dtype == np.float32 and got.shape == fx["y"].shape
    np.testing.assert_allclose(got, fx["y"], rtol=1e-5, atol=1e-5)


def test_fixture_set_is_complete():
    assert len(FIXTURES) == 7


def _gpu(x, u, gamma, beta):
    from ops_rec_b200 import cabi
    out = cabi.ln_mul(*(torch.from_numpy(t).cuda() for t in (x, u, gamma, beta)))
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[:-4] for p in FIXTURES])
def test_gpu_against_the_reference_golden(path):
    fx = np.load(path)
    got = _gpu(fx["x"], fx["u"], fx["gamma"], fx["beta"])
    np.testing.assert_allclose(got, fx["y"], rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("a", [1, 2, 8, 33, 256, 2048])
@pytest.mark.parametrize("r", [1, 4, 8, 16, 31, 64, 100, 128, 1000, 1024, 1025, 2048, 8192, 8193, 20000])
def test_gpu_grid_against_the_oracle(a, r):
    if a * r > 2048 * 8192:
        a = 64
    x, u, gamma, beta = _inputs(a, r)
    got = _gpu(x, u, gamma, beta)
    want64 = LO.ln_mul(x, u, gamma, beta, dtype=np.float64)
    np.testing.assert_allclose(got, want64, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(got, LO.ln_mul(x, u, gamma, beta), rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
def test_gpu_unaligned_views_and_torch_operator():
    import ops_rec_b200 as ops_rec
    x, u, gamma, beta = _inputs(37, 256, seed=3)
    want = LO.ln_mul(x, u, gamma, beta)
    xt, ut, gt, bt = (torch.from_numpy(t).cuda() for t in (x, u, gamma, beta))
    op = ops_rec.ascendc.activation.ln_mul
    np.testing.assert_allclose(op(xt, ut, gt, bt).cpu().numpy(), want, rtol=1e-4, atol=1e-4)
    # non-contiguous inputs are made contiguous by the adapter, as in the reference
    big = torch.zeros(37, 512, device="cuda")
    big[:, ::2] = xt
    np.testing.assert_allclose(op(big[:, ::2], ut, gt, bt).cpu().numpy(), want, rtol=1e-4, atol=1e-4)
    # a base that is only 4-byte aligned takes the scalar path
    flat = torch.zeros(37 * 256 + 1, device="cuda")
    flat[1:] = xt.reshape(-1)
    from ops_rec_b200 import cabi
    got = cabi.ln_mul(flat[1:].view(37, 256), ut, gt, bt)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-4)
    with pytest.raises(RuntimeError, match="The x should be 2D"):
        op(xt[0], ut, gt, bt)
    with pytest.raises(RuntimeError, match="identical shape"):
        op(xt, ut[:5], gt, bt)
    with pytest.raises(RuntimeError, match="float32 only"):
        op(xt.half(), ut.half(), gt.half(), bt.half())


@pytest.mark.gpu
def test_gpu_large_mean_rows_keep_their_precision():
    # a one-pass E[x^2] - mean^2 variance would lose these rows; the kernel uses the reference's two passes
    x, u, gamma, beta = _inputs(16, 1024, seed=9)
    x += 1000.0
    got = _gpu(x, u, gamma, beta)
    np.testing.assert_allclose(got, LO.ln_mul(x, u, gamma, beta, dtype=np.float64), rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(got, LO.ln_mul(x, u, gamma, beta), rtol=1e-3, atol=1e-3)
