"""in_linear_silu_backward and the autograd formula of distance_in_linear_silu: the oracle against the outputs of the
reference's two goldens (CPU); the CUDA operator through the C ABI, the torch operator and loss.backward() against the
oracle (GPU).  Input recipe and acceptance follow the reference tests
(in_linear_silu_backward/test/pytest/test_in_linear_silu_backward.py:173-236: uniform inputs, the "double pole"
comparison of max / mean relative error and RMSE against a 16-bit small-operator run with ratios 5 / 1.5 / 1.5;
test_in_linear_silu_autograd.py:176-207: MSE loss against a target, atol 5e-3 / 1e-3 with at most 0.1 % outliers)."""
import glob
import os

import pytest
import torch

from oracle import in_linear_silu_oracle as IO
from tests._util import GOLDEN_DIR, load_fixture

FIXTURES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "linsilu_bwd_*.npz")))
BF16, FP16 = torch.bfloat16, torch.float16


def _fixture(name):
    fx = load_fixture(name)
    dt = FP16 if int(fx["is_fp16"]) else BF16
    t = {k: (fx[k].to(dt) if dt == FP16 else fx[k]) for k in
         ("x", "weight", "user_grad", "value_grad", "query_grad", "key_grad", "linear_output")}
    return fx, dt, t, [int(v) for v in fx["split"]], fx.get("bias")


@pytest.mark.parametrize("name", FIXTURES)
def test_oracle_matches_both_reference_goldens(name):
    fx, dt, t, split, bias = _fixture(name)
    args = (t["x"], t["weight"], bias, t["user_grad"], t["value_grad"], t["query_grad"], t["key_grad"], t["linear_output"])
    xg, wg, bg = IO.in_linear_silu_backward(*args, round_mid=False)
    torch.testing.assert_close(xg, fx["x_grad_fp32"], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(wg, fx["weight_grad_fp32"], rtol=1e-4, atol=1e-4)
    xg, wg, bg16 = IO.in_linear_silu_backward(*args)
    torch.testing.assert_close(xg.float(), fx["x_grad_lowp"], rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(wg.float(), fx["weight_grad_lowp"], rtol=1e-2, atol=1e-2)
    if bias is not None:
        torch.testing.assert_close(bg, fx["bias_grad_fp32"], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(bg16, fx["bias_grad_lowp"], rtol=1e-4, atol=1e-4)


def test_fixture_set_is_complete():
    assert len(FIXTURES) == 3


def _errors(actual, golden):
    a, g = actual.float(), golden.float()
    diff, den = (a - g).abs(), g.abs() + 1e-7
    rel = torch.where(den > 1e-7, diff / den, diff)
    return rel.max().item(), rel.mean().item(), (a - g).pow(2).mean().sqrt().item()


def _double_pole(label, fused, small_op, golden):
    """The reference's acceptance (test_in_linear_silu_backward.py:79-117): the fused operator's errors against the
    fp32 golden may exceed those of the 16-bit small-operator run by at most x5 (max), x1.5 (mean), x1.5 (RMSE)."""
    ef, es = _errors(fused, golden), _errors(small_op, golden)
    for (f, s), ratio, what in zip(zip(ef, es), (5, 1.5, 1.5), ("max rel", "mean rel", "rmse")):
        assert (f / s <= ratio) if s != 0.0 else abs(f - s) < 1e-6, (label, what, f, s)


def _case(m, k, n, dtype, diff, bias, seed=0):
    gen = torch.Generator().manual_seed(seed + m + n)
    h = n // 4
    split = [h - 32, h - 16, h + 16, h + 32] if diff else [h] * 4
    u = lambda *s: (torch.rand(*s, generator=gen) * 2 - 1).to(dtype)
    grads = [torch.rand(m, w, generator=gen).to(dtype) for w in split]
    return dict(x=u(m, k), weight=u(n, k), bias=(torch.rand(n, generator=gen) * 2 - 1) if bias else None,
                grads=grads, linear_output=u(m, n), split=split)


def _run_cabi(c):
    from ops_rec_b200 import cabi
    cu = lambda t: t.cuda() if t is not None else None
    out = cabi.in_linear_silu_backward(cu(c["x"]), cu(c["weight"]), cu(c["bias"]), *[g.cuda() for g in c["grads"]],
                                       cu(c["linear_output"]), c["split"])
    torch.cuda.synchronize()
    return [o.cpu() if o is not None else None for o in out]


def _check(c, got, label):
    args = (c["x"], c["weight"], c["bias"], *c["grads"], c["linear_output"])
    g32 = IO.in_linear_silu_backward(*args, round_mid=False)
    g16 = IO.in_linear_silu_backward(*args)
    for name, a, lo, hi in zip(("x_grad", "weight_grad", "bias_grad"), got, g16, g32):
        if hi is None:
            assert a is None
            continue
        assert a.shape == hi.shape and torch.isfinite(a.float()).all(), (label, name)
        if name == "bias_grad":
            torch.testing.assert_close(a, hi, rtol=1e-4, atol=1e-4 * max(1.0, hi.abs().max().item()))
        else:
            assert a.dtype == c["x"].dtype
            _double_pole(f"{label} {name}", a, lo, hi)
            assert (a.float() - hi).abs().max() <= 2e-2 * hi.abs().max(), (label, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", FIXTURES)
def test_gpu_fixtures(name):
    fx, dt, t, split, bias = _fixture(name)
    c = dict(x=t["x"], weight=t["weight"], bias=bias, grads=[t[k] for k in ("user_grad", "value_grad", "query_grad", "key_grad")],
             linear_output=t["linear_output"], split=split)
    got = _run_cabi(c)
    _double_pole("x_grad", got[0], fx["x_grad_lowp"], fx["x_grad_fp32"])
    _double_pole("weight_grad", got[1], fx["weight_grad_lowp"], fx["weight_grad_fp32"])
    if bias is not None:
        torch.testing.assert_close(got[2], fx["bias_grad_fp32"], rtol=1e-4, atol=1e-4)
    _check(c, got, name)


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 1123, 2048, 3201])
@pytest.mark.parametrize("dim", [(16, 128), (64, 512), (240, 960), (128, 2048)])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("dtype", [FP16, BF16])
@pytest.mark.parametrize("diff", [False, True])
def test_gpu_reference_grid(m, dim, bias, dtype, diff):
    if dim[0] <= 32 and diff:
        pytest.skip("the reference skips unequal splits for the smallest width")
    c = _case(m, dim[0], dim[1], dtype, diff, bias)
    _check(c, _run_cabi(c), f"m{m} {dim} {dtype} diff{diff} bias{bias}")


@pytest.mark.gpu
def test_gpu_large_shapes():
    for m, dim in ((511, (512, 6144)), (7687, (768, 3072)), (20480, (64, 512))):
        c = _case(m, dim[0], dim[1], BF16, False, True)
        _check(c, _run_cabi(c), f"m{m} {dim}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [BF16, FP16])
def test_gpu_autograd_through_the_forward_operator(dtype):
    """loss.backward() through distance_in_linear_silu, against torch autograd of F.linear + F.silu + split in fp32
    (test_in_linear_silu_autograd.py:148-172) with that test's acceptance."""
    import ops_rec_b200 as ops_rec
    torch.manual_seed(0)
    m, k, n = 1123, 64, 512
    split = [n // 4 - 32, n // 4 - 16, n // 4 + 16, n // 4 + 32]
    x = torch.empty(m, k).uniform_(-1, 1).to(dtype)
    w = torch.empty(n, k).uniform_(-1, 1).to(dtype)
    b = torch.empty(n).uniform_(-1, 1)
    target = torch.empty(m, n).uniform_(-1, 1)
    xs, ws, bs = (t.cuda().requires_grad_(True) for t in (x, w, b))
    outs = ops_rec.ascendc.activation.distance_in_linear_silu(xs, ws, bs, split)
    tg = torch.split(target.cuda().to(dtype), split, dim=-1)
    loss = sum(torch.nn.functional.mse_loss(o, t) for o, t in zip(outs[:4], tg)) / 4
    loss.backward()
    xr, wr, br = (t.float().requires_grad_(True) for t in (x, w, b))
    mixed = torch.nn.functional.silu(torch.nn.functional.linear(xr, wr, br))
    ref = sum(torch.nn.functional.mse_loss(o, t) for o, t in zip(torch.split(mixed, split, dim=-1),
                                                               torch.split(target, split, dim=-1))) / 4
    ref.backward()
    atol = 1e-3 if dtype == FP16 else 5e-3
    for name, got, want in (("x", xs.grad, xr.grad), ("weight", ws.grad, wr.grad), ("bias", bs.grad, br.grad)):
        bad = ((got.float().cpu() - want).abs() > atol).float().mean().item()
        assert bad < 1e-3, (name, bad)


@pytest.mark.gpu
def test_gpu_errors_and_meta():
    import ops_rec_b200 as ops_rec
    op = ops_rec.ascendc.activation.in_linear_silu_backward
    c = _case(8, 64, 256, BF16, False, True)
    cu = lambda t: t.cuda()
    with pytest.raises(RuntimeError, match="split_list must have 4"):
        op(cu(c["x"]), cu(c["weight"]), None, *[cu(g) for g in c["grads"]], cu(c["linear_output"]), [64, 64, 64])
    with pytest.raises(RuntimeError, match="linear_output dim"):
        op(cu(c["x"]), cu(c["weight"]), None, *[cu(g) for g in c["grads"]], cu(c["linear_output"][:, :128]), c["split"])
    x = torch.empty(8, 64, device="meta", dtype=BF16)
    w = torch.empty(256, 64, device="meta", dtype=BF16)
    g = torch.empty(8, 64, device="meta", dtype=BF16)
    lo = torch.empty(8, 256, device="meta", dtype=BF16)
    out = op(x, w, torch.empty(256, device="meta"), g, g, g, g, lo, [64] * 4)
    assert out[0].shape == (8, 64) and out[1].shape == (256, 64) and out[2].shape == (256,)
