"""hstu_dense ([B, S, N, D] layout), the reference's second forward entry point
(ascendc/attention/hstu_v1/torch_extension/hstu_dense_plugin.cpp:19-40, 154-162): here it is the jagged forward
over equal lengths.  Oracle against the reference's numpy golden get_golden (fixtures), schema and Meta on CPU,
the operator itself on the GPU."""
import pytest
import torch

from oracle import hstu_oracle as O
from tests._util import dense_fixture_names, load_fixture


def _args(fx):
    B, S, N, D, mask_type = (int(x) for x in fx["meta"])
    return dict(q=fx["q"], k=fx["k"], v=fx["v"], mask=fx.get("mask"), attn_bias=fx.get("rab"), mask_type=mask_type,
                max_seq_len=S, silu_scale=float(fx["silu_scale"]))


@pytest.mark.parametrize("name", dense_fixture_names())
def test_dense_oracle_matches_reference_golden(name):
    fx = load_fixture(name)
    got = O.hstu_dense_forward(**_args(fx), round_p=False, out_dtype=torch.float32)
    torch.testing.assert_close(got, fx["out_v1_numpy"].float(), rtol=1e-5, atol=1e-6)


def test_dense_schema_and_meta():
    import ops_rec_b200 as ops_rec
    sch = torch.ops.ops_rec.hstu_dense.default._schema
    assert [a.name for a in sch.arguments] == ["q", "k", "v", "mask", "attn_bias", "mask_type", "max_seq_len",
                                               "silu_scale"]
    q = torch.empty(2, 9, 3, 32, device="meta", dtype=torch.float16)
    out = ops_rec.ascendc.attention.hstu_dense(q, q, q, None, None, 0, 9, 0.0)
    assert out.shape == q.shape and out.dtype == q.dtype
    with pytest.raises(RuntimeError, match="4D"):
        ops_rec.ascendc.attention.hstu_dense(q[0], q[0], q[0], None, None, 0, 9, 0.0)


@pytest.mark.gpu
@pytest.mark.parametrize("name", dense_fixture_names())
def test_dense_operator_on_fixtures(name):
    import ops_rec_b200 as ops_rec
    fx = load_fixture(name)
    a = _args(fx)
    cu = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in a.items()}
    out = ops_rec.ascendc.attention.hstu_dense(cu["q"], cu["k"], cu["v"], cu["mask"], cu["attn_bias"], cu["mask_type"],
                                               cu["max_seq_len"], cu["silu_scale"])
    torch.testing.assert_close(out.cpu(), fx["out_v1_numpy"].float(), rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("shape,dtype,mask_type,bias", [
    ((4, 256, 4, 128), torch.bfloat16, 0, True),     # tensor-core kernel, whole tiles
    ((3, 300, 2, 64), torch.float16, 2, False),      # tensor-core kernel, ragged tail, no mask
    ((2, 15, 1, 32), torch.float32, 3, True),        # generic kernel, custom mask
    ((16, 1024, 1, 128), torch.bfloat16, 0, False),
])
def test_dense_operator_against_the_oracle(shape, dtype, mask_type, bias):
    import ops_rec_b200 as ops_rec
    B, S, N, D = shape
    g = torch.Generator().manual_seed(S + D)
    q, k, v = ((torch.randn(B, S, N, D, generator=g) * 0.5).to(dtype) for _ in range(3))
    rab = (torch.randn(B, N, S, S, generator=g) * 0.1).to(dtype) if bias else None
    mask = torch.randint(0, 2, (B, N, S, S), generator=g).to(dtype) if mask_type == 3 else None
    out = ops_rec.ascendc.attention.hstu_dense(q.cuda(), k.cuda(), v.cuda(), None if mask is None else mask.cuda(),
                                               None if rab is None else rab.cuda(), mask_type, S, 1.0 / 256).cpu()
    ref = O.hstu_dense_forward(q, k, v, mask, rab, mask_type, S, 1.0 / 256, round_p=False, out_dtype=torch.float32)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    torch.testing.assert_close(out.float(), ref, rtol=tol, atol=tol)
    scale = ref.abs().max()
    assert (out.float() - ref).abs().max() <= (2e-5 if dtype == torch.float32 else 2e-2) * scale
