"""GPU parity of the backward: hstu_jagged_bwd through the C ABI against the CPU oracle and against the fixtures made
by the reference's autograd golden.

Grid and acceptance follow the reference's backward test
(hstu_backward_v1/test/pytest/test_hstu_jagged_backward.py:283-420): head-dim / GQA / mask / bias / dtype / ctx-target
combinations, inputs uniform(-1, 1), alpha 0.5, the double-reference rule with multiplier 5 for 16-bit inputs.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import ops_rec_b200
from oracle import hstu_oracle as O
from ops_rec_b200 import cabi
from tests._parity import to_cuda
from tests._util import bwd_fixture_names, fixture_call_args, load_fixture

pytestmark = pytest.mark.gpu

BF16, FP16, FP32 = torch.bfloat16, torch.float16, torch.float32
NAMES = ("dq", "dk", "dv", "dbias")


def bwd_args(args):
    """Forward-style keyword arguments -> the backward entry point's."""
    a = dict(args)
    a["max_seq_len_k"] = a.get("max_seq_len_k") or a["max_seq_len"]
    if a.get("seq_offset_k") is None:
        a["seq_offset_k"] = a["seq_offset"]
    return a


def run_bwd(grad, args, **extra):
    res, status = cabi.hstu_jagged_backward(grad.cuda(), **to_cuda(bwd_args(args)), **extra, return_status=True)
    torch.cuda.synchronize()
    return [r.cpu() if r is not None else None for r in res], status


def make_bwd_case(B, Hq, Hk, Dqk, Dv, maxL, dtype, *, seed=0, bias=True, ctx=0, tgt=0, g=0, mask_type=0, delta=False,
                  alpha=0.5, silu_scale=0.0, index_dtype=torch.int64):
    """Seeded inputs in the manner of the reference's jagged_data_gen (test_hstu_jagged_backward.py:40-85):
    lengths U[1 + ctx + tgt, maxL], len_q = min(len_q, len_k), values uniform(-1, 1)."""
    rng = np.random.default_rng(seed)
    gen = torch.Generator().manual_seed(seed + 1)
    lo = 1 + ctx + tgt
    len_k = rng.integers(lo, maxL + 1, B)
    len_q = np.minimum(rng.integers(lo, maxL + 1, B), len_k) if delta else len_k.copy()
    offq = torch.from_numpy(np.concatenate([[0], np.cumsum(len_q)])).to(index_dtype)
    offk = torch.from_numpy(np.concatenate([[0], np.cumsum(len_k)])).to(index_dtype)

    def uni(*shape):
        return (torch.rand(*shape, generator=gen) * 2 - 1).to(dtype)

    Tq, Tk = int(offq[-1]), int(offk[-1])
    args = dict(q=uni(Tq, Hq, Dqk), k=uni(Tk, Hk, Dqk), v=uni(Tk, Hk, Dv),
                mask=torch.randint(0, 2, (B, Hq, maxL, maxL), generator=gen).to(dtype) if mask_type == 3 else None,
                attn_bias=uni(B, Hq, maxL, maxL) if bias else None, mask_type=mask_type, max_seq_len=maxL,
                silu_scale=silu_scale, seq_offset=offq,
                num_context=torch.full((B,), ctx, dtype=index_dtype) if (ctx or tgt) else None,
                num_target=torch.full((B,), tgt, dtype=index_dtype) if (ctx or tgt) else None,
                target_group_size=g, alpha=alpha, max_seq_len_k=maxL, seq_offset_k=offk)
    return uni(Tq, Hq, Dv), args


def assert_bwd_parity(got, grad, args, label=""):
    dtype = args["q"].dtype
    ref32 = O.hstu_jagged_backward(grad, **args, round_mid=False, out_dtype=torch.float32)
    lowp = O.hstu_jagged_backward(grad, **args) if dtype != FP32 else None
    for i, name in enumerate(NAMES):
        if ref32[i] is None:
            assert got[i] is None, (label, name)
            continue
        g, r = got[i], ref32[i]
        assert g.shape == r.shape and g.dtype == dtype, (label, name)
        assert torch.isfinite(g.float()).all(), (label, name)
        scale = max(r.abs().max().item(), 1e-30)
        err = (g.float() - r).abs().max().item()
        if dtype == FP32:
            torch.testing.assert_close(g, r, rtol=1e-5, atol=1e-5 * max(scale, 1.0), msg=lambda m: f"{label} {name}: {m}")
            assert err <= 3e-5 * scale, (label, name, err, scale)
        else:
            torch.testing.assert_close(g.float(), r, rtol=1e-2, atol=1e-2 * max(scale, 1.0),
                                       msg=lambda m: f"{label} {name}: {m}")
            ok, detail = O.double_reference_ok(g, lowp[i], r, multiplier=5)
            assert ok, (label, name, detail)
            # and a bound relative to the gradient's own scale (the absolute tolerance alone says little when the
            # gradients are small), as the forward parity has
            assert err <= (3e-2 if dtype == BF16 else 6e-3) * scale, (label, name, err, scale)


@pytest.mark.parametrize("name", bwd_fixture_names())
def test_fixtures_from_the_reference_autograd_golden(name):
    fx = load_fixture(name)
    args = fixture_call_args(fx)
    got, status = run_bwd(fx["grad"], args)
    assert status == 0
    dtype = args["q"].dtype
    for g, key in zip(got, NAMES):
        if key + "_fp32" not in fx:
            assert g is None
            continue
        ref = fx[key + "_fp32"]
        if dtype == FP32:
            torch.testing.assert_close(g, ref, rtol=1e-5, atol=1e-5, msg=lambda m: f"{key}: {m}")
        else:
            ok, detail = O.double_reference_ok(g, fx[key + "_lowp"], ref, multiplier=5)
            assert ok, (key, detail)
            torch.testing.assert_close(g.float(), ref, rtol=1e-2, atol=1e-2 * max(ref.abs().max().item(), 1.0))
    assert_bwd_parity(got, fx["grad"], args, label=name)


@pytest.mark.parametrize("Hk", [8, 4, 2, 1])
@pytest.mark.parametrize("Dqk,Dv", [(1, 16), (16, 32), (32, 16), (72, 32)])
@pytest.mark.parametrize("dtype", [FP16, BF16, FP32])
def test_reference_grid_heads_and_dims(Hk, Dqk, Dv, dtype):
    grad, args = make_bwd_case(2, 8, Hk, Dqk, Dv, 70, dtype, seed=Hk * 100 + Dqk, bias=(Dqk % 32 == 0), delta=True)
    got, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(got, grad, args, label=f"Hk{Hk} D{Dqk}/{Dv} {dtype}")


@pytest.mark.parametrize("maxL,ctx,tgt,g", [(1, 0, 0, 0), (257, 1, 1, 1), (300, 128, 0, 1), (400, 0, 200, 3),
                                            (400, 64, 200, 3)])
@pytest.mark.parametrize("mask_type", [0, 2, 3])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("silu_scale", [0.0, 1.0 / 256])
def test_reference_grid_masks(maxL, ctx, tgt, g, mask_type, bias, silu_scale):
    grad, args = make_bwd_case(2, 2, 1, 32, 16, maxL, BF16, seed=maxL + ctx + tgt, bias=bias, ctx=ctx, tgt=tgt, g=g,
                               mask_type=mask_type, silu_scale=silu_scale)
    got, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(got, grad, args, label=f"L{maxL} c{ctx} t{tgt} g{g} m{mask_type}")


@pytest.mark.parametrize("D", [64, 128, 512])
def test_large_head_dims(D):
    grad, args = make_bwd_case(2, 2, 2, D, D, 50, BF16, seed=D, bias=False, alpha=1.0 / D)
    got, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(got, grad, args, label=f"D{D}")


def test_int32_offsets_and_padding():
    grad, args = make_bwd_case(3, 2, 2, 16, 16, 40, FP32, seed=5, index_dtype=torch.int32)
    base, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(base, grad, args)
    off = args["seq_offset"]
    padded = torch.cat([off, off[-1:], off[-1:]])
    pad_bias = torch.cat([args["attn_bias"], torch.zeros_like(args["attn_bias"][:2])])
    args2 = dict(args, seq_offset=padded, seq_offset_k=padded, attn_bias=pad_bias)
    got, status = run_bwd(grad, args2)
    assert status == 0
    for a, b in zip(got[:3], base[:3]):
        assert torch.equal(a, b)
    assert torch.equal(got[3][:3], base[3])
    assert (got[3][3:] == 0).all()     # blocks of empty sequences are written too


def test_bias_gradient_is_fully_written_and_zero_outside():
    grad, args = make_bwd_case(3, 2, 2, 16, 16, 45, BF16, seed=11, ctx=2, tgt=7, g=2)
    (dq, dk, dv, dbias), status = run_bwd(grad, args)
    assert status == 0
    assert torch.isfinite(dbias.float()).all()
    off = args["seq_offset"].tolist()
    for b in range(3):
        L = off[b + 1] - off[b]
        m = torch.from_numpy(O.hstu_mask(L, L, 2, 7, 2, 0))
        blk = dbias[b].float()
        assert (blk[:, L:, :] == 0).all() and (blk[:, :, L:] == 0).all()
        assert (blk[:, :L, :L][:, ~m] == 0).all()


def test_bitwise_reproducible():
    grad, args = make_bwd_case(4, 4, 2, 32, 32, 90, BF16, seed=3)
    a, _ = run_bwd(grad, args)
    b, _ = run_bwd(grad, args)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_alpha_before_bias_flag():
    grad, args = make_bwd_case(2, 2, 2, 16, 16, 33, FP32, seed=8)
    got, status = run_bwd(grad, args, flags=cabi.FLAG_ALPHA_BEFORE_BIAS)
    assert status == 0
    ref = O.hstu_jagged_backward(grad, **args, round_mid=False, alpha_before_bias=True)
    for g, r in zip(got, ref):
        torch.testing.assert_close(g, r, rtol=1e-5, atol=1e-5)


def test_autograd_through_the_forward_operator():
    """loss.backward() through ops_rec.ascendc.attention.hstu_jagged (formula registered like the reference's
    hstu_v1_autograd.py) gives the oracle's gradients; both overloads."""
    grad, args = make_bwd_case(3, 4, 2, 64, 64, 150, BF16, seed=21, ctx=0, tgt=9, g=1, alpha=1.0 / 64)
    ca = to_cuda(args)
    leaves = [ca[n].clone().requires_grad_(True) for n in ("q", "k", "v", "attn_bias")]
    op = ops_rec_b200.ascendc.attention.hstu_jagged
    out = op(leaves[0], leaves[1], leaves[2], None, leaves[3], 0, args["max_seq_len"], 0.0, ca["seq_offset"],
             ca["num_context"], ca["num_target"], 1, args["alpha"])
    got = torch.autograd.grad(out, leaves, grad.cuda())
    assert_bwd_parity([g.cpu() for g in got], grad, args, label="equal")
    out = op(leaves[0], leaves[1], leaves[2], None, None, 0, args["max_seq_len"], args["max_seq_len"], 0.0,
             ca["seq_offset"], ca["seq_offset"], ca["num_context"], ca["num_target"], 1, args["alpha"])
    got = torch.autograd.grad(out, leaves[:3], grad.cuda())
    assert_bwd_parity([g.cpu() for g in got] + [None], grad, dict(args, attn_bias=None), label="delta")


def test_forward_and_backward_replay_from_a_cuda_graph():
    """The operators enqueue on the current stream without any host synchronisation or host read of device data, so a
    step (forward, then the backward of its output's gradient) can be captured in a CUDA graph and replayed on new
    inputs - including the kernels launched with programmatic stream serialization."""
    grad, args = make_bwd_case(5, 4, 2, 64, 64, 300, BF16, seed=31, tgt=11, g=1, alpha=1.0 / 64)
    grad2, args2 = make_bwd_case(5, 4, 2, 64, 64, 300, BF16, seed=31, tgt=11, g=1, alpha=1.0 / 64)
    gen = torch.Generator().manual_seed(77)
    for name in ("q", "k", "v", "attn_bias"):   # same lengths, other values
        args2[name] = (torch.rand(args[name].shape, generator=gen) * 2 - 1).to(BF16)
    grad2 = (torch.rand(grad.shape, generator=gen) * 2 - 1).to(BF16)
    ca = to_cuda(args)
    fwd = ops_rec_b200.ascendc.attention.hstu_jagged
    bwd = ops_rec_b200.ascendc.attention.hstu_jagged_backward
    g_in = grad.cuda()

    def step():
        out = fwd(ca["q"], ca["k"], ca["v"], None, ca["attn_bias"], 0, args["max_seq_len"], 0.0, ca["seq_offset"],
                  ca["num_context"], ca["num_target"], 1, args["alpha"])
        grads = bwd(g_in, ca["q"], ca["k"], ca["v"], None, ca["attn_bias"], 0, args["max_seq_len"], 0.0,
                    ca["seq_offset"], ca["num_context"], ca["num_target"], 1, args["alpha"])
        return out, grads

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, grads = step()
    for a, g in ((args, grad), (args2, grad2)):
        for name in ("q", "k", "v", "attn_bias"):
            ca[name].copy_(a[name])
        g_in.copy_(g)
        graph.replay()
        torch.cuda.synchronize()
        ref = O.hstu_jagged_forward(**a)
        assert (out.float().cpu() - ref.float()).abs().max() <= 2e-2 * max(1.0, float(ref.float().abs().max()))
        got = [t.cpu() if t is not None else None for t in grads[:4]]
        assert_bwd_parity(got, g, a, label="graph replay")


def test_errors():
    grad, args = make_bwd_case(2, 2, 2, 16, 16, 20, BF16, seed=1)
    shared = dict(args, attn_bias=args["attn_bias"][:1])
    with pytest.raises(cabi.HstuError, match="per-sequence attn_bias"):
        run_bwd(grad, shared)
    with pytest.raises(cabi.HstuError, match="maskType"):
        run_bwd(grad, dict(args, mask_type=1))
    with pytest.raises(RuntimeError, match="numTarget is required"):
        ca = to_cuda(args)
        ops_rec_b200.ascendc.attention.hstu_jagged_backward(
            grad.cuda(), ca["q"], ca["k"], ca["v"], None, None, 0, 20, 0.0, ca["seq_offset"],
            torch.zeros(2, dtype=torch.int64, device="cuda"), None, 1, 0.5)


def test_padded_bias_stride_is_rejected():
    # grad_bias is contiguous and addressed like the bias: a bias whose batch blocks are padded apart has no
    # consistent gradient layout (host check, nothing is launched)
    grad, args = make_bwd_case(2, 2, 2, 16, 16, 20, BF16, seed=1)
    ca = to_cuda(bwd_args(args))
    fwd, _ = cabi.make_args(ca["q"], ca["k"], ca["v"], None, ca["seq_offset"], attn_bias=ca["attn_bias"],
                            max_seq_len=ca["max_seq_len"])
    fwd.bias_batch_stride += 64
    a = cabi.HstuJaggedBwdArgs()
    a.struct_bytes = C.sizeof(cabi.HstuJaggedBwdArgs)
    a.fwd = fwd
    n = C.c_uint64(0)
    rc = cabi.load().hstu_jagged_bwd_get_workspace_size(C.byref(a), C.byref(n))
    assert rc == -2 and b"bias_batch_stride" in cabi.load().hstu_last_error()


@pytest.mark.parametrize("B,lo_hi,maxL,bias", [(40, (1, 300), 1500, False), (24, (1, 200), 700, True),
                                               (1100, (1, 40), 64, True), (1300, (1, 30), 256, False)])
def test_tile_lists_of_short_sequences_under_a_large_max_seq_len(B, lo_hi, maxL, bias):
    """The tensor-core kernels draw their tiles from lists the pre-pass writes: only tiles that exist (most of the
    batch x heads x max_seq_len / 128 slots are empty here), more than 1024 sequences (the pre-pass scans in chunks)."""
    grad, args = make_bwd_case(B, 2, 1, 64, 64, lo_hi[1], BF16, seed=B, bias=False, alpha=1.0 / 64)
    args["max_seq_len"] = args["max_seq_len_k"] = maxL
    if bias:
        gen = torch.Generator().manual_seed(B)
        args["attn_bias"] = (torch.rand(B, 2, maxL, maxL, generator=gen) * 2 - 1).to(BF16)
    got, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(got, grad, args, label=f"B{B} maxL{maxL} bias={bias}")


@pytest.mark.parametrize("bias", [False, True])
def test_many_single_step_tiles_per_cta(bias):
    """Eight one-step tiles per CTA (with and without a staged bias): the producer thread, which draws the tiles and
    runs ahead of the other warps, is a whole tile ahead all the time.  310 sequences of 121 - 128 rows x 4 heads."""
    grad, args = make_bwd_case(310, 4, 4, 64, 64, 128, BF16, seed=5, bias=bias, tgt=120, g=1, alpha=1.0 / 64)
    assert int(args["seq_offset"][-1]) * 4 // 128 >= 8 * 148
    got, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(got, grad, args, label=f"310 x 4 tiles, bias={bias}")


def test_no_query_rows_still_writes_every_element_of_grad_bias():
    # all sequences empty: no kernel visits grad_bias, which must come back as zeros, not as uninitialised memory
    B, H, S, D = 3, 2, 40, 64
    z = torch.zeros(0, H, D, dtype=BF16)
    args = dict(q=z, k=z, v=z, mask=None, attn_bias=torch.randn(B, H, S, S).to(BF16), mask_type=0, max_seq_len=S,
                max_seq_len_k=S, silu_scale=0.0, seq_offset=torch.zeros(B + 1, dtype=torch.int64),
                seq_offset_k=torch.zeros(B + 1, dtype=torch.int64), num_context=None, num_target=None,
                target_group_size=0, alpha=0.5)
    (dq, dk, dv, dbias), status = run_bwd(z, args)
    assert status == 0 and dq.numel() == 0 and dk.numel() == 0
    assert (dbias == 0).all()


def test_inconsistent_inputs_set_the_status_word():
    grad, args = make_bwd_case(2, 2, 2, 16, 16, 20, BF16, seed=2)
    bad = dict(args, max_seq_len=5, max_seq_len_k=5, attn_bias=None)
    _, status = run_bwd(grad, bad)
    assert status & cabi.ST_LEN_GT_MAX


# ------------------------------------------------------------------------------------ tensor-core kernels
# bf16 / fp16 with Dqk = Dv in {64, 128} and mask tril / none run on hstu_bwd_tc.cu; FLAG_FORCE_GENERIC keeps the
# CUDA-core kernels, which gives an independent GPU result to compare with.

@pytest.mark.parametrize("D,dtype", [(128, BF16), (64, BF16), (128, FP16), (64, FP16)])
@pytest.mark.parametrize("case", [
    dict(B=3, Hq=2, Hk=2, maxL=130, bias=False),
    dict(B=4, Hq=4, Hk=2, maxL=700, bias=True),
    dict(B=3, Hq=4, Hk=1, maxL=400, bias=True, ctx=5, tgt=40, g=3),
    dict(B=3, Hq=2, Hk=2, maxL=300, bias=False, ctx=0, tgt=64, g=1),
    dict(B=3, Hq=2, Hk=2, maxL=450, bias=True, ctx=130, tgt=150, g=7),
    dict(B=3, Hq=2, Hk=1, maxL=390, bias=False, ctx=70, tgt=33, g=0),
    dict(B=3, Hq=2, Hk=1, maxL=520, bias=True, delta=True),
    dict(B=3, Hq=2, Hk=2, maxL=520, bias=True, delta=True, ctx=3, tgt=50, g=2),
    dict(B=2, Hq=2, Hk=2, maxL=260, bias=True, mask_type=2),
])
def test_tensor_core_backward(D, dtype, case):
    c = dict(case)
    B, Hq, Hk, maxL, bias = c.pop("B"), c.pop("Hq"), c.pop("Hk"), c.pop("maxL"), c.pop("bias")
    grad, args = make_bwd_case(B, Hq, Hk, D, D, maxL, dtype, seed=maxL + D, bias=bias, alpha=1.0 / D, **c)
    got, status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity(got, grad, args, label=f"tc D{D} {dtype} {case}")
    gen, status = run_bwd(grad, args, flags=cabi.FLAG_FORCE_GENERIC)
    assert status == 0
    for a, b_, name in zip(got, gen, NAMES):
        if a is None:
            assert b_ is None
            continue
        scale = max(b_.float().abs().max().item(), 1e-30)
        assert (a.float() - b_.float()).abs().max().item() <= 3e-2 * scale, name


def test_tensor_core_backward_long_sequences_and_bias_padding():
    # several 128-row tiles per sequence, odd max_seq_len (unaligned d_bias rows), d_bias fully written
    grad, args = make_bwd_case(2, 2, 2, 128, 128, 1031, BF16, seed=77, bias=True, alpha=1.0 / 128)
    (dq, dk, dv, dbias), status = run_bwd(grad, args)
    assert status == 0
    assert_bwd_parity([dq, dk, dv, dbias], grad, args, label="long")
    off = args["seq_offset"].tolist()
    for b in range(2):
        L = off[b + 1] - off[b]
        assert (dbias[b, :, L:, :] == 0).all() and (dbias[b, :, :, L:] == 0).all()
        assert (torch.triu(dbias[b, 0, :L, :L].float(), diagonal=1) == 0).all()


def test_tensor_core_backward_bitwise_reproducible():
    grad, args = make_bwd_case(4, 4, 2, 64, 64, 500, BF16, seed=31, alpha=1.0 / 64)
    a, _ = run_bwd(grad, args)
    b, _ = run_bwd(grad, args)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
