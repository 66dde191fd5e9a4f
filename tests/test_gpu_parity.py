"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and the committed fixtures.

The grid follows the reference's own forward test (hstu_forward_v1/test/pytest/test_hstu_jagged.py:227-491):
shapes x bias on/off x dtype x mask variants, the ctx/target boundary values, GQA, padded offsets, int32/int64
offsets, dqk != dv, delta (q shorter than k).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import hstu_oracle as O
from ops_rec_b200 import cabi
from tests._parity import assert_parity, run_cabi, to_cuda
from tests._util import fixture_call_args, fixture_names, load_fixture, make_case

pytestmark = pytest.mark.gpu

BF16, FP16, FP32 = torch.bfloat16, torch.float16, torch.float32


@pytest.mark.parametrize("name", fixture_names())
def test_fixtures_from_the_reference_goldens(name):
    fx = load_fixture(name)
    args = fixture_call_args(fx)
    out, status = run_cabi(args)
    assert status == 0
    ref = fx["out_v2_fp32"]
    if args["q"].dtype == FP32:
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    else:
        torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2)
        ok, detail = O.double_reference_ok(out, fx["out_v2_lowp"], ref, multiplier=5)
        assert ok, detail
    assert_parity(out, args, label=name)


MASKS = [dict(mask_type=2), dict(custom_mask=True), dict(ctx=0, tgt=30, g=1), dict(ctx=0, tgt=30, g=3),
         dict(ctx=6, tgt=0, g=1), dict(ctx=6, tgt=0, g=3), dict(ctx=6, tgt=30, g=1), dict(ctx=6, tgt=30, g=3),
         dict()]


@pytest.mark.parametrize("shape", [(1, 2, 15, 16), (16, 4, 1024, 128), (1, 4, 1024, 16), (16, 2, 15, 128),
                                   (8, 4, 600, 64)])
@pytest.mark.parametrize("bias", [None, "batch"])
@pytest.mark.parametrize("dtype", [FP32, FP16, BF16])
def test_reference_grid_causal(shape, bias, dtype):
    B, H, maxL, D = shape
    if dtype == FP32 and maxL * B > 4096:
        B = 4
    args = make_case(B, H, H, D, D, 1, maxL, dtype, seed=B + maxL, rab=bias)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"{shape} {bias} {dtype}")


@pytest.mark.parametrize("mask", MASKS)
@pytest.mark.parametrize("D,dtype", [(128, BF16), (64, FP16), (32, FP32)])
def test_mask_variants(mask, D, dtype):
    mask = dict(mask)
    args = make_case(4, 2, 2, D, D, 1, 330, dtype, seed=7, rab="batch", **mask)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"{mask} d{D} {dtype}")


@pytest.mark.parametrize("ctx", [255, 256, 257])
@pytest.mark.parametrize("tgt", [511, 512])
def test_ctx_target_boundaries(ctx, tgt):
    args = make_case(2, 2, 2, 128, 128, 1, 200, BF16, seed=ctx + tgt, ctx=ctx, tgt=tgt, g=1)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"ctx{ctx} tgt{tgt}")


@pytest.mark.parametrize("L", [1, 15, 127, 128, 129, 255, 256, 257, 383, 384, 385, 512, 513])
@pytest.mark.parametrize("D", [64, 128])
def test_ragged_tails_single_sequence(L, D):
    # make_case adds ctx + tgt to the base length
    args = make_case(1, 2, 2, D, D, L - min(3, L - 1), L - min(3, L - 1), BF16, seed=L, rab="batch",
                     tgt=min(3, L - 1), g=1)
    assert int(args["seq_offset"][-1]) == L
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"L{L} d{D}")


@pytest.mark.parametrize("Hq,Hk", [(8, 8), (8, 4), (8, 2), (8, 1)])
@pytest.mark.parametrize("dtype,D", [(BF16, 128), (FP32, 16)])
def test_gqa(Hq, Hk, dtype, D):
    args = make_case(3, Hq, Hk, D, D, 1, 300, dtype, seed=Hk, rab="batch")
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"gqa {Hq}:{Hk}")


@pytest.mark.parametrize("dtype", [BF16, FP32])
def test_dqk_differs_from_dv(dtype):
    args = make_case(3, 2, 2, 64, 128, 1, 200, dtype, seed=5, rab="batch", tgt=5, g=1)
    out, status = run_cabi(args)
    assert status == 0 and out.shape[-1] == 128
    assert_parity(out, args, label="dqk64 dv128")


@pytest.mark.parametrize("dtype,D", [(BF16, 128), (BF16, 64), (FP32, 32)])
def test_delta_q_shorter_than_k(dtype, D):
    args = make_case(5, 2, 2, D, D, 1, 400, dtype, seed=11, rab="batch", delta=True)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"delta d{D}")
    args = make_case(5, 2, 2, D, D, 20, 400, dtype, seed=12, delta=True, tgt=9, g=2, ctx=3)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"delta ctx/target d{D}")


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_padded_and_empty_offsets(index_dtype):
    args = make_case(6, 4, 4, 128, 128, 1, 500, BF16, seed=21, rab="batch", index_dtype=index_dtype)
    base, status = run_cabi(args)
    assert status == 0
    assert_parity(base, args, label="base")
    off = args["seq_offset"]
    # repeated last offset (the reference pads like this, test_hstu_jagged.py:58-61) and an empty sequence
    padded = torch.cat([off, off[-1:], off[-1:]])
    bias = torch.cat([args["attn_bias"], args["attn_bias"][:2]])
    out, status = run_cabi(dict(args, seq_offset=padded, seq_offset_k=padded, attn_bias=bias))
    assert status == 0 and torch.equal(out, base)
    mid = torch.cat([off[:3], off[2:]])
    bias = torch.cat([args["attn_bias"][:2], args["attn_bias"][:1], args["attn_bias"][2:]])
    out, status = run_cabi(dict(args, seq_offset=mid, seq_offset_k=mid, attn_bias=bias))
    assert status == 0 and torch.equal(out, base)


@pytest.mark.parametrize("form", ["shared3", "shared4"])
def test_bias_shared_by_the_batch(form):
    args = make_case(5, 4, 4, 64, 64, 1, 300, BF16, seed=3, rab=form, tgt=7, g=1)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=form)
    S = args["max_seq_len"]
    dense = args["attn_bias"].reshape(1, 4, S, S).expand(5, -1, -1, -1).contiguous()
    out2, _ = run_cabi(dict(args, attn_bias=dense))
    assert torch.equal(out, out2)


def test_bias_with_odd_max_seq_len_takes_the_scalar_load_path():
    args = make_case(3, 2, 2, 128, 128, 1, 299, BF16, seed=9, rab="batch", max_seq_len=301)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label="maxL 301")


def test_alpha_before_bias_flag_and_default_order():
    args = make_case(2, 2, 2, 128, 128, 50, 300, BF16, seed=2, rab="batch")
    args["alpha"] = 0.05
    out, _ = run_cabi(args)
    assert_parity(out, args, label="alpha after bias")
    out2, _ = run_cabi(args, flags=cabi.FLAG_ALPHA_BEFORE_BIAS)
    ref2 = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32, alpha_before_bias=True)
    torch.testing.assert_close(out2.float(), ref2, rtol=1e-2, atol=1e-2)
    assert (out2.float() - ref2).abs().max() <= 2e-2 * ref2.abs().max()
    assert (out.float() - ref2).abs().max() > 5e-2 * ref2.abs().max()


@pytest.mark.parametrize("alpha", [0.02, 0.15, 0.5, 2.0])
@pytest.mark.parametrize("D", [64, 128])
def test_score_magnitudes_small_to_saturating(alpha, D):
    # alpha sweeps |alpha * (s + bias)| from << 1 (the near-linear part of SiLU) to >> 1 (the saturated part): the
    # approximate tanh / exp instructions behind the SiLU must hold the tolerance over the whole range
    args = make_case(4, 2, 2, D, D, 100, 500, BF16, seed=int(alpha * 100) + D, rab="batch", tgt=11, g=1)
    args["alpha"] = alpha
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"alpha {alpha} d{D}")


def test_explicit_silu_scale_and_deterministic_flag():
    args = make_case(3, 2, 2, 64, 64, 1, 257, BF16, seed=4)
    args["silu_scale"] = 0.125
    out, _ = run_cabi(args)
    assert_parity(out, args, label="silu_scale")
    out2, _ = run_cabi(args, deterministic=True)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("D,dtype", [(128, BF16), (64, BF16), (128, FP16)])
def test_tensor_core_and_generic_kernels_agree(D, dtype):
    args = make_case(6, 4, 2, D, D, 1, 700, dtype, seed=13, rab="batch", tgt=20, g=2, ctx=4)
    a, _ = cabi.make_args(args["q"], args["k"], args["v"], None, args["seq_offset"], max_seq_len=args["max_seq_len"])
    assert cabi.kernel_kind(a) == 1
    tc, st1 = run_cabi(args)
    gen, st2 = run_cabi(args, flags=cabi.FLAG_FORCE_GENERIC)
    assert st1 == 0 and st2 == 0
    assert_parity(tc, args, label="tc")
    assert_parity(gen, args, label="generic")
    scale = gen.float().abs().max()
    assert (tc.float() - gen.float()).abs().max() <= 2e-2 * scale


@pytest.mark.parametrize("rab", [None, "shared3"])
def test_medium_batches_take_the_limited_look_ahead(rab):
    """Between 4 and 32 work items per CTA the scheduler draws a few items ahead (not one, not the whole ring):
    400 sequences x 4 heads x 1-2 q-pairs on 148 CTAs."""
    args = make_case(400, 4, 4, 64, 64, 200, 400, BF16, seed=29, rab=rab, max_seq_len=400)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"400 sequences, rab={rab}")
    again, _ = run_cabi(args)
    assert torch.equal(out, again)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("rab,lo,hi", [(None, 200, 420), (None, 1030, 1300), ("shared3", 600, 900), ("shared3", 1030, 1300)])
def test_both_forms_of_the_score_stage(D, rab, lo, hi):
    """The kernel exists with its P/O code rolled (short sequences) and unrolled (long ones); the launcher picks by
    mean length and bias mode: below 512 / 1024 with a staged bias rolled, above unrolled."""
    args = make_case(3, 2, 1, D, D, lo, hi, BF16, seed=lo + D, rab=rab, tgt=20, g=1)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label=f"D{D} rab={rab} lengths {lo}-{hi}")


def test_results_are_bitwise_reproducible():
    args = make_case(8, 4, 4, 128, 128, 1, 900, BF16, seed=17, rab="batch")
    a, _ = run_cabi(args)
    for _ in range(3):
        b, _ = run_cabi(args)
        assert torch.equal(a, b)


@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
@pytest.mark.parametrize("D,dtype,rab", [(128, BF16, None), (64, BF16, "batch"), (128, FP16, "shared3"), (32, FP32, None)])
def test_non_finite_values_of_a_neighbouring_sequence_do_not_leak(D, dtype, rab, poison):
    """The reference golden slices every sequence out of the packed tensors, so nothing of one sequence can reach
    another.  Here a K/V tile that runs past a sequence end holds the next sequence's rows: with every second
    sequence's q, k and v made non-finite, the others must come out finite and bit for bit as without the poison."""
    args = make_case(9, 2, 2, D, D, 3, 420, dtype, seed=23, rab=rab)
    clean, status = run_cabi(args)
    assert status == 0
    off = args["seq_offset"].tolist()
    bad = dict(args, q=args["q"].clone(), k=args["k"].clone(), v=args["v"].clone())
    for b in range(1, 9, 2):
        for name in ("q", "k", "v"):
            bad[name][off[b]:off[b + 1]] = poison
    out, status = run_cabi(bad)
    assert status == 0
    for b in range(0, 9, 2):
        rows = slice(off[b], off[b + 1])
        assert torch.isfinite(out[rows].float()).all(), f"sequence {b} (L={off[b + 1] - off[b]})"
        assert torch.equal(out[rows], clean[rows]), f"sequence {b}"


def test_output_rows_outside_the_call_are_untouched():
    args = to_cuda(make_case(5, 2, 2, 128, 128, 1, 300, BF16, seed=19))
    T = args["q"].shape[0]
    pad = 64
    buf = torch.full((T + 2 * pad, 2, 128), 7.0, dtype=BF16, device="cuda")
    out = buf[pad:pad + T]
    cabi.hstu_jagged_forward(**args, out=out)
    torch.cuda.synchronize()
    assert (buf[:pad] == 7.0).all() and (buf[pad + T:] == 7.0).all()
    assert_parity(out.cpu(), {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in args.items()})


def test_inconsistent_inputs_set_the_status_word_and_never_fault():
    args = make_case(4, 2, 2, 128, 128, 10, 300, BF16, seed=23, rab="batch", tgt=5, g=1)
    off = args["seq_offset"].clone()
    bad = off.clone()
    bad[2] = bad[1] - 3                                     # not monotone
    _, status = run_cabi(dict(args, seq_offset=bad, seq_offset_k=bad))
    assert status & cabi.ST_BAD_OFFSETS
    _, status = run_cabi(dict(args, max_seq_len=8, max_seq_len_k=8, attn_bias=None))
    assert status & cabi.ST_LEN_GT_MAX
    big = torch.full_like(args["num_target"], 10_000)
    _, status = run_cabi(dict(args, num_target=big))
    assert status & cabi.ST_BAD_CTX_TARGET
    past = off.clone()
    past[-1] += 1000                                        # points past the end of q
    _, status = run_cabi(dict(args, seq_offset=past, seq_offset_k=past))
    assert status & cabi.ST_BAD_OFFSETS
    # offsets that run back and forth describe more q-pairs than the work list (sized from total_q) can hold:
    # the device clamps the list and ignores what does not fit - flagged, never a fault
    B = off.numel() - 1
    zig = torch.tensor([int(off[-1]) if i % 2 else 0 for i in range(B + 1)], dtype=off.dtype)
    _, status = run_cabi(dict(args, seq_offset=zig, seq_offset_k=zig, max_seq_len=int(off[-1]),
                              max_seq_len_k=int(off[-1]), attn_bias=None))
    assert status & cabi.ST_BAD_OFFSETS
    many = make_case(64, 4, 4, 128, 128, 60, 64, BF16, seed=5)
    T = many["q"].shape[0]
    zig = torch.tensor([T if i % 2 else 0 for i in range(65)], dtype=many["seq_offset"].dtype)
    _, status = run_cabi(dict(many, seq_offset=zig, seq_offset_k=zig, max_seq_len=T, max_seq_len_k=T))
    assert status & cabi.ST_BAD_OFFSETS
    out, status = run_cabi(args)                            # the context is still healthy
    assert status == 0
    assert_parity(out, args, label="after bad inputs")


def test_tensors_on_another_device_are_refused_on_the_host():
    """A CPU (or other-GPU) tensor among CUDA tensors must fail before any pointer reaches a kernel."""
    import ops_rec_b200 as ops_rec
    args = to_cuda(make_case(2, 2, 2, 64, 64, 5, 40, BF16, seed=3, rab="batch", tgt=2, g=1))
    hj = ops_rec.ascendc.attention.hstu_jagged

    def call(**over):
        a = dict(args, **over)
        return hj(a["q"], a["k"], a["v"], a["mask"], a["attn_bias"], a["mask_type"], a["max_seq_len"], 0.0,
                  a["seq_offset"], None, a["num_target"], 1, a["alpha"])

    for name in ("k", "v", "attn_bias", "seq_offset"):
        with pytest.raises(RuntimeError, match="device|CUDA"):
            call(**{name: args[name].cpu()})
    with pytest.raises(RuntimeError, match="device|CUDA"):
        call(mask=torch.ones(2, 2, args["max_seq_len"], args["max_seq_len"], dtype=BF16), mask_type=3)
    with pytest.raises(ValueError, match="is on"):
        cabi.hstu_jagged_forward(**dict(args, attn_bias=args["attn_bias"].cpu()))
    out = call()                                            # and a consistent call still works
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()


def test_device_work_list_equals_host_plan():
    args = to_cuda(make_case(37, 4, 4, 128, 128, 1, 1500, BF16, seed=29))
    out = torch.empty_like(args["q"])
    a, keep = cabi.make_args(args["q"], args["k"], args["v"], out, args["seq_offset"],
                             max_seq_len=args["max_seq_len"], alpha=args["alpha"])
    n = cabi.workspace_size(a)
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
    cabi.check(cabi.load().hstu_jagged_fwd(C.byref(a), ws.data_ptr(), n, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    header = ws[:16].cpu().numpy().view(np.uint32)
    items_dev = ws[256:].cpu().numpy().view(np.uint32).reshape(-1, 2)[: header[1]]
    items_host, status = cabi.plan_host(args["seq_offset"].cpu().numpy(), 4, max_seq_len=args["max_seq_len"])
    assert header[0] == 0 and status == 0
    assert header[1] == len(items_host)
    assert np.array_equal(items_dev, items_host)


def test_large_batch_beyond_the_reference_limit():
    # the reference caps the batch at 2048 (tiling_policy_define.h:107); here it may be larger
    args = make_case(3000, 2, 2, 64, 64, 1, 40, BF16, seed=31)
    out, status = run_cabi(args)
    assert status == 0
    assert_parity(out, args, label="B3000")


@pytest.mark.parametrize("D,dtype", [(128, BF16), (64, BF16), (128, FP16)])
@pytest.mark.parametrize("maxL", [130, 517])
def test_custom_mask_runs_on_the_tensor_core_kernel(D, dtype, maxL):
    """mask_type 3 (the mask's values multiply, hstu_dense_forward_kernel_patten_bsnd.h:388-395): 0/1 masks as in the
    reference tests (test_hstu_jagged.py: torch.randint(0, 2, ...)) and arbitrary multipliers; with an odd
    max_seq_len the mask rows are not 16-byte aligned (scalar loads)."""
    args = make_case(5, 4, 2, D, D, 1, maxL, dtype, seed=maxL + D, custom_mask=True)
    a, _ = cabi.make_args(args["q"], args["k"], args["v"], None, args["seq_offset"], mask=args["mask"], mask_type=3,
                          max_seq_len=args["max_seq_len"])
    assert cabi.kernel_kind(a) == 1
    tc, st = run_cabi(args)
    assert st == 0
    assert_parity(tc, args, label="0/1 mask")
    gen, _ = run_cabi(args, flags=cabi.FLAG_FORCE_GENERIC)
    assert (tc.float() - gen.float()).abs().max() <= 2e-2 * gen.float().abs().max()
    gen_t = torch.Generator().manual_seed(7)
    args["mask"] = (torch.rand(args["mask"].shape, generator=gen_t) * 2 - 0.5).to(dtype)   # multipliers in [-0.5, 1.5)
    tc, st = run_cabi(args)
    assert st == 0
    assert_parity(tc, args, label="multiplier mask")


def test_custom_mask_with_bias_takes_the_generic_kernel():
    args = make_case(3, 2, 2, 128, 128, 1, 200, BF16, seed=9, custom_mask=True, rab="batch")
    a, _ = cabi.make_args(args["q"], args["k"], args["v"], None, args["seq_offset"], mask=args["mask"],
                          attn_bias=args["attn_bias"], mask_type=3, max_seq_len=args["max_seq_len"])
    assert cabi.kernel_kind(a) == 0
    out, st = run_cabi(args)
    assert st == 0
    assert_parity(out, args, label="mask + bias")
