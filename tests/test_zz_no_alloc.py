"""hstu_jagged_fwd_static: the entry point for callers that may not allocate device memory (a serving process
with a frozen memory budget, a plugin whose host forbids allocation while enqueueing, code that cannot afford the
device-wide synchronisation of cudaMalloc).  It keeps the scheduler's scratch in a fixed block inside the library
and must give exactly what the regular entry point gives - also on a second call, when the block still holds the
first call's work list.  This file is named to be collected last; it also passes when run on its own."""
import pytest
import torch

from oracle import hstu_oracle as O
from ops_rec_b200 import cabi
from tests._util import make_case

pytestmark = pytest.mark.gpu


def _cuda(args):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in args.items()}


def _both(args):
    cu = _cuda(args)
    a, _ = cabi.make_args(cu["q"], cu["k"], cu["v"], None, cu["seq_offset"], max_seq_len=cu["max_seq_len"])
    assert cabi.kernel_kind(a) == 1  # the tensor-core kernel: the one that needs scratch (its work list)
    want = cabi.hstu_jagged_forward(**cu)
    got = torch.full_like(want, float("nan"))
    _, status = cabi.hstu_jagged_forward_static(
        cu["q"], cu["k"], cu["v"], got, cu["mask"], cu["attn_bias"], cu["mask_type"], cu["max_seq_len"],
        cu["silu_scale"], cu["seq_offset"], cu["num_context"], cu["num_target"], cu["target_group_size"], cu["alpha"],
        max_seq_len_k=cu["max_seq_len_k"], seq_offset_k=cu["seq_offset_k"], return_status=True)
    torch.cuda.synchronize()
    assert status == 0   # the status word of the built-in block, read without a workspace pointer
    return got.cpu(), want.cpu()


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    # first call: many sequences, long work list; second call: fewer, shorter - stale list entries must not matter
    first = make_case(24, 4, 4, 128, 128, 1, 900, torch.bfloat16, seed=41, rab="batch", tgt=9, g=1)
    second = make_case(3, 2, 1, 64, 64, 1, 300, torch.bfloat16, seed=42, ctx=4)
    for args in (first, second, first):
        got, want = _both(args)
        assert torch.isfinite(got.float()).all()
        # same kernels, same inputs: bit-identical (well inside the rtol = atol = 1e-2 the parity tests use)
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-2)
        assert torch.equal(got, want)
        # and, so that this file stands on its own: the CPU oracle, at the tolerance of the parity tests
        ref = O.hstu_jagged_forward(**args, round_p=False, out_dtype=torch.float32)
        torch.testing.assert_close(got.float(), ref, rtol=1e-2, atol=1e-2)
        assert (got.float() - ref).abs().max() <= 2e-2 * ref.abs().max()


def test_static_scratch_entry_point_rejects_oversized_work_lists():
    # 16 heads x (total_q / 256 + batch) items must fit 1 MiB; a batch of 70000 one-token sequences cannot
    B = 70000
    q = torch.zeros(B, 16, 64, dtype=torch.bfloat16, device="cuda")
    off = torch.arange(B + 1, dtype=torch.int64, device="cuda")
    out = torch.empty_like(q)
    with pytest.raises(cabi.HstuError) as e:
        cabi.hstu_jagged_forward_static(q, q, q, out, None, None, 0, 16, 0.0, off, None, None, 0, 1.0)
    assert e.value.code == cabi.E_SCRATCH_LIMIT and "scratch" in str(e.value)   # the error text is set too
    # the regular entry point takes the same call with a caller workspace
    cabi.hstu_jagged_forward(q, q, q, None, None, 0, 16, 0.0, off, None, None, 0, 1.0)
    torch.cuda.synchronize()


def test_static_scratch_entry_point_reports_the_device_status_word():
    # inconsistent offsets are flagged in the status word of the built-in block (and nothing faults)
    args = _cuda(make_case(4, 2, 2, 64, 64, 10, 200, torch.bfloat16, seed=43))
    bad = args["seq_offset"].clone()
    bad[2] = bad[1] - 3
    out = torch.empty_like(args["q"])
    _, status = cabi.hstu_jagged_forward_static(args["q"], args["k"], args["v"], out, None, None, 0,
                                                args["max_seq_len"], 0.0, bad, None, None, 0, args["alpha"],
                                                return_status=True)
    assert status & cabi.ST_BAD_OFFSETS
