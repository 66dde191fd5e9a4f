"""hstu_paged: the oracle against the fixtures made by the reference's two goldens (CPU), and the CUDA operator
against the oracle and the same fixtures (GPU, through the C ABI).  Grid after the reference's test
(hstu_forward_v1/test/pytest/test_hstu_paged.py:484-520: history / candidate lengths, page sizes 32 / 128 / 256, with
and without previous history in the cache, three dtypes)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import hstu_oracle as O
from oracle import hstu_paged_oracle as PO
from tests._util import GOLDEN_DIR, load_fixture

BF16, FP16, FP32 = torch.bfloat16, torch.float16, torch.float32
NAMES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "paged_*.npz")))


def fixture_args(fx):
    B, Hq, Hk, D, page, max_q, max_k, mask_type = (int(x) for x in fx["meta"])
    return dict(q=fx["q"], k=fx["k"], v=fx["v"], kv_cache=fx["kv_cache"], mask=fx.get("mask"), attn_bias=None,
                mask_type=mask_type, max_seq_len=max_q, max_seq_len_k=max_k, silu_scale=1.0 / max_q,
                seq_offset=fx["seq_offset"], seq_offset_k=fx["seq_offset_k"], seq_offset_t=fx["seq_offset_t"],
                page_offsets=fx["page_offsets"], page_ids=fx["page_ids"], last_page_len=fx["last_page_len"],
                num_target=fx["num_target"], target_group_size=1, alpha=float(fx["alpha"]))


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_the_reference_goldens(name):
    fx = load_fixture(name)
    args = fixture_args(fx)
    got = PO.hstu_paged_forward(**args, round_p=False, out_dtype=torch.float32)
    torch.testing.assert_close(got, fx["out_torch_fp32"], rtol=1e-5, atol=1e-5)
    if "out_torch_lowp" in fx:   # 16-bit golden: every intermediate in the input type; the x5 double-reference rule
        low = PO.hstu_paged_forward(**args)
        ok, detail = O.double_reference_ok(low, fx["out_torch_lowp"], fx["out_torch_fp32"], multiplier=5)
        assert ok, detail
    if "out_numpy_noalpha" in fx:   # the numpy golden applies no alpha
        got = PO.hstu_paged_forward(**dict(args, alpha=1.0), round_p=False, out_dtype=torch.float32)
        torch.testing.assert_close(got, fx["out_numpy_noalpha"], rtol=1e-5, atol=1e-5)


def test_fixture_set_is_present():
    assert len(NAMES) >= 6


def make_paged_case(B, Hq, Hk, D, hist, cand, page, prev, dtype, seed=0, mask_type=0, shuffle_pages=True):
    """Seeded inputs in the spirit of paged_hstu_attn_kernel (test_hstu_paged.py:373-412); pages are handed out in
    a shuffled order so that the page table really indirects."""
    rng = np.random.default_rng(seed)
    gen = torch.Generator().manual_seed(seed + 1)
    new_hist = rng.integers(min(1, hist // 2), hist + 1, B)
    prev_len = rng.integers(1, hist + 1, B) * int(prev)
    cache_len = new_hist + prev_len
    n_cand = rng.integers(1, cand + 1, B) if cand > 0 else np.zeros(B, dtype=np.int64)
    pages_per = (cache_len + page - 1) // page
    total_pages = int(pages_per.sum()) + 3
    order = rng.permutation(total_pages) if shuffle_pages else np.arange(total_pages)
    table = (torch.rand(total_pages, 2, page, Hk, D, generator=gen) * 2 - 1).to(dtype)
    page_ids, page_off, last_len = [], [0], []
    at = 0
    for b in range(B):
        page_ids.extend(int(x) for x in order[at:at + pages_per[b]])
        at += int(pages_per[b])
        page_off.append(len(page_ids))
        rem = int(cache_len[b]) % page
        last_len.append(rem if rem else page)
    lq = new_hist + n_cand
    lk = cache_len + n_cand
    off_q = np.concatenate([[0], np.cumsum(lq)])
    off_k = np.concatenate([[0], np.cumsum(lk)])
    off_t = np.concatenate([[0], np.cumsum(n_cand)])
    T = int(off_q[-1])
    u = lambda *s: (torch.rand(*s, generator=gen) * 2 - 1).to(dtype)
    max_q, max_k = int(lq.max()), int(lk.max())
    mask = None
    if mask_type == 3:
        mask = torch.randint(0, 2, (B, Hq, max_q, max_k), generator=gen).to(dtype)
    i64 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int64)
    return dict(q=u(T, Hq, D), k=u(T, Hk, D), v=u(T, Hk, D), kv_cache=table, mask=mask, attn_bias=None,
                mask_type=mask_type, max_seq_len=max_q, max_seq_len_k=max_k, silu_scale=1.0 / max_q,
                seq_offset=i64(off_q), seq_offset_k=i64(off_k), seq_offset_t=i64(off_t), page_offsets=i64(page_off),
                page_ids=i64(page_ids), last_page_len=i64(last_len), num_target=i64(n_cand), target_group_size=1,
                alpha=1.0 / D ** 0.5)


def test_oracle_gather_follows_the_page_table():
    args = make_paged_case(3, 2, 1, 16, 50, 7, 8, True, FP32, seed=3)
    k_con, v_con, offk = PO.gather_paged_kv(args["k"], args["v"], args["kv_cache"], args["seq_offset"],
                                            args["page_offsets"], args["page_ids"], args["last_page_len"],
                                            args["num_target"])
    assert offk.tolist() == args["seq_offset_k"].tolist()
    b, page = 1, 8
    first = int(args["page_ids"][int(args["page_offsets"][b])])
    assert torch.equal(k_con[int(offk[b]):int(offk[b]) + page], args["kv_cache"][first, 0])
    t = int(args["num_target"][b])
    assert torch.equal(v_con[int(offk[b + 1]) - t:int(offk[b + 1])],
                       args["v"][int(args["seq_offset"][b + 1]) - t:int(args["seq_offset"][b + 1])])


# ------------------------------------------------------------------------------------------------------- GPU
def _run(args, **extra):
    from ops_rec_b200 import cabi
    cu = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in args.items()}
    out, status = cabi.hstu_paged_forward(**cu, **extra, return_status=True)
    torch.cuda.synchronize()
    return out.cpu(), status


def _assert_parity(out, args, label=""):
    dtype = args["q"].dtype
    ref32 = PO.hstu_paged_forward(**args, round_p=False, out_dtype=torch.float32)
    assert out.shape == ref32.shape and out.dtype == dtype, label
    assert torch.isfinite(out.float()).all(), label
    scale = max(ref32.abs().max().item(), 1e-30)
    err = (out.float() - ref32).abs().max().item()
    if dtype == FP32:
        torch.testing.assert_close(out, ref32, rtol=1e-5, atol=1e-5, msg=lambda m: f"{label}: {m}")
        assert err <= 2e-5 * scale, (label, err, scale)
        return
    lowp = PO.hstu_paged_forward(**args)
    torch.testing.assert_close(out.float(), ref32, rtol=1e-2, atol=1e-2, msg=lambda m: f"{label}: {m}")
    ok, detail = O.double_reference_ok(out, lowp, ref32, multiplier=5)
    assert ok, (label, detail)
    assert err <= (2e-2 if dtype == BF16 else 4e-3) * scale, (label, err, scale)


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_gpu_fixtures_of_the_reference_goldens(name):
    fx = load_fixture(name)
    args = fixture_args(fx)
    out, status = _run(args)
    assert status == 0
    dtype = args["q"].dtype
    if dtype == FP32:
        torch.testing.assert_close(out, fx["out_torch_fp32"], rtol=1e-5, atol=1e-5)
    else:
        ok, detail = O.double_reference_ok(out, fx["out_torch_lowp"], fx["out_torch_fp32"], multiplier=5)
        assert ok, detail
        atol = 5e-3 if dtype == BF16 else 1e-3   # test_hstu_paged.py:474-479
        assert O.outlier_fraction_ok(out, fx["out_torch_lowp"], atol, atol)
    _assert_parity(out, args, label=name)


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,D", [(1, 4, 32), (32, 8, 128), (1, 8, 128), (32, 4, 32), (16, 4, 64)])
@pytest.mark.parametrize("dtype", [BF16, FP32, FP16])
@pytest.mark.parametrize("hist,cand", [(100, 0), (200, 25), (750, 80)])
@pytest.mark.parametrize("page", [32, 128, 256])
@pytest.mark.parametrize("prev", [True, False])
def test_gpu_reference_grid(B, H, D, dtype, hist, cand, page, prev):
    if dtype == FP32 and B * hist > 3200:
        B = 2                                   # the fp32 oracle is slow; the kernels behind it do not depend on B
    if dtype != BF16 and (page == 128 or hist == 750) and B > 1:
        pytest.skip("bf16 carries the full grid; the other dtypes a cross-section")
    args = make_paged_case(B, H, H, D, hist, cand, page, prev, dtype, seed=B + hist + page)
    out, status = _run(args)
    assert status == 0
    _assert_parity(out, args, label=f"B{B} H{H} D{D} {dtype} hist{hist} cand{cand} page{page} prev{prev}")


@pytest.mark.gpu
def test_gpu_long_history_gqa_and_custom_mask():
    args = make_paged_case(3, 8, 2, 128, 2048, 300, 128, True, BF16, seed=5)
    out, status = _run(args)
    assert status == 0
    _assert_parity(out, args, label="long gqa")
    args = make_paged_case(3, 2, 2, 64, 150, 20, 32, False, BF16, seed=6, mask_type=3)
    out, status = _run(args)
    assert status == 0
    _assert_parity(out, args, label="custom mask")
    args = make_paged_case(2, 2, 2, 64, 90, 9, 24, True, BF16, seed=7)     # a page size that divides nothing
    out, status = _run(args)
    assert status == 0
    _assert_parity(out, args, label="page 24")


@pytest.mark.gpu
@pytest.mark.parametrize("D", [64, 128])
def test_gpu_nothing_uninitialised_is_read_from_the_workspace(D):
    """With 128-row pages the whole pages of the cache never pass through the staging tensors of the workspace: their
    rows there stay unwritten.  A workspace full of 0xFF bytes (NaN in every 16-bit float) must change nothing."""
    args = make_paged_case(6, 4, 2, D, 700, 40, 128, True, BF16, seed=11)
    clean, status = _run(args)
    assert status == 0
    dirty, status = _run(args, workspace_fill=0xFF)
    assert status == 0
    assert torch.isfinite(dirty.float()).all()
    assert torch.equal(clean, dirty)
    _assert_parity(dirty, args, label="page 128, workspace of NaNs")


@pytest.mark.gpu
def test_gpu_int32_metadata_and_torch_operator():
    import ops_rec_b200 as ops_rec
    args = make_paged_case(4, 4, 2, 64, 300, 30, 32, True, BF16, seed=9)
    cu = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in args.items()}
    i32 = lambda t: t.to(torch.int32)
    out = ops_rec.ascendc.attention.hstu_paged(
        cu["q"], cu["k"], cu["v"], cu["kv_cache"], None, None, 0, cu["max_seq_len"], cu["max_seq_len_k"],
        cu["silu_scale"], i32(cu["seq_offset"]), i32(cu["seq_offset_k"]), i32(cu["seq_offset_t"]),
        i32(cu["page_offsets"]), i32(cu["page_ids"]), i32(cu["last_page_len"]), i32(cu["num_target"]), 1, cu["alpha"])
    torch.cuda.synchronize()
    _assert_parity(out.cpu(), args, label="torch op, int32 metadata")


@pytest.mark.gpu
def test_gpu_inconsistent_page_table_is_flagged_not_followed():
    from ops_rec_b200 import cabi
    args = make_paged_case(3, 2, 2, 64, 100, 10, 32, False, BF16, seed=11)
    bad = dict(args, last_page_len=args["last_page_len"] + 5)           # cache length != seq_offset_k - targets
    _, status = _run(bad)
    assert status & cabi.ST_BAD_PAGES
    bad = dict(args, page_ids=args["page_ids"] + 10_000)                # page ids past the cache
    _, status = _run(bad)
    assert status & cabi.ST_BAD_PAGES
    out, status = _run(args)                                            # the context is still healthy
    assert status == 0
    _assert_parity(out, args, label="after bad page tables")
