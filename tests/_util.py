"""Shared helpers for the tests: fixture loading and seeded input generation."""
from __future__ import annotations

import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_fixture(name):
    """Load tests/golden/<name>.npz into a dict of torch tensors / numpy scalars (bf16 restored)."""
    raw = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for key in raw.files:
        arr = raw[key]
        if key.endswith("__bf16"):
            out[key[:-6]] = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
        elif key in ("meta", "alpha", "silu_scale"):
            out[key] = arr
        else:
            out[key] = torch.from_numpy(np.ascontiguousarray(arr))
    return out


def fixture_names():
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    return [n for n in names if n != "mask_grid" and not n.startswith(("dense_", "bwd_", "lnmul_", "linsilu_", "paged_"))]


def bwd_fixture_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "bwd_*.npz")))


def dense_fixture_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "dense_*.npz")))


def fixture_call_args(fx):
    """Operator arguments (reference schema names) for a loaded fixture."""
    B, Hq, Hk, Dqk, Dv, maxL, ctx, tgt, g, mask_type = (int(x) for x in fx["meta"])
    return dict(
        q=fx["q"], k=fx["k"], v=fx["v"], mask=fx.get("mask"), attn_bias=fx.get("rab"), mask_type=mask_type,
        max_seq_len=maxL, silu_scale=float(fx["silu_scale"]) if "grad" in fx else 0.0, seq_offset=fx["seq_offset"],
        num_context=fx["num_context"] if ctx else None, num_target=fx["num_target"] if tgt else None,
        target_group_size=g, alpha=float(fx["alpha"]), max_seq_len_k=maxL, seq_offset_k=fx["seq_offset_k"])


def make_case(B, Hq, Hk, Dqk, Dv, lo, hi, dtype, *, seed=0, rab=None, ctx=0, tgt=0, g=0, mask_type=0,
              delta=False, max_seq_len=None, value_scale=0.5, index_dtype=torch.int64, custom_mask=False):
    """Seeded jagged inputs in the spirit of the reference's jagged_data_gen
    (test_hstu_jagged.py:41-104): constant ctx/target per test, lengths = U[lo,hi] + ctx + target."""
    rng = np.random.default_rng(seed)
    gen = torch.Generator().manual_seed(seed + 1)
    base = rng.integers(lo, hi + 1, B)
    len_k = base + (ctx + tgt if mask_type == 0 else 0)
    len_q = np.maximum(1, len_k - rng.integers(0, 9, B)) if delta else len_k.copy()
    maxL = int(max_seq_len or max(len_k.max(), 1))
    offq = torch.from_numpy(np.concatenate([[0], np.cumsum(len_q)])).to(index_dtype)
    offk = torch.from_numpy(np.concatenate([[0], np.cumsum(len_k)])).to(index_dtype)
    Tq, Tk = int(offq[-1]), int(offk[-1])
    q = (torch.randn(Tq, Hq, Dqk, generator=gen) * value_scale).to(dtype)
    k = (torch.randn(Tk, Hk, Dqk, generator=gen) * value_scale).to(dtype)
    v = (torch.randn(Tk, Hk, Dv, generator=gen) * value_scale).to(dtype)
    bias = None
    if rab == "batch":
        bias = (torch.randn(B, Hq, maxL, maxL, generator=gen) * 0.1).to(dtype)
    elif rab == "shared3":
        bias = (torch.randn(Hq, maxL, maxL, generator=gen) * 0.1).to(dtype)
    elif rab == "shared4":
        bias = (torch.randn(1, Hq, maxL, maxL, generator=gen) * 0.1).to(dtype)
    mask = None
    if custom_mask:
        mask = torch.randint(0, 2, (B, Hq, maxL, maxL), generator=gen).to(dtype)
        mask_type = 3
    return dict(
        q=q, k=k, v=v, mask=mask, attn_bias=bias, mask_type=mask_type, max_seq_len=maxL, silu_scale=0.0,
        seq_offset=offq, num_context=torch.full((B,), ctx, dtype=index_dtype) if ctx else None,
        num_target=torch.full((B,), tgt, dtype=index_dtype) if tgt else None, target_group_size=g,
        alpha=1.0 / Dqk, max_seq_len_k=maxL, seq_offset_k=offk)
