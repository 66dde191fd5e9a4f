"""Host-side logic of the CUDA library, checked without a GPU through the C ABI's host hooks:
the device mask predicate (same source compiled for the host) against the reference's create_causal_mask,
the K-tile range / "full tile" classifier, and the scheduler's work list."""
import ctypes as C

import numpy as np
import pytest

from oracle import hstu_oracle as O
from ops_rec_b200 import cabi
from tests._util import GOLDEN_DIR


def test_device_mask_predicate_matches_reference_masks():
    raw = np.load(GOLDEN_DIR + "/mask_grid.npz")
    for lq, lk, c, t, g in raw["grid"].tolist():
        want = np.unpackbits(raw[f"m_{lq}_{lk}_{c}_{t}_{g}"])[: lq * lk].reshape(lq, lk).astype(bool)
        got = cabi.debug_mask(lq, lk, c, t, g, 0)
        assert np.array_equal(got, want), (lq, lk, c, t, g)


@pytest.mark.parametrize("lq,lk", [(1, 1), (127, 127), (128, 128), (129, 129), (255, 255), (256, 256), (257, 257),
                                    (300, 340), (513, 513), (700, 700)])
def test_mask_predicate_boundaries_vs_oracle(lq, lk):
    # the reference's boundary grid: ctx in {255,256,257}, target in {511,512} (test_hstu_jagged.py:285-308)
    for c in (0, 6, 255, 256, 257):
        for t in (0, 1, 30, 511, 512):
            for g in (0, 1, 3):
                if c + t > lq:
                    continue
                assert np.array_equal(cabi.debug_mask(lq, lk, c, t, g, 0), O.hstu_mask(lq, lk, c, t, g, 0))
    assert cabi.debug_mask(lq, lk, 0, 0, 0, 2).all()


@pytest.mark.parametrize("rows,bn", [(128, 128), (32, 32)])
def test_tile_range_and_full_classifier(rows, bn):
    rng = np.random.default_rng(3)
    cases = [(1, 1, 0, 0, 0), (129, 129, 0, 0, 0), (300, 300, 6, 30, 1), (300, 340, 0, 17, 3), (513, 513, 257, 0, 1),
             (700, 700, 0, 512, 1), (640, 640, 130, 40, 3)]
    for _ in range(12):
        lk = int(rng.integers(1, 900))
        lq = int(rng.integers(1, lk + 1))
        t = int(rng.integers(0, min(lq, 64) + 1))
        c = int(rng.integers(0, max(1, lq - t) + 1)) if rng.random() < 0.5 else 0
        c = min(c, lq - t)
        cases.append((lq, lk, c, t, int(rng.integers(0, 4))))
    for lq, lk, c, t, g in cases:
        for mask_type in (0, 2):
            m = O.hstu_mask(lq, lk, c, t, g, mask_type)
            for r0 in range(0, lq + rows, rows):
                n, bits = cabi.debug_tiles(lq, lk, c, t, g, mask_type, r0, rows, bn)
                if r0 >= lq:
                    assert n == 0
                    continue
                sub = m[r0:r0 + rows]
                assert n <= (lk + bn - 1) // bn
                # nothing visible beyond the visited range ...
                assert not sub[:, n * bn:].any(), (lq, lk, c, t, g, r0)
                # ... and the last visited tile is not empty (no wasted tile)
                if n > 0:
                    assert sub[:, (n - 1) * bn:n * bn].any(), (lq, lk, c, t, g, r0)
                # "full" must never be claimed for a tile with a hidden element
                for tile in range(min(n, 64)):
                    if bits >> tile & 1:
                        blk = sub[:, tile * bn:(tile + 1) * bn]
                        assert blk.shape[1] == bn and blk.all(), (lq, lk, c, t, g, r0, tile)


def _lengths(kind, B, rng):
    if kind == "uniform":
        return rng.integers(1, 1025, B)
    if kind == "lognormal":
        return np.clip(np.rint(rng.lognormal(np.log(2048), 0.6, B)), 64, 8192).astype(np.int64)
    return np.array([0, 1, 255, 256, 257, 0, 512, 513, 20480][:B])


@pytest.mark.parametrize("kind,B,H", [("uniform", 32, 4), ("lognormal", 64, 8), ("edge", 9, 3)])
def test_work_list_covers_every_q_pair_exactly_once(kind, B, H):
    rng = np.random.default_rng(0)
    L = _lengths(kind, B, rng)
    off = np.concatenate([[0], np.cumsum(L)])
    items, status = cabi.plan_host(off, H)
    assert status == 0
    want = {(b, h, p) for b in range(len(L)) for h in range(H) for p in range((int(L[b]) + 255) // 256)}
    got = [(int(b), int(hp) >> 16, int(hp) & 0xFFFF) for b, hp in items]
    assert len(got) == len(set(got)) == len(want)
    assert set(got) == want
    pairs = [(int(L[b]) + 255) // 256 for b, _, _ in got]
    if H * (int(off[-1]) // 256) < 8 * 148:
        # a call with few items: by steps - the last q-pairs of all sequences first (a q-pair's cost grows with its
        # number), inside a number the sequences with the most pairs first, heads of a sequence together
        numbers = [p for _, _, p in got]
        assert numbers == sorted(numbers, reverse=True)
        for (b0, h0, p0), (b1, h1, p1), n0, n1 in zip(got, got[1:], pairs, pairs[1:]):
            if p0 == p1:
                assert n0 >= n1
                assert (b1, h1) == (b0, h0 + 1) or (b1 != b0 and h0 == H - 1 and h1 == 0)
    else:
        # longest sequences first; inside a (sequence, head) the heaviest q-pair first
        assert pairs == sorted(pairs, reverse=True)
        for (b0, h0, p0), (b1, h1, p1) in zip(got, got[1:]):
            if (b0, h0) == (b1, h1):
                assert p1 == p0 - 1


def test_work_list_flags_inconsistent_inputs():
    off = np.array([0, 10, 5, 20])  # not monotone
    _, status = cabi.plan_host(off, 2)
    assert status & cabi.ST_BAD_OFFSETS
    off = np.array([0, 300, 600])
    _, status = cabi.plan_host(off, 2, max_seq_len=256)
    assert status & cabi.ST_LEN_GT_MAX
    _, status = cabi.plan_host(off, 2, num_context=[200, 0], num_target=[150, 0])
    assert status & cabi.ST_BAD_CTX_TARGET
    items, status = cabi.plan_host(off, 2, num_context=[200, 0], num_target=[100, 0])
    assert status == 0 and len(items) == 2 * 2 * 2


def test_overlapping_offsets_describe_more_items_than_the_list_is_sized_for():
    # The workspace is sized from total_q (heads * (total_q / 256 + batch) items).  Offsets that run back and forth
    # between 0 and T describe far more q-pairs than that; the plan reports them (and flags the offsets), and the
    # device clamps its work list to the capacity it was given instead of reading past it.
    T, B, H = 4096, 64, 4
    off = np.array([T if i % 2 else 0 for i in range(B + 1)], dtype=np.int64)
    items, status = cabi.plan_host(off, H, total_q=T)
    assert status & cabi.ST_BAD_OFFSETS
    bound = H * (T // 256 + B)
    assert len(items) == bound + 1            # the plan stops one past the bound it was given room for ...
    n, _ = cabi.plan_host(off, H, total_q=T, count_only=True)
    assert n > bound                          # ... and counts more than the bound
