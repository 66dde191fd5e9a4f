"""CPU oracle for `hstu_paged`: HSTU attention whose history keys / values live in a paged KV cache.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE (see oracle/hstu_oracle.py for who may import it).

It restates the two goldens of the reference:

  * the torch golden of the operator's test, ascendc/attention/hstu_v1/hstu_forward_v1/test/pytest/
    test_hstu_paged.py:203-277 (`_hstu_paged_kv_attention`: per sequence, K/V = every page of the sequence in
    page-table order, the last page cut to last_page_len, followed by the TARGET rows of the input k / v - the
    last num_target rows of the sequence's segment; the history rows of the input k / v are not used) feeding
    :130-200 (`_hstu_attention_maybe_from_cache`: S = Q.K^T, S += rab, S *= alpha, silu, / max_seq_len_q, * mask);
    its mask (:75-127, `generate_attn_mask`) is a lower triangle over the cache columns shifted by
    (cache length + targets - query rows), and the identity over the target columns;
  * the numpy golden ascendc/attention/hstu_v1/hstu_forward_v1/test/pytest/common.py:255-300
    (`get_golden_paged`: the same without alpha and with cache length == history length).

That mask is the composite mask of the jagged operator with len_k = cache length + targets, num_target targets
and target_group_size 1, so after the gather this oracle hands over to oracle.hstu_oracle.hstu_jagged_forward
(the `.delta` form: len_q = new history + targets <= len_k).

Parity is pinned: tests/golden/paged_*.npz hold inputs made by the reference test's own generators and the outputs
of both reference goldens (tests/golden/make_golden.py), and tests/test_paged.py checks this file against them.
"""
from __future__ import annotations

import torch

from . import hstu_oracle as O


def gather_paged_kv(k, v, kv_cache, seq_offset, page_offsets, page_ids, last_page_len, num_target):
    """(k_con, v_con, seq_offset_k): the keys / values the operator attends over, packed sequence by sequence.

    kv_cache [pages, 2, page_size, heads_k, dim] (0 = keys, 1 = values); pages page_ids[page_offsets[b] :
    page_offsets[b + 1]] belong to sequence b, the last of them holds last_page_len[b] rows.
    """
    off = [int(x) for x in seq_offset]
    po = [int(x) for x in page_offsets]
    ks, vs, offk = [], [], [0]
    page_size = kv_cache.shape[2]
    for b in range(len(off) - 1):
        t = int(num_target[b]) if num_target is not None else 0
        for p in range(po[b], po[b + 1]):
            n = int(last_page_len[b]) if p == po[b + 1] - 1 else page_size
            pid = int(page_ids[p])
            ks.append(kv_cache[pid, 0, :n])
            vs.append(kv_cache[pid, 1, :n])
        if t > 0:
            ks.append(k[off[b + 1] - t:off[b + 1]])
            vs.append(v[off[b + 1] - t:off[b + 1]])
        offk.append(sum(x.shape[0] for x in ks))
    empty = kv_cache.new_zeros((0,) + tuple(kv_cache.shape[3:]))
    k_con = torch.cat(ks) if ks else empty
    v_con = torch.cat(vs) if vs else empty
    return k_con.to(k.dtype), v_con.to(v.dtype), torch.tensor(offk, dtype=torch.int64)


def hstu_paged_forward(q, k, v, kv_cache, mask=None, attn_bias=None, mask_type=O.MASK_TRIL, max_seq_len=0,
                       max_seq_len_k=0, silu_scale=0.0, seq_offset=None, seq_offset_k=None, seq_offset_t=None,
                       page_offsets=None, page_ids=None, last_page_len=None, num_target=None, target_group_size=0,
                       alpha=1.0, **kw):
    """Argument order of ops_rec::hstu_paged (ascendc/attention/hstu_v1/torch_extension/hstu_paged_plugin.cpp:75-98).
    seq_offset_k must agree with the page table (checked); seq_offset_t (offsets of num_target) is implied by
    num_target and only checked.  Extra keywords go to the jagged oracle (round_p, out_dtype, ...)."""
    k_con, v_con, offk = gather_paged_kv(k, v, kv_cache, seq_offset, page_offsets, page_ids, last_page_len, num_target)
    if seq_offset_k is not None:
        assert [int(x) for x in seq_offset_k] == offk.tolist(), "seq_offset_k disagrees with the page table"
    if seq_offset_t is not None and num_target is not None:
        t = [int(x) for x in seq_offset_t]
        assert [t[i + 1] - t[i] for i in range(len(t) - 1)] == [int(x) for x in num_target]
    return O.hstu_jagged_forward(q, k_con, v_con, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset,
                                 None, num_target, target_group_size, alpha, max_seq_len_k=max_seq_len_k or None,
                                 seq_offset_k=offk, **kw)
