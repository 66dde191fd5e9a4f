"""Synthetic HSTU workloads (lengths, targets, work model) and the multi-GPU batch partition.

Everything here is host-side numpy: which sequences exist, how long they are, how much useful arithmetic and
compulsory memory traffic the forward has, and which rank gets which sequence.  Nothing here computes attention.

Generator rules (fixed so that every run sees the same workload): `rng = numpy.random.default_rng(seed)`;
uniform lengths `rng.integers(lo, hi + 1, B)`; lognormal lengths `clip(rint(rng.lognormal(mu, sigma, B)), lo, hi)`;
targets drawn after the lengths from the same rng and clamped to L - 1.

Work model: with n = L - T history rows and T target rows (each target sees the history and itself),
pairs(L, T) = n(n+1)/2 + T(n+1); FLOPs = heads * (2*Dqk + 2*Dv) * sum(pairs); bytes = q + k + v + out
(+ the visible part of the bias).  Masked-out positions, SiLU and scaling are not counted.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Workload:
    name: str
    batch: int
    heads: int
    dim: int
    max_seq_len: int
    lengths: np.ndarray
    targets: np.ndarray | None = None
    rab: str | None = None            # None | "batch" ([B,H,S,S]) | "shared" ([H,S,S], same for all sequences)
    dtype: str = "bf16"
    value_scale: float = 0.5
    alpha: float = field(default=0.0)
    target_group_size: int = 0

    def __post_init__(self):
        if not self.alpha:
            self.alpha = 1.0 / self.dim
        if self.targets is not None and not self.target_group_size:
            self.target_group_size = 1

    @property
    def tokens(self):
        return int(self.lengths.sum())

    def offsets(self):
        return np.concatenate([[0], np.cumsum(self.lengths)]).astype(np.int64)

    def pairs(self):
        L = self.lengths.astype(np.int64)
        T = self.targets.astype(np.int64) if self.targets is not None else np.zeros_like(L)
        n = L - T
        return n * (n + 1) // 2 + T * (n + 1)

    def flops(self):
        return float(self.heads * 4 * self.dim * self.pairs().sum())

    def bytes(self, esize=2):
        qkvo = 4 * self.tokens * self.heads * self.dim * esize
        if self.rab == "batch":
            qkvo += int(self.heads * self.pairs().sum()) * esize
        elif self.rab == "shared":
            S = self.max_seq_len
            qkvo += self.heads * S * (S + 1) // 2 * esize
        return float(qkvo)

    def subset(self, idx, name=None):
        idx = np.asarray(idx, dtype=np.int64)
        return Workload(name or self.name, len(idx), self.heads, self.dim, self.max_seq_len, self.lengths[idx],
                        None if self.targets is None else self.targets[idx], self.rab, self.dtype,
                        self.value_scale, self.alpha, self.target_group_size)


def _uniform(rng, lo, hi, B):
    return rng.integers(lo, hi + 1, B).astype(np.int64)


def _lognormal(rng, mu, sigma, lo, hi, B):
    return np.clip(np.rint(rng.lognormal(mu, sigma, B)), lo, hi).astype(np.int64)


def make_workload(name, seed=0):
    """The five named workloads: cfg1 (fp32 golden case) ... cfg5 (serving-shaped ranking batch)."""
    rng = np.random.default_rng(seed)
    if name == "cfg1":
        return Workload(name, 4, 2, 32, 128, _uniform(rng, 1, 128, 4), dtype="fp32", value_scale=1.0)
    if name == "cfg2":
        return Workload(name, 32, 4, 128, 1024, _uniform(rng, 256, 1024, 32))
    if name == "cfg3":
        L = _uniform(rng, 256, 1024, 32)
        T = np.minimum(rng.integers(0, 33, 32), L - 1).astype(np.int64)
        return Workload(name, 32, 4, 128, 1024, L, T, rab="batch")
    if name == "cfg4":
        return Workload(name, 256, 8, 128, 8192, _lognormal(rng, np.log(2048), 0.6, 64, 8192, 256))
    if name == "cfg5":
        L = _lognormal(rng, np.log(200), 0.8, 8, 2048, 4096)
        T = np.minimum(rng.integers(1, 65, 4096), L - 1).astype(np.int64)
        return Workload(name, 4096, 4, 64, 2048, L, T, rab="shared")
    raise ValueError(f"unknown workload {name!r}")


def partition_lpt(lengths, world_size):
    """Greedy longest-processing-time partition of sequences over ranks by cost L*(L+1) (proportional to the
    useful FLOPs of a causal sequence).  Returns a list of index arrays, one per rank, each in ascending order
    of the original index.  Sequences are never split."""
    lengths = np.asarray(lengths, dtype=np.int64)
    cost = lengths * (lengths + 1)
    order = np.argsort(-cost, kind="stable")
    load = np.zeros(world_size, dtype=np.int64)
    buckets = [[] for _ in range(world_size)]
    for i in order:
        r = int(np.argmin(load))
        buckets[r].append(int(i))
        load[r] += cost[i]
    return [np.array(sorted(b), dtype=np.int64) for b in buckets]


def imbalance(lengths, parts):
    """(max / mean) of the per-rank FLOP cost and of the per-rank token count."""
    lengths = np.asarray(lengths, dtype=np.int64)
    cost = np.array([(lengths[p] * (lengths[p] + 1)).sum() for p in parts], dtype=np.float64)
    toks = np.array([lengths[p].sum() for p in parts], dtype=np.float64)
    return float(cost.max() / cost.mean()), float(toks.max() / toks.mean())


def materialize(w: Workload, device, seed=1, index_dtype=None):
    """Random tensors for a workload on `device` (torch).  Returns the keyword arguments of the operator."""
    import torch

    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[w.dtype]
    gen = torch.Generator(device=device).manual_seed(seed)
    T, H, D = w.tokens, w.heads, w.dim

    def rnd(*shape, scale):
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * scale).to(dtype)

    q, k, v = (rnd(T, H, D, scale=w.value_scale) for _ in range(3))
    bias = None
    if w.rab == "batch":
        bias = rnd(w.batch, H, w.max_seq_len, w.max_seq_len, scale=0.1)
    elif w.rab == "shared":
        bias = rnd(H, w.max_seq_len, w.max_seq_len, scale=0.1)
    idt = index_dtype or torch.int64
    off = torch.from_numpy(w.offsets()).to(device=device, dtype=idt)
    tgt = torch.from_numpy(w.targets).to(device=device, dtype=idt) if w.targets is not None else None
    return dict(q=q, k=k, v=v, mask=None, attn_bias=bias, mask_type=0, max_seq_len=w.max_seq_len, silu_scale=0.0,
                seq_offset=off, num_context=None, num_target=tgt, target_group_size=w.target_group_size,
                alpha=w.alpha)
