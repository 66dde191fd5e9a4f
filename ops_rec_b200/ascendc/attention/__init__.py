"""`ops_rec.ascendc.attention` namespace: every operator registered under torch.ops.ops_rec is reachable by name.

Same proxy behaviour as the reference (ops_rec/ascendc/attention/__init__.py:31-49): known names resolve to the
torch OpOverloadPacket (so `hstu_jagged(...)` picks `.equal` or `.delta` from the argument types, and
`hstu_jagged.equal(...)` works); unknown names raise AttributeError listing what is available.
"""
from __future__ import annotations

import torch

_OPS = ("hstu_jagged", "hstu_jagged_backward", "hstu_dense")


def _available():
    return [n for n in _OPS if hasattr(torch.ops.ops_rec, n)]


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    if name in _OPS and hasattr(torch.ops.ops_rec, name):
        return getattr(torch.ops.ops_rec, name)
    raise AttributeError(
        f"module 'ops_rec.ascendc.attention' has no operator '{name}'. Available ops: {_available()}")


def __dir__():
    return sorted(list(globals().keys()) + _available())
