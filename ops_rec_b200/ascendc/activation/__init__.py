"""`ops_rec.ascendc.activation` namespace (reference: ops_rec/ascendc/activation/__init__.py): the operators of the
steps either side of the attention in an HSTU layer that this package provides.  Same proxy rule as the attention
namespace: known names resolve to the torch OpOverloadPacket, unknown names raise AttributeError."""
from __future__ import annotations

import torch

_OPS = ("ln_mul", "distance_in_linear_silu")


def _available():
    return [n for n in _OPS if hasattr(torch.ops.ops_rec, n)]


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    if name in _OPS and hasattr(torch.ops.ops_rec, name):
        return getattr(torch.ops.ops_rec, name)
    raise AttributeError(
        f"module 'ops_rec.ascendc.activation' has no operator '{name}'. Available ops: {_available()}")


def __dir__():
    return sorted(list(globals().keys()) + _available())
