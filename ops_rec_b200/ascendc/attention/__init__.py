"""`ops_rec.ascendc.attention` namespace: every operator registered under torch.ops.ops_rec is reachable by name.

Same proxy behaviour as the reference (ops_rec/ascendc/attention/__init__.py:31-49, identical in all four group
packages): every registered name resolves to the torch OpOverloadPacket (so `hstu_jagged(...)` picks `.equal` or
`.delta` from the argument types, and `hstu_jagged.equal(...)` works); unknown names raise AttributeError listing
what is available.
"""
from __future__ import annotations

import torch

_NS = torch.ops.ops_rec


def _available():
    """Every operator name registered under ops_rec:: (overload names stripped)."""
    names = {n.split("::", 1)[1].split(".", 1)[0] for n in torch._C._dispatch_get_all_op_names()
             if n.startswith("ops_rec::")}
    return sorted(names)


# Export what is registered at import time, so that `from ops_rec.ascendc.attention import <op>` works
# (ops_rec/ascendc/attention/__init__.py:31-36 does the same with dir(torch.ops.ops_rec)).
__all__ = _available()
for _name in __all__:
    globals()[_name] = getattr(_NS, _name)


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    if hasattr(_NS, name):
        return getattr(_NS, name)
    raise AttributeError(
        f"module 'ops_rec.ascendc.attention' has no attribute '{name}'. Operator '{name}' is not supported or not "
        f"compiled for this device. Available ops: {_available()}")


def __dir__():
    return sorted(set(list(globals().keys()) + _available()))
