"""`ops_rec.ascendc.activation` namespace (reference: ops_rec/ascendc/activation/__init__.py): like the attention
namespace it proxies every operator registered under torch.ops.ops_rec - the reference's group packages do not
partition the operators either - so `ln_mul` and `distance_in_linear_silu` are found here as its users expect.
"""
from __future__ import annotations

import torch

_NS = torch.ops.ops_rec


def _available():
    """Every operator name registered under ops_rec:: (overload names stripped)."""
    names = {n.split("::", 1)[1].split(".", 1)[0] for n in torch._C._dispatch_get_all_op_names()
             if n.startswith("ops_rec::")}
    return sorted(names)


# Export what is registered at import time, so that `from ops_rec.ascendc.activation import <op>` works
# (ops_rec/ascendc/activation/__init__.py:31-36 does the same with dir(torch.ops.ops_rec)).
__all__ = _available()
for _name in __all__:
    globals()[_name] = getattr(_NS, _name)


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    if hasattr(_NS, name):
        return getattr(_NS, name)
    raise AttributeError(
        f"module 'ops_rec.ascendc.activation' has no attribute '{name}'. Operator '{name}' is not supported or not "
        f"compiled for this device. Available ops: {_available()}")


def __dir__():
    return sorted(set(list(globals().keys()) + _available()))
