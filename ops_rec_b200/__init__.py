"""B200-native HSTU jagged attention forward, a drop-in for `ops_rec.ascendc.attention.hstu_jagged`.

Importing this package loads the C-ABI library (CUDA kernels for sm_100a) and the torch shim that registers
`torch.ops.ops_rec.hstu_jagged` (overloads `.equal` and `.delta`) with the reference's schema strings
(ascendc/attention/hstu_v1/torch_extension/hstu_jagged_plugin.cpp:186-231), `hstu_jagged_backward` (same two
overloads) and the autograd formula that binds it to the forward.  The namespace mirrors the reference
package (ops_rec/__init__.py:223-236, ops_rec/ascendc/attention/__init__.py:31-49):

    import ops_rec_b200 as ops_rec
    out = ops_rec.ascendc.attention.hstu_jagged(q, k, v, None, rab, 0, max_seq_len, 0.0, seq_offset,
                                                None, num_target, 1, alpha)

`install_as_ops_rec()` additionally publishes the package under the name `ops_rec`, so unmodified user code
(`import ops_rec`) picks it up.  If a native library is missing the import fails; nothing falls back to Python.
"""
from __future__ import annotations

import os
import sys

from . import cabi

__version__ = "0.1.0"

_PKG = os.path.dirname(os.path.abspath(__file__))
SHIM_PATH = os.path.join(_PKG, "_torch_shim.so")
_loaded = False


def load_native():
    """Load libhstu_b200.so and the torch shim (idempotent). Raises ImportError if either is not built."""
    global _loaded
    if _loaded:
        return
    import torch

    cabi.load()
    if not os.path.exists(SHIM_PATH):
        raise ImportError(f"{SHIM_PATH} is missing: build it with `python ops_rec_b200/_build.py`.")
    torch.ops.load_library(SHIM_PATH)
    _loaded = True


def env_setup_path():
    """Counterpart of ops_rec.env_setup_path() (ops_rec/__init__.py:25-38): the directory holding the native
    libraries.  Nothing needs to be sourced for this implementation."""
    return _PKG


def install_as_ops_rec():
    """Publish this package as `ops_rec` (and its ascendc.attention sub-namespace) in sys.modules."""
    from . import ascendc
    from .ascendc import attention

    sys.modules.setdefault("ops_rec", sys.modules[__name__])
    sys.modules.setdefault("ops_rec.ascendc", ascendc)
    sys.modules.setdefault("ops_rec.ascendc.attention", attention)
    sys.modules.setdefault("ops_rec.ascendc.activation", ascendc.activation)
    return sys.modules["ops_rec"]


load_native()
from . import ascendc  # noqa: E402,F401
from . import autograd as _autograd  # noqa: E402

_autograd.register_autograd()
