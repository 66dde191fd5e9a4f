"""Operator groups, named as in the reference package (ops_rec/ascendc/__init__.py)."""
from . import attention  # noqa: F401
from . import activation  # noqa: F401
