"""Put the reference's own CPU implementation of the forward where the benchmark's reference arm finds it.

    python oracle/fetch_reference.py /path/to/ops-rec

Copies, unmodified, the three files of the reference's PyTorch golden into `baseline/_ref/hstu_v2/` (a folder that is
not part of the repository history):

    ascendc/attention/hstu_v2/test/pytest/backend/pytorch_native_backend.py   Kernel._forward_impl (the golden)
    ascendc/attention/hstu_v2/test/pytest/backend/common.py                   jagged <-> dense helpers it imports
    ascendc/attention/hstu_v2/test/pytest/utils/data.py                       TestDataGenerator.create_causal_mask

`bench.py --impl reference` and its `cpu_baseline` leg time `Kernel._forward_impl` from there when the files are
present ("kind": "reference"), and fall back to the restatement in oracle/hstu_oracle.py otherwise ("kind": "port").
This is test / measurement infrastructure; the library never imports any of it.
"""
from __future__ import annotations

import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref", "hstu_v2")
FILES = (
    ("ascendc/attention/hstu_v2/test/pytest/backend/pytorch_native_backend.py", "backend/pytorch_native_backend.py"),
    ("ascendc/attention/hstu_v2/test/pytest/backend/common.py", "backend/common.py"),
    ("ascendc/attention/hstu_v2/test/pytest/utils/data.py", "utils/data.py"),
)


def fetch(ref_root):
    """Returns True when all files were copied, False when the reference tree is not there."""
    if not all(os.path.isfile(os.path.join(ref_root, src)) for src, _ in FILES):
        return False
    for src, dst in FILES:
        target = os.path.join(DEST, dst)
        os.makedirs(os.path.dirname(target), exist_ok=True)
        shutil.copyfile(os.path.join(ref_root, src), target)
    return True


def load():
    """(Kernel class, create_causal_mask) of the fetched reference files, or None when they are absent.  The files are
    loaded by path under a synthetic package so that the NPU-only sibling backends are never imported, and
    utils/data.py gets an empty stand-in for the `torch_npu` module it imports at the top."""
    import importlib.util
    import types

    paths = [os.path.join(DEST, dst) for _, dst in FILES]
    if os.environ.get("HSTU_NO_REFERENCE_FILES") or not all(os.path.isfile(p) for p in paths):
        return None
    pkg = types.ModuleType("hstu_ref_backend")
    pkg.__path__ = [os.path.join(DEST, "backend")]
    sys.modules["hstu_ref_backend"] = pkg
    mods = {}
    for name in ("common", "pytorch_native_backend"):
        spec = importlib.util.spec_from_file_location(f"hstu_ref_backend.{name}", os.path.join(DEST, "backend", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"hstu_ref_backend.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    sys.modules.setdefault("torch_npu", types.ModuleType("torch_npu"))
    spec = importlib.util.spec_from_file_location("hstu_ref_data", os.path.join(DEST, "utils", "data.py"))
    data = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(data)
    return mods["pytorch_native_backend"].Kernel, data.TestDataGenerator.create_causal_mask


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python oracle/fetch_reference.py <path to the ops-rec tree>")
    ok = fetch(sys.argv[1])
    print("copied to" if ok else "reference tree not found; nothing copied to", DEST)
    sys.exit(0 if ok else 1)
