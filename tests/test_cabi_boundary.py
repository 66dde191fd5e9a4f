"""The drop-in boundary without a GPU: the shared library exports every symbol the header declares, rejects bad
arguments with the reference's error classes, and the torch operator keeps the reference's schema."""
import ctypes as C
import os
import re

import pytest
import torch

from ops_rec_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = "".join(open(os.path.join(ROOT, "include", n)).read() for n in ("hstu_b200.h", "hstu_b200_testing.h"))
    return sorted(set(re.findall(r"HSTU_API\s+[\w\s\*]+?\b((?:hstu|ops_rec)_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = cabi.load()
    declared = _declared_functions()
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/*.h but not exported"
    assert set(declared) == set(cabi.EXPORTS)
    assert lib.hstu_b200_version() >= 100


def test_struct_layout_matches_header():
    # the C side refuses a struct of a different size
    a = cabi.HstuJaggedArgs()
    a.struct_bytes = C.sizeof(cabi.HstuJaggedArgs) - 8
    n = C.c_uint64()
    assert cabi.load().hstu_jagged_fwd_get_workspace_size(C.byref(a), C.byref(n)) == -2
    assert b"struct_bytes" in cabi.load().hstu_last_error()


class _Fake:
    """Stands in for a device tensor: shape / dtype only, address 256-aligned and never dereferenced."""

    def __init__(self, *shape, dtype=torch.bfloat16, addr=0x7F0000000000):
        self.shape, self.dtype, self._addr = shape, dtype, addr

    def dim(self):
        return len(self.shape)

    def element_size(self):
        return torch.empty(0, dtype=self.dtype).element_size()


def _args(**kw):
    H, D = kw.pop("H", 4), kw.pop("D", 128)
    dtype = kw.pop("dtype", torch.bfloat16)
    q = _Fake(1000, H, D, dtype=dtype)
    k = _Fake(1000, kw.pop("Hk", H), D, dtype=dtype)
    v = _Fake(1000, k.shape[1], kw.pop("Dv", D), dtype=dtype)
    off = _Fake(9, dtype=torch.int64)
    base = dict(mask_type=0, max_seq_len=512, alpha=1.0)
    base.update(kw)
    a, _ = cabi.make_args(q, k, v, _Fake(1000, H, v.shape[2], dtype=dtype), off, ptr=lambda t: t._addr, **base)
    return a


def test_workspace_size_and_kernel_choice():
    a = _args()
    assert cabi.kernel_kind(a) == 1                     # bf16 d128 -> tensor-core kernel
    need = cabi.workspace_size(a)
    assert need >= 256 + 8 * 4 * (1000 // 256 + 8) and need % 256 == 0
    assert cabi.kernel_kind(_args(dtype=torch.float32)) == 0
    assert cabi.workspace_size(_args(dtype=torch.float32)) == 256
    assert cabi.kernel_kind(_args(D=96, Dv=96)) == 0    # head dim without a tensor-core instance
    assert cabi.kernel_kind(_args(D=64, Dv=64)) == 1
    assert cabi.kernel_kind(_args(D=128, Dv=64)) == 0   # dim_qk != dim_v
    assert cabi.kernel_kind(_args(flags=cabi.FLAG_FORCE_GENERIC)) == 0
    assert cabi.kernel_kind(_args(dtype=torch.float16, H=8, Hk=2)) == 1


@pytest.mark.parametrize("kw,needle", [
    (dict(mask_type=1), "triu"),
    (dict(mask_type=4), "maskType expect in [0, 3]"),
    (dict(mask_type=3), "custome mask"),
    (dict(max_seq_len=0), "maxSeqLen expect in [1, 20480]"),
    (dict(max_seq_len=20481), "maxSeqLen expect in [1, 20480]"),
    (dict(H=4, Hk=3), "divisible"),
    (dict(H=17, Hk=17), "head count"),
    (dict(Dv=24), "multiple of 16"),
    (dict(D=520, Dv=512), "head dim"),
    (dict(target_group_size=-1), "target_group_size"),
])
def test_invalid_arguments_are_rejected(kw, needle):
    with pytest.raises(cabi.HstuError) as e:
        cabi.workspace_size(_args(**kw))
    assert e.value.code == -2 and needle in str(e.value)
    assert isinstance(e.value, RuntimeError)   # the error type the reference's error tests expect


def test_launch_refuses_missing_or_bad_workspace():
    a = _args()
    lib = cabi.load()
    assert lib.hstu_jagged_fwd(C.byref(a), None, 0, None) == -3
    assert lib.hstu_jagged_fwd(C.byref(a), 0x7F0000000010, 1 << 20, None) == -3   # misaligned
    assert lib.hstu_jagged_fwd(C.byref(a), 0x7F0000000100, 256, None) == -3       # too small
    assert b"needed" in lib.hstu_last_error()
    a.seq_offset_q = None
    assert lib.hstu_jagged_fwd(C.byref(a), 0x7F0000000100, 1 << 20, None) == -1
    assert lib.hstu_jagged_fwd(None, None, 0, None) == -1


def test_torch_operator_schema_is_the_reference_schema():
    import ops_rec_b200  # noqa: F401  (registers the operator)
    eq = torch.ops.ops_rec.hstu_jagged.equal._schema
    names = [a.name for a in eq.arguments]
    assert names == ["q", "k", "v", "mask", "attn_bias", "mask_type", "max_seq_len", "silu_scale", "seq_offset",
                     "num_context", "num_target", "target_group_size", "alpha", "deterministic"]
    de = torch.ops.ops_rec.hstu_jagged.delta._schema
    assert [a.name for a in de.arguments][6:11] == ["max_seq_len", "max_seq_len_k", "silu_scale", "seq_offset",
                                                    "seq_offset_k"]
    defaults = {a.name: a.default_value for a in eq.arguments if a.has_default_value()}
    assert defaults["mask_type"] == 0 and defaults["alpha"] == 1.0 and defaults["target_group_size"] == 0
    assert defaults["silu_scale"] == 0.0 and defaults["deterministic"] is False


def test_meta_dispatch_and_overload_resolution():
    import ops_rec_b200 as ops_rec
    hj = ops_rec.ascendc.attention.hstu_jagged
    q = torch.empty(10, 4, 64, device="meta", dtype=torch.bfloat16)
    k = torch.empty(12, 2, 64, device="meta", dtype=torch.bfloat16)
    v = torch.empty(12, 2, 32, device="meta", dtype=torch.bfloat16)
    off = torch.empty(3, device="meta", dtype=torch.int32)
    out = hj(q, k, v, None, None, 0, 16, 0.0, off, None, None, 0, 0.5)           # .equal
    assert out.shape == (10, 4, 32) and out.dtype == torch.bfloat16 and out.device.type == "meta"
    out = hj(q, k, v, None, None, 0, 16, 16, 0.0, off, off)                       # .delta
    assert out.shape == (10, 4, 32)
    with pytest.raises(AttributeError, match="Available ops"):
        ops_rec.ascendc.attention.fa_infer_with_arbitrary_func
    with pytest.raises(RuntimeError, match="3D"):
        hj(q[0], k, v, None, None, 0, 16, 0.0, off)


def test_cpu_tensors_are_refused_not_computed():
    import ops_rec_b200 as ops_rec
    q = torch.zeros(4, 1, 64, dtype=torch.bfloat16)
    off = torch.tensor([0, 4])
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops_rec.ascendc.attention.hstu_jagged(q, q, q, None, None, 0, 4, 0.0, off)
    with pytest.raises(cabi.HstuError, match="no CPU implementation"):
        cabi.hstu_jagged_forward(q, q, q, None, None, 0, 4, 0.0, off)
