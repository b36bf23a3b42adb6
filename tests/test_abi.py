"""The shared library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from cinnamon_b200 import build
    return build.build()


def _declared():
    text = open(os.path.join(ROOT, "include", "cinnamon_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cinn_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(built):
    lib = ctypes.CDLL(built)
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/cinnamon_b200.h but not exported"


def test_binding_table_matches_header(built):
    from cinnamon_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    assert _lib.lib.cinn_version() >= 100


def test_bad_arguments_are_reported_not_crashed(built):
    from cinnamon_b200 import _lib
    L = _lib.lib
    # null pointers / bad modes are rejected on the host before any CUDA call
    st = L.cinn_quant_rowwise(None, 0, 4, 128, 128, 1, None, None, 128, 0, 0, None)
    assert st == _lib.ERR_INVALID and "null" in _lib.last_error()
    st = L.cinn_quant_rowwise(ctypes.c_void_p(16), 0, 4, 128, 128, 1, ctypes.c_void_p(16), ctypes.c_void_p(16), 128, 0, 7, None)
    assert st == _lib.ERR_INVALID and "div_mode" in _lib.last_error()
    st = L.cinn_fp8_gemm(ctypes.c_void_p(16), ctypes.c_void_p(16), 1, ctypes.c_void_p(16), ctypes.c_void_p(16), 1, 1,
                         ctypes.c_void_p(16), 128, 128, 100, 0, 0, None)
    assert st == _lib.ERR_INVALID and "multiple of 16" in _lib.last_error()
    with pytest.raises(AssertionError):
        _lib.check(st, "cinn_fp8_gemm")
    # empty problems are a successful no-op
    assert L.cinn_quant_rowwise(None, 0, 0, 128, 128, 1, None, None, 128, 0, 0, None) == 0
    assert L.cinn_fp8_gemm(None, None, 1, None, None, 1, 1, None, 0, 128, 128, 0, 0, None) == 0


def test_cpu_tensors_assert_like_the_reference(built):
    import torch
    from cinnamon_b200 import kernels as K
    x = torch.randn(4, 128)
    for fn in (K.quantize_fp8_rowwise, K.quantize_fp8_blockwise):
        with pytest.raises(AssertionError, match="CUDA"):
            fn(x)
    with pytest.raises(AssertionError):
        K.dequantize_fp8(x.to(torch.float8_e4m3fn), torch.ones(1, 1))
    # FP8Linear on CPU is an unquantised linear, as in the reference (src/kernels.py:823-824)
    lin = K.FP8Linear(128, 256)
    assert torch.equal(lin(x), torch.nn.functional.linear(x, lin.weight))


def test_convert_to_fp8_selection_rules(built):
    import torch
    from cinnamon_b200 import kernels as K

    class Blk(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w1 = torch.nn.Linear(256, 512, bias=False)
            self.w3 = torch.nn.Linear(512, 256, bias=True)
            self.attn_proj = torch.nn.Linear(256, 256)
            self.router = torch.nn.Linear(256, 8)
            self.tiny = torch.nn.Linear(64, 256)

    m = torch.nn.Sequential(Blk())
    K.convert_to_fp8(m)
    b = m[0]
    assert isinstance(b.w1, K.FP8Linear) and b.w1.round_scale
    assert isinstance(b.w3, K.FP8Linear) and not b.w3.round_scale and b.w3.bias is not None
    assert type(b.attn_proj) is torch.nn.Linear and type(b.router) is torch.nn.Linear and type(b.tiny) is torch.nn.Linear
    assert sorted(n for n, _ in b.w1.named_parameters()) == ["weight"]
