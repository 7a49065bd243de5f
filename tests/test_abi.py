"""The C-ABI library loads and exports every symbol the header declares; argument validation works
without touching a GPU."""
import ctypes
import os
import re

from torchlib_xpu_b200 import _build, cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200tbe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200tbe_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    _build.build_cabi()
    lib = cabi.lib()
    declared = _declared_symbols()
    assert declared, "no declarations found in include/b200tbe.h"
    for name in declared:
        assert hasattr(lib, name), "libb200tbe.so does not export %s" % name
    assert sorted(cabi.EXPORTS) == declared
    assert lib.b200tbe_abi_version() >= 1


def test_status_strings():
    lib = cabi.lib()
    assert lib.b200tbe_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert lib.b200tbe_status_string(code) not in (b"ok", b"unknown status")
    assert lib.b200tbe_status_string(-99) == b"unknown status"


def test_argument_validation_needs_no_gpu():
    lib = cabi.lib()
    assert lib.b200tbe_forward(None, None) == -1
    assert lib.b200tbe_nbit_forward(None, None) == -1
    assert lib.b200tbe_backward(None, None) == -1
    p = cabi.ForwardParams()
    p.T, p.B = 2, 3  # null pointers
    assert lib.b200tbe_forward(ctypes.byref(p), None) == -1
    p.T = 0          # empty problem: nothing to do, no pointer is read
    assert lib.b200tbe_forward(ctypes.byref(p), None) == 0
    s = cabi.JaggedShape()
    s.num_jagged_dims = 9
    assert lib.b200tbe_jagged_to_padded_dense(ctypes.byref(s), None, None, 0, None) == -4
    s.num_jagged_dims, s.offset_bytes, s.elem_bytes = 1, 8, 3
    assert lib.b200tbe_dense_to_jagged(ctypes.byref(s), None, None, None) == -4
    assert lib.b200tbe_radix_sort_pairs(None, None, None, None, -1, 4, 8, None, 0, None) == -1
    assert lib.b200tbe_radix_sort_scratch_bytes(0) >= 0
    assert lib.b200tbe_backward_scratch_bytes(1 << 20, 25, 128, 8) > (1 << 20) * 8
