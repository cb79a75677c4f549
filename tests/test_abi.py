"""The C-ABI library builds for sm_100a, loads without a GPU, and exports every symbol
the public header declares."""
import ctypes
import os
import re

from conftest import ROOT
from brokefish_b200 import _native


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "brokefish_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bf_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_the_header():
    _native.build()
    L = ctypes.CDLL(_native.LIB_PATH)
    names = declared_symbols()
    assert sorted(_native.EXPORTS) == names
    for n in names:
        assert hasattr(L, n), n
    assert b"sm_100a" in _native.lib().bf_version()


def test_argument_errors_need_no_gpu():
    L = _native.lib()
    out = ctypes.c_void_p(0)
    assert L.bf_create(None, 0, 0, ctypes.byref(out)) == -1
    assert b"blob" in L.bf_last_error()
    assert L.bf_forward(None, None, None, None, None, 4, None, None, None, None) == -1
    assert L.bf_destroy(None) == 0
    assert L.bf_launch_count(None) == 0


def test_kernel_constants_match_the_packer():
    """The quantisation ranges compiled into the kernel equal the host packer's (the reference
    checks the same pair of facts, tests/test_quant.py:233-269)."""
    from brokefish_b200.nn import quant
    L = _native.lib()
    s, u = ctypes.c_int(0), ctypes.c_int(0)
    L.bf_int8_q_max(ctypes.byref(s), ctypes.byref(u))
    assert (s.value, u.value) == (127, 255) == (int(quant.Q_MAX_S8), int(quant.Q_MAX_U8))
    assert L.bf_fp8_q_max() == 8.0 == quant.Q_MAX
    L.bf_int8_q_max(None, None)                              # null outputs are allowed
