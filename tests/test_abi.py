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


def test_host_call_launch_plans():
    """The launch sizes of the host-buffer call need no GPU to compute: they sum to the batch, a
    fast link gives shrinking launches of whole waves with a single wave last, a slow link equal
    launches of about two waves, and a link in between a gentler shrink."""
    L = _native.lib()
    sizes = (ctypes.c_int * 16)()

    def plan(n, gbps, mode=0, sms=148):
        k = L.bf_host_plan(n, sms, mode, gbps, sizes)
        assert 1 <= k <= 16
        got = list(sizes[:k])
        assert sum(got) == n and min(got) > 0
        return got

    wave = 148 * 4
    assert plan(4096, 0.0) == [3504, 592] == plan(4096, 55.0) == plan(4096, 12.0, mode=1)
    assert plan(4096, 26.0) == [2320, 1184, 592]               # copying 2.95 times faster than evaluating
    slow = plan(4096, 12.0)
    assert slow == plan(4096, 55.0, mode=2) and slow[-1] == wave and len(slow) == 4
    assert max(slow[:-1]) - min(slow[:-1]) < 4 and max(slow) <= 2 * wave
    assert plan(100, 55.0) == [100] == plan(100, 5.0)
    for n in (1, 591, 592, 593, 5000, 65536, 131072, 1 << 20):
        for gbps in (0.0, 3.0, 9.0, 14.0, 20.0, 40.0, 80.0):
            for mode in (0, 1, 2):
                got = plan(n, gbps, mode)
                if mode == 1:        # the remainder first, then whole waves, ever fewer
                    assert len(got) == 1 or all(m % wave == 0 for m in got[1:])
                    assert got[1:] == sorted(got[1:], reverse=True)
    assert L.bf_host_plan(0, 148, 0, 0.0, sizes) == -1
    assert L.bf_host_plan(10, 148, 3, 0.0, sizes) == -1
