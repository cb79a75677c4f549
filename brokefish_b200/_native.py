"""Build and load the C-ABI shared library (``libbrokefish_b200.so``).

The library is built in-tree with one ``nvcc`` line for sm_100a; there is no JIT cache
and no fallback: if the library is missing or does not load, every entry point of the
package that needs the GPU raises.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from typing import List, Optional

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
#: The in-tree library; ``BROKEFISH_B200_LIB`` points the loader at another build of it.
LIB_PATH = os.environ.get("BROKEFISH_B200_LIB") or os.path.join(PKG_DIR, "libbrokefish_b200.so")
SOURCES = [os.path.join(PKG_DIR, "csrc", "bf_encoder.cu")]
DEPS = SOURCES + [os.path.join(PKG_DIR, "csrc", name) for name in
                  ("bf_ptx.cuh", "bf_movegen.cuh", "bf_encoder_one.cuh")] + [
                      os.path.join(ROOT, "include", "brokefish_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-diag-suppress", "177,550"]

#: Every symbol ``include/brokefish_b200.h`` declares.
EXPORTS = ["bf_version", "bf_last_error", "bf_create", "bf_destroy", "bf_info", "bf_forward",
           "bf_forward_stage", "bf_forward_stage_at", "bf_forward_capture", "bf_forward_host", "bf_status",
           "bf_launch_count", "bf_profile", "bf_profile_read", "bf_profile_phases",
           "bf_forward_noalloc", "bf_noalloc_status", "bf_noalloc_forget", "bf_host_link_gbps", "bf_host_plan", "bf_selftest_umma", "bf_set_option", "bf_measure_i8_peak", "bf_forward_priors",
           "bf_forward_priors_host", "bf_selftest_timeout", "bf_movegen", "bf_step", "bf_random_ply",
           "bf_forward_leaves", "bf_measure_elementwise", "bf_forward_backbone", "bf_int8_q_max",
           "bf_fp8_q_max", "bf_terminal", "bf_hash", "bf_history_push",
           "bf_repetition_count"]


def nvcc_path() -> str:
    cand = os.environ.get("BROKEFISH_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set BROKEFISH_NVCC")
    return cand


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in DEPS)


def build(force: bool = False, verbose: bool = False, extra: Optional[List[str]] = None) -> str:
    """Compile the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [nvcc_path()] + NVCC_FLAGS + (extra or []) + ["-o", LIB_PATH] + SOURCES
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        print(" ".join(cmd))
        print(res.stdout)
        print(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed with code {res.returncode}:\n{res.stderr[-4000:]}")
    return LIB_PATH


_LIB = None


def lib() -> ctypes.CDLL:
    """The loaded library with argument types declared.  Raises if it is not built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU or PyTorch fallback for the evaluator)")
    L = ctypes.CDLL(LIB_PATH)
    vp, i32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    L.bf_version.restype = ctypes.c_char_p
    L.bf_last_error.restype = ctypes.c_char_p
    L.bf_create.argtypes = [vp, sz, i32, ctypes.POINTER(vp)]
    L.bf_destroy.argtypes = [vp]
    L.bf_info.argtypes = [vp, ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i32)]
    L.bf_forward.argtypes = [vp, vp, vp, vp, vp, i32, vp, vp, vp, vp]
    L.bf_forward_stage.argtypes = [vp, vp, vp, vp, i32, i32, vp, vp]
    L.bf_forward_stage_at.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, vp]
    L.bf_forward_capture.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, vp, vp]
    L.bf_forward_host.argtypes = [vp, vp, vp, vp, vp, i32, vp, vp, vp]
    L.bf_status.argtypes = [vp, ctypes.POINTER(i32)]
    L.bf_set_option.argtypes = [vp, i32, i32]
    L.bf_forward_priors.argtypes = [vp, vp, vp, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp]
    L.bf_selftest_timeout.argtypes = [i32, i32, ctypes.POINTER(i32), ctypes.POINTER(ctypes.c_longlong)]
    L.bf_movegen.argtypes = [i32, vp, vp, i32, vp, vp, vp]
    L.bf_forward_leaves.argtypes = [vp] * 7 + [i32] + [vp] * 3 + [i32] + [vp] * 4
    L.bf_measure_elementwise.argtypes = [i32, i32, i32, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    L.bf_forward_backbone.argtypes = [vp, vp, vp, i32, vp, vp]
    L.bf_int8_q_max.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    L.bf_int8_q_max.restype = None
    L.bf_fp8_q_max.argtypes = []
    L.bf_fp8_q_max.restype = ctypes.c_double
    L.bf_terminal.argtypes = [i32, vp, vp, vp, vp, vp, i32, vp, vp, vp]
    L.bf_hash.argtypes = [i32, vp, vp, i32, vp, vp]
    L.bf_history_push.argtypes = [i32, vp, vp, vp, vp, i32, vp]
    L.bf_repetition_count.argtypes = [i32, vp, vp, vp, i32, vp, vp]
    L.bf_random_ply.argtypes = [i32, vp, vp, vp, vp, vp, i32, vp, vp]
    L.bf_step.argtypes = [i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp]
    L.bf_forward_priors_host.argtypes = [vp, vp, vp, vp, vp, i32, i32, vp, vp, vp, vp]
    L.bf_measure_i8_peak.argtypes = [i32, i32, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    L.bf_launch_count.argtypes = [vp]
    L.bf_launch_count.restype = ctypes.c_longlong
    L.bf_profile.argtypes = [vp, i32]
    L.bf_profile_read.argtypes = [vp, ctypes.POINTER(ctypes.c_longlong), i32]
    L.bf_profile_phases.restype = ctypes.c_char_p
    L.bf_forward_noalloc.argtypes = [i32, vp, sz, vp, vp, vp, vp, i32, vp, vp, vp, vp]
    L.bf_noalloc_status.argtypes = [i32, ctypes.POINTER(i32)]
    L.bf_noalloc_forget.argtypes = [i32]
    L.bf_host_link_gbps.argtypes = [vp]
    L.bf_host_link_gbps.restype = ctypes.c_double
    L.bf_host_plan.argtypes = [i32, i32, i32, ctypes.c_double, ctypes.POINTER(i32)]
    L.bf_selftest_umma.argtypes = [i32, i32, vp, vp, vp]
    for name in EXPORTS:
        fn = getattr(L, name)
        if name not in ("bf_version", "bf_last_error", "bf_launch_count", "bf_profile_phases",
                        "bf_int8_q_max", "bf_fp8_q_max", "bf_host_link_gbps"):
            fn.restype = ctypes.c_int
    _LIB = L
    return L


class NativeError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    """Turn a negative return code into an exception carrying ``bf_last_error()``."""
    if rc == 0:
        return
    msg = lib().bf_last_error().decode("utf-8", "replace")
    if rc == -1:
        raise ValueError(f"{what}: {msg}")
    if rc == -3:
        raise NotImplementedError(f"{what}: {msg}")
    raise NativeError(f"{what} failed ({rc}): {msg}")
