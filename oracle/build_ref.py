"""Build the on-device reference checker: the reference's own encoder kernel, compiled from
where its sources lie, plus the weight slabs its own constructor derives.

TEST INFRASTRUCTURE ONLY.  Nothing the product ships imports this file or what it writes.

    PYTHONDONTWRITEBYTECODE=1 python oracle/build_ref.py --reference <reference checkout>

writes into ``oracle/_ref/`` (ignored by git, never the reference's sources):

* ``brokefish_encoder.so`` -- ``csrc/encoder.cu`` of the reference (with the headers it
  includes: ``mma.cuh``, ``fp8_gemm.cuh``, ``int8_gemm.cuh``), compiled by one ``nvcc`` line
  for sm_100a against the torch headers of this interpreter.  The reference's own build
  helper (``brokefish/nn/_build.py:149-190``) is not run; the flags below are the ones it
  would pass, with the architecture changed from sm_89;
* ``slabs_<set>.npz`` -- for each seeded weight set of the parity tests, the tensors the
  reference's ``FusedEncoder.__init__`` (``brokefish/nn/cuda_impl.py:140-430``) hands to its
  kernel: fp16 weight slab, int8 / e4m3 weight bytes and scales, embedding table, tail,
  re-injection slab and the scalar arguments.  The constructor itself runs, unmodified, on
  the CPU: only the placement calls (``Tensor.cuda()``, ``device="cuda"``) are neutralised
  for the duration.

``tests/test_gpu_reference_kernel.py`` loads both on a GPU box and compares the product's
outputs with the reference kernel's on the same positions; it skips when they are absent.
"""

from __future__ import annotations

import argparse
import contextlib
import os
import subprocess
import sys
import sysconfig

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
SO_NAME = "brokefish_encoder.so"

#: weight sets: name -> (seeded_state kwargs, FusedEncoder kwargs)
SETS = {
    "A_int8": (dict(seed=0, std=0.02, perturb_norms=False), dict(int8=True)),
    "B_int8": (dict(seed=0, std=None, perturb_norms=True), dict(int8=True)),
    "A_e4m3": (dict(seed=0, std=0.02, perturb_norms=False), dict(fp8=True)),
    "B_e4m3": (dict(seed=0, std=None, perturb_norms=True), dict(fp8=True)),
    "A_f16": (dict(seed=0, std=0.02, perturb_norms=False), dict()),
    "B_int8_ffn": (dict(seed=0, std=None, perturb_norms=True), dict(int8=True, int8_scheme="ffn")),
    "B_int8_ffn_qkv": (dict(seed=0, std=None, perturb_norms=True), dict(int8=True, int8_scheme="ffn+qkv")),
    "C_int8_rj": (dict(seed=7, std=None, perturb_norms=True, reinject="both"), dict(int8=True)),
    "C_f16_rj": (dict(seed=7, std=None, perturb_norms=True, reinject="both"), dict()),
    "D_f16_rj1": (dict(seed=8, std=0.02, perturb_norms=True, reinject="ln1"), dict()),
    "V_int8_wdl": (dict(seed=3, std=0.02, perturb_norms=True, n_value=3, value_head="pooled"),
                   dict(int8=True)),
    "P_int8_prenorm": (dict(seed=5, std=None, perturb_norms=True, n_value=3, value_head="prenorm"),
                       dict(int8=True)),
}


def compile_kernel(reference: str, verbose: bool = True) -> str:
    from torch.utils import cpp_extension as ce
    src = os.path.join(reference, "csrc", "encoder.cu")
    out = os.path.join(OUT, SO_NAME)
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    tlib = ce.library_paths()[0]
    inc = [p for p in ce.include_paths() if "cuda" not in p.split(os.sep)[-2:]]
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
           "-DTORCH_EXTENSION_NAME=brokefish_encoder", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           *ce.COMMON_NVCC_FLAGS,
           "-I", os.path.join(reference, "csrc"), *sum((["-isystem", p] for p in inc), []),
           "-isystem", sysconfig.get_paths()["include"],
           src, "-o", out,
           "-L", tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-Xlinker", "-rpath", "-Xlinker", tlib]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return out


@contextlib.contextmanager
def cpu_placement():
    """Make ``.cuda()`` and ``device="cuda"`` no-ops so the reference constructor, which only
    packs weights, can run on a machine without a GPU."""
    saved_cuda = torch.Tensor.cuda
    saved = {name: getattr(torch, name) for name in ("empty", "zeros", "ones", "tensor", "arange")}

    def strip(fn):
        def wrapped(*a, **kw):
            if str(kw.get("device", "")).startswith("cuda"):
                kw.pop("device")
            return fn(*a, **kw)
        return wrapped

    torch.Tensor.cuda = lambda self, *a, **kw: self
    for name, fn in saved.items():
        setattr(torch, name, strip(fn))
    try:
        yield
    finally:
        torch.Tensor.cuda = saved_cuda
        for name, fn in saved.items():
            setattr(torch, name, fn)


def make_slabs(reference: str) -> None:
    sys.path.insert(0, reference)
    sys.path.insert(0, ROOT)
    sys.dont_write_bytecode = True
    from brokefish.nn.cuda_impl import FusedEncoder as RefEncoder     # reference
    from brokefish.nn.model import BrokefishNet as RefNet             # reference
    from brokefish_b200.nn.model import seeded_state                  # ours: weights by seed

    for name, (skw, ekw) in SETS.items():
        state = seeded_state(**skw)
        net_kw = {k: skw[k] for k in ("n_value", "value_head", "reinject") if k in skw}
        net = RefNet(**net_kw).eval()
        net.load_state_dict(state, strict=True)
        with cpu_placement():
            enc = RefEncoder(net, **ekw)
            rj = enc._rj_slab()
        np.savez(os.path.join(OUT, f"slabs_{name}.npz"),
                 weights=enc.weights.numpy(), emb=enc.emb.numpy(), tail=enc.tail.numpy(),
                 wq8=enc._wq8.numpy(), sq8=enc._sq8.numpy(), rj=rj.numpy(),
                 scalars=np.array([enc.n_layers, enc.quant, int(enc.two_boards), enc.n_value,
                                   enc.vmode, enc.rj_mode], dtype=np.int64),
                 eps=np.array([enc.eps], dtype=np.float64))
        print(f"slabs {name}: weights {tuple(enc.weights.shape)} wq8 {tuple(enc._wq8.shape)} "
              f"quant {enc.quant} vmode {enc.vmode} rj_mode {enc.rj_mode}", flush=True)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("BROKEFISH_REFERENCE"), required="BROKEFISH_REFERENCE" not in os.environ,
                    help="checkout of the reference (default: $BROKEFISH_REFERENCE)")
    ap.add_argument("--no-kernel", action="store_true")
    ap.add_argument("--no-slabs", action="store_true")
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.reference, "csrc")):
        print("no reference checkout: nothing built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    if not args.no_slabs:
        make_slabs(args.reference)
    if not args.no_kernel:
        compile_kernel(args.reference)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
