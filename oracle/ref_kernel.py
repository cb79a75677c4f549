"""Run the reference's own encoder kernel (built by ``oracle/build_ref.py``) on a GPU.

TEST INFRASTRUCTURE ONLY: the on-device checker beside the numpy restatement.  The product
never imports this module.  It needs nothing of the reference checkout at run time: the
compiled extension and the weight slabs its constructor derived are both under
``oracle/_ref/``.

The call made is the one ``FusedEncoder.forward_full`` of the reference makes
(``brokefish/nn/cuda_impl.py:487-503``): ``model_forward`` of ``csrc/encoder.cu:1770`` with
the slabs, empty ``y``, stage 0.
"""

from __future__ import annotations

import importlib.util
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
SO_PATH = os.path.join(REF_DIR, "brokefish_encoder.so")

_EXT = None


def available(name: str | None = None) -> bool:
    ok = os.path.exists(SO_PATH)
    if name is not None:
        ok = ok and os.path.exists(os.path.join(REF_DIR, f"slabs_{name}.npz"))
    return ok


def ext():
    global _EXT
    if _EXT is None:
        import torch  # noqa: F401  (the extension links against torch's libraries)
        spec = importlib.util.spec_from_file_location("brokefish_encoder", SO_PATH)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _EXT = mod
    return _EXT


class RefKernel:
    """The reference kernel with one weight set resident on ``device``."""

    def __init__(self, name: str, device: str = "cuda:0"):
        import torch
        z = np.load(os.path.join(REF_DIR, f"slabs_{name}.npz"))
        self.device = torch.device(device)
        put = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        self.weights, self.emb, self.tail = put(z["weights"]), put(z["emb"]), put(z["tail"])
        self.wq8, self.sq8, self.rj = put(z["wq8"]), put(z["sq8"]), put(z["rj"])
        (self.n_layers, self.quant, self.two_boards, self.n_value, self.vmode,
         self.rj_mode) = (int(v) for v in z["scalars"])
        self.eps = float(z["eps"][0])
        self._empty_h = torch.empty(0, dtype=torch.half, device=self.device)
        self._n = -1

    def forward_full(self, boards, control, rep):
        """``boards [n,32] int16, control [n] int16, rep [n] uint8`` (CUDA tensors) ->
        ``(policy [n,32,64] fp16, promo [n,32,4] fp16, value [n] fp32)``."""
        import torch
        n = boards.shape[0]
        if n != self._n:
            self.policy = torch.empty(n, 32, 64, device=self.device, dtype=torch.half)
            self.promo = torch.empty(n, 32, 4, device=self.device, dtype=torch.half)
            self.value = torch.empty(n, device=self.device, dtype=torch.float)
            self._n = n
        ext().model_forward(boards.contiguous(), control.contiguous(), rep.contiguous(),
                            self.weights, self.emb, self.tail,
                            self.policy, self.promo, self.value, self._empty_h,
                            self.n_layers, self.eps, 0, self.wq8, self.sq8, self.quant,
                            self.two_boards, self.n_value, self.vmode, self.rj, self.rj_mode)
        return self.policy, self.promo, self.value

    def forward_stage(self, boards, control, rep, stage: int):
        """Activations ``[n,32,256]`` fp16 at one of the reference's debug stages (9: the
        embedding, 8: the final norm), as ``brokefish/nn/cuda_impl.py:511-530`` asks for them."""
        import torch
        n = boards.shape[0]
        y = torch.empty(n, 32, 256, device=self.device, dtype=torch.half)
        e_f = torch.empty(0, dtype=torch.float, device=self.device)
        ext().model_forward(boards.contiguous(), control.contiguous(), rep.contiguous(),
                            self.weights, self.emb, self.tail,
                            self._empty_h, self._empty_h, e_f, y,
                            self.n_layers, self.eps, int(stage), self.wq8, self.sq8, self.quant,
                            self.two_boards, self.n_value, self.vmode, self.rj, self.rj_mode)
        return y

    def encoder_forward(self, x, alive=None):
        """The reference's backbone-only entry (``encoder_forward`` of ``csrc/encoder.cu:1752``,
        the call ``brokefish/nn/cuda_impl.py:447-461`` makes): ``x [n,32,256]`` fp16 in, the
        residual stream after the last layer out; ``alive [n,32]`` int8 or ``None``."""
        import torch
        out = x.contiguous().clone()
        a = alive.contiguous() if alive is not None else torch.empty(0, dtype=torch.int8, device=self.device)
        ext().encoder_forward(out, self.weights, a, self.n_layers, self.eps, 0)
        return out

