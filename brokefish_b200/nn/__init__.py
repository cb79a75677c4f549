"""The encoder implementations, selected by name.

Mirrors the registry of the reference (brokefish/nn/__init__.py:45-86): a caller asks
for ``encoder_impl("cuda")`` and gets the ``FusedEncoder`` class whose
``forward_full(boards, control, rep)`` maps boards to ``(policy_logits, promo, value)``.
This build has exactly one implementation, the sm_100a kernel; asking for ``"triton"``
is refused because no second backend exists here.

    net = BrokefishNet().eval()
    model = encoder_impl("cuda")(net)
    policy_logits, promo, value = model.forward_full(boards, control, rep)
"""

from __future__ import annotations

IMPLEMENTATIONS = ("cuda",)

_WHY: dict = {}


def encoder_impl(name: str):
    """The ``FusedEncoder`` class of one implementation; ``ValueError`` for an unknown
    name, and the implementation's own import error otherwise."""
    if name == "cuda":
        from brokefish_b200.nn.cuda_impl import FusedEncoder
        return FusedEncoder
    raise ValueError(f"unknown implementation {name!r}, expected one of {IMPLEMENTATIONS}")


def available() -> list:
    """Implementations usable on this machine: the library is built, loads, and a CUDA
    device is present."""
    found = []
    for name in IMPLEMENTATIONS:
        try:
            import torch
            from brokefish_b200 import _native
            encoder_impl(name)
            _native.lib()
            if not torch.cuda.is_available():
                raise RuntimeError("no CUDA device")
        except Exception as exc:  # reported through why_unavailable()
            _WHY[name] = f"{type(exc).__name__}: {exc}"
        else:
            found.append(name)
            _WHY.pop(name, None)
    return found


def why_unavailable() -> dict:
    """Why each missing implementation is missing.  Call :func:`available` first."""
    return dict(_WHY)


__all__ = ["IMPLEMENTATIONS", "encoder_impl", "available", "why_unavailable"]
