"""The engine functions the evaluator's inputs come from, on the GPU.

``movegen(boards, control) -> (mask, in_check)`` with the reference's contract
(brokefish/env/torch_impl.py:254-291): ``mask [n,32]`` int64, bit ``s`` of word ``p`` set when
the piece in slot ``p`` may legally move to square ``s``; ``in_check [n]`` bool for the side
to move.  One warp per board in ``libbrokefish_b200`` (C ABI ``bf_movegen``); CUDA tensors in,
CUDA tensors out, on the current stream.  There is no CPU path.
"""

from __future__ import annotations

import ctypes

import torch

from brokefish_b200 import _native


def movegen(boards: torch.Tensor, control: torch.Tensor):
    n = boards.shape[0]
    if boards.dim() != 2 or boards.shape[1] != 32 or boards.dtype is not torch.int16:
        raise ValueError(f"boards must be [n, 32] int16, got {tuple(boards.shape)} {boards.dtype}")
    if tuple(control.shape) != (n,) or control.dtype is not torch.int16:
        raise ValueError(f"control must be [{n}] int16, got {tuple(control.shape)} {control.dtype}")
    if not (boards.is_cuda and control.is_cuda and boards.device == control.device):
        raise ValueError("movegen takes CUDA tensors on one device; there is no CPU path")
    dev = boards.device
    mask = torch.zeros(n, 32, dtype=torch.int64, device=dev)
    in_check = torch.zeros(n, dtype=torch.uint8, device=dev)
    if n:
        b, c = boards.contiguous(), control.contiguous()
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _native.check(_native.lib().bf_movegen(
            dev.index or 0, ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(c.data_ptr()), n,
            ctypes.c_void_p(mask.data_ptr()), ctypes.c_void_p(in_check.data_ptr()), stream), "bf_movegen")
    return mask, in_check.bool()
