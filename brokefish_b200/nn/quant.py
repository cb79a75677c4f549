"""The int8 quantisation scheme of the evaluator, as host-side torch functions.

Same names, arguments and results as the int8 half of the reference's
``brokefish/nn/quant.py`` (lines 237-305); the packer in :mod:`brokefish_b200.nn.pack`
uses :func:`quantise_weights_int8_bytes`, and the other two exist so that code written
against the reference's scheme functions keeps working.

Scheme: weights are symmetric s8 with one fp32 scale per block of 128 output channels
taken over the whole reduction; activations are symmetric s8 (or u8 for the
non-negative post-ReLU hidden) with one fp32 scale per row; products accumulate exactly
in s32 and are descaled once.
"""

from __future__ import annotations

from typing import Optional

import torch

BLOCK_N = 128
ROW_K = 256
#: The formats' own limits; the kernel uses the same two numbers.
Q_MAX_S8 = 127.0
Q_MAX_U8 = 255.0


#: e4m3 as NVIDIA defines it (no infinities, maximum 448).
E4M3 = torch.float8_e4m3fn
E4M3_MAX = 448.0
#: What a row's (or a weight block's) maximum is mapped to in the e4m3 arithmetic.  The
#: reference fixes 8 because its kernel accumulates 256 products in fp16; the value is kept so
#: that both implementations quantise to the same grid (brokefish/nn/quant.py:97-110).
Q_MAX = 8.0


def _scale_for(amax: torch.Tensor, q_max: float) -> torch.Tensor:
    """``amax / q_max`` in fp32, with 1 for an all-zero group so nothing divides by 0."""
    one = torch.ones((), dtype=amax.dtype, device=amax.device)
    return torch.where(amax > 0, amax / q_max, one)


def quantise_activations_int8(x: torch.Tensor, unsigned: bool = False):
    """``[M, K]`` -> ``(q [M, K] float, scale [M, 1])``: one scale per row,
    round-to-nearest-even, clamped to the format."""
    if unsigned:
        pos = x.clamp(min=0)
        scale = _scale_for(pos.amax(dim=-1, keepdim=True), Q_MAX_U8)
        return (pos / scale).round().clamp(0, Q_MAX_U8), scale
    scale = _scale_for(x.abs().amax(dim=-1, keepdim=True), Q_MAX_S8)
    return (x / scale).round().clamp(-Q_MAX_S8, Q_MAX_S8), scale


def quantise_weights_int8_bytes(w: torch.Tensor, block_n: int = BLOCK_N):
    """``[N, K]`` -> ``(bytes [N, K] uint8, scale [N // block_n] fp32)``: one scale per
    ``block_n`` output rows over the whole of K."""
    n, k = w.shape
    if n % block_n:
        raise ValueError(f"weight {tuple(w.shape)} does not tile into {block_n} rows")
    blocks = w.float().reshape(n // block_n, block_n * k)
    scale = _scale_for(blocks.abs().amax(dim=1), Q_MAX_S8)
    q = (blocks / scale[:, None]).round().clamp(-Q_MAX_S8, Q_MAX_S8).to(torch.int8)
    return q.reshape(n, k).view(torch.uint8), scale.contiguous()


def int8_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                unsigned: bool = False, row_k: int = ROW_K) -> torch.Tensor:
    """``F.linear`` under the scheme: the reduction is cut into ``row_k`` slices, each
    slice has its own activation scale per row and accumulates exactly (float64 holds
    the integers), and the weight scale is applied once at the end."""
    lead = x.shape[:-1]
    a = x.reshape(-1, x.shape[-1]).float()
    wq, ws = quantise_weights_int8_bytes(w.float())
    wq = wq.view(torch.int8).to(torch.float64)
    total = torch.zeros(a.shape[0], w.shape[0], dtype=torch.float64, device=a.device)
    for lo in range(0, a.shape[1], row_k):
        q, sa = quantise_activations_int8(a[:, lo:lo + row_k], unsigned)
        total += (q.to(torch.float64) @ wq[:, lo:lo + row_k].T) * sa.to(torch.float64)
    y = total.float() * ws.repeat_interleave(BLOCK_N)[None, :]
    if bias is not None:
        y = y + bias.float()
    return y.reshape(*lead, w.shape[0]).to(x.dtype)


def quantise_weights_bytes(w: torch.Tensor, q_max: float = Q_MAX, tile_k: Optional[int] = None,
                           block_n: int = BLOCK_N):
    """``[N, K]`` -> ``(e4m3 bytes [N, K] uint8, scale [N // block_n, K // tile_k] fp32)``.

    One scale per ``block_n`` output rows and ``tile_k`` reduction columns (``tile_k=None``:
    the whole of K, which is what the evaluator's single descale needs); values are divided by
    the scale, clamped to +-448 and rounded to e4m3 (brokefish/nn/quant.py:208-224)."""
    n, k = w.shape
    tile_k = k if tile_k is None else tile_k
    if n % block_n or k % tile_k:
        raise ValueError(f"weight {tuple(w.shape)} does not tile into {block_n}x{tile_k} blocks")
    blocks = w.float().reshape(n // block_n, block_n, k // tile_k, tile_k)
    scale = _scale_for(blocks.abs().amax(dim=(1, 3), keepdim=True), q_max)
    q = (blocks / scale).clamp(-E4M3_MAX, E4M3_MAX).to(E4M3).reshape(n, k)
    return q.view(torch.uint8), scale.reshape(n // block_n, k // tile_k).contiguous()
