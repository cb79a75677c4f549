"""Evaluator entry points: what the search calls once per simulation.

``make_evaluator`` has the signature and meaning of the reference's
``brokefish/search/torch_impl.py:186-197``.  ``ShardedEvaluator`` is the multi-GPU form:
one process per GPU, every rank holds a full copy of the packed weights (broadcast once
from rank 0 at construction), positions are split by index and nothing is exchanged on
the evaluation path.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def make_evaluator(net, impl: Optional[str] = None, **kw) -> Callable:
    """``(boards, control, rep) -> (policy_logits, promo, value)``.

    ``impl=None`` calls ``net`` itself, which must then be a network with a forward path (the
    reference's own module; this package's weight container has none); ``"cuda"`` is the fused
    sm_100a evaluator.
    """
    if impl is None:
        return lambda b, c, r: net(b, c, r)
    from brokefish_b200.nn import encoder_impl
    return encoder_impl(impl)(net, **kw).forward_full


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, even split of ``n`` positions: rank ``r`` gets ``[lo, hi)``; the first
    ``n % world`` ranks get one extra."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def broadcast_blob(blob_or_none, device: torch.device, src: int = 0) -> torch.Tensor:
    """Replicate rank ``src``'s packed weight blob to every rank with one broadcast (plus
    one 8-byte broadcast for its length).  Works with the nccl backend (``device`` a CUDA
    device) and with gloo (``device`` CPU)."""
    import torch.distributed as dist
    rank = dist.get_rank()
    size = torch.zeros(1, dtype=torch.int64, device=device)
    if rank == src:
        blob = torch.as_tensor(blob_or_none, dtype=torch.uint8).to(device)
        size[0] = blob.numel()
    dist.broadcast(size, src=src)
    if rank != src:
        blob = torch.empty(int(size.item()), dtype=torch.uint8, device=device)
    dist.broadcast(blob, src=src)
    return blob


class ShardedEvaluator:
    """Position-sharded evaluation: this rank evaluates its slice of every batch.

    ``net`` is needed on rank 0 only (other ranks may pass ``None``); the packed weights
    travel as one blob (int8 by default; ``fp8=True`` the e4m3-FFN arithmetic, ``int8=False`` the
    fp16 arithmetic).  ``forward_shard`` evaluates positions that already live on this
    rank's GPU; ``shard`` tells the caller which slice of a global batch is this rank's.
    """

    def __init__(self, net, rank: int, world: int, device_index: int, fp8: bool = False,
                 int8: bool = True, int8_scheme: str = "all"):
        import torch.distributed as dist
        from brokefish_b200.nn.cuda_impl import FusedEncoder
        from brokefish_b200.nn.pack import pack_blob
        self.rank, self.world = rank, world
        dev = torch.device("cuda", device_index)
        if world > 1:
            fmt = "e4m3" if fp8 else ({"all": "int8", "ffn": "int8_ffn", "ffn+qkv": "int8_ffn_qkv"}[int8_scheme]
                                      if int8 else "f16")
            blob = pack_blob(net, fmt) if rank == 0 else None
            blob_dev = broadcast_blob(blob, dev, src=0)
            torch.cuda.synchronize(dev)
            self.encoder = FusedEncoder.from_blob(blob_dev, device=device_index)
        else:
            self.encoder = FusedEncoder(net, device=device_index, fp8=fp8, int8=bool(int8) and not fp8,
                                        int8_scheme=int8_scheme)

    def shard(self, n: int) -> Tuple[int, int]:
        return shard_bounds(n, self.world, self.rank)

    def forward_shard(self, boards, control, rep, legal=None):
        return self.encoder.forward_full(boards, control, rep, legal)
