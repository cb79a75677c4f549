"""The N > 1 host logic on CPU: two gloo ranks, rank 0 packs the weight blob, one broadcast
replicates it, every rank takes its contiguous slice of the positions and the slices
reassemble to the whole batch.  (The GPU side of a rank is the single-GPU evaluator.)"""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_positions


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from brokefish_b200.evaluator import broadcast_blob, shard_bounds
    blob = None
    if rank == 0:
        from brokefish_b200.nn.model import BrokefishNet, seeded_state
        from brokefish_b200.nn.pack import pack_blob
        net = BrokefishNet().eval()
        net.load_state_dict(seeded_state(seed=0, std=0.02))
        blob = pack_blob(net)
    got = broadcast_blob(blob, torch.device("cpu"), src=0)
    pos = load_positions(256, 0)
    lo, hi = shard_bounds(250, world, rank)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), blob_sum=np.int64(got.numpy().astype(np.int64).sum()),
             blob_len=np.int64(got.numel()), magic=got[:4].numpy(), lo=lo, hi=hi,
             boards=pos["boards"][lo:hi])
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_share_one_blob_and_split_the_positions(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    assert parts[0]["blob_len"] == parts[1]["blob_len"] > 6_000_000
    assert parts[0]["blob_sum"] == parts[1]["blob_sum"]
    assert bytes(parts[1]["magic"]) == b"BFB8"
    assert (parts[0]["lo"], parts[0]["hi"], parts[1]["lo"], parts[1]["hi"]) == (0, 125, 125, 250)
    whole = np.concatenate([p["boards"] for p in parts])
    assert np.array_equal(whole, load_positions(256, 0)["boards"][:250])
