"""Benchmark of the network-evaluation hot path: positions evaluated per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

One step = one pass of the evaluator over one batch of positions per GPU (batch 4096,
the reference's self-play leaf-evaluation batch).  For N > 1 launch under
``python -m torch.distributed.run --nproc-per-node N``; every rank holds a full copy of
the weights (one broadcast from rank 0 before the timed loop), evaluates its own 4096
positions and nothing is exchanged on the evaluation path ("weak" scaling: N x 4096
positions per step).  ``--total 131072`` instead splits a fixed 131072-position step
evenly across the ranks.

Rank 0 prints one JSON line.  ``value`` is device-timed with inputs resident in HBM;
``e2e`` is the same metric through the host-buffer C-ABI call with both copies inside
the timed region; ``roofline`` is the int8 tensor throughput of the one kernel against
the tensor pipe's int8 rate measured in the same run (rank 0's GPU, at every N);
``cpu_baseline`` is the reference's fp32 PyTorch evaluator (restated in
``oracle/fp32_model.py``) on the host cores.  Beside the headline, with timed loops of their
own after it: ``reference_kernel`` (the reference's CUDA kernel compiled for sm_100a, timed
interleaved with this one), ``batch_sweep``, ``fp8_batch16384`` and ``split_131072``.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

OPS_PER_POSITION = 402653184          # int8 ops of the 32 weight GEMMs of one position
BYTES_IN, BYTES_OUT = 67, 4356        # boards+control+rep ; policy+promo+value
PROFILE_NCU = os.path.join(ROOT, "profiles", "encoder_kernel_batch4096_ncu_full.md")
METRIC = "positions evaluated/sec at batch 4096 int8"
WORKLOAD = ("8-layer d256 h8 ff1024 int8 evaluator, N(0,0.02) seed-0 weights, seeded "
            "random-playout positions, batch 4096 per GPU")
WORKLOAD_CPU = ("8-layer d256 h8 ff1024 evaluator in fp32 on the host cores (the reference's CPU path), "
                "N(0,0.02) seed-0 weights, seeded random-playout positions, batch 256 per step")


def profiled_traffic():
    """DRAM bytes per launch at batch 4096 from the committed ncu summary of this kernel
    (its ``dram_bytes_per_launch = ...`` line), or ``None`` when the summary has none."""
    import re
    try:
        m = re.search(r"dram_bytes_per_launch\s*=\s*([0-9.eE+]+)", open(PROFILE_NCU).read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


def load_positions(n: int):
    """``n`` positions: the committed 4096 random-playout positions, tiled when more are
    asked for (a tile keeps the distribution of piece counts, clocks and side to move)."""
    from brokefish_b200.positions import tiled
    return tiled(n)


def sweep(enc, dev, batches=(1, 64, 512, 4096, 16384, 65536), steps=10, warmup=3):
    """Batch sweep with piece counts uniform in 2..32 and side to move 50/50: one JSON line
    per batch size (latency-bound at the small end, throughput-bound at the large end)."""
    from brokefish_b200.positions import varied
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for n in batches:
        b, c, r, _ = varied(n, seed=2)
        d_b, d_c, d_r = (torch.from_numpy(a).to(dev) for a in (b, c, r))
        for _ in range(warmup):
            enc.forward_full(d_b, d_c, d_r)
        torch.cuda.synchronize(dev)
        ms = []
        for i in range(steps):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            enc.forward_full(d_b, d_c, d_r)
            e1.record()
            torch.cuda.synchronize(dev)
            ms.append(e0.elapsed_time(e1))
        enc.check_status()
        t = float(np.median(ms))
        print(json.dumps({"sweep_batch": n, "ms_per_launch_median": t, "positions_per_s": n / t * 1e3,
                          "int8_TOPs": n * OPS_PER_POSITION / t / 1e9, "tiles": (n + 3) // 4,
                          "data": "synthetic: piece counts U{2..32}, side to move 50/50, seed 2"}))


def engine(enc, dev, n=1 << 20, steps=10, warmup=3):
    """The engine kernels beside the evaluator, one JSON line each: the legal-move generator
    and `step` on `n` random-playout positions made on the device (HBM-bound by their
    algorithmic bytes, 323 and 137 B per board; measured against the copy bandwidth), and the
    evaluator's fused expansion with and without the legality words given."""
    import ctypes
    from brokefish_b200 import _native
    from brokefish_b200.env import random_playouts
    hbm = 6650.0
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        hbm = float(json.load(open(path)).get("hbm_gbs", hbm))
    b, c, r, lg, _ = random_playouts(n, 11, device=dev)
    mask = torch.empty(n, 32, dtype=torch.int64, device=dev)
    chk = torch.empty(n, dtype=torch.uint8, device=dev)
    count = (lg != 0).any(dim=1)
    first = (lg != 0).float().argmax(dim=1)
    w = lg[torch.arange(n, device=dev), first]
    low = w & -w
    bit = torch.where(low < 0, torch.full_like(low, 63), torch.log2(low.abs().clamp(min=1).double()).long())
    move = torch.where(count, first * 64 + bit, torch.full_like(first, -1)).to(torch.int32)
    nb, nc = torch.empty_like(b), torch.empty_like(c)
    irr = torch.empty(n, dtype=torch.uint8, device=dev)
    L, stream = _native.lib(), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(warmup):
            fn()
        ms = []
        for i in range(steps):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(dev)
            ms.append(e0.elapsed_time(e1))
        return float(np.median(ms))

    idx = dev.index or 0
    for name, bytes_per_board, fn in (
            ("movegen", 64 + 2 + 256 + 1,
             lambda: _native.check(L.bf_movegen(idx, ptr(b), ptr(c), n, ptr(mask), ptr(chk), stream), "bf_movegen")),
            ("step", 64 + 2 + 4 + 64 + 2 + 1,
             lambda: _native.check(L.bf_step(idx, ptr(b), ptr(c), ptr(move), None, n, ptr(nb), ptr(nc), ptr(irr),
                                             None, None, None, stream), "bf_step")),
            ("step+movegen (play)", 64 + 2 + 4 + 64 + 2 + 1 + 256 + 1,
             lambda: _native.check(L.bf_step(idx, ptr(b), ptr(c), ptr(move), None, n, ptr(nb), ptr(nc), ptr(irr),
                                             ptr(mask), ptr(chk), None, stream), "bf_step"))):
        t = timed(fn)
        gbs = n * bytes_per_board / t / 1e6
        print(json.dumps({"engine_kernel": name, "boards": n, "ms_per_launch_median": t, "boards_per_s": n / t * 1e3,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s",
                                       "frac": gbs / hbm, "algorithmic_bytes_per_board": bytes_per_board},
                          "data": "synthetic: random-playout positions played on the device, seed 11"}))
    m = 4096
    t_given = timed(lambda: enc.forward_priors(b[:m], c[:m], r[:m], lg[:m], 96))
    t_own = timed(lambda: enc.forward_priors(b[:m], c[:m], r[:m], None, 96))
    t_plain = timed(lambda: enc.forward_full(b[:m], c[:m], r[:m]))
    enc.check_status()
    print(json.dumps({"fused_expansion_batch": m, "ms_logits_only": t_plain, "ms_priors_legality_given": t_given,
                      "ms_priors_moves_generated_in_kernel": t_own}))


def timed_ms(fn, dev, launches: int, warmup: int = 2):
    """Mean device time of ``fn`` over ``launches`` back-to-back calls (CUDA events)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / launches


def reference_kernel_leg(enc, args, dev, rounds: int = 8, launches: int = 5):
    """The reference's own CUDA kernel (compiled for sm_100a under ``oracle/_ref``) against this
    library on the same GPU and inputs, with the reference's protocol (bench/bench_model.py:
    172-177): the two candidates interleaved in one process, order reversed on alternate rounds,
    medians over the rounds.  ``None`` where the checker is not built."""
    try:
        from oracle import ref_kernel as R
    except Exception:
        return None
    if not R.available("A_int8"):
        return None
    ref = R.RefKernel("A_int8", device=str(dev))
    cand = {"ours": lambda: enc.forward_full(*args), "reference": lambda: ref.forward_full(*args)}
    ms = {"ours": [], "reference": []}
    for rnd in range(rounds):
        order = ("ours", "reference") if rnd % 2 == 0 else ("reference", "ours")
        for name in order:
            ms[name].append(timed_ms(cand[name], dev, launches, warmup=1))
    enc.check_status()
    n = args[0].shape[0]
    ours, theirs = float(np.median(ms["ours"])), float(np.median(ms["reference"]))
    return {"ms": theirs, "positions_per_s": n / theirs * 1e3, "ours_ms": ours, "ratio": theirs / ours,
            "rounds": rounds, "launches_per_round": launches,
            "protocol": "interleaved in one process, order reversed on alternate rounds, median of rounds; "
                        "the reference's csrc/encoder.cu compiled for sm_100a, int8 'all', same weights and positions",
            "outputs": "bit-identical to ours (tests/test_gpu_reference_kernel.py)"}


def other_configs(net, enc, dev, world, rank, barrier, all_max):
    """The configurations beside the headline, each with a short timed loop of its own:
    the batch sweep (piece counts uniform in 2..32, six sizes, median of 10 launches), the
    e4m3-FFN arithmetic at batch 16384, and one 131072-position step split evenly across the
    GPUs.  Rank 0 runs the first two; every rank takes part in the third."""
    from brokefish_b200.evaluator import shard_bounds
    from brokefish_b200.positions import varied
    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def median_ms(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        ms = []
        for i in range(n):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(dev)
            ms.append(e0.elapsed_time(e1))
        return float(np.median(ms))

    if rank == 0:
        rows = []
        for n in (1, 64, 512, 4096, 16384, 65536):
            b, c, r, _ = varied(n, seed=2)
            d = [torch.from_numpy(a).to(dev) for a in (b, c, r)]
            t = median_ms(lambda: enc.forward_full(*d))
            rows.append({"batch": n, "ms": t, "positions_per_s": n / t * 1e3})
        out["batch_sweep"] = {"rows": rows, "data": "synthetic: piece counts U{2..32}, side to move 50/50, seed 2",
                              "timing": "median of 10 launches, L2 flushed between them"}
        if net is not None:
            from brokefish_b200.nn.cuda_impl import FusedEncoder
            e8 = FusedEncoder(net, fp8=True, device=dev.index or 0)
            b, c, r, _ = load_positions(16384)
            d = [torch.from_numpy(a).to(dev) for a in (b, c, r)]
            t = median_ms(lambda: e8.forward_full(*d))
            e8.check_status()
            e8.close()
            out["fp8_batch16384"] = {"ms": t, "positions_per_s": 16384 / t * 1e3, "dtype": "e4m3 (FFN) + f16",
                                     "int8_equivalent_TOPs": 16384 * OPS_PER_POSITION / t / 1e9}
        enc.check_status()
    total = 131072
    lo, hi = shard_bounds(total, world, rank)
    b, c, r, _ = (a[lo:hi] for a in load_positions(total))
    d = [torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (b, c, r)]
    for _ in range(3):
        enc.forward_full(*d)
    barrier()
    ms = []
    for i in range(5):
        flush.fill_(i & 0xFF)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        enc.forward_full(*d)
        e1.record()
        torch.cuda.synchronize(dev)
        ms.append(e0.elapsed_time(e1))
    barrier()
    enc.check_status()
    t = all_max(float(np.mean(ms)))
    out["split_131072"] = {"ms_per_step": t, "positions_per_s": total / t * 1e3, "positions_per_gpu": hi - lo,
                           "timing": "mean of 5 launches per rank, max over ranks"}
    return out


def d2h_probe(dev, rank, world, barrier, nbytes=4096 * BYTES_OUT, reps=200):
    """What the host side of the box takes: every rank copies `nbytes` (one step's logits) from
    its GPU into pinned host memory `reps` times, all ranks at once, then rank 0 alone.  Prints
    the per-rank and aggregate GB/s: the ceiling of the end-to-end logit stream at N GPUs."""
    import torch.distributed as dist
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    dst = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    out = {}
    for label, active in (("all_ranks", True), ("rank0_alone", rank == 0)):
        for _ in range(5):
            dst.copy_(src, non_blocking=True)
        barrier()
        t0 = time.perf_counter()
        if active:
            for _ in range(reps):
                dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        barrier()
        gbs = torch.tensor([nbytes * reps / dt / 1e9 if active else 0.0], dtype=torch.float64, device=dev)
        if world > 1:
            rows = [torch.zeros_like(gbs) for _ in range(world)]
            dist.all_gather(rows, gbs)
            vals = [float(r[0]) for r in rows]
        else:
            vals = [float(gbs[0])]
        out[label] = {"per_rank_GBps": vals, "aggregate_GBps": sum(vals)}
    if rank == 0:
        print(json.dumps({"d2h_probe": out, "bytes_per_copy": nbytes, "copies": reps, "n_gpus": world,
                          "what": "device -> pinned host copies of one step's logits (4096 x 4356 B), "
                                  "cudaMemcpyAsync back to back; the ceiling this box's host side puts on "
                                  "the end-to-end logit stream is aggregate_GBps / 4356 positions/s"}))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        m = json.load(open(path))
        return 2.0 * float(m["bf16_tflops"]), "2 x measured dense bf16 burst (MEASURED_PEAKS.json)"
    return 2.0 * 1590.0, "2 x fallback dense bf16 (1.59 PFLOP/s)"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.rows, self.proc, self.index, self.first = [], None, index, 0

    def mark(self):
        """The timed region starts here: earlier samples (warm-up) are not reported."""
        self.first = len(self.rows)

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        rows = self.rows[self.first:] or self.rows
        sm = [float(r[0]) for r in rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [nm for i, nm in enumerate(names)
                   if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def cpu_reference(steps: int, warmup: int, batch: int = 256):
    """The reference's CPU evaluator (fp32 PyTorch network, all host threads) on ``batch``
    positions per step; returns positions/s and a description of the sample."""
    from brokefish_b200.nn.model import seeded_state
    from oracle import fp32_model
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    state = seeded_state(seed=0, std=0.02)
    b, c, r, _ = load_positions(batch)
    b, c, r = torch.from_numpy(b), torch.from_numpy(c), torch.from_numpy(r)
    for _ in range(max(1, warmup)):
        fp32_model.forward(state, b, c, r)
    t0 = time.perf_counter()
    for _ in range(steps):
        fp32_model.forward(state, b, c, r)
    dt = time.perf_counter() - t0
    return batch * steps / dt, dt / steps * 1e3, {
        "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"{steps} steps x {batch} positions, fp32 PyTorch evaluator on host threads"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=4096, help="positions per GPU per step")
    ap.add_argument("--total", type=int, default=0,
                    help="fixed number of positions per step split across the GPUs")
    ap.add_argument("--playouts", action="store_true",
                    help="play this rank's positions on the device (random games from the start position, "
                         "seed 100 + rank) instead of tiling the committed 4096")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--d2h-probe", action="store_true",
                    help="measure the device-to-pinned-host copy bandwidth of all ranks at once and exit")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations and the reference-kernel comparison")
    ap.add_argument("--sweep", action="store_true", help="print one line per batch size 1..65536 and exit")
    ap.add_argument("--engine", action="store_true",
                    help="time the engine kernels (movegen, step) and the fused expansion; print their lines and exit")
    ap.add_argument("--phases", action="store_true",
                    help="add the in-kernel phase split (cycles per phase over 5 extra launches) to the line")
    ap.add_argument("--f16", action="store_true",
                    help="time the plain fp16 arithmetic (the reference's default) instead of int8")
    ap.add_argument("--scheme", default="all", choices=["all", "ffn", "ffn+qkv"],
                    help="which matmuls run in int8: all four (the shipped scheme, the metric's), the FFN only, "
                         "or the FFN and QKV (the reference's partial schemes)")
    ap.add_argument("--host-plan", type=int, default=0,
                    help="how the end-to-end host call splits a batch (BF_OPT_HOST_PLAN; 0 = its own choice)")
    ap.add_argument("--fp8", action="store_true",
                    help="time the e4m3-FFN arithmetic instead of int8 (a separate line; not the headline)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(3, args.warmup)

    if args.impl == "reference":
        if rank != 0:
            return 0
        steps = min(args.steps, 40)
        value, ms, info = cpu_reference(steps, min(warmup, 3))
        line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "positions/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": min(warmup, 3), "ms_per_step": ms,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": WORKLOAD_CPU, "positions_per_step": 256, "l2": "n/a (CPU)"},
                "cpu_baseline": dict(info, value=value, unit="positions/s"),
                "e2e": {"value": value, "unit": "positions/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the evaluator")
    import torch.distributed as dist
    from brokefish_b200.evaluator import ShardedEvaluator, shard_bounds
    from brokefish_b200.nn.model import BrokefishNet, seeded_state

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.d2h_probe:
        def probe_barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)
        d2h_probe(dev, rank, world, probe_barrier)
        if world > 1:
            dist.destroy_process_group()
        return 0
    net = None
    if rank == 0 or world == 1:
        net = BrokefishNet().eval()
        net.load_state_dict(seeded_state(seed=0, std=0.02))
    ev = ShardedEvaluator(net, rank, world, local, fp8=args.fp8, int8=not args.f16, int8_scheme=args.scheme)   # one broadcast of the packed blob
    enc = ev.encoder
    if args.host_plan:
        enc.set_host_plan(args.host_plan)

    if args.sweep:
        if rank == 0:
            sweep(enc, dev)
        return 0
    if args.engine:
        if rank == 0:
            engine(enc, dev)
        return 0

    if args.total:
        lo, hi = shard_bounds(args.total, world, rank)
        n_local, n_global, scaling = hi - lo, args.total, "strong"
        b, c, r, lg = (a[lo:hi] for a in load_positions(args.total))
    else:
        n_local, n_global, scaling = args.batch, args.batch * world, "weak"
        b, c, r, lg = load_positions(args.batch)
    data = "synthetic"
    if args.playouts:
        from brokefish_b200.env import random_playouts
        pb, pc, pr, pl, _ = random_playouts(n_local, 100 + rank, device=dev)
        b, c, r = pb.cpu().numpy(), pc.cpu().numpy(), pr.cpu().numpy()
        lg = pl.cpu().numpy().view(np.uint64)
        data = f"synthetic: {n_local} random-playout positions per rank played on the device, seed 100 + rank"
    d_b, d_c, d_r = (torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (b, c, r))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(warmup):
        enc.forward_full(d_b, d_c, d_r)
    barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    launches0 = enc.launches
    barrier()
    sampler.mark()
    t_wall = time.perf_counter()
    for i in range(args.steps):
        flush.fill_(i & 0xFF)                      # L2 flush between timed iterations
        starts[i].record()
        enc.forward_full(d_b, d_c, d_r)
        stops[i].record()
    barrier()
    t_wall = time.perf_counter() - t_wall
    enc.check_status()
    kernel_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    dev_ms = float(sum(kernel_ms))
    launches = enc.launches - launches0

    # end to end: pinned host buffers in, pinned host buffers out, every step
    h_b, h_c, h_r = (torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in (b, c, r))
    h_pol = torch.empty(n_local, 32, 64, dtype=torch.half).pin_memory()
    h_pro = torch.empty(n_local, 32, 4, dtype=torch.half).pin_memory()
    h_val = torch.empty(n_local, dtype=torch.float).pin_memory()
    for _ in range(3):
        enc.forward_host(h_b, h_c, h_r, h_pol, h_pro, h_val)
    barrier()
    e2e_steps = args.steps
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        enc.forward_host(h_b, h_c, h_r, h_pol, h_pro, h_val)
    torch.cuda.synchronize(dev)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    # the same end-to-end step with the expansion fused in: edge lists back instead of logits
    h_lg = torch.from_numpy(np.ascontiguousarray(lg).view(np.int64).copy()).pin_memory()
    e_cap = 96
    h_pri = torch.empty(n_local, e_cap, dtype=torch.half).pin_memory()
    h_mov = torch.empty(n_local, e_cap, dtype=torch.int16).pin_memory()
    h_ne = torch.empty(n_local, dtype=torch.int32).pin_memory()
    for _ in range(3):
        enc.forward_priors_host(h_b, h_c, h_r, h_lg, h_pri, h_mov, h_ne, h_val)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        enc.forward_priors_host(h_b, h_c, h_r, h_lg, h_pri, h_mov, h_ne, h_val)
    torch.cuda.synchronize(dev)
    e2e_pri_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if rank == 0 else None
    phases = None
    if args.phases and rank == 0:
        enc.set_profile(True)
        enc.read_profile()
        for _ in range(5):
            enc.forward_full(d_b, d_c, d_r)
        phases = {k: v / 5 for k, v in enc.read_profile().items() if k}
        enc.set_profile(False)

    def all_max(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    headline = not (args.fp8 or args.f16 or args.scheme != "all" or args.total or args.playouts
                    or args.batch != 4096)
    extras, ref_leg = {}, None
    if headline and not args.no_extras:
        # outside the timed regions: the other configurations, and the reference's own kernel
        # timed against this one on the same GPU
        extras = other_configs(net, enc, dev, world, rank, barrier, all_max)
        if rank == 0:
            ref_leg = reference_kernel_leg(enc, (d_b, d_c, d_r), dev)

    times = torch.tensor([dev_ms, e2e_ms, e2e_pri_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, e2e_pri_ms = float(times[0]), float(times[1]), float(times[2])
    if rank != 0:
        if world > 1:
            # rank 0 still has its probes and the CPU baseline to run: wait for it on the
            # rendezvous store (a blocking socket read), not in a collective, whose waiters spin
            # on host cores and would take them from the CPU baseline
            from datetime import timedelta
            dist.distributed_c10d._get_default_store().wait(["bench_rank0_done"], timedelta(minutes=20))
            dist.destroy_process_group()
        return 0

    value = n_global * args.steps / (dev_ms * 1e-3)
    e2e = n_global * e2e_steps / (e2e_ms * 1e-3)
    peak, peak_src = peaks()
    kern_avg_ms = float(np.mean(kernel_ms))
    achieved = n_local * OPS_PER_POSITION / (kern_avg_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": "positions/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": "e4m3 (FFN) + f16" if args.fp8 else ("f16" if args.f16 else
                                                      {"all": "s8", "ffn": "s8 (FFN) + f16",
                                                       "ffn+qkv": "s8 (FFN, QKV) + f16"}[args.scheme]),
        "data": data,
        "config": {"workload": WORKLOAD, "positions_per_step": n_global, "parallelism": f"dp{world}",
                   "l2": "flushed between timed iterations (256 MiB fill)",
                   "timing": "CUDA events per launch on the launching stream, summed; max over ranks",
                   "wall_ms_incl_flush": t_wall * 1e3},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "peak_source": peak_src + "; int8 dense nominal 4500",
                     "traffic": profiled_traffic() if (n_local == 4096 and not args.fp8 and not args.f16
                                                       and args.scheme == "all") else None,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this "
                                       "kernel at batch 4096, read from profiles/encoder_kernel_batch4096_ncu_full.md",
                     "hbm_algorithmic_GBps": n_local * (BYTES_IN + BYTES_OUT) / (kern_avg_ms * 1e-3) / 1e9},
        "e2e": {"value": e2e, "unit": "positions/s", "h2d_bytes_per_step": n_local * BYTES_IN,
                "d2h_bytes_per_step": n_local * BYTES_OUT,
                "host_link_GBps_rank0": enc.host_link_gbps,
                "launch_sizes_rank0": enc.host_plan(n_local),
                "plan": "the call sizes its launches by the device-to-host rate it measured on its previous "
                        "call: each launch as many times the next as copying a position is faster than "
                        "evaluating it (at most 6), the last a single wave; under 1.5 times, equal two-wave "
                        "launches with the last wave written straight into the pinned buffers"},
        "e2e_fused_expansion": {"value": n_global * e2e_steps / (e2e_pri_ms * 1e-3), "unit": "positions/s",
                                "what": "the same step through forward_priors_host: legality words in, "
                                        "edge lists (fp16 priors, move labels, counts) and values out",
                                "h2d_bytes_per_step": n_local * (BYTES_IN + 256),
                                "d2h_bytes_per_step": n_local * (e_cap * 4 + 8)},
        "gpu_launches": launches, "clocks": clocks,
    }
    if phases is not None:
        line["phases_cycles_per_launch"] = phases
    line.update(extras)
    if ref_leg is not None:
        line["reference_kernel"] = ref_leg
    if True:
        # the tensor pipe's own int8 rate on this GPU (rank 0's, at every N) (a tcgen05 kind::i8 loop on resident
        # operands) is the denominator when it can be measured; the fractions of 2 x the measured
        # bf16 rate and of the nominal int8 rate are kept beside it
        import ctypes
        from brokefish_b200 import _native
        tops, ms = ctypes.c_double(0), ctypes.c_double(0)
        rf = line["roofline"]
        rf["frac_of_2x_bf16_measured"], rf["frac_of_nominal_4500"] = achieved / peak, achieved / 4500.0
        if _native.lib().bf_measure_i8_peak(local, 16384, ctypes.byref(tops), ctypes.byref(ms)) == 0:
            rf["peak"], rf["frac"] = tops.value, achieved / tops.value
            rf["peak_source"] = ("measured on this GPU in this run: tcgen05.mma kind::i8 loop on resident "
                                 "operands (bf_measure_i8_peak); 2 x measured dense bf16 burst "
                                 "(MEASURED_PEAKS.json) = %.0f; int8 dense nominal 4500" % peak)
        # the second roof: the time the element-wise arithmetic between the GEMMs needs on the
        # CUDA cores at the rate the row warps' own device functions reach in isolation
        # (per position and layer: 32 rows x the widths below; attention, heads and embedding
        # are not counted, so the floor is an underestimate)
        if not args.f16 and not args.fp8 and args.scheme == "all":
            widths = {0: 1024, 1: 768 + 256, 2: 1024, 3: 2 * 256, 4: 2 * 256, 5: 256}
            rates, floor_s = {}, 0.0
            for block, width in widths.items():
                eps = ctypes.c_double(0)
                if _native.lib().bf_measure_elementwise(local, block, 4000, ctypes.byref(eps), None) != 0:
                    rates = None
                    break
                rates[block] = eps.value
                floor_s += n_local * 8 * 32 * width / eps.value
            # the same sum for the cheaper, no longer bit-exact forms of the blocks (one combined
            # scale, requantisation in fp16 or fused into the normalise): what a tolerance arm
            # could save at most on the CUDA cores
            cheap_s, cheap = 0.0, {8: 1024, 10: 768 + 256, 11: 1024, 3: 2 * 256, 9: 2 * 256, 5: 256}
            for block, width in cheap.items():
                eps = ctypes.c_double(0)
                if rates is None or _native.lib().bf_measure_elementwise(local, block, 4000, ctypes.byref(eps), None) != 0:
                    cheap_s = None
                    break
                cheap_s += n_local * 8 * 32 * width / eps.value
            if cheap_s:
                rf["cuda_core_floor_cheaper_arithmetic_ms"] = cheap_s * 1e3
            if rates:
                names = ["ff1_epilogue", "descale_bias", "ff2_step", "norm_statistics", "normalise_quantise", "quantise"]
                rf["cuda_core_floor"] = {
                    "ms": floor_s * 1e3, "frac_of_step": floor_s * 1e3 / kern_avg_ms,
                    "elements_per_ns_per_sm": {names[b]: r / 1e9 / 148 for b, r in rates.items()},
                    "what": "sum over the element-wise blocks of elements per launch / isolated rate "
                            "(bf_measure_elementwise: same device functions, operands in shared memory, "
                            "16 warps per SM, no tensor-memory loads, exchanges or barriers)"}
    if not args.no_cpu_baseline:
        cv, cms, info = cpu_reference(25, 3)
        line["cpu_baseline"] = dict(info, value=cv, unit="positions/s")
    print(json.dumps(line))
    if world > 1:
        dist.distributed_c10d._get_default_store().set("bench_rank0_done", "1")
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
