"""Prior-space validation of an evaluator: does it still agree where the search looks?

The reference judges a quantised or fused evaluator not in logit space but by the quantity
its search consumes, the prior over a node's legal edges (brokefish/nn/validate.py:1-57), and
obtains that prior from the search's own expansion step.  This module restates that step
(:func:`expand_priors`, after ``Search._expand``, brokefish/search/torch_impl.py:962-1033) as
a plain function of logits and a legality mask, and the reference's metrics
(:func:`compare`, after brokefish/nn/validate.py:314-388), so that the B200 evaluator can be
scored the same way without the search or the rules engine:

    python -m brokefish_b200.validate --positions tests/golden/positions_4096_seed1.npz

Positions arrive with their legal-move words (bit ``s`` of word ``p`` set when the move of
slot ``p`` to square ``s`` is legal); positions without a legal move are dropped, as the
reference drops terminal positions (validate.py:172-177).

The expansion: a candidate is a legal (slot, square) pair, times the four promotion types
when the moving piece is a pawn reaching its last rank.  Its logit is the policy logit plus,
for promotions, the log-softmax of the slot's four promotion logits; the prior is the
softmax over the node's candidates.  When a node has more than ``e_cap`` candidates the
``e_cap`` largest are kept (ties by canonical order: slot, then square, then N B R Q) and
the prior is renormalised over them.  Priors are stored as fp16, as the search stores them.
"""

from __future__ import annotations

import argparse
import copy
import os
import sys
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Sequence

import numpy as np
import torch

PAWN = 0                        # piece type code (brokefish/env/torch_impl.py:45)
PROMO_SHIFT = 11                # move label: field (slot * 64 + square) | promotion type << 11
FP16_SUBNORMAL_MIN = 5.9604644775390625e-08


def legal_to_bool(legal: torch.Tensor) -> torch.Tensor:
    """``[N,32]`` int64 words -> ``[N,32,64]`` bool."""
    rng = torch.arange(64, device=legal.device, dtype=torch.int64)
    return ((legal.to(torch.int64)[..., None] >> rng) & 1).bool()


def promotion_targets(boards: torch.Tensor, control: torch.Tensor) -> torch.Tensor:
    """``[N,32,64]``: the slot holds a live pawn and the square is on the mover's last rank
    (rank 0 when ``control < 0``, else rank 7; torch_impl.py:950-959)."""
    words = boards.to(torch.int32)
    pawn = (((words >> 6) & 0b111) == PAWN) & (((words >> 11) & 1) == 0)
    last_rank = torch.where(control < 0, 0, 7).long()
    sq = torch.arange(64, device=boards.device)
    on_last = (sq[None, :] // 8) == last_rank[:, None]
    return pawn[:, :, None] & on_last[:, None, :]


def _largest(score: torch.Tensor, live: torch.Tensor, k: int) -> torch.Tensor:
    """Of the live entries of each row, mark the ``k`` with the highest score; equal scores
    go to the lower index (a stable ascending sort of the negated score)."""
    neg = torch.where(live, -score, torch.full_like(score, float("inf")))
    by_rank = neg.argsort(dim=-1, stable=True)
    place = torch.empty_like(by_rank)
    place.scatter_(1, by_rank, torch.arange(score.shape[1], device=score.device).expand_as(by_rank))
    return live & (place < k)


@torch.no_grad()
def expand_priors(boards, control, legal, policy, promo, e_cap: int = 96):
    """``(prior [N, e_cap] fp32 read back from fp16, move [N, e_cap] int16, nedges [N])``.

    The arithmetic of ``Search._expand``: fp32 log-softmax of the promotion logits, fp32
    softmax over the kept candidates, fp16 storage; edges in canonical order."""
    n, dev = boards.shape[0], boards.device
    moves_ok = legal_to_bool(legal)                                           # [N,32,64]
    promotes = promotion_targets(boards, control) & moves_ok
    # candidate (slot, square, type): type 0 for every legal move, types 1-3 only for promotions
    types = torch.arange(4, device=dev)
    live = (moves_ok[..., None] & ((types == 0) | promotes[..., None])).reshape(n, -1)
    type_logp = torch.log_softmax(promo.float(), dim=-1)[:, :, None, :]       # [N,32,1,4]
    score = policy.float()[..., None] + torch.where(promotes[..., None], type_logp,
                                                    torch.zeros((), device=dev))
    score = score.reshape(n, -1)                                              # [N, 32*64*4]
    total = live.sum(-1)
    kept = _largest(score, live, e_cap) if int(total.max() if n else 0) > e_cap else live
    dist = torch.softmax(score.masked_fill(~kept, float("-inf")), dim=-1)
    where_n, where_c = kept.nonzero(as_tuple=True)
    edge = (kept.cumsum(-1) - 1)[where_n, where_c]                            # canonical order
    priors = torch.zeros((n, e_cap), dtype=torch.float16, device=dev)
    labels = torch.zeros((n, e_cap), dtype=torch.int16, device=dev)
    priors[where_n, edge] = dist[where_n, where_c].to(torch.float16)
    labels[where_n, edge] = ((where_c // 4) | ((where_c % 4) << PROMO_SHIFT)).to(torch.int16)
    return priors.float(), labels, kept.sum(-1)


@dataclass
class Delta:
    """One variant scored against the fp32 network, in probability space (the fields of the
    reference's ``Delta``, brokefish/nn/validate.py:288-311)."""
    name: str
    max_abs: float
    p95_abs: float
    max_rel: float
    max_kl: float
    mean_kl: float
    top1_disagree: float
    top3_miss: float
    flip_risk: float
    flushed: int
    edge_set_differs: int
    max_abs_logit: float
    nonfinite: int
    max_abs_value: float
    aliases_across_calls: bool = False

    def line(self) -> str:
        return (f"  {self.name:<10} |dp| max {self.max_abs:.3e}  p95 {self.p95_abs:.3e}"
                f"   rel {self.max_rel:7.2%}   KL max {self.max_kl:.2e}"
                f"   top1 {self.top1_disagree:6.3%}  flip {self.flip_risk:6.3%}"
                f"   flush {self.flushed:5d}")


def compare(name: str, ref, got, rel_floor: float = 1e-3) -> Delta:
    """``ref`` and ``got`` are ``(prior, move, nedges, policy, promo, value)``.  Positions
    whose kept edge set differs are counted in ``edge_set_differs`` and left out of the
    probability metrics; with nothing comparable the maxima are ``inf``, never 0."""
    pr, mr, nr = ref[0], ref[1], ref[2]
    pg, mg, ng, pol_g, pro_g, val_g = got
    width = pr.shape[1]
    in_node = torch.arange(width, device=pr.device)[None, :] < nr[:, None]
    comparable = (nr == ng) & ((mr == mg) | ~in_node).all(-1)        # same edges, same order
    use = in_node & comparable[:, None]
    err = (pg - pr).abs().masked_fill(~use, 0.0)
    picked = comparable.nonzero(as_tuple=True)[0]
    denom = max(int(picked.numel()), 1)

    # KL(ref || got); a prior flushed to zero is clamped at the smallest positive fp16
    ratio = pr.clamp(min=1e-30) / pg.clamp(min=FP16_SUBNORMAL_MIN)
    kl = (pr * ratio.log()).masked_fill(~(use & (pr > 0)), 0.0).sum(-1)[picked]

    lowest = torch.finfo(torch.float32).min
    ranked_ref = pr.masked_fill(~use, lowest)
    ranked_got = pg.masked_fill(~use, lowest)
    best_ref = ranked_ref.argmax(-1)
    moved = (best_ref != ranked_got.argmax(-1))[picked]
    in_top3 = (ranked_got.topk(min(3, width), dim=-1).indices == best_ref[:, None]).any(-1)[picked]
    lead = ranked_ref.topk(min(2, width), dim=-1).values
    margin = lead[:, 0] - lead[:, 1] if lead.shape[1] == 2 else torch.ones_like(lead[:, 0])
    could_flip = (err.max(-1).values > margin)[picked]

    weighty = use & (pr >= rel_floor)
    bad_numbers = sum(int((~torch.isfinite(t.float())).sum()) for t in (pol_g, pro_g, val_g))
    return Delta(
        name=name,
        max_abs=float(err.max()) if bool(use.any()) else float("inf"),
        p95_abs=float(torch.quantile(err[use], 0.95)) if bool(use.any()) else float("inf"),
        max_rel=float((err[weighty] / pr[weighty]).max()) if bool(weighty.any()) else float("inf"),
        max_kl=float(kl.max()) if kl.numel() else 0.0,
        mean_kl=float(kl.mean()) if kl.numel() else 0.0,
        top1_disagree=float(moved.sum()) / denom,
        top3_miss=float((~in_top3).sum()) / denom,
        flip_risk=float(could_flip.sum()) / denom,
        flushed=int((use & (pr > 0) & (pg == 0)).sum()),
        edge_set_differs=int((~comparable).sum()),
        max_abs_logit=float(pol_g.float().abs().max()),
        nonfinite=bad_numbers,
        max_abs_value=float((val_g.float() - ref[5].float()).abs().max()))


def _same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    kind = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
    return bool((a.contiguous().view(kind) == b.contiguous().view(kind)).all())


@torch.no_grad()
def aliases_across_calls(fn, boards, control, rep) -> bool:
    """Does a second call overwrite what the first returned?  (It does for ``FusedEncoder``:
    outputs are views of reused buffers, as in the reference, validate.py:203-234.)"""
    n = boards.shape[0]
    if n < 2:
        return False
    half = max(n // 2, 1)
    first = fn(boards[:half], control[:half], rep[:half])
    keep = tuple(t.clone() for t in first)
    fn(boards[half:2 * half], control[half:2 * half], rep[half:2 * half])
    return not all(_same_bits(k, t) for k, t in zip(keep, first))


@torch.no_grad()
def run_logits(fn, boards, control, rep, chunk: int = 1024):
    """Any forward, chunked, every chunk cloned (the outputs may be reused buffers)."""
    pol, pro, val = [], [], []
    for lo in range(0, boards.shape[0], chunk):
        p, q, v = fn(boards[lo:lo + chunk], control[lo:lo + chunk], rep[lo:lo + chunk])
        pol.append(p.clone())
        pro.append(q.clone())
        val.append(v.clone())
    return torch.cat(pol), torch.cat(pro), torch.cat(val)


@torch.no_grad()
def validate(net, boards, control, rep, legal, forwards: Dict[str, Callable], e_cap: int = 96,
             rel_floor: float = 1e-3, verbose: bool = True) -> Dict[str, Delta]:
    """Every forward in ``forwards`` (name -> ``(boards, control, rep) -> (policy, promo,
    value)``) against the fp32 network on fp16-rounded weights, plus the two yardsticks of the
    reference: ``store`` (the fp32 logits rounded to fp16, the floor of the storage format) and
    ``torch16`` (the same module in fp16 arithmetic, where the device supports it)."""
    keep = (legal != 0).any(-1).nonzero(as_tuple=True)[0]
    boards, control, rep, legal = (t[keep].contiguous() for t in (boards, control, rep, legal))
    if boards.shape[0] == 0:
        raise RuntimeError("every position was terminal; nothing to validate")
    dev = boards.device
    net16 = copy.deepcopy(net).to(dev).half().eval()
    net32 = copy.deepcopy(net16).float()

    def bundle(policy, promo, value):
        pri, mov, ne = expand_priors(boards, control, legal, policy, promo, e_cap)
        return (pri, mov, ne, policy, promo, value)

    ref_logits = run_logits(net32, boards, control, rep)
    ref = bundle(*ref_logits)
    variants = {"store": bundle(ref_logits[0].half().float(), ref_logits[1].half().float(), ref_logits[2])}
    if dev.type == "cuda":
        variants["torch16"] = bundle(*run_logits(net16, boards, control, rep))
    aliasing = {}
    for name, fn in forwards.items():
        aliasing[name] = aliases_across_calls(fn, boards, control, rep)
        variants[name] = bundle(*run_logits(fn, boards, control, rep))
    if verbose:
        print(f"positions   {boards.shape[0]} non-terminal, E = {e_cap}, max |policy logit| "
              f"{float(ref_logits[0].abs().max()):.2f}, mean edges {float(ref[2].float().mean()):.1f}, "
              f"max {int(ref[2].max())}")
    out = {}
    for name, got in variants.items():
        out[name] = compare(name, ref, got, rel_floor=rel_floor)
        out[name].aliases_across_calls = bool(aliasing.get(name, False))
        if verbose:
            print(out[name].line())
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--positions", required=True, help=".npz with boards, control, rep, legal")
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--e-cap", type=int, default=96)
    ap.add_argument("--std", type=float, default=0.02, help="N(0, std) seed-0 weights; 0 = default init scale")
    ap.add_argument("--reference", default=os.environ.get("BROKEFISH_REFERENCE", ""),
                    help="checkout of the reference: its BrokefishNet is the fp32 yardstick "
                         "(default: $BROKEFISH_REFERENCE)")
    args = ap.parse_args(argv)
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import seeded_state
    # the fp32 yardstick is the reference's own network, called as the reference's validator
    # calls it; this package holds weights and the kernel, not a second torch forward path
    if not args.reference or not os.path.isdir(os.path.join(args.reference, "brokefish")):
        raise SystemExit("validate needs the reference's network as its yardstick: pass --reference "
                         "<checkout> or set BROKEFISH_REFERENCE")
    sys.path.insert(0, args.reference)
    from brokefish.nn.model import BrokefishNet
    z = np.load(args.positions)
    n = args.limit or z["boards"].shape[0]
    dev = torch.device("cuda")
    boards, control, rep = (torch.from_numpy(np.ascontiguousarray(z[k][:n])).to(dev) for k in ("boards", "control", "rep"))
    legal = torch.from_numpy(z["legal"][:n].view(np.int64).copy()).to(dev)
    net = BrokefishNet().eval()
    net.load_state_dict(seeded_state(seed=0, std=args.std or None, perturb_norms=not args.std))
    net = net.half().float()
    forwards = {"b200-int8": encoder_impl("cuda")(net, int8=True).forward_full,
                "b200-e4m3": encoder_impl("cuda")(net, fp8=True).forward_full}
    validate(net, boards, control, rep, legal, forwards, e_cap=args.e_cap)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
