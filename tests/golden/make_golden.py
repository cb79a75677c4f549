"""Generate the committed golden fixtures from the reference's own Python.

Run in a container that holds the reference checkout (read-only), from the repo root:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <reference checkout>

It imports the reference (``brokefish.nn.model``, ``brokefish.nn.quant``,
``brokefish.nn.cuda_impl._fold_norm``, ``brokefish.env.torch_impl``) on CPU and writes,
next to this script:

* ``positions_256_seed0.npz``, ``positions_4096_seed1.npz`` -- boards / control / rep /
  legal-move words from uniformly random legal playouts of 0-120 plies with the
  reference's move generator (the recipe of the reference's tests/boards.py, with a
  per-position ply count);
* ``ref_outputs_A.npz``, ``ref_outputs_B.npz`` -- for two seeded weight sets, the
  reference network's fp32 outputs, its int8-emulated outputs, its fp16 embedding and
  digests of its folded + quantised weights;
* ``ref_outputs_C.npz`` -- the reference fp32 network's outputs for a network with per-layer
  input re-injection at both norms and nonzero coefficients;
* ``ref_priors.npz`` -- priors, move labels and edge counts that the reference's search
  (``Search.root_init`` -> ``_expand``) derives from its fp32 network's fp16 logits on 160
  non-terminal positions, at edge caps 96 and 12, and the reference validator's metrics on a
  perturbed copy of those logits;
* ``ref_movegen.npz`` -- the reference move generator's legal words and check flags on 17
  hand-picked positions (its adversarial FENs, castling, en passant, pins, mates), and its check
  flags for the two playout sets;
* ``scheme_kats.npz`` -- known answers of the reference's int8 scheme functions.

The fixtures are what ``tests/test_oracle_golden.py`` pins the CPU oracle against; the
GPU box never needs the reference.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def playout_positions(env, n: int, seed: int, max_plies: int = 120):
    """Uniform-random legal playouts, game i snapshotted after ``plies[i]`` moves."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    plies = torch.randint(0, max_plies + 1, (n,), generator=gen)
    boards, control = env.initial_boards(n, device="cpu")
    mask, _ = env.movegen(boards, control)
    out_b, out_c, out_m = boards.clone(), control.clone(), mask.clone()
    for ply in range(max_plies + 1):
        snap = plies == ply
        out_b[snap], out_c[snap], out_m[snap] = boards[snap], control[snap], mask[snap]
        if ply == max_plies:
            break
        legal = env.bitset_to_bool(mask).reshape(n, 32 * 64)
        counts = legal.sum(dim=1)
        live = counts > 0
        r = torch.rand(n, generator=gen)
        pick = (r * counts.clamp(min=1).float()).long()
        pick = torch.minimum(pick, (counts - 1).clamp(min=0))
        move = (legal.cumsum(dim=1) > pick[:, None]).float().argmax(dim=1)
        move = torch.where(live, move, torch.zeros_like(move))
        promo = torch.randint(0, 4, (n,), generator=gen)
        nb, nc, nm, _ = env.play(boards, control, move.to(torch.int64), promo=promo)
        boards = torch.where(live[:, None], nb, boards)
        control = torch.where(live, nc, control)
        mask = torch.where(live[:, None], nm, mask)
        if ply % 20 == 0:
            print(f"  ply {ply}: {int(live.sum())}/{n} games live", flush=True)
    rep = (torch.arange(n) % 3).to(torch.uint8)
    return (out_b.numpy().astype(np.int16), out_c.numpy().astype(np.int16),
            rep.numpy(), out_m.numpy().astype(np.int64).view(np.uint64), plies.numpy())


def step_answers(env) -> None:
    """The engine's `step` / `play` on one random legal move (random promotion type) from each of
    the 4096 playout positions -- every 16th board gets the null move -- and on hand-picked
    castling, en passant and promotion moves: new words, control, the irreversible flag and the
    next position's legal words and check flag."""
    z = np.load(os.path.join(HERE, "positions_4096_seed1.npz"))
    boards, control = torch.from_numpy(z["boards"]), torch.from_numpy(z["control"])
    mask = torch.from_numpy(z["legal"].view(np.int64))
    n = boards.shape[0]
    gen = torch.Generator(device="cpu").manual_seed(7)
    legal = env.bitset_to_bool(mask).reshape(n, 32 * 64)
    counts = legal.sum(dim=1)
    pick = torch.minimum((torch.rand(n, generator=gen) * counts.clamp(min=1).float()).long(), (counts - 1).clamp(min=0))
    move = (legal.cumsum(dim=1) > pick[:, None]).float().argmax(dim=1)
    move = torch.where((counts > 0) & (torch.arange(n) % 16 != 5), move, torch.full_like(move, -1))
    promo = torch.randint(0, 4, (n,), generator=gen)
    nb, nc, _, irr = env.step(boards, control, move, promo=promo)
    nm, chk = env.movegen(nb, nc)
    out = {"move": move.numpy().astype(np.int32), "promo": promo.numpy().astype(np.int8),
           "boards": nb.numpy().astype(np.int16), "control": nc.numpy().astype(np.int16),
           "irreversible": irr.numpy(), "legal": nm.numpy().astype(np.int64).view(np.uint64),
           "in_check": chk.numpy()}
    # hand-picked: (FEN, from, to, promotion type or -1 for the default)
    sq = lambda name: (ord(name[0]) - 97) + 8 * (int(name[1]) - 1)
    cases = [("r3k2r/pppppppp/8/8/8/8/PPPPPPPP/R3K2R w KQkq - 0 1", "e1", "g1", -1),
             ("r3k2r/pppppppp/8/8/8/8/PPPPPPPP/R3K2R w KQkq - 0 1", "e1", "c1", -1),
             ("r3k2r/8/8/8/8/8/8/R3K2R b KQkq - 0 1", "e8", "g8", -1),
             ("r3k2r/8/8/8/8/8/8/R3K2R b KQkq - 0 1", "e8", "c8", -1),
             ("r3k2r/8/8/8/8/8/8/R3K2R b KQkq - 5 9", "a8", "a1", -1),       # rook takes rook: both lose rights
             ("r3k2r/8/8/8/8/8/8/R3K2R w KQkq - 5 9", "h1", "h4", -1),       # quiet rook move: a right goes
             ("rnbqkbnr/ppp1p1pp/8/3pPp2/8/8/PPPP1PPP/RNBQKBNR w KQkq f6 0 3", "e5", "f6", -1),
             ("rnbqkbnr/ppp1p1pp/8/3pPp2/8/8/PPPP1PPP/RNBQKBNR w KQkq f6 0 3", "e5", "e6", -1),
             ("rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1", "e2", "e4", -1),
             ("rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1", "g1", "f3", -1),
             ("8/2P5/8/8/8/8/5p2/K2k4 w - - 0 1", "c7", "c8", -1),
             ("8/2P5/8/8/8/8/5p2/K2k4 w - - 0 1", "c7", "c8", 0),
             ("8/2P5/8/8/8/8/5p2/K2k4 w - - 0 1", "c7", "c8", 1),
             ("8/2P5/8/8/8/8/5p2/K2k4 b - - 0 1", "f2", "f1", 2),
             ("8/2P5/8/8/8/8/5p2/K2k4 b - - 0 1", "f2", "f1", 3),
             ("4k3/8/8/8/8/8/8/4K2R w K - 12 30", "e1", "e2", -1)]           # quiet king move: the counter goes up
    fb, fc, fmv, fpr = [], [], [], []
    for fen, a, b, pr in cases:
        bb, cc = env.from_fen(fen)
        slot = int((((bb[0] & 63) == sq(a)) & ((bb[0] >> 11) == 0)).int().argmax())
        fb.append(bb); fc.append(cc); fmv.append(slot * 64 + sq(b)); fpr.append(3 if pr < 0 else pr)
    fb, fc = torch.cat(fb), torch.cat(fc)
    fmv, fpr = torch.tensor(fmv), torch.tensor(fpr)
    legal_before, _ = env.movegen(fb, fc)
    ok = (legal_before[torch.arange(len(cases)), fmv // 64] >> (fmv % 64)) & 1
    assert bool(ok.all()), "a hand-picked move is not legal"
    hb, hc, _, hirr = env.step(fb, fc, fmv, promo=fpr)
    hm, hchk = env.movegen(hb, hc)
    out.update({"case_boards_in": fb.numpy().astype(np.int16), "case_control_in": fc.numpy().astype(np.int16),
                "case_move": fmv.numpy().astype(np.int32), "case_promo": fpr.numpy().astype(np.int8),
                "case_boards": hb.numpy().astype(np.int16), "case_control": hc.numpy().astype(np.int16),
                "case_irreversible": hirr.numpy(), "case_legal": hm.numpy().astype(np.int64).view(np.uint64),
                "case_in_check": hchk.numpy(), "cases": np.array([f"{f} {a}{b}" for f, a, b, _ in cases])})
    np.savez_compressed(os.path.join(HERE, "ref_step.npz"), **out)


def shuffled_answers(env) -> None:
    """The engine on boards whose slots do not keep the colours apart: 512 playout positions with
    the thirty non-king slots permuted at random (the kings stay in slots 15 and 31), one random
    legal move each.  Every rule reads colour, type and square from the word, so the reference's
    answers are the same moves under the same permutation; a kernel that walks "its own sixteen
    slots" must notice that it cannot here."""
    z = np.load(os.path.join(HERE, "positions_4096_seed1.npz"))
    n = 512
    gen = torch.Generator(device="cpu").manual_seed(21)
    boards, control = torch.from_numpy(z["boards"][:n]).clone(), torch.from_numpy(z["control"][:n])
    others = torch.tensor([i for i in range(32) if i not in (15, 31)])
    for i in range(n):
        boards[i, others] = boards[i, others[torch.randperm(30, generator=gen)]]
    mask, chk = env.movegen(boards, control)
    legal = env.bitset_to_bool(mask).reshape(n, 32 * 64)
    counts = legal.sum(dim=1)
    pick = torch.minimum((torch.rand(n, generator=gen) * counts.clamp(min=1).float()).long(), (counts - 1).clamp(min=0))
    move = (legal.cumsum(dim=1) > pick[:, None]).float().argmax(dim=1)
    move = torch.where(counts > 0, move, torch.full_like(move, -1))
    promo = torch.randint(0, 4, (n,), generator=gen)
    nb, nc, _, irr = env.step(boards, control, move, promo=promo)
    nm, nchk = env.movegen(nb, nc)
    np.savez_compressed(os.path.join(HERE, "ref_shuffled.npz"),
                        boards=boards.numpy().astype(np.int16), control=control.numpy().astype(np.int16),
                        legal=mask.numpy().astype(np.int64).view(np.uint64), in_check=chk.numpy(),
                        move=move.numpy().astype(np.int32), promo=promo.numpy().astype(np.int8),
                        next_boards=nb.numpy().astype(np.int16), next_control=nc.numpy().astype(np.int16),
                        irreversible=irr.numpy(), next_legal=nm.numpy().astype(np.int64).view(np.uint64),
                        next_in_check=nchk.numpy())


def terminal_answers(env) -> None:
    """The engine's `terminal` (no history) on the two playout sets and on hand-made positions:
    bare kings, one minor piece, bishops on one and on two colours of squares, two knights, a
    pawn, the fifty-move counter at and just under its limit, mate and stalemate (also with the
    counter at its limit: mate comes first)."""
    fens = ["8/8/8/4k3/8/8/8/4K3 w - - 0 1", "8/8/8/4k3/8/8/8/4KN2 w - - 0 1", "8/8/8/4k3/8/8/8/4KB2 b - - 0 1",
            "8/8/8/4k3/8/8/8/2B1KB2 w - - 0 1", "8/8/8/4k3/8/8/2B5/4KB2 w - - 0 1", "8/8/8/3bk3/8/8/8/4KB2 w - - 0 1",
            "8/8/8/2b1k3/8/8/8/4KB2 w - - 0 1", "8/8/8/4k3/8/8/8/3NKN2 w - - 0 1", "8/8/8/4k3/8/8/8/3NKB2 w - - 0 1",
            "8/8/8/3nk3/8/8/8/4KN2 w - - 0 1", "8/8/8/4k3/8/8/4P3/4K3 w - - 0 1", "8/8/8/4k3/8/8/8/4KR2 b - - 0 1",
            "8/8/8/4k3/8/8/4P3/4K3 w - - 100 80", "8/8/8/4k3/8/8/4P3/4K3 b - - 99 80", "8/8/8/4k3/8/8/4P3/4K3 b - - 120 90",
            "7k/5Q2/6K1/8/8/8/8/8 b - - 0 1", "7k/6Q1/6K1/8/8/8/8/8 b - - 0 1", "7k/6Q1/6K1/8/8/8/8/8 b - - 100 70",
            "7k/5Q2/6K1/8/8/8/8/8 b - - 100 70", "rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1",
            "1r1r2Rk/pp5p/4b2n/1P5P/n1Ppp3/R4P1p/1B1KP3/8 b - - 1 1"]
    fb, fc = zip(*(env.from_fen(f) for f in fens))
    fb, fc = torch.cat(fb), torch.cat(fc)
    fm, fk = env.movegen(fb, fc)
    code, result = env.terminal(fm, fk, fc, fb)
    out = {"fens": np.array(fens), "fen_boards": fb.numpy().astype(np.int16), "fen_control": fc.numpy().astype(np.int16),
           "fen_legal": fm.numpy().astype(np.int64).view(np.uint64), "fen_in_check": fk.numpy(),
           "fen_code": code.numpy(), "fen_result": result.numpy()}
    for n_pos, seed in ((256, 0), (4096, 1)):
        z = np.load(os.path.join(HERE, f"positions_{n_pos}_seed{seed}.npz"))
        b, c = torch.from_numpy(z["boards"]), torch.from_numpy(z["control"])
        m, k = env.movegen(b, c)
        code, result = env.terminal(m, k, c, b)
        out[f"code_{n_pos}"], out[f"result_{n_pos}"] = code.numpy(), result.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_terminal.npz"), **out)


def history_answers(env) -> None:
    """Position keys, the repetition ring and the threefold rule along 192 random games of up to
    100 plies -- half from the start position, half from positions with three or four pieces,
    where random play repeats itself often -- as the reference engine counts them: per ply the
    move played, the repetition count of the position reached and its terminal code with the
    history given.  And pairs of positions with the reference's verdict on whether their keys
    are equal (en passant flags that do and do not count, castling rights, side to move)."""
    sparse = ["8/8/8/4k3/8/8/8/R3K3 w Q - 0 1", "8/8/8/4k3/8/8/8/4KQ2 w - - 0 1", "8/8/8/3nk3/8/8/8/4KN2 b - - 0 1",
              "8/8/8/4k3/8/8/8/2B1KB2 w - - 0 1", "8/8/4k3/8/8/8/4P3/4K2R w K - 0 1", "6k1/8/8/8/8/8/8/R3K2R b KQ - 0 1"]
    n, plies = 192, 100
    bs, cs = [], []
    for i in range(n):
        b, c = env.initial_boards(1) if i < n // 2 else env.from_fen(sparse[i % len(sparse)])
        bs.append(b); cs.append(c)
    boards, control = torch.cat(bs), torch.cat(cs)
    gen = torch.Generator(device="cpu").manual_seed(33)
    mask, chk = env.movegen(boards, control)
    h = env.hash_position(boards, control)
    ring, length = env.empty_history(n)
    active = torch.ones(n, dtype=torch.bool)
    moves = np.full((plies, n), -1, dtype=np.int32)
    promos = np.zeros((plies, n), dtype=np.int8)
    counts = np.zeros((plies, n), dtype=np.uint8)
    codes = np.zeros((plies, n), dtype=np.uint8)
    for ply in range(plies):
        legal = env.bitset_to_bool(mask).reshape(n, 32 * 64)
        cnt = legal.sum(dim=1)
        pick = torch.minimum((torch.rand(n, generator=gen) * cnt.clamp(min=1).float()).long(), (cnt - 1).clamp(min=0))
        move = (legal.cumsum(dim=1) > pick[:, None]).float().argmax(dim=1)
        move = torch.where(active & (cnt > 0), move, torch.full_like(move, -1))
        promo = torch.randint(0, 4, (n,), generator=gen)
        nb, nc, nh, irr = env.step(boards, control, move, promo=promo, hash=h)
        played = move >= 0
        r2, l2 = env.push_history(ring, length, h, irr)
        ring = torch.where(played[:, None], r2, ring)
        length = torch.where(played, l2, length)
        boards, control, h = nb, nc, nh
        mask, chk = env.movegen(boards, control)
        code, _ = env.terminal(mask, chk, control, boards, h, ring, length)
        moves[ply], promos[ply] = move.numpy(), promo.numpy()
        counts[ply] = env.repetition_count(h, ring, length).clamp(max=255).numpy()
        codes[ply] = code.numpy()
        active &= code == 0
    pairs = [("rnbqkbnr/ppp1p1pp/8/3pPp2/8/8/PPPP1PPP/RNBQKBNR w KQkq f6 0 3", "rnbqkbnr/ppp1p1pp/8/3pPp2/8/8/PPPP1PPP/RNBQKBNR w KQkq - 0 3"),
             ("4k3/8/8/8/4Pp2/8/8/4K3 b - e3 0 1", "4k3/8/8/8/4Pp2/8/8/4K3 b - - 0 1"),
             ("4k3/8/8/8/4P3/8/8/4K3 b - e3 0 1", "4k3/8/8/8/4P3/8/8/4K3 b - - 0 1"),
             ("8/8/8/8/k2Pp2Q/8/8/4K3 b - d3 0 1", "8/8/8/8/k2Pp2Q/8/8/4K3 b - - 0 1"),
             ("r3k2r/8/8/8/8/8/8/R3K2R w KQkq - 0 1", "r3k2r/8/8/8/8/8/8/R3K2R w KQ - 0 1"),
             ("r3k2r/8/8/8/8/8/8/R3K2R w KQkq - 0 1", "r3k2r/8/8/8/8/8/8/R3K2R b KQkq - 0 1"),
             ("r3k2r/8/8/8/8/8/8/R3K2R w KQkq - 0 1", "r3k2r/8/8/8/8/8/8/R3K2R w KQkq - 7 9")]
    pa, pc, qa, qc = [], [], [], []
    for a, b in pairs:
        x, y = env.from_fen(a), env.from_fen(b)
        pa.append(x[0]); pc.append(x[1]); qa.append(y[0]); qc.append(y[1])
    pa, pc, qa, qc = torch.cat(pa), torch.cat(pc), torch.cat(qa), torch.cat(qc)
    same = env.hash_position(pa, pc) == env.hash_position(qa, qc)
    np.savez_compressed(os.path.join(HERE, "ref_history.npz"),
                        boards=torch.cat(bs).numpy().astype(np.int16), control=torch.cat(cs).numpy().astype(np.int16),
                        moves=moves, promos=promos, counts=counts, codes=codes,
                        pair_a=pa.numpy().astype(np.int16), pair_a_control=pc.numpy().astype(np.int16),
                        pair_b=qa.numpy().astype(np.int16), pair_b_control=qc.numpy().astype(np.int16),
                        pair_same=same.numpy(), pairs=np.array([f"{a} | {b}" for a, b in pairs]))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("BROKEFISH_REFERENCE"), required="BROKEFISH_REFERENCE" not in os.environ,
                    help="checkout of the reference (default: $BROKEFISH_REFERENCE)")
    ap.add_argument("--skip-positions", action="store_true")
    ap.add_argument("--only-step", action="store_true", help="write ref_step.npz and stop")
    ap.add_argument("--only-shuffled", action="store_true", help="write ref_shuffled.npz and stop")
    ap.add_argument("--only-terminal", action="store_true", help="write ref_terminal.npz and stop")
    ap.add_argument("--only-history", action="store_true", help="write ref_history.npz and stop")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    torch.manual_seed(0)

    from brokefish.env import torch_impl as env                      # reference
    if args.only_step:
        step_answers(env)
        return 0
    if args.only_shuffled:
        shuffled_answers(env)
        return 0
    if args.only_terminal:
        terminal_answers(env)
        return 0
    if args.only_history:
        history_answers(env)
        return 0
    from brokefish.nn import quant as rq                             # reference
    from brokefish.nn.cuda_impl import _fold_norm                    # reference
    from brokefish.nn.model import BrokefishNet as RefNet            # reference
    from brokefish_b200.nn.model import seeded_state                 # ours: weights by seed

    for n, seed in ((256, 0), (4096, 1)):
        path = os.path.join(HERE, f"positions_{n}_seed{seed}.npz")
        if args.skip_positions and os.path.exists(path):
            continue
        print(f"positions n={n} seed={seed}", flush=True)
        b, c, r, m, plies = playout_positions(env, n, seed)
        np.savez_compressed(path, boards=b, control=c, rep=r, legal=m, plies=plies)

    pos = np.load(os.path.join(HERE, "positions_256_seed0.npz"))
    boards = torch.from_numpy(pos["boards"])
    control = torch.from_numpy(pos["control"])
    rep = torch.from_numpy(pos["rep"])

    sets = {"A": dict(seed=0, std=0.02, perturb_norms=False),
            "B": dict(seed=0, std=None, perturb_norms=True)}
    for name, kw in sets.items():
        print(f"weight set {name}", flush=True)
        state = seeded_state(**kw)
        net = RefNet().eval()
        net.load_state_dict(state, strict=True)
        out = {"state_sha": sha(np.concatenate(
            [state[k].numpy().reshape(-1).astype(np.float32) for k in sorted(state)]))}
        n_fp32, n_emu = 64, 32
        with torch.no_grad():
            p, pr, v = net(boards[:n_fp32], control[:n_fp32], rep[:n_fp32])
            out["fp32_policy"] = p.numpy().astype(np.float32)
            out["fp32_promo"] = pr.numpy().astype(np.float32)
            out["fp32_value"] = v.numpy().astype(np.float32)
            fwd = rq.emulated_forward(net, rq.QuantConfig(fmt="int8"))
            p, pr, v = fwd(boards[:n_emu], control[:n_emu], rep[:n_emu])
            out["emu_policy"] = p.numpy().astype(np.float32)
            out["emu_promo"] = pr.numpy().astype(np.float32)
            out["emu_value"] = v.numpy().astype(np.float32)
            # the reference's e4m3 arithmetic as its kernel ships it: the two FFN matmuls,
            # weights and activations, q_max 8, one scale over the whole 256-deep reduction
            cfg8 = rq.QuantConfig(fmt="e4m3", weights=True, activations=True, acc16=False,
                                  q_max=rq.Q_MAX, tile_k=rq.ROW_K)
            p, pr, v = rq.emulated_forward(net, cfg8, which=("ffn1", "ffn2"))(
                boards[:n_emu], control[:n_emu], rep[:n_emu])
            out["e4m3_policy"] = p.numpy().astype(np.float16)
            out["e4m3_value"] = v.numpy().astype(np.float32)
            half = RefNet().eval()
            half.load_state_dict(state, strict=True)
            half = half.half()
            x, alive = half.embed(boards, control, rep)
            out["embed_sha"] = sha(x.numpy())
            out["embed_first4"] = x[:4].numpy()
            out["alive"] = alive.numpy()
        # folded + quantised weights exactly as the reference constructor derives them
        # (brokefish/nn/cuda_impl.py:194-210, 356-369)
        digests, fb_qkv, fb_ff1 = [], [], []
        for li, lay in enumerate(net.encoder.layers):
            w_qkv = lay.self_attn.in_proj_weight.detach().float().clone()
            b_qkv = lay.self_attn.in_proj_bias.detach().float().clone()
            w_qkv[:256] *= 32 ** -0.5
            b_qkv[:256] *= 32 ** -0.5
            w_ff1 = lay.linear1.weight.detach().float().clone()
            b_ff1 = lay.linear1.bias.detach().float().clone()
            w_qkv, b_qkv = _fold_norm(w_qkv, b_qkv, lay.norm1)
            w_ff1, b_ff1 = _fold_norm(w_ff1, b_ff1, lay.norm2)
            for tag, wmat in (("qkv", w_qkv), ("o", lay.self_attn.out_proj.weight.detach()),
                              ("ff1", w_ff1), ("ff2", lay.linear2.weight.detach())):
                qb, sc = rq.quantise_weights_int8_bytes(wmat.float())
                digests.append(f"{li}.{tag}.q={sha(qb.numpy())}")
                digests.append(f"{li}.{tag}.s={sha(sc.numpy())}")
            fb_qkv.append(b_qkv.half().numpy())
            fb_ff1.append(b_ff1.half().numpy())
        out["weight_digests"] = np.array(digests)
        out["folded_b_qkv"] = np.stack(fb_qkv)
        out["folded_b_ff1"] = np.stack(fb_ff1)
        np.savez_compressed(os.path.join(HERE, f"ref_outputs_{name}.npz"), **out)

    # per-layer input re-injection (both norms), nonzero coefficients: fp32 reference outputs
    print("weight set C (re-injection)", flush=True)
    kw = dict(seed=7, std=None, perturb_norms=True, reinject="both")
    state = seeded_state(**kw)
    net = RefNet(reinject="both").eval()
    net.load_state_dict(state, strict=True)
    with torch.no_grad():
        p, pr, v = net(boards[:32], control[:32], rep[:32])
    np.savez_compressed(os.path.join(HERE, "ref_outputs_C.npz"),
                        state_sha=sha(np.concatenate([state[k].numpy().reshape(-1).astype(np.float32)
                                                      for k in sorted(state)])),
                        fp32_policy=p.numpy().astype(np.float16), fp32_promo=pr.numpy().astype(np.float16),
                        fp32_value=v.numpy().astype(np.float32))

    # the search's own expansion step on reference logits: priors, move labels and edge counts
    # (brokefish/nn/validate.py:248-280 run_priors -> Search.root_init -> Search._expand), with
    # the default edge cap and with a small one so that the truncation branch is exercised
    print("priors through the reference search", flush=True)
    from brokefish.nn.validate import compare as ref_compare, run_priors      # reference
    legal_words = torch.from_numpy(pos["legal"].view(np.int64).copy())
    rows = (legal_words != 0).any(-1).nonzero(as_tuple=True)[0][:160]
    state = seeded_state(**sets["B"])
    net = RefNet().eval()
    net.load_state_dict(state, strict=True)
    with torch.no_grad():
        pol, pro, val = net(boards[rows], control[rows], rep[rows])
    pol16, pro16 = pol.half(), pro.half()
    out = {"rows": rows.numpy(), "policy": pol16.numpy(), "promo": pro16.numpy(), "value": val.numpy()}
    for cap in (96, 12):
        pri, mov, ne = run_priors(boards[rows], control[rows], pol16, pro16, val, cap)
        out[f"prior_{cap}"] = pri.numpy().astype(np.float16)
        out[f"move_{cap}"] = mov.numpy()
        out[f"nedges_{cap}"] = ne.numpy()
    # the reference's metrics on a perturbed copy of the logits, as known answers for compare()
    g = torch.Generator().manual_seed(99)
    pol_b = (pol16.float() + 0.05 * torch.randn(pol16.shape, generator=g)).half()
    ref_b = (*run_priors(boards[rows], control[rows], pol16, pro16, val, 96), pol16, pro16, val)
    got_b = (*run_priors(boards[rows], control[rows], pol_b, pro16, val + 0.01, 96), pol_b, pro16, val + 0.01)
    dl = ref_compare("perturbed", ref_b, got_b)
    out["policy_perturbed"] = pol_b.numpy()
    out["delta_perturbed"] = np.array([dl.max_abs, dl.p95_abs, dl.max_rel, dl.max_kl, dl.mean_kl,
                                       dl.top1_disagree, dl.top3_miss, dl.flip_risk, dl.flushed,
                                       dl.edge_set_differs, dl.max_abs_logit, dl.nonfinite,
                                       dl.max_abs_value], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "ref_priors.npz"), **out)

    # the engine's move generator on positions no random playout reaches (the adversarial FENs
    # of brokefish/nn/validate.py:81-87 plus castling, en passant, pins and checks) and the check
    # flag of the two playout sets (their legal words are already in the position files)
    print("movegen known answers", flush=True)
    fens = [f for _, f in __import__("brokefish.nn.validate", fromlist=["ADVERSARIAL"]).ADVERSARIAL] + [
        "r3k2r/pppppppp/8/8/8/8/PPPPPPPP/R3K2R w KQkq - 0 1",
        "r3k2r/8/8/8/8/8/8/R3K2R b KQkq - 0 1",
        "r3k2r/8/8/8/8/8/6r1/R3K2R w KQkq - 0 1",          # g1 / f1 covered: no short castle
        "4k3/8/8/8/8/8/8/R3K2r w Q - 0 1",                  # in check: no castle
        "rnbqkbnr/ppp1p1pp/8/3pPp2/8/8/PPPP1PPP/RNBQKBNR w KQkq f6 0 3",   # en passant available
        "8/8/8/8/k2Pp2Q/8/8/4K3 b - d3 0 1",                # en passant would expose the king
        "4k3/8/8/8/8/4r3/4B3/4K3 w - - 0 1",                # pinned bishop
        "4k3/8/8/8/8/8/3n4/4K3 w - - 0 1",                  # knight check
        "7k/5Q2/6K1/8/8/8/8/8 b - - 0 1",                   # stalemate
        "7k/6Q1/6K1/8/8/8/8/8 b - - 0 1",                   # checkmate
        "8/2P5/8/8/8/8/5p2/K2k4 w - - 0 1",                 # promotions for both sides
        "8/2P5/8/8/8/8/5p2/K2k4 b - - 0 1",
    ]
    fb, fc = zip(*(env.from_fen(f) for f in fens))
    fb, fc = torch.cat(fb), torch.cat(fc)
    fm, fchk = env.movegen(fb, fc)
    out = {"fen_boards": fb.numpy().astype(np.int16), "fen_control": fc.numpy().astype(np.int16),
           "fen_legal": fm.numpy().astype(np.int64).view(np.uint64), "fen_in_check": fchk.numpy(),
           "fens": np.array(fens)}
    for n_pos, seed in ((256, 0), (4096, 1)):
        z = np.load(os.path.join(HERE, f"positions_{n_pos}_seed{seed}.npz"))
        m, chk = env.movegen(torch.from_numpy(z["boards"]), torch.from_numpy(z["control"]))
        assert np.array_equal(m.numpy().astype(np.int64).view(np.uint64), z["legal"])
        out[f"in_check_{n_pos}"] = chk.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_movegen.npz"), **out)

    print("step known answers", flush=True)
    step_answers(env)
    shuffled_answers(env)
    terminal_answers(env)
    history_answers(env)

    print("scheme known answers", flush=True)
    g = torch.Generator().manual_seed(1234)
    wmat = torch.randn(256, 256, generator=g) * 0.05
    wmat[128:] *= 3.0
    qb, sc = rq.quantise_weights_int8_bytes(wmat)
    acts = torch.randn(16, 256, generator=g)
    acts[3] = 0.0
    acts[4, :8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 127.0, -127.0])
    acts16 = acts.half().float()
    qs, ss = rq.quantise_activations_int8(acts16)
    qu, su = rq.quantise_activations_int8(acts16.relu(), unsigned=True)
    qb8, sc8 = rq.quantise_weights_bytes(wmat, rq.Q_MAX, tile_k=wmat.shape[1])
    lin = rq.int8_linear(acts16, wmat, torch.linspace(-1, 1, 256))
    np.savez_compressed(os.path.join(HERE, "scheme_kats.npz"),
                        w=wmat.numpy(), w_q=qb.numpy(), w_s=sc.numpy(),
                        acts=acts16.numpy(), q_s8=qs.numpy(), s_s8=ss.numpy(),
                        q_u8=qu.numpy(), s_u8=su.numpy(), lin=lin.numpy(),
                        q_max=np.array([rq.Q_MAX_S8, rq.Q_MAX_U8]),
                        w_e4m3=qb8.numpy(), w_e4m3_s=sc8.numpy(), q_max_e4m3=np.array([rq.Q_MAX]))
    print("done")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
