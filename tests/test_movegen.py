"""The move generator (brokefish_b200/csrc/bf_movegen.cuh, C ABI bf_movegen) against the
reference engine's own answers, committed under tests/golden/ by make_golden.py: the legal words
of 4352 random-playout positions (0-120 plies: captures, castling, en passant, promotions,
checks, mates) and of 17 hand-picked positions, and the check flags.  Bit-exact."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN


@pytest.fixture(scope="module")
def gold():
    z = np.load(os.path.join(GOLDEN, "ref_movegen.npz"))
    return {k: z[k] for k in z.files}


def popcount(words):
    return np.array([bin(int(w)).count("1") for w in np.asarray(words).reshape(-1)]).reshape(np.asarray(words).shape)


def test_golden_answers_are_the_known_move_counts(gold):
    """The fixture itself: 218 moves in the maximum-mobility position, 20 from the start
    position, mate and stalemate have none, and the hand-picked cases say what they should."""
    counts = popcount(gold["fen_legal"]).sum(-1)
    fens = list(gold["fens"])
    by = {f.split()[0] + " " + f.split()[1]: int(c) for f, c in zip(fens, counts)}
    assert by["R6R/3Q4/1Q4Q1/4Q3/2Q4Q/Q4Q2/pp1Q4/kBNN1KB1 w"] == 218
    assert by["rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w"] == 20
    assert by["7k/5Q2/6K1/8/8/8/8/8 b"] == 0 and by["7k/6Q1/6K1/8/8/8/8/8 b"] == 0
    chk = dict(zip(fens, gold["fen_in_check"]))
    assert not chk["7k/5Q2/6K1/8/8/8/8/8 b - - 0 1"] and chk["7k/6Q1/6K1/8/8/8/8/8 b - - 0 1"]
    # white castles both ways from the bare position: the king's word has bits 2 and 6 set
    i = fens.index("r3k2r/pppppppp/8/8/8/8/PPPPPPPP/R3K2R w KQkq - 0 1")
    king = gold["fen_legal"][i][15]
    assert (int(king) >> 6) & 1 and (int(king) >> 2) & 1
    # rook on g2 covers g1 and f1... the short castle is gone, the long one stays
    i = fens.index("r3k2r/8/8/8/8/8/6r1/R3K2R w KQkq - 0 1")
    king = gold["fen_legal"][i][15]
    assert not (int(king) >> 6) & 1 and (int(king) >> 2) & 1
    # the en passant capture that would expose the king is not there
    i = fens.index("8/8/8/8/k2Pp2Q/8/8/4K3 b - d3 0 1")
    assert all(not (int(w) >> 19) & 1 for w in gold["fen_legal"][i])


@pytest.mark.gpu
def test_movegen_equals_the_reference_engine(gold, pos256, pos4096):
    from brokefish_b200.env import movegen
    cases = [(gold["fen_boards"], gold["fen_control"], gold["fen_legal"], gold["fen_in_check"]),
             (pos256["boards"], pos256["control"], pos256["legal"], gold["in_check_256"]),
             (pos4096["boards"], pos4096["control"], pos4096["legal"], gold["in_check_4096"])]
    for boards, control, legal, in_check in cases:
        b = torch.from_numpy(np.ascontiguousarray(boards)).cuda()
        c = torch.from_numpy(np.ascontiguousarray(control)).cuda()
        mask, chk = movegen(b, c)
        got = mask.cpu().numpy().view(np.uint64)
        bad = np.argwhere(got != legal)
        assert bad.size == 0, (bad[:5], [hex(int(got[tuple(i)])) for i in bad[:3]], [hex(int(legal[tuple(i)])) for i in bad[:3]])
        assert np.array_equal(chk.cpu().numpy(), in_check.astype(bool))
    assert in_check.any() and (popcount(pos256["legal"]).sum(-1) == 0).any()      # checks and mates occur
    # an empty batch and wrong inputs
    m, k = movegen(b[:0], c[:0])
    assert m.shape == (0, 32) and k.shape == (0,)
    with pytest.raises(ValueError):
        movegen(b.cpu(), c.cpu())


@pytest.mark.gpu
def test_fused_expansion_generates_its_own_moves(pos4096):
    """`forward_priors` without legality words: the kernel's expansion warp generates them (lane
    = slot) and the result equals the call that was given the engine's words."""
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import BrokefishNet, seeded_state
    net = BrokefishNet().eval()
    net.load_state_dict(seeded_state(seed=0, std=None, perturb_norms=True))
    n = 1111
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a[:n])).cuda()
    boards, control, rep = t(pos4096["boards"]), t(pos4096["control"]), t(pos4096["rep"])
    legal = torch.from_numpy(pos4096["legal"][:n].view(np.int64).copy()).cuda()
    enc = encoder_impl("cuda")(net, int8=True)
    for cap in (96, 12):
        want = [x.clone() for x in enc.forward_priors(boards, control, rep, legal, cap)]
        got = [x.clone() for x in enc.forward_priors(boards, control, rep, None, cap)]
        assert torch.equal(got[0].view(torch.int16), want[0].view(torch.int16))
        assert torch.equal(got[1], want[1]) and torch.equal(got[2], want[2]) and torch.equal(got[3], want[3])
    enc.check_status()
    with pytest.raises(ValueError):
        enc.forward_priors(boards, control, rep, None, 96, logits=True)
    enc.close()


@pytest.fixture(scope="module")
def gold_step():
    z = np.load(os.path.join(GOLDEN, "ref_step.npz"))
    return {k: z[k] for k in z.files}


def test_step_fixture_covers_the_special_moves(gold_step, pos4096):
    """The reference's answers themselves: castling moves the rook too, en passant removes the
    pawn beside the target, promotions take the asked type, the null move changes nothing."""
    g = gold_step
    cases = list(g["cases"])
    i = cases.index("r3k2r/pppppppp/8/8/8/8/PPPPPPPP/R3K2R w KQkq - 0 1 e1g1")
    assert (g["case_boards"][i][15] & 63) == 6 and (g["case_boards"][i][13] & 63) == 5
    i = cases.index("rnbqkbnr/ppp1p1pp/8/3pPp2/8/8/PPPP1PPP/RNBQKBNR w KQkq f6 0 3 e5f6")
    assert (g["case_boards"][i] == 0x800).sum() == (g["case_boards_in"][i] == 0x800).sum() + 1
    types = [(int(g["case_boards"][i][g["case_move"][i] >> 6]) >> 6) & 7
             for i, c in enumerate(cases) if c.endswith("w - - 0 1 c7c8")]
    assert types == [4, 1, 2]
    null = g["move"] < 0
    assert null.sum() > 200 and np.array_equal(g["boards"][null], pos4096["boards"][null])
    assert not g["irreversible"][null].any() and 0.2 < g["irreversible"].mean() < 0.5
    assert not g["case_irreversible"][cases.index("rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1 g1f3")]


@pytest.mark.gpu
def test_step_and_play_equal_the_reference_engine(gold_step, pos4096):
    from brokefish_b200.env import play, step
    g = gold_step
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sets = [(pos4096["boards"], pos4096["control"], g["move"], g["promo"], g["boards"], g["control"],
             g["irreversible"], g["legal"], g["in_check"]),
            (g["case_boards_in"], g["case_control_in"], g["case_move"], g["case_promo"], g["case_boards"],
             g["case_control"], g["case_irreversible"], g["case_legal"], g["case_in_check"])]
    for b0, c0, mv, pr, b1, c1, irr, legal, chk in sets:
        nb, nc, h, ir = step(cu(b0), cu(c0), cu(mv), cu(pr))
        assert h is None
        assert np.array_equal(nb.cpu().numpy(), b1) and np.array_equal(nc.cpu().numpy(), c1)
        assert np.array_equal(ir.cpu().numpy(), irr.astype(bool))
        pb, pc, pm, pk = play(cu(b0), cu(c0), cu(mv).long(), cu(pr))
        assert torch.equal(pb, nb) and torch.equal(pc, nc)
        assert np.array_equal(pm.cpu().numpy().view(np.uint64), legal)
        assert np.array_equal(pk.cpu().numpy(), chk.astype(bool))
    # the default promotion is the queen (the hand-picked set asks for 3 where it wants the default)
    q = g["case_promo"] == 3
    nb2, _, _, _ = step(cu(g["case_boards_in"][q]), cu(g["case_control_in"][q]), cu(g["case_move"][q]))
    assert np.array_equal(nb2.cpu().numpy(), g["case_boards"][q])
    with pytest.raises(ValueError):
        step(cu(b0), cu(c0), cu(mv)[:3])


@pytest.mark.gpu
def test_random_playouts_on_the_gpu_reproduce_the_reference_made_position_files(pos256, pos4096):
    """Up to 120 plies of movegen -> pick -> step chained on the device, with the random draws of
    the fixture script: the positions and their legal words come out equal to the files the
    reference engine wrote, and the start position is the reference's."""
    from brokefish_b200.env import initial_boards, random_playouts
    for pos, n, seed in ((pos256, 256, 0), (pos4096, 4096, 1)):
        b, c, rep, legal, plies = random_playouts(n, seed)
        assert np.array_equal(plies.numpy(), pos["plies"])
        assert np.array_equal(b.cpu().numpy(), pos["boards"])
        assert np.array_equal(c.cpu().numpy(), pos["control"])
        assert np.array_equal(rep.cpu().numpy(), pos["rep"])
        assert np.array_equal(legal.cpu().numpy().view(np.uint64), pos["legal"])
    i = int(np.argmax(pos256["plies"] == 0))
    sb, sc = initial_boards(2)
    assert np.array_equal(sb[1].cpu().numpy(), pos256["boards"][i]) and int(sc[0]) == 1


@pytest.mark.gpu
def test_boards_that_do_not_keep_the_colours_apart_by_slot():
    """512 positions with their thirty non-king slots permuted at random: the stand-alone kernels
    (which normally walk only the mover's sixteen slots) and the evaluator's in-kernel generator
    give the reference engine's legal words, check flags, moved boards and next legal words."""
    from brokefish_b200.env import movegen, play
    z = np.load(os.path.join(GOLDEN, "ref_shuffled.npz"))
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    b, c = cu(z["boards"]), cu(z["control"])
    mask, chk = movegen(b, c)
    assert np.array_equal(mask.cpu().numpy().view(np.uint64), z["legal"])
    assert np.array_equal(chk.cpu().numpy(), z["in_check"].astype(bool))
    nb, nc, nm, nk = play(b, c, cu(z["move"]), cu(z["promo"]))
    assert np.array_equal(nb.cpu().numpy(), z["next_boards"]) and np.array_equal(nc.cpu().numpy(), z["next_control"])
    assert np.array_equal(nm.cpu().numpy().view(np.uint64), z["next_legal"])
    assert np.array_equal(nk.cpu().numpy(), z["next_in_check"].astype(bool))
    # the warp-per-board form inside the evaluator: generated moves == given moves
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import BrokefishNet, seeded_state
    net = BrokefishNet().eval()
    net.load_state_dict(seeded_state(seed=0, std=0.02))
    enc = encoder_impl("cuda")(net, int8=True)
    rep = torch.zeros(b.shape[0], dtype=torch.uint8, device="cuda")
    legal = torch.from_numpy(z["legal"].view(np.int64).copy()).cuda()
    want = [x.clone() for x in enc.forward_priors(b, c, rep, legal, 96)]
    got = enc.forward_priors(b, c, rep, None, 96)
    assert torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])
    assert torch.equal(got[0].view(torch.int16), want[0].view(torch.int16))
    enc.close()


@pytest.fixture(scope="module")
def gold_terminal():
    z = np.load(os.path.join(GOLDEN, "ref_terminal.npz"))
    return {k: z[k] for k in z.files}


def test_terminal_fixture_says_what_the_rules_say(gold_terminal):
    g = gold_terminal
    by = dict(zip(g["fens"], zip(g["fen_code"], g["fen_result"])))
    assert by["8/8/8/4k3/8/8/8/4K3 w - - 0 1"] == (5, 0) and by["8/8/8/4k3/8/8/8/3NKN2 w - - 0 1"] == (0, 0)
    assert by["8/8/8/4k3/8/8/8/2B1KB2 w - - 0 1"] == (0, 0) and by["8/8/8/4k3/8/8/2B5/4KB2 w - - 0 1"] == (5, 0)
    assert by["8/8/8/4k3/8/8/4P3/4K3 w - - 100 80"] == (3, 0) and by["8/8/8/4k3/8/8/4P3/4K3 b - - 99 80"] == (0, 0)
    assert by["7k/6Q1/6K1/8/8/8/8/8 b - - 100 70"] == (1, -1) and by["7k/5Q2/6K1/8/8/8/8/8 b - - 100 70"] == (2, 0)
    assert (g["code_4096"] == 1).sum() == 53 and (g["result_4096"] == -1).sum() == 53


@pytest.mark.gpu
def test_terminal_codes_equal_the_reference_engine(gold_terminal, pos256, pos4096):
    """`env.terminal` on this library's own legal words and check flags: the reference's codes
    and results on the hand-made positions and on both playout sets."""
    from brokefish_b200.env import movegen, terminal
    g = gold_terminal
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for boards, control, code, result in ((g["fen_boards"], g["fen_control"], g["fen_code"], g["fen_result"]),
                                          (pos256["boards"], pos256["control"], g["code_256"], g["result_256"]),
                                          (pos4096["boards"], pos4096["control"], g["code_4096"], g["result_4096"])):
        b, c = cu(boards), cu(control)
        mask, chk = movegen(b, c)
        got_code, got_result = terminal(mask, chk, c, b)
        assert got_code.dtype is torch.uint8 and got_result.dtype is torch.int8
        assert np.array_equal(got_code.cpu().numpy(), code) and np.array_equal(got_result.cpu().numpy(), result)
    e = terminal(mask[:0], chk[:0], c[:0], b[:0])
    assert e[0].shape == (0,)
    with pytest.raises(ValueError):
        terminal(mask[:5], chk, c, b)


@pytest.mark.gpu
def test_position_keys_repetition_ring_and_threefold_rule():
    """192 games replayed move by move (half from the start position, half from three- and
    four-piece positions where random play repeats itself): after every ply the repetition count
    of the position reached and the terminal code with the history given equal the reference
    engine's (68 second and 19 third occurrences among 15,060 moves).  The keys themselves are
    this library's own; what is checked is everything the reference derives from them."""
    from brokefish_b200 import env
    z = np.load(os.path.join(GOLDEN, "ref_history.npz"))
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    boards, control = cu(z["boards"]), cu(z["control"])
    n = boards.shape[0]
    h = env.hash_position(boards, control)
    ring, length = env.empty_history(n)
    assert (z["counts"] >= 2).sum() > 50 and (z["codes"] == 4).any()
    for ply in range(z["moves"].shape[0]):
        move, promo = cu(z["moves"][ply]), cu(z["promos"][ply])
        nb, nc, nh, irr, mask, chk = env.step(boards, control, move, promo, with_moves=True, hash=h)
        played = move >= 0
        r2, l2 = env.push_history(ring, length, h, irr)
        ring = torch.where(played[:, None], r2, ring)
        length = torch.where(played, l2, length)
        boards, control, h = nb, nc, nh
        assert torch.equal(h, env.hash_position(boards, control))        # the fused key is the stand-alone one
        count = env.repetition_count(h, ring, length)
        code, result = env.terminal(mask, chk, control, boards, h, ring, length)
        assert np.array_equal(count.clamp(max=255).cpu().numpy().astype(np.uint8), z["counts"][ply]), ply
        assert np.array_equal(code.cpu().numpy(), z["codes"][ply]), ply
        assert ((result == -1) == (code == 1)).all()
    # pairs of positions: equal keys exactly where the reference's are (an en passant flag counts
    # only when the capture is available and legal; rights and side to move always count; the
    # fifty-move counter never does)
    same = env.hash_position(cu(z["pair_a"]), cu(z["pair_a_control"])) == \
        env.hash_position(cu(z["pair_b"]), cu(z["pair_b_control"]))
    assert np.array_equal(same.cpu().numpy(), z["pair_same"]), list(zip(z["pairs"], same.cpu().numpy()))
    assert list(z["pair_same"]) == [False, False, True, True, False, False, True]
    # distinct positions get distinct keys on the playout sets (no collision among 4096)
    p = np.load(os.path.join(GOLDEN, "positions_4096_seed1.npz"))
    keys = env.hash_position(cu(p["boards"]), cu(p["control"])).cpu().numpy()
    packed = np.concatenate([p["boards"].view(np.uint16).astype(np.int64), p["control"][:, None].astype(np.int64)], axis=1)
    assert len(np.unique(keys)) <= len(np.unique(packed, axis=0))
    assert len(np.unique(keys)) >= 0.9 * len(np.unique(packed, axis=0))
