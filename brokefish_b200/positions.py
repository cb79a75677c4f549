"""Seeded synthetic position batches for benchmarks and tests.

The base material is a fixture of real random-playout positions (boards, control words,
repetition counts, legal-move words) produced once with the reference's move generator.
From it this module derives batches of any size with the distributions the benchmark
configurations ask for: tiling for size, captures down to a piece count drawn uniformly from
2..32 (kings are never captured), and side to move flipped with probability 1/2 by negating the
control word.  Everything is a pure function of the seed.
"""

from __future__ import annotations

import os

import numpy as np

FIXTURE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                       "tests", "golden", "positions_4096_seed1.npz")
DEAD = np.int16(1 << 11)
KING_SLOTS = (15, 31)


def load_base(path: str = FIXTURE):
    z = np.load(path)
    return z["boards"], z["control"], z["rep"], z["legal"]


def tiled(n: int, path: str = FIXTURE):
    """``n`` positions: the fixture repeated as often as needed."""
    b, c, r, lg = load_base(path)
    reps = (n + b.shape[0] - 1) // b.shape[0]
    cut = lambda a: np.ascontiguousarray(np.concatenate([a] * reps)[:n])
    return cut(b), cut(c), cut(r), cut(lg)


def varied(n: int, seed: int, path: str = FIXTURE):
    """``n`` positions with piece counts uniform in 2..32 and side to move 50/50.

    Slots beyond the drawn count are captured (word ``0x800``, legal word 0) in a random
    order that never touches the two king slots; a position that already has fewer pieces
    keeps what it has.  Flipping the side to move negates the control word only (the
    null-move construction the reference's tests use), so a flipped position's legal words
    are no longer the mover's: they are kept as an arbitrary mask.
    """
    b, c, r, lg = tiled(n, path)
    b, c, lg = b.copy(), c.copy(), lg.copy()
    rng = np.random.default_rng(seed)
    want = rng.integers(2, 33, size=n)
    order = rng.random((n, 32))
    order[:, KING_SLOTS] = 2.0                      # kings sort last: never captured
    alive = (b.view(np.uint16) >> 11 & 1) == 0
    order[~alive] = -1.0                            # already dead: first in line, no effect
    rank = order.argsort(axis=1).argsort(axis=1)    # 0 = first to be captured
    n_alive = alive.sum(axis=1)
    kill = rank < (32 - np.maximum(want, 2))[:, None]
    kill &= alive & (n_alive[:, None] > want[:, None])
    kill[:, KING_SLOTS] = False
    b[kill] = DEAD
    lg[kill] = 0
    flip = rng.random(n) < 0.5
    c[flip] = -c[flip]
    return b, c, r, lg
