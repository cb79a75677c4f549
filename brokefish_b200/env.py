"""The engine functions the evaluator's inputs come from, on the GPU.

``movegen(boards, control) -> (mask, in_check)`` with the reference's contract
(brokefish/env/torch_impl.py:254-291): ``mask [n,32]`` int64, bit ``s`` of word ``p`` set when
the piece in slot ``p`` may legally move to square ``s``; ``in_check [n]`` bool for the side
to move.  ``step`` and ``play`` apply a move per board (torch_impl.py:412-548, 680-685),
``hash_position``, ``push_history``, ``repetition_count`` and ``terminal`` are the repetition and
game-end rules (torch_impl.py:374-401, 571-676), ``initial_boards`` is the start position (torch_impl.py:692-697)
and ``random_playouts`` plays uniform-random games to make evaluator inputs.  One thread per board
in ``libbrokefish_b200`` (C ABI ``bf_movegen``, ``bf_step``, ``bf_random_ply``, ``bf_hash`` ...); CUDA tensors
in, CUDA tensors out, on the current stream.  There is no CPU path.
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


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _check_position(boards, control):
    n = boards.shape[0]
    if boards.dim() != 2 or boards.shape[1] != 32 or boards.dtype is not torch.int16:
        raise ValueError(f"boards must be [n, 32] int16, got {tuple(boards.shape)} {boards.dtype}")
    if tuple(control.shape) != (n,) or control.dtype is not torch.int16:
        raise ValueError(f"control must be [{n}] int16, got {tuple(control.shape)} {control.dtype}")
    if not (boards.is_cuda and control.is_cuda and boards.device == control.device):
        raise ValueError("the engine kernels take CUDA tensors on one device; there is no CPU path")
    return n


def initial_boards(n: int = 1, device="cuda"):
    """``n`` copies of the start position, white to move (brokefish/env/torch_impl.py:692-697).
    Slots: white pawns a-h, knights, bishops, rooks, queen, king, then black in the same order."""
    squares = list(range(8, 16)) + [1, 6, 2, 5, 0, 7, 3, 4]
    types = [0] * 8 + [1, 1, 2, 2, 3, 3, 4, 5]
    white = [(t << 6) | s for t, s in zip(types, squares)]
    black = [(1 << 10) | (t << 6) | (s ^ 56) for t, s in zip(types, squares)]
    start = torch.tensor(white + black, dtype=torch.int16, device=device)
    return start.unsqueeze(0).expand(n, -1).clone(), torch.ones(n, dtype=torch.int16, device=device)


def step(boards, control, move, promo=None, with_moves: bool = False, hash=None):
    """Apply ``move [n]`` (``slot * 64 + target``, -1 = no move) with ``promo [n]`` (0..3 =
    N B R Q, default queen): ``(boards, control, hash, irreversible)`` as the reference's
    ``step`` returns them (brokefish/env/torch_impl.py:412-548); the third element is ``None``
    unless ``hash`` (the key of the position before the move; any non-None value asks for it) is
    given, in which case it is the new position's key, computed in the same launch.  With
    ``with_moves`` the new positions' ``(mask, in_check)`` are generated in that launch too and
    appended.  Moves are not checked for legality."""
    n = _check_position(boards, control)
    dev = boards.device
    if tuple(move.shape) != (n,) or not move.is_cuda:
        raise ValueError(f"move must be a CUDA tensor of shape [{n}]")
    mv = move.to(torch.int32).contiguous()
    pr = promo.to(device=dev, dtype=torch.int8).contiguous() if promo is not None else None
    if pr is not None and tuple(pr.shape) != (n,):
        raise ValueError(f"promo must have shape [{n}]")
    nb = torch.empty(n, 32, dtype=torch.int16, device=dev)
    nc = torch.empty(n, dtype=torch.int16, device=dev)
    irr = torch.zeros(n, dtype=torch.uint8, device=dev)
    mask = torch.zeros(n, 32, dtype=torch.int64, device=dev) if with_moves else None
    chk = torch.zeros(n, dtype=torch.uint8, device=dev) if with_moves else None
    new_hash = torch.zeros(n, dtype=torch.int64, device=dev) if hash is not None else None
    if n:
        b, c = boards.contiguous(), control.contiguous()
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _native.check(_native.lib().bf_step(dev.index or 0, _ptr(b), _ptr(c), _ptr(mv), _ptr(pr), n, _ptr(nb),
                                            _ptr(nc), _ptr(irr), _ptr(mask), _ptr(chk), _ptr(new_hash), stream),
                      "bf_step")
    out = (nb, nc, new_hash, irr.bool())
    return out + (mask, chk.bool()) if with_moves else out


def play(boards, control, move, promo=None):
    """``step`` then ``movegen`` in one launch: ``(boards, control, mask, in_check)``
    (brokefish/env/torch_impl.py:680-685)."""
    nb, nc, _, _, mask, chk = step(boards, control, move, promo, with_moves=True)
    return nb, nc, mask, chk


NONE, CHECKMATE, STALEMATE, FIFTY_MOVE, REPETITION, INSUFFICIENT = range(6)
MAX_HISTORY = 100


def hash_position(boards, control):
    """``[n] int64`` position keys (brokefish/env/torch_impl.py:374-401): pieces by (colour,
    type, square), side to move, castling rights and the file of an en passant capture that is
    really available.  The key values are this library's own; equal positions have equal keys,
    which is all the repetition rules use."""
    n = _check_position(boards, control)
    h = torch.zeros(n, dtype=torch.int64, device=boards.device)
    if n:
        stream = ctypes.c_void_p(torch.cuda.current_stream(boards.device).cuda_stream)
        _native.check(_native.lib().bf_hash(boards.device.index or 0, _ptr(boards.contiguous()),
                                            _ptr(control.contiguous()), n, _ptr(h), stream), "bf_hash")
    return h


def empty_history(n: int, device="cuda"):
    """A per-game repetition ring ``[n, 100] int64`` and its length ``[n] int64``
    (brokefish/env/torch_impl.py:571-575)."""
    return (torch.zeros(n, MAX_HISTORY, dtype=torch.int64, device=device),
            torch.zeros(n, dtype=torch.int64, device=device))


def push_history(ring, length, hash, irreversible):
    """Record the position being left (``hash`` = its key, ``irreversible`` = what ``step`` said
    about the move), as the reference's ``push_history`` (brokefish/env/torch_impl.py:578-593):
    new ``(ring, length)``; an irreversible move empties the ring."""
    n = ring.shape[0]
    if tuple(ring.shape) != (n, MAX_HISTORY) or ring.dtype is not torch.int64 or not ring.is_cuda:
        raise ValueError(f"ring must be a CUDA int64 tensor [n, {MAX_HISTORY}]")
    if tuple(length.shape) != (n,) or length.dtype is not torch.int64 or tuple(hash.shape) != (n,) \
            or hash.dtype is not torch.int64 or tuple(irreversible.shape) != (n,):
        raise ValueError("length, hash [n] int64 and irreversible [n] are needed")
    ring, length = ring.clone(), length.clone()
    irr = irreversible.to(torch.uint8).contiguous()
    if n:
        stream = ctypes.c_void_p(torch.cuda.current_stream(ring.device).cuda_stream)
        _native.check(_native.lib().bf_history_push(ring.device.index or 0, _ptr(ring), _ptr(length),
                                                    _ptr(hash.contiguous()), _ptr(irr), n, stream), "bf_history_push")
    return ring, length


def repetition_count(hash, ring, length):
    """``[n] int64``: how many times the position has occurred, the present one included
    (brokefish/env/torch_impl.py:596-603); what the network's repetition input and the threefold
    rule read."""
    n = ring.shape[0]
    count = torch.ones(n, dtype=torch.int32, device=ring.device)
    if n:
        stream = ctypes.c_void_p(torch.cuda.current_stream(ring.device).cuda_stream)
        _native.check(_native.lib().bf_repetition_count(ring.device.index or 0, _ptr(hash.contiguous()),
                                                        _ptr(ring.contiguous()), _ptr(length.contiguous()), n,
                                                        _ptr(count), stream), "bf_repetition_count")
    return count.long()


def terminal(mask, in_check, control, boards, hash=None, ring=None, length=None):
    """``(code [n] uint8, result [n] int8)``: why each game is over (1 checkmate, 2 stalemate,
    3 fifty-move rule, 5 insufficient material, 0 not over; the first that applies) and its result
    for the side to move (-1 checkmate, else 0) -- the reference's ``terminal``
    (brokefish/env/torch_impl.py:632-676).  Threefold repetition (code 4) is tested when the
    position's key and the game's ring are given, and skipped otherwise, as in the reference."""
    n = _check_position(boards, control)
    rep = None
    if hash is not None and ring is not None and length is not None:
        rep = repetition_count(hash, ring, length).to(torch.int32)
    dev = boards.device
    if tuple(mask.shape) != (n, 32) or mask.dtype is not torch.int64 or not mask.is_cuda:
        raise ValueError(f"mask must be a CUDA int64 tensor of shape [{n}, 32]")
    if tuple(in_check.shape) != (n,) or not in_check.is_cuda:
        raise ValueError(f"in_check must be a CUDA tensor of shape [{n}]")
    chk = in_check.to(torch.uint8).contiguous()
    code = torch.zeros(n, dtype=torch.uint8, device=dev)
    result = torch.zeros(n, dtype=torch.int8, device=dev)
    if n:
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _native.check(_native.lib().bf_terminal(dev.index or 0, _ptr(mask.contiguous()), _ptr(chk),
                                                _ptr(control.contiguous()), _ptr(boards.contiguous()), _ptr(rep),
                                                n, _ptr(code), _ptr(result), stream), "bf_terminal")
    return code, result


def random_playouts(n: int, seed: int, max_plies: int = 120, device="cuda"):
    """``n`` uniform-random legal games from the start position, game ``i`` stopped after
    ``plies[i]`` moves (uniform in 0..max_plies) or at its end: ``(boards, control, rep, legal,
    plies)`` with ``rep = i % 3``.  The random draws come from a CPU generator seeded with
    ``seed`` in a fixed order (plies; then per ply one fp32 uniform and one promotion type per
    game), so the positions depend on ``seed`` alone; the rules run on the GPU, one launch per
    ply."""
    dev = torch.device(device)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    plies = torch.randint(0, max_plies + 1, (n,), generator=gen)
    boards, control = initial_boards(n, dev)
    mask, _ = movegen(boards, control)
    left = plies.to(dev)
    out_b, out_c, out_m = boards.clone(), control.clone(), mask.clone()
    lib, stream = _native.lib(), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for ply in range(max_plies):
        r = torch.rand(n, generator=gen).to(dev)
        promo = torch.randint(0, 4, (n,), generator=gen).to(device=dev, dtype=torch.int8)
        if n:
            _native.check(lib.bf_random_ply(dev.index or 0, _ptr(boards), _ptr(control), _ptr(mask), _ptr(r),
                                            _ptr(promo), n, None, stream), "bf_random_ply")
        snap = left == ply + 1
        out_b[snap], out_c[snap], out_m[snap] = boards[snap], control[snap], mask[snap]
    rep = (torch.arange(n, device=dev) % 3).to(torch.uint8)
    return out_b, out_c, rep, out_m, plies
