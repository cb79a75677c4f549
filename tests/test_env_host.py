"""Host side of the engine wrappers (brokefish_b200/env.py): what can be checked without a GPU.
The kernels themselves are checked against the reference engine in tests/test_movegen.py."""
import numpy as np
import pytest
import torch

from brokefish_b200 import env


def test_start_position_is_the_reference_s(pos256):
    boards, control = env.initial_boards(3, device="cpu")
    i = int(np.argmax(pos256["plies"] == 0))
    assert boards.dtype is torch.int16 and control.dtype is torch.int16
    assert np.array_equal(boards[2].numpy(), pos256["boards"][i]) and control.tolist() == [1, 1, 1]
    words = boards[0].to(torch.int32)
    assert ((words >> 10) & 1).tolist() == [0] * 16 + [1] * 16          # white in slots 0-15, black in 16-31
    assert (((words[15] >> 6) & 7), ((words[31] >> 6) & 7)) == (5, 5)   # the kings' slots


def test_cpu_tensors_are_refused_not_evaluated():
    b, c = env.initial_boards(2, device="cpu")
    move = torch.tensor([12 * 64 + 28, -1])
    mask = torch.zeros(2, 32, dtype=torch.int64)
    for call in (lambda: env.movegen(b, c), lambda: env.step(b, c, move), lambda: env.play(b, c, move),
                 lambda: env.hash_position(b, c), lambda: env.terminal(mask, torch.zeros(2, dtype=torch.bool), c, b)):
        with pytest.raises(ValueError):
            call()
    with pytest.raises(ValueError):
        env.movegen(b.to(torch.int32), c)
    with pytest.raises(ValueError):
        env.movegen(b, c[:1])
    with pytest.raises(ValueError):
        env.push_history(torch.zeros(2, 100, dtype=torch.int64), torch.zeros(2, dtype=torch.int64),
                         torch.zeros(2, dtype=torch.int64), torch.zeros(2, dtype=torch.bool))


def test_terminal_code_names_follow_the_reference():
    assert (env.NONE, env.CHECKMATE, env.STALEMATE, env.FIFTY_MOVE, env.REPETITION, env.INSUFFICIENT) == tuple(range(6))
    assert env.MAX_HISTORY == 100
    ring, length = env.empty_history(5, device="cpu")
    assert ring.shape == (5, 100) and ring.dtype is torch.int64 and length.tolist() == [0] * 5
