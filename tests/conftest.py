import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")

WEIGHT_SETS = {"A": dict(seed=0, std=0.02, perturb_norms=False),
               "B": dict(seed=0, std=None, perturb_norms=True)}
#: Per-layer input re-injection at both norms with nonzero coefficients.
REINJECT_SET = dict(seed=7, std=None, perturb_norms=True, reinject="both")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_positions(n: int, seed: int):
    z = np.load(os.path.join(GOLDEN, f"positions_{n}_seed{seed}.npz"))
    return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def pos256():
    return load_positions(256, 0)


@pytest.fixture(scope="session")
def pos4096():
    return load_positions(4096, 1)


@pytest.fixture(scope="session")
def states():
    from brokefish_b200.nn.model import seeded_state
    return {k: seeded_state(**kw) for k, kw in WEIGHT_SETS.items()}


@pytest.fixture(scope="session")
def oracle_weights(states):
    from oracle import int8_encoder as O
    return {k: O.prepare({n: t.numpy() for n, t in s.items()}) for k, s in states.items()}


@pytest.fixture(scope="session")
def nets(states):
    """The two weight sets as callable torch networks (the product's weight container plus the
    test oracle's forward path)."""
    from oracle.torch_net import TorchNet
    out = {}
    for k, s in states.items():
        net = TorchNet().eval()
        net.load_state_dict(s)
        out[k] = net
    return out
