"""The network's weights on the host: a container with the reference's parameter tree.

``BrokefishNet`` here holds the fp32 master weights under the constructor arguments,
attribute names and ``state_dict`` keys of the reference's ``BrokefishNet``
(brokefish/nn/model.py:268-361), so a checkpoint written by the reference loads here
unchanged and one written here loads there.  It is what
:class:`brokefish_b200.nn.cuda_impl.FusedEncoder` packs its blob from when no reference
checkout is at hand (the reference's own module is accepted just the same).  It has no
``forward``: evaluating positions is the sm_100a kernel's job, and the plain PyTorch
evaluation of these weights, which only the tests and the CPU baseline need, lives with the
test oracles.

Architecture (brokefish/nn/model.py:38-47): 32 piece tokens, width 256, 8 pre-norm
encoder layers with 8 heads of 32 and a 1024-wide ReLU FFN, a final LayerNorm, and
three bias-free heads (64 policy logits and 4 promotion logits per token, value from
the side-to-move king's token).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

D_MODEL, N_LAYERS, N_HEADS, D_FF, T = 256, 8, 8, 1024, 32
N_SQUARE, N_TYPE_SPECIAL, N_COLOR_TURN, N_CLOCK, N_REP = 64, 12, 4, 101, 3
KING_SLOT_WHITE, KING_SLOT_BLACK = 15, 31
N_POLICY, N_PROMO = 64, 4
VALUE_CLASSES = (1, 3)
VALUE_HEADS = ("king", "pooled", "prenorm")
VALUE_MODE_ID = {"pooled": 1, "prenorm": 2}
REINJECT_MODES = ("none", "ln1", "both")
REINJECT_MODE_ID = {"ln1": 1, "both": 2}
N_SOURCES = 5

EMB_TABLES = ("emb_square", "emb_type_special", "emb_color_turn", "emb_clock", "emb_rep")


def n_value_of(state: dict) -> int:
    return int(state["value.weight"].shape[0])


def value_head_of(state: dict) -> str:
    if "value_mode" not in state:
        return "king"
    got = int(state["value_mode"])
    for name, i in VALUE_MODE_ID.items():
        if i == got:
            return name
    raise ValueError(f"unknown value_mode {got}")


def reinject_of(state: dict) -> str:
    """Which per-layer input re-injection a ``state_dict`` was written with; absence of the
    marker means none (brokefish/nn/model.py:210-225)."""
    if "reinject_mode" not in state:
        return "none"
    got = int(state["reinject_mode"])
    for name, i in REINJECT_MODE_ID.items():
        if i == got:
            return name
    raise ValueError(f"unknown reinject_mode {got}")


def net_for_state(state: dict, **kw) -> "BrokefishNet":
    """An empty network shaped to hold ``state`` (brokefish/nn/model.py:243-248)."""
    if "rule_features_mode" in state:
        raise NotImplementedError("rule-feature networks are not supported by this build")
    return BrokefishNet(n_value=n_value_of(state), value_head=value_head_of(state),
                        reinject=reinject_of(state), **kw)


class BrokefishNet(nn.Module):
    """Weight container of the piece-token transformer; same parameters and key names as the
    reference's module, no forward path."""

    def __init__(self, d_model: int = D_MODEL, n_layers: int = N_LAYERS,
                 n_heads: int = N_HEADS, d_ff: int = D_FF, eps: float = 1e-5,
                 n_value: int = 1, value_head: str = "king", reinject: str = "none",
                 rule_features: bool = False):
        super().__init__()
        if n_value not in VALUE_CLASSES:
            raise ValueError(f"n_value must be one of {VALUE_CLASSES}, got {n_value}")
        if value_head not in VALUE_HEADS:
            raise ValueError(f"value_head must be one of {VALUE_HEADS}, got {value_head!r}")
        if reinject not in REINJECT_MODES:
            raise ValueError(f"reinject must be one of {REINJECT_MODES}, got {reinject!r}")
        if rule_features:
            raise NotImplementedError("rule-derived inputs are a torch-only prototype of the "
                                      "reference and are not built here")
        self.d_model, self.n_layers, self.n_value = d_model, n_layers, n_value
        self.value_head, self.reinject, self.rule_features = value_head, reinject, False
        self.n_sites = 0 if reinject == "none" else n_layers * (2 if reinject == "both" else 1)

        self.emb_square = nn.Embedding(N_SQUARE, d_model)
        self.emb_type_special = nn.Embedding(N_TYPE_SPECIAL, d_model)
        self.emb_color_turn = nn.Embedding(N_COLOR_TURN, d_model)
        self.emb_clock = nn.Embedding(N_CLOCK, d_model)
        self.emb_rep = nn.Embedding(N_REP, d_model)
        layer = nn.TransformerEncoderLayer(
            d_model=d_model, nhead=n_heads, dim_feedforward=d_ff, batch_first=True,
            norm_first=True, dropout=0.0, layer_norm_eps=eps)
        self.encoder = nn.TransformerEncoder(layer, num_layers=n_layers, norm=None,
                                             enable_nested_tensor=False)
        self.norm_f = nn.LayerNorm(d_model, eps=eps)
        self.policy = nn.Linear(d_model, N_POLICY, bias=False)
        self.promo = nn.Linear(d_model, N_PROMO, bias=False)
        self.value = nn.Linear(d_model, n_value, bias=False)
        if value_head in VALUE_MODE_ID:
            self.register_buffer("value_mode",
                                 torch.tensor(VALUE_MODE_ID[value_head], dtype=torch.int64))
        if reinject in REINJECT_MODE_ID:
            # zero-initialised: an untrained re-injecting network is the plain one exactly
            self.reinject_c = nn.Parameter(torch.zeros(self.n_sites, N_SOURCES))
            self.register_buffer("reinject_mode",
                                 torch.tensor(REINJECT_MODE_ID[reinject], dtype=torch.int64))
        std = d_model ** -0.5
        for mod in (self.emb_square, self.emb_type_special, self.emb_color_turn,
                    self.emb_clock, self.emb_rep, self.policy, self.promo, self.value):
            nn.init.normal_(mod.weight, mean=0.0, std=std)

    @property
    def value_absolute(self) -> bool:
        """Pooled and prenorm value heads score the position in White's frame."""
        return self.value_head in ("pooled", "prenorm")


def seeded_state(seed: int = 0, std: Optional[float] = 0.02, perturb_norms: bool = False,
                 n_value: int = 1, value_head: str = "king", reinject: str = "none",
                 reinject_scale: float = 0.5) -> dict:
    """A reproducible ``state_dict``, independent of module construction order.

    Keys are visited in sorted order and each tensor is drawn from its own
    ``torch.Generator`` seeded with ``seed`` and the key's position, so the same call
    gives the same bytes on any machine with the same torch build.

    ``std`` set: every tensor with two or more dimensions is N(0, std); LayerNorm
    gammas are 1 and every bias / beta is 0.  ``std=None``: matrices are
    N(0, 1/16) (tables and heads) or N(0, 1/sqrt(fan_in)) (projections).
    ``perturb_norms``: LayerNorm gamma/beta and all biases get N(1, .1) / N(0, .1), so
    the LayerNorm folds and the bias paths carry signal.  ``reinject``: the coefficient
    matrix is N(0, reinject_scale).
    """
    net = BrokefishNet(n_value=n_value, value_head=value_head, reinject=reinject)
    state = net.state_dict()
    out = {}
    for i, key in enumerate(sorted(state)):
        t = state[key]
        if not t.is_floating_point():
            out[key] = t.clone()
            continue
        g = torch.Generator(device="cpu").manual_seed(seed * 100003 + i)
        if key == "reinject_c":
            out[key] = reinject_scale * torch.randn(t.shape, generator=g)
        elif t.dim() >= 2:
            s = std if std is not None else (
                1.0 / 16 if (key.startswith("emb_") or key.split(".")[0] in
                             ("policy", "promo", "value")) else t.shape[-1] ** -0.5)
            out[key] = torch.randn(t.shape, generator=g) * s
        elif perturb_norms:
            base = 1.0 if key.endswith("weight") else 0.0
            out[key] = base + 0.1 * torch.randn(t.shape, generator=g)
        else:
            # construction-time values of Linear biases come from the global RNG, so
            # they are replaced by fixed ones: LayerNorm gamma 1, everything else 0
            is_gamma = "norm" in key and key.endswith("weight")
            out[key] = torch.ones_like(t) if is_gamma else torch.zeros_like(t)
    return out
