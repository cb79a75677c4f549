"""TEST INFRASTRUCTURE, not product code: the plain PyTorch evaluation of a network's weights.

``TorchNet`` is the product's weight container (``brokefish_b200.nn.model.BrokefishNet``)
plus a ``forward`` that computes what the reference's module computes
(brokefish/nn/model.py:365-397 embedding, 481-538 encoder with per-layer input re-injection,
551-617 heads, 621-645 forward), written as one functional pass over the container's
parameters.  The tests use it wherever the reference would call its own network on the CPU:
as the fp32 yardstick of the prior-space validator, as the fp16 embedding check, and as the
torch side of the host-API tests.  ``tests/test_oracle_golden.py`` and
``tests/test_host_api.py`` pin it to outputs of the reference's module committed under
``tests/golden/``.  Only ``tests/`` may import this module.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from brokefish_b200.nn.model import BrokefishNet

T, H = 32, 8


def token_indices(boards: torch.Tensor, control: torch.Tensor, rep: torch.Tensor):
    """Row numbers into the five embedding tables for every token, the per-slot colour row that
    re-injection uses, and the alive mask.  Piece word: bit 11 captured, bit 10 colour, bit 9
    special, bits 6-8 type, bits 0-5 square (brokefish/nn/model.py:251-265)."""
    w = boards.long() & 0xFFFF
    black_to_move = (control < 0).long()[:, None]
    slot_is_black = (torch.arange(T, device=boards.device) >= T // 2).long()[None, :]
    rows = {
        "square": w & 63,
        "type_special": ((w >> 6) & 7) * 2 + ((w >> 9) & 1),
        "color_turn": ((w >> 10) & 1) * 2 + black_to_move,
        "clock": (control.abs().long() - 1).clamp(0, 100),
        "rep": rep.long().clamp(0, 2),
        "slot_color_turn": slot_is_black * 2 + black_to_move,
    }
    return rows, ((w >> 11) & 1) == 0


class TorchNet(BrokefishNet):
    """The weight container with the reference network's forward path."""

    def embed(self, boards, control, rep):
        """``((square + type_special) + color_turn) + (clock + rep)`` in the parameters' dtype,
        and the alive mask."""
        rows, alive = token_indices(boards, control, rep)
        board_part = self.emb_clock.weight[rows["clock"]] + self.emb_rep.weight[rows["rep"]]
        x = self.emb_square.weight[rows["square"]] + self.emb_type_special.weight[rows["type_special"]]
        x = x + self.emb_color_turn.weight[rows["color_turn"]]
        return x + board_part[:, None, :], alive

    def _injection(self, rows, coef):
        """``sum_k coef[k] * table_k[row_k]`` of one re-injection site; the colour table is read by
        slot colour, not by the decoded word."""
        per_token = (F.embedding(rows["square"], coef[0] * self.emb_square.weight)
                     + F.embedding(rows["type_special"], coef[1] * self.emb_type_special.weight)
                     + F.embedding(rows["slot_color_turn"], coef[2] * self.emb_color_turn.weight))
        per_board = (F.embedding(rows["clock"], coef[3] * self.emb_clock.weight)
                     + F.embedding(rows["rep"], coef[4] * self.emb_rep.weight))
        return per_token + per_board[:, None, :]

    def _block(self, layer, x, dead_key_bias, inject1=None, inject2=None):
        """One pre-norm encoder block; a norm sees ``x + injection`` while the residual stream
        stays ``x``."""
        n = x.shape[0]
        d = x.shape[-1]
        attn = layer.self_attn
        h = layer.norm1(x if inject1 is None else x + inject1)
        q, k, v = (t.reshape(n, T, H, d // H).transpose(1, 2)
                   for t in F.linear(h, attn.in_proj_weight, attn.in_proj_bias).chunk(3, dim=-1))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=dead_key_bias)
        x = x + attn.out_proj(o.transpose(1, 2).reshape(n, T, d))
        h = layer.norm2(x if inject2 is None else x + inject2)
        return x + layer.linear2(F.relu(layer.linear1(h)))

    def forward(self, boards, control, rep, with_logits: bool = False):
        rows, alive = token_indices(boards, control, rep)
        x, _ = self.embed(boards, control, rep)
        dead_key_bias = torch.zeros(x.shape[0], 1, 1, T, dtype=x.dtype, device=x.device)
        dead_key_bias.masked_fill_(~alive[:, None, None, :], float("-inf"))
        both = self.reinject == "both"
        for i, layer in enumerate(self.encoder.layers):
            inj1 = inj2 = None
            if self.reinject != "none":
                site = 2 * i if both else i
                inj1 = self._injection(rows, self.reinject_c[site])
                if both:
                    inj2 = self._injection(rows, self.reinject_c[site + 1])
            x = self._block(layer, x, dead_key_bias, inj1, inj2)
        tokens = self.norm_f(x)
        live = alive.unsqueeze(-1).to(x.dtype)
        n_live = live.sum(1).clamp(min=1)
        if self.value_head == "prenorm":
            summary = self.norm_f((x * live).sum(1) / n_live)
        elif self.value_head == "pooled":
            summary = (tokens * live).sum(1) / n_live
        else:
            mover_king = torch.where(control < 0, 31, 15).long()
            summary = tokens[torch.arange(tokens.shape[0], device=tokens.device), mover_king]
        raw = self.value(summary).float()
        if self.n_value == 1:
            value = torch.tanh(raw).squeeze(-1)
        else:
            p = torch.softmax(raw, dim=-1)
            value = p[..., 2] - p[..., 0]
        if self.value_absolute:
            value = torch.where(control > 0, value, -value)
        if with_logits:
            return self.policy(tokens), self.promo(tokens), value, raw
        return self.policy(tokens), self.promo(tokens), value


def net_for_state(state: dict) -> TorchNet:
    """An empty ``TorchNet`` shaped to hold ``state``."""
    from brokefish_b200.nn import model
    return TorchNet(n_value=model.n_value_of(state), value_head=model.value_head_of(state),
                    reinject=model.reinject_of(state))
