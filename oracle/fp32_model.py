"""TEST / BASELINE INFRASTRUCTURE, not product code: the reference's fp32 PyTorch
evaluator restated with functional torch ops, for timing on host cores.

The reference's CPU evaluator is its ``BrokefishNet`` called under ``torch.no_grad()``
(brokefish/search/torch_impl.py:186-197 with ``impl=None``; brokefish/nn/model.py:621-645).
This module computes the same function from a ``state_dict`` without ``nn.Module``
plumbing: embedding sum (model.py:383-397), eight pre-norm blocks with key-padding-masked
attention and a ReLU FFN (``nn.TransformerEncoderLayer(norm_first=True)``), final
LayerNorm, three bias-free heads, king-row value through ``tanh`` (model.py:551-617).
``tests/test_oracle_golden.py`` pins it to the reference's committed fp32 outputs.
Only ``tests/`` and ``bench.py`` (``cpu_baseline`` and ``--impl reference``) import it.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

H, DH, T = 8, 32, 32


@torch.no_grad()
def forward(state: dict, boards: torch.Tensor, control: torch.Tensor, rep: torch.Tensor):
    """``(policy [n,32,64], promo [n,32,4], value [n])`` in fp32 on the tensors' device."""
    w = boards.long() & 0xFFFF
    stm = (control < 0).long()
    alive = ((w >> 11) & 1) == 0
    per_board = state["emb_clock.weight"][(control.abs().long() - 1).clamp(0, 100)] \
        + state["emb_rep.weight"][rep.long().clamp(0, 2)]
    x = state["emb_square.weight"][w & 63]
    x = x + state["emb_type_special.weight"][((w >> 6) & 7) * 2 + ((w >> 9) & 1)]
    x = x + state["emb_color_turn.weight"][((w >> 10) & 1) * 2 + stm[:, None]]
    x = x + per_board[:, None, :]
    n = x.shape[0]
    bias = torch.zeros(n, 1, 1, T, dtype=x.dtype, device=x.device)
    bias.masked_fill_(~alive[:, None, None, :], float("-inf"))
    n_layers = 1 + max(int(k.split(".")[2]) for k in state if k.startswith("encoder.layers."))
    for i in range(n_layers):
        p = f"encoder.layers.{i}."
        h = F.layer_norm(x, (256,), state[p + "norm1.weight"], state[p + "norm1.bias"], 1e-5)
        qkv = F.linear(h, state[p + "self_attn.in_proj_weight"], state[p + "self_attn.in_proj_bias"])
        q, k, v = (t.reshape(n, T, H, DH).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        o = o.transpose(1, 2).reshape(n, T, 256)
        x = x + F.linear(o, state[p + "self_attn.out_proj.weight"], state[p + "self_attn.out_proj.bias"])
        h = F.layer_norm(x, (256,), state[p + "norm2.weight"], state[p + "norm2.bias"], 1e-5)
        h = F.relu(F.linear(h, state[p + "linear1.weight"], state[p + "linear1.bias"]))
        x = x + F.linear(h, state[p + "linear2.weight"], state[p + "linear2.bias"])
    hn = F.layer_norm(x, (256,), state["norm_f.weight"], state["norm_f.bias"], 1e-5)
    king = torch.where(control < 0, 31, 15).long()
    raw = F.linear(hn[torch.arange(n), king], state["value.weight"])
    return (F.linear(hn, state["policy.weight"]), F.linear(hn, state["promo.weight"]),
            torch.tanh(raw).squeeze(-1))
