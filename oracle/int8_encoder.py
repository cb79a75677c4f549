"""TEST INFRASTRUCTURE, not product code: a CPU restatement (numpy) of the reference's
int8 evaluator, boards in, logits out.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl
reference`` legs of ``bench.py`` may import this module.  Nothing under
``brokefish_b200/`` does.

What it restates, step by step, with the reference lines each step follows (paths are
the reference project's own):

* weight folding and quantisation ............ brokefish/nn/cuda_impl.py:194-227, 339-371;
                                                brokefish/nn/quant.py:263-278
* embedding sum, fp16, normative grouping ..... csrc/encoder.cu:817-889; nn/model.py:383-397
* LayerNorm (one-pass fp32 stats, fp16 out) ... csrc/encoder.cu:584-616
* per-row s8/u8 activation quantiser .......... csrc/int8_gemm.cuh:159-199
* s8/u8 x s8 GEMM, exact s32, one descale ..... csrc/int8_gemm.cuh:276-297
* bias / ReLU / residual in fp16 .............. csrc/encoder.cu:631-686, 1482-1489
* attention, dead keys masked, fp32 softmax ... csrc/encoder.cu:715-797
* layer order and the ff2 fp16 running total .. csrc/encoder.cu:1319-1557
* final norm (affine), fp16 heads, value ...... csrc/encoder.cu:894-1079; nn/model.py:551-617

Parity status: PINNED.  ``tests/test_oracle_golden.py`` checks this file against outputs
of the reference's own Python (its fp32 network, its int8 emulation, its scheme
functions, its embedding) generated in a container that holds the reference and
committed under ``tests/golden/`` with the generating script.

Where the reference's GPU arithmetic cannot be reproduced bit for bit on a CPU
(``rsqrtf``, ``__expf``, the internal order of tensor-core accumulation), this file
uses correctly rounded fp32 (``1/sqrt`` rounded once, ``exp``), models the attention
products as fp16 accumulation in two steps of 16 with an exact sum inside a step, and
accumulates the head product in fp32; the LayerNorm statistics follow the reference
kernel's own summation order; every other rounding point is the reference's.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

D, DFF, H, DH, T, L = 256, 1024, 8, 32, 32, 8
N_CLOCK, N_REP, N_TYPE_SPECIAL = 101, 3, 12
N_POLICY, N_PROMO = 64, 4
EPS = np.float32(1e-5)
F32, F16 = np.float32, np.float16

#: The statistics' summation order is the reference kernel's (csrc/encoder.cu:566-583): lane l
#: of a warp owns columns 8l..8l+7 and adds them one after the other; the 32 partial sums are
#: then combined by the butterfly 16, 8, 4, 2, 1 (every lane ends with the same total).
_LANES, _LANE_COLS = 32, 8


def f16(x) -> np.ndarray:
    return np.asarray(x).astype(F16)


def add_f16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """fp16 + fp16 rounded once to fp16 (float64 holds the exact sum)."""
    return (a.astype(np.float64) + b.astype(np.float64)).astype(F16)


# ---------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------

def round_e4m3(x) -> np.ndarray:
    """Round to the e4m3 grid (4 exponent bits, bias 7, 3 mantissa bits, no infinities),
    nearest-even, saturating at +-448; returned as float32 values."""
    x = np.asarray(x).astype(np.float64)
    a = np.minimum(np.abs(x), 448.0)
    e = np.maximum(np.floor(np.log2(np.maximum(a, 2.0 ** -9))), -6.0)
    step = 2.0 ** (e - 3.0)
    return (np.sign(x) * np.rint(a / step) * step).astype(F32)


def decode_e4m3(b) -> np.ndarray:
    """e4m3 bytes -> float32 values."""
    b = np.asarray(b).astype(np.int64)
    e, m = (b >> 3) & 15, b & 7
    mag = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    return np.where(b >> 7, -mag, mag).astype(F32)


def quantise_weights_e4m3(w: np.ndarray):
    """``[N, K]`` fp32 -> ``(values on the e4m3 grid [N, K] fp32, scale [N/128] fp32)``: one
    scale ``amax/8`` per 128 output rows over all of K (brokefish/nn/quant.py:208-224 with
    ``q_max=8, tile_k=K``; brokefish/nn/cuda_impl.py:323-335)."""
    n, k = w.shape
    b = w.astype(F32).reshape(n // 128, 128 * k)
    amax = np.abs(b).max(axis=1)
    scale = np.where(amax > 0, amax / F32(8.0), F32(1.0)).astype(F32)
    return round_e4m3((b / scale[:, None]).astype(F32)).reshape(n, k), scale


def quantise_weights_s8(w: np.ndarray):
    """``[N, K]`` fp32 -> ``(q [N, K] int8, scale [N/128] fp32)``; one scale per 128
    output rows over all of K, ``amax/127``, round-half-even, clamp +-127."""
    n, k = w.shape
    b = w.astype(F32).reshape(n // 128, 128 * k)
    amax = np.abs(b).max(axis=1)
    scale = np.where(amax > 0, amax / F32(127.0), F32(1.0)).astype(F32)
    q = np.clip(np.rint(b / scale[:, None]), -127, 127).astype(np.int8)
    return q.reshape(n, k), scale


@dataclass
class LayerW:
    q_qkv: np.ndarray; s_qkv: np.ndarray; b_qkv: np.ndarray
    q_o: np.ndarray; s_o: np.ndarray; b_o: np.ndarray
    q_ff1: np.ndarray; s_ff1: np.ndarray; b_ff1: np.ndarray
    q_ff2: np.ndarray; s_ff2: np.ndarray; b_ff2: np.ndarray


@dataclass
class Weights:
    layers: List[LayerW]
    emb: Dict[str, np.ndarray]            # fp16 tables
    lnf_w: np.ndarray; lnf_b: np.ndarray  # fp16
    head: np.ndarray                      # [96, 256] fp16
    n_value: int
    vmode: int
    rj_mode: int = 0                      # 0 none, 1 attention norms, 2 both norms
    rj_coef: Optional[np.ndarray] = None  # [sites, 5] fp16
    #: "int8_ffn": the FFN as in "int8", QKV and out-projection as in "f16".
    #: "int8": the four matmuls in s8/u8.  "e4m3": the two FFN matmuls in e4m3 (q_* hold grid
    #: values as fp32), QKV and out-projection in fp16 (q_* hold the fp16 matrices, scales 1).
    fmt: str = "int8"


def prepare(state: Dict[str, np.ndarray], fmt: str = "int8") -> Weights:
    """Fold, quantise and round a fp32 ``state_dict`` (numpy arrays)."""
    if fmt not in ("int8", "e4m3", "f16", "int8_ffn", "int8_ffn_qkv"):
        raise ValueError(fmt)
    s = {k: np.asarray(v) for k, v in state.items()}
    n_layers = 1 + max(int(k.split(".")[2]) for k in s if k.startswith("encoder.layers."))
    layers = []
    for i in range(n_layers):
        p = f"encoder.layers.{i}."
        w_qkv = s[p + "self_attn.in_proj_weight"].astype(F32).copy()
        b_qkv = s[p + "self_attn.in_proj_bias"].astype(F32).copy()
        sc = F32(DH ** -0.5)
        w_qkv[:D] *= sc
        b_qkv[:D] *= sc
        g1, e1 = s[p + "norm1.weight"].astype(F32), s[p + "norm1.bias"].astype(F32)
        # bias uses W before gamma; the dot product is taken in float64 and rounded once
        b_qkv = (b_qkv.astype(np.float64) + w_qkv.astype(np.float64) @ e1.astype(np.float64)).astype(F32)
        w_qkv = w_qkv * g1[None, :]
        w_ff1 = s[p + "linear1.weight"].astype(F32).copy()
        b_ff1 = s[p + "linear1.bias"].astype(F32).copy()
        g2, e2 = s[p + "norm2.weight"].astype(F32), s[p + "norm2.bias"].astype(F32)
        b_ff1 = (b_ff1.astype(np.float64) + w_ff1.astype(np.float64) @ e2.astype(np.float64)).astype(F32)
        w_ff1 = w_ff1 * g2[None, :]
        if fmt == "int8":
            q_qkv, s_qkv = quantise_weights_s8(w_qkv)
            q_o, s_o = quantise_weights_s8(s[p + "self_attn.out_proj.weight"])
            q_ff1, s_ff1 = quantise_weights_s8(w_ff1)
            q_ff2, s_ff2 = quantise_weights_s8(s[p + "linear2.weight"])
        else:
            q_qkv, s_qkv = f16(w_qkv), np.ones(6, dtype=F32)
            q_o, s_o = f16(s[p + "self_attn.out_proj.weight"]), np.ones(2, dtype=F32)
            if fmt == "int8_ffn_qkv":  # the reference's "ffn+qkv" scheme: only the out-projection stays fp16
                q_qkv, s_qkv = quantise_weights_s8(w_qkv)
            if fmt in ("int8_ffn", "int8_ffn_qkv"):      # int8 FFN ("ffn": fp16 QKV and out-projection)
                q_ff1, s_ff1 = quantise_weights_s8(w_ff1)
                q_ff2, s_ff2 = quantise_weights_s8(s[p + "linear2.weight"])
            elif fmt == "e4m3":
                q_ff1, s_ff1 = quantise_weights_e4m3(w_ff1)
                q_ff2, s_ff2 = quantise_weights_e4m3(s[p + "linear2.weight"].astype(F32))
            else:               # the reference's default arithmetic: every matrix fp16
                q_ff1, s_ff1 = f16(w_ff1), np.ones(8, dtype=F32)
                q_ff2, s_ff2 = f16(s[p + "linear2.weight"]), np.ones(2, dtype=F32)
        layers.append(LayerW(q_qkv, s_qkv, f16(b_qkv), q_o, s_o,
                             f16(s[p + "self_attn.out_proj.bias"]),
                             q_ff1, s_ff1, f16(b_ff1), q_ff2, s_ff2,
                             f16(s[p + "linear2.bias"])))
    nv = int(s["value.weight"].shape[0])
    head = np.zeros((96, D), dtype=F16)
    head[:64] = f16(s["policy.weight"])
    head[64:68] = f16(s["promo.weight"])
    head[68:68 + nv] = f16(s["value.weight"])
    emb = {k: f16(s[k + ".weight"]) for k in
           ("emb_square", "emb_type_special", "emb_color_turn", "emb_clock", "emb_rep")}
    vmode = int(s["value_mode"]) if "value_mode" in s else 0
    rj_mode = int(s["reinject_mode"]) if "reinject_mode" in s else 0
    rj_coef = f16(s["reinject_c"]) if rj_mode else None
    return Weights(layers, emb, f16(s["norm_f.weight"]), f16(s["norm_f.bias"]), head, nv, vmode,
                   rj_mode, rj_coef, fmt)


# ---------------------------------------------------------------------------
# stages
# ---------------------------------------------------------------------------

def embed(w: Weights, boards: np.ndarray, control: np.ndarray, rep: np.ndarray):
    """``[n,32]`` words -> (``[n,32,256]`` fp16 tokens, ``[n,32]`` alive)."""
    wd = boards.astype(np.int64) & 0xFFFF
    ctl = control.astype(np.int64)
    stm = (ctl < 0).astype(np.int64)
    sq = wd & 63
    ts = np.minimum(((wd >> 6) & 7) * 2 + ((wd >> 9) & 1), N_TYPE_SPECIAL - 1)
    ct = ((wd >> 10) & 1) * 2 + stm[:, None]
    clk = np.clip(np.abs(ctl) - 1, 0, N_CLOCK - 1)
    rp = np.minimum(rep.astype(np.int64), N_REP - 1)
    per_board = add_f16(w.emb["emb_clock"][clk], w.emb["emb_rep"][rp])
    x = add_f16(w.emb["emb_square"][sq], w.emb["emb_type_special"][ts])
    x = add_f16(x, w.emb["emb_color_turn"][ct])
    x = add_f16(x, per_board[:, None, :])
    return x, ((wd >> 11) & 1) == 0


def fma_f16(a, b, c) -> np.ndarray:
    """fp16 fused multiply-add, rounded once (float64 holds a*b + c exactly)."""
    return (np.asarray(a).astype(np.float64) * np.asarray(b).astype(np.float64)
            + np.asarray(c).astype(np.float64)).astype(F16)


def reinject(w: Weights, x16: np.ndarray, boards, control, rep, site: int) -> np.ndarray:
    """What a block's LayerNorm is given under per-layer input re-injection:
    ``x + sum_k c[site, k] * E_k`` in the reference kernel's fp16 order
    (csrc/encoder.cu:439-583): ``pb = fma(c_clk, clock, c_rep * rep)``,
    ``cs = fma(c_ct, color_turn[slot colour], pb)``, then per token
    ``fma(c_ts, type_special, fma(c_sq, square, x)) + cs``.  The colour row is chosen by the
    slot index (0-15 white, 16-31 black), not by the decoded word."""
    n = boards.shape[0]
    c = w.rj_coef[site]
    wd = boards.astype(np.int64) & 0xFFFF
    ctl = control.astype(np.int64)
    stm = (ctl < 0).astype(np.int64)
    sq = wd & 63
    ts = np.minimum(((wd >> 6) & 7) * 2 + ((wd >> 9) & 1), N_TYPE_SPECIAL - 1)
    clk = np.clip(np.abs(ctl) - 1, 0, N_CLOCK - 1)
    rp = np.minimum(rep.astype(np.int64), N_REP - 1)
    slot_col = (np.arange(T) >= T // 2).astype(np.int64)
    pb = fma_f16(c[3], w.emb["emb_clock"][clk], (c[4].astype(np.float64)
                                                 * w.emb["emb_rep"][rp].astype(np.float64)).astype(F16))
    cs = fma_f16(c[2], w.emb["emb_color_turn"][slot_col[None, :] * 2 + stm[:, None]], pb[:, None, :])
    t = fma_f16(c[0], w.emb["emb_square"][sq], x16.reshape(n, T, D))
    t = fma_f16(c[1], w.emb["emb_type_special"][ts], t)
    return add_f16(t, cs).reshape(n * T, D)


def ln_stats(x16: np.ndarray):
    """Row mean and 1/std of fp16 rows ``[M, 256]`` in the fixed summation order."""
    v = x16.astype(F32).reshape(-1, _LANES, _LANE_COLS)
    tot = np.zeros(v.shape[:2], dtype=F32)
    totq = np.zeros(v.shape[:2], dtype=F32)
    for j in range(_LANE_COLS):
        tot = (tot + v[:, :, j]).astype(F32)
        totq = (totq + v[:, :, j] * v[:, :, j]).astype(F32)    # the square of an fp16 is exact in fp32
    while tot.shape[1] > 1:
        h = tot.shape[1] // 2
        tot = (tot[:, :h] + tot[:, h:]).astype(F32)
        totq = (totq[:, :h] + totq[:, h:]).astype(F32)
    tot, totq = tot[:, 0], totq[:, 0]
    mean = (tot * F32(1.0 / 256)).astype(F32)
    t = (totq * F32(1.0 / 256)).astype(F32)
    var = (t.astype(np.float64) - mean.astype(np.float64) ** 2).astype(F32)   # one fma
    var = np.maximum(var, F32(0))
    v = (var + EPS).astype(F32)
    rstd = (1.0 / np.sqrt(v.astype(np.float64))).astype(F32)
    return mean, rstd


def layernorm(x16: np.ndarray, gamma: Optional[np.ndarray] = None,
              beta: Optional[np.ndarray] = None) -> np.ndarray:
    mean, rstd = ln_stats(x16)
    xn = ((x16.astype(F32) - mean[:, None]).astype(F32) * rstd[:, None]).astype(F32)
    if gamma is not None:
        xn = (xn.astype(np.float64) * gamma.astype(np.float64)[None, :]
              + beta.astype(np.float64)[None, :]).astype(F32)
    return xn.astype(F16)


def quantise_rows(x16: np.ndarray, unsigned: bool = False):
    """fp16 rows -> (int values as float32, per-row fp32 scale)."""
    x = x16.astype(F32)
    if unsigned:
        amax = x.max(axis=1)
        amax = np.maximum(amax, F32(0))
        qmax = F32(255.0)
    else:
        amax = np.abs(x).max(axis=1)
        qmax = F32(127.0)
    sc = np.where(amax > 0, (amax / qmax).astype(F32), F32(1.0)).astype(F32)
    inv = (F32(1.0) / sc).astype(F32)
    q = np.rint((x * inv[:, None]).astype(F32))
    q = np.clip(q, 0 if unsigned else -128, 255 if unsigned else 127).astype(F32)
    return q, sc


def quantise_rows_e4m3(x16: np.ndarray):
    """fp16 rows -> (values on the e4m3 grid as fp32, per-row fp32 scale ``amax/8``); the
    scaled value is rounded to fp16 before the e4m3 conversion, as the reference's
    quantiser does (csrc/fp8_gemm.cuh:147-208)."""
    x = x16.astype(F32)
    amax = np.abs(x).max(axis=1)
    sc = np.where(amax > 0, (amax / F32(8.0)).astype(F32), F32(1.0)).astype(F32)
    inv = (F32(1.0) / sc).astype(F32)
    return round_e4m3((x * inv[:, None]).astype(F32).astype(F16)), sc


def gemm_int(q_a: np.ndarray, q_w: np.ndarray) -> np.ndarray:
    """``A @ W^T`` in float32.  For int8 operands this is the exact integer product: every
    partial sum is below 2^24 (255 * 127 * 256 = 8.29e6), so fp32 accumulation is exact in
    any order.  For e4m3 operands it is an fp32-accumulated product (the tensor cores'
    summation order is not reproduced)."""
    return q_a.astype(F32) @ q_w.astype(F32).T


def descale(acc: np.ndarray, sa: np.ndarray, sw_blocks: np.ndarray, n0: int = 0):
    """``(float(acc) * sa[row]) * sw[col // 128]`` in fp32, two roundings."""
    n = acc.shape[1]
    sw = sw_blocks[(n0 + np.arange(n)) // 128].astype(F32)
    return ((acc.astype(F32) * sa[:, None]).astype(F32) * sw[None, :]).astype(F32)


def _mma_f16acc(a: np.ndarray, b: np.ndarray, acc: Optional[np.ndarray] = None) -> np.ndarray:
    """``a @ b`` for fp16 operands with the contraction cut into steps of 16 and an fp16
    accumulator between the steps, the shape of the reference's ``mma.sync m16n8k16`` with
    fp16 accumulators (csrc/mma.cuh:68-75).  Inside a step the sum is taken exactly and rounded
    once; the hardware's own order inside a step is not documented, so this is a model of it,
    not a transcript."""
    for k0 in range(0, a.shape[-1], 16):
        part = np.matmul(a[..., k0:k0 + 16].astype(np.float64), b[..., k0:k0 + 16, :].astype(np.float64))
        acc = part.astype(F16) if acc is None else (acc.astype(np.float64) + part).astype(F16)
    return acc


def attention(q16, k16, v16, alive):
    """``[n,32,256]`` fp16 Q, K, V (scale pre-folded) -> ``[n,32,256]`` fp16, in the
    reference's arithmetic (csrc/encoder.cu:715-797): both products accumulate in fp16 in two
    steps of 16, the softmax is fp32 (``exp`` here where the kernel has the hardware
    ``__expf``; the row sum's order is not mirrored)."""
    n = q16.shape[0]
    q = q16.reshape(n, T, H, DH).transpose(0, 2, 1, 3)
    k = k16.reshape(n, T, H, DH).transpose(0, 2, 1, 3)
    v = v16.reshape(n, T, H, DH).transpose(0, 2, 1, 3)
    s = _mma_f16acc(q, k.transpose(0, 1, 3, 2)).astype(F32)          # [n,H,32,32]
    s = np.where(alive[:, None, None, :], s, F32(-np.inf))
    with np.errstate(invalid="ignore"):
        mx = s.max(axis=-1, keepdims=True)
        p = np.exp((s - mx).astype(F32)).astype(F32)
        inv = (F32(1.0) / p.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)
        pn = (p * inv).astype(F16)
        o = _mma_f16acc(pn, v)
    return o.transpose(0, 2, 1, 3).reshape(n, T, D).astype(F16)


@dataclass
class Trace:
    """Optional per-stage outputs; keys follow the reference's ``debug_stage`` numbers
    for layer 0 (9 embed, 1 LN1, 5/6/7 Q/K/V, 4 attention out, 2 residual after
    attention, 3 LN2, 8 final norm) plus GEMM captures ``(layer, op)`` ->
    ``(A int values, s32 accumulators)`` with op in qkv, out, ff1_c, ff2_c."""
    stages: Dict[int, np.ndarray] = field(default_factory=dict)
    gemms: Dict[tuple, tuple] = field(default_factory=dict)
    #: (layer, stage) -> activations for every layer; stage 10 = residual at layer end
    by_layer: Dict[tuple, np.ndarray] = field(default_factory=dict)


def forward(w: Weights, boards, control, rep, legal=None, trace: Optional[Trace] = None,
            capture_layers=()):
    """Boards to ``(policy fp16 [n,32,64], promo fp16 [n,32,4], value fp32 [n])``.

    ``legal`` (``[n,32]`` uint64, bit s of word p set when the move p->s is legal) turns
    every illegal policy entry into -inf, bitwise.
    """
    boards = np.asarray(boards)
    control = np.asarray(control)
    rep = np.asarray(rep)
    n = boards.shape[0]
    x, alive = embed(w, boards, control, rep)
    if trace is not None:
        trace.stages[9] = x.copy()
    x = x.reshape(n * T, D)

    def cap(layer, op, qa, acc):
        if trace is not None and layer in capture_layers:
            trace.gemms[(layer, op)] = (qa.copy(), acc.astype(np.int32))

    for li, lw in enumerate(w.layers):
        first = li == 0 and trace is not None
        site1 = li * 2 if w.rj_mode == 2 else li
        xn = layernorm(reinject(w, x, boards, control, rep, site1) if w.rj_mode else x)
        if first:
            trace.stages[1] = xn.reshape(n, T, D).copy()
        e4 = w.fmt in ("e4m3", "f16", "int8_ffn", "int8_ffn_qkv")       # fp16 out-projection
        if e4 and w.fmt != "int8_ffn_qkv":       # fp16 QKV with fp16 accumulators, 16 steps of 16 (csrc/encoder.cu:1366-1368)
            qkv = add_f16(_mma_f16acc(xn, lw.q_qkv.astype(F16).T), lw.b_qkv[None, :])
        else:
            qa, sa = quantise_rows(xn)
            acc = gemm_int(qa, lw.q_qkv)
            cap(li, "qkv", qa, acc)
            qkv = add_f16(descale(acc, sa, lw.s_qkv).astype(F16), lw.b_qkv[None, :])
        q16, k16, v16 = (qkv[:, i * D:(i + 1) * D].reshape(n, T, D) for i in range(3))
        if first:
            trace.stages[5], trace.stages[6], trace.stages[7] = q16.copy(), k16.copy(), v16.copy()
        o = attention(q16, k16, v16, alive)
        if first:
            trace.stages[4] = o.copy()
        if e4:
            y = add_f16(_mma_f16acc(o.reshape(n * T, D), lw.q_o.astype(F16).T), lw.b_o[None, :])
        else:
            qa, sa = quantise_rows(o.reshape(n * T, D))
            acc = gemm_int(qa, lw.q_o)
            cap(li, "out", qa, acc)
            y = add_f16(descale(acc, sa, lw.s_o).astype(F16), lw.b_o[None, :])
        x = add_f16(x, y)
        if trace is not None:
            trace.by_layer[(li, 4)] = o.copy()
            trace.by_layer[(li, 2)] = x.reshape(n, T, D).copy()
        if first:
            trace.stages[2] = x.reshape(n, T, D).copy()
        xn = layernorm(reinject(w, x, boards, control, rep, li * 2 + 1) if w.rj_mode == 2 else x)
        if first:
            trace.stages[3] = xn.reshape(n, T, D).copy()
        if w.fmt == "f16":
            # fp16 FFN (csrc/encoder.cu:1431-1556 without quantisation): ff1 per chunk with fp16
            # accumulators, + bias, ReLU; the ff2 accumulators run on through all four chunks
            ff = None
            for c in range(DFF // 256):
                hid = add_f16(_mma_f16acc(xn, lw.q_ff1[256 * c:256 * c + 256].astype(F16).T),
                              lw.b_ff1[None, 256 * c:256 * c + 256])
                hid = np.maximum(hid, F16(0))
                ff = _mma_f16acc(hid, lw.q_ff2[:, 256 * c:256 * c + 256].astype(F16).T, acc=ff)
            x = add_f16(x, add_f16(ff, lw.b_ff2[None, :]))
            if trace is not None:
                trace.by_layer[(li, 10)] = x.reshape(n, T, D).copy()
            continue
        qa, sa = quantise_rows_e4m3(xn) if w.fmt == "e4m3" else quantise_rows(xn)
        run = np.zeros((n * T, D), dtype=F16)
        e4 = w.fmt == "e4m3"
        for c in range(DFF // 256):
            acc = gemm_int(qa, lw.q_ff1[256 * c:256 * c + 256])
            if not e4:
                cap(li, f"ff1_{c}", qa, acc)
            hid = add_f16(descale(acc, sa, lw.s_ff1, n0=256 * c).astype(F16),
                          lw.b_ff1[None, 256 * c:256 * c + 256])
            hid = np.maximum(hid, F16(0))
            qh, sh = quantise_rows_e4m3(hid) if e4 else quantise_rows(hid, unsigned=True)
            acc2 = gemm_int(qh, lw.q_ff2[:, 256 * c:256 * c + 256])
            if not e4:
                cap(li, f"ff2_{c}", qh, acc2)
            # `float(acc) * sa * sw + float(run)` (csrc/int8_gemm.cuh:285-294): the compiler fuses
            # the second product with the sum, so it is one fma (float64 holds it exactly)
            sw2 = lw.s_ff2[np.arange(D) // 128].astype(np.float64)
            prod = (acc2.astype(F32) * sh[:, None]).astype(F32)
            o32 = (prod.astype(np.float64) * sw2[None, :] + run.astype(np.float64)).astype(F32)
            run = o32.astype(F16)
        y = add_f16(run, lw.b_ff2[None, :])
        x = add_f16(x, y)
        if trace is not None:
            trace.by_layer[(li, 10)] = x.reshape(n, T, D).copy()

    hn = layernorm(x, w.lnf_w, w.lnf_b)
    if trace is not None:
        trace.stages[8] = hn.reshape(n, T, D).copy()
    logits = _mma_f16acc(hn, w.head.T).reshape(n, T, 96)        # fp16 accumulators, 16 steps of 16
    policy = logits[:, :, :N_POLICY].copy()
    promo = logits[:, :, N_POLICY:N_POLICY + N_PROMO].copy()
    vcols = logits[:, :, 68:68 + w.n_value].astype(F32)
    ctl = control.astype(np.int64)
    if w.vmode == 0:
        king = np.where(ctl < 0, 31, 15)
        raw = vcols[np.arange(n), king]
    elif w.vmode == 1:
        m = alive.astype(F32)
        raw = (vcols * m[:, :, None]).sum(axis=1, dtype=F32) / np.maximum(
            m.sum(axis=1, dtype=F32), F32(1))[:, None]
    else:
        # "prenorm": mean of the raw residual over live tokens, final LayerNorm with affine,
        # value rows, all fp32 (csrc/encoder.cu:1008-1057; nn/model.py:576-584)
        m = alive.astype(F32)
        xr = x.reshape(n, T, D).astype(F32)
        pooled = (xr * m[:, :, None]).sum(axis=1, dtype=F32) / np.maximum(m.sum(axis=1, dtype=F32), F32(1))[:, None]
        mu = pooled.mean(axis=1, dtype=F32)
        var = np.maximum((pooled * pooled).mean(axis=1, dtype=F32) - mu * mu, F32(0))
        rs = (F32(1) / np.sqrt(var + EPS)).astype(F32)
        nv = ((pooled - mu[:, None]) * rs[:, None] * w.lnf_w.astype(F32)[None, :] + w.lnf_b.astype(F32)[None, :])
        raw = (nv.astype(F32) @ w.head[68:68 + w.n_value].astype(F32).T).astype(F32)
    if w.n_value == 1:
        value = np.tanh(raw[:, 0]).astype(F32)
    else:
        e = np.exp(raw - raw.max(axis=1, keepdims=True))
        value = ((e[:, 2] - e[:, 0]) / e.sum(axis=1)).astype(F32)
    if w.vmode != 0:
        value = np.where(ctl < 0, -value, value).astype(F32)
    if legal is not None:
        bits = (np.asarray(legal).astype(np.uint64)[:, :, None]
                >> np.arange(64, dtype=np.uint64)[None, None, :]) & np.uint64(1)
        policy = np.where(bits.astype(bool), policy, F16(-np.inf))
    return policy, promo, value


def masked_argmax(policy: np.ndarray, legal: np.ndarray) -> np.ndarray:
    """Argmax of ``where(legal, logit, -inf)`` over the 2048 moves, lowest index on
    ties; -1 for a position with no legal move."""
    n = policy.shape[0]
    bits = ((np.asarray(legal).astype(np.uint64)[:, :, None]
             >> np.arange(64, dtype=np.uint64)[None, None, :]) & np.uint64(1)).astype(bool)
    flat = np.where(bits, policy.astype(F32), F32(-np.inf)).reshape(n, -1)
    best = flat.argmax(axis=1)
    return np.where(bits.reshape(n, -1).any(axis=1), best, -1)
