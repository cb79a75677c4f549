"""Fold, quantise and lay out a network's weights as the blob the sm_100a kernel streams.

What happens here, once per weight snapshot (the reference does the same work in
``FusedEncoder.__init__`` / ``_pack_int8`` / ``_pack_tail``, brokefish/nn/cuda_impl.py:
194-227, 339-371, 375-406):

* ``1/sqrt(d_head)`` is folded into the Q rows of ``in_proj`` (weight and bias);
* each block's LayerNorm affine is folded into the GEMM that consumes it
  (``W <- W * gamma``, ``b <- b + W @ beta`` with the *unfolded* ``W``);
* the four folded matrices per layer are quantised to s8 with one fp32 scale per 128
  output rows (:func:`brokefish_b200.nn.quant.quantise_weights_int8_bytes`);
* the bytes are written out as *stage images*: the exact shared-memory picture of a
  K-major, 128-byte-swizzled tensor-core B operand, in the order the kernel's bulk
  copy engine consumes them, so one linear ``cp.async.bulk`` per stage is all the
  device does.

Blob layout (all offsets 256-byte aligned, little endian; mirrored by
``include/brokefish_b200.h``):

    header   256 B   magic, version, n_layers, n_value, vmode, eps, rj_mode, quant, section table
                     (offset, bytes of wstream, lparams, emb, tail, rj), total bytes
    wstream  n_layers * 786432 B + 49152 B
                     per layer 8 QKV stages [192 rows x 128 B], then 36 stages
                     [128 rows x 128 B]: out-proj (2 units) and the FFN units in
                     issue order; after the last layer the [96 x 256] fp16 head matrix
                     (policy rows 0-63, promo 64-67, value from 68) as 4 stages
                     [96 rows x 128 B], one per K-slab of 64 columns
    lparams  n_layers * 4736 B
                     per layer 18 fp32 weight scales (qkv 6, out 2, ff1 8, ff2 2; padded
                     to 128 B) then fp16 biases: qkv (chunk order) 768, out 256,
                     ff1 1024, ff2 256
    emb      184 * 256 fp16: square, type_special, color_turn, clock, rep tables
    tail     1280 fp16: norm_f gamma, beta, then the value head's rows as three plain
             row-major vectors (zero rows beyond n_value)
    rj       (only with per-layer input re-injection) sites * 8 fp16: five coefficients per
             site (square, type_special, color_turn, clock, rep), padded to 8; 16 sites
             when both norms of a layer inject, 8 when only the attention norm does

A QKV "chunk" j (0..3) holds heads 2j and 2j+1: rows 0-63 are their Q rows, 64-127
their K rows, 128-191 their V rows.  A stage image stores row r's 16-byte group c at
byte ``r*128 + ((c ^ (r & 7)) * 16)``.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import List

import numpy as np
import torch

from brokefish_b200.nn.model import (BrokefishNet, EMB_TABLES, N_POLICY, N_PROMO,
                                     REINJECT_MODE_ID, VALUE_MODE_ID)
from brokefish_b200.nn.quant import Q_MAX, quantise_weights_bytes, quantise_weights_int8_bytes

MAGIC = 0x38424642          # "BFB8"
VERSION = 4
HEADER_BYTES = 256
D, DFF, H, DH, T = 256, 1024, 8, 32, 32
NHEAD = 96                   # head matrix rows: 64 policy, 4 promo, 1-3 value, zero pad
VALUE_ROW = N_POLICY + N_PROMO
LAYER_STREAM_BYTES = 786432
LAYER_STREAM_BYTES_E4M3 = 1048576
LAYER_STREAM_BYTES_F16 = 1572864
LAYER_STREAM_BYTES_QKV8 = 851968      # s8 QKV, fp16 out-projection, s8 FFN
#: Arithmetic of a blob, by the reference's kernel mode number: 3 = int8 on all four
#: matmuls, 1 = e4m3 on the two FFN matmuls with fp16 QKV and out-projection.
QUANT_INT8, QUANT_E4M3, QUANT_F16, QUANT_INT8_FFN, QUANT_INT8_FFN_QKV = 3, 1, 0, 2, 4
HEAD_STREAM_BYTES = 4 * NHEAD * 128
LPARAM_STRIDE = 4736
LP_SW_QKV, LP_SW_O, LP_SW_FF1, LP_SW_FF2 = 0, 24, 32, 64
LP_B_QKV, LP_B_O, LP_B_FF1, LP_B_FF2 = 128, 1664, 2176, 4224
#: The FFN's sixteen GEMM units in issue order: (kind, hidden chunk c, half j).
#: kind 1 = ff1 rows ``256c + 128j ..`` over K = 256; kind 2 = ff2 rows ``128j ..`` over
#: hidden columns ``256c ..``.
FFN_UNITS = [(1, 0, 0), (1, 0, 1), (1, 1, 0), (1, 1, 1), (2, 0, 0), (2, 0, 1),
             (1, 2, 0), (1, 2, 1), (2, 1, 0), (2, 1, 1), (1, 3, 0), (1, 3, 1),
             (2, 2, 0), (2, 2, 1), (2, 3, 0), (2, 3, 1)]


def fold_norm(w: torch.Tensor, b: torch.Tensor, norm):
    """``LN(x) W^T + b == x_hat (W * gamma)^T + (b + W beta)``; fp32 in, fp32 out."""
    gamma = norm.weight.detach().float()
    beta = norm.bias.detach().float()
    return w * gamma[None, :], b + w @ beta


def qkv_chunk_rows() -> np.ndarray:
    """``[4, 192]``: the ``in_proj`` row behind each row of each QKV chunk."""
    rows = np.empty((4, 192), dtype=np.int64)
    for j in range(4):
        for i in range(192):
            rows[j, i] = (i // 64) * D + 64 * j + (i % 64)
    return rows


def sw128_image(tile: np.ndarray) -> np.ndarray:
    """``[R, 128]`` bytes -> the same bytes in 128-byte-swizzled K-major order."""
    r = tile.shape[0]
    if tile.shape[1] != 128 or tile.dtype != np.uint8:
        raise ValueError("a stage image is built from [rows, 128] uint8")
    groups = tile.reshape(r, 8, 16)
    dst = np.arange(8)[None, :] ^ (np.arange(r)[:, None] & 7)        # [r, 8]
    out = np.empty_like(groups)
    out[np.arange(r)[:, None], dst] = groups
    return out.reshape(-1)


@dataclass
class FoldedLayer:
    """One layer after folding and quantisation (natural row order, no layout yet).  In the
    e4m3 arithmetic ``q_qkv`` / ``q_o`` are the fp16 matrices viewed as bytes ``[N, 512]``
    and their scales are ones."""
    q_qkv: np.ndarray; s_qkv: np.ndarray; b_qkv: np.ndarray     # [768,256] u8, [6], [768] f16
    q_o: np.ndarray; s_o: np.ndarray; b_o: np.ndarray
    q_ff1: np.ndarray; s_ff1: np.ndarray; b_ff1: np.ndarray
    q_ff2: np.ndarray; s_ff2: np.ndarray; b_ff2: np.ndarray


def fold_and_quantise(net: BrokefishNet, fmt: str = "int8") -> List[FoldedLayer]:
    """The per-layer folded matrices, scales and fp16 biases.  ``fmt="int8"``: all four
    matrices s8.  ``fmt="e4m3"``: the two FFN matrices e4m3 with ``amax/8`` scales, QKV and
    out-projection fp16 (brokefish/nn/cuda_impl.py:303-337).  ``fmt="f16"``: all four fp16, the
    folded fp32 matrices rounded once (cuda_impl.py:194-228).  ``fmt="int8_ffn"``: the reference's
    "ffn" int8 scheme (quant 2): the two FFN matrices s8, QKV and out-projection fp16.
    ``fmt="int8_ffn_qkv"``: its "ffn+qkv" scheme (quant 4): only the out-projection stays fp16."""
    if fmt not in ("int8", "e4m3", "f16", "int8_ffn", "int8_ffn_qkv"):
        raise ValueError(f"fmt must be 'int8', 'int8_ffn', 'int8_ffn_qkv', 'e4m3' or 'f16', got {fmt!r}")
    out = []
    scale = DH ** -0.5
    for lay in net.encoder.layers:
        w_qkv = lay.self_attn.in_proj_weight.detach().float().clone()
        b_qkv = lay.self_attn.in_proj_bias.detach().float().clone()
        w_qkv[:D] *= scale
        b_qkv[:D] *= scale
        w_qkv, b_qkv = fold_norm(w_qkv, b_qkv, lay.norm1)
        w_ff1, b_ff1 = fold_norm(lay.linear1.weight.detach().float().clone(),
                                 lay.linear1.bias.detach().float().clone(), lay.norm2)
        mats = {}
        for name, w in (("qkv", w_qkv), ("o", lay.self_attn.out_proj.weight.detach()),
                        ("ff1", w_ff1), ("ff2", lay.linear2.weight.detach())):
            if (fmt == "int8" or (fmt == "int8_ffn" and name in ("ff1", "ff2"))
                    or (fmt == "int8_ffn_qkv" and name != "o")):
                qb, sc = quantise_weights_int8_bytes(w.float())
            elif fmt == "e4m3" and name in ("ff1", "ff2"):
                qb, sc = quantise_weights_bytes(w.float(), Q_MAX, tile_k=w.shape[1])
                sc = sc.reshape(-1)
            else:
                qb = w.float().half().contiguous().view(torch.uint8).reshape(w.shape[0], -1)
                sc = torch.ones(w.shape[0] // 128)
            mats[name] = (qb.cpu().numpy(), sc.cpu().numpy().astype(np.float32))

        def f16(v):
            return v.detach().float().half().cpu().numpy()
        out.append(FoldedLayer(
            mats["qkv"][0], mats["qkv"][1], f16(b_qkv),
            mats["o"][0], mats["o"][1], f16(lay.self_attn.out_proj.bias),
            mats["ff1"][0], mats["ff1"][1], f16(b_ff1),
            mats["ff2"][0], mats["ff2"][1], f16(lay.linear2.bias)))
    return out


def head_matrix(net: BrokefishNet) -> np.ndarray:
    """``[96, 256]`` fp16: policy rows 0-63, promo 64-67, value from 68, zeros after."""
    head = torch.zeros(NHEAD, D, dtype=torch.half)
    head[:N_POLICY] = net.policy.weight.detach().half().cpu()
    head[N_POLICY:VALUE_ROW] = net.promo.weight.detach().half().cpu()
    nv = int(net.value.weight.shape[0])
    head[VALUE_ROW:VALUE_ROW + nv] = net.value.weight.detach().half().cpu()
    return head.numpy()


def _layer_stream(fl: FoldedLayer) -> np.ndarray:
    parts = []
    rows = qkv_chunk_rows()
    slabs = fl.q_qkv.shape[1] // 128          # 2 for s8 (K = 256 bytes), 4 for fp16 (512 bytes)
    slabs_o = fl.q_o.shape[1] // 128
    for j in range(4):
        chunk = fl.q_qkv[rows[j]]                                   # [192, K bytes]
        for s in range(slabs):
            parts.append(sw128_image(np.ascontiguousarray(chunk[:, 128 * s:128 * s + 128])))
    for u in range(2):
        for s in range(slabs_o):
            parts.append(sw128_image(np.ascontiguousarray(
                fl.q_o[128 * u:128 * u + 128, 128 * s:128 * s + 128])))
    if fl.q_ff1.shape[1] == 512:
        # fp16 FFN: units of 4 K-slabs of 64 halves each; the ff2 accumulators run on through
        # the chunks, so its units follow the chunk order
        def ff1_unit(c, j):
            return [sw128_image(np.ascontiguousarray(
                fl.q_ff1[256 * c + 128 * j:256 * c + 128 * j + 128, 128 * s:128 * s + 128])) for s in range(4)]

        def ff2_unit(c, j):
            return [sw128_image(np.ascontiguousarray(
                fl.q_ff2[128 * j:128 * j + 128, 512 * c + 128 * s:512 * c + 128 * s + 128])) for s in range(4)]

        # issue order of the MMA schedule: F1 c0 j0, F1 c0 j1, then per chunk c: F1 c+1 j0,
        # F2 c j0, F2 c j1, F1 c+1 j1
        parts += ff1_unit(0, 0) + ff1_unit(0, 1)
        for c in range(4):
            if c < 3:
                parts += ff1_unit(c + 1, 0)
            parts += ff2_unit(c, 0) + ff2_unit(c, 1)
            if c < 3:
                parts += ff1_unit(c + 1, 1)
    else:
        for kind, c, j in FFN_UNITS:
            for s in range(2):
                if kind == 1:
                    blk = fl.q_ff1[256 * c + 128 * j:256 * c + 128 * j + 128,
                                   128 * s:128 * s + 128]
                else:
                    blk = fl.q_ff2[128 * j:128 * j + 128,
                                   256 * c + 128 * s:256 * c + 128 * s + 128]
                parts.append(sw128_image(np.ascontiguousarray(blk)))
    stream = np.concatenate(parts)
    assert stream.size == (LAYER_STREAM_BYTES_F16 if fl.q_ff1.shape[1] == 512 else
                           LAYER_STREAM_BYTES_E4M3 if slabs == 4 else
                           LAYER_STREAM_BYTES if slabs_o == 2 else LAYER_STREAM_BYTES_QKV8)
    return stream


def _layer_params(fl: FoldedLayer) -> np.ndarray:
    buf = np.zeros(LPARAM_STRIDE, dtype=np.uint8)
    buf[LP_SW_QKV:LP_SW_QKV + 24] = fl.s_qkv.astype("<f4").view(np.uint8)
    buf[LP_SW_O:LP_SW_O + 8] = fl.s_o.astype("<f4").view(np.uint8)
    buf[LP_SW_FF1:LP_SW_FF1 + 32] = fl.s_ff1.astype("<f4").view(np.uint8)
    buf[LP_SW_FF2:LP_SW_FF2 + 8] = fl.s_ff2.astype("<f4").view(np.uint8)
    b_qkv = fl.b_qkv[qkv_chunk_rows().reshape(-1)]
    buf[LP_B_QKV:LP_B_QKV + 1536] = b_qkv.astype("<f2").view(np.uint8)
    buf[LP_B_O:LP_B_O + 512] = fl.b_o.astype("<f2").view(np.uint8)
    buf[LP_B_FF1:LP_B_FF1 + 2048] = fl.b_ff1.astype("<f2").view(np.uint8)
    buf[LP_B_FF2:LP_B_FF2 + 512] = fl.b_ff2.astype("<f2").view(np.uint8)
    return buf


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def pack_blob(net: BrokefishNet, fmt: str = "int8") -> np.ndarray:
    """The whole device blob for ``net`` as a ``uint8`` array, in the int8 arithmetic, in the
    e4m3-FFN arithmetic (a layer's stream is 16 QKV stages and 8 out-projection stages of fp16
    followed by the 32 FFN stages of e4m3 bytes: 1,048,576 B per layer) or in the fp16
    arithmetic (``fmt="f16"``: 16 + 8 + 64 stages of fp16, 1,572,864 B per layer)."""
    if (net.d_model, len(net.encoder.layers)) != (D, net.n_layers):
        raise ValueError("unexpected network shape")
    first = net.encoder.layers[0]
    if (first.self_attn.embed_dim, first.self_attn.num_heads,
            first.linear1.out_features) != (D, H, DFF):
        raise ValueError(
            f"kernel is compiled for d_model={D}, d_ff={DFF}, heads={H}; got "
            f"{first.self_attn.embed_dim}, {first.linear1.out_features}, "
            f"{first.self_attn.num_heads}")
    layers = fold_and_quantise(net, fmt)
    if fmt in ("e4m3", "int8_ffn", "int8_ffn_qkv") and getattr(net, "reinject", "none") != "none":
        raise NotImplementedError("input re-injection is built for the int8 and fp16 arithmetics only")
    head_bytes = np.ascontiguousarray(head_matrix(net)).view(np.uint8).reshape(NHEAD, 2 * D)
    wstream = np.concatenate([_layer_stream(fl) for fl in layers] +
                             [sw128_image(np.ascontiguousarray(head_bytes[:, 128 * s:128 * s + 128]))
                              for s in range(4)])
    lparams = np.concatenate([_layer_params(fl) for fl in layers])
    emb = np.concatenate([getattr(net, n).weight.detach().half().cpu().numpy().reshape(-1)
                          for n in EMB_TABLES]).astype("<f2").view(np.uint8)
    val = np.zeros((3, D), dtype=np.float16)
    val[:int(net.value.weight.shape[0])] = net.value.weight.detach().half().cpu().numpy()
    tail = np.concatenate([net.norm_f.weight.detach().half().cpu().numpy(),
                           net.norm_f.bias.detach().half().cpu().numpy(), val.reshape(-1)]
                          ).astype("<f2").view(np.uint8)
    rj_mode = REINJECT_MODE_ID.get(getattr(net, "reinject", "none"), 0)
    rj = np.zeros(0, dtype=np.uint8)
    if rj_mode:
        coef = net.reinject_c.detach().float().half().cpu().numpy()          # [sites, 5]
        slab = np.zeros((coef.shape[0], 8), dtype=np.float16)
        slab[:, :coef.shape[1]] = coef
        rj = slab.reshape(-1).astype("<f2").view(np.uint8)
    sections = [wstream, lparams, emb, tail, rj]
    offs, cur = [], HEADER_BYTES
    for sec in sections:
        offs.append(cur)
        cur = _align(cur + sec.size)
    total = cur
    vmode = VALUE_MODE_ID.get(getattr(net, "value_head", "king"), 0)
    header = struct.pack("<IIIIIfII", MAGIC, VERSION, len(layers),
                         int(net.value.weight.shape[0]), vmode, float(first.norm1.eps), rj_mode,
                         {"int8": QUANT_INT8, "e4m3": QUANT_E4M3, "f16": QUANT_F16, "int8_ffn": QUANT_INT8_FFN,
                          "int8_ffn_qkv": QUANT_INT8_FFN_QKV}[fmt])
    for off, sec in zip(offs, sections):
        header += struct.pack("<QQ", off, sec.size)
    header += struct.pack("<Q", total)
    blob = np.zeros(total, dtype=np.uint8)
    blob[:len(header)] = np.frombuffer(header, dtype=np.uint8)
    for off, sec in zip(offs, sections):
        blob[off:off + sec.size] = sec
    return blob
