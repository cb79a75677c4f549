"""Pins the CPU oracle (oracle/int8_encoder.py) to outputs of the reference's own
Python, committed under tests/golden/ by tests/golden/make_golden.py."""
import hashlib
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import int8_encoder as O


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def kats():
    return np.load(os.path.join(GOLDEN, "scheme_kats.npz"))


def test_weight_quantiser_matches_reference_bytes(kats):
    q, s = O.quantise_weights_s8(kats["w"])
    assert np.array_equal(q.view(np.uint8), kats["w_q"])
    assert np.array_equal(s, kats["w_s"])
    assert tuple(kats["q_max"]) == (127.0, 255.0)


def test_activation_quantiser_matches_reference(kats):
    a16 = kats["acts"].astype(np.float16)
    q, s = O.quantise_rows(a16)
    assert np.array_equal(q, kats["q_s8"])
    assert np.array_equal(s, kats["s_s8"][:, 0])
    # ties go to even, the zero row gets scale 1
    assert list(q[4, :6] * s[4]) == pytest.approx([0.5, 1.5, 2.5, -0.5, -1.5, -2.5], abs=1.0)
    assert s[3] == 1.0 and not q[3].any()
    qu, su = O.quantise_rows(np.maximum(a16, np.float16(0)), unsigned=True)
    assert np.array_equal(qu, kats["q_u8"])
    assert np.array_equal(su, kats["s_u8"][:, 0])


def test_int8_linear_matches_reference(kats):
    a16 = kats["acts"].astype(np.float16)
    qw, sw = O.quantise_weights_s8(kats["w"])
    qa, sa = O.quantise_rows(a16)
    acc = O.gemm_int(qa, qw)
    exact = qa.astype(np.int64) @ qw.astype(np.int64).T
    assert np.array_equal(acc.astype(np.int64), exact)
    out = O.descale(acc, sa, sw) + np.linspace(-1, 1, 256, dtype=np.float32)[None, :]
    assert np.abs(out - kats["lin"]).max() <= 2e-6 * np.abs(kats["lin"]).max() + 1e-6


@pytest.mark.parametrize("name", ["A", "B"])
def test_seeded_weights_are_the_golden_ones(name, states):
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    st = states[name]
    flat = np.concatenate([st[k].numpy().reshape(-1).astype(np.float32) for k in sorted(st)])
    assert sha(flat) == str(g["state_sha"])


@pytest.mark.parametrize("name", ["A", "B"])
def test_fold_and_quantise_matches_reference_digests(name, oracle_weights):
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    want = dict(x.split("=") for x in g["weight_digests"])
    for li, lw in enumerate(oracle_weights[name].layers):
        for tag, q, s in (("qkv", lw.q_qkv, lw.s_qkv), ("o", lw.q_o, lw.s_o),
                          ("ff1", lw.q_ff1, lw.s_ff1), ("ff2", lw.q_ff2, lw.s_ff2)):
            assert sha(q.view(np.uint8)) == want[f"{li}.{tag}.q"], (li, tag)
            assert sha(s) == want[f"{li}.{tag}.s"], (li, tag)
        # the folded biases go through a 256-long fp32 dot product whose summation order is
        # the BLAS library's: equal to within one fp16 step, and almost always equal
        for mine, ref in ((lw.b_qkv, g["folded_b_qkv"][li]), (lw.b_ff1, g["folded_b_ff1"][li])):
            step = np.abs(mine.view(np.int16).astype(np.int32) - ref.view(np.int16).astype(np.int32))
            assert step.max() <= 1 and (step == 0).mean() >= 0.99


@pytest.mark.parametrize("name", ["A", "B"])
def test_embedding_is_bit_exact(name, oracle_weights, pos256):
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    x, alive = O.embed(oracle_weights[name], pos256["boards"], pos256["control"], pos256["rep"])
    assert sha(x) == str(g["embed_sha"])
    assert np.array_equal(x[:4], g["embed_first4"])
    assert np.array_equal(alive, g["alive"])


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_against_reference_fp32_and_int8_emulation(name, oracle_weights, pos256):
    """The reference's own bar for a quantised path against its fp32 network is 8 % of
    max|logit| (its tests/test_quant.py:342-356); against its int8 *emulation* (which
    quantises the unfolded weights and keeps fp32 activations) half of that."""
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    n = g["fp32_policy"].shape[0]
    pol, pro, val = O.forward(oracle_weights[name], pos256["boards"][:n], pos256["control"][:n],
                              pos256["rep"][:n])
    top = np.abs(g["fp32_policy"]).max()
    assert np.isfinite(pol.astype(np.float32)).all()
    assert np.abs(pol.astype(np.float32) - g["fp32_policy"]).max() <= 0.08 * top
    assert np.abs(pro.astype(np.float32) - g["fp32_promo"]).max() <= 0.08 * top
    assert np.abs(val - g["fp32_value"]).max() <= 0.08
    m = g["emu_policy"].shape[0]
    assert np.abs(pol[:m].astype(np.float32) - g["emu_policy"]).max() <= 0.05 * top
    assert np.abs(val[:m] - g["emu_value"]).max() <= 0.08


def test_dead_slots_are_inert_and_batch_composition_does_not_matter(oracle_weights, pos256):
    w = oracle_weights["A"]
    b, c, r = pos256["boards"][:8].copy(), pos256["control"][:8], pos256["rep"][:8]
    p1, _, v1 = O.forward(w, b, c, r)
    p2, _, v2 = O.forward(w, b[3:5], c[3:5], r[3:5])
    assert np.array_equal(p1[3:5], p2) and np.array_equal(v1[3:5], v2)


def test_legal_mask_and_argmax(oracle_weights, pos256):
    w = oracle_weights["A"]
    sl = slice(0, 8)
    raw, _, _ = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl])
    msk, _, _ = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl],
                          legal=pos256["legal"][sl])
    bits = ((pos256["legal"][sl][:, :, None] >> np.arange(64, dtype=np.uint64)) & np.uint64(1)).astype(bool)
    assert np.array_equal(msk[bits], raw[bits])
    assert np.all(np.isneginf(msk[~bits].astype(np.float32)))
    am = O.masked_argmax(raw, pos256["legal"][sl])
    assert all(bits.reshape(8, -1)[i, a] for i, a in enumerate(am) if a >= 0)


@pytest.mark.parametrize("name", ["A", "B"])
def test_fp32_port_matches_reference_fp32(name, states, pos256):
    """The functional fp32 restatement timed as the CPU baseline equals the reference's own
    fp32 network on the committed outputs."""
    import torch
    from oracle import fp32_model
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    n = g["fp32_policy"].shape[0]
    p, pr, v = fp32_model.forward(states[name], torch.from_numpy(pos256["boards"][:n]),
                                  torch.from_numpy(pos256["control"][:n]),
                                  torch.from_numpy(pos256["rep"][:n]))
    assert np.abs(p.numpy() - g["fp32_policy"]).max() < 1e-4
    assert np.abs(pr.numpy() - g["fp32_promo"]).max() < 1e-4
    assert np.abs(v.numpy() - g["fp32_value"]).max() < 1e-4


def test_reinjection_against_reference_fp32(pos256):
    """A re-injecting network (both norms, nonzero coefficients): the oracle's int8 path
    against the reference's fp32 outputs at the reference's 8 % bar; with all-zero
    coefficients the injecting path is bit-identical to the plain one."""
    import copy
    from conftest import REINJECT_SET
    from brokefish_b200.nn.model import seeded_state
    g = np.load(os.path.join(GOLDEN, "ref_outputs_C.npz"))
    st = seeded_state(**REINJECT_SET)
    flat = np.concatenate([st[k].numpy().reshape(-1).astype(np.float32) for k in sorted(st)])
    assert sha(flat) == str(g["state_sha"])
    w = O.prepare({k: v.numpy() for k, v in st.items()})
    assert w.rj_mode == 2 and w.rj_coef.shape == (16, 5)
    n = g["fp32_policy"].shape[0]
    pol, pro, val = O.forward(w, pos256["boards"][:n], pos256["control"][:n], pos256["rep"][:n])
    top = np.abs(g["fp32_policy"].astype(np.float32)).max()
    assert np.abs(pol.astype(np.float32) - g["fp32_policy"].astype(np.float32)).max() <= 0.08 * top
    assert np.abs(val - g["fp32_value"]).max() <= 0.08
    plain = copy.deepcopy(w)
    plain.rj_mode = 0
    differs = O.forward(plain, pos256["boards"][:4], pos256["control"][:4], pos256["rep"][:4])[0]
    assert not np.array_equal(differs, pol[:4])              # the injection does something
    zero = copy.deepcopy(w)
    zero.rj_coef = np.zeros_like(w.rj_coef)
    same = O.forward(zero, pos256["boards"][:4], pos256["control"][:4], pos256["rep"][:4])[0]
    assert np.array_equal(same.view(np.uint16), differs.view(np.uint16))


def test_e4m3_scheme_against_reference(kats, states, pos256):
    """The e4m3 FFN arithmetic: weight bytes and scales equal the reference's
    `quantise_weights_bytes(q_max=8, tile_k=K)`; end to end, the oracle stays within 12 % of
    max|logit| of the reference fp32 network and of the reference's own e4m3 emulation (which
    itself is 7-8 % from fp32 on these networks: three mantissa bits)."""
    q, s = O.quantise_weights_e4m3(kats["w"])
    assert np.array_equal(O.decode_e4m3(kats["w_e4m3"]), q)
    assert np.array_equal(s, kats["w_e4m3_s"].reshape(-1)) and kats["q_max_e4m3"][0] == 8.0
    grid = O.round_e4m3(np.array([0.0, 448.0, 500.0, -600.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 0.0145], np.float32))
    assert list(grid) == [0.0, 448.0, 448.0, -448.0, 2.0 ** -9, 0.0, 2.0 ** -8, 0.013671875]
    for name in ("A", "B"):
        g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
        w = O.prepare({k: v.numpy() for k, v in states[name].items()}, fmt="e4m3")
        n = g["e4m3_policy"].shape[0]
        pol, _, val = O.forward(w, pos256["boards"][:n], pos256["control"][:n], pos256["rep"][:n])
        top = np.abs(g["fp32_policy"]).max()
        assert np.abs(pol.astype(np.float32) - g["fp32_policy"][:n]).max() <= 0.12 * top
        assert np.abs(pol.astype(np.float32) - g["e4m3_policy"].astype(np.float32)).max() <= 0.12 * top
        assert np.abs(val - g["fp32_value"][:n]).max() <= 0.15
