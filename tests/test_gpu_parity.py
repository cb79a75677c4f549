"""Parity of the sm_100a kernel against the CPU oracle, through the C ABI.

Bars: s32 GEMM accumulators bit-exact (always).  On the weights the metric is quoted on
(set A: N(0, 0.02), max|logit| about 1.1): fp16 logits and value within max-abs 2e-2;
masked-policy argmax over non-terminal positions agrees wherever the oracle's best and
second-best legal logits are further apart than that tolerance, and in >= 99.5 % of all
positions (measured: 99.7 % on the 4096-position set; every disagreement is a near tie).

Why the logit bar is a tolerance and not equality: everything up to layer 0's Q/K/V is
bit-identical to the oracle (tested below), but the two attention products accumulate
in fp32 inside the tensor cores in an order a CPU cannot reproduce, so about one fp16
value in 3000 of the first attention output lands on the other side of a rounding
boundary.  Each such flip moves an int8 operand by one step (0.8 % of its row maximum),
and from there the two computations drift apart to a fraction of the int8 quantisation
noise itself -- about 1.5 % of max|logit| after eight layers -- whichever two
implementations are compared.  Set B (reference default init scale, LayerNorm affines
and biases perturbed, max|logit| about 3) is therefore held to the same 2 % in relative
terms and to 98 % argmax agreement."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import int8_encoder as O

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2
VALUE_TOL = 2e-2
ARGMAX_MIN = {"A": 0.995, "B": 0.98}


def logit_tol(name, ref_logits):
    top = float(np.abs(ref_logits.astype(np.float32)).max())
    return LOGIT_TOL if name == "A" else LOGIT_TOL * max(1.0, top)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def inputs(pos, sl):
    return dev(pos["boards"][sl]), dev(pos["control"][sl]), dev(pos["rep"][sl])


@pytest.fixture(scope="module")
def encoders(nets):
    """The product with correctly rounded 1/sqrt in the norms, the form the numpy oracle can
    reproduce; the default (the hardware approximation, as the reference kernel) is what
    `encoders_hw` and tests/test_gpu_reference_kernel.py run."""
    from brokefish_b200.nn import encoder_impl
    out = {k: encoder_impl("cuda")(n, int8=True) for k, n in nets.items()}
    for e in out.values():
        e.exact_rsqrt = True
    yield out
    for e in out.values():
        e.close()


@pytest.fixture(scope="module")
def encoders_hw(nets):
    from brokefish_b200.nn import encoder_impl
    out = {k: encoder_impl("cuda")(n, int8=True) for k, n in nets.items()}
    yield out
    for e in out.values():
        e.close()


def aligned_oracle(oracle_weights, name, enc):
    """The oracle's weights with its two folded biases replaced by the product's after
    checking they agree to one fp16 step (the fold is a BLAS dot product whose summation
    order differs between numpy and torch)."""
    import copy
    from brokefish_b200.nn.pack import fold_and_quantise
    w = copy.deepcopy(oracle_weights[name])
    for lw, fl in zip(w.layers, fold_and_quantise(enc.net)):
        for attr in ("b_qkv", "b_ff1"):
            a, b = getattr(lw, attr), getattr(fl, attr)
            assert np.abs(a.view(np.int16).astype(np.int32) - b.view(np.int16).astype(np.int32)).max() <= 1
            setattr(lw, attr, b.copy())
    return w


def assert_disagreements_are_near_ties(opol, legal, mine, theirs, tol):
    """Where the two argmaxes differ, the oracle itself rates the kernel's move within `tol`
    of its own best move."""
    n = opol.shape[0]
    flat = opol.astype(np.float32).reshape(n, -1)
    for i in np.where((theirs >= 0) & (mine != theirs))[0]:
        assert flat[i, theirs[i]] - flat[i, mine[i]] <= tol, (i, flat[i, theirs[i]], flat[i, mine[i]])


# ---------------------------------------------------------------- tensor-core self test
@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
def test_umma_tile_against_exact_integer_product(mode):
    """One tcgen05 GEMM tile against an exact host product (the method of the reference's
    csrc/tests/tint8.cu:268-337): operands span the full range including -128/255."""
    from brokefish_b200 import _native
    from brokefish_b200.nn.pack import sw128_image
    rng = np.random.default_rng(mode)
    n = {0: 128, 1: 128, 2: 192, 3: 96, 4: 128}[mode]
    if mode == 4:
        # e4m3 operands chosen from small exactly representable values: every sum is exact
        vals = np.array([-2.0, -1.0, -0.5, 0.0, 0.5, 1.0, 2.0, 4.0], dtype=np.float32)
        a = vals[rng.integers(0, 8, size=(128, 256))]
        w = vals[rng.integers(0, 8, size=(n, 256))]
        enc = lambda m: torch.from_numpy(m).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        a_bytes, w_bytes = enc(a), enc(w)
        want = a.astype(np.float64) @ w.astype(np.float64).T
    elif mode == 3:
        a = (rng.standard_normal((128, 256)) * 0.5).astype(np.float16)
        w = (rng.standard_normal((n, 256)) * 0.5).astype(np.float16)
        a_bytes, w_bytes = a.view(np.uint8), w.view(np.uint8)
        want = a.astype(np.float64) @ w.astype(np.float64).T
    else:
        a = rng.integers(0 if mode == 1 else -128, 256 if mode == 1 else 128, size=(128, 256))
        w = rng.integers(-128, 128, size=(n, 256))
        a[0, :] = 255 if mode == 1 else -128
        w[0, :] = -128
        a_bytes = a.astype(np.uint8 if mode == 1 else np.int8).view(np.uint8)
        w_bytes = w.astype(np.int8).view(np.uint8)
        want = a.astype(np.int64) @ w.astype(np.int64).T
    slabs = w_bytes.shape[1] // 128
    image = np.concatenate([sw128_image(np.ascontiguousarray(w_bytes[:, 128 * s:128 * s + 128]))
                            for s in range(slabs)])
    d_a, d_w = dev(a_bytes), dev(image)
    d_out = torch.zeros(128, n, dtype=torch.int32, device="cuda")
    _native.check(_native.lib().bf_selftest_umma(0, mode, ctypes.c_void_p(d_a.data_ptr()),
                                                 ctypes.c_void_p(d_w.data_ptr()),
                                                 ctypes.c_void_p(d_out.data_ptr())), "selftest")
    got = d_out.cpu().numpy()
    if mode == 4:
        assert np.array_equal(got.view(np.float32).astype(np.float64), want)
    elif mode == 3:
        got = got.view(np.float32)
        assert np.abs(got - want).max() <= 1e-3
    else:
        assert np.array_equal(got.astype(np.int64), want)


# ---------------------------------------------------------------- stages
@pytest.mark.parametrize("name", ["A", "B"])
def test_embedding_is_bit_exact(name, encoders, oracle_weights, pos256):
    enc = encoders[name]
    got = enc.forward_stage(*inputs(pos256, slice(0, 256)), 9).cpu().numpy()
    want, _ = O.embed(oracle_weights[name], pos256["boards"], pos256["control"], pos256["rep"])
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    enc.check_status()


def test_embedding_over_every_clock_sign_and_repetition(encoders, oracle_weights, nets, pos256):
    """Every half-move-clock row (1..101, and the clamp beyond), both signs of the control word
    and every repetition value including the clamp (the reference's tests/test_b2.py:110-133),
    bit-exact against the oracle and against the torch module in fp16."""
    enc = encoders["B"]
    clocks = np.arange(1, 111)
    control = np.concatenate([clocks, -clocks]).astype(np.int16)
    grid_c = np.repeat(control, 5)
    grid_r = np.tile(np.arange(5, dtype=np.uint8), len(control))
    boards = np.tile(pos256["boards"][7][None, :], (len(grid_c), 1))
    got = enc.forward_stage(dev(boards), dev(grid_c), dev(grid_r), 9).cpu().numpy()
    want, _ = O.embed(oracle_weights["B"], boards, grid_c, grid_r)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    half = __import__("copy").deepcopy(nets["B"]).half()
    with torch.no_grad():
        x, _ = half.embed(torch.from_numpy(boards), torch.from_numpy(grid_c), torch.from_numpy(grid_r))
    assert np.array_equal(got.view(np.uint16), x.numpy().view(np.uint16))


@pytest.mark.parametrize("name", ["A", "B"])
def test_layer0_stages(name, encoders, oracle_weights, pos256):
    """LN1, Q/K/V and LN2-side stages of layer 0.  LN1 and Q/K/V are reproducible exactly;
    downstream of the first attention a few fp16 last-place differences are expected."""
    enc = encoders[name]
    w = aligned_oracle(oracle_weights, name, enc)
    sl = slice(0, 32)
    tr = O.Trace()
    O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl], trace=tr)
    live = ((pos256["boards"][sl].view(np.uint16) >> 11) & 1) == 0
    for stage in (1, 5, 6, 7):
        got = enc.forward_stage(*inputs(pos256, sl), stage).cpu().numpy()
        assert np.array_equal(got.view(np.uint16), tr.stages[stage].view(np.uint16)), stage
    for stage, tol in ((4, 2e-3), (2, 4e-3), (3, 8e-3), (8, 3e-2)):
        got = enc.forward_stage(*inputs(pos256, sl), stage).cpu().numpy().astype(np.float32)
        want = tr.stages[stage].astype(np.float32)
        err = np.abs(got - want)
        assert np.isfinite(got).all()
        assert err.max() <= tol * max(1.0, np.abs(want).max()), (stage, err.max())
        if stage in (4, 2, 3):
            assert (err[live] == 0).mean() >= 0.98, (stage, (err[live] == 0).mean())
    enc.check_status()


# ---------------------------------------------------------------- accumulators
@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 0), ("A", 5), ("B", 7)])
def test_s32_accumulators_are_bit_exact(name, layer, encoders, oracle_weights, pos256):
    """Every weight GEMM of a layer: the captured A bytes times the packed s8 weights,
    recomputed on the host in int64, equals the captured tensor-core accumulators."""
    from brokefish_b200.nn.pack import qkv_chunk_rows
    enc = encoders[name]
    lw = oracle_weights[name].layers[layer]
    sl = slice(100, 133)            # 33 boards: a ragged last tile
    args = inputs(pos256, sl)
    perm = qkv_chunk_rows().reshape(-1)
    cases = [(0, lw.q_qkv[perm], False), (1, lw.q_o, False), (2, lw.q_ff1, False)]
    cases += [(3 + c, lw.q_ff2[:, 256 * c:256 * c + 256], True) for c in range(4)]
    for op, wq, unsigned in cases:
        a, acc = enc.capture_gemm(*args, layer=layer, op=op)
        a = a.cpu().numpy()
        a_int = a.astype(np.int64) if unsigned else a.view(np.int8).astype(np.int64)
        want = a_int @ wq.astype(np.int64).T
        assert np.array_equal(acc.cpu().numpy().astype(np.int64), want), (op,)
        assert a_int.any()
    enc.check_status()


@pytest.mark.parametrize("name", ["A", "B"])
def test_layer0_operands_equal_the_oracles(name, encoders, oracle_weights, pos256):
    """The quantised LN1 operand of layer 0 and its accumulators against the oracle's."""
    from brokefish_b200.nn.pack import qkv_chunk_rows
    enc = encoders[name]
    sl = slice(0, 16)
    tr = O.Trace()
    O.forward(oracle_weights[name], pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl],
              trace=tr, capture_layers=(0,))
    qa, acc = tr.gemms[(0, "qkv")]
    a, got = enc.capture_gemm(*inputs(pos256, sl), layer=0, op=0)
    assert np.array_equal(a.cpu().numpy().view(np.int8).astype(np.float32), qa)
    assert np.array_equal(got.cpu().numpy(), acc[:, qkv_chunk_rows().reshape(-1)])


# ---------------------------------------------------------------- outputs
@pytest.mark.parametrize("hw_rsqrt", [False, True])
@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_value_and_argmax(name, hw_rsqrt, encoders, encoders_hw, oracle_weights, pos256):
    enc = (encoders_hw if hw_rsqrt else encoders)[name]
    assert enc.exact_rsqrt == (not hw_rsqrt)
    w = aligned_oracle(oracle_weights, name, enc)
    sl = slice(0, 256)
    pol, pro, val = (t.cpu().numpy() for t in enc.forward_full(*inputs(pos256, sl)))
    enc.check_status()
    opol, opro, oval = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl])
    assert np.isfinite(pol.astype(np.float32)).all() and np.isfinite(val).all()
    tol = logit_tol(name, opol)
    assert np.abs(pol.astype(np.float32) - opol.astype(np.float32)).max() <= tol
    assert np.abs(pro.astype(np.float32) - opro.astype(np.float32)).max() <= tol
    assert np.abs(val - oval).max() <= VALUE_TOL
    legal = pos256["legal"][sl]
    mine, theirs = O.masked_argmax(pol, legal), O.masked_argmax(opol, legal)
    playable = theirs >= 0
    assert (mine[playable] == theirs[playable]).mean() >= ARGMAX_MIN[name]
    assert (mine[~playable] == -1).all()
    assert_disagreements_are_near_ties(opol, legal, mine, theirs, tol)


def test_against_reference_fp32_golden(encoders, pos256):
    """The reference's own bar for a quantised path: 8 % of max|logit| against its fp32
    network (tests/test_quant.py:342-356), on the committed reference outputs."""
    import os
    from conftest import GOLDEN
    for name in ("A", "B"):
        g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
        n = g["fp32_policy"].shape[0]
        pol, pro, val = (t.cpu().numpy() for t in encoders[name].forward_full(*inputs(pos256, slice(0, n))))
        top = np.abs(g["fp32_policy"]).max()
        assert np.abs(pol.astype(np.float32) - g["fp32_policy"]).max() <= 0.08 * top
        assert np.abs(pro.astype(np.float32) - g["fp32_promo"]).max() <= 0.08 * top
        assert np.abs(val - g["fp32_value"]).max() <= 0.08


def test_legal_mask_is_a_bitwise_select(encoders, pos256):
    enc = encoders["A"]
    sl = slice(0, 67)
    raw = enc.forward_full(*inputs(pos256, sl))[0].cpu().numpy()
    legal = pos256["legal"][sl]
    msk = enc.forward_full(*inputs(pos256, sl), legal=dev(legal.view(np.int64)))[0].cpu().numpy()
    bits = ((legal[:, :, None] >> np.arange(64, dtype=np.uint64)) & np.uint64(1)).astype(bool)
    assert np.array_equal(msk.view(np.uint16)[bits], raw.view(np.uint16)[bits])
    assert (msk.view(np.uint16)[~bits] == 0xFC00).all()


def test_deterministic_and_independent_of_batch_composition(encoders, pos256):
    """Same bytes on a repeat, and a position's outputs do not depend on which positions
    share its launch or its tile (the reference's tests/test_quant.py:309-339)."""
    enc = encoders["B"]
    full = [t.cpu().numpy().copy() for t in enc.forward_full(*inputs(pos256, slice(0, 256)))]
    again = [t.cpu().numpy().copy() for t in enc.forward_full(*inputs(pos256, slice(0, 256)))]
    for a, b in zip(full, again):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    for n in (1, 2, 3, 5, 31, 33, 127):
        part = [t.cpu().numpy() for t in enc.forward_full(*inputs(pos256, slice(7, 7 + n)))]
        for a, b in zip(full, part):
            assert np.array_equal(a[7:7 + n].view(np.uint8), b.view(np.uint8)), n
    enc.check_status()


def test_dead_slots_are_inert(encoders, pos256):
    """Rewriting a captured slot's word cannot happen (it is 0x800 by definition), but a
    dead token's *embedding inputs* must not reach live tokens: flipping rep/clock-free
    fields is not possible either, so the check is the reference's (tests/test_b2.py:
    270-293): outputs of live rows are unchanged when dead rows' words get other
    colour/type/square bits."""
    enc = encoders["A"]
    b = pos256["boards"][:64].copy()
    dead = ((b.view(np.uint16) >> 11) & 1) == 1
    assert dead.any()
    base = enc.forward_full(dev(b), dev(pos256["control"][:64]), dev(pos256["rep"][:64]))[0].cpu().numpy().copy()
    b2 = b.copy()
    b2.view(np.uint16)[dead] = 0x800 | 0x400 | (3 << 6) | 17
    got = enc.forward_full(dev(b2), dev(pos256["control"][:64]), dev(pos256["rep"][:64]))[0].cpu().numpy()
    assert np.array_equal(base.view(np.uint16)[~dead], got.view(np.uint16)[~dead])


def test_full_size_batch_properties(encoders, oracle_weights, pos4096):
    """Batch 4096 (the configuration the metric is quoted on): finite outputs, value in
    [-1, 1], equal to the same positions evaluated in small launches, and within
    tolerance of the oracle on a 384-position sample."""
    enc = encoders["A"]
    args = inputs(pos4096, slice(0, 4096))
    pol, pro, val = (t.cpu().numpy().copy() for t in enc.forward_full(*args))
    enc.check_status()
    assert np.isfinite(pol.astype(np.float32)).all() and np.isfinite(pro.astype(np.float32)).all()
    assert np.abs(val).max() <= 1.0
    for lo in (0, 1111, 4000):
        part = enc.forward_full(*inputs(pos4096, slice(lo, lo + 96)))[0].cpu().numpy()
        assert np.array_equal(part.view(np.uint16), pol[lo:lo + 96].view(np.uint16))
    idx = np.arange(0, 4096, 4096 // 384)[:384]
    w = aligned_oracle(oracle_weights, "A", enc)
    opol, _, oval = O.forward(w, pos4096["boards"][idx], pos4096["control"][idx], pos4096["rep"][idx])
    assert np.abs(pol[idx].astype(np.float32) - opol.astype(np.float32)).max() <= LOGIT_TOL
    assert np.abs(val[idx] - oval).max() <= VALUE_TOL
    legal = pos4096["legal"][idx]
    mine, theirs = O.masked_argmax(pol[idx], legal), O.masked_argmax(opol, legal)
    ok = theirs >= 0
    assert (mine[ok] == theirs[ok]).mean() >= ARGMAX_MIN["A"]
    assert_disagreements_are_near_ties(opol, legal, mine, theirs, LOGIT_TOL)


def test_largest_configured_batch_is_a_tiling_of_the_4096_batch(encoders_hw, pos4096):
    """131,072 positions in one launch (the largest step size of the configurations; the 4096
    fixture tiled 32 times, shifted by 5 positions so that copies straddle tiles differently):
    every copy's outputs equal the 4096-position launch's bit for bit — an evaluation does not
    depend on its index in the batch, on what shares its tile, or on the batch size."""
    enc = encoders_hw["A"]
    base = [t.clone() for t in enc.forward_full(*inputs(pos4096, slice(0, 4096)))]
    reps, shift = 32, 5
    big = []
    for key in ("boards", "control", "rep"):
        a = np.roll(pos4096[key], shift, axis=0)
        big.append(dev(np.concatenate([a] * reps, axis=0)))
    pol, pro, val = enc.forward_full(*big)
    enc.check_status()
    assert pol.shape[0] == 131072
    want = [torch.roll(t, shift, dims=0) for t in base]
    for k in (0, 1, 17, 31):
        lo = 4096 * k
        assert torch.equal(pol[lo:lo + 4096].view(torch.int16), want[0].view(torch.int16))
        assert torch.equal(pro[lo:lo + 4096].view(torch.int16), want[1].view(torch.int16))
        assert torch.equal(val[lo:lo + 4096].view(torch.int32), want[2].view(torch.int32))
    # a checksum over all copies: the remaining 28 agree with the first as well
    folded = pol.view(torch.int16).to(torch.int32).reshape(reps, -1)
    assert bool((folded == folded[0]).all())


@pytest.mark.parametrize("plan", [1, 2, 0])
@pytest.mark.parametrize("pinned", [True, False])
def test_end_to_end_host_call_matches_device_call(pinned, plan, encoders, pos4096):
    """Pinned and pageable host buffers; more positions than one wave (592 on a 148-SM part) and
    not a multiple of it, so that several launches and their overlapped copies run.  Both ways of
    splitting the batch (1: shrinking launches, largest first; 2: equal launches with the last
    wave written straight into pinned buffers) and the automatic choice give the device call's
    bits."""
    enc = encoders["A"]
    enc.set_host_plan(plan)
    n = 2500 if plan == 2 else 1500
    pin = (lambda t: t.pin_memory()) if pinned else (lambda t: t)
    b = pin(torch.from_numpy(pos4096["boards"][:n].copy()))
    c = pin(torch.from_numpy(pos4096["control"][:n].copy()))
    r = pin(torch.from_numpy(pos4096["rep"][:n].copy()))
    pol = pin(torch.zeros(n, 32, 64, dtype=torch.half))
    pro = pin(torch.zeros(n, 32, 4, dtype=torch.half))
    val = pin(torch.zeros(n, dtype=torch.float))
    enc.forward_host(b, c, r, pol, pro, val)
    enc.set_host_plan(0)
    dpol, dpro, dval = (t.cpu() for t in enc.forward_full(b.cuda(), c.cuda(), r.cuda()))
    assert torch.equal(pol.view(torch.int16), dpol.view(torch.int16))
    assert torch.equal(pro.view(torch.int16), dpro.view(torch.int16))
    assert torch.equal(val, dval)
    assert enc.host_link_gbps > 0.0
    assert sum(enc.host_plan(n)) == n


def test_value_head_variants(pos256):
    """Win/draw/loss rows and the pooled head (the reference's tests/test_b2.py:404-690)."""
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import BrokefishNet, seeded_state
    for nv, head in ((3, "king"), (1, "pooled"), (3, "pooled"), (1, "prenorm"), (3, "prenorm")):
        st = seeded_state(seed=5, std=None, perturb_norms=True, n_value=nv, value_head=head)
        net = BrokefishNet(n_value=nv, value_head=head).eval()
        net.load_state_dict(st)
        enc = encoder_impl("cuda")(net, int8=True)
        enc.exact_rsqrt = True
        w = O.prepare({k: v.numpy() for k, v in st.items()})
        sl = slice(0, 48)
        val = enc.forward_full(*inputs(pos256, sl))[2].cpu().numpy()
        oval = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl])[2]
        assert np.abs(val - oval).max() <= 2e-2, (nv, head)
        enc.close()


def test_input_rejection_and_empty_batch(encoders):
    enc = encoders["A"]
    z = torch.zeros(0, 32, dtype=torch.int16, device="cuda")
    p, pr, v = enc.forward_full(z, torch.zeros(0, dtype=torch.int16, device="cuda"),
                                torch.zeros(0, dtype=torch.uint8, device="cuda"))
    assert p.shape == (0, 32, 64) and v.shape == (0,)
    b = torch.zeros(2, 32, dtype=torch.int16)
    with pytest.raises(ValueError):
        enc.forward_full(b, torch.ones(2, dtype=torch.int16), torch.zeros(2, dtype=torch.uint8))
    with pytest.raises(ValueError):
        enc.forward_stage(b.cuda(), torch.ones(2, dtype=torch.int16, device="cuda"),
                          torch.zeros(2, dtype=torch.uint8, device="cuda"), 42)


def test_phase_profile_hooks(encoders, pos256):
    """The in-kernel phase clock: off by default, sums cycles per phase when on, and leaves
    the outputs untouched (the reference's bench/bench_phases.py protocol)."""
    enc = encoders["A"]
    args = inputs(pos256, slice(0, 256))
    base = enc.forward_full(*args)[0].cpu().numpy().copy()
    enc.set_profile(True)
    got = enc.forward_full(*args)[0].cpu().numpy().copy()
    prof = enc.read_profile()
    enc.set_profile(False)
    assert np.array_equal(base.view(np.uint16), got.view(np.uint16))
    assert set(prof) >= {"layernorm_quantise", "wait_mma_ff1", "attention", "ff1_epilogue", "heads"}
    assert all(v >= 0 for v in prof.values()) and prof["ff1_epilogue"] > 0 and prof["attention"] > 0
    enc.check_status()


@pytest.mark.parametrize("mode", ["ln1", "both"])
def test_reinjection(mode, pos256):
    """Per-layer input re-injection (the reference's tests/test_b2.py:734-754): layer-0 LN1
    output and Q/K/V bit-identical to the oracle, logits within the relative tolerance, and with
    all-zero coefficients bit-identical to the same network without injection, odd batch."""
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import net_for_state, seeded_state
    st = seeded_state(seed=7, std=None, perturb_norms=True, reinject=mode)
    net = net_for_state(st).eval()
    net.load_state_dict(st)
    enc = encoder_impl("cuda")(net, int8=True)
    enc.exact_rsqrt = True
    assert enc.rj_mode == {"ln1": 1, "both": 2}[mode]
    w = aligned_oracle({"X": O.prepare({k: v.numpy() for k, v in st.items()})}, "X", enc)
    sl = slice(0, 48)
    tr = O.Trace()
    opol, _, oval = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl], trace=tr)
    for stage in (1, 5, 6, 7):
        got = enc.forward_stage(*inputs(pos256, sl), stage).cpu().numpy()
        assert np.array_equal(got.view(np.uint16), tr.stages[stage].view(np.uint16)), stage
    pol, _, val = (t.cpu().numpy() for t in enc.forward_full(*inputs(pos256, sl)))
    assert np.abs(pol.astype(np.float32) - opol.astype(np.float32)).max() <= logit_tol("B", opol)
    assert np.abs(val - oval).max() <= 3e-2
    enc.check_status()
    enc.close()
    # zero coefficients == no injection, bit for bit, on an odd batch
    st0 = {k: (torch.zeros_like(v) if k == "reinject_c" else v) for k, v in st.items()}
    net0 = net_for_state(st0).eval()
    net0.load_state_dict(st0)
    plain_state = {k: v for k, v in st0.items() if not k.startswith("reinject")}
    plain = net_for_state(plain_state).eval()
    plain.load_state_dict(plain_state)
    e0, e1 = encoder_impl("cuda")(net0, int8=True), encoder_impl("cuda")(plain, int8=True)
    odd = slice(3, 3 + 131)
    a = [t.cpu().numpy().copy() for t in e0.forward_full(*inputs(pos256, odd))]
    b = [t.cpu().numpy().copy() for t in e1.forward_full(*inputs(pos256, odd))]
    for x, y in zip(a, b):
        assert np.array_equal(x.view(np.uint8), y.view(np.uint8))
    e0.close()
    e1.close()


@pytest.mark.parametrize("name", ["A", "B"])
def test_e4m3_ffn_arithmetic(name, nets, states, pos256):
    """`FusedEncoder(net, fp8=True)`: FFN in e4m3 (amax/8 scales), QKV and out-projection in
    fp16.  LN1 output is bit-identical to the oracle; everything after the first fp16 GEMM is a
    tolerance (e4m3 steps are 6-12 % of a value, so two implementations that differ in one
    rounding drift further apart than in int8): logits within 8 % of max|logit| of the e4m3
    oracle (measured 6.0 % on set A, less on B) and within 12 % of the reference fp32 network (the reference's own e4m3 emulation is
    7-8 % from fp32 on these weights)."""
    import os
    from conftest import GOLDEN
    from brokefish_b200.nn import encoder_impl
    enc = encoder_impl("cuda")(nets[name], fp8=True)
    enc.exact_rsqrt = True
    assert enc.quant == 1 and enc.label.startswith("e4m3")
    w = O.prepare({k: v.numpy() for k, v in states[name].items()}, fmt="e4m3")
    sl = slice(0, 64)
    tr = O.Trace()
    opol, opro, oval = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl], trace=tr)
    got = enc.forward_stage(*inputs(pos256, sl), 1).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), tr.stages[1].view(np.uint16))
    for stage in (5, 6, 7, 4):
        got = enc.forward_stage(*inputs(pos256, sl), stage).cpu().numpy().astype(np.float32)
        want = tr.stages[stage].astype(np.float32)
        assert np.abs(got - want).max() <= 4e-3 * max(1.0, np.abs(want).max()), stage
    pol, pro, val = (t.cpu().numpy() for t in enc.forward_full(*inputs(pos256, sl)))
    enc.check_status()
    top = float(np.abs(opol.astype(np.float32)).max())
    assert np.isfinite(pol.astype(np.float32)).all()
    assert np.abs(pol.astype(np.float32) - opol.astype(np.float32)).max() <= 0.08 * top
    assert np.abs(val - oval).max() <= 0.08
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    assert np.abs(pol.astype(np.float32) - g["fp32_policy"]).max() <= 0.12 * np.abs(g["fp32_policy"]).max()
    # deterministic, and independent of what shares the launch
    again = enc.forward_full(*inputs(pos256, sl))[0].cpu().numpy()
    assert np.array_equal(again.view(np.uint16), pol.view(np.uint16))
    part = enc.forward_full(*inputs(pos256, slice(5, 5 + 33)))[0].cpu().numpy()
    assert np.array_equal(part.view(np.uint16), pol[5:5 + 33].view(np.uint16))
    with pytest.raises(NotImplementedError):
        enc.capture_gemm(*inputs(pos256, slice(0, 4)), layer=0, op=0)
    enc.close()


def test_divergence_report(encoders, encoders_hw, oracle_weights, pos256):
    """Not a bar: prints, layer by layer, how far the kernel and the numpy oracle are apart
    (`pytest tests/test_gpu_parity.py -m gpu -s -k divergence_report`), for both 1/sqrt modes.
    Stage 4 = attention output, 2 = residual after the attention block, 10 = residual at the end
    of the layer."""
    sl = slice(0, 256)
    for mode, encs in (("correctly rounded 1/sqrt", encoders), ("hardware 1/sqrt", encoders_hw)):
        enc = encs["A"]
        w = aligned_oracle(oracle_weights, "A", enc)
        tr = O.Trace()
        opol, _, oval = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl], trace=tr)
        print(f"\nset A, {mode}: layer | stage 4 max / exact | stage 2 max / exact | stage 10 max / exact")
        for layer in range(8):
            cells = []
            for stage in (4, 2, 10):
                got = enc.forward_stage(*inputs(pos256, sl), stage, layer=layer).cpu().numpy()
                want = tr.by_layer[(layer, stage)].reshape(got.shape)
                d = np.abs(got.astype(np.float32) - want.astype(np.float32)).max()
                same = (got.view(np.uint16) == want.view(np.uint16)).mean()
                cells.append(f"{d:.4f} / {same:.4f}")
            print(f"  {layer} | " + " | ".join(cells))
        pol, _, val = (t.cpu().numpy() for t in enc.forward_full(*inputs(pos256, sl)))
        d = np.abs(pol.astype(np.float32) - opol.astype(np.float32))
        same = (pol.view(np.uint16) == opol.view(np.uint16)).mean()
        am, ao = O.masked_argmax(pol, pos256["legal"][sl]), O.masked_argmax(opol, pos256["legal"][sl])
        ok = ao >= 0
        print(f"  logits max {d.max():.4f}, {same:.3f} bit-identical, value max {np.abs(val - oval).max():.4f}, "
              f"masked argmax {(am[ok] == ao[ok]).sum()} / {ok.sum()}")


def test_int8_peak_probe_runs_and_is_plausible():
    """The tcgen05 kind::i8 loop used as the roofline's measured denominator: runs clean and
    lands between half of and a little above the nominal dense int8 rate (4500 TOP/s)."""
    from brokefish_b200 import _native
    tops, ms = ctypes.c_double(0), ctypes.c_double(0)
    rc = _native.lib().bf_measure_i8_peak(0, 4096, ctypes.byref(tops), ctypes.byref(ms))
    assert rc == 0, _native.lib().bf_last_error()
    assert 2000.0 < tops.value < 5500.0, (tops.value, ms.value)
    assert _native.lib().bf_measure_i8_peak(0, 1, ctypes.byref(tops), None) != 0     # iters out of range


def test_elementwise_probe_gives_the_cuda_core_roof():
    """The second roof: the row warps' own element-wise functions in isolation.  The ff1
    epilogue is the slowest block per element, the norm statistics the fastest, and the time
    they imply for a 4096-position launch is below the launch's measured time."""
    from brokefish_b200 import _native
    L = _native.lib()
    rate = {}
    for block in range(6):
        eps, ms = ctypes.c_double(0), ctypes.c_double(0)
        assert L.bf_measure_elementwise(0, block, 2000, ctypes.byref(eps), ctypes.byref(ms)) == 0, L.bf_last_error()
        rate[block] = eps.value / 1e9 / 148                    # elements per ns per SM
        assert 3.0 < rate[block] < 400.0, (block, rate[block], ms.value)
    # (relations between timings are held to a margin: a shared GPU's clocks move)
    assert rate[0] < 1.15 * min(rate.values()) and rate[3] > 0.85 * max(rate.values()), rate
    widths = {0: 1024, 1: 1024, 2: 1024, 3: 512, 4: 512, 5: 256}
    floor_ms = sum(4096 * 8 * 32 * w / (rate[b] * 148 * 1e9) for b, w in widths.items()) * 1e3
    print(f"\nelements/ns/SM {dict((b, round(r, 1)) for b, r in rate.items())}; floor for 4096 positions {floor_ms:.3f} ms")
    assert 0.4 < floor_ms < 2.0
    # the ff1 epilogue with 8 and with 32 warps per SM: sixteen are within 10 % of thirty-two
    for block in (6, 7):
        assert L.bf_measure_elementwise(0, block, 2000, ctypes.byref(eps), None) == 0, L.bf_last_error()
        rate[block] = eps.value / 1e9 / 148
    print(f"ff1 epilogue, elements/ns/SM at 8 / 16 / 32 warps: {rate[6]:.1f} / {rate[0]:.1f} / {rate[7]:.1f}")
    assert rate[6] < rate[0] * 1.15 and rate[0] > 0.8 * rate[7], rate
    # the cheaper, not bit-exact forms of the ff1 epilogue, the normalise + quantise, the descale
    # and the ff2 step (blocks 8-11): what a tolerance arm could save on the CUDA cores at most
    for block in (8, 9, 10, 11):
        assert L.bf_measure_elementwise(0, block, 2000, ctypes.byref(eps), None) == 0, L.bf_last_error()
        rate[block] = eps.value / 1e9 / 148
    cheap = {8: 1024, 10: 1024, 11: 1024, 3: 512, 9: 512, 5: 256}
    cheap_ms = sum(4096 * 8 * 32 * w / (rate[b] * 148 * 1e9) for b, w in cheap.items()) * 1e3
    print(f"cheaper forms, elements/ns/SM: ff1 {rate[8]:.1f} (exact {rate[0]:.1f}), normalise+quantise {rate[9]:.1f} "
          f"({rate[4]:.1f}), descale {rate[10]:.1f} ({rate[1]:.1f}), ff2 {rate[11]:.1f} ({rate[2]:.1f}); "
          f"floor {cheap_ms:.3f} ms against {floor_ms:.3f} ms")
    assert rate[8] > 0.9 * rate[0] and rate[9] > 0.9 * rate[4] and cheap_ms < 1.1 * floor_ms, rate
    assert L.bf_measure_elementwise(0, 12, 100, ctypes.byref(eps), None) != 0
    assert L.bf_measure_elementwise(0, 0, 0, ctypes.byref(eps), None) != 0


def test_a_wait_that_nothing_satisfies_times_out_and_reports():
    """Failure detection without a fault: the bounded wait gives up after its limit, the kernel
    returns, the status word carries the code, a later waiter returns at once, and the device
    keeps working afterwards."""
    from brokefish_b200 import _native
    L = _native.lib()
    status = ctypes.c_int(0)
    waited = (ctypes.c_longlong * 2)()
    assert L.bf_selftest_timeout(0, 7, ctypes.byref(status), waited) == 0, L.bf_last_error()
    assert status.value == 7
    assert waited[0] >= 400_000_000 and waited[0] < 4_000_000_000      # the limit, not forever
    assert waited[1] < 10_000_000                                      # the second waiter saw the flag
    assert L.bf_selftest_timeout(0, 0, ctypes.byref(status), None) != 0
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0


def test_fp16_arithmetic_against_the_oracle_and_the_fp32_network(nets, states, pos256):
    """`FusedEncoder(net, int8=False)` against the oracle's fp16 restatement (same roundings up
    to the hardware's exp and the order inside a tensor-core step): logits within 1 % of
    max|logit|; and within 1 % of the reference fp32 network's committed outputs (fp16 arithmetic
    has no quantisation noise)."""
    import os
    from conftest import GOLDEN
    from brokefish_b200.nn import encoder_impl
    enc = encoder_impl("cuda")(nets["A"], int8=False)
    enc.exact_rsqrt = True
    w = O.prepare({k: v.numpy() for k, v in states["A"].items()}, fmt="f16")
    sl = slice(0, 64)
    tr = O.Trace()
    opol, opro, oval = O.forward(w, pos256["boards"][sl], pos256["control"][sl], pos256["rep"][sl], trace=tr)
    got = enc.forward_stage(*inputs(pos256, sl), 1).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), tr.stages[1].view(np.uint16))
    pol, pro, val = (t.cpu().numpy() for t in enc.forward_full(*inputs(pos256, sl)))
    enc.check_status()
    top = float(np.abs(opol.astype(np.float32)).max())
    assert np.abs(pol.astype(np.float32) - opol.astype(np.float32)).max() <= 0.01 * max(1.0, top)
    assert np.abs(val - oval).max() <= 5e-3
    g = np.load(os.path.join(GOLDEN, "ref_outputs_A.npz"))
    n = g["fp32_policy"].shape[0]
    assert np.abs(pol[:n].astype(np.float32) - g["fp32_policy"]).max() <= 0.01 * np.abs(g["fp32_policy"]).max()
    # determinism and independence of what shares the launch
    a = enc.forward_full(*inputs(pos256, slice(5, 5 + 33)))[0].cpu().numpy().copy()
    b = enc.forward_full(*inputs(pos256, slice(0, 64)))[0].cpu().numpy()[5:38]
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    enc.close()


def test_the_parity_checks_bite(nets, pos256):
    """A validator nobody has watched fail is an assertion, not a measurement (the reference's
    tests/test_validate.py): flip one weight byte, one scale bit or one bias bit in the packed
    blob and the outputs must move; an untouched copy of the blob must reproduce them exactly."""
    import struct
    from brokefish_b200.nn.cuda_impl import FusedEncoder
    from brokefish_b200.nn.pack import pack_blob
    blob = pack_blob(nets["A"])
    args = inputs(pos256, slice(0, 64))
    base_enc = FusedEncoder.from_blob(blob.copy())
    base = [t.clone() for t in base_enc.forward_full(*args)]
    base_enc.close()
    off_w, bytes_w, off_lp = struct.unpack_from("<QQQ", blob, 32)
    mutants = {"weight byte, layer 5": off_w + 5 * 786432 + 123457,
               "weight scale, layer 2 ff1": off_lp + 2 * 4736 + 32 + 2,
               "bias, layer 7 ff2": off_lp + 7 * 4736 + 4224 + 11}
    for what, at in mutants.items():
        m = blob.copy()
        m[at] ^= 0x10
        enc = FusedEncoder.from_blob(m)
        pol = enc.forward_full(*args)[0]
        assert not torch.equal(pol.view(torch.int16), base[0].view(torch.int16)), what
        enc.close()
    again = FusedEncoder.from_blob(blob.copy())
    out = again.forward_full(*args)
    assert all(torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a.view(torch.int16),
                           b.view(torch.int32) if b.dtype == torch.float32 else b.view(torch.int16))
               for a, b in zip(out, base))
    again.close()
