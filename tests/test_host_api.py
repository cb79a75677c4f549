"""Host-side behaviour of the reference-facing Python surface that needs no GPU."""
import numpy as np
import pytest
import torch

from brokefish_b200.nn import encoder_impl, available, why_unavailable, IMPLEMENTATIONS
from brokefish_b200.nn.cuda_impl import FusedEncoder, SCHEMES, SCHEME
from brokefish_b200.nn.model import BrokefishNet, net_for_state, seeded_state
from brokefish_b200.nn import quant
from brokefish_b200.evaluator import make_evaluator, shard_bounds


def test_registry():
    assert IMPLEMENTATIONS == ("cuda",)
    assert encoder_impl("cuda") is FusedEncoder
    with pytest.raises(ValueError):
        encoder_impl("triton")
    got = available()
    assert got in ([], ["cuda"])
    if not got:
        assert "cuda" in why_unavailable()
    assert SCHEMES[SCHEME] == 3


def test_constructor_refusals(nets):
    net = nets["A"]
    with pytest.raises(ValueError):
        FusedEncoder(net, acc_dtype="bf16")
    with pytest.raises(NotImplementedError):
        FusedEncoder(net, acc_dtype="fp32")
    with pytest.raises(ValueError):
        FusedEncoder(net, fp8=True, int8=True)
    with pytest.raises(ValueError):
        FusedEncoder(net, int8_scheme="nope")
    with pytest.raises(ValueError):
        FusedEncoder(BrokefishNet(d_ff=512))
    # a bare encoder stack is accepted but has no boards->logits path
    bare = FusedEncoder(net.encoder)
    z = torch.zeros(1, 32, dtype=torch.int16)
    with pytest.raises(ValueError):
        bare.forward_full(z, torch.ones(1, dtype=torch.int16), torch.zeros(1, dtype=torch.uint8))
    with pytest.raises(ValueError):
        bare(torch.zeros(1, 32, 256))                       # the backbone entry takes CUDA fp16 tensors
    with pytest.raises(ValueError):
        bare(torch.zeros(1, 32, 128))


def test_input_checks():
    chk = FusedEncoder._check_inputs
    b = torch.zeros(3, 32, dtype=torch.int16)
    c = torch.ones(3, dtype=torch.int16)
    r = torch.zeros(3, dtype=torch.uint8)
    assert chk(b, c, r) == 3
    for bad in ((b[:, :31], c, r), (b.int(), c, r), (b, c[:2], r), (b, c.int(), r), (b, c, r.int())):
        with pytest.raises(ValueError):
            chk(*bad)


def test_model_mirror_matches_reference_fp32_outputs(nets, pos256):
    import os
    from conftest import GOLDEN
    for name in ("A", "B"):
        g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
        n = g["fp32_policy"].shape[0]
        ev = make_evaluator(nets[name], None)
        with torch.no_grad():
            p, pr, v = ev(torch.from_numpy(pos256["boards"][:n]), torch.from_numpy(pos256["control"][:n]),
                          torch.from_numpy(pos256["rep"][:n]))
        assert np.abs(p.numpy() - g["fp32_policy"]).max() < 1e-4
        assert np.abs(pr.numpy() - g["fp32_promo"]).max() < 1e-4
        assert np.abs(v.numpy() - g["fp32_value"]).max() < 1e-4


def test_state_dict_round_trip_and_variants():
    st = seeded_state(seed=3, n_value=3, value_head="pooled")
    net = net_for_state(st)
    net.load_state_dict(st)
    assert net.n_value == 3 and net.value_head == "pooled" and net.value_absolute
    with pytest.raises(ValueError):
        BrokefishNet(n_value=2)
    with pytest.raises(NotImplementedError):
        BrokefishNet(rule_features=True)
    rj = seeded_state(seed=3, reinject="both")
    assert rj["reinject_c"].shape == (16, 5) and int(rj["reinject_mode"]) == 2
    assert net_for_state(rj).reinject == "both" and net_for_state(rj).n_sites == 16


def test_scheme_functions_against_reference_answers():
    import os
    from conftest import GOLDEN
    k = np.load(os.path.join(GOLDEN, "scheme_kats.npz"))
    qb, sc = quant.quantise_weights_int8_bytes(torch.from_numpy(k["w"]))
    assert np.array_equal(qb.numpy(), k["w_q"]) and np.array_equal(sc.numpy(), k["w_s"])
    q, s = quant.quantise_activations_int8(torch.from_numpy(k["acts"]))
    assert np.array_equal(q.numpy(), k["q_s8"]) and np.array_equal(s.numpy(), k["s_s8"])
    q, s = quant.quantise_activations_int8(torch.from_numpy(k["acts"]).relu(), unsigned=True)
    assert np.array_equal(q.numpy(), k["q_u8"]) and np.array_equal(s.numpy(), k["s_u8"])
    lin = quant.int8_linear(torch.from_numpy(k["acts"]), torch.from_numpy(k["w"]), torch.linspace(-1, 1, 256))
    assert np.array_equal(lin.numpy(), k["lin"])
    assert (quant.Q_MAX_S8, quant.Q_MAX_U8) == tuple(k["q_max"])
    with pytest.raises(ValueError):
        quant.quantise_weights_int8_bytes(torch.zeros(100, 256))


def test_shard_bounds():
    for n in (0, 1, 7, 4096, 131072):
        for world in (1, 2, 3, 8):
            cuts = [shard_bounds(n, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


class _Twin(torch.nn.Module):
    """A module with the reference network's parts that is NOT this package's class: what
    ``FusedEncoder`` sees when a trainer hands it the reference's own ``BrokefishNet``."""

    def __init__(self, src):
        super().__init__()
        import copy
        for part in ("encoder", "norm_f", "policy", "promo", "value", "emb_square", "emb_type_special",
                     "emb_color_turn", "emb_clock", "emb_rep"):
            setattr(self, part, copy.deepcopy(getattr(src, part)))
        self.d_model, self.n_layers, self.n_value = src.d_model, src.n_layers, src.n_value
        self.value_head, self.reinject = src.value_head, src.reinject


def test_network_is_recognised_by_its_parts_not_its_class(nets):
    """The constructor takes any module shaped like the reference's network (the class
    `PackedWeights.pack` passes is the reference's own, brokefish/train/sync.py:60-86), packs
    the same blob from it as from this package's container, from fp32 master weights and from
    the `.half()` copy alike (tests/test_b2.py:61-67), and keeps the reference's defaults:
    plain fp16 arithmetic unless `int8` or `fp8` is asked for."""
    import inspect
    from brokefish_b200.nn import pack
    from brokefish_b200.nn.cuda_impl import is_whole_network
    net = nets["B"]
    twin = _Twin(net)
    assert not isinstance(twin, BrokefishNet)
    assert is_whole_network(twin) and is_whole_network(net) and not is_whole_network(net.encoder)
    want = pack.pack_blob(net, "int8")
    assert np.array_equal(pack.pack_blob(twin, "int8"), want)
    half = _Twin(net).half()
    net_h = __import__("copy").deepcopy(net).half()
    assert np.array_equal(pack.pack_blob(half, "int8"), pack.pack_blob(net_h, "int8"))
    sig = inspect.signature(FusedEncoder.__init__).parameters
    assert sig["int8"].default is False and sig["fp8"].default is False and sig["acc_dtype"].default == "fp16"
    assert list(sig)[1:7] == ["source", "acc_dtype", "fp8", "int8", "two_boards", "int8_scheme"]
    if not torch.cuda.is_available():
        # recognised as a whole network: the constructor gets as far as asking for the device
        with pytest.raises(RuntimeError, match="CUDA device"):
            FusedEncoder(twin, int8=True)


def test_reference_network_packs_to_the_same_blob(states):
    """Where a checkout of the reference is at hand (``BROKEFISH_REFERENCE``, else a directory
    ``reference`` beside this repository), its own ``BrokefishNet`` -- fp32 and ``.half()`` --
    gives the blob bytes this package's container gives for the same state."""
    import os
    import sys
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("BROKEFISH_REFERENCE") or os.path.join(os.path.dirname(here), "reference")
    if not os.path.isdir(os.path.join(ref, "brokefish")):
        pytest.skip("no checkout of the reference here (BROKEFISH_REFERENCE)")
    sys.path.insert(0, ref)
    try:
        from brokefish.nn.model import BrokefishNet as RefNet
    finally:
        sys.path.remove(ref)
    from brokefish_b200.nn import pack
    from brokefish_b200.nn.cuda_impl import is_whole_network
    for name, fmt in (("A", "int8"), ("B", "int8"), ("B", "f16"), ("B", "e4m3")):
        theirs, ours = RefNet().eval(), BrokefishNet().eval()
        theirs.load_state_dict(states[name], strict=True)
        ours.load_state_dict(states[name], strict=True)
        assert is_whole_network(theirs)
        assert np.array_equal(pack.pack_blob(theirs, fmt), pack.pack_blob(ours, fmt))
        assert np.array_equal(pack.pack_blob(theirs.half(), fmt), pack.pack_blob(ours.half(), fmt))
