"""The backbone-only entry (C ABI bf_forward_backbone, FusedEncoder.forward / __call__):
activations in, the residual stream after the last layer out, always on the fp16 arithmetic
(brokefish/nn/cuda_impl.py:447-463; csrc/encoder.cu:1752-1767)."""
import numpy as np
import pytest
import torch

from oracle import ref_kernel as R

pytestmark = pytest.mark.gpu

SET_A = dict(seed=0, std=0.02, perturb_norms=False)


def make(state_kw, **enc_kw):
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import net_for_state, seeded_state
    st = seeded_state(**state_kw)
    net = net_for_state(st).eval()
    net.load_state_dict(st)
    return net, encoder_impl("cuda")(net, **enc_kw)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def case(pos256):
    n = 203
    boards, control, rep = dev(pos256["boards"][:n]), dev(pos256["control"][:n]), dev(pos256["rep"][:n])
    alive = ((boards.to(torch.int32) >> 11) & 1) == 0
    net, enc = make(SET_A, int8=False)
    x = enc.forward_stage(boards, control, rep, 9).clone()                   # the embedding
    want = enc.forward_stage(boards, control, rep, 10, layer=7).clone()      # residual after layer 7
    yield dict(net=net, enc=enc, x=x, alive=alive, want=want, boards=boards, control=control, rep=rep)
    enc.check_status()
    enc.close()


def same(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_backbone_continues_the_embedding_to_the_last_layer_s_residual(case):
    """Fed the embedding of real boards and their alive flags, the backbone gives the bits the
    boards-in call has in its residual stream after the last layer; in place too."""
    enc, x, alive, want = case["enc"], case["x"], case["alive"], case["want"]
    got = enc(x, alive)
    assert got.shape == x.shape and got.dtype is torch.half and same(got, want)
    assert same(enc.forward(x, alive.view(torch.int8)), want)
    buf = x.clone()
    assert enc.forward(buf, alive, out=buf) is buf and same(buf, want)
    # a ragged batch and an empty one
    assert same(enc(x[:5], alive[:5]).clone(), want[:5])
    assert enc(x[:0], alive[:0]).shape == (0, 32, 256)


def test_alive_flags_only_mask_keys(case):
    """Without flags every token is a key: the answer changes on boards with captured pieces
    and stays on boards without."""
    enc, x, alive, want = case["enc"], case["x"], case["alive"], case["want"]
    everyone = enc(x, None).clone()
    assert same(everyone, enc(x, torch.ones_like(alive)).clone())
    full = alive.all(dim=1)
    assert full.any() and (~full).any()
    assert same(everyone[full], want[full])
    assert not same(everyone[~full], want[~full])


def test_other_sources_reach_the_same_bits(case):
    """An int8 instance packs an fp16 handle on first use (the reference keeps its fp16 slab
    beside the quantised ones); a bare nn.TransformerEncoder is a valid source for this entry
    and for nothing else."""
    from brokefish_b200.nn import encoder_impl
    x, alive, want, net = case["x"], case["alive"], case["want"], case["net"]
    e8 = encoder_impl("cuda")(net, int8=True)
    assert e8.quant == 3 and same(e8(x, alive), want)
    pol = e8.forward_full(case["boards"], case["control"], case["rep"])[0]
    assert torch.isfinite(pol.float()).all()                 # its own arithmetic still runs
    e8.close()
    bare = encoder_impl("cuda")(net.encoder)
    assert same(bare(x, alive), want)
    with pytest.raises(ValueError):
        bare.forward_full(case["boards"], case["control"], case["rep"])
    bare.close()


def test_against_torch_fp32_stack(case):
    """nn.TransformerEncoder in fp32 on the CPU with the same weights and key mask: the fp16
    kernel stays within 1 % of the largest activation on live rows."""
    x, alive, net = case["x"][:64], case["alive"][:64], case["net"]
    got = case["enc"](x, alive).float().cpu()
    with torch.no_grad():
        ref = net.encoder(x.float().cpu(), src_key_padding_mask=~alive.cpu())
    live = alive.cpu()
    err = (got - ref)[live].abs().max().item()
    scale = ref[live].abs().max().item()
    print(f"\nbackbone vs torch fp32: max|d| {err:.4f} of max|x| {scale:.3f}")
    assert err <= 0.01 * scale                                # tolerance: 1 % of max |activation|


@pytest.mark.skipif(not R.available("A_f16"), reason="oracle/_ref not built")
def test_bit_identical_to_the_reference_kernel_s_backbone_entry(case):
    ref = R.RefKernel("A_f16")
    x, alive = case["x"], case["alive"]
    for a in (alive.view(torch.int8), None):
        want = ref.encoder_forward(x, a)
        torch.cuda.synchronize()
        assert same(case["enc"](x, None if a is None else alive).clone(), want)


def test_refusals(case):
    enc, x, alive = case["enc"], case["x"], case["alive"]
    with pytest.raises(ValueError):
        enc(x[:, :, :128], alive)
    with pytest.raises(ValueError):
        enc(x.float(), alive)
    with pytest.raises(ValueError):
        enc(x, alive[:3])
    with pytest.raises(ValueError):
        enc(x, alive.float())
    with pytest.raises(ValueError):
        enc(x.cpu(), None)
    # the C entry refuses a handle that carries another arithmetic
    import ctypes
    from brokefish_b200 import _native
    from brokefish_b200.nn import encoder_impl
    e8 = encoder_impl("cuda")(case["net"], int8=True)
    rc = _native.lib().bf_forward_backbone(e8._handle, ctypes.c_void_p(x.data_ptr()), None, 4,
                                           ctypes.c_void_p(x.clone().data_ptr()), None)
    assert rc != 0 and b"fp16" in _native.lib().bf_last_error()
    e8.close()
