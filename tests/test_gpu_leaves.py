"""The compacted leaf list interface (C ABI bf_forward_leaves, FusedEncoder.forward_leaves):
positions named by an index list whose length lives in device memory.  What it must do: give
each listed position the bits the dense call gives it, at the position's own place; touch no
other place; honour a count the host never saw; run short when the list is short."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def enc():
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import BrokefishNet, seeded_state
    net = BrokefishNet().eval()
    net.load_state_dict(seeded_state(seed=0, std=None, perturb_norms=True))
    e = encoder_impl("cuda")(net, int8=True)
    yield e
    e.check_status()
    e.close()


def staged(pos, n):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a[:n])).cuda()
    legal = torch.from_numpy(pos["legal"][:n].view(np.int64).copy()).cuda()
    return t(pos["boards"]), t(pos["control"]), t(pos["rep"]), legal


def test_listed_positions_get_the_dense_call_s_bits_at_their_own_place(enc, pos4096):
    n = 1000
    boards, control, rep, _ = staged(pos4096, n)
    want = [x.clone() for x in enc.forward_full(boards, control, rep)]
    g = torch.Generator().manual_seed(3)
    for k in (333, 1, 4, 1000):
        idx = torch.randperm(n, generator=g)[:k].to(torch.int32).cuda()
        count = torch.tensor([k], dtype=torch.int32, device="cuda")
        enc.policy_out.fill_(float("nan")); enc.promo_out.fill_(float("nan")); enc.value_out.fill_(float("nan"))
        pol, pro, val = enc.forward_leaves(boards, control, rep, idx, count)
        sel = idx.long()
        assert torch.equal(pol[sel].view(torch.int16), want[0][sel].view(torch.int16))
        assert torch.equal(pro[sel].view(torch.int16), want[1][sel].view(torch.int16))
        assert torch.equal(val[sel], want[2][sel])
        rest = torch.ones(n, dtype=torch.bool, device="cuda")
        rest[sel] = False
        assert torch.isnan(val[rest]).all() and torch.isnan(pol[rest].float()).all()


def test_the_count_is_read_on_the_device(enc, pos4096):
    """The count comes out of device work queued just before the launch (a reduction), is
    clamped to the list's capacity, and zero or a negative count evaluates nothing."""
    n = 512
    boards, control, rep, _ = staged(pos4096, n)
    want = enc.forward_full(boards, control, rep)[2].clone()
    idx = torch.arange(n - 1, -1, -1, dtype=torch.int32, device="cuda")
    active = torch.zeros(n, dtype=torch.bool, device="cuda")
    active[:77] = True
    count = torch.zeros(1, dtype=torch.int32, device="cuda")
    for expect, fill in ((77, None), (n, 10_000), (0, 0), (0, -5)):
        enc.value_out.fill_(float("nan"))
        if fill is None:
            count.copy_(active.sum().to(torch.int32))          # no .item(): the host never learns it
        else:
            count.fill_(fill)
        val = enc.forward_leaves(boards, control, rep, idx, count)[2]
        done = ~torch.isnan(val)
        assert int(done.sum()) == expect
        if expect:
            sel = idx[:expect].long()
            assert done[sel].all() and torch.equal(val[sel], want[sel])


def test_fused_expansion_over_a_leaf_list(enc, pos4096):
    n = 777
    boards, control, rep, legal = staged(pos4096, n)
    want = [x.clone() for x in enc.forward_priors(boards, control, rep, legal, 64)]
    idx = torch.arange(0, n, 3, dtype=torch.int32, device="cuda")
    count = torch.tensor([idx.numel() - 2], dtype=torch.int32, device="cuda")
    for lg in (legal, None):
        enc.prior_out.fill_(float("nan")); enc.nedges_out.fill_(-1)
        pri, mov, ne, val = enc.forward_leaves(boards, control, rep, idx, count, legal=lg, e_cap=64)
        sel = idx[:-2].long()
        assert torch.equal(pri[sel].view(torch.int16), want[0][sel].view(torch.int16))
        assert torch.equal(mov[sel], want[1][sel]) and torch.equal(ne[sel], want[2][sel])
        assert torch.equal(val[sel], want[3][sel])
        assert (ne[idx[-2:].long()] == -1).all() and (ne[1::3] == -1).all()


def test_a_short_list_runs_short(enc, pos4096):
    """128 live leaves of a 4096-place staging area against the dense call on all 4096: the
    reference's evaluator would cost the full batch either way."""
    n = 4096
    boards, control, rep, _ = staged(pos4096, n)
    idx = torch.randperm(n, generator=torch.Generator().manual_seed(0)).to(torch.int32).cuda()
    count = torch.tensor([128], dtype=torch.int32, device="cuda")

    def time_ms(fn):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 10

    dense = time_ms(lambda: enc.forward_full(boards, control, rep))
    short = time_ms(lambda: enc.forward_leaves(boards, control, rep, idx, count))
    count.fill_(4096)
    full = time_ms(lambda: enc.forward_leaves(boards, control, rep, idx, count))
    print(f"\ndense 4096: {dense:.3f} ms; leaf list 128 of 4096: {short:.3f} ms; leaf list 4096 (permuted): {full:.3f} ms")
    assert short < 0.4 * dense and full < 1.25 * dense


def test_wrong_arguments_are_refused(enc, pos4096):
    boards, control, rep, _ = staged(pos4096, 16)
    idx = torch.arange(16, dtype=torch.int32, device="cuda")
    count = torch.tensor([16], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        enc.forward_leaves(boards, control, rep, idx.long(), count)
    with pytest.raises(ValueError):
        enc.forward_leaves(boards, control, rep, idx, count.long())
    with pytest.raises(ValueError):
        enc.forward_leaves(boards, control, rep, torch.arange(17, dtype=torch.int32, device="cuda"), count)
    with pytest.raises(ValueError):
        enc.forward_leaves(boards, control, rep, idx.cpu(), count)
