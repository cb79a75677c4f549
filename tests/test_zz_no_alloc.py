"""The entry point that allocates nothing (`bf_forward_noalloc`), through the C ABI.

It serves callers that are not allowed to allocate device memory while they run -- for
instance an evaluator embedded in a process whose GPU memory was handed out in advance --
so the weights stay in a buffer the caller already owns and the kernel's status word lives
in a small fixed array inside the library.  The check: on two calls in a row its three
outputs are bit-identical to those of the ordinary handle-based `bf_forward` on the same
inputs (same kernel, same arithmetic, so the tolerance is zero), and the shared status word
reads clean.  This file sorts last so that a run stopping at the first failure has already
run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_noalloc_entry_point_matches_the_handle_path_twice(nets, pos256):
    from brokefish_b200 import _native
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.pack import pack_blob

    L = _native.lib()
    dev = torch.device("cuda", 0)
    net = nets["B"]
    blob = torch.from_numpy(pack_blob(net)).to(dev)          # caller-owned device copy
    assert blob.data_ptr() % 256 == 0
    enc = encoder_impl("cuda")(net, int8=True, device=0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(0).cuda_stream)

    for lo, n in ((0, 101), (50, 206)):                      # two calls in a row, ragged tiles
        b = torch.from_numpy(pos256["boards"][lo:lo + n].copy()).to(dev)
        c = torch.from_numpy(pos256["control"][lo:lo + n].copy()).to(dev)
        r = torch.from_numpy(pos256["rep"][lo:lo + n].copy()).to(dev)
        want = [t.clone() for t in enc.forward_full(b, c, r)]
        pol = torch.zeros(n, 32, 64, dtype=torch.half, device=dev)
        pro = torch.zeros(n, 32, 4, dtype=torch.half, device=dev)
        val = torch.zeros(n, dtype=torch.float, device=dev)
        rc = L.bf_forward_noalloc(0, _ptr(blob), blob.numel(), _ptr(b), _ptr(c), _ptr(r), None, n,
                                  _ptr(pol), _ptr(pro), _ptr(val), stream)
        assert rc == 0, L.bf_last_error()
        st = ctypes.c_int(-1)
        assert L.bf_noalloc_status(0, ctypes.byref(st)) == 0 and st.value == 0
        assert torch.equal(pol.view(torch.int16), want[0].view(torch.int16))
        assert torch.equal(pro.view(torch.int16), want[1].view(torch.int16))
        assert torch.equal(val, want[2])
    enc.close()


def test_noalloc_rejects_what_it_cannot_serve(nets):
    from brokefish_b200 import _native
    from brokefish_b200.nn.pack import pack_blob
    L = _native.lib()
    dev = torch.device("cuda", 0)
    blob = torch.from_numpy(pack_blob(nets["A"])).to(dev)
    z = torch.zeros(8, dtype=torch.uint8, device=dev)
    too_many = 1048576 + 1
    rc = L.bf_forward_noalloc(0, _ptr(blob), blob.numel(), _ptr(z), _ptr(z), _ptr(z), None, too_many,
                              None, None, None, None)
    assert rc == -1 and b"BF_NOALLOC_MAX_POSITIONS" in L.bf_last_error()
    rc = L.bf_forward_noalloc(0, _ptr(blob), blob.numel() - 256, _ptr(z), _ptr(z), _ptr(z), None, 1,
                              None, None, None, None)
    assert rc == -1 and b"header" in L.bf_last_error()
    # a blob this entry point cannot run is refused with the reason, not as a malformed blob:
    # another arithmetic (fp16, e4m3) or a re-injecting network needs a handle
    from brokefish_b200.nn.model import BrokefishNet, seeded_state
    for fmt, word in (("f16", b"arithmetic 0"), ("e4m3", b"arithmetic 1")):
        other = torch.from_numpy(pack_blob(nets["A"], fmt)).to(dev)
        rc = L.bf_forward_noalloc(0, _ptr(other), other.numel(), _ptr(z), _ptr(z), _ptr(z), None, 1,
                                  None, None, None, None)
        assert rc == -3 and word in L.bf_last_error(), L.bf_last_error()
    rj = BrokefishNet(reinject="ln1")
    rj.load_state_dict(seeded_state(seed=3, std=None, perturb_norms=True, reinject="ln1"))
    other = torch.from_numpy(pack_blob(rj, "int8")).to(dev)
    rc = L.bf_forward_noalloc(0, _ptr(other), other.numel(), _ptr(z), _ptr(z), _ptr(z), None, 1,
                              None, None, None, None)
    assert rc == -3 and b"re-injecting" in L.bf_last_error()


def test_noalloc_repacked_buffer_needs_forget(pos256):
    """The weight-refresh pattern of a caller with one fixed weight buffer: a second network of
    the same blob size (another value head: king scalar, then pooled win/draw/loss) is copied
    over the first at the same device address.  The entry point remembers a blob's header by
    address and size, so the caller says `bf_noalloc_forget` after the copy; the values that
    come back are then the new head's (equal to a handle built from the new network), and the
    caller's current device is left as it was."""
    from brokefish_b200 import _native
    from brokefish_b200.nn import encoder_impl
    from brokefish_b200.nn.model import BrokefishNet, seeded_state
    from brokefish_b200.nn.pack import pack_blob
    L = _native.lib()
    dev = torch.device("cuda", 0)
    n = 64
    b, c, r = (torch.from_numpy(pos256[k][:n].copy()).to(dev) for k in ("boards", "control", "rep"))
    stream = ctypes.c_void_p(torch.cuda.current_stream(0).cuda_stream)
    nets_ = []
    for kw in (dict(n_value=1, value_head="king"), dict(n_value=3, value_head="pooled")):
        net = BrokefishNet(**kw).eval()
        net.load_state_dict(seeded_state(seed=5, std=None, perturb_norms=True, **kw))
        nets_.append(net)
    blobs = [pack_blob(net, "int8") for net in nets_]
    assert blobs[0].size == blobs[1].size                      # the tail section has a fixed size
    buf = torch.empty(blobs[0].size, dtype=torch.uint8, device=dev)
    val = torch.zeros(n, dtype=torch.float, device=dev)
    for net, blob in zip(nets_, blobs):
        buf.copy_(torch.from_numpy(blob))
        torch.cuda.synchronize()
        assert L.bf_noalloc_forget(0) == 0
        rc = L.bf_forward_noalloc(0, _ptr(buf), buf.numel(), _ptr(b), _ptr(c), _ptr(r), None, n,
                                  None, None, _ptr(val), stream)
        assert rc == 0, L.bf_last_error()
        enc = encoder_impl("cuda")(net, int8=True, device=0)
        want = enc.forward_full(b, c, r)[2].clone()
        enc.close()
        torch.cuda.synchronize()
        assert torch.equal(val, want)
    assert torch.cuda.current_device() == 0
