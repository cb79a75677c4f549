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
    enc = encoder_impl("cuda")(net, device=0)
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
