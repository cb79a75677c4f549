"""Host-side packing: the product's folded / quantised weights against the oracle's and
the reference's, and the stage-image layout re-derived independently."""
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN
from brokefish_b200.nn import pack


@pytest.fixture(scope="module")
def folded(nets):
    return {k: pack.fold_and_quantise(n) for k, n in nets.items()}


@pytest.mark.parametrize("name", ["A", "B"])
def test_quantised_weights_equal_oracle_and_reference(name, folded, oracle_weights):
    g = np.load(os.path.join(GOLDEN, f"ref_outputs_{name}.npz"))
    for li, (fl, lw) in enumerate(zip(folded[name], oracle_weights[name].layers)):
        for tag in ("qkv", "o", "ff1", "ff2"):
            assert np.array_equal(getattr(fl, "q_" + tag), getattr(lw, "q_" + tag).view(np.uint8))
            assert np.array_equal(getattr(fl, "s_" + tag), getattr(lw, "s_" + tag))
        assert np.array_equal(fl.b_o, lw.b_o) and np.array_equal(fl.b_ff2, lw.b_ff2)
        for mine, ref in ((fl.b_qkv, g["folded_b_qkv"][li]), (fl.b_ff1, g["folded_b_ff1"][li])):
            step = np.abs(mine.view(np.int16).astype(np.int32) - ref.view(np.int16).astype(np.int32))
            assert step.max() <= 1 and (step == 0).mean() >= 0.99


def test_stage_image_is_the_128_byte_swizzle():
    rng = np.random.default_rng(0)
    tile = rng.integers(0, 256, size=(192, 128), dtype=np.uint8)
    img = pack.sw128_image(tile)
    assert img.size == tile.size
    for r in (0, 1, 7, 8, 13, 191):
        for c in range(8):
            at = r * 128 + ((c ^ (r & 7)) * 16)
            assert np.array_equal(img[at:at + 16], tile[r, 16 * c:16 * c + 16])
    with pytest.raises(ValueError):
        pack.sw128_image(np.zeros((8, 64), dtype=np.uint8))


def test_qkv_chunk_rows_cover_in_proj_once():
    rows = pack.qkv_chunk_rows()
    assert sorted(rows.reshape(-1).tolist()) == list(range(768))
    assert rows[1, 0] == 64 and rows[1, 64] == 256 + 64 and rows[3, 191] == 512 + 255


def test_blob_layout_decodes_back(nets, folded):
    net, fl = nets["B"], folded["B"]
    blob = pack.pack_blob(net)
    magic, ver, nl, nv, vm, eps = struct.unpack_from("<IIIIIf", blob, 0)
    assert (magic, ver, nl, nv, vm) == (pack.MAGIC, 4, 8, 1, 0) and abs(eps - 1e-5) < 1e-12
    offs = struct.unpack_from("<11Q", blob, 32)
    off_w, bytes_w, off_lp, bytes_lp, off_emb, bytes_emb, off_tail, bytes_tail, off_rj, bytes_rj, total = offs
    assert bytes_rj == 0 and bytes_tail == 2560
    assert total == blob.size and bytes_w == 8 * 786432 + 4 * 96 * 128 and bytes_lp == 8 * 4736
    assert all(o % 256 == 0 for o in (off_w, off_lp, off_emb, off_tail))
    # layer 3, FFN unit 9 = ff2, hidden chunk 1, output half 1; its K-slab 1
    layer, unit, slab = 3, 9, 1
    kind, c, j = pack.FFN_UNITS[unit]
    assert (kind, c, j) == (2, 1, 1)
    at = off_w + layer * 786432 + 8 * 24576 + 4 * 16384 + (unit * 2 + slab) * 16384
    r, grp = 77, 5
    got = blob[at + r * 128 + ((grp ^ (r & 7)) * 16):][:16]
    want = fl[layer].q_ff2[128 * j + r, 256 * c + 128 * slab + 16 * grp:][:16]
    assert np.array_equal(got, want)
    # QKV chunk 2, K-slab 0, row 130 = V row of head 4 (in_proj row 512 + 128 + 2)
    at = off_w + layer * 786432 + (2 * 2 + 0) * 24576
    r, grp = 130, 3
    got = blob[at + r * 128 + ((grp ^ (r & 7)) * 16):][:16]
    assert np.array_equal(got, fl[layer].q_qkv[512 + 128 + 2, 16 * grp:16 * grp + 16])
    # scales and the permuted qkv bias
    lp = blob[off_lp + layer * 4736:][:4736]
    assert np.array_equal(lp[:24].view("<f4"), fl[layer].s_qkv)
    assert np.array_equal(lp[64:72].view("<f4"), fl[layer].s_ff2)
    bq = lp[128:128 + 1536].view("<f2")
    assert bq[2 * 192 + 130] == fl[layer].b_qkv[512 + 128 + 2]
    # the head matrix closes the weight stream: 4 K-slabs of [96 rows][128 B], swizzled like
    # every other stage; row 68 is the first value row
    head = pack.head_matrix(net)
    slab, r, grp = 2, 68, 6
    at = off_w + 8 * 786432 + slab * 96 * 128
    got = blob[at + r * 128 + ((grp ^ (r & 7)) * 16):][:16].view("<f2")
    assert np.array_equal(got, head[r, 64 * slab + 8 * grp:64 * slab + 8 * grp + 8])
    tail = blob[off_tail:off_tail + bytes_tail].view("<f2")
    assert np.array_equal(tail[:256], net.norm_f.weight.detach().half().numpy())
    assert np.array_equal(tail[512:768], head[68])


def test_packer_rejects_other_widths():
    import torch
    from brokefish_b200.nn.model import BrokefishNet
    with pytest.raises(ValueError):
        pack.pack_blob(BrokefishNet(d_ff=512))
