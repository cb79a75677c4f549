"""``FusedEncoder``: the evaluator object the search and the trainer call.

Same constructor, attributes, methods and errors as the reference's CUDA implementation
(brokefish/nn/cuda_impl.py:119-531), backed by the sm_100a kernel through the C ABI in
``include/brokefish_b200.h``.  PyTorch is used for device memory and the current stream
only.

All five arithmetics of the reference are built: its ``int8=True`` path (scheme ``"all"``:
QKV, out-projection and both FFN matmuls in int8, heads and attention in fp16), whose
outputs equal the reference kernel's bit for bit; the partial schemes
``int8_scheme="ffn"`` and ``"ffn+qkv"`` (the other GEMMs in fp16), bit for bit as well; its
``fp8=True`` path (the two FFN matmuls in e4m3 with ``amax/8`` scales, QKV and out-projection
in fp16), a tolerance; and the plain fp16 arithmetic (the default, as in the
reference; every weight GEMM fp16 with fp16 accumulators on tcgen05, which carry the bits of
the reference's fp16-accumulate ``mma.sync``), bit for bit.

The weights are a *snapshot*: folded, quantised and uploaded once in the constructor.
After a weight update, build a new ``FusedEncoder``.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from brokefish_b200 import _native
from brokefish_b200.nn.model import BrokefishNet, N_POLICY, N_PROMO
from brokefish_b200.nn.pack import pack_blob

#: Which matmuls int8 covers, by the reference's kernel mode number.
SCHEMES = {"ffn": 2, "ffn+qkv": 4, "all": 3}
SCHEME = "all"

OP_QKV, OP_OUT, OP_FF1, OP_FF2 = 0, 1, 2, 3
_OP_WIDTH = {OP_QKV: 768, OP_OUT: 256, OP_FF1: 1024}


#: What makes a module "the whole network" for the constructor: the parts the blob is packed from.
_NETWORK_PARTS = ("encoder", "norm_f", "policy", "promo", "value", "emb_square", "emb_type_special",
                  "emb_color_turn", "emb_clock", "emb_rep")


def is_whole_network(source) -> bool:
    """True for anything shaped like the reference's ``BrokefishNet`` (whichever class it is an
    instance of), False for a bare encoder stack."""
    return all(hasattr(source, part) for part in _NETWORK_PARTS)


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else ctypes.c_void_p(0)


class FusedEncoder:
    """Inference-only fused forward on one B200."""

    D, DFF, T, H = 256, 1024, 32, 8
    ACC_DTYPES = ("fp16", "fp32")
    NHEAD = 96
    VALUE_ROW = N_POLICY + N_PROMO
    VMODE = {"king": 0, "pooled": 1, "prenorm": 2}
    RJMODE = {"none": 0, "ln1": 1, "both": 2}
    n_value = 1
    vmode = 0
    rj_mode = 0

    def __init__(self, source, acc_dtype: str = "fp16", fp8: bool = False, int8: bool = False,
                 two_boards: Optional[bool] = None, int8_scheme: str = SCHEME,
                 device: Optional[int] = None):
        """``source``: a whole network -- any module with the reference network's parts
        (``encoder.layers``, ``norm_f``, the ``policy`` / ``promo`` / ``value`` heads and the five
        embedding tables; the reference's own ``BrokefishNet`` in fp32 or ``.half()``, or this
        package's weight container) -- or a bare ``nn.TransformerEncoder`` for the backbone
        entry alone.  Keywords and their defaults are the reference's
        (brokefish/nn/cuda_impl.py:160-162): plain fp16 arithmetic unless ``int8`` or ``fp8``
        is asked for."""
        if acc_dtype not in self.ACC_DTYPES:
            raise ValueError(f"acc_dtype must be one of {self.ACC_DTYPES}, got {acc_dtype!r}")
        if acc_dtype == "fp32":
            raise NotImplementedError(
                "acc_dtype='fp32' is not built: the weight GEMMs accumulate exactly in s32, and "
                "the attention and head products keep the fp16 accumulators of the reference's "
                "shipped kernel so that outputs equal that kernel's bit for bit")
        if fp8 and int8:
            raise ValueError("fp8 and int8 quantise the same two matmuls; pick one")
        if int8_scheme not in SCHEMES:
            raise ValueError(f"int8_scheme must be one of {sorted(SCHEMES)}, got {int8_scheme!r}")
        net = source if is_whole_network(source) else None
        encoder = source.encoder if net is not None else source
        if not hasattr(encoder, "layers") or len(encoder.layers) == 0:
            raise ValueError("source must be a network with an `encoder`, or an nn.TransformerEncoder")
        block = encoder.layers[0]
        self.acc_dtype = acc_dtype
        self.n_layers = len(encoder.layers)
        self.d_model = int(block.self_attn.embed_dim)
        self.n_heads = int(block.self_attn.num_heads)
        self.d_ff = int(block.linear1.out_features)
        self.d_head = self.d_model // self.n_heads
        self.eps = float(block.norm1.eps)
        if (self.d_model, self.d_ff, self.n_heads) != (self.D, self.DFF, self.H):
            raise ValueError(
                f"kernel is compiled for d_model={self.D}, d_ff={self.DFF}, heads={self.H}; "
                f"got {self.d_model}, {self.d_ff}, {self.n_heads}")
        self.fp8, self.int8 = bool(fp8), bool(int8)
        self.int8_scheme = int8_scheme
        # the reference's kernel mode numbers: 3 = int8 on all four matmuls, 1 = e4m3 FFN,
        # 0 = the plain fp16 arithmetic (the reference's default; here `int8=False`)
        self.quant = 1 if self.fp8 else (SCHEMES[int8_scheme] if self.int8 else 0)
        # Kept for callers that read it; the number of boards sharing a CTA never changes
        # a board's arithmetic, here as in the reference.
        self.two_boards = True if two_boards is None else bool(two_boards)
        self.debug_stage = 0
        self.net = net
        self._source_encoder = encoder
        self._bb_handle = None
        self._handle = ctypes.c_void_p(0)
        self._exact_rsqrt = False
        self._host_plan = 0
        self._buffered = 0
        self._buffered_full = 0
        if net is not None:
            if not torch.cuda.is_available():
                raise RuntimeError("FusedEncoder needs a CUDA device (sm_100a); there is no "
                                   "CPU fallback")
            self.device = torch.cuda.current_device() if device is None else int(device)
            self.n_value = int(net.value.weight.shape[0])
            self.vmode = self.VMODE[getattr(net, "value_head", "king")]
            self.rj_mode = self.RJMODE[getattr(net, "reinject", "none")]
            if self.quant in (1, 2, 4) and self.rj_mode:
                raise NotImplementedError("input re-injection is built for the int8 and the fp16 arithmetic "
                                          "(as in the reference, brokefish/nn/cuda_impl.py:413-420); this "
                                          "encoder is " + self.label)
            self.blob = pack_blob(net, {3: "int8", 2: "int8_ffn", 4: "int8_ffn_qkv", 1: "e4m3", 0: "f16"}[self.quant])
            self._create(self.blob)

    # -- construction helpers --------------------------------------------------
    def _create(self, blob: np.ndarray) -> None:
        L = _native.lib()
        h = ctypes.c_void_p(0)
        _native.check(L.bf_create(ctypes.c_void_p(blob.ctypes.data), blob.size, self.device,
                                  ctypes.byref(h)), "bf_create")
        self._handle = h

    @classmethod
    def from_blob(cls, blob, device: Optional[int] = None) -> "FusedEncoder":
        """Build from an already packed blob (``numpy`` uint8 array or a CUDA ``uint8``
        tensor, e.g. one received by a broadcast) without a network object."""
        self = cls.__new__(cls)
        self.acc_dtype, self.fp8, self.int8 = "fp16", False, True
        self.int8_scheme, self.quant, self.two_boards, self.debug_stage = "all", 3, True, 0
        self.d_model, self.d_ff, self.n_heads, self.d_head = cls.D, cls.DFF, cls.H, 32
        self.net = None
        self._exact_rsqrt = False
        self._host_plan = 0
        self._buffered = self._buffered_full = 0
        self.device = torch.cuda.current_device() if device is None else int(device)
        L = _native.lib()
        h = ctypes.c_void_p(0)
        if isinstance(blob, torch.Tensor):
            ptr, size = ctypes.c_void_p(blob.data_ptr()), blob.numel()
        else:
            ptr, size = ctypes.c_void_p(blob.ctypes.data), blob.size
        _native.check(L.bf_create(ptr, size, self.device, ctypes.byref(h)), "bf_create")
        self._handle = h
        nl, nv, vm = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        _native.check(L.bf_info(h, ctypes.byref(nl), ctypes.byref(nv), ctypes.byref(vm)), "bf_info")
        self.n_layers, self.n_value, self.vmode = nl.value, nv.value, vm.value
        head = blob[:32].cpu().numpy() if isinstance(blob, torch.Tensor) else np.asarray(blob[:32])
        self.rj_mode, self.quant = (int(v) for v in head.view(np.uint32)[6:8])
        self.fp8, self.int8 = self.quant == 1, self.quant == 3
        self.eps = 1e-5
        self._from_blob = True
        return self

    def close(self) -> None:
        if getattr(self, "_handle", None) and self._handle.value:
            _native.lib().bf_destroy(self._handle)
            self._handle = ctypes.c_void_p(0)
        if getattr(self, "_bb_handle", None) is not None and self._bb_handle.value:
            _native.lib().bf_destroy(self._bb_handle)
            self._bb_handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def label(self) -> str:
        """What this instance runs, for a bench header or a run log."""
        base = {1: "e4m3 FFN", 0: "fp16", 2: "int8 FFN", 3: "int8 FFN+QKV+out_proj", 4: "int8 FFN+QKV"}[self.quant]
        return base + ", 4 boards/CTA, tcgen05 (sm_100a)"

    @property
    def launches(self) -> int:
        return int(_native.lib().bf_launch_count(self._handle)) if self._handle.value else 0

    def _require_net(self, what: str):
        if not self._handle.value:
            raise ValueError(
                f"{what} needs the whole model: build this from a BrokefishNet, not from a "
                "bare nn.TransformerEncoder")

    # -- the backbone-only path: activations in, activations out ------------------------
    def _backbone_handle(self):
        """The handle the backbone entry runs on: this instance's own when it carries the fp16
        arithmetic, else a second one packed from the same weights on first use (the reference
        keeps an fp16 slab beside the quantised ones for the same purpose,
        brokefish/nn/cuda_impl.py:228, 460)."""
        if self.quant == 0 and self._handle.value:
            return self._handle
        if getattr(self, "_bb_handle", None) is not None and self._bb_handle.value:
            return self._bb_handle
        if getattr(self, "_from_blob", False):
            raise NotImplementedError("an encoder built from a packed blob has no weights to pack the fp16 "
                                      "backbone from; build it from the network")
        net = self.net
        if net is None:
            # a bare nn.TransformerEncoder: the stack is all there is; embeddings, final norm and
            # heads of a throw-away network fill the blob's other sections and are never read
            if not torch.cuda.is_available():
                raise RuntimeError("FusedEncoder needs a CUDA device (sm_100a); there is no CPU fallback")
            if not hasattr(self, "device"):
                self.device = torch.cuda.current_device()
            net = BrokefishNet(n_layers=self.n_layers, eps=self.eps)
            net.encoder = self._source_encoder
        blob = pack_blob(net, "f16")
        h = ctypes.c_void_p(0)
        _native.check(_native.lib().bf_create(ctypes.c_void_p(blob.ctypes.data), blob.size, self.device,
                                              ctypes.byref(h)), "bf_create")
        self._bb_handle = h
        return h

    def forward(self, x, alive=None, out=None):
        """Backbone only (brokefish/nn/cuda_impl.py:447-463): ``x [n,32,256]`` fp16 through the
        encoder layers, no embedding, no final norm, no heads; ``alive [n,32]`` bool or int8
        masks dead tokens as attention keys.  Always the fp16 arithmetic, as in the reference.
        Returns ``out`` (or an internal buffer the next call overwrites)."""
        if x.dim() != 3:
            raise ValueError(f"x must be [n, 32, {self.D}], got {tuple(x.shape)}")
        n_boards, seq_len, d_model = x.shape
        if d_model != self.d_model:
            raise ValueError(f"expected d_model={self.d_model}, got {d_model}")
        if seq_len != self.T:
            raise ValueError(f"expected {self.T} tokens per board, got {seq_len}")
        if not x.is_cuda or x.dtype is not torch.half:
            raise ValueError("x must be a CUDA fp16 tensor")
        alive_arg = None
        if alive is not None:
            if tuple(alive.shape) != (n_boards, seq_len):
                raise ValueError(f"alive must be [{n_boards}, {seq_len}], got {tuple(alive.shape)}")
            if alive.dtype is torch.bool:
                alive = alive.view(torch.int8)
            elif alive.dtype is not torch.int8:
                raise ValueError(f"alive must be bool or int8, got {alive.dtype}")
            alive_arg = alive.contiguous()
        h = self._backbone_handle()
        self._check_device(x, alive_arg, out)
        if out is None:
            if self._buffered != n_boards:
                self.state = torch.empty(n_boards, seq_len, d_model, dtype=torch.half,
                                         device=torch.device("cuda", self.device))
                self._buffered = n_boards
            out = self.state
        elif tuple(out.shape) != tuple(x.shape) or out.dtype is not torch.half or not out.is_contiguous():
            raise ValueError("out must be a contiguous fp16 tensor of x's shape")
        xin = x.contiguous()
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(_native.lib().bf_forward_backbone(h, _ptr(xin), _ptr(alive_arg), n_boards, _ptr(out), stream),
                      "bf_forward_backbone")
        return out

    __call__ = forward

    # -- boards in, logits out ---------------------------------------------------------
    def _ensure_full_buffers(self, n: int) -> None:
        if self._buffered_full != n:
            dev = torch.device("cuda", self.device)
            self.policy_out = torch.empty(n, self.T, N_POLICY, device=dev, dtype=torch.half)
            self.promo_out = torch.empty(n, self.T, N_PROMO, device=dev, dtype=torch.half)
            self.value_out = torch.empty(n, device=dev, dtype=torch.float)
            self._buffered_full = n

    @staticmethod
    def _check_inputs(boards, control, rep):
        n = boards.shape[0]
        if boards.dim() != 2 or boards.shape[1] != FusedEncoder.T:
            raise ValueError(f"boards must be [n, 32], got {tuple(boards.shape)}")
        if boards.dtype is not torch.int16:
            raise ValueError(f"boards must be int16, got {boards.dtype}")
        if control.shape != (n,) or control.dtype is not torch.int16:
            raise ValueError(f"control must be [{n}] int16, got {tuple(control.shape)} {control.dtype}")
        if rep.shape != (n,) or rep.dtype is not torch.uint8:
            raise ValueError(f"rep must be [{n}] uint8, got {tuple(rep.shape)} {rep.dtype}")
        return n

    def _check_device(self, *tensors):
        for t in tensors:
            if t is not None and (not t.is_cuda or t.device.index != self.device):
                raise ValueError(f"inputs must live on cuda:{self.device}, got {t.device}")

    def forward_full(self, boards, control, rep, legal=None):
        """Boards to ``(policy_logits [n,32,64] fp16, promo [n,32,4] fp16, value [n] fp32)``
        in one launch on the current stream.

        ``policy_logits`` is raw unless ``legal`` (``[n,32]`` int64 legality words, bit s of
        word p set when p->s is legal) is given, in which case illegal entries are -inf.
        Returns views on internal buffers, which the next call overwrites.
        """
        self._require_net("forward_full")
        n = self._check_inputs(boards, control, rep)
        self._check_device(boards, control, rep, legal)
        if legal is not None and (tuple(legal.shape) != (n, self.T) or legal.dtype is not torch.int64):
            raise ValueError(f"legal must be [{n}, 32] int64, got {tuple(legal.shape)} {legal.dtype}")
        self._ensure_full_buffers(n)
        b, c, r = boards.contiguous(), control.contiguous(), rep.contiguous()
        lg = legal.contiguous() if legal is not None else None
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(_native.lib().bf_forward(
            self._handle, _ptr(b), _ptr(c), _ptr(r), _ptr(lg), n, _ptr(self.policy_out),
            _ptr(self.promo_out), _ptr(self.value_out), stream), "bf_forward")
        return self.policy_out, self.promo_out, self.value_out

    def forward_priors(self, boards, control, rep, legal, e_cap: int = 96, logits: bool = False):
        """Evaluate and expand in one launch: ``(prior [n,e_cap] fp16, move [n,e_cap] int16,
        nedges [n] int32, value [n] fp32)`` — the edges of each position's search node in
        canonical order with their priors, what the reference's search computes from the
        logits in ``Search._expand`` (brokefish/search/torch_impl.py:962-1033).  ``legal`` is
        the ``[n,32]`` int64 legality words, or ``None`` to let the kernel generate the legal
        moves itself (the rules of :func:`brokefish_b200.env.movegen`).  With ``logits=True`` the masked policy and the
        promotion logits are written as well (``self.policy_out``, ``self.promo_out``).
        Returns views on internal buffers, which the next call overwrites."""
        self._require_net("forward_priors")
        n = self._check_inputs(boards, control, rep)
        self._check_device(boards, control, rep, legal)
        if legal is not None and (tuple(legal.shape) != (n, self.T) or legal.dtype is not torch.int64):
            raise ValueError(f"legal must be [{n}, 32] int64 or None")
        if legal is None and logits:
            raise ValueError("the masked policy needs the legality words; pass them or leave logits off")
        if not 1 <= int(e_cap) <= 255:
            raise ValueError(f"e_cap must be in 1..255, got {e_cap}")
        self._ensure_full_buffers(n)
        dev = torch.device("cuda", self.device)
        if getattr(self, "_prior_shape", None) != (n, int(e_cap)):
            self.prior_out = torch.zeros(n, int(e_cap), device=dev, dtype=torch.half)
            self.move_out = torch.zeros(n, int(e_cap), device=dev, dtype=torch.int16)
            self.nedges_out = torch.zeros(n, device=dev, dtype=torch.int32)
            self._prior_shape = (n, int(e_cap))
        b, c, r = boards.contiguous(), control.contiguous(), rep.contiguous()
        lg = legal.contiguous() if legal is not None else None
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(_native.lib().bf_forward_priors(
            self._handle, _ptr(b), _ptr(c), _ptr(r), _ptr(lg), n, int(e_cap), _ptr(self.prior_out),
            _ptr(self.move_out), _ptr(self.nedges_out), _ptr(self.value_out),
            _ptr(self.policy_out) if logits else None, _ptr(self.promo_out) if logits else None, stream),
            "bf_forward_priors")
        return self.prior_out, self.move_out, self.nedges_out, self.value_out

    def forward_leaves(self, boards, control, rep, leaf_index, leaf_count, legal=None, e_cap: int = 0):
        """Evaluate a compacted leaf list: positions ``leaf_index[: leaf_count]`` of the staged
        arrays, where ``leaf_count`` is a one-element int32 CUDA tensor the kernel reads when it
        starts (no host synchronisation; clamped to ``len(leaf_index)``) -- the staging interface
        the reference's retrospective asks for in place of "all B staged leaves, active or not"
        (brokefish/search/cuda_impl.py:304-320).  A short list runs short: CTAs beyond the
        count's tiles leave at once.  Returns ``(policy, promo, value)`` sized like the staged
        arrays, rows not in the list untouched since the last call; with ``e_cap > 0`` the fused
        expansion runs as well and ``(prior, move, nedges, value)`` is returned (``legal`` words
        optional as in :meth:`forward_priors`, and the masked policy is written when they are
        given).  Views on internal buffers."""
        self._require_net("forward_leaves")
        n = self._check_inputs(boards, control, rep)
        self._check_device(boards, control, rep, legal, leaf_index, leaf_count)
        if leaf_index.dim() != 1 or leaf_index.dtype is not torch.int32 or leaf_index.shape[0] > n:
            raise ValueError(f"leaf_index must be int32 [k], k <= {n}")
        if leaf_count.dtype is not torch.int32 or leaf_count.numel() != 1:
            raise ValueError("leaf_count must be a one-element int32 tensor")
        if legal is not None and (tuple(legal.shape) != (n, self.T) or legal.dtype is not torch.int64):
            raise ValueError(f"legal must be [{n}, 32] int64 or None")
        e_cap = int(e_cap)
        if not 0 <= e_cap <= 255:
            raise ValueError(f"e_cap must be in 0..255, got {e_cap}")
        self._ensure_full_buffers(n)
        dev = torch.device("cuda", self.device)
        if e_cap and getattr(self, "_prior_shape", None) != (n, e_cap):
            self.prior_out = torch.zeros(n, e_cap, device=dev, dtype=torch.half)
            self.move_out = torch.zeros(n, e_cap, device=dev, dtype=torch.int16)
            self.nedges_out = torch.zeros(n, device=dev, dtype=torch.int32)
            self._prior_shape = (n, e_cap)
        capacity = int(leaf_index.shape[0])
        if capacity == 0:
            return ((self.prior_out, self.move_out, self.nedges_out, self.value_out) if e_cap
                    else (self.policy_out, self.promo_out, self.value_out))
        b, c, r, li = boards.contiguous(), control.contiguous(), rep.contiguous(), leaf_index.contiguous()
        lg = legal.contiguous() if legal is not None else None
        want_policy = not e_cap or lg is not None
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(_native.lib().bf_forward_leaves(
            self._handle, _ptr(b), _ptr(c), _ptr(r), _ptr(lg), _ptr(li), _ptr(leaf_count), capacity,
            _ptr(self.policy_out) if want_policy else None, _ptr(self.promo_out) if want_policy else None,
            _ptr(self.value_out), e_cap, _ptr(self.prior_out) if e_cap else None,
            _ptr(self.move_out) if e_cap else None, _ptr(self.nedges_out) if e_cap else None, stream),
            "bf_forward_leaves")
        if e_cap:
            return self.prior_out, self.move_out, self.nedges_out, self.value_out
        return self.policy_out, self.promo_out, self.value_out

    def forward_stage(self, boards, control, rep, stage: int, layer: int = 0):
        """Activations ``[n,32,256]`` fp16 at an intermediate stage: 9 embedding; layer 0:
        1 LN1, 5/6/7 Q/K/V, 4 attention output, 2 residual after attention, 3 LN2; 8 final
        norm.  ``layer`` (an extension) selects another layer for stages 1-7 and allows
        stage 10, the residual stream at the end of that layer."""
        self._require_net("forward_stage")
        n = self._check_inputs(boards, control, rep)
        self._check_device(boards, control, rep)
        if self._buffered != n:
            self.state = torch.zeros(n, self.T, self.D, device=torch.device("cuda", self.device),
                                     dtype=torch.half)
            self._buffered = n
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        if layer == 0 and stage != 10:
            rc = _native.lib().bf_forward_stage(
                self._handle, _ptr(boards.contiguous()), _ptr(control.contiguous()),
                _ptr(rep.contiguous()), n, int(stage), _ptr(self.state), stream)
        else:
            rc = _native.lib().bf_forward_stage_at(
                self._handle, _ptr(boards.contiguous()), _ptr(control.contiguous()),
                _ptr(rep.contiguous()), n, int(layer), int(stage), _ptr(self.state), stream)
        _native.check(rc, "bf_forward_stage")
        return self.state

    def capture_gemm(self, boards, control, rep, layer: int, op: int):
        """``(A bytes [n*32,256] uint8, accumulators [n*32,N] int32)`` of one GEMM of one
        layer, exactly as the tensor cores saw and produced them."""
        self._require_net("capture_gemm")
        n = self._check_inputs(boards, control, rep)
        width = _OP_WIDTH.get(op, 256)
        dev = torch.device("cuda", self.device)
        a = torch.zeros(n * self.T, 256, device=dev, dtype=torch.uint8)
        acc = torch.zeros(n * self.T, width, device=dev, dtype=torch.int32)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(_native.lib().bf_forward_capture(
            self._handle, _ptr(boards.contiguous()), _ptr(control.contiguous()),
            _ptr(rep.contiguous()), n, int(layer), int(op), _ptr(a), _ptr(acc), stream),
            "bf_forward_capture")
        return a, acc

    def forward_host(self, boards, control, rep, policy, promo, value, legal=None):
        """End-to-end call on HOST tensors (pinned for speed): copies in, runs, copies the
        three outputs into the given host tensors and synchronises."""
        self._require_net("forward_host")
        n = self._check_inputs(boards, control, rep)
        for t in (boards, control, rep, policy, promo, value):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("forward_host takes contiguous CPU tensors")
        _native.check(_native.lib().bf_forward_host(
            self._handle, _ptr(boards), _ptr(control), _ptr(rep), _ptr(legal), n, _ptr(policy),
            _ptr(promo), _ptr(value)), "bf_forward_host")
        return policy, promo, value

    def forward_priors_host(self, boards, control, rep, legal, prior, move, nedges, value):
        """``forward_priors`` end to end on HOST tensors (pinned for speed): ``prior [n,E]``
        fp16, ``move [n,E]`` int16, ``nedges [n]`` int32 and ``value [n]`` fp32 are filled;
        ``E = prior.shape[1]``."""
        self._require_net("forward_priors_host")
        n = self._check_inputs(boards, control, rep)
        for t in (boards, control, rep, legal, prior, move, nedges, value):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("forward_priors_host takes contiguous CPU tensors")
        e_cap = int(prior.shape[1])
        if (tuple(legal.shape) != (n, self.T) or legal.dtype is not torch.int64
                or tuple(move.shape) != (n, e_cap) or move.dtype is not torch.int16
                or prior.dtype is not torch.half or tuple(nedges.shape) != (n,)
                or nedges.dtype is not torch.int32 or tuple(value.shape) != (n,)
                or value.dtype is not torch.float32):
            raise ValueError("forward_priors_host: legal [n,32] int64, prior [n,E] fp16, move [n,E] int16, "
                             "nedges [n] int32, value [n] fp32")
        _native.check(_native.lib().bf_forward_priors_host(
            self._handle, _ptr(boards), _ptr(control), _ptr(rep), _ptr(legal), n, e_cap, _ptr(prior),
            _ptr(move), _ptr(nedges), _ptr(value)), "bf_forward_priors_host")
        return prior, move, nedges, value

    # -- in-kernel phase accounting (the reference's set_profile / read_profile hooks) ----
    def set_profile(self, on: bool) -> None:
        _native.check(_native.lib().bf_profile(self._handle, int(bool(on))), "bf_profile")

    def read_profile(self) -> dict:
        """``{phase: cycles}`` summed over CTAs since the last read; synchronises."""
        buf = (ctypes.c_longlong * 16)()
        _native.check(_native.lib().bf_profile_read(self._handle, buf, 16), "bf_profile_read")
        names = _native.lib().bf_profile_phases().decode().split(",")
        return {n: int(buf[i]) for i, n in enumerate(names)}

    # -- 1/sqrt of the norms: hardware approximation (default, as the reference kernel's
    #    rsqrtf, csrc/encoder.cu:597) or correctly rounded (what a CPU can reproduce) ------
    @property
    def exact_rsqrt(self) -> bool:
        return self._exact_rsqrt

    @exact_rsqrt.setter
    def exact_rsqrt(self, on: bool) -> None:
        _native.check(_native.lib().bf_set_option(self._handle, 1, int(bool(on))), "bf_set_option")
        self._exact_rsqrt = bool(on)

    def set_one_board(self, boards_per_sm: int) -> None:
        """Batches of at most this many boards per SM run in the small-batch form of the int8
        kernel (one board per tile, sixteen row warps per board); 0 switches it off."""
        _native.check(_native.lib().bf_set_option(self._handle, 5, int(boards_per_sm)), "bf_set_option")

    # -- how forward_host splits a batch: by the measured host link (0), or forced (1 fast, 2 slow)
    def set_host_plan(self, plan: int) -> None:
        _native.check(_native.lib().bf_set_option(self._handle, 4, int(plan)), "bf_set_option")
        self._host_plan = int(plan)

    @property
    def host_link_gbps(self) -> float:
        """GB/s the first device-to-host copy of the last ``forward_host`` call reached."""
        return float(_native.lib().bf_host_link_gbps(self._handle))

    def host_plan(self, n: int):
        """The launch sizes ``forward_host`` would use for ``n`` positions now."""
        sizes = (ctypes.c_int * 16)()
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        k = _native.lib().bf_host_plan(int(n), sms, self._host_plan, self.host_link_gbps, sizes)
        _native.check(min(k, 0), "bf_host_plan")
        return list(sizes[:k])

    def check_status(self) -> None:
        """Synchronise and raise if any launch hit a device-side time-out."""
        st = ctypes.c_int(0)
        _native.check(_native.lib().bf_status(self._handle, ctypes.byref(st)), "bf_status")
