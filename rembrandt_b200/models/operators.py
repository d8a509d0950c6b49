"""Operator library: one class per layer kind, each with a CUDA path (hand-written kernels, bf16 NHWC) and
a reference path (plain torch fp32, used on CPU and as the numerical oracle).

Mirrors the reference's ``Operator`` protocol (src/operator/mod.rs:61-99): parameters live in flat
vectors owned by the network; an operator reads its input activation from the previous operator, writes
its own output buffer, and on backward accumulates parameter gradients (beta = 1, as cuDNN/cuBLAS are
called in the reference) and writes the previous operator's delta buffer. Where the previous operator
ends in a ReLU, the delta is masked by that operator's output in the same kernel that produces it (the
reference does this as a separate in-place pass at the start of each backward).
"""
from __future__ import annotations

import contextlib
import math
from typing import List, Optional

import torch
import torch.nn.functional as F

import os

from ..ops import layout
from ..ops import native_ops as K
from ..ops.conv_strided import dgrad_strided_tc
from ..ops.native_ops import pad_channels
from . import config as C


def _strided_dgrad_on_tensor_cores() -> bool:
    """Strided data-grad by output phases on the tensor-core kernel (ops/conv_strided.py) instead of the CUDA-core
    kernel; RB_STRIDED_DGRAD_TC=0 selects the latter."""
    return os.environ.get("RB_STRIDED_DGRAD_TC", "1") == "1"


class ParamSeg:
    """A parameter tensor inside the flat vectors."""

    def __init__(self, name, shape, decay=True, trainable=True):
        self.name = name
        self.shape = tuple(shape)
        self.numel = int(math.prod(shape))
        self.decay = decay
        self.trainable = trainable
        self.offset = -1  # assigned by the network


class Op:
    """Base operator. Shapes are (H, W, C) logical plus the padded channel count `cp`."""

    has_params = False

    def __init__(self, name, cfg):
        self.name = name
        self.cfg = cfg
        self.net = None
        self.prev: Optional[Op] = None
        self.out_hwc = None
        self.out_cp = 0
        self.has_relu = False
        self.act_kind = 0
        self.act_param = 0.0
        self.segs: List[ParamSeg] = []
        self.out = None    # activation buffer (CUDA path)
        self.dout = None   # delta w.r.t. `out`, written by the consumer

    # ---- construction
    def setup(self, net, prev):
        self.net, self.prev = net, prev

    def alloc(self):
        h, w, _ = self.out_hwc
        n = self.net.batch
        self.out = torch.zeros((n, h, w, self.out_cp), dtype=torch.bfloat16, device=self.net.device)
        if self.net.training_capable:
            self.dout = torch.zeros_like(self.out)

    def bind(self):
        """Called after the flat vectors exist."""

    # ---- parameters
    def init_params(self, rng):
        pass

    def encode_params(self) -> list:
        return []

    def decode_params(self, arrays: list) -> int:
        return 0

    def state_segs(self) -> List[ParamSeg]:
        return [s for s in self.segs if s.trainable]

    # ---- execution
    def forward(self, train: bool, t: int):
        raise NotImplementedError

    def backward(self):
        pass

    def ref_forward(self, x, train: bool, t: int):
        raise NotImplementedError

    # ---- helpers
    def view(self, seg: ParamSeg, which="params"):
        return self.net.seg_view(seg, which)

    @property
    def in_hwc(self):
        return self.prev.out_hwc

    @property
    def in_cp(self):
        return self.prev.out_cp

    # ---- activations other than ReLU (ReLU is fused into the producing kernel's epilogue and the consumer's mask)
    def _setup_act(self, act, param=None):
        self.has_relu = act == C.Act.RECT
        self.act_kind = {C.Act.LOGISTIC: K.ACT_LOGISTIC, C.Act.TANH: K.ACT_TANH,
                         C.Act.BOUNDED_RECT: K.ACT_BOUNDED_RECT,
                         C.Act.SCALED_LOGISTIC: K.ACT_SCALED_LOGISTIC}.get(act, 0)
        default = C.ACT_BETA if act == C.Act.SCALED_LOGISTIC else C.ACT_BOUND
        self.act_param = float(default if param is None else param)

    def _act_rows(self):
        h, w, _ = self.out_hwc
        return self.net.batch * h * w

    def _act_forward(self):
        if self.act_kind:
            K.act_fwd(self.out, self._act_rows(), self.out_cp, self.out_hwc[2], self.act_kind, self.act_param)

    def _act_backward(self):
        """Turn the delta w.r.t. the activation into the delta w.r.t. the pre-activation, in place."""
        if self.act_kind:
            K.act_bwd(self.dout, self.out, self._act_rows(), self.out_cp, self.out_hwc[2], self.act_kind,
                      self.act_param)

    def _ref_act(self, y):
        if self.has_relu:
            return torch.relu(y)
        if self.act_kind == K.ACT_LOGISTIC:
            return torch.sigmoid(y)
        if self.act_kind == K.ACT_TANH:
            return torch.tanh(y)
        if self.act_kind == K.ACT_BOUNDED_RECT:
            return y.clamp(0.0, self.act_param)
        if self.act_kind == K.ACT_SCALED_LOGISTIC:
            return torch.sigmoid(self.act_param * y)
        return y

    def mask_src(self):
        """Activation to mask the delta of `prev` with, or None."""
        return self.prev.out if self.prev.has_relu else None

    def wants_prev_delta(self):
        return self.prev is not None and self.prev.dout is not None and not isinstance(self.prev, DataOp)


def _draw(kind: C.ParamsInit, rng, shape, fan_in, fan_out):
    n = int(math.prod(shape))
    if kind.kind == "disabled":
        return torch.zeros(shape)
    if kind.kind == "uniform":
        return rng.uniform(n, -kind.half_range, kind.half_range).reshape(shape)
    if kind.kind == "normal":
        return rng.normal(n, kind.mean, kind.std).reshape(shape)
    if kind.kind == "xavier":
        h = math.sqrt(6.0 / (fan_in + fan_out))
        return rng.uniform(n, -h, h).reshape(shape)
    if kind.kind == "kaiming_fwd":
        return rng.normal(n, 0.0, math.sqrt(2.0 / fan_in)).reshape(shape)
    raise ValueError(kind.kind)


# =============================================================================================== input
class DataOp(Op):
    """Fixed-size input operator: u8 staging -> cast / normalise / mean / crop / flip / PCA noise.

    Reference: Data3dOperator (src/operator/mod.rs:386-836). Differences by design: crop offsets and flip
    coins are drawn per sample unless `per_batch_draws` is set; the crop may extend beyond the image by
    `pad` pixels (zero fill), which gives the usual pad-and-crop augmentation.
    """

    def setup(self, net, prev):
        super().setup(net, prev)
        cfg: C.Data3dCfg = self.cfg
        w, h, c = cfg.in_dims
        self.src_hwc = (h, w, c)
        self.crop_h, self.crop_w, self.pad = h, w, 0
        self.flip = False
        self.mean = None
        self.mean_scale = 1.0
        self.pca = None
        for p in cfg.preprocs:
            if p.kind == "crop":
                self.crop_w, self.crop_h, self.pad = p.crop_width, p.crop_height, p.pad
            elif p.kind == "flip_x":
                self.flip = True
            elif p.kind == "subtract_mean":
                self.mean = p
            elif p.kind == "pca_noise":
                self.pca = p
            elif p.kind == "scale_bicubic":
                self.scale_range = (p.lower, p.upper)
            else:
                raise ValueError(f"unknown preprocessing stage {p.kind!r}")
        self.scale = cfg.scale if cfg.scale is not None else (1.0 / 255.0 if cfg.normalize else 1.0)
        self.out_hwc = (self.crop_h, self.crop_w, c)
        self.out_cp = pad_channels(c)
        self.mode = "nhwc"
        self.f = 1
        self.extra_pad = 0      # padding absorbed from a space-to-depth'd first convolution
        self.mean_dev = None
        self.stage = None

    # layout requests from the first hidden operator
    def request_s2d(self, f, s2d_hw, conv_pad):
        self.mode, self.f, self.extra_pad = "s2d", f, conv_pad
        c = self.out_hwc[2]
        self.s2d_hw = s2d_hw
        self.out_cp = pad_channels(f * f * c)

    def request_flat(self):
        h, w, c = self.out_hwc
        self.mode, self.f = "flat", max(h, w)
        self.out_cp = pad_channels(self.f * self.f * c)

    def out_buffer_shape(self):
        n = self.net.batch
        if self.mode == "s2d":
            return (n, self.s2d_hw, self.s2d_hw, self.out_cp)
        if self.mode == "flat":
            return (n, 1, 1, self.out_cp)
        return (n, self.crop_h, self.crop_w, self.out_cp)

    def alloc(self):
        h, w, c = self.src_hwc
        dev = self.net.device
        self.out = torch.zeros(self.out_buffer_shape(), dtype=torch.bfloat16, device=dev)
        self.stage = torch.zeros((self.net.batch, c, h, w), dtype=torch.uint8, device=dev)
        if self.mean is not None:
            m = self.mean.mean
            if m is None and self.mean.mean_path:
                from ..utils import blob
                m = blob.read_array_file(self.mean.mean_path, "f32")
            m = torch.as_tensor(m, dtype=torch.float32).reshape(c, h, w)
            self.mean_dev = m.to(dev)
            self.mean_scale = self.scale if self.mean.normalize or self.cfg.normalize else 1.0

    def load_batch(self, images_u8: torch.Tensor, non_blocking=True):
        """Copy a [B,C,H,W] uint8 batch (host, ideally pinned, or device) into the staging buffer."""
        self.stage.copy_(images_u8.reshape(self.stage.shape), non_blocking=non_blocking)

    def forward(self, train, t):
        h, w, c = self.src_hwc
        cfg = self.cfg
        n = self.net.batch
        if self.mode == "nhwc":
            oh, ow, f = self.crop_h, self.crop_w, 1
        elif self.mode == "s2d":
            oh = ow = self.s2d_hw
            f = self.f
        else:
            oh = ow = 1
            f = self.f
        ep = self.extra_pad
        # a crop window enlarged by the absorbed convolution padding
        ch, cw = self.crop_h + 2 * ep, self.crop_w + 2 * ep
        lo_y, hi_y = -(self.pad + ep), h - self.crop_h + self.pad - ep
        lo_x, hi_x = -(self.pad + ep), w - self.crop_w + self.pad - ep
        rnd_crop = train and (hi_y > lo_y or hi_x > lo_x)
        pv = pe = None
        sigma = 0.0
        if self.pca is not None and train:
            sigma, pv, pe = self.pca.std, list(self.pca.eigenvalues), list(self.pca.eigenvectors)
        K.input_u8(self.stage, self.mean_dev, self.out, n, c, h, w, ch, cw, oh, ow, self.out_cp, f, lo_y, hi_y, lo_x,
                   hi_x, rnd_crop, train and self.flip, cfg.per_batch_draws, self.scale, self.mean_scale, sigma, pv,
                   pe, self.net.data_seed, 0, self.net.step_counter)

    def ref_forward(self, x, train, t):
        """x: [B,C,H,W] uint8 or float. Centre crop / no flip at inference, torch RNG draws when training."""
        h, w, c = self.src_hwc
        x = x.float() * self.scale
        if self.mean is not None:
            m = torch.as_tensor(self.mean.mean, dtype=torch.float32).reshape(1, c, h, w).to(x.device)
            x = x - (self.scale if (self.mean.normalize or self.cfg.normalize) else 1.0) * m
        p = self.pad
        if p:
            x = F.pad(x, (p, p, p, p))
        hh, ww = x.shape[2], x.shape[3]
        g = self.net.ref_generator
        n = x.shape[0]
        draws = 1 if self.cfg.per_batch_draws else n       # one offset / coin per batch (reference) or per sample
        if (hh, ww) != (self.crop_h, self.crop_w):
            if train:
                oys = torch.randint(0, hh - self.crop_h + 1, (draws,), generator=g).tolist()
                oxs = torch.randint(0, ww - self.crop_w + 1, (draws,), generator=g).tolist()
            else:
                oys, oxs = [(hh - self.crop_h) // 2], [(ww - self.crop_w) // 2]
            if len(oys) == 1:
                x = x[:, :, oys[0]:oys[0] + self.crop_h, oxs[0]:oxs[0] + self.crop_w]
            else:
                x = torch.stack([x[i, :, oy:oy + self.crop_h, ox:ox + self.crop_w]
                                 for i, (oy, ox) in enumerate(zip(oys, oxs))])
        if train and self.flip:
            coins = torch.randint(0, 2, (draws,), generator=g).bool()
            if draws == 1:
                x = x.flip(-1) if bool(coins[0]) else x
            else:
                x = torch.where(coins.reshape(n, 1, 1, 1), x.flip(-1), x)
        if train and self.pca is not None and c == 3 and self.pca.std > 0:
            # lighting noise: per sample, shift[c] = sum_j alpha_j * eigenvalue_j * eigenvector[c][j], alpha ~ N(0, std)
            al = torch.randn(x.shape[0], 3, generator=self.net.ref_generator) * self.pca.std
            vals = torch.tensor(list(self.pca.eigenvalues), dtype=torch.float32)
            vecs = torch.tensor(list(self.pca.eigenvectors), dtype=torch.float32).reshape(3, 3)
            x = x + ((al * vals) @ vecs.t()).reshape(-1, 3, 1, 1)
        return x


class VarDataOp(DataOp):
    """Variable-size input operator: every sample has its own width / height (up to `max_dims`).

    Reference: VarData3dOperator (src/operator/input.rs:49-538) with its ScaleBicubic -> Crop -> FlipX -> PCA-noise
    chain. Here the whole chain is one kernel (csrc/var_input.cu) that interpolates only the pixels of the crop
    window. Training draws, per sample: the target length of the shorter side in [lower, upper], the crop offset
    and the flip coin; inference uses `lower`, the centred crop and no flip (input.rs:318-321, 428-431).
    A batch is a list of uint8 [C, h, w] tensors, or a pair (padded uint8 [B, C*maxH*maxW], int32 [B, 2] of (w, h)).
    """

    def setup(self, net, prev):
        cfg: C.Data3dCfg = self.cfg
        md = cfg.max_dims or cfg.in_dims
        Op.setup(self, net, prev)
        mw, mh, c = md
        self.max_hwc = (mh, mw, c)
        self.src_hwc = (mh, mw, c)
        self.crop_h, self.crop_w, self.pad = mh, mw, 0
        self.flip, self.pca, self.mean = False, None, None
        self.scale_range = (0, 0)
        for p in cfg.preprocs:
            if p.kind == "crop":
                self.crop_w, self.crop_h = p.crop_width, p.crop_height
            elif p.kind == "flip_x":
                self.flip = True
            elif p.kind == "pca_noise":
                self.pca = p
            elif p.kind == "scale_bicubic":
                self.scale_range = (int(p.lower), int(p.upper))
            else:
                raise ValueError(f"variable-size input does not support the stage {p.kind!r}")
        if c > 4:
            raise ValueError("variable-size input handles up to 4 channels")
        self.scale = cfg.scale if cfg.scale is not None else (1.0 / 255.0 if cfg.normalize else 1.0)
        self.channel_mean = list(cfg.channel_mean) if cfg.channel_mean is not None else [0.0] * c
        self.out_hwc = (self.crop_h, self.crop_w, c)
        self.out_cp = pad_channels(c)
        self.mode, self.f, self.extra_pad = "nhwc", 1, 0
        self.mean_dev = None
        self.stage = None

    def request_flat(self):
        raise ValueError("a variable-size input cannot feed an affine operator directly")

    def alloc(self):
        mh, mw, c = self.max_hwc
        dev = self.net.device
        n = self.net.batch
        self.in_stride = c * mh * mw
        self.out = torch.zeros(self.out_buffer_shape(), dtype=torch.bfloat16, device=dev)
        self.stage = torch.zeros((n, self.in_stride), dtype=torch.uint8, device=dev)
        self.shapes = torch.ones((n, 2), dtype=torch.int32, device=dev)
        self.draws = torch.zeros((n, 4), dtype=torch.int32, device=dev)

    @staticmethod
    def pack(images, in_stride):
        """List of uint8 [C, h, w] tensors -> (padded [B, in_stride] uint8, [B, 2] int32 of (w, h)) on the host."""
        padded = torch.zeros((len(images), in_stride), dtype=torch.uint8)
        shapes = torch.zeros((len(images), 2), dtype=torch.int32)
        for i, im in enumerate(images):
            c, h, w = im.shape
            if c * h * w > in_stride:
                raise ValueError(f"sample {i} ({w}x{h}) exceeds the configured maximum")
            padded[i, : c * h * w] = im.reshape(-1)
            shapes[i, 0], shapes[i, 1] = w, h
        return padded, shapes

    def load_batch(self, images, non_blocking=True):
        if isinstance(images, torch.Tensor) and images.dim() == 4:
            images = list(images)                       # a batch of equally sized images
        if isinstance(images, (list,)) or (isinstance(images, tuple) and images[0].dim() == 3):
            images = self.pack(list(images), self.in_stride)
        padded, shapes = images
        self.stage.copy_(padded.reshape(self.stage.shape), non_blocking=non_blocking)
        self.shapes.copy_(shapes.reshape(self.shapes.shape).int(), non_blocking=non_blocking)

    def forward(self, train, t):
        mh, mw, c = self.max_hwc
        cfg = self.cfg
        if self.mode == "s2d":
            oh = ow = self.s2d_hw
        else:
            oh, ow = self.crop_h, self.crop_w
        pv = pe = None
        sigma = 0.0
        if self.pca is not None and train:
            sigma, pv, pe = self.pca.std, list(self.pca.eigenvalues), list(self.pca.eigenvectors)
        K.var_input_u8(self.stage, self.shapes, self.out, self.draws, self.in_stride, self.net.batch, c, self.crop_h,
                       self.crop_w, self.out_cp, self.f, self.extra_pad, oh, ow, self.scale_range[0],
                       self.scale_range[1], train, self.flip, cfg.per_batch_draws, self.scale, self.channel_mean,
                       sigma, pv, pe, self.net.data_seed, 0, self.net.step_counter)

    # ---- plain-torch restatement (one sample), the oracle of the kernel
    @staticmethod
    def scaled_dims(w, h, sdim):
        if sdim <= 0:
            return w, h
        f32 = torch.float32
        if w <= h:
            return sdim, int(torch.round(torch.tensor(sdim, dtype=f32) / torch.tensor(w, dtype=f32) * h))
        return int(torch.round(torch.tensor(sdim, dtype=f32) / torch.tensor(h, dtype=f32) * w)), sdim

    @staticmethod
    def ref_sample(img, sdim, ox, oy, flip, crop_w, crop_h):
        """img: [C, h, w] (any dtype). Returns float32 [C, crop_h, crop_w]: Catmull-Rom rescale so that the shorter
        side is `sdim` (0 = none), window at (ox, oy) of the rescaled image, zeros outside it, optional flip."""
        img = img.float()
        c, h, w = img.shape
        rw, rh = VarDataOp.scaled_dims(w, h, sdim)
        xs = torch.arange(crop_w)
        X = ox + (crop_w - 1 - xs if flip else xs)
        Y = oy + torch.arange(crop_h)
        inside = ((Y >= 0) & (Y < rh))[:, None] & ((X >= 0) & (X < rw))[None, :]
        if (rw, rh) == (w, h):
            out = img[:, Y.clamp(0, h - 1)][:, :, X.clamp(0, w - 1)]
            return out * inside

        def taps(P, src, dst):
            f = (P.float() + 0.5) * (torch.tensor(float(src)) / torch.tensor(float(dst))) - 0.5
            fl = torch.floor(f)
            t = f - fl
            t2, t3 = t * t, t * t * t
            wts = torch.stack([-0.5 * t3 + t2 - 0.5 * t, 1.5 * t3 - 2.5 * t2 + 1.0, -1.5 * t3 + 2.0 * t2 + 0.5 * t,
                               0.5 * t3 - 0.5 * t2], 1)                         # [n, 4]
            idx = (fl.long()[:, None] - 1 + torch.arange(4)[None, :]).clamp(0, src - 1)
            return wts, idx

        wx, xi = taps(X, w, rw)
        wy, yi = taps(Y, h, rh)
        rows = img[:, yi.reshape(-1)].reshape(c, crop_h, 4, w)                 # [C, ch, 4, w]
        cols = rows[:, :, :, xi.reshape(-1)].reshape(c, crop_h, 4, crop_w, 4)  # [C, ch, 4(j), cw, 4(k)]
        horiz = (cols * wx[None, None, None]).sum(-1)                           # [C, ch, 4, cw]
        out = (horiz * wy[None, :, :, None]).sum(2)
        return out.clamp(0.0, 255.0) * inside

    def ref_forward(self, x, train, t):
        if isinstance(x, tuple) and not (x[0].dim() == 3):
            padded, shapes = x
            images = []
            c = self.max_hwc[2]
            for i in range(padded.shape[0]):
                w, h = int(shapes[i, 0]), int(shapes[i, 1])
                images.append(padded[i, : c * h * w].reshape(c, h, w))
        else:
            images = list(x)
        g = self.net.ref_generator
        outs = []
        lo, hi = self.scale_range
        mean = torch.tensor(self.channel_mean, dtype=torch.float32).reshape(-1, 1, 1)
        for im in images:
            c, h, w = im.shape
            sdim = (int(torch.randint(lo, hi + 1, (1,), generator=g)) if train else lo) if lo > 0 else 0
            rw, rh = self.scaled_dims(w, h, sdim)
            if train and rw > self.crop_w:
                ox = int(torch.randint(0, rw - self.crop_w + 1, (1,), generator=g))
            else:
                ox = (rw - self.crop_w) // 2
            if train and rh > self.crop_h:
                oy = int(torch.randint(0, rh - self.crop_h + 1, (1,), generator=g))
            else:
                oy = (rh - self.crop_h) // 2
            flip = bool(train and self.flip and int(torch.randint(0, 2, (1,), generator=g)))
            v = self.ref_sample(im, sdim, ox, oy, flip, self.crop_w, self.crop_h)
            xs = torch.arange(self.crop_w)
            X = ox + (self.crop_w - 1 - xs if flip else xs)
            Y = oy + torch.arange(self.crop_h)
            inside = ((Y >= 0) & (Y < rh))[:, None] & ((X >= 0) & (X < rw))[None, :]
            v = v * self.scale - mean
            if train and self.pca is not None and c == 3 and self.pca.std > 0:
                # lighting noise, one draw per image (as in the fixed-size operator)
                al = torch.randn(3, generator=g) * self.pca.std
                vals = torch.tensor(list(self.pca.eigenvalues), dtype=torch.float32)
                vecs = torch.tensor(list(self.pca.eigenvectors), dtype=torch.float32).reshape(3, 3)
                v = v + (vecs @ (al * vals)).reshape(3, 1, 1)
            outs.append(v * inside)
        return torch.stack(outs)


# =============================================================================================== graph plumbing
class _SplitArm:
    """One arm of a Split as its consumer sees it: the shared activation and a delta buffer of its own."""

    def __init__(self, split, index):
        self.split, self.index = split, index
        self.name = f"{split.name}:{index}"
        self.dout = None

    out = property(lambda self: self.split.prev.out)
    out_hwc = property(lambda self: self.split.out_hwc)
    out_cp = property(lambda self: self.split.out_cp)
    # the consumer masks its delta with the shared activation when the producer ends in a ReLU
    has_relu = property(lambda self: self.split.prev.has_relu)


class SplitOp(Op):
    """Fan-out: the activation is shared (no copy), the arms' deltas are summed on backward
    (src/operator/mod.rs:301-384)."""

    def setup(self, net, prev):
        super().setup(net, prev)
        self.out_hwc, self.out_cp = prev.out_hwc, prev.out_cp
        self.arms = [_SplitArm(self, i) for i in range(self.cfg.num_out_arms)]

    def alloc(self):
        if self.net.training_capable:
            for a in self.arms:
                a.dout = torch.zeros_like(self.prev.out)

    def forward(self, train, t):
        pass

    def backward(self):
        if not self.wants_prev_delta():
            return
        d = self.prev.dout
        d.copy_(self.arms[0].dout)
        for a in self.arms[1:]:
            K.add_bf16(d, a.dout, d.numel())

    def ref_forward(self, x, train, t):
        return x


class JoinOp(Op):
    """Fan-in by summation: out = sum of the arms; every arm receives the output's delta."""

    def setup(self, net, prev):
        prevs = list(prev)
        Op.setup(self, net, prevs[0])
        self.prevs = prevs
        for p in prevs[1:]:
            if p.out_hwc != prevs[0].out_hwc:
                raise ValueError(f"join {self.name!r}: arm shapes differ ({p.out_hwc} vs {prevs[0].out_hwc})")
        self.out_hwc, self.out_cp = prevs[0].out_hwc, prevs[0].out_cp

    def forward(self, train, t):
        self.out.copy_(self.prevs[0].out)
        for p in self.prevs[1:]:
            K.add_bf16(self.out, p.out, self.out.numel())

    def backward(self):
        for p in self.prevs:
            if p.dout is None or isinstance(p, DataOp):
                continue
            p.dout.copy_(self.dout)
            if p.has_relu:
                K.relu_mask(p.dout, p.out, p.dout.numel())

    def ref_forward(self, xs, train, t):
        out = xs[0]
        for x in xs[1:]:
            out = out + x
        return out


# =============================================================================================== conv
def conv_out(n, k, s, p):
    return (n + 2 * p - k) // s + 1


class Conv2dOp(Op):
    """Convolution + bias + optional ReLU (src/operator/mod.rs:1366-2003), on the tcgen05 implicit-GEMM kernel."""

    has_params = True

    def setup(self, net, prev):
        super().setup(net, prev)
        cfg = self.cfg
        h, w, c = prev.out_hwc
        self.in_c = c
        k, s, p = cfg.conv_size, cfg.conv_stride, cfg.conv_pad
        self.P, self.Q = conv_out(h, k, s, p), conv_out(w, k, s, p)
        self.s2d = False
        if isinstance(prev, DataOp) and s > 1 and c <= 4 and h == w and prev.mode == "nhwc":
            f, r2, out_hw, s2d_hw = layout.s2d_geometry(k, s, h + 2 * p)
            prev.request_s2d(f, s2d_hw, p)
            self.s2d, self.f, self.r2, self.s2d_hw = True, f, r2, s2d_hw
        self.cp = prev.out_cp
        self.out_hwc = (self.P, self.Q, cfg.out_channels)
        self.out_cp = pad_channels(cfg.out_channels)
        self._setup_act(cfg.act, getattr(cfg, "act_param", None))
        self.direct = getattr(cfg, "backend", C.ConvBackend.TENSOR_CORE) == C.ConvBackend.DIRECT
        rs = self.r2 * self.r2 if self.s2d else k * k
        self.rs = rs
        self.seg_w = ParamSeg(self.name + ".w", (cfg.out_channels, rs, self.cp))
        self.segs = [self.seg_w]
        self.seg_b = None
        if getattr(cfg, "bias", True):
            self.seg_b = ParamSeg(self.name + ".b", (cfg.out_channels,))
            self.segs.append(self.seg_b)
        self.wt16 = None

    def alloc(self):
        super().alloc()
        if self.net.training_capable and self.wants_prev_delta() and self.cfg.conv_stride == 1:
            self.wt16 = torch.zeros((self.cp, self.rs, self.out_cp), dtype=torch.bfloat16, device=self.net.device)
        if self.net.device.type == "cuda" and not self.direct:
            self._tune()

    def _tune(self):
        """Measure the tile plans of this layer's forward and data-grad shapes once, on scratch operands."""
        h, w, r, s, p = self._geom()
        n, ko = self.net.batch, self.cfg.out_channels
        K.tune_conv(n, h, w, self.cp, ko, r, r, s, p, p, self.P, self.Q, self.out_cp, relu=self.has_relu,
                    has_bias=self.seg_b is not None, n_valid=ko, n_store=self.out_cp)
        if self.wt16 is not None:
            K.tune_conv(n, self.P, self.Q, self.out_cp, self.cp, r, r, 1, r - 1 - p, r - 1 - p, h, w, self.cp,
                        has_mask=self.mask_src() is not None, n_valid=self.in_c, n_store=self.cp)

    # geometry the kernels see (the s2d form is a stride-1, pad-0 convolution on the rearranged input)
    def _geom(self):
        if self.s2d:
            return self.s2d_hw, self.s2d_hw, self.r2, 1, 0
        h, w, _ = self.prev.out_hwc
        return h, w, self.cfg.conv_size, self.cfg.conv_stride, self.cfg.conv_pad

    def forward(self, train, t):
        h, w, r, s, p = self._geom()
        ko = self.cfg.out_channels
        if self.direct:
            K.conv_direct_fwd(self.prev.out, self.view(self.seg_w, "params16"),
                              self.view(self.seg_b) if self.seg_b else None, self.out, self.net.batch, h, w, self.cp,
                              ko, self.out_cp, r, r, s, p, p, self.P, self.Q, self.has_relu)
            self._act_forward()
            return
        if train and self.wt16 is not None:
            # the data-grad reads the filters transposed and flipped; re-packing them depends on the weights alone,
            # so it runs beside the forward pass
            w16 = self.view(self.seg_w, "params16")
            self.net.side(lambda: K.pack_dgrad_filters(w16, self.wt16, ko, self.out_cp, r * r, self.cp))
        K.conv_fprop_tc(self.prev.out, self.net.batch, h, w, self.cp, self.view(self.seg_w, "params16"), ko, r, r, s,
                        p, p, self.P, self.Q, self.out, self.out_cp,
                        bias=self.view(self.seg_b) if self.seg_b else None, relu=self.has_relu, n_valid=ko,
                        n_store=self.out_cp)
        self._act_forward()

    def backward(self):
        h, w, r, s, p = self._geom()
        n, ko = self.net.batch, self.cfg.out_channels
        rows = n * self.P * self.Q
        self._act_backward()
        if self.seg_b:
            gb = self.view(self.seg_b, "grads")
            self.net.side(lambda: K.colsum(self.dout, rows, self.out_cp, ko, gb))     # beside weight- and data-grad
        gw = self.view(self.seg_w, "grads")
        if self.direct:
            K.conv_direct_wgrad(self.prev.out, self.dout, gw, n, h, w, self.cp, ko, self.out_cp, r, r, s, p, p, self.P,
                                self.Q)
        else:
            K.conv_wgrad_tc(self.prev.out, n, h, w, self.cp, self.dout, self.out_cp, ko, r, r, s, p, p, self.P,
                            self.Q, gw)
        if self.s2d:
            K.zero_s2d_structural(gw, ko, self.r2, self.cp, self.f, self.in_c, self.cfg.conv_size)
        if self.wants_prev_delta():
            mask = self.mask_src()
            w16 = self.view(self.seg_w, "params16")
            if self.direct:
                K.conv_direct_dgrad(self.dout, w16, self.prev.dout, mask, n, h, w, self.cp, ko, self.out_cp, r, r, s,
                                    p, p, self.P, self.Q)
            elif s == 1:
                K.conv_fprop_tc(self.dout, n, self.P, self.Q, self.out_cp, self.wt16, self.cp, r, r, 1, r - 1 - p,
                                r - 1 - p, h, w, self.prev.dout, self.cp, mask_src=mask, n_valid=self.in_c,
                                n_store=self.cp)
            else:
                done = False
                if _strided_dgrad_on_tensor_cores():
                    if not hasattr(self, "_sd_cache"):
                        self._sd_cache = {}
                    done = dgrad_strided_tc(self.dout, n, self.P, self.Q, self.out_cp, w16, ko, self.cp, self.in_c, r, r,
                                            s, p, h, w, self.prev.dout, mask, cache=self._sd_cache)
                if not done:
                    K.conv_direct_dgrad(self.dout, w16, self.prev.dout, mask, n, h, w, self.cp, ko, self.out_cp, r, r,
                                        s, p, p, self.P, self.Q)

    # ---- parameters in reference layout
    def _w_ref(self, w_int):
        k = self.cfg.conv_size
        if self.s2d:
            return layout.s2d_weight_from_internal(w_int, self.in_c, k, self.f)
        return layout.conv_weight_from_internal(w_int, self.in_c, k, k)

    def _w_int(self, w_oihw):
        if self.s2d:
            return layout.s2d_weight_to_internal(w_oihw, self.f, self.cp)
        return layout.conv_weight_to_internal(w_oihw, self.cp)

    def init_params(self, rng):
        cfg = self.cfg
        k = cfg.conv_size
        if cfg.init_weights.kind == "xavier":
            raise NotImplementedError("Xavier initialisation is not defined for convolutions in the reference "
                                      "(src/operator/mod.rs:1576-1579)")
        w = _draw(cfg.init_weights, rng, (cfg.out_channels, self.in_c, k, k), k * k * self.in_c, cfg.out_channels)
        self.view(self.seg_w).copy_(self._w_int(w))
        if self.seg_b:
            self.view(self.seg_b).zero_()

    def encode_params(self):
        cfg = self.cfg
        k = cfg.conv_size
        w = self._w_ref(self.view(self.seg_w).detach().float().cpu())
        out = [(w.reshape(-1), (k * k * self.in_c, cfg.out_channels))]
        if self.seg_b:
            out.append((self.view(self.seg_b).detach().float().cpu(), (1, cfg.out_channels)))
        return out

    def decode_params(self, arrays):
        cfg = self.cfg
        k = cfg.conv_size
        w = torch.as_tensor(arrays[0][0]).reshape(cfg.out_channels, self.in_c, k, k)
        self.view(self.seg_w).copy_(self._w_int(w))
        if self.seg_b:
            self.view(self.seg_b).copy_(torch.as_tensor(arrays[1][0]).reshape(-1))
            return 2
        return 1

    def ref_forward(self, x, train, t):
        cfg = self.cfg
        w = self._w_ref(self.view(self.seg_w))
        b = self.view(self.seg_b) if self.seg_b else None
        y = F.conv2d(x, w, b, stride=cfg.conv_stride, padding=cfg.conv_pad)
        return self._ref_act(y)


class ResConv2dOp(Conv2dOp):
    """out = act(conv(x) + b + x): a residual convolution without normalisation (ResidualConv2dLayer,
    src/layer_new.rs:1179-1418). The convolution and its gradients are those of `Conv2dOp`; the identity path is an
    elementwise add before the activation in forward and an add into the producer's delta in backward."""

    def setup(self, net, prev):
        rc = self.cfg
        h, w, c = prev.out_hwc
        if rc.conv_size % 2 == 0:
            raise ValueError("a residual convolution needs an odd filter size (same-size output)")
        self.res_cfg = rc
        self.cfg = C.Conv2dCfg(rc.conv_size, 1, rc.conv_size // 2, c, C.Act.IDENTITY, rc.init_weights, rc.bias)
        super().setup(net, prev)
        if self.s2d or self.out_cp != prev.out_cp:
            raise ValueError("a residual convolution cannot be the first hidden operator of a strided input")
        self._setup_act(rc.act, rc.act_param)     # applied after the sum, not in the convolution's epilogue

    @contextlib.contextmanager
    def _conv_only(self):
        """While active, the inherited forward / backward see a plain linear convolution."""
        saved = (self.has_relu, self.act_kind)
        self.has_relu, self.act_kind = False, 0
        try:
            yield
        finally:
            self.has_relu, self.act_kind = saved

    def forward(self, train, t):
        with self._conv_only():
            super().forward(train, t)
        K.add_bf16(self.out, self.prev.out, self.out.numel())
        if self.has_relu:
            K.act_fwd(self.out, self._act_rows(), self.out_cp, self.out_hwc[2], K.ACT_RECT, 0.0)
        else:
            self._act_forward()

    def backward(self):
        self._act_backward()          # smooth activations; a ReLU was already applied to dout by the consumer
        with self._conv_only():
            super().backward()
        if self.wants_prev_delta():
            n = self.dout.numel()
            K.add_bf16(self.prev.dout, self.dout, n)
            if self.prev.has_relu:    # the identity path passes through the producer's ReLU as well
                K.relu_mask(self.prev.dout, self.prev.out, n)

    def ref_forward(self, x, train, t):
        cfg = self.cfg
        w = self._w_ref(self.view(self.seg_w))
        b = self.view(self.seg_b) if self.seg_b else None
        return self._ref_act(F.conv2d(x, w, b, stride=1, padding=cfg.conv_pad) + x)


# =============================================================================================== affine
class AffineOp(Op):
    """Fully connected layer + bias + optional ReLU (src/operator/mod.rs:838-1364).

    Forward and data-gradient split their reduction over many CTAs (the batch gives a single 128-row tile),
    accumulate in an fp32 workspace with red.add and finish with a small bias/activation kernel.
    """

    has_params = True

    def setup(self, net, prev):
        super().setup(net, prev)
        cfg = self.cfg
        if isinstance(prev, DataOp) and prev.mode == "nhwc" and prev.out_hwc[0] == prev.out_hwc[1]:
            prev.request_flat()
        h, w, c = prev.out_hwc
        self.in_hw_c = (h, w, c)
        if isinstance(prev, DataOp) and prev.mode == "flat":
            self.in_pixel_cp = c            # flat mode packs pixels tightly, padding only at the end
            self.k_in = prev.out_cp
        else:
            self.in_pixel_cp = prev.out_cp
            self.k_in = h * w * prev.out_cp
        self.out_hwc = (1, 1, cfg.out_channels)
        self.out_cp = pad_channels(cfg.out_channels)
        self._setup_act(cfg.act, getattr(cfg, "act_param", None))
        self.seg_w = ParamSeg(self.name + ".w", (cfg.out_channels, self.k_in))
        self.seg_b = ParamSeg(self.name + ".b", (cfg.out_channels,)) if getattr(cfg, "bias", True) else None
        self.segs = [self.seg_w] + ([self.seg_b] if self.seg_b else [])

    def alloc(self):
        super().alloc()
        n = self.net.batch
        self.ws = torch.zeros((n, self.out_cp), dtype=torch.float32, device=self.net.device)
        self.ws_in = None
        if self.net.training_capable and self.wants_prev_delta():
            self.ws_in = torch.zeros((n, self.k_in), dtype=torch.float32, device=self.net.device)

    @staticmethod
    def _bn_cap(n_cols, m_tiles=1):
        """Tile width of the forward / data-grad GEMMs. The batch gives one 128-row tile, so every column tile loads
        the whole activation panel again: wide tiles keep those re-reads (the larger share of the rows the TMA unit
        has to fetch) down, and the reduction split spreads the work over the SMs instead."""
        forced = os.environ.get("RB_FC_BN")
        if forced:
            return int(forced)
        if n_cols >= 2048:
            return 256
        if n_cols >= 1024:
            return 128
        return 64

    def forward(self, train, t):
        n, ko = self.net.batch, self.cfg.out_channels
        x = self.prev.out
        K.gemm_tc(x, 0, self.k_in, self.view(self.seg_w, "params16"), 0, self.k_in, n, ko, self.k_in, self.ws,
                  self.out_cp, epi=K.EPI_F32_ATOMIC, n_store=self.out_cp, split_k=0, bn_cap=self._bn_cap(ko))
        K.bias_act(self.ws, n, self.out_cp, ko, self.view(self.seg_b) if self.seg_b else None, self.has_relu,
                   self.out)
        self._act_forward()

    def backward(self):
        n, ko = self.net.batch, self.cfg.out_channels
        self._act_backward()
        if self.seg_b:
            gb = self.view(self.seg_b, "grads")
            self.net.side(lambda: K.colsum(self.dout, n, self.out_cp, ko, gb))
        # dW[out][in] += dY^T X : both operands are read "MN-major" straight from their row-major buffers
        # one pass over the batch: overwrite when this is the only micro-batch of the iteration, else accumulate
        epi = K.EPI_F32_ATOMIC if self.net.accumulate else K.EPI_F32_STORE
        K.gemm_tc(self.dout, 1, self.out_cp, self.prev.out, 1, self.k_in, ko, self.k_in, n,
                  self.view(self.seg_w, "grads"), self.k_in, epi=epi, n_store=self.k_in, split_k=1)
        if self.wants_prev_delta():
            K.gemm_tc(self.dout, 0, self.out_cp, self.view(self.seg_w, "params16"), 1, self.k_in, n, self.k_in,
                      ko, self.ws_in, self.k_in, epi=K.EPI_F32_ATOMIC, n_store=self.k_in, split_k=0,
                      bn_cap=self._bn_cap(self.k_in))
            K.bias_act(self.ws_in, n, self.k_in, self.k_in, None, False, self.prev.dout, mask_src=self.mask_src())

    def _w_ref(self, w_int):
        h, w, c = self.in_hw_c
        o = self.cfg.out_channels
        tight = w_int[:, : h * w * self.in_pixel_cp] if self.in_pixel_cp == c else w_int
        return layout.affine_weight_from_internal(tight, c, h, w, self.in_pixel_cp)

    def _w_int(self, w_ref):
        h, w, c = self.in_hw_c
        t = layout.affine_weight_to_internal(w_ref, c, h, w, self.in_pixel_cp)
        out = torch.zeros((w_ref.shape[0], self.k_in), dtype=w_ref.dtype)
        out[:, : t.shape[1]] = t
        return out

    def init_params(self, rng):
        cfg = self.cfg
        h, w, c = self.in_hw_c
        fan_in = h * w * c
        wr = _draw(cfg.init_weights, rng, (cfg.out_channels, fan_in), fan_in, cfg.out_channels)
        self.view(self.seg_w).copy_(self._w_int(wr))
        if self.seg_b:
            self.view(self.seg_b).zero_()

    def encode_params(self):
        h, w, c = self.in_hw_c
        o = self.cfg.out_channels
        wr = self._w_ref(self.view(self.seg_w).detach().float().cpu())
        recs = [(wr.reshape(-1), (h * w * c, o))]
        if self.seg_b:
            recs.append((self.view(self.seg_b).detach().float().cpu(), (1, o)))
        return recs

    def decode_params(self, arrays):
        h, w, c = self.in_hw_c
        o = self.cfg.out_channels
        self.view(self.seg_w).copy_(self._w_int(torch.as_tensor(arrays[0][0]).reshape(o, h * w * c)))
        if not self.seg_b:
            return 1
        self.view(self.seg_b).copy_(torch.as_tensor(arrays[1][0]).reshape(-1))
        return 2

    def ref_forward(self, x, train, t):
        wr = self._w_ref(self.view(self.seg_w))
        y = x.flatten(1) @ wr.t()
        y = self._ref_act(y + self.view(self.seg_b) if self.seg_b else y)
        return y.reshape(y.shape[0], -1, 1, 1)


# =============================================================================================== pool / lrn / dropout
class Pool2dOp(Op):
    """Max / average pooling with optional fused ReLU (src/operator/mod.rs:2005-2132; act_func on pool layers
    appears in examples/imagenet_alexnet.model:38-44)."""

    def setup(self, net, prev):
        super().setup(net, prev)
        cfg = self.cfg
        h, w, c = prev.out_hwc
        k, s, p = cfg.pool_size, cfg.pool_stride, cfg.pool_pad

        def out(n):
            if cfg.ceil_mode:
                o = -(-(n + 2 * p - k) // s) + 1
                if (o - 1) * s >= n + p:   # the last window must start inside the image or its left padding
                    o -= 1
                return o
            return (n + 2 * p - k) // s + 1

        self.P, self.Q = out(h), out(w)
        self.out_hwc = (self.P, self.Q, c)
        self.out_cp = prev.out_cp
        self.is_max = cfg.kind == C.PoolKind.MAX
        if cfg.act not in (C.Act.RECT, C.Act.IDENTITY):
            raise ValueError(f"{self.name}: a pooling operator takes a rect activation or none, not {cfg.act.value}")
        self.fused_relu = cfg.act == C.Act.RECT
        # the output is non-negative if this op or its producer applied a ReLU; consumers then mask by it
        self.has_relu = self.fused_relu
        self.idx = None

    def alloc(self):
        super().alloc()
        if self.is_max:
            self.idx = torch.zeros(self.out.shape, dtype=torch.uint8, device=self.net.device)

    def forward(self, train, t):
        h, w, _ = self.prev.out_hwc
        cfg = self.cfg
        K.pool_fwd(self.prev.out, self.out, self.idx, self.net.batch, h, w, self.out_cp, self.P, self.Q, cfg.pool_size,
                   cfg.pool_stride, cfg.pool_pad, self.is_max, self.fused_relu)

    def backward(self):
        if not self.wants_prev_delta():
            return
        h, w, _ = self.prev.out_hwc
        cfg = self.cfg
        K.pool_bwd(self.dout, self.idx, self.out if (self.fused_relu and not self.is_max) else None, self.prev.dout,
                   self.mask_src(), self.net.batch, h, w, self.out_cp, self.P, self.Q, cfg.pool_size, cfg.pool_stride,
                   cfg.pool_pad, self.is_max)

    def ref_forward(self, x, train, t):
        cfg = self.cfg
        if self.is_max:
            y = F.max_pool2d(x, cfg.pool_size, cfg.pool_stride, cfg.pool_pad, ceil_mode=cfg.ceil_mode)
        else:
            y = F.avg_pool2d(x, cfg.pool_size, cfg.pool_stride, cfg.pool_pad, ceil_mode=cfg.ceil_mode,
                             count_include_pad=True)
        return torch.relu(y) if self.fused_relu else y


class LrnOp(Op):
    """Cross-channel local response normalisation (a real one; the reference's is a pass-through stub,
    src/layer.rs:1846-1899)."""

    def setup(self, net, prev):
        super().setup(net, prev)
        self.out_hwc = prev.out_hwc
        self.out_cp = prev.out_cp
        cfg = self.cfg
        self.alpha_eff = cfg.scale / cfg.cross_size if cfg.alpha_div_n else cfg.scale
        self.has_relu = False

    def forward(self, train, t):
        h, w, _ = self.out_hwc
        cfg = self.cfg
        K.lrn_fwd(self.prev.out, self.out, self.net.batch * h * w, self.out_cp, cfg.cross_size, self.alpha_eff,
                  cfg.power, cfg.min_div)

    def backward(self):
        if not self.wants_prev_delta():
            return
        h, w, _ = self.out_hwc
        cfg = self.cfg
        K.lrn_bwd(self.prev.out, self.dout, self.prev.dout, self.mask_src(), self.net.batch * h * w, self.out_cp,
                  cfg.cross_size, self.alpha_eff, cfg.power, cfg.min_div)

    def ref_forward(self, x, train, t):
        cfg = self.cfg
        return F.local_response_norm(x, cfg.cross_size, alpha=self.alpha_eff * cfg.cross_size, beta=cfg.power,
                                     k=cfg.min_div)


class DropoutOp(Op):
    """Inverted dropout with an in-kernel Philox mask (src/operator/mod.rs:2134-2255); inference is a copy."""

    def setup(self, net, prev):
        super().setup(net, prev)
        self.out_hwc = prev.out_hwc
        self.out_cp = prev.out_cp
        self.has_relu = False
        self.stream_id = net.next_stream_id()
        self._t = 0

    def forward(self, train, t):
        n = self.out.numel()
        self._t = t
        if train:
            K.dropout(self.prev.out, self.out, n, self.cfg.drop_ratio, self.net.dropout_seed, self.stream_id,
                      step_ptr=self.net.step_counter)
        else:
            self.out.copy_(self.prev.out)

    def backward(self):
        if not self.wants_prev_delta():
            return
        K.dropout(self.dout, self.prev.dout, self.dout.numel(), self.cfg.drop_ratio, self.net.dropout_seed,
                  self.stream_id, mask_src=self.mask_src(), step_ptr=self.net.step_counter)

    def ref_forward(self, x, train, t):
        if not train:
            return x
        p = self.cfg.drop_ratio
        keep = (torch.rand(x.shape, generator=self.net.ref_generator) >= p).to(x.dtype)
        return x * keep / (1.0 - p)


# =============================================================================================== loss
class SoftmaxKLLossOp(Op):
    """Softmax + cross-entropy head with per-sample weights (src/operator/loss.rs:20-262).

    Optional admissibility masks (`load_mask`): categories whose mask byte is zero get probability zero and the rest
    is renormalised, as the gen-2 head does for legal moves (src/layer_new.rs:2057-2096).
    """

    heads = 1

    def setup(self, net, prev):
        super().setup(net, prev)
        self.k = self.cfg.num_categories
        self.heads = int(getattr(self.cfg, "num_heads", 1))
        h, w, c = prev.out_hwc
        if h * w * c != self.k * self.heads:
            raise ValueError(f"loss expects {self.k * self.heads} inputs, previous operator produces {h * w * c}")
        self.out_hwc = prev.out_hwc
        self.out_cp = prev.out_cp
        self.cat_weights = None
        self.mask = None
        self._cpu_mask = None
        self.soft = None          # target distributions (distillation), [B * heads, K] float32
        self._setup_flat()

    def _setup_flat(self):
        """A spatial producer (e.g. the 19 x 19 x 1 move plane of a Go network) leaves its outputs pixel-major with
        padded channels; the head wants one dense row per sample in the reference's order (channel slowest:
        index = x + W * (y + H * c)). `flat` / `dflat` are that row and its delta; copies in and out are strided
        device copies into fixed buffers."""
        h, w, c = self.prev.out_hwc
        self.spatial = h * w > 1
        self.flat = self.dflat = None
        self.ld = pad_channels(h * w * c) if self.spatial else self.prev.out_cp

    def _alloc_flat(self):
        if self.spatial and self.net.is_cuda:
            n = self.net.batch
            self.flat = torch.zeros((n, self.ld), dtype=torch.bfloat16, device=self.net.device)
            if self.net.training_capable:
                self.dflat = torch.zeros_like(self.flat)

    def _as_planes(self, buf):
        h, w, c = self.prev.out_hwc
        return buf[:, : h * w * c].view(self.net.batch, c, h, w)

    def _logits(self):
        """(logits buffer, its delta buffer or None) handed to the loss kernel."""
        if not self.spatial:
            return self.prev.out, self.prev.dout
        c = self.prev.out_hwc[2]
        self._as_planes(self.flat).copy_(self.prev.out[..., :c].permute(0, 3, 1, 2))
        return self.flat, self.dflat

    def _scatter_delta(self):
        if self.spatial:
            c = self.prev.out_hwc[2]
            self.prev.dout[..., :c].copy_(self._as_planes(self.dflat).permute(0, 2, 3, 1))

    def alloc(self):
        dev = self.net.device
        n = self.net.batch
        self.labels = torch.zeros(n * self.heads, dtype=torch.int32, device=dev)
        self.weights = None
        self.loss_sum = torch.zeros(1, dtype=torch.float32, device=dev)
        self.correct = torch.zeros(1, dtype=torch.int32, device=dev)
        self.argmax = torch.zeros(n, dtype=torch.int32, device=dev)
        self.loss_per = torch.zeros(n * self.heads, dtype=torch.float32, device=dev)
        self.probs = None
        self._alloc_flat()

    def load_labels(self, labels, non_blocking=True):
        self.labels.copy_(labels.reshape(-1), non_blocking=non_blocking)

    def load_weights(self, weights):
        if self.weights is None:
            self.weights = torch.zeros(self.net.batch, dtype=torch.float32, device=self.net.device)
        self.weights.copy_(weights)

    def load_mask(self, mask):
        """mask: [B, K] (or [B, heads, K]), non-zero = admissible; None removes the mask."""
        if mask is None:
            self.mask = self._cpu_mask = None
            return
        m = (torch.as_tensor(mask) != 0).reshape(self.net.batch * self.heads, self.k)
        if self.net.is_cuda:
            if self.mask is None:
                self.mask = torch.zeros(m.shape, dtype=torch.uint8, device=self.net.device)
            self.mask.copy_(m.to(torch.uint8))
        else:
            self._cpu_mask = m

    def enable_probs(self):
        """Keep the softmax probabilities of every forward pass (a teacher network's output)."""
        if self.net.is_cuda and self.probs is None:
            self.probs = torch.zeros((self.net.batch * self.heads, self.k), dtype=torch.float32,
                                     device=self.net.device)
        self.keep_probs = True

    def sample_categories(self, temperature: float = 1.0, generator=None, seed: Optional[int] = None) -> torch.Tensor:
        """Draw one category per sample (head 0) from softmax(logits / temperature), restricted to the admissible
        categories when a mask is loaded: the Boltzmann sampling of the gen-1 softmax head (src/layer.rs:2456,
        prefix-sum CDF + uniform draw). Call after `forward`. On a GPU this is one kernel (per-sample warp, prefix
        sums, Philox draw keyed by `seed` and the number of draws so far); on CPU `torch.multinomial`."""
        n = self.net.batch
        if self.net.device.type == "cuda":
            logits = self.flat if self.spatial else self.prev.out.reshape(n, -1)
            mask = None
            if self.mask is not None:
                mask = self.mask.reshape(n, self.heads, self.k)[:, 0].contiguous()
            if not hasattr(self, "_sampled"):
                self._sampled = torch.zeros(n, dtype=torch.int32, device=self.net.device)
                self._draws = 0
            self._draws += 1
            K.sample_categories(logits, n, self.k, logits.shape[1], mask, max(float(temperature), 1e-6),
                                self.net.dropout_seed if seed is None else seed, self._draws, self._sampled)
            return self._sampled.long()
        if self.net.is_cuda:
            logits = (self.flat if self.spatial else self.prev.out.reshape(n, -1))[:, : self.k].float()
            mask = None if self.mask is None else self.mask.reshape(n, self.heads, self.k)[:, 0].bool()
        else:
            logits = self.net._cpu_logits.flatten(1)[:, : self.k].float()
            mask = None if self._cpu_mask is None else self._cpu_mask.reshape(n, self.heads, self.k)[:, 0]
        logits = logits / max(float(temperature), 1e-6)
        if mask is not None:
            logits = logits.masked_fill(~mask, float("-inf"))
        probs = torch.softmax(logits, dim=1)
        return torch.multinomial(probs, 1, generator=generator).squeeze(1)

    def load_soft_targets(self, q):
        """q: [B * heads, K] distribution that replaces the one-hot labels; None returns to hard labels."""
        if q is None:
            self.soft = None
            return
        q = q.reshape(self.net.batch * self.heads, self.k).float()
        if self.net.is_cuda:
            # a persistent buffer: captured graphs keep reading the same address
            if self.soft is None:
                self.soft = torch.zeros_like(q, device=self.net.device)
            self.soft.copy_(q, non_blocking=True)
        else:
            self.soft = q

    def forward(self, train, t):
        logits, dbuf = self._logits()
        delta = dbuf if (train and self.prev.dout is not None) else None
        K.softmax_ce(logits, self.net.batch, self.k, self.ld, self.labels, self.weights,
                     self.net.sample_weight, delta, probs=self.probs, loss_sum=self.loss_sum, correct=self.correct,
                     loss_per=self.loss_per, argmax_out=self.argmax, cat_weights=self.cat_weights, mask=self.mask,
                     heads=self.heads, soft=self.soft)
        if delta is not None:
            self._scatter_delta()

    def ref_loss(self, logits, labels, weights=None):
        """Returns (weighted loss sum, number correct, argmax)."""
        n = logits.shape[0]
        logits = logits.flatten(1).reshape(n * self.heads, self.k)
        if self.cat_weights is not None and logits.requires_grad:
            # per-category weights act on the gradient only (as in the kernel): delta[b, k] *= cw[k]
            cw = self.cat_weights.to(logits.device).reshape(1, -1)
            logits = logits * 1.0
            logits.register_hook(lambda g: g * cw)
        if self._cpu_mask is not None:
            logits = logits.masked_fill(~self._cpu_mask, float("-inf"))
        labels = labels.long().reshape(-1)
        live = (labels >= 0) & (labels < self.k)
        lp = F.log_softmax(logits, dim=1)
        if getattr(self, "keep_probs", False):
            self.probs = lp.detach().exp()
        if self.soft is not None:
            q = self.soft.to(lp.device)
            nll = -(torch.where(q > 0, q * lp, torch.zeros_like(lp))).sum(1)
        else:
            nll = -lp.gather(1, labels.clamp(0, self.k - 1).reshape(-1, 1)).squeeze(1)
            nll = torch.where(live, nll, torch.zeros_like(nll))
        if weights is not None:
            w = weights.reshape(-1, 1).expand(n, self.heads).reshape(-1)
        else:
            w = torch.full_like(nll, self.net.sample_weight)
        am = logits.reshape(n, self.heads, self.k)[:, 0].argmax(1)
        first = labels.reshape(n, self.heads)[:, 0]
        return (w * nll).sum(), int((am == first).sum()), am


class MultiSoftmaxKLLossOp(SoftmaxKLLossOp):
    """k-step look-ahead heads: `num_heads` blocks of `num_categories` logits per sample, one label per head
    (negative = no target for that step); the loss is the sum over heads, accuracy is that of the first head
    (src/layer_new.rs:2969-3118)."""


class PointwiseLossOp(SoftmaxKLLossOp):
    """Heads that compare every output with a float target: logistic (binary cross-entropy on the logit; the gen-2
    LogisticIndicatorLossLayer, src/layer_new.rs) and L2 (the gen-1 L2LossLayer, src/layer.rs). Targets are loaded
    with `load_labels` as [B, K] floats (a [B] integer tensor is taken as K = 1 binary labels)."""

    def setup(self, net, prev):
        Op.setup(self, net, prev)
        self.k = self.cfg.num_outputs
        self.heads = 1
        self.mode = {"logistic": 0, "l2": 1}[self.cfg.kind]
        h, w, c = prev.out_hwc
        if h * w * c != self.k:
            raise ValueError(f"loss expects {self.k} inputs, previous operator produces {h * w * c}")
        self.out_hwc, self.out_cp = prev.out_hwc, prev.out_cp
        self.cat_weights = self.mask = self._cpu_mask = self.soft = None
        self._setup_flat()

    def alloc(self):
        super().alloc()
        self.targets = torch.zeros((self.net.batch, self.k), dtype=torch.float32, device=self.net.device)

    # True: the targets are written by `load_targets` (e.g. a teacher network's activations) and the labels that
    # arrive with a batch are ignored
    hold_targets = False

    def load_labels(self, labels, non_blocking=True):
        if self.hold_targets:
            return
        self.targets.copy_(labels.reshape(self.net.batch, self.k).float(), non_blocking=non_blocking)

    def load_targets(self, targets, non_blocking=True):
        """Float targets [B, K] from elsewhere than the batch's labels; they stay until the next call."""
        self.hold_targets = True
        if not hasattr(self, "targets"):     # host path: no device buffers are allocated
            self.targets = torch.zeros((self.net.batch, self.k), dtype=torch.float32)
        self.targets.copy_(targets.reshape(self.net.batch, self.k).float(), non_blocking=non_blocking)

    def forward(self, train, t):
        logits, dbuf = self._logits()
        delta = dbuf if (train and self.prev.dout is not None) else None
        K.pointwise_loss(logits, self.net.batch, self.k, self.ld, self.targets, self.weights,
                         self.net.sample_weight, delta, loss_sum=self.loss_sum, correct=self.correct, mode=self.mode)
        if delta is not None:
            self._scatter_delta()

    def ref_loss(self, logits, labels, weights=None):
        n = logits.shape[0]
        x = logits.flatten(1)
        t = self.targets.to(x.device) if self.hold_targets else labels.reshape(n, self.k).float()
        if self.mode == 0:
            per = F.binary_cross_entropy_with_logits(x, t, reduction="none").sum(1)
            correct = int(((x[:, 0] > 0) == (t[:, 0] > 0.5)).sum())
        else:
            per = 0.5 * ((x - t) ** 2).sum(1)
            correct = 0
        w = weights if weights is not None else torch.full_like(per, self.net.sample_weight)
        return (w * per).sum(), correct, (x[:, 0] > 0).long()


class CategoricalObjLossOp(SoftmaxKLLossOp):
    """Softmax indicator, antilogistic + KL and antilogistic indicator heads (src/layer_new.rs:2136, :2637, :2859).

    The reference's kernels for these heads are not in its tree; the maths is inferred from the call sites and written
    out in `csrc/softmax_ce.cu` (`categorical_obj_kernel`): the indicator heads maximise the (normalised) mass on the
    target, loss = 1 - mass; the antilogistic heads normalise non-negative scores by their plain sum instead of a
    softmax. `set_target_weights` gives the softmax indicator a weight per category in place of the one-hot label
    (the marginalised form of src/operator/loss.rs:264-407)."""

    KINDS = {"softmax_ind": K.OBJ_SOFTMAX_IND, "antilogistic_kl": K.OBJ_ANTILOGISTIC_KL,
             "antilogistic_ind": K.OBJ_ANTILOGISTIC_IND}

    def setup(self, net, prev):
        super().setup(net, prev)
        if self.cfg.kind not in self.KINDS:
            raise ValueError(f"unknown categorical objective {self.cfg.kind!r}")
        self.objective = self.KINDS[self.cfg.kind]
        self.target_w = None

    def set_target_weights(self, tw):
        if self.objective != K.OBJ_SOFTMAX_IND:
            raise ValueError("category weights exist for the softmax indicator head only")
        self.target_w = None if tw is None else torch.as_tensor(tw, dtype=torch.float32, device=self.net.device)

    def forward(self, train, t):
        logits, dbuf = self._logits()
        delta = dbuf if (train and self.prev.dout is not None) else None
        K.categorical_loss(logits, self.net.batch, self.k, self.ld, self.labels, self.weights, self.net.sample_weight,
                           delta, self.objective, probs=self.probs, loss_sum=self.loss_sum, correct=self.correct,
                           argmax_out=self.argmax, mask=self.mask, target_w=self.target_w)
        if delta is not None:
            self._scatter_delta()

    def ref_loss(self, logits, labels, weights=None):
        n = logits.shape[0]
        x = logits.flatten(1).reshape(n, self.k)
        labels = labels.long().reshape(-1)
        live = (labels >= 0) & (labels < self.k)
        keep = None if self._cpu_mask is None else self._cpu_mask.reshape(n, self.k)
        if self.objective == K.OBJ_SOFTMAX_IND:
            v = torch.softmax(x if keep is None else x.masked_fill(~keep, float("-inf")), dim=1)
        else:
            pos = x.clamp_min(0.0) if keep is None else x.clamp_min(0.0) * keep
            v = pos / pos.sum(1, keepdim=True).clamp_min(1e-6)
        if self.target_w is not None:
            mass = (v * self.target_w.to(v.device).reshape(1, -1)).sum(1)
            live = torch.ones_like(live)
        else:
            mass = v.gather(1, labels.clamp(0, self.k - 1).reshape(-1, 1)).squeeze(1)
        per = -torch.log(mass.clamp_min(1e-6)) if self.objective == K.OBJ_ANTILOGISTIC_KL else 1.0 - mass
        per = torch.where(live, per, torch.zeros_like(per))
        if getattr(self, "keep_probs", False):
            self.probs = v.detach()
        w = weights.reshape(-1) if weights is not None else torch.full_like(per, self.net.sample_weight)
        masked = x if keep is None else x.masked_fill(~keep, float("-inf"))
        am = masked.argmax(1)
        return (w * per).sum(), int((am == labels).sum()), am


class MarginalizedSoftmaxIndLossOp(SoftmaxKLLossOp):
    """Softmax head whose gradient is weighted per category (src/operator/loss.rs:264-407)."""

    def set_category_weights(self, cw):
        self.cat_weights = torch.as_tensor(cw, dtype=torch.float32, device=self.net.device)
