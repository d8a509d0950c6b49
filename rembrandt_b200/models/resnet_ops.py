"""Batch-normalised convolution and the two residual basic blocks.

Counterparts of the reference's ``BNormConv2dOperator`` (src/operator/conv.rs:52-912),
``StackResConv2dOperator`` (:914-2182, identity shortcut) and ``ProjStackResConv2dOperator`` (:2184-3852,
1x1 strided projection shortcut). Convolutions run on the tcgen05 implicit-GEMM kernel without bias;
normalisation, the residual add and the ReLU are one apply kernel after a statistics pass. Parameters per
normalised convolution: filter, scale, bias, running mean, running variance, in that order in the blob
(conv.rs:379-406); only filter, scale and bias receive gradients; none of the normalisation parameters is
L2-regularised (conv.rs:637-651).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import layout
from ..ops import native_ops as K
from ..ops.native_ops import pad_channels
from .operators import Op, ParamSeg, _draw, conv_out


class _BnConv:
    """conv (no bias) -> batch norm [-> + residual] [-> ReLU], with its buffers and parameter segments."""

    def __init__(self, op: Op, tag, in_hw, in_c, in_cp, out_c, k, stride, pad, init, mov_avg, eps, s2d=None):
        """`s2d` = (f, r2, s2d_hw): the input operator hands over a space-to-depth'd image (a strided first layer on
        <= 4 channels), on which this convolution is r2 x r2, stride 1, pad 0 over `in_cp` = pad(f * f * in_c)
        channels; (k, stride, pad) stay the reference geometry (parameters, host path)."""
        self.op, self.tag = op, tag
        self.h, self.w = in_hw
        self.in_c, self.cp = in_c, in_cp
        self.ko, self.kp = out_c, pad_channels(out_c)
        self.k, self.s, self.p = k, stride, pad
        self.P, self.Q = conv_out(self.h, k, stride, pad), conv_out(self.w, k, stride, pad)
        self.init, self.mov_avg, self.eps = init, mov_avg, eps
        self.s2d = s2d
        if s2d is not None:
            self.f, r2, s2d_hw = s2d
            # what the kernels see
            self.gh = self.gw = s2d_hw
            self.gk, self.gs, self.gp = r2, 1, 0
        else:
            self.gh, self.gw, self.gk, self.gs, self.gp = self.h, self.w, k, stride, pad
        n = op.name + "." + tag
        self.seg_w = ParamSeg(n + ".w", (out_c, self.gk * self.gk, in_cp))
        self.seg_g = ParamSeg(n + ".scale", (self.kp,), decay=False)
        self.seg_b = ParamSeg(n + ".bias", (self.kp,), decay=False)
        self.seg_rm = ParamSeg(n + ".run_mean", (self.kp,), decay=False, trainable=False)
        self.seg_rv = ParamSeg(n + ".run_var", (self.kp,), decay=False, trainable=False)
        self.segs = [self.seg_w, self.seg_g, self.seg_b, self.seg_rm, self.seg_rv]

    def alloc(self, need_dx_filters):
        net = self.op.net
        dev, n = net.device, net.batch
        self.conv_out = torch.zeros((n, self.P, self.Q, self.kp), dtype=torch.bfloat16, device=dev)
        self.mean = torch.zeros(self.kp, device=dev)
        self.istd = torch.ones(self.kp, device=dev)
        self.sums = torch.zeros(2 * self.kp, device=dev)
        self.dconv = torch.zeros_like(self.conv_out) if net.training_capable else None
        self.wt16 = None
        if net.training_capable and need_dx_filters and self.gs == 1:
            self.wt16 = torch.zeros((self.cp, self.gk * self.gk, self.kp), dtype=torch.bfloat16, device=dev)
        if dev.type == "cuda":
            # tile plans of the forward and data-grad shapes, measured once on scratch operands
            K.tune_conv(n, self.gh, self.gw, self.cp, self.ko, self.gk, self.gk, self.gs, self.gp, self.gp, self.P,
                        self.Q, self.kp, n_valid=self.ko, n_store=self.kp)
            if self.wt16 is not None:
                for has_mask in (False, True):
                    K.tune_conv(n, self.P, self.Q, self.kp, self.cp, self.gk, self.gk, 1, self.gk - 1 - self.gp,
                                self.gk - 1 - self.gp, self.gh, self.gw, self.cp, has_mask=has_mask,
                                n_valid=self.in_c, n_store=self.cp)

    def v(self, seg, which="params"):
        return self.op.net.seg_view(seg, which)

    def forward(self, x, out, residual, relu, train, t):
        net = self.op.net
        n = net.batch
        K.conv_fprop_tc(x, n, self.gh, self.gw, self.cp, self.v(self.seg_w, "params16"), self.ko, self.gk, self.gk,
                        self.gs, self.gp, self.gp, self.P, self.Q, self.conv_out, self.kp, n_valid=self.ko,
                        n_store=self.kp)
        rows = n * self.P * self.Q
        if train:
            # the factor comes from the device-side step counter, so that graph replays keep averaging correctly
            kind = 1 if self.mov_avg.kind == "cumulative" else 2
            K.bn_fwd_train(self.conv_out, rows, self.kp, self.ko, self.sums, self.eps, self.mov_avg.factor,
                           self.mean, self.istd, self.v(self.seg_rm), self.v(self.seg_rv), self.v(self.seg_g),
                           self.v(self.seg_b), residual, out, relu, avg_kind=kind, step_ptr=net.step_counter)
        else:
            K.bn_fwd_infer(self.conv_out, rows, self.kp, self.ko, self.eps, self.v(self.seg_rm), self.v(self.seg_rv),
                           self.istd, self.v(self.seg_g), self.v(self.seg_b), residual, out, relu)

    def backward(self, x, dout, y_relu, dx, mask):
        """dout: delta w.r.t. the normalised output (masked by `y_relu` here if given)."""
        net = self.op.net
        n = net.batch
        rows = n * self.P * self.Q
        K.bn_bwd(self.conv_out, dout, y_relu, rows, self.kp, self.ko, self.sums, self.mean, self.istd,
                 self.v(self.seg_g), self.v(self.seg_g, "grads"), self.v(self.seg_b, "grads"), self.dconv)
        gw = self.v(self.seg_w, "grads")
        K.conv_wgrad_tc(x, n, self.gh, self.gw, self.cp, self.dconv, self.kp, self.ko, self.gk, self.gk, self.gs,
                        self.gp, self.gp, self.P, self.Q, gw)
        if self.s2d is not None:
            # entries of the rearranged filter that no tap of the original filter maps to stay zero
            K.zero_s2d_structural(gw, self.ko, self.gk, self.cp, self.f, self.in_c, self.k)
        if dx is not None:
            if self.s2d is not None:
                raise RuntimeError("a space-to-depth'd convolution is a first layer: it has no input delta")
            w16 = self.v(self.seg_w, "params16")
            if self.s == 1:
                K.pack_dgrad_filters(w16, self.wt16, self.ko, self.kp, self.k * self.k, self.cp)
                K.conv_fprop_tc(self.dconv, n, self.P, self.Q, self.kp, self.wt16, self.cp, self.k, self.k, 1,
                                self.k - 1 - self.p, self.k - 1 - self.p, self.h, self.w, dx, self.cp, mask_src=mask,
                                n_valid=self.in_c, n_store=self.cp)
            else:
                from .operators import _strided_dgrad_on_tensor_cores
                from ..ops.conv_strided import dgrad_strided_tc
                done = False
                if _strided_dgrad_on_tensor_cores():
                    if not hasattr(self, "_sd_cache"):
                        self._sd_cache = {}
                    done = dgrad_strided_tc(self.dconv, n, self.P, self.Q, self.kp, w16, self.ko, self.cp, self.in_c,
                                            self.k, self.k, self.s, self.p, self.h, self.w, dx, mask,
                                            cache=self._sd_cache)
                if not done:
                    K.conv_direct_dgrad(self.dconv, w16, dx, mask, n, self.h, self.w, self.cp, self.ko, self.kp, self.k,
                                        self.k, self.s, self.p, self.p, self.P, self.Q)

    # ---- parameters
    def _w_int(self, w_oihw):
        if self.s2d is not None:
            return layout.s2d_weight_to_internal(w_oihw, self.f, self.cp)
        return layout.conv_weight_to_internal(w_oihw, self.cp)

    def _w_ref(self, w_int):
        if self.s2d is not None:
            return layout.s2d_weight_from_internal(w_int, self.in_c, self.k, self.f)
        return layout.conv_weight_from_internal(w_int, self.in_c, self.k, self.k)

    def init_params(self, rng):
        w = _draw(self.init, rng, (self.ko, self.in_c, self.k, self.k), self.k * self.k * self.in_c, self.ko)
        self.v(self.seg_w).copy_(self._w_int(w))
        self.v(self.seg_g).zero_()
        self.v(self.seg_g)[: self.ko] = 1.0
        self.v(self.seg_b).zero_()
        self.v(self.seg_rm).zero_()
        self.v(self.seg_rv).zero_()
        self.v(self.seg_rv)[: self.ko] = 1.0

    def encode(self):
        w = self._w_ref(self.v(self.seg_w).detach().float().cpu())
        out = [(w.reshape(-1), (self.k * self.k * self.in_c, self.ko))]
        for seg in (self.seg_g, self.seg_b, self.seg_rm, self.seg_rv):
            out.append((self.v(seg).detach().float().cpu()[: self.ko].clone(), (1, self.ko)))
        return out

    def decode(self, arrays):
        w = torch.as_tensor(arrays[0][0]).reshape(self.ko, self.in_c, self.k, self.k)
        self.v(self.seg_w).copy_(self._w_int(w))
        for seg, (a, _) in zip((self.seg_g, self.seg_b, self.seg_rm, self.seg_rv), arrays[1:5]):
            self.v(seg).zero_()
            self.v(seg)[: self.ko] = torch.as_tensor(a).reshape(-1)
        return 5

    def ref(self, x, residual, relu, train, t):
        w = self._w_ref(self.v(self.seg_w))
        y = F.conv2d(x, w, None, stride=self.s, padding=self.p)
        g, b = self.v(self.seg_g)[: self.ko], self.v(self.seg_b)[: self.ko]
        # `.data` views: running statistics are updated in place without touching autograd's version counter
        rm, rv = self.v(self.seg_rm).data[: self.ko], self.v(self.seg_rv).data[: self.ko]
        if train:
            rm2, rv2 = rm.clone(), rv.clone()
            y = F.batch_norm(y, rm2, rv2, g, b, training=True, momentum=self.mov_avg.at_iter(t), eps=self.eps)
            with torch.no_grad():
                rm.copy_(rm2)
                rv.copy_(rv2)
        else:
            y = F.batch_norm(y, rm, rv, g, b, training=False, eps=self.eps)
        if residual is not None:
            y = y + residual
        return torch.relu(y) if relu else y


class _BlockBase(Op):
    has_params = True
    units = ()

    def state_segs(self):
        return [s for s in self.segs if s.trainable]

    def init_params(self, rng):
        for u in self.units:
            u.init_params(rng)

    def encode_params(self):
        out = []
        for u in self.units:
            out.extend(u.encode())
        return out

    def decode_params(self, arrays):
        i = 0
        for u in self.units:
            i += u.decode(arrays[i:])
        return i


class BNormConv2dOp(_BlockBase):
    def setup(self, net, prev):
        super().setup(net, prev)
        cfg = self.cfg
        h, w, c = prev.out_hwc
        s2d = None
        from .operators import DataOp
        if isinstance(prev, DataOp) and cfg.conv_stride > 1 and c <= 4 and h == w and prev.mode == "nhwc":
            # a strided first layer on a few channels (the 7 x 7 / 2 stem): the input operator writes the image
            # space-to-depth'd, and the convolution becomes stride 1 over f * f * c channels instead of a strided
            # one whose 3 channels are padded to 32 per filter tap
            f, r2, _out_hw, s2d_hw = layout.s2d_geometry(cfg.conv_size, cfg.conv_stride, h + 2 * cfg.conv_pad)
            prev.request_s2d(f, s2d_hw, cfg.conv_pad)
            s2d = (f, r2, s2d_hw)
        self.u = _BnConv(self, "conv", (h, w), c, prev.out_cp, cfg.out_channels, cfg.conv_size, cfg.conv_stride,
                         cfg.conv_pad, cfg.init_weights, cfg.bnorm_mov_avg, cfg.bnorm_epsilon, s2d=s2d)
        self.units = (self.u,)
        self.segs = list(self.u.segs)
        self.out_hwc = (self.u.P, self.u.Q, cfg.out_channels)
        self.out_cp = self.u.kp
        self._setup_act(cfg.act, getattr(cfg, "act_param", None))

    def alloc(self):
        super().alloc()
        self.u.alloc(self.wants_prev_delta())

    def forward(self, train, t):
        self.u.forward(self.prev.out, self.out, None, self.has_relu, train, t)
        self._act_forward()

    def backward(self):
        self._act_backward()
        dx = self.prev.dout if self.wants_prev_delta() else None
        # the consumer already masked dout by this operator's ReLU
        self.u.backward(self.prev.out, self.dout, None, dx, self.mask_src())

    def ref_forward(self, x, train, t):
        y = self.u.ref(x, None, self.has_relu, train, t)
        return y if self.has_relu else self._ref_act(y)


class StackResConv2dOp(_BlockBase):
    """out = relu(x + bn2(conv3x3(relu(bn1(conv3x3(x))))))"""

    def setup(self, net, prev):
        super().setup(net, prev)
        cfg = self.cfg
        h, w, c = prev.out_hwc
        mk = lambda tag: _BnConv(self, tag, (h, w), c, prev.out_cp, c, 3, 1, 1, cfg.init_weights, cfg.bnorm_mov_avg,
                                 cfg.bnorm_epsilon)
        self.u1, self.u2 = mk("conv1"), mk("conv2")
        self.units = (self.u1, self.u2)
        self.segs = self.u1.segs + self.u2.segs
        self.out_hwc = (h, w, c)
        self.out_cp = prev.out_cp
        self.has_relu = True

    def alloc(self):
        super().alloc()
        self.u1.alloc(self.wants_prev_delta())
        self.u2.alloc(True)
        self.a1 = torch.zeros_like(self.out)
        self.da1 = torch.zeros_like(self.out) if self.net.training_capable else None

    def forward(self, train, t):
        x = self.prev.out
        self.u1.forward(x, self.a1, None, True, train, t)
        self.u2.forward(self.a1, self.out, x, True, train, t)

    def backward(self):
        x = self.prev.out
        self.u2.backward(self.a1, self.dout, None, self.da1, self.a1)
        if self.wants_prev_delta():
            self.u1.backward(x, self.da1, None, self.prev.dout, None)
            K.add_bf16(self.prev.dout, self.dout, self.dout.numel())
            if self.prev.has_relu:
                K.relu_mask(self.prev.dout, self.prev.out, self.dout.numel())
        else:
            self.u1.backward(x, self.da1, None, None, None)

    def ref_forward(self, x, train, t):
        a1 = self.u1.ref(x, None, True, train, t)
        return self.u2.ref(a1, x, True, train, t)


class ProjStackResConv2dOp(_BlockBase):
    """out = relu(bn2(conv3x3(relu(bn1(conv3x3_s(x))))) + bn3(conv1x1_s(x)))"""

    def setup(self, net, prev):
        super().setup(net, prev)
        cfg = self.cfg
        h, w, c = prev.out_hwc
        out_hw = cfg.out_hw if cfg.out_hw is not None else (h if cfg.out_channels == c else (h + 1) // 2)
        if out_hw == h:
            s = 1
        elif out_hw == (h + 1) // 2 or out_hw == h // 2:
            s = 2
        else:
            raise ValueError("projection block output must be the input size or half of it")
        ko = cfg.out_channels
        args = (cfg.init_weights, cfg.bnorm_mov_avg, cfg.bnorm_epsilon)
        self.u1 = _BnConv(self, "conv1", (h, w), c, prev.out_cp, ko, 3, s, 1, *args)
        self.u2 = _BnConv(self, "conv2", (self.u1.P, self.u1.Q), ko, self.u1.kp, ko, 3, 1, 1, *args)
        self.u3 = _BnConv(self, "proj", (h, w), c, prev.out_cp, ko, 1, s, 0, *args)
        self.units = (self.u1, self.u2, self.u3)
        self.segs = self.u1.segs + self.u2.segs + self.u3.segs
        self.out_hwc = (self.u1.P, self.u1.Q, ko)
        self.out_cp = self.u1.kp
        self.has_relu = True

    def alloc(self):
        super().alloc()
        need = self.wants_prev_delta()
        self.u1.alloc(need)
        self.u2.alloc(True)
        self.u3.alloc(need)
        self.a1 = torch.zeros_like(self.out)
        self.sc = torch.zeros_like(self.out)
        if self.net.training_capable:
            self.da1 = torch.zeros_like(self.out)
            self.dx2 = torch.zeros_like(self.prev.out) if need else None

    def forward(self, train, t):
        x = self.prev.out
        self.u3.forward(x, self.sc, None, False, train, t)
        self.u1.forward(x, self.a1, None, True, train, t)
        self.u2.forward(self.a1, self.out, self.sc, True, train, t)

    def backward(self):
        x = self.prev.out
        need = self.wants_prev_delta()
        self.u2.backward(self.a1, self.dout, None, self.da1, self.a1)
        self.u1.backward(x, self.da1, None, self.prev.dout if need else None, None)
        self.u3.backward(x, self.dout, None, self.dx2 if need else None, None)
        if need:
            K.add_bf16(self.prev.dout, self.dx2, self.dx2.numel())
            if self.prev.has_relu:
                K.relu_mask(self.prev.dout, self.prev.out, self.dx2.numel())

    def ref_forward(self, x, train, t):
        sc = self.u3.ref(x, None, False, train, t)
        a1 = self.u1.ref(x, None, True, train, t)
        return self.u2.ref(a1, sc, True, train, t)
