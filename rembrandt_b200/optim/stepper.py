"""Applies the SGD rules to a network's flat vectors.

On CUDA this is the fused one-pass kernel (csrc/sgd_fused.cu), launched once for the regularised range and
once for the unregularised tail; on CPU it is ``reference_step``. ``phase`` lets the training loop split
"accumulate into the momentum buffer" from "apply to the parameters" when a parameter exchange sits between
the two (the reference's SyncParamsThenStep order, src/opt/sgd/new.rs:408-431).
"""
from __future__ import annotations

import torch

from ..ops import native_ops as K
from .sgd import Momentum, reference_step


class SgdStepper:
    def __init__(self, net, momentum: Momentum, mu: float, l2: float):
        self.net = net
        self.mode = int(momentum)
        self.mu = float(mu) if momentum != Momentum.ZERO else 0.0
        self.l2 = float(l2)

    def _ranges(self, lo, hi):
        """Split [lo, hi) at the boundary between regularised and unregularised parameters."""
        d = self.net.decay_len
        out = []
        if lo < min(hi, d):
            out.append((lo, min(hi, d), self.l2))
        if max(lo, d) < hi:
            out.append((max(lo, d), hi, 0.0))
        return out

    def step(self, lr: float, grad_scale: float = 1.0, phase: int = 7, lo: int = 0, hi: int = None, grid=None):
        """`grid` = (blocks, threads) launches the sweep with small blocks (used when it runs beside backward)."""
        net = self.net
        hi = net.flat_len if hi is None else hi
        for a, b, l2 in self._ranges(lo, hi):
            n = b - a
            if net.is_cuda and grid is not None:
                K.sgd_fused_grid(net.params[a:b], net.grads[a:b], net.mom[a:b], net.params16[a:b], n, lr, self.mu,
                                 l2, grad_scale, self.mode, phase, grid[0], grid[1])
            elif net.is_cuda:
                K.sgd_fused(net.params[a:b], net.grads[a:b], net.mom[a:b], net.params16[a:b], n, lr, self.mu, l2,
                            grad_scale, self.mode, phase)
            else:
                with torch.no_grad():
                    reference_step(net.params[a:b], net.grads[a:b], net.mom[a:b], lr, self.mu, l2, grad_scale,
                                   self.mode, phase)

    def nesterov_lookahead(self, sign: float = 1.0):
        """w += sign * mu * v: the reference keeps Nesterov parameters at the look-ahead point and applies this
        once before training (src/opt/sgd/new.rs:257-262)."""
        net = self.net
        if net.is_cuda:
            K.axpy_shadow(net.params, net.mom, net.params16, net.flat_len, sign * self.mu)
        else:
            with torch.no_grad():
                net.params.add_(net.mom, alpha=sign * self.mu)
