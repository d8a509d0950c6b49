"""Data-gradient of a strided convolution on the tensor-core kernel, by output phases.

For stride s the input position (y, x) = (s i + a, s j + b) only receives contributions from the filter taps
r = r0 + s u, c = c0 + s v with r0 = (a + pad) mod s, c0 = (b + pad) mod s, and

    dX[n, s i + a, s j + b, :] = sum_{u, v} dY[n, i + qa - u, j + qb - v, :] . W[:, r0 + s u, c0 + s v, :]
    qa = (a + pad - r0) / s,   qb = (b + pad - c0) / s

which is a stride-1 convolution of dY with the flipped sub-filter, top / left padding (U - 1) - qa, (V - 1) - qb.
Each of the s x s phases runs through the forward convolution path (`conv_fprop_tc`) into a compact tensor that is
then interleaved into dX; phases with no tap (e.g. three of the four phases of a 1 x 1 stride-2 projection) are zero.

`phase_plan` is pure arithmetic (tested on CPU against autograd through `dgrad_by_phases_reference`); the device
path below only swaps the plain-torch convolution for the kernel.
"""
from __future__ import annotations

from typing import List, NamedTuple

import torch
import torch.nn.functional as F


class Phase(NamedTuple):
    a: int          # row phase of dX
    b: int          # column phase
    r0: int         # first filter row / column that reaches this phase
    c0: int
    U: int          # taps of the sub-filter
    V: int
    pad_t: int      # top / left padding of the equivalent stride-1 convolution over dY
    pad_l: int
    Hp: int         # extent of this phase of dX
    Wp: int


def phase_plan(H: int, W: int, R: int, S: int, stride: int, pad: int) -> List[Phase]:
    out = []
    for a in range(stride):
        for b in range(stride):
            r0, c0 = (a + pad) % stride, (b + pad) % stride
            U, V = len(range(r0, R, stride)), len(range(c0, S, stride))
            qa, qb = (a + pad - r0) // stride, (b + pad - c0) // stride
            out.append(Phase(a, b, r0, c0, U, V, (U - 1) - qa, (V - 1) - qb, len(range(a, H, stride)),
                             len(range(b, W, stride))))
    return out


def dgrad_by_phases_reference(dy: torch.Tensor, w: torch.Tensor, H: int, W: int, stride: int, pad: int) -> torch.Tensor:
    """dy [N, K, P, Q], w [K, C, R, S] (torch layouts, fp32) -> dX [N, C, H, W] through the phase decomposition, with
    plain torch convolutions. The oracle of the decomposition itself (compared with autograd in the tests)."""
    N, K, P, Q = dy.shape
    _, C, R, S = w.shape
    dx = torch.zeros(N, C, H, W, dtype=dy.dtype)
    for ph in phase_plan(H, W, R, S, stride, pad):
        if ph.U == 0 or ph.V == 0 or ph.Hp == 0 or ph.Wp == 0:
            continue
        # sub-filter, flipped, as a correlation kernel that maps K channels of dY to C channels of dX
        sub = w[:, :, ph.r0::stride, ph.c0::stride].flip(2, 3).permute(1, 0, 2, 3)        # [C, K, U, V]
        # explicit padding: top / left as planned (cropping when negative), bottom / right to reach Hp x Wp
        need_h, need_w = ph.Hp + ph.U - 1, ph.Wp + ph.V - 1
        src = dy
        t, l = ph.pad_t, ph.pad_l
        if t < 0:
            src, t = src[:, :, -t:], 0
        if l < 0:
            src, l = src[:, :, :, -l:], 0
        bpad, rpad = max(0, need_h - t - src.shape[2]), max(0, need_w - l - src.shape[3])
        src = F.pad(src, (l, rpad, t, bpad))[:, :, :need_h, :need_w]
        dx[:, :, ph.a::stride, ph.b::stride] = F.conv2d(src, sub)
    return dx


def dgrad_strided_tc(dy, n, P, Q, kp, w16, ko, cp, in_c, R, S, stride, pad, H, W, dx, mask=None, cache=None):
    """Device path. dy: bf16 [n, P, Q, kp]; w16: bf16 filters [ko][R*S][cp]; dx: bf16 [n, H, W, cp] (overwritten);
    mask: optional bf16 [n, H, W, cp], dx is zeroed where mask <= 0. Returns False when a phase needs a negative
    padding (the caller then uses the direct kernel). `cache` (a dict owned by the calling operator) keeps the
    per-phase filter and output buffers between calls, so that a training step allocates nothing here."""
    from . import native_ops as K
    plan = phase_plan(H, W, R, S, stride, pad)
    if any(ph.U and ph.V and (ph.pad_t < 0 or ph.pad_l < 0) for ph in plan):
        return False
    w4 = w16[: ko * R * S * cp].view(ko, R, S, cp)
    for ph in plan:
        view = dx[:, ph.a::stride, ph.b::stride, :]
        if ph.U == 0 or ph.V == 0:
            view.zero_()
            continue
        # flipped sub-filter in the forward kernel's layout: [output channel = c][tap][input channel = k], k padded
        sub = w4[:, ph.r0::stride, ph.c0::stride, :].flip(1, 2).permute(3, 1, 2, 0).reshape(cp, ph.U * ph.V, ko)
        key = (ph.a, ph.b)
        bufs = cache.get(key) if cache is not None else None
        if bufs is None:
            bufs = (torch.zeros((cp, ph.U * ph.V, kp), dtype=torch.bfloat16, device=dy.device),
                    torch.empty((n, ph.Hp, ph.Wp, cp), dtype=torch.bfloat16, device=dy.device))
            if cache is not None:
                cache[key] = bufs
        wt, tmp = bufs
        wt[:, :, :ko].copy_(sub)
        K.conv_fprop_tc(dy, n, P, Q, kp, wt, cp, ph.U, ph.V, 1, ph.pad_t, ph.pad_l, ph.Hp, ph.Wp, tmp, cp,
                        n_valid=in_c, n_store=cp)
        view.copy_(tmp)
    if mask is not None:
        K.relu_mask(dx, mask, dx.numel())
    return True
