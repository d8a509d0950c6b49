"""Conversions between the reference's tensor conventions and the internal compute layouts.

Reference conventions (all "first dimension fastest"): activations ``(W,H,C,N)`` = torch NCHW; convolution
filters ``[k*k*Cin, Cout]`` = cuDNN ``(w,h,cin,cout)`` = torch OIHW; affine weights ``[in,out]`` = torch
``Linear.weight`` ``[out,in]`` whose ``in`` index runs over ``(w,h,c)`` = a CHW flatten.

Internal layouts: activations NHWC bf16 with padded channels; filters ``[Kout][R*S][Cp]``; affine weights
``[out][H*W*Cp]`` (an HWC flatten with padded channels); strided first layers run on a space-to-depth'd
input with filters ``[Kout][R2*S2][Cp2]`` where channel = ``(dy*f+dx)*Cin + c``.
"""
from __future__ import annotations

import torch


def to_nhwc_padded(x_nchw: torch.Tensor, cp: int, dtype=torch.bfloat16) -> torch.Tensor:
    n, c, h, w = x_nchw.shape
    out = torch.zeros((n, h, w, cp), dtype=dtype, device=x_nchw.device)
    out[..., :c] = x_nchw.permute(0, 2, 3, 1).to(dtype)
    return out


def from_nhwc_padded(x_nhwc: torch.Tensor, c: int) -> torch.Tensor:
    return x_nhwc[..., :c].permute(0, 3, 1, 2).float().contiguous()


def conv_weight_to_internal(w_oihw: torch.Tensor, cp: int) -> torch.Tensor:
    k, c, r, s = w_oihw.shape
    out = torch.zeros((k, r * s, cp), dtype=w_oihw.dtype, device=w_oihw.device)
    out[:, :, :c] = w_oihw.permute(0, 2, 3, 1).reshape(k, r * s, c)
    return out


def conv_weight_from_internal(w_int: torch.Tensor, c: int, r: int, s: int) -> torch.Tensor:
    k = w_int.shape[0]
    return w_int[:, :, :c].reshape(k, r, s, c).permute(0, 3, 1, 2).contiguous()


def s2d_geometry(ksize: int, stride: int, in_hw: int):
    """Geometry of the stride-1 equivalent of a `ksize` x `ksize`, stride-`stride`, pad-0 convolution."""
    f = stride
    r2 = (ksize + f - 1) // f
    out_hw = (in_hw - ksize) // stride + 1
    s2d_hw = out_hw + r2 - 1          # rows of the space-to-depth'd input that are read
    return f, r2, out_hw, s2d_hw


def s2d_weight_to_internal(w_oihw: torch.Tensor, f: int, cp2: int) -> torch.Tensor:
    k, c, r, s = w_oihw.shape
    r2 = (r + f - 1) // f
    s2 = (s + f - 1) // f
    wp = torch.zeros((k, c, r2 * f, s2 * f), dtype=w_oihw.dtype, device=w_oihw.device)
    wp[:, :, :r, :s] = w_oihw
    # (k, c, R2, dy, S2, dx) -> (k, R2, S2, dy, dx, c)
    wp = wp.reshape(k, c, r2, f, s2, f).permute(0, 2, 4, 3, 5, 1).reshape(k, r2 * s2, f * f * c)
    out = torch.zeros((k, r2 * s2, cp2), dtype=w_oihw.dtype, device=w_oihw.device)
    out[:, :, : f * f * c] = wp
    return out


def s2d_weight_from_internal(w_int: torch.Tensor, c: int, ksize: int, f: int) -> torch.Tensor:
    k = w_int.shape[0]
    r2 = (ksize + f - 1) // f
    wp = w_int[:, :, : f * f * c].reshape(k, r2, r2, f, f, c).permute(0, 5, 1, 3, 2, 4)
    wp = wp.reshape(k, c, r2 * f, r2 * f)
    return wp[:, :, :ksize, :ksize].contiguous()


def s2d_input(x_nchw: torch.Tensor, f: int, out_hw: int, cp2: int, dtype=torch.bfloat16) -> torch.Tensor:
    """Space-to-depth of an NCHW tensor into NHWC with `out_hw` rows/cols (zero beyond the image)."""
    n, c, h, w = x_nchw.shape
    xp = torch.zeros((n, c, out_hw * f, out_hw * f), dtype=x_nchw.dtype, device=x_nchw.device)
    hh, ww = min(h, out_hw * f), min(w, out_hw * f)
    xp[:, :, :hh, :ww] = x_nchw[:, :, :hh, :ww]
    xp = xp.reshape(n, c, out_hw, f, out_hw, f).permute(0, 2, 4, 3, 5, 1).reshape(n, out_hw, out_hw, f * f * c)
    out = torch.zeros((n, out_hw, out_hw, cp2), dtype=dtype, device=x_nchw.device)
    out[..., : f * f * c] = xp.to(dtype)
    return out


def affine_weight_to_internal(w_out_in: torch.Tensor, c: int, h: int, w: int, cp: int) -> torch.Tensor:
    """[out][c*h*w] (CHW flatten) -> [out][h*w*cp] (HWC flatten, padded channels)."""
    o = w_out_in.shape[0]
    t = w_out_in.reshape(o, c, h, w).permute(0, 2, 3, 1)
    out = torch.zeros((o, h, w, cp), dtype=w_out_in.dtype, device=w_out_in.device)
    out[..., :c] = t
    return out.reshape(o, h * w * cp)


def affine_weight_from_internal(w_int: torch.Tensor, c: int, h: int, w: int, cp: int) -> torch.Tensor:
    o = w_int.shape[0]
    return w_int.reshape(o, h, w, cp)[..., :c].permute(0, 3, 1, 2).reshape(o, c * h * w).contiguous()
