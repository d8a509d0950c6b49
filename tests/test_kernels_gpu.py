"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op (GPU only).

Inputs are rounded to bf16 first so that the reference sees exactly the values the kernel reads; outputs
are NaN-poisoned before the launch so that unwritten elements are caught.
"""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from rembrandt_b200.ops import layout, native_ops as K

DEV = "cuda"


def bf(x):
    return x.to(torch.bfloat16).float()


def close(a, b, rtol=2e-2, atol=None):
    a, b = a.float(), b.float()
    if atol is None:
        atol = 2e-2 * float(b.abs().max().clamp_min(1e-6))
    bad = (a - b).abs() > atol + rtol * b.abs()
    assert not torch.isnan(a).any(), "NaN in kernel output (unwritten element?)"
    assert not bad.any(), f"mismatch: max abs err {(a - b).abs().max().item():.4g}, ref max {b.abs().max().item():.4g}"


def status_ok():
    torch.cuda.synchronize()
    assert K.read_status() == 0


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K_", [(128, 256, 512), (200, 96, 96), (77, 32, 64), (384, 512, 1024), (128, 1024, 160)])
def test_gemm_kmajor_bf16_epilogue(M, N, K_, tile_mode):
    torch.manual_seed(0)
    a = bf(torch.randn(M, K_, device=DEV))
    b = bf(torch.randn(N, K_, device=DEV))
    bias = torch.randn(N, device=DEV)
    d = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(a.bfloat16(), 0, K_, b.bfloat16(), 0, K_, M, N, K_, d, N, epi=K.EPI_BF16, bias=bias, relu=True)
    status_ok()
    close(d, torch.relu(a @ b.t() + bias))


def test_gemm_mask_and_padding_columns():
    torch.manual_seed(1)
    M, N, Np, K_ = 130, 50, 64, 128
    a = bf(torch.randn(M, K_, device=DEV))
    b = bf(torch.randn(N, K_, device=DEV))
    mask = bf(torch.randn(M, Np, device=DEV))
    d = torch.full((M, Np), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(a.bfloat16(), 0, K_, b.bfloat16(), 0, K_, M, N, K_, d, Np, epi=K.EPI_BF16, mask_src=mask.bfloat16(),
              n_valid=N, n_store=Np)
    status_ok()
    ref = torch.zeros(M, Np, device=DEV)
    ref[:, :N] = a @ b.t()
    ref = ref * (mask > 0)
    close(d, ref)


@pytest.mark.parametrize("M,N,K_", [(128, 256, 256), (100, 192, 320), (128, 4096, 512)])
def test_gemm_b_mn_major(M, N, K_):
    """dX = dY * W with W stored [K][N] (N contiguous): the affine data-gradient form."""
    torch.manual_seed(2)
    a = bf(torch.randn(M, K_, device=DEV))
    w = bf(torch.randn(K_, N, device=DEV))
    d = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(a.bfloat16(), 0, K_, w.bfloat16(), 1, N, M, N, K_, d, N, epi=K.EPI_BF16)
    status_ok()
    close(d, a @ w)


@pytest.mark.parametrize("M,N,K_,split", [(256, 384, 128, 1), (96, 200, 1000, 0), (4096, 1024, 128, 1)])
def test_gemm_both_mn_major_atomic(M, N, K_, split, tile_mode):
    """dW[M][N] += dY^T X with dY [K][M], X [K][N]: the affine weight-gradient form (fp32 accumulate)."""
    torch.manual_seed(3)
    Np = (N + 31) // 32 * 32
    Mp = (M + 7) // 8 * 8
    dy = torch.zeros(K_, Mp, device=DEV)
    dy[:, :M] = bf(torch.randn(K_, M, device=DEV))
    x = torch.zeros(K_, Np, device=DEV)
    x[:, :N] = bf(torch.randn(K_, N, device=DEV))
    d = torch.ones(M, Np, device=DEV)
    K.gemm_tc(dy.bfloat16(), 1, Mp, x.bfloat16(), 1, Np, M, N, K_, d, Np, epi=K.EPI_F32_ATOMIC, split_k=split,
              n_store=Np)
    status_ok()
    close(d, 1.0 + dy[:, :M].t() @ x, rtol=1e-2)


def test_gemm_f32_store():
    torch.manual_seed(4)
    M, N, K_ = 128, 64, 192
    a = bf(torch.randn(M, K_, device=DEV))
    b = bf(torch.randn(N, K_, device=DEV))
    d = torch.full((M, N), float("nan"), device=DEV)
    K.gemm_tc(a.bfloat16(), 0, K_, b.bfloat16(), 0, K_, M, N, K_, d, N, epi=K.EPI_F32_STORE)
    status_ok()
    close(d, a @ b.t(), rtol=1e-2)


# ----------------------------------------------------------------------------- convolution
CONV_CASES = [
    # N, C, H, W, Kout, R, stride, pad
    (2, 64, 13, 13, 128, 3, 1, 1),
    (3, 96, 27, 27, 256, 5, 1, 2),
    (2, 20, 12, 12, 50, 5, 1, 0),
    (4, 256, 13, 13, 384, 3, 1, 1),
    (2, 64, 16, 16, 64, 1, 1, 0),
    (2, 128, 15, 15, 96, 3, 2, 1),
    (1, 32, 6, 6, 40, 3, 1, 1),
    (130, 32, 8, 8, 32, 5, 1, 2),
    (2, 64, 14, 14, 96, 3, 1, 1),     # data-grad reduces over 96 channels: a half-empty 64-channel chunk
    (2, 160, 9, 9, 64, 3, 1, 1),
    (1, 32, 40, 40, 64, 3, 1, 1),     # halo mode: row pitch 64 (two output rows per sub-tile)
    (1, 32, 70, 66, 32, 3, 1, 1),     # halo mode: row pitch 128, non-square
    (128, 64, 13, 13, 64, 3, 1, 1),   # 169 row tiles on 148 SMs: the 21 of the last wave are cut along the reduction
    (128, 32, 13, 13, 320, 3, 1, 1),  # the same with one 320-column tile (two MMAs side by side)
    (40, 64, 27, 27, 64, 5, 1, 2),    # box loads: 4 output rows per sub-tile, 280 tiles, ragged last band of each tile
    (3, 64, 20, 23, 96, 3, 1, 0),     # box loads without padding: output narrower than the input
]


def _conv_setup(N, C, H, W, Ko, R, stride, pad, seed=0):
    torch.manual_seed(seed)
    Cp, Kp = K.pad_channels(C), K.pad_channels(Ko)
    x = bf(torch.randn(N, C, H, W, device=DEV))
    w = bf(torch.randn(Ko, C, R, R, device=DEV) / math.sqrt(C * R * R))
    b = torch.randn(Ko, device=DEV)
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - R) // stride + 1
    return Cp, Kp, x, w, b, P, Q


@pytest.fixture(params=["auto", "halo", "mt1", "mt2", "mt1_resident", "mt2_resident", "mt1_taps2", "mt2_taps3", "tail",
                        "wide", "wide_tail", "box", "box_mt2", "box_tail", "box_wide", "pair", "pair_mt1", "tuned"])
def tile_mode(request):
    """Force the kernel's tile-shape planner through each of its modes (two sub-tiles per item, resident B,
    column-shifted halo tiles for stride-1 convolutions, the last wave cut along the reduction, one tile as wide as
    the layer, tap-shifted box loads of whole output rows, CTA pairs issuing 256-row MMAs, plans chosen by
    measurement)."""
    mode = request.param
    opts = {}
    if mode == "halo":
        opts["force_halo"] = 1
    elif mode != "auto":
        opts["force_halo"] = 0
    if mode.startswith("mt"):
        opts["force_mt"] = 2 if "mt2" in mode else 1
        opts["force_resident"] = 1 if "resident" in mode else 0
        if "taps" in mode:
            opts["force_taps"] = int(mode[-1])
    if "box" in mode:
        opts["force_box"] = 1
        if "mt2" in mode:
            opts["force_mt"] = 2
    if "pair" in mode:
        opts["force_pair"] = 1
        if "mt1" in mode:
            opts["force_mt"] = 1
    if "tail" in mode:
        opts["force_tail"] = 1
    if "wide" in mode:
        opts["force_wide"] = 1
    if mode == "tuned":
        K.gemm_clear_plans()
        with K.gemm_tuning():
            yield mode
        K.gemm_clear_plans()
        return
    with K.gemm_options(**opts):
        yield mode


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_fprop_tc(case, tile_mode):
    N, C, H, W, Ko, R, stride, pad = case
    Cp, Kp, x, w, b, P, Q = _conv_setup(*case)
    xi = layout.to_nhwc_padded(x, Cp)
    wi = layout.conv_weight_to_internal(w, Cp).bfloat16()
    y = torch.full((N, P, Q, Kp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.conv_fprop_tc(xi, N, H, W, Cp, wi, Ko, R, R, stride, pad, pad, P, Q, y, Kp, bias=b, relu=True, n_valid=Ko,
                    n_store=Kp)
    status_ok()
    ref = torch.relu(F.conv2d(x, w, b, stride=stride, padding=pad))
    close(layout.from_nhwc_padded(y, Ko), ref)
    assert (y[..., Ko:].float() == 0).all(), "padded output channels must be zero"
    # the direct kernel must agree as well
    y2 = torch.full_like(y, float("nan"))
    K.conv_direct_fwd(xi, wi, b, y2, N, H, W, Cp, Ko, Kp, R, R, stride, pad, pad, P, Q, True)
    close(layout.from_nhwc_padded(y2, Ko), ref)


@pytest.mark.parametrize("case", [c for c in CONV_CASES if c[6] == 1])
def test_conv_dgrad_tc(case, tile_mode):
    N, C, H, W, Ko, R, stride, pad = case
    Cp, Kp, x, w, b, P, Q = _conv_setup(*case, seed=5)
    dy = bf(torch.randn(N, Ko, P, Q, device=DEV))
    dyi = layout.to_nhwc_padded(dy, Kp)
    wi = layout.conv_weight_to_internal(w, Cp).bfloat16()
    wt = torch.full((Cp, R * R, Kp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.pack_dgrad_filters(wi, wt, Ko, Kp, R * R, Cp)
    mask = bf(torch.randn(N, C, H, W, device=DEV))
    maski = layout.to_nhwc_padded(mask, Cp)
    dx = torch.full((N, H, W, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    # data-gradient = forward convolution of dY with flipped filters, padding R-1-pad
    K.conv_fprop_tc(dyi, N, P, Q, Kp, wt, Cp, R, R, 1, R - 1 - pad, R - 1 - pad, H, W, dx, Cp, mask_src=maski,
                    n_valid=C, n_store=Cp)
    status_ok()
    ref = F.conv_transpose2d(dy, w, stride=1, padding=pad) * (mask > 0)
    close(layout.from_nhwc_padded(dx, C), ref)
    dx2 = torch.full_like(dx, float("nan"))
    K.conv_direct_dgrad(dyi, wi, dx2, maski, N, H, W, Cp, Ko, Kp, R, R, 1, pad, pad, P, Q)
    close(layout.from_nhwc_padded(dx2, C), ref)


def test_conv_direct_dgrad_strided():
    case = (2, 32, 15, 15, 48, 3, 2, 1)
    N, C, H, W, Ko, R, stride, pad = case
    Cp, Kp, x, w, b, P, Q = _conv_setup(*case, seed=6)
    dy = bf(torch.randn(N, Ko, P, Q, device=DEV))
    dx = torch.full((N, H, W, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.conv_direct_dgrad(layout.to_nhwc_padded(dy, Kp), layout.conv_weight_to_internal(w, Cp).bfloat16(), dx, None, N,
                        H, W, Cp, Ko, Kp, R, R, stride, pad, pad, P, Q)
    ref = torch.autograd.grad(F.conv2d(x.requires_grad_(), w, stride=stride, padding=pad), x, dy)[0]
    close(layout.from_nhwc_padded(dx, C), ref)


@pytest.mark.parametrize("case", [(2, 32, 15, 15, 48, 3, 2, 1), (2, 64, 16, 16, 64, 1, 2, 0), (3, 32, 12, 14, 32, 3, 2, 1),
                                  (2, 64, 28, 28, 128, 3, 2, 1)])
def test_conv_dgrad_strided_by_phases_on_tensor_cores(case):
    """Strided data-grad as s x s stride-1 sub-convolutions on the tensor-core kernel, with the ReLU mask."""
    from rembrandt_b200.ops.conv_strided import dgrad_strided_tc
    N, C, H, W, Ko, R, stride, pad = case
    Cp, Kp, x, w, b, P, Q = _conv_setup(*case, seed=8)
    dy = bf(torch.randn(N, Ko, P, Q, device=DEV))
    mask = bf(torch.randn(N, C, H, W, device=DEV))
    dx = torch.full((N, H, W, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    wi = layout.conv_weight_to_internal(w, Cp).bfloat16()
    ok = dgrad_strided_tc(layout.to_nhwc_padded(dy, Kp), N, P, Q, Kp, wi, Ko, Cp, C, R, R, stride, pad, H, W, dx,
                          layout.to_nhwc_padded(mask, Cp))
    assert ok
    status_ok()
    ref = torch.autograd.grad(F.conv2d(x.requires_grad_(), w, stride=stride, padding=pad), x, dy)[0] * (mask > 0)
    close(layout.from_nhwc_padded(dx, C), ref)
    assert (dx[..., C:].float() == 0).all()


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_wgrad_tc(case, tile_mode):
    N, C, H, W, Ko, R, stride, pad = case
    Cp, Kp, x, w, b, P, Q = _conv_setup(*case, seed=7)
    dy = bf(torch.randn(N, Ko, P, Q, device=DEV))
    xi = layout.to_nhwc_padded(x, Cp)
    dyi = layout.to_nhwc_padded(dy, Kp)
    dw = torch.ones((Ko, R * R, Cp), device=DEV)
    K.conv_wgrad_tc(xi, N, H, W, Cp, dyi, Kp, Ko, R, R, stride, pad, pad, P, Q, dw)
    status_ok()
    wr = w.clone().requires_grad_()
    ref = torch.autograd.grad(F.conv2d(x, wr, stride=stride, padding=pad), wr, dy)[0]
    got = layout.conv_weight_from_internal(dw - 1.0, C, R, R)
    close(got, ref, rtol=2e-2)
    assert ((dw - 1.0)[:, :, C:] == 0).all(), "gradient of padded channels must stay zero"
    dw2 = torch.zeros_like(dw)
    K.conv_direct_wgrad(xi, dyi, dw2, N, H, W, Cp, Ko, Kp, R, R, stride, pad, pad, P, Q)
    close(layout.conv_weight_from_internal(dw2, C, R, R), ref, rtol=2e-2)


def test_deterministic_option_makes_weight_gradients_bit_identical():
    """With the `deterministic` option no two CTAs add into the same element, so two launches on the same operands
    agree bit for bit (the default splits long reductions over CTAs, whose additions arrive in any order)."""
    case = (16, 64, 27, 27, 128, 5, 1, 2)
    N, C, H, W, Ko, R, stride, pad = case
    Cp, Kp, x, w, b, P, Q = _conv_setup(*case, seed=9)
    dy = bf(torch.randn(N, Ko, P, Q, device=DEV))
    xi, dyi = layout.to_nhwc_padded(x, Cp), layout.to_nhwc_padded(dy, Kp)
    outs = []
    with K.gemm_options(deterministic=1):
        for _ in range(3):
            dw = torch.zeros((Ko, R * R, Cp), device=DEV)
            K.conv_wgrad_tc(xi, N, H, W, Cp, dyi, Kp, Ko, R, R, stride, pad, pad, P, Q, dw)
            outs.append(dw)
    status_ok()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    wr = w.clone().requires_grad_()
    ref = torch.autograd.grad(F.conv2d(x, wr, stride=stride, padding=pad), wr, dy)[0]
    close(layout.conv_weight_from_internal(outs[0], C, R, R), ref, rtol=2e-2)


@pytest.mark.parametrize("ks,st,HW", [(11, 4, 67), (7, 2, 31), (5, 2, 20)])
def test_conv_s2d_first_layer_matches_strided_conv(ks, st, HW):
    """A strided k x k convolution on 3 channels == a stride-1 convolution on the space-to-depth input."""
    torch.manual_seed(8)
    N, C, Ko = 2, 3, 96
    f, r2, out_hw, s2d_hw = layout.s2d_geometry(ks, st, HW)
    cp2 = K.pad_channels(f * f * C)
    x = bf(torch.randn(N, C, HW, HW, device=DEV))
    w = bf(torch.randn(Ko, C, ks, ks, device=DEV) / math.sqrt(C * ks * ks))
    b = torch.randn(Ko, device=DEV)
    xi = layout.s2d_input(x, f, s2d_hw, cp2)
    wi = layout.s2d_weight_to_internal(w, f, cp2).bfloat16()
    Kp = K.pad_channels(Ko)
    y = torch.full((N, out_hw, out_hw, Kp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.conv_fprop_tc(xi, N, s2d_hw, s2d_hw, cp2, wi, Ko, r2, r2, 1, 0, 0, out_hw, out_hw, y, Kp, bias=b, n_valid=Ko,
                    n_store=Kp)
    status_ok()
    close(layout.from_nhwc_padded(y, Ko), F.conv2d(x, w, b, stride=st))
    # weight-gradient in the s2d layout, structural zeros removed, maps back to the 11x11 gradient
    dy = bf(torch.randn(N, Ko, out_hw, out_hw, device=DEV))
    dw = torch.zeros((Ko, r2 * r2, cp2), device=DEV)
    K.conv_wgrad_tc(xi, N, s2d_hw, s2d_hw, cp2, layout.to_nhwc_padded(dy, Kp), Kp, Ko, r2, r2, 1, 0, 0, out_hw,
                    out_hw, dw)
    K.zero_s2d_structural(dw, Ko, r2, cp2, f, C, ks)
    status_ok()
    wr = w.clone().requires_grad_()
    ref = torch.autograd.grad(F.conv2d(x, wr, stride=st), wr, dy)[0]
    close(layout.s2d_weight_from_internal(dw, C, ks, f), ref)
    back = layout.s2d_weight_to_internal(layout.s2d_weight_from_internal(dw, C, ks, f), f, cp2)
    assert torch.equal(back, dw), "structural entries of the s2d gradient must be zero"


# ----------------------------------------------------------------------------- memory-bound ops
@pytest.mark.parametrize("kind,k,stride,pad,ceil,relu", [("max", 3, 2, 0, False, False), ("max", 3, 2, 0, True, True),
                                                         ("max", 2, 2, 0, False, False), ("avg", 3, 2, 0, False, False),
                                                         ("avg", 3, 2, 1, False, True), ("avg", 6, 1, 0, False, False)])
def test_pool(kind, k, stride, pad, ceil, relu):
    torch.manual_seed(9)
    N, C, H = 3, 40, 13
    Cp = K.pad_channels(C)
    x = bf(torch.randn(N, C, H, H, device=DEV)).requires_grad_()
    if kind == "max":
        ref = F.max_pool2d(x, k, stride, pad, ceil_mode=ceil)
    else:
        ref = F.avg_pool2d(x, k, stride, pad, ceil_mode=ceil, count_include_pad=True)
    if relu:
        ref = torch.relu(ref)
    P = ref.shape[2]
    xi = layout.to_nhwc_padded(x.detach(), Cp)
    y = torch.full((N, P, P, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    idx = torch.zeros((N, P, P, Cp), device=DEV, dtype=torch.uint8)
    K.pool_fwd(xi, y, idx, N, H, H, Cp, P, P, k, stride, pad, kind == "max", relu)
    close(layout.from_nhwc_padded(y, C), ref.detach())
    dy = bf(torch.randn_like(ref))
    gref = torch.autograd.grad(ref, x, dy)[0]
    dx = torch.full((N, H, H, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.pool_bwd(layout.to_nhwc_padded(dy, Cp), idx, y if relu else None, dx, None, N, H, H, Cp, P, P, k, stride, pad,
               kind == "max")
    close(layout.from_nhwc_padded(dx, C), gref)


@pytest.mark.parametrize("k,stride,pad,ceil,relu,C,H", [(3, 2, 0, False, False, 96, 29), (3, 2, 0, True, True, 96, 29),
                                                        (3, 2, 1, False, False, 40, 31), (2, 2, 0, False, True, 256, 14),
                                                        (3, 1, 1, False, False, 64, 17)])
def test_maxpool_row_mapped_kernels(k, stride, pad, ceil, relu, C, H):
    """Shapes wide enough for the row-mapped max-pooling kernels (forward and backward), with a ReLU mask."""
    torch.manual_seed(19)
    N = 3
    Cp = K.pad_channels(C)
    x = bf(torch.randn(N, C, H, H, device=DEV)).requires_grad_()
    ref = F.max_pool2d(x, k, stride, pad, ceil_mode=ceil)
    if relu:
        ref = torch.relu(ref)
    P = ref.shape[2]
    assert P * (Cp // 8) >= 64 and H * (Cp // 8) >= 64
    xi = layout.to_nhwc_padded(x.detach(), Cp)
    y = torch.full((N, P, P, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    idx = torch.zeros((N, P, P, Cp), device=DEV, dtype=torch.uint8)
    K.pool_fwd(xi, y, idx, N, H, H, Cp, P, P, k, stride, pad, True, relu)
    close(layout.from_nhwc_padded(y, C), ref.detach())
    dy = bf(torch.randn_like(ref))
    gref = torch.autograd.grad(ref, x, dy)[0]
    # the producer of the delta masks it with the ReLU'd activation below the pooling layer
    below = bf(torch.randn(N, C, H, H, device=DEV))
    gref = gref * (below > 0)
    dx = torch.full((N, H, H, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.pool_bwd(layout.to_nhwc_padded(dy, Cp), idx, y if relu else None, dx, layout.to_nhwc_padded(below, Cp), N, H, H,
               Cp, P, P, k, stride, pad, True)
    close(layout.from_nhwc_padded(dx, C), gref)
    assert (dx[..., C:].float() == 0).all()


def test_lrn():
    torch.manual_seed(10)
    N, C, H = 2, 96, 7
    Cp = K.pad_channels(C)
    size, alpha, beta, k = 5, 1e-2, 0.75, 2.0
    x = (bf(torch.randn(N, C, H, H, device=DEV)) * 3).requires_grad_()
    # torch divides alpha by the window size; the kernel takes the effective coefficient
    ref = F.local_response_norm(x, size, alpha=alpha * size, beta=beta, k=k)
    xi = layout.to_nhwc_padded(x.detach(), Cp)
    y = torch.full((N, H, H, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.lrn_fwd(xi, y, N * H * H, Cp, size, alpha, beta, k)
    close(layout.from_nhwc_padded(y, C), ref.detach())
    dy = bf(torch.randn_like(ref))
    gref = torch.autograd.grad(ref, x, dy)[0]
    dx = torch.full((N, H, H, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.lrn_bwd(xi, layout.to_nhwc_padded(dy, Cp), dx, None, N * H * H, Cp, size, alpha, beta, k)
    close(layout.from_nhwc_padded(dx, C), gref)


def test_dropout_mask_is_reproducible_and_scaled():
    n, p = 1 << 16, 0.5
    x = torch.ones(n, device=DEV, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    K.dropout(x, y, n, p, seed=123, stream_id=7)
    keep = (y.float() > 0).float().mean().item()
    assert abs(keep - 0.5) < 0.02
    assert set(y.float().unique().tolist()) <= {0.0, 2.0}
    g = torch.full_like(x, 3.0)
    dx = torch.empty_like(x)
    K.dropout(g, dx, n, p, seed=123, stream_id=7)
    assert torch.equal((dx.float() > 0), (y.float() > 0))
    y2 = torch.empty_like(x)
    K.dropout(x, y2, n, p, seed=124, stream_id=7)
    assert not torch.equal(y, y2)


def test_softmax_ce():
    torch.manual_seed(11)
    B, Kc = 37, 1000
    ld = K.pad_channels(Kc)
    logits = bf(torch.randn(B, Kc, device=DEV) * 3)
    li = torch.zeros(B, ld, device=DEV, dtype=torch.bfloat16)
    li[:, :Kc] = logits.bfloat16()
    labels = torch.randint(0, Kc, (B,), device=DEV, dtype=torch.int32)
    w = 1.0 / B
    delta = torch.full((B, ld), float("nan"), device=DEV, dtype=torch.bfloat16)
    loss = torch.zeros(1, device=DEV)
    correct = torch.zeros(1, device=DEV, dtype=torch.int32)
    K.softmax_ce(li, B, Kc, ld, labels, None, w, delta, loss_sum=loss, correct=correct)
    lr = logits.clone().requires_grad_()
    ref_loss = F.cross_entropy(lr, labels.long(), reduction="sum") * w
    ref_delta = torch.autograd.grad(ref_loss, lr)[0]
    assert abs(loss.item() - ref_loss.item()) < 1e-3 * max(1.0, abs(ref_loss.item()))
    close(delta[:, :Kc], ref_delta, atol=1e-4)
    assert (delta[:, Kc:].float() == 0).all()
    assert correct.item() == int((logits.argmax(1) == labels.long()).sum())


def test_softmax_ce_masks_and_lookahead_heads():
    torch.manual_seed(13)
    B, Kc, L = 9, 361, 3
    ld = K.pad_channels(Kc * L)
    logits = bf(torch.randn(B, L, Kc, device=DEV) * 2)
    li = torch.zeros(B, ld, device=DEV, dtype=torch.bfloat16)
    li[:, :Kc * L] = logits.reshape(B, -1).bfloat16()
    mask = (torch.rand(B, L, Kc, device=DEV) > 0.3)
    labels = torch.randint(0, Kc, (B, L), device=DEV)
    mask.scatter_(2, labels.unsqueeze(-1), True)          # a target is always admissible
    mask[:, :, 0] = True                                  # so is the stand-in index of a skipped head
    labels[2, 1] = -1                                      # a head without a target
    labels[5, 2] = -1
    w = 0.25
    delta = torch.full((B, ld), float("nan"), device=DEV, dtype=torch.bfloat16)
    loss = torch.zeros(1, device=DEV)
    correct = torch.zeros(1, device=DEV, dtype=torch.int32)
    am = torch.zeros(B, device=DEV, dtype=torch.int32)
    K.softmax_ce(li, B, Kc, ld, labels.int().contiguous(), None, w, delta, loss_sum=loss, correct=correct,
                 argmax_out=am, mask=mask.to(torch.uint8).contiguous(), heads=L)
    lr = logits.clone().requires_grad_()
    masked = lr.masked_fill(~mask, float("-inf")).reshape(B * L, Kc)
    live = labels.reshape(-1) >= 0
    nll = F.cross_entropy(masked, labels.reshape(-1).clamp_min(0), reduction="none")
    ref_loss = torch.where(live, nll, torch.zeros_like(nll)).sum() * w
    ref_delta = torch.autograd.grad(ref_loss, lr)[0].reshape(B, L * Kc)
    assert abs(loss.item() - ref_loss.item()) < 2e-3 * max(1.0, abs(ref_loss.item()))
    close(delta[:, :Kc * L], ref_delta, atol=2e-3)
    assert (delta[:, Kc * L:].float() == 0).all()
    assert (delta[:, :Kc * L].float().reshape(B, L, Kc)[~mask] == 0).all()
    first = masked.reshape(B, L, Kc)[:, 0].argmax(1)
    assert torch.equal(am.long(), first)
    assert correct.item() == int((first == labels[:, 0]).sum())


@pytest.mark.parametrize("mode", [0, 1])
def test_pointwise_loss(mode):
    torch.manual_seed(14)
    B, Kc = 21, 5
    ld = K.pad_channels(Kc)
    x = bf(torch.randn(B, Kc, device=DEV) * 4)
    xi = torch.zeros(B, ld, device=DEV, dtype=torch.bfloat16)
    xi[:, :Kc] = x.bfloat16()
    t = (torch.rand(B, Kc, device=DEV) > 0.5).float() if mode == 0 else torch.randn(B, Kc, device=DEV)
    w = 0.125
    delta = torch.full((B, ld), float("nan"), device=DEV, dtype=torch.bfloat16)
    loss = torch.zeros(1, device=DEV)
    correct = torch.zeros(1, device=DEV, dtype=torch.int32)
    K.pointwise_loss(xi, B, Kc, ld, t, None, w, delta, loss_sum=loss, correct=correct, mode=mode)
    xr = x.clone().requires_grad_()
    if mode == 0:
        ref = F.binary_cross_entropy_with_logits(xr, t, reduction="sum") * w
    else:
        ref = 0.5 * ((xr - t) ** 2).sum() * w
    ref_delta = torch.autograd.grad(ref, xr)[0]
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    close(delta[:, :Kc], ref_delta, atol=2e-3, rtol=1e-2)
    assert (delta[:, Kc:].float() == 0).all()
    if mode == 0:
        assert correct.item() == int(((x[:, 0] > 0) == (t[:, 0] > 0.5)).sum())


def test_sample_categories_follows_the_tempered_masked_softmax():
    torch.manual_seed(17)
    B, Kc = 4096, 37
    ld = K.pad_channels(Kc)
    row = torch.randn(Kc, device=DEV) * 1.5
    x = torch.zeros(B, ld, device=DEV, dtype=torch.bfloat16)
    x[:, :Kc] = row.bfloat16()
    mask = torch.ones(B, Kc, device=DEV, dtype=torch.uint8)
    mask[:, ::5] = 0
    out = torch.full((B,), -7, device=DEV, dtype=torch.int32)
    counts = torch.zeros(Kc, device=DEV)
    for step in range(8):
        K.sample_categories(x, B, Kc, ld, mask, 0.7, 1234, step, out)
        assert int(out.min()) >= 0 and int(out.max()) < Kc
        counts += torch.bincount(out.long(), minlength=Kc).float()
    assert float(counts[::5].sum()) == 0, "a masked category was drawn"
    p = torch.softmax((row.bfloat16().float() / 0.7).masked_fill(mask[0] == 0, float("-inf")), 0)
    freq = counts / counts.sum()
    assert float((freq - p).abs().max()) < 0.01, (freq, p)
    # the same (seed, step) gives the same draws; another step gives others
    a = torch.empty_like(out)
    K.sample_categories(x, B, Kc, ld, mask, 0.7, 1234, 7, a)
    assert torch.equal(a, out)
    K.sample_categories(x, B, Kc, ld, mask, 0.7, 1234, 8, a)
    assert not torch.equal(a, out)


@pytest.mark.parametrize("objective", [1, 2, 3])
@pytest.mark.parametrize("marginal", [False, True])
def test_categorical_objective_heads(objective, marginal):
    """Softmax indicator (also with a weight per category), antilogistic + KL, antilogistic indicator against
    autograd of the formulas."""
    if marginal and objective != 1:
        pytest.skip("category weights exist for the softmax indicator only")
    torch.manual_seed(15)
    B, Kc = 19, 11
    ld = K.pad_channels(Kc)
    x = bf(torch.randn(B, Kc, device=DEV) * 2) if objective == 1 else bf(torch.rand(B, Kc, device=DEV) * 3 + 0.05)
    xi = torch.zeros(B, ld, device=DEV, dtype=torch.bfloat16)
    xi[:, :Kc] = x.bfloat16()
    y = torch.randint(0, Kc, (B,), device=DEV, dtype=torch.int32)
    mask = (torch.rand(B, Kc, device=DEV) > 0.25)
    mask[torch.arange(B), y.long()] = True
    tw = torch.rand(Kc, device=DEV) if marginal else None
    w = 0.2
    delta = torch.full((B, ld), float("nan"), device=DEV, dtype=torch.bfloat16)
    probs = torch.full((B, Kc), float("nan"), device=DEV)
    loss = torch.zeros(1, device=DEV)
    correct = torch.zeros(1, device=DEV, dtype=torch.int32)
    am = torch.zeros(B, device=DEV, dtype=torch.int32)
    K.categorical_loss(xi, B, Kc, ld, y, None, w, delta, objective, probs=probs, loss_sum=loss, correct=correct,
                       argmax_out=am, mask=mask.to(torch.uint8), target_w=tw)
    xr = x.clone().requires_grad_()
    if objective == 1:
        v = torch.softmax(xr.masked_fill(~mask, float("-inf")), 1)
    else:
        pos = xr.clamp_min(0) * mask
        v = pos / pos.sum(1, keepdim=True)
    mass = (v * tw).sum(1) if marginal else v[torch.arange(B), y.long()]
    ref = ((-torch.log(mass) if objective == 2 else 1 - mass) * w).sum()
    ref_delta = torch.autograd.grad(ref, xr)[0]
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    close(delta[:, :Kc], ref_delta, atol=3e-3, rtol=2e-2)
    close(probs, v.detach(), atol=1e-3, rtol=1e-2)
    assert (delta[:, Kc:].float() == 0).all()
    first = x.masked_fill(~mask, float("-inf")).argmax(1)
    assert torch.equal(am.long(), first) and correct.item() == int((first == y.long()).sum())


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 5])
def test_sgd_fused_rules(mode):
    from rembrandt_b200.optim.sgd import reference_step
    torch.manual_seed(12)
    n = 4099
    w = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV)
    v = torch.randn(n, device=DEV) * 0.1
    w16 = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    rw, rg, rv = reference_step(w.clone(), g.clone(), v.clone(), lr=0.1, mu=0.9, l2=5e-4, grad_scale=0.5, mode=mode)
    K.sgd_fused(w, g, v, w16, n, 0.1, 0.9, 5e-4, 0.5, mode)
    close(w, rw, rtol=1e-5, atol=1e-5)
    close(v, rv, rtol=1e-5, atol=1e-5)
    close(g, rg, rtol=1e-5, atol=1e-5)
    close(w16, rw.bfloat16(), rtol=1e-2, atol=1e-2)


def test_colsum_and_bias_act():
    torch.manual_seed(13)
    rows, C = 1000, 96
    x = bf(torch.randn(rows, C, device=DEV))
    out = torch.ones(C, device=DEV)
    K.colsum(x.bfloat16(), rows, C, C, out)
    close(out, 1 + x.sum(0), rtol=1e-3)
    acc = torch.randn(rows, C, device=DEV)
    bias = torch.randn(80, device=DEV)
    y = torch.full((rows, C), float("nan"), device=DEV, dtype=torch.bfloat16)
    ref = torch.zeros(rows, C, device=DEV)
    ref[:, :80] = torch.relu(acc[:, :80] + bias)
    K.bias_act(acc, rows, C, 80, bias, True, y)
    close(y, ref)
    assert (acc == 0).all()


@pytest.mark.parametrize("N,C,H", [(4, 64, 5), (6, 128, 9), (3, 512, 7), (5, 96, 6), (2, 320, 8), (33, 64, 12),
                                   (2, 1024, 4)])
def test_bn_forward_backward(N, C, H):
    """Channel counts whose 8-channel groups divide a block (64, 128, 512, 1024) take the reduction that spreads
    rows over the lanes; 96 and 320 take the slab-per-block one."""
    torch.manual_seed(14)
    rows = N * H * H
    x = bf(torch.randn(N, C, H, H, device=DEV) * 2 + 1).requires_grad_()
    gamma = (torch.rand(C, device=DEV) + 0.5).requires_grad_()
    beta = torch.randn(C, device=DEV).requires_grad_()
    rm, rv = torch.zeros(C, device=DEV), torch.ones(C, device=DEV)
    ref = torch.relu(F.batch_norm(x, rm.clone(), rv.clone(), gamma, beta, training=True, momentum=0.1, eps=1e-5))
    xi = layout.to_nhwc_padded(x.detach(), C)
    sums = torch.zeros(2 * C, device=DEV)
    mean, istd = torch.empty(C, device=DEV), torch.empty(C, device=DEV)
    y = torch.full((N, H, H, C), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.bn_fwd_train(xi, rows, C, C, sums, 1e-5, 0.1, mean, istd, rm, rv, gamma.detach(), beta.detach(), None, y, True)
    close(layout.from_nhwc_padded(y, C), ref.detach())
    assert (sums == 0).all()
    dy = bf(torch.randn_like(ref))
    gx, gg, gb = torch.autograd.grad(ref, [x, gamma, beta], dy)
    dgamma, dbeta = torch.zeros(C, device=DEV), torch.zeros(C, device=DEV)
    dx = torch.full((N, H, H, C), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.bn_bwd(xi, layout.to_nhwc_padded(dy, C), y, rows, C, C, sums, mean, istd, gamma.detach(), dgamma, dbeta, dx)
    close(layout.from_nhwc_padded(dx, C), gx, rtol=5e-2)
    close(dgamma, gg, rtol=5e-2)
    close(dbeta, gb, rtol=5e-2)


def test_bn_statistics_of_channels_whose_mean_dwarfs_their_spread():
    """Channels at 200 +- 0.5 in bf16 (values on a grid of 1): E[x^2] - E[x]^2 in fp32 would lose the variance;
    the shifted sums keep it."""
    torch.manual_seed(16)
    rows, C = 4096, 32
    x = (200.0 + torch.randn(rows, C, device=DEV) * 0.5).bfloat16()
    xf = x.float()
    sums = torch.zeros(2 * C, device=DEV)
    mean, istd = torch.empty(C, device=DEV), torch.empty(C, device=DEV)
    rm, rv = torch.zeros(C, device=DEV), torch.ones(C, device=DEV)
    g, b = torch.ones(C, device=DEV), torch.zeros(C, device=DEV)
    y = torch.empty(rows, C, device=DEV, dtype=torch.bfloat16)
    K.bn_fwd_train(x, rows, C, C, sums, 1e-5, 1.0, mean, istd, rm, rv, g, b, None, y, False)
    var = xf.var(0, unbiased=False)
    assert torch.allclose(mean, xf.mean(0), rtol=0, atol=1e-3)
    assert torch.allclose(istd, torch.rsqrt(var + 1e-5), rtol=1e-3)
    assert torch.allclose(rv, xf.var(0, unbiased=True), rtol=1e-3)


def test_input_pipeline_center_crop_and_s2d():
    torch.manual_seed(15)
    N, C, H = 3, 3, 40
    src = torch.randint(0, 256, (N, C, H, H), device=DEV, dtype=torch.uint8)
    mean = torch.rand(C, H, H, device=DEV) * 255
    crop = 32
    Cp = 32
    dst = torch.full((N, crop, crop, Cp), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.input_u8(src, mean, dst, N, C, H, H, crop, crop, crop, crop, Cp, 1, 0, H - crop, 0, H - crop, False, False,
               False, 1 / 255.0, 1 / 255.0, 0.0, None, None, 1, 0)
    o = (H - crop) // 2
    ref = (src.float() - mean)[:, :, o:o + crop, o:o + crop] / 255.0
    close(layout.from_nhwc_padded(dst, C), ref, atol=1e-2)
    # space-to-depth output equals the host-side rearrangement
    f, out_hw = 4, 10
    cp2 = 64
    dst2 = torch.full((N, out_hw, out_hw, cp2), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.input_u8(src, None, dst2, N, C, H, H, H, H, out_hw, out_hw, cp2, f, 0, 0, 0, 0, False, False, False, 1.0, 0.0,
               0.0, None, None, 1, 0)
    assert torch.equal(dst2, layout.s2d_input(src.float(), f, out_hw, cp2))


def test_input_pipeline_random_crop_flip_is_a_crop_of_the_source():
    N, C, H, crop = 8, 3, 32, 32
    src = torch.randint(0, 256, (N, C, H, H), device=DEV, dtype=torch.uint8)
    dst = torch.empty((N, crop, crop, 32), device=DEV, dtype=torch.bfloat16)
    # pad-4 random crop: the window's corner ranges over [-4, 4]
    K.input_u8(src, None, dst, N, C, H, H, crop, crop, crop, crop, 32, 1, -4, 4, -4, 4, True, True, False, 1.0, 0.0,
               0.0, None, None, 99, 3)
    out = layout.from_nhwc_padded(dst, C)
    padded = F.pad(src.float(), (4, 4, 4, 4))
    for n in range(N):
        found = False
        for oy in range(9):
            for ox in range(9):
                win = padded[n, :, oy:oy + crop, ox:ox + crop]
                if torch.equal(out[n], win) or torch.equal(out[n], win.flip(-1)):
                    found = True
        assert found, f"sample {n} is not a (flipped) crop of its source"


@pytest.mark.parametrize("n,k,nnz,transposed", [(361, 2000, 400, True), (361, 2000, 400, False), (2000, 361, 10, True),
                                                (77, 129, 129, False), (361, 20000, 2000, True)])
def test_gemv_sparse_matches_dense_product(n, k, nnz, transposed):
    """Matrix x sparse vector (the board-game layers of tools/bench-cublas.rs) against the dense product in fp32."""
    torch.manual_seed(31)
    w = torch.randn(n, k, device=DEV)
    ind = torch.randperm(k, device=DEV)[:nnz].int()
    val = torch.randn(nnz, device=DEV)
    x = torch.zeros(k, device=DEV)
    x[ind.long()] = val
    y0 = torch.randn(n, device=DEV)
    y = y0.clone()
    wm = w.t().contiguous() if transposed else w
    K.gemv_sparse(wm, n, k, transposed, val, ind, nnz, y, alpha=0.5, beta=2.0)
    status_ok()
    ref = 2.0 * y0 + 0.5 * (w.double() @ x.double()).float()
    assert torch.allclose(y, ref, rtol=1e-4, atol=1e-3 * float(ref.abs().max()))
    y = torch.full((n,), float("nan"), device=DEV)
    K.gemv_sparse(wm, n, k, transposed, val, ind, nnz, y)       # beta = 0 overwrites whatever was there
    assert torch.allclose(y, (w.double() @ x.double()).float(), rtol=1e-4, atol=1e-3 * float(ref.abs().max()))

