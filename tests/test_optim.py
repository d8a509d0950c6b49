"""Momentum rules, phase splitting and step-size schedules against closed-form NumPy statements (CPU)."""
import numpy as np
import pytest
import torch

from rembrandt_b200.optim.sgd import Momentum, StepSizeSchedule, reference_step


def numpy_rule(mode, w, g, v, lr, mu, l2, scale):
    gp = scale * g + l2 * w
    if mode == Momentum.ZERO:
        v = -lr * gp
        w = w + v
    elif mode == Momentum.UPDATE:
        v = mu * v - lr * gp
        w = w + v
    elif mode == Momentum.UPDATE_NESTEROV:
        w = w - mu * v
        v = mu * v - lr * gp
        w = w + v + mu * v
    elif mode == Momentum.GRADIENT:
        v = mu * v + gp
        w = w - lr * v
    elif mode == Momentum.GRADIENT_NESTEROV:
        v = mu * v + gp
        w = w - lr * gp - lr * mu * v
    return w, v


@pytest.mark.parametrize("mode", [Momentum.ZERO, Momentum.UPDATE, Momentum.UPDATE_NESTEROV, Momentum.GRADIENT,
                                  Momentum.GRADIENT_NESTEROV])
def test_rules_match_closed_form_over_several_steps(mode):
    rng = np.random.default_rng(int(mode))
    w = rng.standard_normal(50)
    v = np.zeros(50)
    tw, tv = torch.tensor(w), torch.tensor(v)
    for step in range(4):
        g = rng.standard_normal(50)
        w, v = numpy_rule(mode, w, g, v, 0.1, 0.9, 1e-3, 0.5)
        tg = torch.tensor(g)
        reference_step(tw, tg, tv, 0.1, 0.9, 1e-3, 0.5, mode)
        assert np.allclose(tw.numpy(), w) and np.allclose(tv.numpy(), v)
        assert float(tg.abs().max()) == 0.0


def test_nesterov_update_keeps_parameters_at_the_lookahead_point():
    """theta_stored = theta + mu v: stepping the stored form equals classical momentum on theta."""
    rng = np.random.default_rng(1)
    theta = rng.standard_normal(20)
    v = np.zeros(20)
    stored, tv = torch.tensor(theta.copy()), torch.zeros(20, dtype=torch.float64)
    for _ in range(5):
        g = rng.standard_normal(20)
        v = 0.9 * v - 0.05 * g
        theta = theta + v
        reference_step(stored, torch.tensor(g), tv, 0.05, 0.9, 0.0, 1.0, Momentum.UPDATE_NESTEROV)
        assert np.allclose(stored.numpy(), theta + 0.9 * v)


def test_grad_decay_rule_scales_gradients_instead_of_zeroing():
    w, g, v = torch.ones(4), torch.full((4,), 2.0), torch.zeros(4)
    reference_step(w, g, v, 0.1, 0.5, 0.0, 1.0, Momentum.GRAD_DECAY)
    assert torch.allclose(w, torch.full((4,), 0.8)) and torch.allclose(g, torch.full((4,), 1.0))


@pytest.mark.parametrize("mode", [Momentum.UPDATE, Momentum.GRADIENT, Momentum.UPDATE_NESTEROV])
def test_split_phases_equal_the_fused_step(mode):
    torch.manual_seed(0)
    w1, g1, v1 = torch.randn(30), torch.randn(30), torch.randn(30) * 0.1
    w2, g2, v2 = w1.clone(), g1.clone(), v1.clone()
    reference_step(w1, g1, v1, 0.1, 0.9, 1e-3, 1.0, mode, phase=7)
    reference_step(w2, g2, v2, 0.1, 0.9, 1e-3, 1.0, mode, phase=1)
    reference_step(w2, g2, v2, 0.1, 0.9, 1e-3, 1.0, mode, phase=6)
    assert torch.allclose(w1, w2) and torch.allclose(v1, v2) and float(g2.abs().max()) == 0.0


def test_second_generation_schedule_names():
    s = StepSizeSchedule.step_twice(0.1, 10, 0.01, 20, 0.001)
    assert [s.at_iter(t) for t in (0, 9, 10, 19, 20, 99)] == [0.1, 0.1, 0.01, 0.01, 0.001, 0.001]
    assert StepSizeSchedule.decay_once(0.5, 3, 0.05).at_iter(3) == 0.05 and StepSizeSchedule.fixed(0.2).at_iter(7) == 0.2
    d = StepSizeSchedule.decay(1.0, 0.5, 4)
    assert [d.at_iter(t) for t in (0, 3, 4, 8)] == [1.0, 1.0, 0.5, 0.25]


def test_schedules():
    assert StepSizeSchedule.constant(0.3).at_iter(10**6) == 0.3
    a2 = StepSizeSchedule.anneal2(0.1, 18750, 0.01, 37500, 0.001)
    assert [a2.at_iter(t) for t in (0, 18749, 18750, 37499, 37500)] == [0.1, 0.1, 0.01, 0.01, 0.001]
    a4 = StepSizeSchedule.anneal4(1.0, 10, 0.5, 20, 0.25, 30, 0.125, 40, 0.0625)
    assert a4.at_iter(35) == 0.125 and a4.at_iter(40) == 0.0625
    inv = StepSizeSchedule.inverse(0.1, 0.01)
    assert abs(inv.at_iter(100) - 0.1 / (1 + 0.1 * 0.01 * 100)) < 1e-12
    dec = StepSizeSchedule.decay(0.01, 0.1, 200000)
    assert dec.at_iter(199999) == 0.01 and abs(dec.at_iter(400000) - 1e-4) < 1e-15
    assert abs(StepSizeSchedule.inv(0.1, 50.0).at_iter(50) - 0.05) < 1e-12
    pol = StepSizeSchedule.from_annealing_policy(0.01, {"kind": "step", "step_iters": 10, "decay": 0.5})
    assert pol.at_iter(25) == 0.01 * 0.25
    assert StepSizeSchedule.from_annealing_policy(0.02, None).at_iter(5) == 0.02


import pytest as _pytest


@_pytest.mark.parametrize("k,stride,pad,hw", [(3, 2, 1, 15), (3, 2, 1, 16), (1, 2, 0, 14), (7, 2, 3, 21), (5, 3, 2, 17),
                                              (3, 2, 0, 11), (4, 2, 1, 12)])
def test_strided_data_grad_phase_decomposition_equals_autograd(k, stride, pad, hw):
    """The arithmetic of the phase-by-phase strided data-grad (what the tensor-core path computes) against autograd."""
    import torch
    import torch.nn.functional as F
    from rembrandt_b200.ops.conv_strided import dgrad_by_phases_reference, phase_plan
    torch.manual_seed(k * 100 + stride * 10 + pad)
    N, C, Ko = 2, 5, 7
    x = torch.randn(N, C, hw, hw + 1, dtype=torch.float64, requires_grad=True)
    w = torch.randn(Ko, C, k, k, dtype=torch.float64)
    y = F.conv2d(x, w, stride=stride, padding=pad)
    dy = torch.randn_like(y)
    ref = torch.autograd.grad(y, x, dy)[0]
    got = dgrad_by_phases_reference(dy, w, hw, hw + 1, stride, pad)
    assert torch.allclose(got, ref, atol=1e-10), float((got - ref).abs().max())
    assert len(phase_plan(hw, hw + 1, k, k, stride, pad)) == stride * stride


def test_strided_data_grad_device_path_packing_with_an_emulated_kernel(monkeypatch):
    """`dgrad_strided_tc` itself (filter slicing / flipping / padding, phase interleave, mask) with the forward kernel
    replaced by a plain-torch emulation of its contract, so the layout logic is checked without a GPU."""
    import torch
    import torch.nn.functional as F
    from rembrandt_b200.ops import conv_strided, layout
    from rembrandt_b200.ops import native_ops as K

    def fake_fprop(x, N, H, W, Cp, w, Kout, R, S, stride, pad_h, pad_w, P, Q, y, ldy, bias=None, relu=False,
                   mask_src=None, n_valid=0, n_store=0):
        assert stride == 1 and pad_h >= 0 and pad_w >= 0
        xi = x.float().permute(0, 3, 1, 2)                                     # [N, Cp, H, W]
        wi = w.float().view(Kout, R, S, Cp).permute(0, 3, 1, 2)                # [Kout, Cp, R, S]
        need_h, need_w = P + R - 1, Q + S - 1
        xi = F.pad(xi, (pad_w, max(0, need_w - pad_w - W), pad_h, max(0, need_h - pad_h - H)))[:, :, :need_h, :need_w]
        out = F.conv2d(xi, wi)                                                 # [N, Kout, P, Q]
        out[:, n_valid:] = 0
        y.copy_(out.permute(0, 2, 3, 1).to(y.dtype))

    def fake_mask(d, m, n):
        d.mul_((m.float() > 0).to(d.dtype))

    monkeypatch.setattr(K, "conv_fprop_tc", fake_fprop)
    monkeypatch.setattr(K, "relu_mask", fake_mask)
    torch.manual_seed(4)
    for (C, Ko, R, stride, pad, H, W) in ((5, 7, 3, 2, 1, 9, 10), (8, 6, 1, 2, 0, 8, 8), (3, 4, 5, 3, 2, 11, 13)):
        N = 2
        Cp, Kp = K.pad_channels(C), K.pad_channels(Ko)
        x = torch.randn(N, C, H, W, requires_grad=True)
        w = torch.randn(Ko, C, R, R)
        y = F.conv2d(x, w, stride=stride, padding=pad)
        dy = torch.randn_like(y)
        mask = torch.randn(N, C, H, W)
        ref = torch.autograd.grad(y, x, dy)[0] * (mask > 0)
        dx = torch.full((N, H, W, Cp), float("nan"))
        wi = layout.conv_weight_to_internal(w, Cp)
        cache = {}
        for _ in range(2):   # the second call reuses the cached per-phase buffers
            ok = conv_strided.dgrad_strided_tc(layout.to_nhwc_padded(dy, Kp).float(), N, y.shape[2], y.shape[3], Kp, wi,
                                               Ko, Cp, C, R, R, stride, pad, H, W, dx,
                                               layout.to_nhwc_padded(mask, Cp).float(), cache=cache)
            assert ok
        assert len(cache) == sum(1 for ph in conv_strided.phase_plan(H, W, R, R, stride, pad) if ph.U and ph.V)
        got = layout.from_nhwc_padded(dx, C)
        assert torch.allclose(got.float(), ref, atol=2e-2, rtol=2e-2), float((got.float() - ref).abs().max())
        assert (dx[..., C:] == 0).all()
