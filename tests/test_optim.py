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
