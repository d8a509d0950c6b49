"""SGD configuration, momentum rules and step-size schedules.

Mirrors the reference's ``SgdOptConfig`` family (src/opt/sgd/mod.rs:20-161) and the update rules of its
training loop (src/opt/sgd/new.rs:377-463), plus the gen-2 / gen-1 schedules (src/opt_new.rs:73-118,
src/old_opt.rs:18-47). ``reference_step`` is the plain-torch statement of each rule: it is the CPU path
of the optimizer and the oracle the fused CUDA kernel is tested against.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional, Sequence



class Momentum(enum.IntEnum):
    """Momentum rule; the integer is the `mode` of the fused kernel."""
    ZERO = 0
    UPDATE = 1
    UPDATE_NESTEROV = 2
    GRADIENT = 3
    GRADIENT_NESTEROV = 4
    GRAD_DECAY = 5  # gen-2: gradients are scaled by mu instead of zeroed


class SyncOrder(enum.Enum):
    STEP_THEN_SYNC_PARAMS = "step_then_sync_params"
    SYNC_PARAMS_THEN_STEP = "sync_params_then_step"
    SYNC_GRADS_THEN_STEP = "sync_grads_then_step"
    SYNC_PARAMS_AND_GRADS_THEN_STEP = "sync_params_and_grads_then_step"


class StepSizeReference(enum.Enum):
    LOCAL = "local"            # schedule evaluated every iteration
    CHECKPOINT = "checkpoint"  # schedule evaluated only at checkpoints


class CheckpointBehavior(enum.Enum):
    DISCARD = "discard"  # validate on the averaged model, keep training the local one
    KEEP = "keep"


class InitBehavior(enum.Enum):
    INIT_OR_RESUME = "init_or_resume"
    RESUME_FROM = "resume_from"


# ------------------------------------------------------------------------------------------ schedules
@dataclass
class StepSizeSchedule:
    """Step size as a function of the iteration counter.

    kinds: constant | anneal (piecewise constant: ``steps`` = [(t_threshold, value), ...]) |
    inverse (s/(1+s*lambda*t)) | decay (s*rate^(t // iters)) | inv (s/(1+t/tau)) | step (s*decay^(t // iters))
    """
    kind: str = "constant"
    step0: float = 0.01
    steps: Sequence[tuple] = ()
    lam: float = 0.0
    rate: float = 1.0
    iters: int = 1
    tau: float = 1.0

    def at_iter(self, t: int) -> float:
        k = self.kind
        if k == "constant":
            return self.step0
        if k == "anneal":
            s = self.step0
            for thr, val in self.steps:
                if t >= thr:
                    s = val
            return s
        if k == "inverse":
            return self.step0 / (1.0 + self.step0 * self.lam * t)
        if k in ("decay", "step"):
            return self.step0 * (self.rate ** (t // max(1, self.iters)))
        if k == "inv":
            return self.step0 / (1.0 + t / self.tau)
        raise ValueError(f"unknown schedule kind {k!r}")

    # constructors named after the reference variants
    @staticmethod
    def constant(step0):
        return StepSizeSchedule("constant", step0)

    @staticmethod
    def anneal1(step0, t1, step1):
        return StepSizeSchedule("anneal", step0, [(t1, step1)])

    @staticmethod
    def anneal2(step0, t1, step1, t2, step2):
        return StepSizeSchedule("anneal", step0, [(t1, step1), (t2, step2)])

    @staticmethod
    def anneal4(step0, t1, s1, t2, s2, t3, s3, t4, s4):
        return StepSizeSchedule("anneal", step0, [(t1, s1), (t2, s2), (t3, s3), (t4, s4)])

    @staticmethod
    def inverse(step0, lam):
        return StepSizeSchedule("inverse", step0, lam=lam)

    @staticmethod
    def decay(step0, rate, iters):
        return StepSizeSchedule("decay", step0, rate=rate, iters=iters)

    @staticmethod
    def inv(step0, tau):
        return StepSizeSchedule("inv", step0, tau=tau)

    # the second generation's names (src/opt_new.rs:52-106): all piecewise-constant or geometric forms of the above
    @staticmethod
    def fixed(lr):
        return StepSizeSchedule.constant(lr)

    @staticmethod
    def step_once(lr0, lr0_iters, lr_final):
        return StepSizeSchedule.anneal1(lr0, lr0_iters, lr_final)

    decay_once = step_once

    @staticmethod
    def step_twice(lr0, lr0_iters, lr1, lr1_iters, lr_final):
        return StepSizeSchedule.anneal2(lr0, lr0_iters, lr1, lr1_iters, lr_final)

    @staticmethod
    def from_annealing_policy(step0: float, policy: Optional[dict]):
        """`annealing_policy` table of a .model file's [opt] section."""
        if not policy or policy.get("kind") in (None, "none"):
            return StepSizeSchedule.constant(step0)
        kind = policy["kind"]
        if kind == "step":
            return StepSizeSchedule.decay(step0, policy.get("decay", 0.1), policy["step_iters"])
        if kind == "step_once":
            return StepSizeSchedule.anneal1(step0, policy["step_iters"], step0 * policy.get("decay", 0.1))
        if kind == "step_twice":
            d = policy.get("decay", 0.1)
            return StepSizeSchedule.anneal2(step0, policy["first_step"], step0 * d, policy["second_step"],
                                            step0 * d * d)
        if kind == "inv":
            return StepSizeSchedule.inv(step0, policy["time_scale"])
        raise ValueError(f"unknown annealing policy {kind!r}")


@dataclass
class SgdOptConfig:
    init: InitBehavior = InitBehavior.INIT_OR_RESUME
    resume_t: int = 0
    minibatch_size: int = 128          # per worker; a multiple of the batch size => gradient accumulation
    step_size: StepSizeSchedule = field(default_factory=StepSizeSchedule)
    step_ref: StepSizeReference = StepSizeReference.LOCAL
    momentum: Momentum = Momentum.UPDATE
    mu: float = 0.9
    l2_reg_coef: float = 0.0
    sync_order: SyncOrder = SyncOrder.SYNC_GRADS_THEN_STEP
    comm_interval: int = 1
    checkpoint: CheckpointBehavior = CheckpointBehavior.DISCARD
    display_iters: int = 100
    checkpoint_iters: int = 0          # 0 = never
    save_iters: int = 0
    valid_iters: int = 0
    checkpoint_dir: Optional[str] = None
    max_iters: int = 0


# ------------------------------------------------------------------------------------------ rules
def reference_step(w, g, v, lr, mu, l2, grad_scale, mode, phase=7):
    """One optimizer step on plain tensors (modified in place, also returned).

    Same contract as the fused kernel: ``phase`` bit 1 = regularise + accumulate into ``v``, bit 2 = apply
    to ``w``, bit 4 = zero ``g``.
    """
    mode = int(mode)
    acc, upd, zero = bool(phase & 1), bool(phase & 2), bool(phase & 4)
    gp = grad_scale * g + l2 * w
    if mode in (0, 1):
        if acc:
            v.copy_((0.0 if mode == 0 else mu) * v - lr * gp)
        if upd:
            w.add_(v)
    elif mode == 2:
        if acc:
            w.sub_(mu * v)
            v.copy_(mu * v - lr * gp)
        if upd:
            w.add_(v + mu * v)
    elif mode == 3:
        if acc:
            v.copy_(mu * v + gp)
        if upd:
            w.sub_(lr * v)
    elif mode == 4:
        if acc:
            v.copy_(mu * v + gp)
        if upd:
            w.sub_(lr * gp + lr * mu * v)
    elif mode == 5:
        if upd:   # the decay of the gradient belongs to the applying phase, so that split phases decay it once
            w.sub_(lr * gp)
            g.copy_(mu * gp)
    else:
        raise ValueError(mode)
    if zero and mode != 5:
        g.zero_()
    return w, g, v
