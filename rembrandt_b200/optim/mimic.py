"""Distillation ("mimic") training: a student network is fitted to a teacher network.

Counterpart of the reference's ``MimicSgdOptimizer`` (src/old_opt.rs:372-470), which runs a trained "target"
network in inference mode on every batch and hands its result to the loss layer of the network being trained. The
reference has two forms of that hand-over: the teacher's output probabilities (``recv_target_probs``, the one left
enabled, src/old_opt.rs:427-430) and the activations that enter the teacher's loss layer (``recv_target``, commented
out there, src/old_opt.rs:420-425). Both exist here:

* ``target="probs"`` (default): the teacher's probabilities become the soft targets of the student's softmax head
  (delta = w (p - q), loss = -sum q log p, one fused kernel on the GPU);
* ``target="activations"``: the student ends in an L2 head (``pointwise_loss`` with kind "l2") whose targets are the
  teacher's pre-softmax activations, the form used to fit a low-rank (``mimic_affine``) network to a wide one.

Labels still drive the reported accuracy of the softmax form.
"""
from __future__ import annotations

import torch

from ..trainer import SgdOpt


class MimicSgdOpt(SgdOpt):
    def __init__(self, config, engine, teacher, target="probs", **kw):
        super().__init__(config, engine, **kw)
        if teacher.batch != self.net.batch:
            raise ValueError("teacher and student must use the same batch size")
        if teacher.loss_op.k * teacher.loss_op.heads != self.net.loss_op.k * self.net.loss_op.heads:
            raise ValueError("teacher and student must have the same number of outputs")
        if target not in ("probs", "activations"):
            raise ValueError(f"unknown distillation target {target!r}")
        if target == "activations" and not hasattr(self.net.loss_op, "load_targets"):
            raise ValueError("distilling activations needs a student that ends in an L2 head (pointwise_loss 'l2')")
        self.teacher = teacher
        self.target = target
        if target == "probs":
            teacher.loss_op.enable_probs()

    def _teacher_output(self):
        t = self.teacher
        if self.target == "probs":
            return t.loss_op.probs
        if t.is_cuda:
            logits, _ = t.loss_op._logits()       # [batch, ..., padded outputs]
            return logits.reshape(t.batch, -1)[:, : t.loss_op.k * t.loss_op.heads]
        return t._cpu_logits.flatten(1)

    def _hand_over(self):
        out = self._teacher_output()
        if self.target == "probs":
            self.net.loss_op.load_soft_targets(out)
        else:
            self.net.loss_op.load_targets(out.detach())

    def before_step(self, images, labels):
        t, eng = self.teacher, self.engine
        if t.is_cuda:
            with torch.cuda.stream(eng.compute_stream):
                t.load_batch(images.to(t.device, non_blocking=True), labels.to(t.device, non_blocking=True).int())
                t.forward(False)
                self._hand_over()
        else:
            t.load_batch(images, labels)
            with torch.no_grad():
                t.forward(False)
            t.read_stats()
            self._hand_over()
