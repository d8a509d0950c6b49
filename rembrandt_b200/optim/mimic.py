"""Distillation ("mimic") training: a student network is fitted to a teacher network's softmax output.

Counterpart of the reference's ``MimicSgdOptimizer`` (src/old_opt.rs), which trains a compressed network against the
activations of a trained one. Here the target is the teacher's output distribution: before every batch the teacher
runs an inference pass on the same batch, its probabilities become the soft targets of the student's softmax head
(delta = w (p - q), loss = -sum q log p, one fused kernel on the GPU), and the usual SGD step follows. Labels still
drive the reported accuracy.
"""
from __future__ import annotations

import torch

from ..trainer import SgdOpt


class MimicSgdOpt(SgdOpt):
    def __init__(self, config, engine, teacher, **kw):
        super().__init__(config, engine, **kw)
        if teacher.batch != self.net.batch:
            raise ValueError("teacher and student must use the same batch size")
        if teacher.loss_op.k * teacher.loss_op.heads != self.net.loss_op.k * self.net.loss_op.heads:
            raise ValueError("teacher and student must have the same number of outputs")
        self.teacher = teacher
        teacher.loss_op.enable_probs()

    def before_step(self, images, labels):
        t, eng = self.teacher, self.engine
        if t.is_cuda:
            with torch.cuda.stream(eng.compute_stream):
                t.load_batch(images.to(t.device, non_blocking=True), labels.to(t.device, non_blocking=True).int())
                t.forward(False)
                self.net.loss_op.load_soft_targets(t.loss_op.probs)
        else:
            t.load_batch(images, labels)
            with torch.no_grad():
                t.forward(False)
            t.read_stats()
            self.net.loss_op.load_soft_targets(t.loss_op.probs)
