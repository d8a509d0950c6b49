"""SGD loop without the shared checkpoint barrier: every worker checkpoints, validates and continues on its own
clock, on its own local model (the reference's older ``AsyncSgdOpt``, src/opt/sgd/async.rs, which pre-dates the
shared ``OptSharedData`` barrier and is no longer compiled there).

Intended for the gossip / elastic backends, whose exchanges tolerate workers that are steps apart; a backend that has
a lock-step and an asynchronous form (push gossip, pull gossip, elastic averaging on the kernel backend) must be in
its asynchronous form, or its own cross-GPU barriers would put the ranks back in step. Differences to
``SgdOpt``: no barrier before or after the checkpoint window, no exact synchronisation of the parameters at a
checkpoint (each rank writes its own parameter files under ``<checkpoint_dir>/rank<r>``), and the displayed training
statistics are this rank's alone.
"""
from __future__ import annotations

import os

from ..optim.sgd import CheckpointBehavior
from ..trainer import SgdOpt
from ..utils import checkpoint as ckpt


class _LocalStats:
    """Stand-in for the shared statistics exchange: a rank reports its own numbers."""

    def sync(self, values):
        return list(values)


class AsyncSgdOpt(SgdOpt):
    def __init__(self, config, engine, **kw):
        super().__init__(config, engine, **kw)
        self.shared = _LocalStats()
        if self.world > 1 and getattr(self.comm, "synchronous", False):
            raise ValueError(f"{self.comm.name} is in its lock-step form (synchronous=True): its exchanges contain "
                             "cross-GPU barriers, which a barrier-free loop must not run")

    # the loop's own barriers do nothing here; the communication backend is left as it is
    def _signal_barrier(self):
        pass

    def _wait_barrier(self) -> bool:
        return True

    def _barrier(self):
        pass

    def _checkpoint_window(self, t, valid_data, t_start):
        cfg, eng, net = self.cfg, self.engine, self.net
        eng.flush()
        eng.synchronize()
        self._check_device_status(t)
        if cfg.checkpoint == CheckpointBehavior.DISCARD:
            net.save_params()
        if cfg.checkpoint_dir:
            local_dir = os.path.join(cfg.checkpoint_dir, f"rank{self.rank}")
            os.makedirs(local_dir, exist_ok=True)
            if cfg.save_iters and t % cfg.save_iters == 0:
                ckpt.checkpoint_state(net, local_dir, self.rank)
            ckpt.checkpoint_params(net, t, local_dir)
        if valid_data is not None and cfg.valid_iters:
            self.validate(valid_data, cfg.valid_iters, t, t_start)
        if cfg.checkpoint == CheckpointBehavior.DISCARD:
            net.restore_params()
