"""The training loop: ``SgdOpt``.

Follows the reference's ``SgdOpt::train`` / ``validate`` (src/opt/sgd/new.rs:209-765) step for step:

1. initialise or resume (``InitOrResume`` looks for a checkpoint, ``ResumeFrom{t}`` loads a given iteration);
2. Nesterov variants move the parameters to the look-ahead point once before training;
3. parameter-server backends upload rank 0's parameters (``first_one_way_sync``); all ranks pass a barrier;
4. per batch: load, forward, backward; per iteration (= minibatch_size / batch_size batches): regularise,
   exchange and update in the configured ``SyncOrder``, reset gradients, write a ``step`` row to the per-rank CSV
   trace, print a progress line on rank 0 every ``display_iters``;
5. every ``checkpoint_iters``: snapshot the local parameters (``Discard``), write the per-rank state blob every
   ``save_iters``, average the parameters exactly over all ranks, write the parameter blob on rank 0, validate,
   restore the local parameters, pass a barrier and re-evaluate the step size (``StepSizeReference::Checkpoint``).

What differs is underneath: batches go through ``StepEngine`` (pinned staging, CUDA graph, one-step-lagged
loss), throughput is measured on the device with CUDA events and reported as images/s, and the straggler
injection of the reference's experiment configuration (src/worker/gossip_dist.rs:1027-1031,1577-1582) is a
host-side sleep before the next launch, never a device-side stall.
"""
from __future__ import annotations

import csv
import os
import random
import sys
import time
from dataclasses import dataclass, field
from typing import Iterable, List, Optional

import torch

from .engine import StepEngine
from .optim.sgd import (CheckpointBehavior, InitBehavior, Momentum, SgdOptConfig, StepSizeReference)
from .utils import checkpoint as ckpt


@dataclass
class ExperimentConfig:
    straggler_ranks: List[int] = field(default_factory=list)
    straggler_max_delay_ms: int = 0


class OptSharedData:
    """Cross-rank accumulators for the progress line (the reference shares atomics between worker threads,
    src/opt/sgd/mod.rs:163-182; ranks here are processes, so the sums go through the comm backend)."""

    def __init__(self, comm):
        self.comm = comm

    def sync(self, values):
        return self.comm.allreduce_stats(values)


class TraceLog:
    """Per-rank CSV trace ``trace_sgd.{rank}.log`` with header ``t,event,loss,error,elapsed``; an existing file is
    never overwritten: the next free ``.N`` suffix is used (src/opt/sgd/new.rs:149-197)."""

    def __init__(self, directory: Optional[str], rank: int):
        self.file = None
        if not directory:
            return
        os.makedirs(directory, exist_ok=True)
        base = os.path.join(directory, f"trace_sgd.{rank}.log")
        path, n = base, 0
        while os.path.exists(path):
            n += 1
            path = f"{base}.{n}"
        self.path = path
        self.file = open(path, "w", newline="")
        self.writer = csv.writer(self.file)
        self.writer.writerow(["t", "event", "loss", "error", "elapsed"])
        self.file.flush()

    def row(self, t, event, loss, error, elapsed):
        if self.file:
            self.writer.writerow([t, event, f"{loss:.6f}", f"{error:.6f}", f"{elapsed:.6f}"])
            self.file.flush()

    def close(self):
        if self.file:
            self.file.close()
            self.file = None


class DeviceWaitTimeout(RuntimeError):
    """A kernel gave up a bounded wait on another rank (its flag never arrived): that rank is gone or stuck."""


class SgdOpt:
    def __init__(self, config: SgdOptConfig, engine: StepEngine, experiment: Optional[ExperimentConfig] = None,
                 log_dir: Optional[str] = None, report=None, quiet: bool = False):
        self.cfg = config
        self.engine = engine
        self.net = engine.net
        self.comm = engine.comm
        self.rank, self.world = self.comm.rank, self.comm.num_workers()
        self.experiment = experiment or ExperimentConfig()
        self.shared = OptSharedData(self.comm)
        self.trace = TraceLog(log_dir or config.checkpoint_dir, self.rank)
        self.report = report
        self.quiet = quiet
        self.history = []          # (iteration, loss, accuracy) at display points
        self.valid_history = []    # (iteration, loss, accuracy)
        self._straggle_rng = random.Random(1234 + self.rank)

    # ------------------------------------------------------------------ initialisation
    def _init_or_resume(self) -> int:
        cfg, net = self.cfg, self.net
        init_t = 0
        if cfg.init == InitBehavior.INIT_OR_RESUME:
            t = ckpt.can_rollback(cfg.checkpoint_dir, self.rank)
            if t is not None:
                ckpt.rollback_state(net, cfg.checkpoint_dir, self.rank)
                init_t = t
        elif cfg.init == InitBehavior.RESUME_FROM:
            init_t = ckpt.rollback_params(net, cfg.checkpoint_dir, cfg.resume_t)
        return init_t

    def _log(self, msg):
        if self.rank == 0 and not self.quiet:
            print(msg, file=sys.stderr, flush=True)

    def _exchange_rate(self, iters: int, device_ms: float) -> Optional[float]:
        """GB/s of exchange traffic per rank averaged over the device time of `iters` iterations: the flat vector
        once per exchange, times 2 (N - 1) / N for the all-reduce backends (the usual bus-bandwidth convention).
        The exchange overlaps the backward pass, so this is a rate the step sustains, not the speed of the exchange
        kernels alone (that is what `cli/bench_allreduce.py` measures)."""
        if self.world <= 1 or device_ms <= 0:
            return None
        exchanges = iters / max(1, self.cfg.comm_interval)
        payload = self.net.flat_len * 4.0 * exchanges
        if "allreduce" in self.comm.name and "gossip" not in self.comm.name:
            payload *= 2.0 * (self.world - 1) / self.world
        return payload / (device_ms * 1e-3) / 1e9

    # ------------------------------------------------------------------ failure detection
    def _device_status(self) -> int:
        """The status word in which the kernels record a wait that ran out (0 = healthy). One small device read;
        called only where the loop has just synchronised anyway."""
        if not self.engine.is_cuda:
            return 0
        from .ops import native_ops as K
        return K.read_status()

    def _check_device_status(self, t: int) -> None:
        """The exchange kernels never hang on a missing peer: they give up after a deadline, set a bit in the status
        word and return, and the step goes on with whatever data was there. The reference panics on any MPI / CUDA
        error (e.g. src/worker/allreduce_dist.rs:231); here the loop stops at the next display point instead: no
        collective can be trusted once a peer is gone, so this rank writes its own state beside the regular
        checkpoints (`state.abort.blob.<rank>`, never over them) and raises."""
        arena = getattr(self.comm, "arena", None)
        damaged = arena.damaged() if arena is not None else []
        if damaged:   # only with RB_ARENA_GUARD=1: some kernel wrote outside a peer-visible buffer
            raise RuntimeError(f"rank {self.rank}: guard bands of peer-visible buffers overwritten: {damaged}")
        status = self._device_status()
        if status == 0:
            return
        saved = None
        if self.cfg.checkpoint_dir:
            saved = ckpt.checkpoint_state(self.net, self.cfg.checkpoint_dir, self.rank, name="state.abort.blob")
        self.trace.row(t, "abort", float(status), 0.0, 0.0)
        self.trace.close()
        raise DeviceWaitTimeout(f"rank {self.rank}: device status {status:#x} at iteration {t}: a bounded wait on a "
                                f"peer ran out" + (f"; local state written to {saved}" if saved else ""))

    # ---- the checkpoint barrier of the synchronous loop (the barrier-free loop overrides these three)
    def _signal_barrier(self):
        self.comm.signal_barrier()

    def _wait_barrier(self) -> bool:
        return self.comm.wait_barrier()

    def _barrier(self):
        self.comm.barrier()

    def before_step(self, images, labels):
        """Hook run before every batch is fed (used by the distillation optimizer)."""

    # ------------------------------------------------------------------ training
    def train(self, train_data: Iterable, valid_data: Optional[Iterable] = None, max_iters: Optional[int] = None):
        cfg, eng, net, comm = self.cfg, self.engine, self.net, self.comm
        max_iters = max_iters if max_iters is not None else (cfg.max_iters or None)
        init_t = self._init_or_resume()
        eng.iter = init_t
        if cfg.momentum == Momentum.UPDATE_NESTEROV:
            eng.stepper.nesterov_lookahead(+1.0)
        with torch.no_grad():
            comm.first_one_way_sync(net.params)
        net.refresh_shadow()
        self._signal_barrier()
        while not self._wait_barrier():
            time.sleep(0.001)
        net.reset_grads()
        chkpt_step = cfg.step_size.at_iter(init_t)
        eng.set_lr(chkpt_step)

        batches_per_iter = eng.accum
        disp_loss = disp_correct = disp_samples = 0.0
        t_start = time.time()
        dev_t0 = dev_t1 = None
        if eng.is_cuda:
            dev_t0, dev_t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dev_t0.record(eng.compute_stream)
        disp_wall = time.time()
        epoch = 0
        done = False
        pending_rows = []  # iterations whose (lagged) loss has not arrived yet
        while not done:
            for images, labels in train_data:
                it_before = eng.iter
                self.before_step(images, labels)
                eng.feed(images, labels)
                stats = eng.step()
                if self.rank in self.experiment.straggler_ranks and self.experiment.straggler_max_delay_ms > 0:
                    time.sleep(self._straggle_rng.uniform(0, self.experiment.straggler_max_delay_ms) / 1e3)
                if stats is not None:
                    loss, correct = stats
                    disp_loss += loss
                    disp_correct += correct
                    disp_samples += net.batch
                    if pending_rows:
                        t_row = pending_rows.pop(0)
                        self.trace.row(t_row, "step", loss, 1.0 - correct / net.batch, time.time() - t_start)
                if eng.iter == it_before:
                    continue   # inside a gradient-accumulation group
                t = eng.iter
                pending_rows.append(t) if eng.is_cuda else self.trace.row(
                    t, "step", stats[0], 1.0 - stats[1] / net.batch, time.time() - t_start)
                if cfg.step_ref == StepSizeReference.LOCAL:
                    eng.set_lr(cfg.step_size.at_iter(t))
                else:
                    eng.set_lr(chkpt_step)
                comm.hack_set_step_size(eng.lr)

                if cfg.display_iters and t % cfg.display_iters == 0:
                    ips = bus = None
                    if eng.is_cuda:
                        dev_t1.record(eng.compute_stream)
                        dev_t1.synchronize()
                        ms = dev_t0.elapsed_time(dev_t1)
                        ips = cfg.display_iters * batches_per_iter * net.batch * self.world / (ms / 1e3)
                        bus = self._exchange_rate(cfg.display_iters, ms)
                        dev_t0, dev_t1 = dev_t1, torch.cuda.Event(enable_timing=True)
                    self._check_device_status(t)
                    sums = self.shared.sync([disp_loss, disp_correct, disp_samples])
                    n = max(1.0, sums[2])
                    avg_loss = sums[0] * batches_per_iter / max(1.0, sums[2] / net.batch)
                    acc = sums[1] / n
                    self.history.append((t, avg_loss, acc))
                    if self.report is not None:
                        self.report.update_training(t, avg_loss, acc)
                    wall = time.time() - disp_wall
                    disp_wall = time.time()
                    self._log(f"iter {t} epoch {epoch} step {eng.lr:.6g} loss {avg_loss:.4f} accuracy {acc:.4f} "
                              f"elapsed {wall:.3f}s" + (f" device {ips:.0f} images/s" if ips else "") +
                              (f" exchange {bus:.1f} GB/s" if bus else ""))
                    disp_loss = disp_correct = disp_samples = 0.0

                if cfg.checkpoint_iters and t % cfg.checkpoint_iters == 0:
                    self._signal_barrier()
                    self._checkpoint_window(t, valid_data, t_start)
                    chkpt_step = cfg.step_size.at_iter(t)
                if max_iters and t >= max_iters:
                    done = True
                    break
            epoch += 1
            if max_iters is None and not done:
                done = True   # a finite iterable without an iteration limit: one pass
        last = eng.flush()
        if last is not None and pending_rows:
            self.trace.row(pending_rows.pop(0), "step", last[0], 1.0 - last[1] / net.batch, time.time() - t_start)
        eng.synchronize()
        return self.history

    @torch.no_grad()   # on CPU the flat parameter vector is an autograd leaf; the averaging mixes it in place
    def _checkpoint_window(self, t, valid_data, t_start):
        cfg, eng, net, comm = self.cfg, self.engine, self.net, self.comm
        eng.flush()
        eng.synchronize()
        self._check_device_status(t)
        while not self._wait_barrier():
            time.sleep(0.001)
        # a backend that shards the fp32 master (fused all-reduce + SGD) holds only this rank's shard up to date:
        # the snapshot, the state blob and the restore below all need the complete vector
        if hasattr(comm, "gather_master"):
            comm.gather_master()
        # the training loop keeps Nesterov parameters at the look-ahead point w + mu v; the reference takes the
        # extra momentum off before the update and puts it back after the checkpoint window
        # (src/opt/sgd/new.rs:360-369,623-634), so blobs hold the plain w and a resumed run applies it once
        nesterov = cfg.momentum == Momentum.UPDATE_NESTEROV
        if nesterov:
            eng.stepper.nesterov_lookahead(-1.0)
        if cfg.checkpoint == CheckpointBehavior.DISCARD:
            net.save_params()
        if cfg.checkpoint_dir and cfg.save_iters and t % cfg.save_iters == 0:
            ckpt.checkpoint_state(net, cfg.checkpoint_dir, self.rank)
        comm.exact_sync(net.params)
        net.refresh_shadow()
        if self.rank == 0 and cfg.checkpoint_dir:
            ckpt.checkpoint_params(net, t, cfg.checkpoint_dir)
        if valid_data is not None and cfg.valid_iters:
            self.validate(valid_data, cfg.valid_iters, t, t_start)
        if cfg.checkpoint == CheckpointBehavior.DISCARD:
            net.restore_params()
        if nesterov:
            eng.stepper.nesterov_lookahead(+1.0)
        self._barrier()

    # ------------------------------------------------------------------ validation
    def validate(self, valid_data: Iterable, num_batches: int, t: int = 0, t_start: Optional[float] = None):
        """Inference over `num_batches` batches of this rank's shard; statistics are summed over ranks."""
        eng, net = self.engine, self.net
        t0 = time.time()
        loss = correct = total = 0.0
        n = 0
        net.read_stats()
        for images, labels in valid_data:
            l, c = eng.eval_batch(images, labels)
            # the loss head weights samples by 1/minibatch; report the per-sample mean
            loss += l * net.minibatch_size
            correct += c
            total += net.batch
            n += 1
            if n >= num_batches:
                break
        sums = self.shared.sync([1.0, correct, total, loss])
        acc = sums[1] / max(1.0, sums[2])
        mean_loss = sums[3] / max(1.0, sums[2])
        self.valid_history.append((t, mean_loss, acc))
        self.trace.row(t, "valid", mean_loss, 1.0 - acc, (time.time() - t_start) if t_start else time.time() - t0)
        if self.report is not None:
            self.report.update_validation(t, mean_loss, acc)
        self._log(f"valid iter {t} loss {mean_loss:.4f} accuracy {acc:.4f} ({int(sums[2])} samples, "
                  f"{time.time() - t0:.3f}s)")
        return mean_loss, acc
