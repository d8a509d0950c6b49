"""Step engine: one replica's forward / backward / exchange / update, fed from pinned host memory.

This is the device-side half of the reference's training loop body (src/opt/sgd/new.rs:325-495): where the
reference issues one H2D copy per image, synchronises the stream several times per batch and launches every
kernel individually, the engine

* stages batches through two pinned-to-device buffers on a copy stream, so the H2D copy of batch i+1 overlaps
  the compute of batch i;
* captures forward + backward (+ exchange + update when the backend's kernels can be captured) in one CUDA
  graph and replays it per step;
* returns loss / accuracy with a one-step lag through a pinned host mirror, so the host never blocks on the
  step it has just launched.

On CPU the same interface runs the reference path eagerly.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .models.net import Net
from .optim.sgd import SgdOptConfig, SyncOrder
from .optim.stepper import SgdStepper
from .ops import native_ops as K
from .parallel.comm import CommWorker, NullComm
from .utils.trace import span


class StepEngine:
    def __init__(self, net: Net, opt: SgdOptConfig, comm: Optional[CommWorker] = None, use_graph: bool = True):
        self.net = net
        self.opt = opt
        self.comm = comm or NullComm()
        self.stepper = SgdStepper(net, opt.momentum, opt.mu, opt.l2_reg_coef)
        self.is_cuda = net.is_cuda
        self.use_graph = use_graph and self.is_cuda
        self.accum = max(1, opt.minibatch_size // net.batch)   # batches per optimizer iteration
        self.lr = opt.step_size.at_iter(0)
        self.iter = 0
        self._graphs = {}
        self._pending = None
        self._lag_stats = None
        self.launches_per_step = 0
        if self.is_cuda:
            dev = net.device
            self.compute_stream = torch.cuda.Stream(dev)
            self.copy_stream = torch.cuda.Stream(dev)
            io = net.input_op
            self._stage_imgs = [torch.zeros_like(io.stage) for _ in range(2)]
            self._stage_lbls = [torch.zeros_like(net.loss_op.labels) for _ in range(2)]
            # variable-size input: the per-sample (w, h) table travels with the padded pixel rows
            self._stage_shapes = [torch.ones_like(io.shapes) for _ in range(2)] if hasattr(io, "shapes") else None
            self._copy_done = [torch.cuda.Event() for _ in range(2)]
            self._consumed = [torch.cuda.Event() for _ in range(2)]
            self._slot = 0
            self._stats_dev = torch.zeros(2, dtype=torch.float32, device=dev)
            self._stats_host = [torch.zeros(2, dtype=torch.float32).pin_memory() for _ in range(2)]
            self._stats_ready = [torch.cuda.Event() for _ in range(2)]
            self._lr_dev = None
            # optional timing of the host-to-device copies (`time_h2d(True)`): pairs of events around each copy
            self._h2d_timing = False
            self._h2d_events = []
            if hasattr(self.comm, "attach"):
                self.comm.attach(self)

    # ------------------------------------------------------------------ feeding
    def feed(self, images_u8, labels: torch.Tensor) -> None:
        """Queue one batch: async H2D into the free staging slot (pinned source for a true async copy).

        Fixed-size input: a uint8 [B, C, H, W] tensor. Variable-size input: a list of uint8 [C, h, w] tensors, or the
        pair (padded uint8 [B, C * maxH * maxW], int32 [B, 2] of (w, h)) that `VarDataOp.pack` makes of such a list."""
        if not self.is_cuda:
            self.net.load_batch(images_u8, labels)
            return
        shapes = None
        if self._stage_shapes is not None:
            io = self.net.input_op
            if isinstance(images_u8, list) or images_u8[0].dim() == 3:
                images_u8 = io.pack(list(images_u8), io.in_stride)
            images_u8, shapes = images_u8
        s = self._slot
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self._consumed[s])
            if self._h2d_timing:
                t0 = torch.cuda.Event(enable_timing=True)
                t0.record(self.copy_stream)
            self._stage_imgs[s].copy_(images_u8.reshape(self._stage_imgs[s].shape), non_blocking=True)
            self._stage_lbls[s].copy_(labels.reshape(-1), non_blocking=True)
            if shapes is not None:
                self._stage_shapes[s].copy_(shapes.reshape(self._stage_shapes[s].shape).int(), non_blocking=True)
            self._copy_done[s].record(self.copy_stream)
            if self._h2d_timing:
                t1 = torch.cuda.Event(enable_timing=True)
                t1.record(self.copy_stream)
                self._h2d_events.append((t0, t1))
        self._pending = s
        self._slot ^= 1

    def time_h2d(self, on: bool) -> None:
        """Start (and clear) or stop the device timing of the staging copies that `feed` issues."""
        self._h2d_timing = bool(on) and self.is_cuda
        if on:
            self._h2d_events = []

    def h2d_ms(self) -> Optional[float]:
        """Mean device time of one staging copy (images + labels) since `time_h2d(True)`; None without samples. The
        copy stream must have finished them (`synchronize`)."""
        if not self._h2d_events:
            return None
        return sum(a.elapsed_time(b) for a, b in self._h2d_events) / len(self._h2d_events)

    def h2d_bytes_per_step(self) -> int:
        if not self.is_cuda:
            return 0
        extra = self._stage_shapes[0].numel() * 4 if self._stage_shapes is not None else 0
        return self._stage_imgs[0].numel() + self._stage_lbls[0].numel() * 4 + extra

    # ------------------------------------------------------------------ one batch
    def _bind_inputs(self, slot):
        """Point the input and loss operators at a staging slot (device-to-device, on the compute stream)."""
        self.net.input_op.stage.copy_(self._stage_imgs[slot], non_blocking=True)
        self.net.loss_op.labels.copy_(self._stage_lbls[slot], non_blocking=True)
        if self._stage_shapes is not None:
            self.net.input_op.shapes.copy_(self._stage_shapes[slot], non_blocking=True)

    def _fwd_bwd(self, train=True, hook=None):
        with span("forward"):
            self.net.forward(train, None)
        if train:
            with span("backward"):
                self.net.backward(hook)
        if self.is_cuda:
            self.net.step_counter.add_(1)

    def _update(self):
        """Exchange + optimizer step for one iteration, in the configured order."""
        # no_grad: on CPU the flat parameter vector is an autograd leaf, and the exchanges mix it in place
        with span("update"), torch.no_grad():
            self._update_in_order()

    def _update_in_order(self):
        o, c, st, net = self.opt, self.comm, self.stepper, self.net
        lr = self.lr
        # the reference counts the iteration before it tests the interval (src/opt/sgd/new.rs:372,402): exchanges
        # happen at iterations k, 2k, ...
        communicate = c.num_workers() > 1 and ((self.iter + 1) % max(1, o.comm_interval) == 0)
        if o.sync_order == SyncOrder.SYNC_GRADS_THEN_STEP:
            if self._overlapped():
                c.fused_grads_step(st, lr)
            else:
                if communicate:
                    c.allreduce_average(net.grads)
                st.step(lr)
        elif o.sync_order == SyncOrder.STEP_THEN_SYNC_PARAMS:
            st.step(lr)
            if communicate:
                c.sync_params(net.params)
                net.refresh_shadow()
        elif o.sync_order == SyncOrder.SYNC_PARAMS_THEN_STEP:
            st.step(lr, phase=1)
            if communicate:
                c.sync_params(net.params)
            st.step(lr, phase=6)
        elif o.sync_order == SyncOrder.SYNC_PARAMS_AND_GRADS_THEN_STEP:
            if communicate:
                c.sync_params(net.params)
                c.sync_params(net.grads, repeat=True)
            st.step(lr)
        else:
            raise ValueError(o.sync_order)

    def _overlapped(self) -> bool:
        o, c = self.opt, self.comm
        return ((c.num_workers() > 1 or getattr(c, "overlap_single", False)) and hasattr(c, "on_op_backward") and
                o.sync_order == SyncOrder.SYNC_GRADS_THEN_STEP and max(1, o.comm_interval) == 1)

    def _graph_safe_update(self) -> bool:
        c = self.comm
        return c.num_workers() <= 1 or getattr(c, "graph_safe", False)

    def _run_step(self, last_of_iteration: bool):
        """Forward + backward (+ update when this batch completes a minibatch) on the compute stream."""
        key = (last_of_iteration, self.lr if last_of_iteration else 0.0)
        full = last_of_iteration and self._graph_safe_update()
        hook = None
        if last_of_iteration and self._overlapped():
            # the exchange of a gradient bucket starts from inside backward, as soon as the bucket is complete
            self.comm.prepare(self.stepper, self.lr)
            hook = self.comm.on_op_backward
        if self.use_graph:
            g = self._graphs.get(key)
            if g is None:
                # first use of this configuration runs eagerly (allocations, lazy init); the second captures
                before = K.LAUNCHES[0]
                self._fwd_bwd(hook=hook)
                if full:
                    self._update()
                self.launches_per_step = K.LAUNCHES[0] - before
                self._graphs[key] = "warm"
            else:
                if g == "warm":
                    torch.cuda.current_stream().synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
                        self._fwd_bwd(hook=hook)
                        if full:
                            self._update()
                    self._graphs[key] = g
                g.replay()
            if last_of_iteration and not full:
                self._update()
        else:
            before = K.LAUNCHES[0]
            self._fwd_bwd(hook=hook)
            if last_of_iteration:
                self._update()
            self.launches_per_step = K.LAUNCHES[0] - before

    def step(self) -> Optional[Tuple[float, int]]:
        """Run the queued batch. Returns (loss, correct) of the *previous* call on CUDA (one-step lag), of this
        call on CPU; None when nothing is available yet."""
        net = self.net
        last = ((net.t + 1) % self.accum) == 0
        if not self.is_cuda:
            self._fwd_bwd()
            if last:
                self._update()
                self.iter += 1
                self.comm.next()
            net.t += 1
            return net.read_stats()
        slot = self._pending
        cs = self.compute_stream
        with torch.cuda.stream(cs):
            cs.wait_event(self._copy_done[slot])
            self._bind_inputs(slot)
            self._consumed[slot].record(cs)
            self._run_step(last)
            # publish loss / correct through the pinned mirror, then clear the accumulators
            lo = net.loss_op
            self._stats_dev[0:1].copy_(lo.loss_sum, non_blocking=True)
            self._stats_dev[1:2].copy_(lo.correct, non_blocking=True)
            i = net.t & 1
            self._stats_host[i].copy_(self._stats_dev, non_blocking=True)
            self._stats_ready[i].record(cs)
            lo.loss_sum.zero_()
            lo.correct.zero_()
        prev = None
        if self._lag_stats is not None:
            j = self._lag_stats
            self._stats_ready[j].synchronize()
            prev = (float(self._stats_host[j][0]), int(self._stats_host[j][1]))
        self._lag_stats = net.t & 1
        if last:
            self.iter += 1
            self.comm.next()
        net.t += 1
        return prev

    def flush(self) -> Optional[Tuple[float, int]]:
        """Wait for the last launched step and return its (loss, correct)."""
        if not self.is_cuda or self._lag_stats is None:
            return None
        j = self._lag_stats
        self._stats_ready[j].synchronize()
        self._lag_stats = None
        return float(self._stats_host[j][0]), int(self._stats_host[j][1])

    def d2h_bytes_per_step(self) -> int:
        return 8 if self.is_cuda else 0

    def set_lr(self, lr: float):
        self.lr = float(lr)

    # ------------------------------------------------------------------ inference
    def eval_batch(self, images_u8, labels) -> Tuple[float, int]:
        net = self.net
        if not self.is_cuda:
            net.load_batch(images_u8, labels)
            net.read_stats()
            net.forward(False)
            return net.read_stats()
        with torch.cuda.stream(self.compute_stream):
            if self._stage_shapes is None:
                images_u8 = images_u8.to(net.device, non_blocking=True)
            net.load_batch(images_u8, labels.to(net.device, non_blocking=True).int())
            net.forward(False)
        self.compute_stream.synchronize()
        return net.read_stats()

    def synchronize(self):
        if self.is_cuda:
            self.compute_stream.synchronize()
            self.copy_stream.synchronize()
