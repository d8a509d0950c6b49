"""The network container: a sequential chain input -> hidden operators -> loss over flat parameter vectors.

Counterpart of the reference's ``SequentialOperatorWorker`` (src/operator/worker.rs:230-477): it assigns
every operator its offset into the flat parameter / gradient / momentum vectors, runs forward in order and
backward in reverse, derives per-operator seeds from one shared seed, and encodes / decodes parameters
and optimizer state as concatenated NdArray records in hidden-operator order.

Memory layout: three fp32 vectors (master parameters, gradients, momentum) plus, on CUDA, a bf16 copy of
the parameters that the tensor-core kernels read. Tensors that receive L2 regularisation come first
(``[0, decay_len)``), the rest (batch-norm scale / bias / running statistics) after, so the fused
optimizer needs two launches at most. Each tensor starts on a 256-byte boundary.

On a CUDA device the operators launch the hand-written kernels; on CPU the same container runs the plain
torch fp32 reference path with autograd, which is the oracle for the GPU path and what CPU-only runs use.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..utils import blob
from ..utils.rng import XorShift128Plus
from ..utils.trace import span
from . import config as C
from . import operators as O

ALIGN = 64  # elements


def _op_table():
    from . import resnet_ops as R
    return {
        C.Data3dCfg: O.DataOp,
        C.Conv2dCfg: O.Conv2dOp,
        C.ResConv2dCfg: O.ResConv2dOp,
        C.AffineCfg: O.AffineOp,
        C.Pool2dCfg: O.Pool2dOp,
        C.LrnCfg: O.LrnOp,
        C.DropoutCfg: O.DropoutOp,
        C.SoftmaxKLLossCfg: O.SoftmaxKLLossOp,
        C.MarginalizedSoftmaxIndLossCfg: O.MarginalizedSoftmaxIndLossOp,
        C.MultiSoftmaxKLLossCfg: O.MultiSoftmaxKLLossOp,
        C.PointwiseLossCfg: O.PointwiseLossOp,
        C.CategoricalObjLossCfg: O.CategoricalObjLossOp,
        C.BNormConv2dCfg: R.BNormConv2dOp,
        C.StackResConv2dCfg: R.StackResConv2dOp,
        C.ProjStackResConv2dCfg: R.ProjStackResConv2dOp,
        C.SplitCfg: O.SplitOp,
        C.JoinCfg: O.JoinOp,
    }


class Net:
    # Tests set this to run the device code path (padded bf16 buffers, kernel fronts) on CPU tensors, with the kernel
    # fronts replaced by plain-torch stand-ins; it has no other use.
    device_path_on_cpu = False

    def __init__(self, cfg: C.SequentialOperatorConfig, batch_size: int, device="cuda", seed=(0x5EED, 0xC0FFEE),
                 minibatch_size: Optional[int] = None, training: bool = True,
                 flat_allocator: Optional[Callable[[str, int, torch.dtype], torch.Tensor]] = None):
        cfg.validate()
        self.cfg = cfg
        self.batch = int(batch_size)
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda" or self.device_path_on_cpu
        self.training_capable = training
        self.minibatch_size = int(minibatch_size or batch_size)
        self.sample_weight = 1.0 / self.minibatch_size
        self.accumulate = self.minibatch_size > self.batch   # gradients of several batches are summed per iteration
        self.shared_seed = tuple(seed)
        self.data_seed = (seed[0] * 0x9E3779B97F4A7C15 + 1) & (2**63 - 1)
        self.dropout_seed = (seed[1] * 0xD1B54A32D192ED03 + 7) & (2**62 - 1)
        self.ref_generator = torch.Generator().manual_seed(seed[0] & 0x7FFFFFFF)
        self._stream_ids = 0
        self.t = 0
        self._flat_allocator = flat_allocator

        table = _op_table()
        if isinstance(cfg, C.GraphOperatorConfig):
            entries = cfg.linearize()
        else:
            named = [cfg.input_op] + list(cfg.hidden_ops) + [cfg.loss_op]
            entries = [(no.name, no.cfg, [named[i - 1].name] if i else []) for i, no in enumerate(named)]
        self.ops: List[O.Op] = []
        produced = {}            # producer key -> operator (or one arm of a split)
        for name, ocfg, ins in entries:
            cls = table.get(type(ocfg))
            if isinstance(ocfg, C.Data3dCfg) and ocfg.variable_size:
                cls = O.VarDataOp
            if cls is None:
                raise NotImplementedError(f"no operator for configuration {type(ocfg).__name__}")
            op = cls(name, ocfg)
            op.input_keys = list(ins)
            prevs = [produced[k] for k in ins]
            op.setup(self, prevs if isinstance(op, O.JoinOp) else (prevs[0] if prevs else None))
            self.ops.append(op)
            produced[name] = op
            if isinstance(op, O.SplitOp):
                for arm in op.arms:
                    produced[arm.name] = arm
        if not isinstance(self.ops[0], O.DataOp):
            raise ValueError("the first operator in execution order must be the input operator")
        self.input_op: O.DataOp = self.ops[0]
        self.hidden_ops = self.ops[1:-1]
        self.loss_op: O.SoftmaxKLLossOp = self.ops[-1]

        # ---- flat parameter layout: regularised tensors first
        segs = [s for op in self.ops for s in op.segs]
        off = 0
        for grp in (True, False):
            for s in segs:
                if s.decay == grp:
                    s.offset = off
                    off += (s.numel + ALIGN - 1) // ALIGN * ALIGN
            if grp:
                self.decay_len = off
        self.flat_len = off
        self.segs = segs

        dev = self.device
        alloc = self._alloc_flat
        self.params = alloc("params", self.flat_len, torch.float32)
        self.grads = alloc("grads", self.flat_len, torch.float32)
        self.mom = alloc("mom", self.flat_len, torch.float32)
        self.params16 = alloc("params16", self.flat_len, torch.bfloat16) if self.is_cuda else None
        self.saved_params = None
        # device-side step counter read by the dropout and input kernels (so captured graphs stay fresh)
        self.step_counter = torch.zeros(1, dtype=torch.int32, device=dev) if self.is_cuda else None
        if not self.is_cuda:
            self.params.requires_grad_(True)
            self.params.grad = self.grads
        # Small kernels that depend on nothing the main stream is about to produce (bias-gradient column sums, the
        # re-packing of filters for the data-grad) run on a side stream beside the tensor-core kernels, which leave
        # DRAM and most of the register file idle; `side` forks, `join_side` joins (both are captured into graphs).
        self._side = None
        self._side_dirty = False
        if self.device.type == "cuda":
            self._side = torch.cuda.Stream(self.device)
            self._side_fork, self._side_join = torch.cuda.Event(), torch.cuda.Event()
        if self.is_cuda:
            for op in self.ops:
                op.alloc()
        for op in self.ops:
            op.bind()
        self._cpu_loss = None
        self._cpu_stats = [0.0, 0]
        self._cpu_batch = None
        self.params_len = sum(self._ref_numel(op) for op in self.hidden_ops)
        self.init_params(self.shared_seed)

    # ------------------------------------------------------------------ memory
    def _alloc_flat(self, name, n, dtype):
        n = max(n, ALIGN)
        if self._flat_allocator is not None and self.is_cuda:
            t = self._flat_allocator(name, n, dtype)
            t.zero_()
            return t
        return torch.zeros(n, dtype=dtype, device=self.device)

    def seg_view(self, seg: O.ParamSeg, which="params"):
        buf = getattr(self, which)
        return buf[seg.offset: seg.offset + seg.numel].view(seg.shape)

    def next_stream_id(self):
        self._stream_ids += 1
        return self._stream_ids

    @staticmethod
    def _ref_numel(op):
        return sum(int(torch.as_tensor(a).numel()) for a, _ in op.encode_params()) if op.has_params else 0

    # ------------------------------------------------------------------ parameters
    def init_params(self, seed):
        """Every operator draws from its own stream derived from the shared seed, in operator order."""
        root = XorShift128Plus(int(seed[0]), int(seed[1]))
        with torch.no_grad():
            self.params.zero_()
            for op in self.hidden_ops:
                op.init_params(root.derive())
            self.grads.zero_()
            self.mom.zero_()
        self.refresh_shadow()

    def refresh_shadow(self):
        """Re-derive the bf16 compute copy from the fp32 master parameters."""
        if self.is_cuda:
            self.params16.copy_(self.params)

    def encode_params(self) -> bytes:
        recs = []
        for op in self.hidden_ops:
            recs.extend(op.encode_params())
        return blob.encode_many(recs)

    def decode_params(self, buf: bytes, offset=0) -> int:
        with torch.no_grad():
            for op in self.hidden_ops:
                n = len(op.encode_params()) if op.has_params else 0
                if n == 0:
                    continue
                recs, offset = blob.decode_records(buf, "f32", offset, count=n)
                if len(recs) != n:
                    raise blob.BlobError(f"parameter blob ends inside operator {op.name!r}")
                op.decode_params([(r[0], r[1]) for r in recs])
        self.refresh_shadow()
        return offset

    def encode_state(self) -> bytes:
        """Per operator: its parameters followed by its momentum buffers (src/worker/gossip_dist.rs:1290-1294)."""
        out = []
        for op in self.hidden_ops:
            if not op.has_params:
                continue
            out.append(blob.encode_many(op.encode_params()))
            for s in op.state_segs():
                v = self.seg_view(s, "mom").detach().float().cpu().reshape(-1)
                out.append(blob.encode_record(v.numpy(), (v.numel(), 1)))
        return b"".join(out)

    def decode_state(self, buf: bytes) -> None:
        offset = 0
        with torch.no_grad():
            for op in self.hidden_ops:
                if not op.has_params:
                    continue
                n = len(op.encode_params())
                recs, offset = blob.decode_records(buf, "f32", offset, count=n)
                op.decode_params([(r[0], r[1]) for r in recs])
                for s in op.state_segs():
                    recs, offset = blob.decode_records(buf, "f32", offset, count=1)
                    self.seg_view(s, "mom").copy_(torch.from_numpy(recs[0][0]).reshape(s.shape))
        self.refresh_shadow()

    def save_params(self):
        """Device-side snapshot (validate on the averaged model, keep training the local one)."""
        if self.saved_params is None:
            self.saved_params = torch.empty_like(self.params)
        with torch.no_grad():
            self.saved_params.copy_(self.params)

    def restore_params(self):
        with torch.no_grad():
            self.params.copy_(self.saved_params)
        self.refresh_shadow()

    def reset_grads(self):
        with torch.no_grad():
            self.grads.zero_()

    def set_grads_with_params_diff(self):
        """grads = saved_params - params (the reference's hook for parameter-difference communication)."""
        with torch.no_grad():
            self.grads.copy_(self.saved_params - self.params)

    # ------------------------------------------------------------------ side stream
    def side(self, fn):
        """Run `fn` (kernel launches) on the side stream, ordered after everything issued so far on the current one."""
        if self._side is None:
            fn()
            return
        self._side_fork.record(torch.cuda.current_stream())
        self._side.wait_event(self._side_fork)
        with torch.cuda.stream(self._side):
            fn()
        self._side_dirty = True

    def join_side(self):
        """Make the current stream wait for everything issued on the side stream."""
        if self._side is not None and self._side_dirty:
            self._side_join.record(self._side)
            torch.cuda.current_stream().wait_event(self._side_join)
            self._side_dirty = False

    # ------------------------------------------------------------------ data
    def load_batch(self, images_u8: torch.Tensor, labels: torch.Tensor, weights: Optional[torch.Tensor] = None):
        if self.is_cuda:
            self.input_op.load_batch(images_u8)
            self.loss_op.load_labels(labels)
            if weights is not None:
                self.loss_op.load_weights(weights)
        else:
            self._cpu_batch = (images_u8, labels, weights)

    # ------------------------------------------------------------------ execution
    def forward(self, train: bool = True, t: Optional[int] = None):
        if self.is_cuda:
            if t is not None:
                self.step_counter.fill_(int(t))
            for op in self.ops:
                with span(op.name):
                    op.forward(train, self.t if t is None else t)
            self.join_side()
            return None
        t = self.t if t is None else t
        images, labels, weights = self._cpu_batch
        ctx = torch.enable_grad() if train else torch.no_grad()
        with ctx:
            vals = {}
            x = images
            for op in self.ops[:-1]:
                if op.input_keys:
                    ins = [vals[k.split(":")[0]] for k in op.input_keys]
                    x = ins if isinstance(op, O.JoinOp) else ins[0]
                x = op.ref_forward(x, train, t)
                vals[op.name] = x
            x = vals[self.loss_op.input_keys[0].split(":")[0]] if self.loss_op.input_keys else x
            loss, correct, am = self.loss_op.ref_loss(x, labels, weights)
        self._cpu_loss = loss if train else None
        self._cpu_stats[0] += float(loss.detach())
        self._cpu_stats[1] += correct
        self._cpu_logits = x.detach()
        return None

    def backward(self, hook=None):
        """Backward in reverse operator order. `hook(i)` is called after operator i has produced its parameter
        gradients (the communication backends start a bucket's exchange from it)."""
        if self.is_cuda:
            for i in range(len(self.ops) - 2, 0, -1):
                with span(self.ops[i].name):
                    self.ops[i].backward()
                if hook is not None:
                    self.join_side()      # the hook hands this operator's gradients to the exchange
                    hook(i)
            self.join_side()
            return
        self._cpu_loss.backward()
        self._cpu_loss = None

    def read_stats(self, reset=True):
        """(weighted loss sum, number correct) accumulated since the last reset; one small device read."""
        if self.is_cuda:
            lo = self.loss_op
            loss = float(lo.loss_sum.item())
            correct = int(lo.correct.item())
            if reset:
                lo.loss_sum.zero_()
                lo.correct.zero_()
            return loss, correct
        loss, correct = self._cpu_stats
        if reset:
            self._cpu_stats = [0.0, 0]
        return loss, correct

    def output_categories(self) -> torch.Tensor:
        if self.is_cuda:
            return self.loss_op.argmax.clone()
        return self._cpu_logits.flatten(1).argmax(1)

    # ------------------------------------------------------------------ introspection
    def describe(self) -> str:
        lines = []
        for op in self.ops:
            h, w, c = op.out_hwc
            n = sum(s.numel for s in op.segs)
            lines.append(f"{op.name:>12s} {type(op).__name__:<22s} out {h:>3d}x{w:<3d}x{c:<5d} (cp {op.out_cp:<5d}) params {n}")
        lines.append(f"params_len {self.params_len} (internal {self.flat_len})")
        return "\n".join(lines)
