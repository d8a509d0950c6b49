"""Public entry points a user of the framework starts from.

``build_replica`` assembles one data-parallel replica (network + optimizer + communication backend + step
engine) for a named model; ``build_net`` gives just the network. With more than one rank
(``torch.distributed`` initialised, one process per GPU) the replica joins the default process group.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .engine import StepEngine
from .models import zoo
from .models.config import Preproc
from .models.net import Net
from .optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule, SyncOrder
from .parallel import comm as comm_mod

# uniform bytes have mean 127.5 and standard deviation 73.9: this maps them to zero mean / unit variance
SYNTH_MEAN, SYNTH_STD = 127.5, 73.9

_MODEL_FN = {"alexnet": zoo.alexnet, "nin": zoo.nin, "lenet": zoo.lenet, "cifar": zoo.cifar_krizh26}


def model_config(model: str, synthetic_norm: bool = True, **kw):
    """Template configuration by name; with `synthetic_norm` the input operator standardises uniform bytes."""
    if model not in _MODEL_FN and model not in zoo.TEMPLATES:
        raise ValueError(f"unknown model {model!r}")
    fn = _MODEL_FN.get(model) or zoo.TEMPLATES[model]
    if model == "cifar":
        kw.setdefault("augment", True)
    cfg = fn(**kw)
    if synthetic_norm:
        d = cfg.input_op.cfg
        w, h, c = d.in_dims
        d.scale = 1.0 / SYNTH_STD
        d.normalize = False
        if not any(p.kind == "subtract_mean" for p in d.preprocs):
            d.preprocs.insert(0, Preproc("subtract_mean", mean=np.full((c, h, w), SYNTH_MEAN, np.float32),
                                         normalize=True))
    return cfg


def default_opt(batch: int, comm_name: str = "null", lr: float = 0.01) -> SgdOptConfig:
    order = SyncOrder.SYNC_GRADS_THEN_STEP
    if comm_name.startswith("gossip") or comm_name.startswith("group_allreduce_gossip"):
        order = SyncOrder.STEP_THEN_SYNC_PARAMS
    elif comm_name.startswith("elastic"):
        order = SyncOrder.SYNC_PARAMS_THEN_STEP
    return SgdOptConfig(minibatch_size=batch, step_size=StepSizeSchedule.constant(lr), momentum=Momentum.UPDATE,
                        mu=0.9, l2_reg_coef=5e-4, sync_order=order)


def build_net(model: str, batch: int, device="cuda", seed=(0x5EED, 0xC0FFEE), **kw) -> Net:
    return Net(model_config(model, **kw), batch, device=device, seed=seed)


def build_replica(model: str, batch: int, device="cuda", comm: str = "auto", use_graph: bool = True,
                  opt: Optional[SgdOptConfig] = None, seed=(0x5EED, 0xC0FFEE), **model_kw) -> StepEngine:
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = torch.device(device)
    if world <= 1:
        # measured on AlexNet / NIN: the overlapped update is no faster than one sweep after backward (2.72 vs
        # 2.68 ms per step), so it is opt-in
        overlap = device.type == "cuda" and comm == "local_overlap"
        worker = comm_mod.LocalOverlapComm() if overlap else comm_mod.NullComm()
    else:
        name = comm
        if name == "auto":
            name = "fused_allreduce_sgd" if device.type == "cuda" else "allreduce"
        worker = comm_mod.make_comm(name)
    seed = worker.broadcast_seed(seed)
    allocator = getattr(worker, "flat_allocator", None)
    net = Net(model_config(model, **model_kw), batch, device=device, seed=seed, flat_allocator=allocator)
    opt = opt or default_opt(batch, worker.name)
    return StepEngine(net, opt, worker, use_graph=use_graph)
