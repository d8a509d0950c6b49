"""Shared driver of the training entry points.

The reference's tools hard-code their configuration in ``main()`` (no argument parsing anywhere); the entry
points here keep those values as defaults and expose them as flags. Multi-GPU runs are launched with
``python -m torch.distributed.run --nproc-per-node N -m rembrandt_b200.cli.<tool> ...`` (one rank per GPU).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from ..data import (AsyncPoolDataIter, AsyncQueueDataIter, BatchIter, RaggedBatchIter, RandomIndexIter, CyclicSampleDataIter, RandomSampleDataIter, SyntheticDataSource,
                    open_data_file, open_split, partition_shard)
from ..engine import StepEngine
from ..models.net import Net
from ..optim.sgd import (CheckpointBehavior, InitBehavior, Momentum, SgdOptConfig, StepSizeReference, StepSizeSchedule,
                         SyncOrder)
from ..parallel import comm as comm_mod
from ..trainer import ExperimentConfig, SgdOpt

MOMENTA = {"zero": Momentum.ZERO, "update": Momentum.UPDATE, "nesterov": Momentum.UPDATE_NESTEROV,
           "gradient": Momentum.GRADIENT, "gradient_nesterov": Momentum.GRADIENT_NESTEROV,
           "grad_decay": Momentum.GRAD_DECAY}
ORDERS = {o.value: o for o in SyncOrder}


def base_parser(desc, **defaults):
    ap = argparse.ArgumentParser(description=desc)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--batch", type=int, default=defaults.get("batch", 64))
    ap.add_argument("--minibatch", type=int, default=defaults.get("minibatch", 0), help="0 = batch")
    ap.add_argument("--lr", type=float, default=defaults.get("lr", 0.01))
    ap.add_argument("--momentum", choices=sorted(MOMENTA), default=defaults.get("momentum", "nesterov"))
    ap.add_argument("--mu", type=float, default=defaults.get("mu", 0.9))
    ap.add_argument("--l2", type=float, default=defaults.get("l2", 5e-4))
    ap.add_argument("--iters", type=int, default=defaults.get("iters", 200))
    ap.add_argument("--display-iters", type=int, default=defaults.get("display_iters", 50))
    ap.add_argument("--checkpoint-iters", type=int, default=defaults.get("checkpoint_iters", 0))
    ap.add_argument("--save-iters", type=int, default=0)
    ap.add_argument("--valid-iters", type=int, default=defaults.get("valid_iters", 0))
    ap.add_argument("--checkpoint-dir", default=None,
                    help="checkpoints and traces go here; a run started in a directory that holds a checkpoint resumes")
    ap.add_argument("--resume-from", type=int, default=None, metavar="T",
                    help="start from the parameter file of iteration T in --checkpoint-dir instead of the latest state")
    ap.add_argument("--keep-averaged", action="store_true",
                    help="continue from the averaged model after a checkpoint (default: every rank keeps its own)")
    ap.add_argument("--comm", default=defaults.get("comm", "auto"),
                    help="exchange backend: auto (fused_allreduce_sgd on GPUs, allreduce on CPU ranks) | kernel backends "
                         "fused_allreduce_sgd, gossip_p2p, gossip_pull_p2p, gossip_push_p2p, group_allreduce_gossip_p2p, "
                         "elastic_p2p | library backends allreduce, gossip_pair, gossip_pull, gossip_push, "
                         "group_allreduce_gossip, elastic, and on CPU ranks their asynchronous forms gossip_push_async, "
                         "elastic_async | null")
    ap.add_argument("--sync-order", choices=sorted(ORDERS), default=None)
    ap.add_argument("--comm-interval", type=int, default=1)
    ap.add_argument("--step-ref", choices=["local", "checkpoint"], default="local",
                    help="checkpoint: the step size is re-evaluated only at checkpoints")
    ap.add_argument("--data", default=None, help=".data descriptor; synthetic data when absent")
    ap.add_argument("--synthetic-size", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--native-loader", type=int, default=-1, metavar="THREADS",
                    help="assemble training batches with this many C++ prefetch threads (shuffled epochs over the "
                         "rank's shard, pinned ring buffers) instead of the Python iterators; 0 = Python iterators; "
                         "default: 2 threads for sources that map to arrays (MNIST, CIFAR-10 files), else Python")
    ap.add_argument("--decode-threads", type=int, default=1,
                    help="decode samples (JPEG records, database cursors) on this many Python threads, order preserved")
    ap.add_argument("--straggler-ranks", type=int, nargs="*", default=[])
    ap.add_argument("--straggler-max-delay-ms", type=int, default=0)
    ap.add_argument("--report-port", type=int, default=0, help="serve a live loss report on this port")
    add_rendezvous_args(ap)
    return ap


def add_rendezvous_args(ap):
    ap.add_argument("--rendezvous-dir", default=os.environ.get("RB_RENDEZVOUS_DIR"),
                    help="meet the other ranks through a file in this shared directory instead of a launcher's "
                         "environment (the reference's directory-based worker, src/worker/gossip_dist_dir.rs): start "
                         "every rank by hand with --rank R --world-size N")
    ap.add_argument("--rank", type=int, default=None)
    ap.add_argument("--world-size", type=int, default=None)


def init_distributed(device: str, args=None):
    """Join the process group. Under `torch.distributed.run` the launcher's environment says who we are; with
    `--rendezvous-dir` the ranks are started by hand and meet through a file in a directory that all of them see."""
    shared = getattr(args, "rendezvous_dir", None)
    if shared and getattr(args, "world_size", None):
        os.environ["WORLD_SIZE"] = str(args.world_size)
        os.environ["RANK"] = str(args.rank or 0)
        if "LOCAL_RANK" not in os.environ:
            per_node = torch.cuda.device_count() if device == "cuda" else 0
            os.environ["LOCAL_RANK"] = str((args.rank or 0) % per_node if per_node else 0)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        how = {}
        if shared:
            os.makedirs(shared, exist_ok=True)
            how = {"init_method": "file://" + os.path.join(os.path.abspath(shared), "rendezvous"),
                   "rank": int(os.environ["RANK"]), "world_size": world}
        if device == "cuda":
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            if os.environ.get("RB_NUMA_BIND", "1") == "1":
                # host threads (loader, pinned staging memory) stay on the NUMA node of this rank's GPU
                from ..utils.numa import bind_to_gpu_node
                bind_to_gpu_node(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local), **how)
        else:
            dist.init_process_group("gloo", **how)
    rank = dist.get_rank() if dist.is_initialized() else 0
    return rank, world


def make_comm(name, device, world):
    if world <= 1:
        return comm_mod.NullComm()
    if name == "auto":
        name = "fused_allreduce_sgd" if device == "cuda" else "allreduce"
    return comm_mod.make_comm(name)


def default_order(comm_name):
    if "gossip" in comm_name:
        return SyncOrder.STEP_THEN_SYNC_PARAMS
    if "elastic" in comm_name:
        return SyncOrder.SYNC_PARAMS_THEN_STEP
    return SyncOrder.SYNC_GRADS_THEN_STEP


def run_training(args, model_cfg, schedule: StepSizeSchedule = None, source=None, valid_source=None):
    rank, world = init_distributed(args.device, args)
    device = torch.device(args.device, int(os.environ.get("LOCAL_RANK", "0")) if args.device == "cuda" else None) \
        if args.device == "cuda" else torch.device("cpu")
    worker = make_comm(args.comm, args.device, world)
    seed = worker.broadcast_seed((args.seed, args.seed * 7919 + 13))
    dims = model_cfg.input_op.cfg.in_dims
    classes = model_cfg.loss_op.cfg.num_categories
    if source is None:
        source = (open_data_file(args.data, "train") if args.data else
                  SyntheticDataSource(args.synthetic_size, dims, classes, seed=args.seed, separable=True))
    if valid_source is None and args.valid_iters:
        if args.data:
            from ..data.datasets import load_data
            splits = load_data(args.data)
            held_out = next((s for s in ("valid", "test") if s in splits), None)
            valid_source = open_split(splits[held_out]) if held_out else None
        else:
            valid_source = SyntheticDataSource(max(256, args.synthetic_size // 8), dims, classes, seed=args.seed + 1,
                                               separable=True)
    # a `source = "synthetic"` split of a .data file has no shape of its own: give it the model's
    def fit(src, seed_):
        if isinstance(src, SyntheticDataSource) and (tuple(src.dims) != tuple(dims) or src.num_classes != classes):
            return SyntheticDataSource(len(src), dims, classes, seed=seed_, separable=True)
        return src
    source, valid_source = fit(source, args.seed), fit(valid_source, args.seed + 1)
    minibatch = args.minibatch or args.batch
    opt = SgdOptConfig(minibatch_size=minibatch, step_size=schedule or StepSizeSchedule.constant(args.lr),
                       momentum=MOMENTA[args.momentum], mu=args.mu, l2_reg_coef=args.l2,
                       sync_order=ORDERS[args.sync_order] if args.sync_order else default_order(worker.name),
                       comm_interval=args.comm_interval, step_ref=StepSizeReference(args.step_ref),
                       checkpoint=CheckpointBehavior.KEEP if args.keep_averaged else CheckpointBehavior.DISCARD,
                       init=InitBehavior.RESUME_FROM if args.resume_from is not None else InitBehavior.INIT_OR_RESUME,
                       resume_t=args.resume_from or 0,
                       display_iters=args.display_iters, checkpoint_iters=args.checkpoint_iters,
                       save_iters=args.save_iters or args.checkpoint_iters, valid_iters=args.valid_iters,
                       checkpoint_dir=args.checkpoint_dir, max_iters=args.iters)
    net = Net(model_cfg, args.batch, device=device, seed=seed, minibatch_size=minibatch,
              flat_allocator=getattr(worker, "flat_allocator", None))
    if rank == 0:
        print(net.describe())
    engine = StepEngine(net, opt, worker, use_graph=not args.no_graph)
    ragged = bool(getattr(model_cfg.input_op.cfg, "variable_size", False))    # images of different sizes
    if args.native_loader < 0:      # the Python chain assembles ~18 000 samples/s whatever their size: too slow for one GPU
        args.native_loader = 2 if hasattr(source, "as_arrays") and not ragged else 0
    if args.native_loader > 0 and not ragged:
        from ..data.datasets import source_arrays
        from ..data.native_loader import NativeBatchLoader
        from ..utils.rng import partition_range
        shard = partition_range(len(source), world, rank)
        w, h, c = dims
        train_iter = None
        if getattr(source, "lmdb_path", None):
            try:   # raw image records: pixels go from the memory-mapped database to the pinned slots in C++
                train_iter = NativeBatchLoader.from_caffe_lmdb(source.lmdb_path, (c, h, w), args.batch, mode="shuffled",
                                                               seed=args.seed + rank, threads=args.native_loader,
                                                               shard=shard)
            except RuntimeError:
                train_iter = None          # encoded (JPEG) records need the Python decoder
        if train_iter is None:
            imgs, lbls = source_arrays(source)
            train_iter = NativeBatchLoader(imgs, lbls, args.batch, mode="shuffled", seed=args.seed + rank,
                                           threads=args.native_loader, shard=shard)
    else:
        shard = partition_shard(source, rank, world)
        if args.decode_threads > 1:    # e.g. JPEG records: the decoder releases the interpreter lock, so threads scale
            samples = AsyncPoolDataIter(RandomIndexIter(len(shard), seed=(args.seed + rank, 99)), shard.__getitem__,
                                        num_workers=args.decode_threads)
        else:
            samples = AsyncQueueDataIter(RandomSampleDataIter(shard, seed=(args.seed + rank, 99)))
        if ragged:
            train_iter = RaggedBatchIter(samples, args.batch, model_cfg.input_op.cfg.max_dims or dims)
        else:
            train_iter = BatchIter(samples, args.batch, dims)
    valid_iter = None
    if valid_source is not None:
        vs = CyclicSampleDataIter(partition_shard(valid_source, rank, world))
        valid_iter = (RaggedBatchIter(vs, args.batch, model_cfg.input_op.cfg.max_dims or dims) if ragged else
                      BatchIter(vs, args.batch, dims))
    report = None
    if args.report_port and rank == 0:
        from ..utils.report import ReportServer
        report = ReportServer(port=args.report_port)
    sgd = SgdOpt(opt, engine, ExperimentConfig(args.straggler_ranks, args.straggler_max_delay_ms), report=report)
    sgd.train(_repeat(train_iter), valid_iter, max_iters=args.iters)
    if valid_iter is not None and args.valid_iters:
        sgd.validate(valid_iter, args.valid_iters, engine.iter)
    worker.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return sgd


def _repeat(it):
    while True:
        for x in it:
            yield x
