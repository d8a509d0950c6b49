"""bench-straggler: what one slow rank costs the others, per exchange backend.

The reference injects stragglers with a host-side sleep on chosen ranks (its experiment configuration,
src/worker/gossip_dist.rs:1027-1031,1577-1582) to show what its asynchronous exchanges are for: with a lock-step
exchange every rank runs at the slowest rank's pace, with an asynchronous one the others keep their own. This tool
trains a network on synthetic batches with one rank sleeping `--delay-ms` before each of its steps and reports every
rank's wall-clock time per step (the sleep is on the host, so device time would not show it), for the backend as
given and, with `--both`, for its lock-step and its asynchronous form side by side.

    python -m torch.distributed.run --nproc-per-node 4 -m rembrandt_b200.cli.bench_straggler \\
        --comm gossip_push_p2p --both --delay-ms 20

`--device cpu` runs the same experiment on gloo ranks with the library backends that have both forms
(`--comm gossip_push` or `elastic`; LeNet by default there).
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from ..api import default_opt, model_config
from ..engine import StepEngine
from ..models.net import Net
from ..ops import native_ops as K
from ..parallel import comm as comm_mod
from ..parallel import p2p

SHAPES = {"alexnet": (227, 3, 1000), "nin": (224, 3, 1000), "lenet": (28, 1, 10), "cifar": (32, 3, 10)}


def run(model, batch, comm_name, synchronous, straggler, delay_ms, steps, warmup, device="cuda"):
    rank, world = dist.get_rank(), dist.get_world_size()
    on_gpu = device == "cuda"
    if on_gpu:
        kw = {} if synchronous is None else {"synchronous": bool(synchronous)}
        worker = p2p.make(comm_name, **kw)
    else:
        worker = comm_mod.make_comm(comm_name, asynchronous=not synchronous if synchronous is not None else False)
    net = Net(model_config(model), batch, device=device, seed=worker.broadcast_seed((0x5EED, 0xC0FFEE)),
              flat_allocator=getattr(worker, "flat_allocator", None))
    eng = StepEngine(net, default_opt(batch, worker.name), worker, use_graph=on_gpu)
    hw, ch, classes = SHAPES[model]
    g = torch.Generator().manual_seed(77 + rank)
    x = torch.randint(0, 256, (batch, ch, hw, hw), dtype=torch.uint8, generator=g)
    y = torch.randint(0, classes, (batch,), dtype=torch.int32, generator=g)
    if on_gpu:
        x, y = x.pin_memory(), y.pin_memory()
    with torch.no_grad():
        worker.first_one_way_sync(net.params)
    if on_gpu:
        net.refresh_shadow()

    def step(i):
        if rank == straggler and delay_ms > 0:
            time.sleep(delay_ms / 1e3)
        eng.feed(x, y)
        eng.step()

    for i in range(warmup):
        step(i)
    eng.flush()
    eng.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(steps):
        step(i)
    eng.flush()
    eng.synchronize()
    mine = torch.tensor([(time.perf_counter() - t0) / steps * 1e3], device=device)
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    dist.barrier()
    per_rank = [round(float(t), 3) for t in everyone]
    others = [t for r, t in enumerate(per_rank) if r != straggler or delay_ms <= 0]
    skipped = worker.skipped_exchanges() if hasattr(worker, "skipped_exchanges") else None
    out = {"model": model, "batch": batch, "ranks": world, "device": device, "comm": worker.name,
           "synchronous": getattr(worker, "synchronous", None), "straggler_rank": straggler if delay_ms > 0 else None,
           "delay_ms": delay_ms, "steps": steps, "ms_per_step_by_rank": per_rank,
           "ms_per_step_of_the_other_ranks": round(sum(others) / len(others), 3),
           "device_status": K.read_status() if on_gpu else 0}
    if skipped is not None:
        out["skipped_exchanges_on_this_rank"] = skipped
    worker.close()
    del eng, net, worker
    if on_gpu:
        torch.cuda.empty_cache()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--model", default=None, choices=sorted(SHAPES), help="default: nin on GPUs, lenet on CPU ranks")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--comm", default=None,
                    help="GPUs: gossip_push_p2p (default) | elastic_p2p | gossip_pull_p2p | gossip_p2p | "
                         "fused_allreduce_sgd; CPU ranks: gossip_push (default) | elastic")
    ap.add_argument("--synchronous", type=int, default=-1, help="1 / 0 for backends that have both forms; -1 = default")
    ap.add_argument("--both", action="store_true", help="run the lock-step and the asynchronous form, with and without delay")
    ap.add_argument("--straggler-rank", type=int, default=1)
    ap.add_argument("--delay-ms", type=float, default=20.0)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.device == "cuda":
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    args.model = args.model or ("nin" if args.device == "cuda" else "lenet")
    args.comm = args.comm or ("gossip_push_p2p" if args.device == "cuda" else "gossip_push")
    forms = [True, False] if args.both else [None if args.synchronous < 0 else bool(args.synchronous)]
    delays = [0.0, args.delay_ms] if args.both else [args.delay_ms]
    for sync in forms:
        for delay in delays:
            row = run(args.model, args.batch, args.comm, sync, args.straggler_rank, delay, args.steps, args.warmup,
                      args.device)
            if dist.get_rank() == 0:
                print(json.dumps(row), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
