"""Helper: run a function as `world` gloo ranks on CPU (child processes, file rendezvous, time limit)."""
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, init_file, fn, args, timeout_s, errors):
    try:
        import datetime
        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
        torch.manual_seed(1000 + rank)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:
        errors.put((rank, traceback.format_exc()))
        raise


def run_ranks(world, fn, *args, timeout_s=60, expect_failure=False):
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rdzv")
        procs = [ctx.Process(target=_entry, args=(r, world, init_file, fn, args, timeout_s, errors))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout_s + 30)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:
            p.kill()
        msgs = []
        while not errors.empty():
            msgs.append(errors.get())
        codes = [p.exitcode for p in procs]
    if expect_failure:
        return codes, msgs
    assert not hung, "ranks did not finish in time"
    assert all(c == 0 for c in codes), "\n".join(f"rank {r}:\n{m}" for r, m in msgs)
    return codes, msgs
