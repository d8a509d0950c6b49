"""bench-link: what SM-issued traffic gets out of one NVLink direction, as a function of how much each thread
keeps in flight. Rank r reads from / writes to the symmetric buffer of rank (r+1) % N; all ranks run at once, so
every GPU serves one reader (or absorbs one writer) while it drives its own traffic.

    python -m torch.distributed.run --nproc-per-node 2 -m rembrandt_b200.cli.bench_link --mb 256

Prints one JSON line per (mode, blocks, threads, unroll): GB/s per direction per GPU, device-timed, max over ranks.
The fused collectives size their grids and per-thread unrolling from these numbers.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ..parallel import p2p
from ..parallel import p2p_kernels as PK
from .._native import check


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--mb", type=float, default=256)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--blocks", type=int, nargs="*", default=[148, 296, 592])
    ap.add_argument("--threads", type=int, nargs="*", default=[128, 512])
    ap.add_argument("--unroll", type=int, nargs="*", default=[1, 4, 16])
    ap.add_argument("--modes", nargs="*", default=["read", "write", "copy_out", "copy_in", "local"])
    args = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    arena = p2p.SymmetricArena()
    n = int(args.mb * (1 << 20) / 4) // 4096 * 4096
    sym = arena.alloc("probe", n, torch.float32)
    loc = torch.zeros(n, device="cuda")
    loc2 = torch.zeros(n, device="cuda")
    sink = torch.zeros(4, device="cuda")
    peer = arena.ptrs("probe")[(rank + 1) % world]
    st = torch.cuda.current_stream().cuda_stream
    fn = PK.fn("rb_link_probe")
    # (src, dst, kernel mode)
    table = {"read": (peer, loc.data_ptr(), 0), "write": (loc.data_ptr(), peer, 1),
             "copy_out": (loc.data_ptr(), peer, 2), "copy_in": (peer, loc.data_ptr(), 2),
             "local": (loc.data_ptr(), loc2.data_ptr(), 2)}
    for mode in args.modes:
        src, dst, km = table[mode]
        for th in args.threads:
            for bl in args.blocks:
                for un in args.unroll:
                    def run():
                        check(fn(src, dst, sink.data_ptr(), n, km, un, bl, th, st), "rb_link_probe")
                    run()
                    torch.cuda.synchronize()
                    dist.barrier()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(args.iters):
                        run()
                    e1.record()
                    torch.cuda.synchronize()
                    t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ms = float(t.item())
                    if rank == 0:
                        print(json.dumps({"mode": mode, "n_gpus": world, "mb": args.mb, "blocks": bl, "threads": th,
                                          "unroll": un, "ms": round(ms, 4),
                                          "gbs": round(n * 4 / ms / 1e6, 1),
                                          "bytes_in_flight_mb": round(bl * th * un * 16 / 1e6, 2)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
