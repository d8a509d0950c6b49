"""test-dist: rendezvous smoke test, the counterpart of the reference's test-mpich / test-openmpi (tools/test-openmpi.rs
initialises MPI and prints rank and size). Every rank joins the process group, all-reduces its rank and prints what it
sees; exit status 0 means the launcher, the rendezvous and one collective work.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m rembrandt_b200.cli.test_dist
    python -m rembrandt_b200.cli.test_dist --rendezvous-dir /shared/run1 --rank R --world-size N     # one per rank, by hand
"""
import argparse

import torch
import torch.distributed as dist

from .common import add_rendezvous_args, init_distributed


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    add_rendezvous_args(ap)
    args = ap.parse_args(argv)
    rank, world = init_distributed(args.device, args)
    total = torch.tensor([float(rank)], device="cuda" if args.device == "cuda" and world > 1 else "cpu")
    if world > 1:
        dist.all_reduce(total)
    expect = world * (world - 1) / 2
    print(f"rank {rank} of {world}: sum of ranks {int(total.item())} (expected {int(expect)})", flush=True)
    ok = float(total.item()) == expect
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit(1)
    return rank, world


if __name__ == "__main__":
    main()
