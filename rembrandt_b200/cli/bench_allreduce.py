"""bench-allreduce: the fused all-reduce + 1/N + SGD kernel alone, per bucket size, against NCCL all-reduce followed
by the separate fused-SGD kernel. Device-timed (CUDA events), max over ranks; reports bus bandwidth
(S/t * 2(N-1)/N, the usual all-reduce convention) and the fraction of the NVLink roofline.

    python -m torch.distributed.run --nproc-per-node 8 -m rembrandt_b200.cli.bench_allreduce --sizes-mb 1 4 16 25 64 256

Roofline of the fused exchange (two-shot, sharded optimizer): every GPU sends (N-1)/N * S bytes of fp32 gradients
(its contribution to the other ranks' shards) and (N-1)/N * S/2 bytes of new bf16 weights (its shard, to every
peer), and receives as much; both travel in the same direction of its links, so the bound is
1.5 * (N-1)/N * S / link_bandwidth with the measured 770 GB/s per direction (multimem.st broadcasts the weights
through the switch and shrinks the outbound weight term to S/2N). The plain all-reduce (op 1) moves fp32 both ways:
2 * (N-1)/N * S / link_bandwidth.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import native_ops as K
from ..parallel import p2p

LINK_GBS = 770.0


def timed(fn, iters, warmup, stream=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class _FakeNet:
    """Just the flat vectors the communication backend touches."""

    def __init__(self, n, comm):
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.flat_len = n
        self.decay_len = n
        self.grads = comm.flat_allocator("grads", n, torch.float32)
        self.params16 = comm.flat_allocator("params16", n, torch.bfloat16)
        self.params = torch.zeros(n, device=dev)
        self.mom = torch.zeros(n, device=dev)
        self.ops = []


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--sizes-mb", type=float, nargs="*", default=[1, 4, 16, 25, 64, 256])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=148)
    ap.add_argument("--multimem", type=int, default=-1, help="1/0 force; -1 = RB_MULTIMEM")
    ap.add_argument("--bucket-mb", type=float, default=32,
                    help="also time each size cut into buckets of this size alternating over two streams, as in training")
    args = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    max_n = int(max(args.sizes_mb) * (1 << 20) / 4) // 512 * 512
    mm = None if args.multimem < 0 else bool(args.multimem)
    comm = p2p.FusedAllreduceSgdComm(bucket_bytes=1 << 40, blocks=args.blocks, use_multimem=mm)
    net = _FakeNet(max_n, comm)
    comm.net = net
    comm.comm_stream = torch.cuda.current_stream()
    comm._ready, comm._done = torch.cuda.Event(), torch.cuda.Event()
    comm.mc_grads = comm.arena.multicast_ptr("grads") if comm.use_multimem else 0
    comm.mc_w16 = comm.arena.multicast_ptr("params16") if comm.use_multimem else 0
    bn = int(args.bucket_mb * (1 << 20) / 4) // 512 * 512
    # slot 0: the whole vector as one bucket; slots 1..: the same range cut into buckets of --bucket-mb
    comm.launches = [(0, 0, max_n, 0)] + [(0, o, min(bn, max_n - o), 1 + i) for i, o in enumerate(range(0, max_n, bn))]
    comm.one_shot_elems = 0
    comm.setup_stage(avg_elems=max_n)
    side = [torch.cuda.Stream(priority=-1), torch.cuda.Stream(priority=-1)]
    ev_ready, ev_done = torch.cuda.Event(), [torch.cuda.Event(), torch.cuda.Event()]
    comm._avg_cap = max_n
    comm._hyper = (0.01, 0.9, 5e-4, 1.0 / world, 1)
    net.grads.normal_()
    rows = []
    for mb in args.sizes_mb:
        n = int(mb * (1 << 20) / 4) // 512 * 512
        fused = lambda: comm._launch(0, n, 0, op=0)
        t_fused = timed(fused, args.iters, args.warmup)
        plain = lambda: comm._launch(0, n, comm.num_slots - 1, op=1)
        t_plain = timed(plain, args.iters, args.warmup)

        def bucketed():
            cur = torch.cuda.current_stream()
            ev_ready.record(cur)
            comm.comm_streams = side
            for st in side:
                st.wait_event(ev_ready)
            for _, o, m, slot in comm.launches[1:]:
                if o < n:
                    comm._launch(o, min(m, n - o), slot, op=0)
            for st, ev in zip(side, ev_done):
                ev.record(st)
                cur.wait_event(ev)
            comm.comm_streams = None
        t_bucketed = timed(bucketed, args.iters, args.warmup) if n > bn else None

        def nccl():
            dist.all_reduce(net.grads[:n])
            K.sgd_fused(net.params[:n], net.grads[:n], net.mom[:n], net.params16[:n], n, 0.01, 0.9, 5e-4, 1.0 / world, 1)
        t_nccl = timed(nccl, args.iters, args.warmup)
        s = n * 4.0
        busbw = lambda ms: s / (ms * 1e-3) * 2 * (world - 1) / world / 1e9
        bound_ms = 1.5 * (world - 1) / world * s / (LINK_GBS * 1e9) * 1e3
        rows.append({"bucket_mb": mb, "n_gpus": world, "multimem": bool(comm.mc_grads),
                     "fused_allreduce_sgd_ms": round(t_fused, 4), "fused_busbw_gbs": round(busbw(t_fused), 1),
                     "fused_fraction_of_roofline": round(bound_ms / t_fused, 3),
                     "fused_bucketed_two_streams_ms": round(t_bucketed, 4) if t_bucketed else None,
                     "bucketed_fraction_of_roofline": round(bound_ms / t_bucketed, 3) if t_bucketed else None,
                     "p2p_allreduce_only_ms": round(t_plain, 4), "p2p_allreduce_busbw_gbs": round(busbw(t_plain), 1),
                     "nccl_allreduce_plus_sgd_ms": round(t_nccl, 4), "nccl_path_busbw_gbs": round(busbw(t_nccl), 1)})
    torch.cuda.synchronize()
    status = K.read_status()
    if rank == 0:
        for r in rows:
            r["status"] = status
            print(json.dumps(r))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
