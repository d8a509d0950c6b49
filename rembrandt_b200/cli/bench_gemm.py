"""bench-gemm: time the tcgen05 GEMM on the three affine-layer forms (forward, data-grad, weight-grad) and report
TFLOP/s and GB/s (counterpart of the reference's tools/bench-cublas.rs, which printed sgemm Gflop/s), and with
`--sparse` the matrix x sparse-vector product that tool also times (19 x 19 board layers whose input is mostly zeros:
tools/bench-cublas.rs:40-64 lists the shapes).

    python -m rembrandt_b200.cli.bench_gemm --batch 128 --inp 9216 --out 4096
    python -m rembrandt_b200.cli.bench_gemm --sparse
"""
import argparse
import json

import torch

from ..ops import native_ops as K
from ..utils.timing import time_fn


def run(batch, inp, out, iters, warmup):
    dev = "cuda"
    outp = K.pad_channels(out)
    x = torch.randn(batch, inp, device=dev).bfloat16()
    w = (torch.randn(out, inp, device=dev) * 0.02).bfloat16()
    dy = torch.zeros(batch, outp, device=dev, dtype=torch.bfloat16)
    dy[:, :out] = torch.randn(batch, out, device=dev).bfloat16()
    ws = torch.zeros(batch, outp, device=dev)
    ws_in = torch.zeros(batch, inp, device=dev)
    gw = torch.zeros(out, inp, device=dev)
    flops = 2.0 * batch * inp * out
    res = {"batch": batch, "in": inp, "out": out}

    def cap(n_cols):
        bn = (n_cols + 147) // 148
        return max(64, min(256, (bn + 63) // 64 * 64))

    fns = {
        "fwd": lambda: K.gemm_tc(x, 0, inp, w, 0, inp, batch, out, inp, ws, outp, epi=K.EPI_F32_ATOMIC, n_store=outp,
                                 split_k=0, bn_cap=cap(out)),
        "dgrad": lambda: K.gemm_tc(dy, 0, outp, w, 1, inp, batch, inp, out, ws_in, inp, epi=K.EPI_F32_ATOMIC,
                                   n_store=inp, split_k=0, bn_cap=cap(inp)),
        "wgrad_add": lambda: K.gemm_tc(dy, 1, outp, x, 1, inp, out, inp, batch, gw, inp, epi=K.EPI_F32_ATOMIC,
                                       n_store=inp, split_k=1),
        "wgrad_store": lambda: K.gemm_tc(dy, 1, outp, x, 1, inp, out, inp, batch, gw, inp, epi=K.EPI_F32_STORE,
                                         n_store=inp, split_k=1),
    }
    for name, fn in fns.items():
        ms = time_fn(fn, iters, warmup)
        res[name + "_ms"] = round(ms, 4)
        res[name + "_tflops"] = round(flops / ms / 1e9, 1)
    res["weight_mb"] = round(inp * out * 2 / 1e6, 1)
    torch.cuda.synchronize()
    res["status"] = K.read_status()
    return res


# (n outputs, k inputs, non-zeros): shallow second layer, first, middle and last layer of the reference's tool
SPARSE_SHAPES = {"shallow_second": (361, 361 * 16, 361 * 4), "first": (2000, 361, 10), "middle": (361, 20000, 2000),
                 "last": (361, 2000, 400)}


def run_sparse(name, iters, warmup):
    n, k, nnz = SPARSE_SHAPES[name]
    dev = "cuda"
    w = torch.randn(k, n, device=dev)                  # [k][n]: the weights of an input entry are contiguous
    wn = w.t().contiguous()                            # [n][k]
    ind = torch.randperm(k, device=dev)[:nnz].int()
    val = torch.randn(nnz, device=dev)
    x = torch.zeros(k, device=dev)
    x[ind.long()] = val
    y = torch.zeros(n, device=dev)
    res = {"shape": name, "n": n, "k": k, "nnz": nnz, "flop": 2 * n * nnz}
    for tag, fn in (("sparse_kn", lambda: K.gemv_sparse(w, n, k, True, val, ind, nnz, y)),
                    ("sparse_nk", lambda: K.gemv_sparse(wn, n, k, False, val, ind, nnz, y)),
                    ("dense_torch", lambda: torch.mv(wn, x, out=y))):
        ms = time_fn(fn, iters, warmup)
        res[tag + "_us"] = round(ms * 1e3, 2)
        res[tag + "_gflops"] = round(2.0 * n * nnz / ms / 1e6, 1)
    res["status"] = K.read_status()
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--inp", type=int, default=9216)
    ap.add_argument("--out", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--sparse", action="store_true", help="time the matrix x sparse-vector product instead")
    args = ap.parse_args(argv)
    if args.sparse:
        for name in SPARSE_SHAPES:
            print(json.dumps(run_sparse(name, args.iters, args.warmup)))
        return
    print(json.dumps(run(args.batch, args.inp, args.out, args.iters, args.warmup)))


if __name__ == "__main__":
    main()
