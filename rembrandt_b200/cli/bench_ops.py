"""bench-ops: the memory-bound kernels of a training step, one by one, on the AlexNet shapes (or a smaller batch for
profiling): device time (CUDA events after warm-up, operands larger than the L2 or an L2 flush between iterations),
the bytes the operator must move by its definition, the rate that makes, and the fraction of the measured copy
bandwidth of this GPU.

    python -m rembrandt_b200.cli.bench_ops                      # every kernel, batch 128
    python -m rembrandt_b200.cli.bench_ops --only pool --batch 32    # a small case for a profiler

"Algorithmic bytes" count every tensor once in each direction it has to travel: e.g. max-pool backward reads the output
gradient, the one-byte window codes and the ReLU mask of its input and writes the input gradient; re-reads of the
output gradient by overlapping windows are not counted (they are what a cache is for).
"""
import argparse
import json

import torch

from ..ops import native_ops as K

HBM_GBS = 6464.9       # copy bandwidth measured on this pool's B200 (read + write bytes / time); --hbm-gbs overrides


def _flush_l2(buf):
    buf.add_(1)


def time_ms(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            _flush_l2(flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bf(*shape):
    return torch.randn(*shape, device="cuda").bfloat16()


def cases(batch):
    """(name, function, algorithmic bytes) for the operators of AlexNet at the given batch."""
    out = []
    n = batch
    # ---- input: 3 x 227 x 227 bytes -> space-to-depth 57 x 57 x 64 bf16
    src = torch.randint(0, 256, (n, 3, 227, 227), dtype=torch.uint8, device="cuda")
    mean = torch.full((3, 227, 227), 127.5, device="cuda")
    dst = torch.empty((n, 57, 57, 64), dtype=torch.bfloat16, device="cuda")
    out.append(("input_u8_s2d", lambda: K.input_u8(src, mean, dst, n, 3, 227, 227, 227, 227, 57, 57, 64, 4, 0, 0, 0, 0,
                                                   False, False, False, 1 / 73.9, 1 / 73.9, 0.0, None, None, 1, 0),
                src.numel() + dst.numel() * 2))
    # ---- LRN on the conv1 output (55 x 55 x 96), forward and backward
    x1, y1 = bf(n, 55, 55, 96).abs_(), torch.empty((n, 55, 55, 96), dtype=torch.bfloat16, device="cuda")
    d1, dx1 = bf(n, 55, 55, 96), torch.empty((n, 55, 55, 96), dtype=torch.bfloat16, device="cuda")
    px = n * 55 * 55
    out.append(("lrn_fwd", lambda: K.lrn_fwd(x1, y1, px, 96, 5, 1e-4, 0.75, 2.0), 2 * x1.numel() * 2))
    out.append(("lrn_bwd", lambda: K.lrn_bwd(x1, d1, dx1, x1, px, 96, 5, 1e-4, 0.75, 2.0), 3 * x1.numel() * 2))
    # ---- max pooling 3 x 3 stride 2: 55 -> 27 (96 channels), 27 -> 13 (256), 13 -> 6 (256)
    for tag, hw, c in (("pool1", 55, 96), ("pool2", 27, 256), ("pool5", 13, 256)):
        p = (hw - 3) // 2 + 1
        x, y = bf(n, hw, hw, c), torch.empty((n, p, p, c), dtype=torch.bfloat16, device="cuda")
        idx = torch.empty((n, p, p, c), dtype=torch.uint8, device="cuda")
        dy, dx = bf(n, p, p, c), torch.empty((n, hw, hw, c), dtype=torch.bfloat16, device="cuda")
        out.append((f"{tag}_fwd", (lambda x=x, y=y, idx=idx, hw=hw, c=c, p=p: K.pool_fwd(
            x, y, idx, n, hw, hw, c, p, p, 3, 2, 0, True, False)), x.numel() * 2 + y.numel() * 3))
        K.pool_fwd(x, y, idx, n, hw, hw, c, p, p, 3, 2, 0, True, False)
        out.append((f"{tag}_bwd", (lambda dy=dy, idx=idx, dx=dx, x=x, hw=hw, c=c, p=p: K.pool_bwd(
            dy, idx, None, dx, x, n, hw, hw, c, p, p, 3, 2, 0, True)), y.numel() * 3 + 2 * x.numel() * 2))
    # ---- bias-gradient column sums of the conv1 / conv2 output gradients
    for tag, rows, c in (("colsum_conv1", n * 55 * 55, 96), ("colsum_conv2", n * 27 * 27, 256)):
        d, o = bf(rows, c), torch.zeros(c, device="cuda")
        out.append((tag, (lambda d=d, o=o, rows=rows, c=c: K.colsum(d, rows, c, c, o)), d.numel() * 2))
    # ---- fully connected helpers on [batch, 4096]
    acc, yb = torch.zeros(n, 4096, device="cuda"), torch.empty((n, 4096), dtype=torch.bfloat16, device="cuda")
    bias = torch.zeros(4096, device="cuda")
    out.append(("bias_act_4096", lambda: K.bias_act(acc, n, 4096, 4096, bias, True, yb), acc.numel() * 8 + yb.numel() * 2))
    out.append(("dropout_4096", lambda: K.dropout(yb, yb, yb.numel(), 0.5, 1, 1), 2 * yb.numel() * 2))
    # ---- softmax + cross-entropy on 1000 classes
    logits = torch.zeros((n, 1024), dtype=torch.bfloat16, device="cuda")
    logits[:, :1000] = bf(n, 1000)
    labels = torch.randint(0, 1000, (n,), dtype=torch.int32, device="cuda")
    delta = torch.empty_like(logits)
    ls, cr = torch.zeros(1, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    out.append(("softmax_ce_1000", lambda: K.softmax_ce(logits, n, 1000, 1024, labels, None, 1.0 / n, delta, loss_sum=ls,
                                                        correct=cr), 2 * logits.numel() * 2))
    # ---- the optimizer sweep over AlexNet's 62.4 M parameters (26 bytes per parameter: w, g, v read; w, v, g = 0 and
    # the bf16 copy written); batch-independent
    np_ = 62_378_344 // 64 * 64
    w, g, v = (torch.zeros(np_, device="cuda") for _ in range(3))
    w16 = torch.zeros(np_, dtype=torch.bfloat16, device="cuda")
    out.append(("sgd_fused_62M", lambda: K.sgd_fused(w, g, v, w16, np_, 0.01, 0.9, 5e-4, 1.0, 1), np_ * 26))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--only", default="", help="substring of the kernel names to run")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hbm-gbs", type=float, default=HBM_GBS)
    ap.add_argument("--no-flush", action="store_true", help="do not write a 256 MB buffer between iterations")
    args = ap.parse_args(argv)
    flush = None if args.no_flush else torch.zeros(64 << 20, device="cuda")      # 256 MB > the 126 MB L2
    for name, fn, nbytes in cases(args.batch):
        if args.only and args.only not in name:
            continue
        ms = time_ms(fn, args.iters, args.warmup, flush)
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "batch": args.batch, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 2),
                          "gb_per_s": round(gbs, 1), "fraction_of_hbm_copy": round(gbs / args.hbm_gbs, 3),
                          "floor_ms": round(nbytes / args.hbm_gbs / 1e6, 4), "status": K.read_status()}), flush=True)


if __name__ == "__main__":
    main()
