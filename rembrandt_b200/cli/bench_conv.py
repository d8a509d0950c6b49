"""bench-conv: time the implicit-GEMM convolution kernels on given or built-in shapes and report achieved
TFLOP/s (counterpart of the reference's tools/bench-cudnn.rs, which timed cuDNN on NIN / AlexNet-shaped
convolutions). Timing uses CUDA events around replays of a CUDA graph that holds `--iters` launches (what a layer
costs inside a captured step; `--eager` launches from the host instead); `--pass` selects fprop / dgrad / wgrad.

    python -m rembrandt_b200.cli.bench_conv --shape alexnet_conv2 --batch 128 --pass all
"""
import argparse
import json

import torch

from ..ops import native_ops as K
from ..utils.timing import time_fn, time_graph

SHAPES = {
    # name: (C, H, W, Kout, R, stride, pad)
    "alexnet_conv1_s2d": (48, 57, 57, 96, 3, 1, 0),
    "alexnet_conv2": (96, 27, 27, 256, 5, 1, 2),
    "alexnet_conv3": (256, 13, 13, 384, 3, 1, 1),
    "alexnet_conv4": (384, 13, 13, 384, 3, 1, 1),
    "alexnet_conv5": (384, 13, 13, 256, 3, 1, 1),
    "nin_conv1_s2d": (48, 56, 56, 96, 3, 1, 0),       # 11 x 11 stride 4 on 224 x 224 after space-to-depth by 4
    "nin_cccp1": (96, 54, 54, 96, 1, 1, 0),
    "nin_conv2": (96, 27, 27, 256, 5, 1, 2),
    "nin_cccp3": (256, 27, 27, 256, 1, 1, 0),
    "nin_conv3": (256, 13, 13, 384, 3, 1, 1),
    "nin_conv4": (384, 6, 6, 1024, 3, 1, 1),
    "nin_cccp5": (384, 13, 13, 384, 1, 1, 0),
    "nin_cccp7": (1024, 6, 6, 1024, 1, 1, 0),
    "nin_cccp8": (1024, 6, 6, 1000, 1, 1, 0),
    # the small board-game shapes the reference's tool also times (tools/bench-cudnn.rs:10-60: 8 x 8 boards at batch
    # 1024, 19 x 19 Go boards at batch 8) and the 128-channel Go layers of tools/train-gogod.rs
    "board8_conv1": (12, 8, 8, 16, 5, 1, 2),
    "board8_conv2": (16, 8, 8, 6, 3, 1, 1),
    "go19_conv1": (16, 19, 19, 16, 5, 1, 2),
    "go19_hidden": (16, 19, 19, 16, 3, 1, 1),
    "go19_res128": (128, 19, 19, 128, 3, 1, 1),
    # the residual stages of ResNet-18 / 34 (run them with --batch 32, the reference tool's batch)
    "resnet_stage1": (64, 56, 56, 64, 3, 1, 1),
    "resnet_stage2": (128, 28, 28, 128, 3, 1, 1),
    "resnet_stage3": (256, 14, 14, 256, 3, 1, 1),
    "resnet_stage4": (512, 7, 7, 512, 3, 1, 1),
}


PEAK_TFLOPS = 1658.7      # cuBLAS bf16 matmul measured on this pool's B200 (burst); fractions are "of measured"


def run(name, batch, passes, iters, warmup, tune=True, roles=False, eager=False):
    C, H, W, Ko, R, s, p = SHAPES[name]
    Cp, Kp = K.pad_channels(C), K.pad_channels(Ko)
    P, Q = (H + 2 * p - R) // s + 1, (W + 2 * p - R) // s + 1
    dev = "cuda"
    if tune:
        # what a network does when it is built: the tile plans of the two overwrite-mode passes are measured once
        K.tune_conv(batch, H, W, Cp, Ko, R, R, s, p, p, P, Q, Kp, relu=True, has_bias=True, n_valid=Ko, n_store=Kp)
        if s == 1:
            K.tune_conv(batch, P, Q, Kp, Cp, R, R, 1, R - 1 - p, R - 1 - p, H, W, Cp, has_mask=True, n_valid=C,
                        n_store=Cp)
    x = torch.randn(batch, H, W, Cp, device=dev).bfloat16()
    w = (torch.randn(Ko, R * R, Cp, device=dev) * 0.05).bfloat16()
    wt = torch.zeros(Cp, R * R, Kp, device=dev, dtype=torch.bfloat16)
    K.pack_dgrad_filters(w, wt, Ko, Kp, R * R, Cp)
    b = torch.zeros(Ko, device=dev)
    y = torch.zeros(batch, P, Q, Kp, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(batch, P, Q, Kp, device=dev).bfloat16()
    dx = torch.zeros_like(x)
    dw = torch.zeros(Ko, R * R, Cp, device=dev)
    flops = 2.0 * batch * P * Q * Ko * R * R * C
    out = {"shape": name, "batch": batch, "gflop": flops / 1e9}
    fns = {
        "fprop": lambda: K.conv_fprop_tc(x, batch, H, W, Cp, w, Ko, R, R, s, p, p, P, Q, y, Kp, bias=b, relu=True,
                                         n_valid=Ko, n_store=Kp),
        "dgrad": lambda: K.conv_fprop_tc(dy, batch, P, Q, Kp, wt, Cp, R, R, 1, R - 1 - p, R - 1 - p, H, W, dx, Cp,
                                         mask_src=x, n_valid=C, n_store=Cp),
        "wgrad": lambda: K.conv_wgrad_tc(x, batch, H, W, Cp, dy, Kp, Ko, R, R, s, p, p, P, Q, dw),
    }
    for name_, fn in fns.items():
        if passes != "all" and passes != name_:
            continue
        if name_ == "dgrad" and s != 1:
            continue
        if roles:
            fn()
            K.gemm_role_profile()      # clear: what the tuning and the first launch left
        # replayed from a CUDA graph unless asked otherwise: launched from the host, a kernel shorter than ~20 us is
        # timed at the host's pace
        ms = time_fn(fn, iters, warmup) if (eager or roles) else time_graph(fn, iters, warmup)
        out[name_ + "_plan"] = K.gemm_last_launch()
        out[name_ + "_ms"] = round(ms, 4)
        out[name_ + "_tflops"] = round(flops / ms / 1e9, 1)
        out[name_ + "_of_peak"] = round(flops / ms / 1e9 / PEAK_TFLOPS, 3)
        if roles:
            c = K.gemm_role_profile()
            if c and c[4]:
                out[name_ + "_waiting_pct"] = {"a_producer": round(100.0 * c[0] / c[4], 1),
                                               "b_producer": round(100.0 * c[1] / c[4], 1),
                                               "mma_on_operands": round(100.0 * c[2] / c[4], 1),
                                               "mma_on_epilogue": round(100.0 * c[3] / c[4], 1),
                                               # one epilogue warp: idle; fence + issue of its stores; slabs on
                                               # their way from TMEM through registers into shared memory
                                               "epilogue_idle": round(100.0 * c[5] / c[4], 1),
                                               "epilogue_store_issue": round(100.0 * c[6] / c[4], 1),
                                               "epilogue_tmem_to_smem": round(100.0 * c[7] / c[4], 1)}
    torch.cuda.synchronize()
    out["status"] = K.read_status()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--shape", default="all", choices=["all"] + sorted(SHAPES))
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--pass", dest="passes", default="all", choices=["all", "fprop", "dgrad", "wgrad"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-tune", action="store_true", help="take the cost model's tile plans instead of measured ones")
    ap.add_argument("--eager", action="store_true", help="launch from the host instead of replaying a captured graph")
    ap.add_argument("--roles", action="store_true",
                    help="also print the share of a CTA's run that each role spends waiting (needs the library built "
                         "with `python -m rembrandt_b200._build --profile`)")
    args = ap.parse_args(argv)
    names = sorted(SHAPES) if args.shape == "all" else [args.shape]
    for n in names:
        print(json.dumps(run(n, args.batch, args.passes, args.iters, args.warmup, tune=not args.no_tune,
                             roles=args.roles, eager=args.eager)))


if __name__ == "__main__":
    main()
