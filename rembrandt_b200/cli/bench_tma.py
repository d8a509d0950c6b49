"""bench-tma: fill-only TMA probes (csrc/tma_probe.cu): what the TMA path delivers into shared memory with no MMA
behind it, per SM and in aggregate. One JSON line per configuration, CUDA-event timed.

    python -m rembrandt_b200.cli.bench_tma                 # both sweeps
    python -m rembrandt_b200.cli.bench_tma --only tiled    # tiled 2-D boxes: box size, row pitch, issuing threads
    python -m rembrandt_b200.cli.bench_tma --only stage    # one conv2-forward pipeline stage: im2col A + tiled B
"""
import argparse
import json

import torch

from .. import _native
from ..ops import native_ops as K
from ..ops.native_ops import check, stream_handle


def _time(fn, reps=3):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def tiled(args):
    lib = _native.cuda()
    status = K.status_word()
    src = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")          # 64 MB: resident in the L2
    cases = [  # box_rows, stages, iters, inner bytes, pitch, issuers, lanes-of-one-warp, blocks
        (64, 8, 4000, 128, 128, 1, 0, 148), (128, 2, 2000, 128, 128, 1, 0, 148), (128, 8, 2000, 128, 128, 1, 0, 148),
        (256, 4, 1000, 128, 128, 1, 0, 148), (128, 4, 2000, 128, 128, 1, 0, 1), (128, 4, 2000, 128, 128, 1, 0, 16),
        (128, 4, 2000, 128, 512, 1, 0, 148), (128, 4, 2000, 128, 4608, 1, 0, 148), (128, 4, 2000, 64, 192, 1, 0, 148),
        (256, 4, 1000, 64, 4800, 1, 0, 148), (128, 2, 2000, 128, 128, 2, 0, 148), (128, 2, 2000, 128, 128, 4, 0, 148),
        (128, 2, 2000, 128, 128, 2, 1, 148), (128, 2, 2000, 128, 128, 4, 1, 148), (128, 2, 2000, 128, 4608, 4, 0, 148),
    ]
    for box, stages, iters, inner, pitch, issuers, lanes, blocks in cases:
        rows = (64 << 20) // pitch

        def run():
            check(lib.rb_tma_probe_tiled(src.data_ptr(), rows, box, stages, iters, 0, blocks, inner, pitch, issuers, lanes,
                                         status.data_ptr(), stream_handle()), "rb_tma_probe_tiled")
        ms = _time(run)
        gb = blocks * iters * box * inner / 1e9
        print(json.dumps({"probe": "tiled", "box_rows": box, "row_bytes": inner, "row_pitch": pitch, "stages": stages,
                          "issuers": issuers, "issuers_are_lanes": bool(lanes), "blocks": blocks,
                          "ns_per_box_per_issuer": round(ms * 1e6 / (iters / issuers), 1),
                          "per_sm_gbs": round(gb / ms * 1e3 / blocks, 1), "total_gbs": round(gb / ms * 1e3, 1),
                          "status": K.read_status()}), flush=True)


def stage(args):
    lib = _native.cuda()
    status = K.status_word()
    for C, bk, stages in ((96, 32, 6), (128, 64, 2)):
        x = torch.zeros(128 * 27 * 27 * C, dtype=torch.bfloat16, device="cuda")
        w = torch.zeros(256 * 25 * C, dtype=torch.bfloat16, device="cuda")
        for do_a, do_b, lanes, blocks in ((1, 1, 2, 148), (1, 0, 2, 148), (0, 1, 2, 148), (1, 0, 1, 148), (1, 0, 4, 148),
                                          (1, 0, 8, 148), (1, 1, 2, 8)):
            iters = 3000

            def run():
                check(lib.rb_tma_probe_conv_stage(x.data_ptr(), w.data_ptr(), C, bk, stages, iters, do_a, do_b, lanes,
                                                  blocks, status.data_ptr(), stream_handle()), "rb_tma_probe_conv_stage")
            ms = _time(run)
            print(json.dumps({"probe": "conv_stage", "channels": C, "bk": bk, "stages": stages, "im2col_A": bool(do_a),
                              "tiled_B": bool(do_b), "a_issuing_lanes": lanes, "blocks": blocks,
                              "ns_per_stage": round(ms * 1e6 / iters, 1), "status": K.read_status()}), flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", choices=["tiled", "stage"], default=None)
    args = ap.parse_args(argv)
    if args.only in (None, "tiled"):
        tiled(args)
    if args.only in (None, "stage"):
        stage(args)


if __name__ == "__main__":
    main()
