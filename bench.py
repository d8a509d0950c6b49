#!/usr/bin/env python
"""Headline benchmark: training throughput (images/s) of AlexNet / NIN on synthetic ImageNet-shaped data.

    python bench.py --gpus N --steps K --warmup W [--model alexnet|nin|lenet|cifar] [--impl ours|torch_ddp|reference]

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N``
(one rank per GPU; RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* are read from the environment). Rank 0 prints one
JSON line. Two numbers are measured, both on the device with CUDA events, max over ranks:

* ``value``: K optimizer steps with the batch already staged on the device (input kernel, forward, backward,
  gradient exchange, SGD update all inside the timed region);
* ``e2e.value``: K steps through the public ``StepEngine.feed/step`` API, each with a host->device copy of a
  fresh pinned uint8 batch + labels and a device->host read of the loss (one-step lag).

The region of K steps is timed again and again until ``--min-seconds`` (2 s) of device time has been measured, so
that the figure is a sustained one under the power cap and not a 40 ms burst; ``value`` is the median region and
``timing`` gives the spread. After the framework's own arm the same process times stock PyTorch (DDP + cuDNN /
cuBLAS) in the variants of ``--baseline-variants`` and reports the fastest as ``baseline_same_lease``; with more than
one rank the line also carries ``replicas_identical`` and ``device_status``.

Weak scaling: the per-GPU batch is fixed. Data is synthetic (uniform uint8 pixels normalised to zero mean /
unit variance, uniform labels), weights are randomly initialised. The per-step working set (activations,
deltas, 250 MB of fp32 weights plus gradients and momentum) is several times the 126 MB L2, so no explicit L2
flush is needed between iterations; this is stated in ``config``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    # name: (input hw, channels, classes, per-GPU batch)
    "alexnet": (227, 3, 1000, 128),
    "nin": (224, 3, 1000, 64),
    "lenet": (28, 1, 10, 128),
    "cifar": (32, 3, 10, 128),
    # the reference's enabled ImageNet tool trains ResNet-18 at batch 32 per worker (tools/new-dist-train-imagenet.rs):
    # 256 x 256 staged images, random 224 crop + flip + lighting noise on the GPU
    "resnet18": (256, 3, 1000, 32),
}


def read_baseline(model, n):
    """Baseline images/s for (model, n GPUs): a published figure of the reference if BASELINE.json lists one, else
    the recorded torch-DDP measurement on this hardware (baseline/recorded.json)."""
    for path, key in ((os.path.join(ROOT, "BASELINE.json"), "published"),
                      (os.path.join(ROOT, "baseline", "recorded.json"), None)):
        try:
            with open(path) as f:
                tab = json.load(f)
            tab = tab.get(key, {}) if key else tab
            v = tab.get(f"{model}_images_per_s", {}).get(str(n))
            if v:
                return v
        except (OSError, ValueError, AttributeError):
            pass      # no such file, or not the JSON layout expected: try the next source
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        # an int, or a comma-separated list of local GPU indices (every GPU of a multi-rank run)
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None      # no nvidia-smi on this machine

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, per_gpu = [], [], set(), {}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                per_gpu.setdefault(parts[0], []).append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower() == "active":
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "sm_mhz_slowest_gpu": min(statistics.median(v) for v in per_gpu.values()) if per_gpu else None,
                "gpus_sampled": len(per_gpu), "samples": len(sm), "reasons": sorted(reasons)}


def timed_regions(fn, finish, steps, barrier, stream, world, dev, min_seconds, max_repeats):
    """Time `steps` calls of `fn` between device events, again and again until at least `min_seconds` of device time
    have been measured (at least one region, at most `max_repeats`). Returns the per-region times in ms (maximum
    over ranks) and whatever `finish()` returned last."""
    import torch
    import torch.distributed as dist
    times, total, last = [], 0.0, None
    while True:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
        for i in range(steps):
            fn(i)
        last = finish()
        with torch.cuda.stream(stream):
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        times.append(ms)
        total += ms
        if total >= min_seconds * 1e3 or len(times) >= max_repeats:
            return times, last


def spread(times, steps, clocks):
    """Median / min / max ms per step over the timed regions, and median ms x median SM MHz (a clock-independent
    figure for comparing runs whose clocks differed)."""
    per = sorted(t / steps for t in times)
    med = statistics.median(per)
    mhz = (clocks or {}).get("sm_mhz")
    return {"regions": len(per), "timed_seconds": round(sum(times) / 1e3, 3), "ms_per_step_median": round(med, 4),
            "ms_per_step_min": round(per[0], 4), "ms_per_step_max": round(per[-1], 4),
            "median_ms_x_sm_mhz": round(med * mhz, 1) if mhz else None}


def run_arm(args, impl, variant, world, rank, local_rank, dev, host_imgs, host_lbls, batch, sampler_ids):
    """Build one arm (this framework, or stock PyTorch in one of its variants), warm it up, and time both modes:
    batch resident on the device, and end to end through feed/step with a pinned host batch per step."""
    import torch
    import torch.distributed as dist
    pool = len(host_imgs)
    extra = {}
    if impl == "ours":
        from rembrandt_b200.api import build_replica
        from rembrandt_b200.ops import native_ops as K
        engine = build_replica(args.model, batch, device=dev, comm=args.comm, use_graph=not args.no_graph)

        def feed_step(i):
            engine.feed(host_imgs[i % pool], host_lbls[i % pool])
            return engine.step()

        def resident_step(i):
            return engine.step()

        finish, sync, stream = engine.flush, engine.synchronize, engine.compute_stream
        h2d, d2h, comm_name = engine.h2d_bytes_per_step(), engine.d2h_bytes_per_step(), engine.comm.name
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        from torch_ddp import TorchBaseline
        tb = TorchBaseline(args.model, batch, world, rank, dev, variant=variant)
        dev_imgs = [t.to(dev) for t in host_imgs[:2]]
        dev_lbls = [t.to(dev) for t in host_lbls[:2]]
        last = {}

        def feed_step(i):
            prev = last.get("loss")
            val = float(prev.item()) if prev is not None else None   # lagged read, like our engine
            last["loss"] = tb.step(host_imgs[i % pool], host_lbls[i % pool])
            return val

        def resident_step(i):
            last["loss"] = tb.step(dev_imgs[i % 2], dev_lbls[i % 2])

        def finish():
            return float(last["loss"].item())

        sync, stream = torch.cuda.synchronize, torch.cuda.current_stream()
        h2d, d2h = host_imgs[0].numel() + host_lbls[0].numel() * 4, 4
        comm_name = "nccl_ddp" if world > 1 else "none"

    def barrier():
        sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (captures the CUDA graph where there is one)
    for i in range(args.warmup):
        feed_step(i)
    finish()
    if impl == "ours":
        engine.feed(host_imgs[0], host_lbls[0])      # resident mode: the last fed batch stays staged
    for i in range(2):
        resident_step(i)
    finish()

    sampler = ClockSampler(sampler_ids)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    t_dev, last_loss = timed_regions(resident_step, finish, args.steps, barrier, stream, world, dev, args.min_seconds,
                                     args.max_repeats)
    if impl == "ours":
        engine.time_h2d(True)
    t_e2e, _ = timed_regions(feed_step, finish, args.steps, barrier, stream, world, dev, args.min_seconds,
                             args.max_repeats)
    clocks = sampler.stop() if rank == 0 else None
    if impl == "ours":
        # device time of one staging copy, slowest rank: what the host side of the end-to-end path costs per step
        engine.time_h2d(False)
        h2d_ms = torch.tensor([engine.h2d_ms() or 0.0], device=dev)
        if world > 1:
            dist.all_reduce(h2d_ms, op=dist.ReduceOp.MAX)
        extra["h2d_copy_ms_slowest_rank"] = round(float(h2d_ms), 4)
        extra["numa_node"] = args.numa_node
    if impl == "ours":
        extra["gpu_launches"] = engine.launches_per_step * args.steps
        extra["device_status"] = K.read_status()
        if world > 1:
            # replicas must hold bit-identical compute weights after the same number of exchanges
            w16 = engine.net.params16
            check = w16.view(torch.int16).to(torch.int64).sum().reshape(1)
            sums = [torch.zeros_like(check) for _ in range(world)]
            dist.all_gather(sums, check)
            extra["replicas_identical"] = bool(all(int(x) == int(sums[0]) for x in sums))
    res = {"impl": impl, "variant": variant, "comm": comm_name, "h2d": h2d, "d2h": d2h, "clocks": clocks,
           "loss": last_loss[0] if isinstance(last_loss, tuple) else last_loss, "times_dev": t_dev, "times_e2e": t_e2e}
    res.update(extra)
    if impl == "ours":
        del engine
    else:
        del tb
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--model", default="alexnet", choices=sorted(MODELS))
    ap.add_argument("--impl", default="ours", choices=["ours", "torch_ddp", "reference"])
    ap.add_argument("--comm", default="auto", help="ours: auto | fused_allreduce_sgd | allreduce | gossip_p2p | "
                    "gossip_pull_p2p | gossip_push_p2p | elastic_p2p | group_allreduce_gossip_p2p")
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the configuration's)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="repeat the timed region of K steps until this much device time has been measured")
    ap.add_argument("--max-repeats", type=int, default=400)
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="do not restrict the rank's host threads to the NUMA node of its GPU")
    ap.add_argument("--baseline-variants", default="auto",
                    help="stock-PyTorch variants timed in the same process (eager, graph, bf16_graph, compiled); the "
                         "fastest is reported. auto = graph,compiled,eager on one GPU (compiling takes about two "
                         "minutes) and graph,eager on several; none = no same-lease baseline.")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)

    if args.impl == "reference":
        # The reference is a Rust-nightly-2016 crate whose GPU runtime lives in 17 sibling crates that are not
        # in its tree; pip cannot install it and there is no Rust toolchain here.
        if int(os.environ.get("RANK", "0")) == 0:      # one line per job, also under a multi-rank launcher
            print(json.dumps({"impl": "reference", "unavailable":
                              "peterhj/rembrandt is a Rust crate (no Python packaging, cargo/rustc absent, 17 path "
                              "dependencies and cuDNN v4 missing): `pip install --target baseline/_ref` finds nothing "
                              "to build; compare against --impl torch_ddp instead"}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    # the pinned staging batches below are placed on the node of the thread that touches them first: stay on the GPU's
    args.numa_node = None
    if not args.no_numa_bind:
        from rembrandt_b200.utils.numa import bind_to_gpu_node
        args.numa_node = bind_to_gpu_node(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    hw, ch, classes, batch = MODELS[args.model]
    if args.batch:
        batch = args.batch
    dev = torch.device("cuda", local_rank)

    # ---- synthetic data: a small pool of pinned uint8 batches, cycled (each step copies a full batch H2D)
    gen = torch.Generator().manual_seed(1234 + rank)
    pool = 4
    host_imgs = [torch.randint(0, 256, (batch, ch, hw, hw), dtype=torch.uint8, generator=gen).pin_memory()
                 for _ in range(pool)]
    host_lbls = [torch.randint(0, classes, (batch,), dtype=torch.int32, generator=gen).pin_memory()
                 for _ in range(pool)]
    sampler_ids = ",".join(str(i) for i in range(world)) if world > 1 else local_rank
    if args.baseline_variants == "auto":
        # several GPUs: eager DDP only. Capturing a DDP step in a CUDA graph is fragile (the autograd engine and the
        # reducer must stay off the legacy stream), and a variant that fails on a rank ends the run for all of them;
        # `--baseline-variants graph,eager` asks for it explicitly.
        args.baseline_variants = "graph,compiled,eager" if world == 1 else "eager"
    variants = [v for v in args.baseline_variants.split(",") if v and v != "none"]

    def torch_arms():
        """Every requested stock-PyTorch variant, timed here and now; a variant that cannot be built is reported."""
        out, failed = [], {}
        for v in variants:
            try:
                out.append(run_arm(args, "torch_ddp", v, world, rank, local_rank, dev, host_imgs, host_lbls, batch,
                                   sampler_ids))
            except (RuntimeError, ImportError, AttributeError) as e:
                failed[v] = f"{type(e).__name__}: {str(e)[:160]}"
                if world > 1:
                    # ranks must stay in step, so nothing more is run after a failure; the line with our own arm's
                    # numbers (already measured) is still printed, then every rank leaves without further collectives
                    failed["_stopped_after"] = v
                    break
        return out, failed

    global_batch = batch * world

    def rate(times):
        return global_batch * args.steps / (statistics.median(times) / 1e3)

    if args.impl == "ours":
        main_arm = run_arm(args, "ours", None, world, rank, local_rank, dev, host_imgs, host_lbls, batch, sampler_ids)
        base_arms, base_failed = torch_arms() if variants else ([], {})
    else:
        base_arms, base_failed = torch_arms()
        if not base_arms:
            raise SystemExit(f"no stock-PyTorch variant could be run: {base_failed}")
        main_arm = max(base_arms, key=lambda a: rate(a["times_dev"]))

    if rank == 0:
        value, e2e = rate(main_arm["times_dev"]), rate(main_arm["times_e2e"])
        med_dev = statistics.median(main_arm["times_dev"])
        med_e2e = statistics.median(main_arm["times_e2e"])
        base = read_baseline(args.model, world)
        out = {
            "metric": f"{args.model}_train_images_per_sec", "value": round(value, 1), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(med_dev / args.steps, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (round(value / base, 4) if base else None), "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": args.model, "global_batch": global_batch, "per_gpu_batch": batch,
                       "input": [ch, hw, hw], "parallelism": f"dp{world}", "comm": main_arm["comm"],
                       "optimizer": "sgd momentum 0.9 wd 5e-4 lr 0.01, fp32 master weights",
                       "l2_policy": "no flush: per-step working set (activations + deltas + fp32 weights, "
                                    "gradients, momentum) is several times the 126 MB L2",
                       "cuda_graph": (not args.no_graph) if args.impl == "ours" else main_arm["variant"] != "eager",
                       "timing": "the region of `steps` steps is repeated until min_seconds of device time; value "
                                 "and ms_per_step are the median region"},
            "timing": spread(main_arm["times_dev"], args.steps, main_arm["clocks"]),
            "e2e": {"value": round(e2e, 1), "unit": "images/s", "ms_per_step": round(med_e2e / args.steps, 4),
                    "h2d_bytes_per_step": main_arm["h2d"], "d2h_bytes_per_step": main_arm["d2h"],
                    "h2d_copy_ms_slowest_rank": main_arm.get("h2d_copy_ms_slowest_rank"),
                    "host_threads_bound_to_numa_node": main_arm.get("numa_node"),
                    "timing": spread(main_arm["times_e2e"], args.steps, main_arm["clocks"]),
                    "note": "pinned uint8 batch + int32 labels copied every step; loss read back with a one-step lag"},
            "gpu_launches": main_arm.get("gpu_launches", 0),
            "final_loss": main_arm["loss"],
            "clocks": main_arm["clocks"],
        }
        if args.impl == "ours":
            out["device_status"] = main_arm.get("device_status")
            if world > 1:
                out["replicas_identical"] = main_arm.get("replicas_identical")
        else:
            out["variant"] = main_arm["variant"]
        if base_arms:
            # stock PyTorch timed in this same process, on this same GPU, minutes apart at most
            best = max(base_arms, key=lambda a: rate(a["times_dev"]))
            out["baseline_same_lease"] = {
                "what": "torch DDP + cuDNN/cuBLAS, same model / batch / optimizer, fastest of the variants run",
                "variant": best["variant"], "value": round(rate(best["times_dev"]), 1),
                "e2e_value": round(rate(best["times_e2e"]), 1),
                "variants": {a["variant"]: {"value": round(rate(a["times_dev"]), 1),
                                            "e2e_value": round(rate(a["times_e2e"]), 1),
                                            "timing": spread(a["times_dev"], args.steps, a["clocks"]),
                                            "clocks": a["clocks"]} for a in base_arms},
            }
            if args.impl == "ours":
                out["vs_baseline_same_lease"] = round(value / rate(best["times_dev"]), 4)
                out["e2e_vs_baseline_same_lease"] = round(e2e / rate(best["times_e2e"]), 4)
        if base_failed:
            out["baseline_variants_failed"] = base_failed
        print(json.dumps(out), flush=True)
    if world > 1:
        if base_failed.get("_stopped_after"):
            os._exit(0)      # the process group may hold a half-captured collective: no clean shutdown to be had
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
