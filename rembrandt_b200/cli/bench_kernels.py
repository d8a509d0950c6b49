"""bench-kernels and sleep-test: host-side overheads of driving the device, in microseconds.

The reference measures the cost of a kernel launch, of a device switch and of event record / synchronise
(tools/bench-kernels.rs:12-46) and the granularity of thread sleeps (tools/sleep-test.rs, which matters for its
polling barriers). Here:

* sleep granularity: requested vs observed duration of `time.sleep` (runs anywhere);
* on a GPU: wall-clock cost per call of a tiny kernel launch through the ctypes binding, of an event record, of
  `torch.cuda.set_device`, of a stream synchronise after one tiny kernel, and the device-side cost per kernel of
  replaying a captured CUDA graph of such launches (what the training step pays instead of the launch cost).
"""
import argparse
import json
import time

import torch


def sleep_granularity(requests_us=(1, 10, 100, 1000, 10000), repeats=20):
    rows = []
    for us in requests_us:
        t0 = time.perf_counter()
        for _ in range(repeats):
            time.sleep(us * 1e-6)
        rows.append({"requested_us": us, "observed_us": (time.perf_counter() - t0) / repeats * 1e6})
    return rows


def _per_call_us(fn, calls):
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(calls):
        fn()
    host = (time.perf_counter() - t0) / calls * 1e6
    torch.cuda.synchronize()
    return host


def device_overheads(calls=2000, graph_kernels=200):
    from ..ops import native_ops as K
    x = torch.zeros(1024, dtype=torch.float32, device="cuda")
    y = torch.zeros_like(x)
    launch = lambda: K.axpby(x, y, x.numel(), 1.0, 0.0)
    for _ in range(10):
        launch()
    ev = torch.cuda.Event(enable_timing=True)
    dev = torch.cuda.current_device()
    out = {
        "kernel_launch_us": _per_call_us(launch, calls),
        "event_record_us": _per_call_us(lambda: ev.record(), calls),
        "set_device_us": _per_call_us(lambda: torch.cuda.set_device(dev), calls),
    }

    def launch_and_sync():
        launch()
        torch.cuda.current_stream().synchronize()
    out["launch_plus_stream_sync_us"] = _per_call_us(launch_and_sync, max(1, calls // 10))
    # device time per kernel: eager back-to-back launches vs one graph replay
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(graph_kernels):
        launch()
    end.record()
    torch.cuda.synchronize()
    out["eager_device_us_per_kernel"] = start.elapsed_time(end) * 1e3 / graph_kernels
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        launch()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(graph_kernels):
                launch()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    out["graph_device_us_per_kernel"] = start.elapsed_time(end) * 1e3 / graph_kernels
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--calls", type=int, default=2000)
    ap.add_argument("--no-device", action="store_true", help="only the host-side sleep test")
    args = ap.parse_args(argv)
    result = {"sleep": sleep_granularity()}
    for r in result["sleep"]:
        print(f"sleep {r['requested_us']:>6d} us -> {r['observed_us']:9.1f} us")
    if torch.cuda.is_available() and not args.no_device:
        result["device"] = device_overheads(args.calls)
        for k, v in result["device"].items():
            print(f"{k:<30s} {v:9.2f}")
    print(json.dumps(result))
    return result


if __name__ == "__main__":
    main()
