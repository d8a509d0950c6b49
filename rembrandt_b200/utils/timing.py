"""Device-side timing helpers (CUDA events on the launching stream, never wall clock).

The reference only measures wall-clock time around minibatches (src/opt/sgd/new.rs:273-275,498-503);
these helpers give per-operator forward / backward times and whole-step times on the device.
"""
from __future__ import annotations

from typing import Callable, Dict, List

import torch


def time_fn(fn: Callable[[], None], iters: int = 10, warmup: int = 3) -> float:
    """Mean device milliseconds of `fn` over `iters` calls after `warmup` calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def time_graph(fn: Callable[[], None], iters: int = 10, warmup: int = 3, replays: int = 5) -> float:
    """Mean device milliseconds of `fn` when `iters` calls of it are captured in one CUDA graph and replayed: what a
    kernel costs inside a captured training step. `time_fn` launches from the host, so for kernels shorter than a
    launch takes to issue (~10-20 us through Python) it reports the host's pace, not the device's."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(replays):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(end) / iters)
    return best


def time_ops(net, iters: int = 5, warmup: int = 2, train: bool = True) -> List[Dict]:
    """Per-operator forward and backward device time in milliseconds."""
    for _ in range(warmup):
        net.forward(train)
        net.backward()
    rows = []
    ev = lambda: torch.cuda.Event(enable_timing=True)
    fwd = {id(op): 0.0 for op in net.ops}
    bwd = {id(op): 0.0 for op in net.ops}
    for _ in range(iters):
        marks = []
        for op in net.ops:
            a, b = ev(), ev()
            a.record()
            op.forward(train, net.t)
            b.record()
            marks.append((op, "f", a, b))
        for op in reversed(net.ops[1:-1]):
            a, b = ev(), ev()
            a.record()
            op.backward()
            b.record()
            marks.append((op, "b", a, b))
        torch.cuda.synchronize()
        for op, kind, a, b in marks:
            (fwd if kind == "f" else bwd)[id(op)] += a.elapsed_time(b)
    for op in net.ops:
        rows.append({"name": op.name, "type": type(op).__name__, "fwd_ms": fwd[id(op)] / iters,
                     "bwd_ms": bwd[id(op)] / iters})
    return rows


def format_op_times(rows) -> str:
    out = [f"{'op':>12s} {'type':<22s} {'fwd ms':>9s} {'bwd ms':>9s}"]
    for r in rows:
        out.append(f"{r['name']:>12s} {r['type']:<22s} {r['fwd_ms']:9.3f} {r['bwd_ms']:9.3f}")
    out.append(f"{'total':>12s} {'':<22s} {sum(r['fwd_ms'] for r in rows):9.3f} {sum(r['bwd_ms'] for r in rows):9.3f}")
    return "\n".join(out)


def time_phases(engine, iters: int = 5, warmup: int = 2) -> Dict[str, float]:
    """Device milliseconds per phase of one eager training step on the batch already loaded into the network:
    forward, backward (the launches of an overlapped gradient exchange are issued from inside it) and the tail from the
    end of backward to the end of the update (exchange not hidden behind backward + optimizer step). On several ranks
    every figure is the maximum over ranks. Call between steps, never inside a graph capture."""
    import torch.distributed as dist

    net = engine.net

    def one(record):
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if record else None
        hook = None
        if engine._overlapped():
            engine.comm.prepare(engine.stepper, engine.lr)
            hook = engine.comm.on_op_backward
        if record:
            marks[0].record()
        net.forward(True, None)
        if record:
            marks[1].record()
        net.backward(hook)
        if record:
            marks[2].record()
        net.step_counter.add_(1)
        engine._update()
        if record:
            marks[3].record()
        return marks

    with torch.cuda.stream(engine.compute_stream):
        for _ in range(warmup):
            one(False)
        acc = [0.0, 0.0, 0.0]
        for _ in range(iters):
            m = one(True)
            m[3].synchronize()
            for i in range(3):
                acc[i] += m[i].elapsed_time(m[i + 1])
    out = torch.tensor([a / iters for a in acc], dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dev = out.cuda() if dist.get_backend() == "nccl" else out
        dist.all_reduce(dev, op=dist.ReduceOp.MAX)
        out = dev.cpu()
    fwd, bwd, tail = (float(v) for v in out)
    return {"forward_ms": fwd, "backward_ms": bwd, "exchange_update_tail_ms": tail, "step_ms": fwd + bwd + tail}
