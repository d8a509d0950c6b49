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
