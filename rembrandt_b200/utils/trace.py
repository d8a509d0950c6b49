"""NVTX ranges around the phases of a training step (forward / backward / update) and around every operator.

Off unless the environment has ``RB_NVTX=1``: the ranges only matter under a timeline profiler, and the reference
has no tracing beyond wall-clock times around minibatches (src/opt/sgd/new.rs:273-275). When the step runs as a CUDA
graph the ranges mark the capture, not the replays; profile with ``--no-graph`` to see them per step.
"""
from __future__ import annotations

import contextlib
import os

import torch

ENABLED = os.environ.get("RB_NVTX", "0") == "1"
_NULL = contextlib.nullcontext()


class _Range:
    __slots__ = ("name",)

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


def span(name: str):
    """Context manager: an NVTX range called `name` when tracing is on and CUDA is present, else nothing."""
    if ENABLED and torch.cuda.is_available():
        return _Range(name)
    return _NULL


def enable(on: bool = True) -> None:
    global ENABLED
    ENABLED = bool(on)
