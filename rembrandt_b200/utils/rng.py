"""Seeded xorshift128+ streams (native, csrc/host/rng_util.cc).

The reference seeds every operator from one shared ``[u64; 2]`` seed broadcast from rank 0
(src/operator/worker.rs:361-367, src/worker/gossip_dist.rs:1088-1095), so that all replicas start equal;
``derive`` plays that role here.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .. import _native


class XorShift128Plus:
    def __init__(self, s0: int, s1: int = 0):
        self._st = _native.XorShift()
        self._lib = _native.host()
        self._lib.rb_xs_seed(C.byref(self._st), s0 & (2**64 - 1), s1 & (2**64 - 1))

    def next_u64(self) -> int:
        return int(self._lib.rb_xs_next(C.byref(self._st)))

    def unit(self) -> float:
        return float(self._lib.rb_xs_unit(C.byref(self._st)))

    def below(self, n: int) -> int:
        return int(self._lib.rb_xs_below(C.byref(self._st), n))

    def uniform(self, n: int, lo: float, hi: float) -> torch.Tensor:
        out = np.empty(n, dtype=np.float32)
        self._lib.rb_xs_fill_uniform(C.byref(self._st), out.ctypes.data, n, lo, hi)
        return torch.from_numpy(out)

    def normal(self, n: int, mean: float, std: float) -> torch.Tensor:
        out = np.empty(n, dtype=np.float32)
        self._lib.rb_xs_fill_normal(C.byref(self._st), out.ctypes.data, n, mean, std)
        return torch.from_numpy(out)

    def permutation(self, n: int) -> list:
        out = np.empty(n, dtype=np.int32)
        self._lib.rb_xs_permutation(C.byref(self._st), out.ctypes.data, n)
        return out.tolist()

    def derive(self) -> "XorShift128Plus":
        """A child stream seeded from two draws of this one (per-operator seeds)."""
        return XorShift128Plus(self.next_u64(), self.next_u64())


def partition_range(n: int, parts: int, idx: int):
    """Balanced contiguous split of [0, n) (src/util.rs:3-21)."""
    lo, hi = C.c_uint64(), C.c_uint64()
    _native.host().rb_partition_range(n, parts, idx, C.byref(lo), C.byref(hi))
    return int(lo.value), int(hi.value)


def cyclic_partition_range(n: int, parts: int, idx: int, shift: int):
    """Like ``partition_range`` but rotated by `shift` with wrap-around (src/util.rs:23-41).

    Returns one or two (lo, hi) pieces.
    """
    lo, hi = partition_range(n, parts, idx)
    if n == 0 or hi == lo:
        return []            # an empty part stays empty however it is rotated
    length = hi - lo
    lo = (lo + shift) % n
    hi = lo + length
    if hi <= n:
        return [(lo, hi)]
    return [(lo, n), (0, hi - n)]
