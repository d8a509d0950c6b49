"""Python front of the native prefetching batch loader (csrc/host/batch_loader.cc).

    loader = NativeBatchLoader(images_u8 [n, ...], labels_i32 [n], batch=128, mode="shuffled", threads=4)
    for images, labels in loader:          # torch uint8 [batch, ...] / int32 [batch] views of pinned ring slots
        engine.feed(images, labels); engine.step()

C++ worker threads fill a ring of pinned host buffers while the training loop runs; a slot handed out by the
iterator stays valid until the next-but-`hold` batch is requested (default: the two most recent batches stay
valid, which covers the engine's double-buffered H2D copies). The order of samples is a function of
(mode, seed, position) only, so a run can be resumed at any batch number and does not depend on thread timing.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native

MODES = {"cyclic": 0, "random": 1, "shuffled": 2}


class NativeBatchLoader:
    def __init__(self, images: np.ndarray, labels: Optional[np.ndarray], batch: int, mode: str = "shuffled",
                 seed: int = 0, threads: int = 2, slots: int = 4, shard: Optional[Tuple[int, int]] = None,
                 pin: Optional[bool] = None, hold: int = 2, max_batches: Optional[int] = None):
        self._images = np.ascontiguousarray(images, dtype=np.uint8)
        self._labels = None if labels is None else np.ascontiguousarray(labels, dtype=np.int32)
        n = self._images.shape[0]
        self.lo, self.hi = shard if shard is not None else (0, n)
        if not (0 <= self.lo < self.hi <= n):
            raise ValueError("empty or out-of-range shard")
        ip, lp = self._make_slots(tuple(self._images.shape[1:]), batch, mode, seed, slots, pin, hold, max_batches)
        self._h = self._lib.rb_loader_create(self._images.ctypes.data,
                                             None if self._labels is None else self._labels.ctypes.data, self.elems,
                                             self.lo, self.hi, self.batch, self.mode, self.seed, threads, slots, ip, lp)
        if not self._h:
            raise RuntimeError("rb_loader_create rejected its arguments")

    def _make_slots(self, sample_shape, batch, mode, seed, slots, pin, hold, max_batches):
        if slots < hold + 2:
            raise ValueError("need at least hold + 2 slots")
        self.sample_shape = tuple(sample_shape)
        self.elems = int(np.prod(self.sample_shape)) if self.sample_shape else 1
        self.batch, self.mode, self.seed = int(batch), MODES[mode], int(seed)
        self.hold, self.max_batches = hold, max_batches
        pin = torch.cuda.is_available() if pin is None else pin
        self._img_slots = [torch.empty((batch,) + self.sample_shape, dtype=torch.uint8, pin_memory=pin)
                           for _ in range(slots)]
        self._lbl_slots = [torch.empty(batch, dtype=torch.int32, pin_memory=pin) for _ in range(slots)]
        self._lib = _native.host()
        self._held = []
        self._given = 0
        self._h = None
        return ((C.c_void_p * slots)(*[t.data_ptr() for t in self._img_slots]),
                (C.c_void_p * slots)(*[t.data_ptr() for t in self._lbl_slots]))

    @classmethod
    def from_caffe_lmdb(cls, path: str, sample_shape: Tuple[int, int, int], batch: int, mode: str = "shuffled",
                        seed: int = 0, threads: int = 2, slots: int = 4, shard: Optional[Tuple[int, int]] = None,
                        pin: Optional[bool] = None, hold: int = 2, max_batches: Optional[int] = None):
        """A loader over the raw images of a Caffe image database (the reference's `lmdb_caffe` source,
        src/data/lmdb_data.rs:50-152): the environment is memory-mapped and indexed once, then the worker threads
        copy pixels of shape `sample_shape` = (C, H, W) straight from the mapping into the pinned slots. `shard` is
        a range of record numbers in key order; sample positions count from the start of the shard."""
        self = cls.__new__(cls)
        self._images = self._labels = None
        ip, lp = self._make_slots(sample_shape, batch, mode, seed, slots, pin, hold, max_batches)
        lo, hi = shard if shard is not None else (0, 2**62)
        err = C.c_int32(0)
        self._h = self._lib.rb_loader_create_lmdb(path.encode(), self.elems, lo, hi, self.batch, self.mode, self.seed,
                                                  threads, slots, ip, lp, C.byref(err))
        if not self._h:
            raise RuntimeError({1: "cannot open the environment", 2: "malformed record",
                                3: "a record is encoded or not of the given shape",
                                4: "empty shard or bad arguments"}.get(err.value, f"error {err.value}") + f": {path}")
        self.lo, self.hi = 0, None      # positions are relative to the shard
        return self

    def __iter__(self):
        return self

    def __next__(self):
        if self.max_batches is not None and self._given >= self.max_batches:
            raise StopIteration
        while len(self._held) >= self.hold:
            self._lib.rb_loader_release(self._h, self._held.pop(0))
        number = C.c_uint64()
        slot = self._lib.rb_loader_acquire(self._h, C.byref(number))
        if slot < 0:
            raise StopIteration
        self._held.append(slot)
        self._given += 1
        return self._img_slots[slot], self._lbl_slots[slot]

    def sample_index(self, pos: int) -> int:
        """Dataset index of the sample at stream position `pos` (batch k holds positions k*batch .. k*batch+batch-1)."""
        if self.hi is None:
            raise ValueError("a database-backed loader does not know its length on the Python side")
        return int(self._lib.rb_loader_sample_index(self.lo, self.hi, self.mode, self.seed, pos))

    def close(self):
        if self._h:
            self._lib.rb_loader_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
