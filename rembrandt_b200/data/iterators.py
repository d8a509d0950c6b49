"""Shards, sample iterators and asynchronous prefetching, after the reference's data API
(src/data/mod.rs:23-809): a *shard* is an indexable range of a source; an *iterator* yields samples;
asynchronous wrappers move the work to threads.

* ``RangeDataShard`` / ``partition_shard``  contiguous (balanced) part of a source for one rank;
* ``SequentialSampleIter``, ``RandomSampleDataIter`` (uniform with replacement), ``CyclicSampleDataIter``;
* ``TransformDataIter``                     applies a host-side transform per sample;
* ``AsyncQueueDataIter``                    one prefetch thread, bounded queue (256 by default);
* ``AsyncPoolDataIter``                     N transform threads, original order restored;
* ``ParallelJoinDataIter``                  N independent producers, unordered;
* ``BatchIter``                             packs samples into pinned uint8 / int32 batch tensors.
"""
from __future__ import annotations

import queue
import threading
from typing import Callable, Iterable, List, Optional

import numpy as np
import torch

from ..utils.rng import XorShift128Plus, cyclic_partition_range, partition_range


class RangeDataShard:
    def __init__(self, source, lo: int = 0, hi: Optional[int] = None):
        self.source, self.lo, self.hi = source, lo, len(source) if hi is None else hi

    def __len__(self):
        return self.hi - self.lo

    def __getitem__(self, i):
        if not 0 <= i < len(self):
            raise IndexError(i)
        return self.source[self.lo + i]


class RangeWrapDataShard:
    """A shard made of up to two pieces of the source (wrap-around partitions, src/util.rs:23-41)."""

    def __init__(self, source, pieces):
        self.source, self.pieces = source, list(pieces)
        self._len = sum(b - a for a, b in self.pieces)

    def __len__(self):
        return self._len

    def __getitem__(self, i):
        for a, b in self.pieces:
            if i < b - a:
                return self.source[a + i]
            i -= b - a
        raise IndexError


def partition_shard(source, rank: int, world: int) -> RangeDataShard:
    lo, hi = partition_range(len(source), world, rank)
    return RangeDataShard(source, lo, hi)


def cyclic_partition_shard(source, rank: int, world: int, shift: int) -> RangeWrapDataShard:
    return RangeWrapDataShard(source, cyclic_partition_range(len(source), world, rank, shift))


class SequentialSampleIter:
    def __init__(self, shard):
        self.shard = shard

    def __iter__(self):
        for i in range(len(self.shard)):
            yield self.shard[i]


class RandomSampleDataIter:
    """Uniform sampling with replacement; one pass yields len(shard) samples."""

    def __init__(self, shard, seed=(1, 2)):
        self.shard, self.rng = shard, XorShift128Plus(*seed)

    def __iter__(self):
        n = len(self.shard)
        for _ in range(n):
            yield self.shard[self.rng.below(n)]


class RandomIndexIter:
    """The index stream of `RandomSampleDataIter` without the samples (uniform with replacement, len(shard) per pass):
    fed to `AsyncPoolDataIter` with `shard.__getitem__` as the transform, it decodes samples on several threads while
    keeping the order of the draws."""

    def __init__(self, n: int, seed=(1, 2)):
        self.n, self.rng = n, XorShift128Plus(*seed)

    def __iter__(self):
        for _ in range(self.n):
            yield self.rng.below(self.n)


class CyclicSampleDataIter:
    """Endless sequential passes (validation in the reference iterates a fixed number of samples off this)."""

    def __init__(self, shard):
        self.shard, self.pos = shard, 0

    def __iter__(self):
        n = len(self.shard)
        while True:
            yield self.shard[self.pos]
            self.pos = (self.pos + 1) % n


# ---- the episode-based iterators of the reference's older data API (src/data_new.rs:97-279) ----------------
def episode_ranges(source):
    """[first, end) sample ranges of the episodes of `source`; a source without episodes has one per sample."""
    if hasattr(source, "episode_ranges"):
        return [r for r in source.episode_ranges() if r[1] > r[0]]
    return [(i, i + 1) for i in range(len(source))]


SampleIterator = SequentialSampleIter   # every sample once, episode by episode (data_new.rs:122-147)


class RandomEpisodeIterator:
    """len(source) draws per pass: a uniformly random episode, then a uniformly random sample of it
    (data_new.rs:149-230). Long and short games are therefore equally likely to be visited."""

    def __init__(self, source, seed=(1, 2)):
        self.source, self.rng = source, XorShift128Plus(*seed)
        self.episodes = episode_ranges(source)

    def __iter__(self):
        for _ in range(len(self.source)):
            lo, hi = self.episodes[self.rng.below(len(self.episodes))]
            yield self.source[lo + self.rng.below(hi - lo)]


class CyclicEpisodeIterator:
    """Walks the episodes in order, again and again, taking one random sample from each, until len(source)
    samples have been drawn (data_new.rs:232-279)."""

    def __init__(self, source, seed=(1, 2)):
        self.source, self.rng = source, XorShift128Plus(*seed)
        self.episodes = episode_ranges(source)

    def __iter__(self):
        limit, count = len(self.source), 0
        while count < limit:
            for lo, hi in self.episodes:
                yield self.source[lo + self.rng.below(hi - lo)]
                count += 1
                if count >= limit:
                    return


class PartitionDataSource(RangeDataShard):
    """The part of a source that belongs to worker `rank` of `world` (data_new.rs:480-549). Sources with episodes are
    cut at episode boundaries, so that no game is split between workers."""

    def __init__(self, rank: int, world: int, source):
        if hasattr(source, "episode_ranges"):
            eps = episode_ranges(source)
            e_lo, e_hi = partition_range(len(eps), world, rank)
            lo = eps[e_lo][0] if e_lo < e_hi else 0
            hi = eps[e_hi - 1][1] if e_lo < e_hi else 0
            self._eps = [(a - lo, b - lo) for a, b in eps[e_lo:e_hi]]
        else:
            lo, hi = partition_range(len(source), world, rank)
            self._eps = None
        super().__init__(source, lo, hi)

    def episode_ranges(self):
        return list(self._eps) if self._eps is not None else [(i, i + 1) for i in range(len(self))]


class AugmentDataSource:
    """A source whose samples pass through `augment(image, label) -> (image, label)` on the host
    (data_new.rs:429-478); episodes are those of the inner source."""

    def __init__(self, augment: Callable, inner):
        self.augment, self.inner = augment, inner
        if hasattr(inner, "dims"):
            self.dims = inner.dims
        if hasattr(inner, "episode_ranges"):
            self.episode_ranges = inner.episode_ranges

    def __len__(self):
        return len(self.inner)

    def __getitem__(self, i):
        image, label = self.inner[i]
        return self.augment(image, label)


class TransformDataIter:
    def __init__(self, inner: Iterable, transform: Callable):
        self.inner, self.transform = inner, transform

    def __iter__(self):
        for s in self.inner:
            yield self.transform(s)


_END = object()


class AsyncQueueDataIter:
    """One producer thread fills a bounded queue; iteration can be restarted (each `iter()` starts a new pass and
    waits for the previous producer to acknowledge the stop request)."""

    def __init__(self, inner: Iterable, capacity: int = 256):
        self.inner, self.capacity = inner, capacity
        self._thread = None
        self._stop = None

    def _produce(self, q, stop):
        try:
            for s in self.inner:
                while not stop.is_set():
                    try:
                        q.put(s, timeout=0.05)
                        break
                    except queue.Full:
                        continue
                if stop.is_set():
                    return
            q.put(_END)
        except BaseException as e:  # surface producer failures to the consumer
            q.put(e)

    def __iter__(self):
        self.close()
        q = queue.Queue(self.capacity)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._produce, args=(q, self._stop), daemon=True)
        self._thread.start()
        while True:
            item = q.get()
            if item is _END:
                return
            if isinstance(item, BaseException):
                raise item
            yield item

    def close(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=5)
            self._thread = None


class AsyncPoolDataIter:
    """N worker threads apply `transform`; results come out in the order of the inner iterator."""

    def __init__(self, inner: Iterable, transform: Callable, num_workers: int = 4, window: int = 64):
        self.inner, self.transform, self.num_workers, self.window = inner, transform, num_workers, window

    def __iter__(self):
        tasks: "queue.Queue" = queue.Queue(self.window)
        results = {}
        cond = threading.Condition()

        def work():
            while True:
                item = tasks.get()
                if item is _END:
                    return
                idx, s = item
                try:
                    r = self.transform(s)
                except BaseException as e:
                    r = e
                with cond:
                    results[idx] = r
                    cond.notify_all()

        workers = [threading.Thread(target=work, daemon=True) for _ in range(self.num_workers)]
        for w in workers:
            w.start()
        submitted = 0
        emitted = 0
        it = iter(self.inner)
        done = False
        try:
            while True:
                while not done and submitted - emitted < self.window:
                    try:
                        tasks.put((submitted, next(it)))
                        submitted += 1
                    except StopIteration:
                        done = True
                if emitted == submitted and done:
                    return
                with cond:
                    while emitted not in results:
                        cond.wait(timeout=0.1)
                    r = results.pop(emitted)
                emitted += 1
                if isinstance(r, BaseException):
                    raise r
                yield r
        finally:
            for _ in workers:
                tasks.put(_END)


class ParallelJoinDataIter:
    """N independent producers (each with its own inner iterator) feeding one queue; order is arbitrary."""

    def __init__(self, inners: List[Iterable], capacity: int = 256):
        self.inners, self.capacity = inners, capacity

    def __iter__(self):
        q: "queue.Queue" = queue.Queue(self.capacity)
        stop = threading.Event()

        def produce(inner):
            try:
                for s in inner:
                    while not stop.is_set():
                        try:
                            q.put(s, timeout=0.05)
                            break
                        except queue.Full:
                            continue
                    if stop.is_set():
                        return
            finally:
                q.put(_END)

        threads = [threading.Thread(target=produce, args=(i,), daemon=True) for i in self.inners]
        for t in threads:
            t.start()
        live = len(threads)
        try:
            while live:
                item = q.get()
                if item is _END:
                    live -= 1
                    continue
                yield item
        finally:
            stop.set()


class BatchIter:
    """Packs (image [C,H,W] uint8, label) samples into batch tensors; pinned when CUDA is available so that the
    engine's host-to-device copies are asynchronous. A pool of `depth` buffers is cycled."""

    def __init__(self, inner: Iterable, batch: int, dims, depth: int = 4, drop_last: bool = True):
        w, h, c = dims
        self.inner, self.batch, self.drop_last = inner, batch, drop_last
        pin = torch.cuda.is_available()
        self.imgs = [torch.zeros((batch, c, h, w), dtype=torch.uint8) for _ in range(depth)]
        self.lbls = [torch.zeros(batch, dtype=torch.int32) for _ in range(depth)]
        if pin:
            self.imgs = [t.pin_memory() for t in self.imgs]
            self.lbls = [t.pin_memory() for t in self.lbls]
        # numpy views of the same (pinned) memory: a per-sample numpy assignment costs a fraction of a torch call
        self._imgs_np = [t.numpy() for t in self.imgs]
        self._lbls_np = [t.numpy() for t in self.lbls]

    def __iter__(self):
        k, slot = 0, 0
        shape = self._imgs_np[0].shape[1:]
        for img, label in self.inner:
            self._imgs_np[slot][k] = np.asarray(img).reshape(shape)
            self._lbls_np[slot][k] = label
            k += 1
            if k == self.batch:
                yield self.imgs[slot], self.lbls[slot]
                slot = (slot + 1) % len(self.imgs)
                k = 0
        if k and not self.drop_last:
            yield self.imgs[slot][:k], self.lbls[slot][:k]


class RaggedBatchIter:
    """Packs samples of different sizes (image [C,h,w] uint8, label) for the variable-size input operator: a batch is
    ((padded uint8 [B, C * maxH * maxW], int32 [B, 2] of (w, h)), labels int32 [B]); every image is stored densely at
    the start of its row. Buffers are pinned when CUDA is available and cycled like `BatchIter`'s."""

    def __init__(self, inner: Iterable, batch: int, max_dims, depth: int = 4):
        mw, mh, c = max_dims
        self.inner, self.batch, self.max_hw, self.c = inner, batch, (mh, mw), c
        self.stride = c * mh * mw
        pin = torch.cuda.is_available()
        mk = (lambda t: t.pin_memory()) if pin else (lambda t: t)
        self.imgs = [mk(torch.zeros((batch, self.stride), dtype=torch.uint8)) for _ in range(depth)]
        self.shapes = [mk(torch.ones((batch, 2), dtype=torch.int32)) for _ in range(depth)]
        self.lbls = [mk(torch.zeros(batch, dtype=torch.int32)) for _ in range(depth)]

    def __iter__(self):
        k, slot = 0, 0
        for img, label in self.inner:
            a = torch.from_numpy(np.ascontiguousarray(img))
            c, h, w = a.shape
            if c != self.c or h > self.max_hw[0] or w > self.max_hw[1]:
                raise ValueError(f"sample of {w} x {h} x {c} exceeds the configured maximum")
            self.imgs[slot][k, : c * h * w].copy_(a.reshape(-1))
            self.shapes[slot][k, 0], self.shapes[slot][k, 1] = w, h
            self.lbls[slot][k] = int(label)
            k += 1
            if k == self.batch:
                yield (self.imgs[slot], self.shapes[slot]), self.lbls[slot]
                slot = (slot + 1) % len(self.imgs)
                k = 0
