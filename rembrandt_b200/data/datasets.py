"""Data sources: seeded synthetic images, MNIST (IDX), CIFAR-10 (binary), NdArray blobs.

Counterparts of the reference's sources (src/data_new.rs:551-997) behind one small interface: ``len(src)``,
``src[i] -> (uint8 array [C,H,W], int label)``. File parsing is done by the native host library
(csrc/host/rng_util.cc). LMDB / varraydb / episodb readers are not provided: those crates are absent from
the reference tree and their on-disk formats are not visible; the Caffe ``Datum`` decoder in ``codecs.py`` covers
the record format for anyone who brings an LMDB binding.
"""
from __future__ import annotations

import ctypes as C
import mmap
import os
from typing import Optional, Tuple

import numpy as np

from .. import _native
from ..models.descriptor import DatasetSplit, load_data


def source_arrays(source):
    """(images uint8 [n, C, H, W], labels int32 [n]) of a whole source, for the native batch loader. MNIST and
    CIFAR-10 files map directly (no per-sample Python work); any other source is materialised sample by sample."""
    if hasattr(source, "as_arrays"):
        return source.as_arrays()
    n = len(source)
    first, _ = source[0]
    imgs = np.empty((n,) + tuple(np.asarray(first).shape), dtype=np.uint8)
    lbls = np.empty(n, dtype=np.int32)
    for i in range(n):
        im, lb = source[i]
        imgs[i], lbls[i] = im, lb
    return imgs, lbls


class DataSource:
    dims: Tuple[int, int, int]   # (W, H, C) as in the reference
    num_classes: int

    def __len__(self):
        raise NotImplementedError

    def __getitem__(self, i):
        raise NotImplementedError


class SyntheticDataSource(DataSource):
    """Seeded synthetic images: sample i is a pure function of (seed, i). With `separable` the mean brightness of
    a class-dependent patch encodes the label, so a network can actually learn it (convergence smoke tests)."""

    def __init__(self, n: int, dims=(28, 28, 1), num_classes=10, seed=0, separable=False):
        self.n, self.dims, self.num_classes, self.seed, self.separable = n, tuple(dims), num_classes, seed, separable

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        w, h, c = self.dims
        rng = np.random.default_rng((self.seed * 1000003 + int(i)) & 0x7FFFFFFF)
        label = int(rng.integers(0, self.num_classes))
        img = rng.integers(0, 256, size=(c, h, w), dtype=np.uint8)
        if self.separable:
            img = (img // 4).astype(np.uint8)
            band = max(1, h // self.num_classes)
            y0 = (label * band) % max(1, h - band + 1)
            img[:, y0:y0 + band, :] = 255 - img[:, y0:y0 + band, :] // 2
        return img, label

    def as_arrays(self):
        """All samples as (uint8 [n, C, H, W], int32 [n]), built once: what the native batch loader reads. Without it
        the training tools would assemble synthetic batches sample by sample in Python, at a tenth of what a GPU eats."""
        if getattr(self, "_arrays", None) is None:
            w, h, c = self.dims
            imgs = np.empty((self.n, c, h, w), dtype=np.uint8)
            lbls = np.empty(self.n, dtype=np.int32)
            for i in range(self.n):
                imgs[i], lbls[i] = self[i]
            self._arrays = (imgs, lbls)
        return self._arrays


class _Mapped:
    def __init__(self, path):
        self._f = open(path, "rb")
        self.size = os.fstat(self._f.fileno()).st_size
        self.mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.arr = np.frombuffer(self.mm, dtype=np.uint8)


class MnistDataSource(DataSource):
    """IDX files: big-endian magic {0,0,type,ndim}, u32 dims, raw bytes; images become (W,H,1)
    (src/data_new.rs:648-795)."""

    def __init__(self, data_path: str, labels_path: str):
        lib = _native.host()
        self._img, self._lbl = _Mapped(data_path), _Mapped(labels_path)

        def header(m):
            dt, nd, off = C.c_uint32(), C.c_uint32(), C.c_uint64()
            dims = (C.c_uint32 * 4)()
            rc = lib.rb_idx_header(m.arr.ctypes.data, m.size, C.byref(dt), C.byref(nd), C.byref(dims), C.byref(off))
            if rc != 0:
                raise ValueError(f"bad IDX file (code {rc})")
            return int(nd.value), [int(d) for d in dims], int(off.value)

        nd, dims, self._ioff = header(self._img)
        if nd != 3:
            raise ValueError("image file must have 3 dimensions")
        self.n, h, w = dims[0], dims[1], dims[2]
        self.dims = (w, h, 1)
        ndl, dl, self._loff = header(self._lbl)
        if dl[0] != self.n:
            raise ValueError("label count does not match image count")
        self.num_classes = 10

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        w, h, _ = self.dims
        o = self._ioff + i * w * h
        return self._img.arr[o:o + w * h].reshape(1, h, w), int(self._lbl.arr[self._loff + i])

    def as_arrays(self):
        w, h, _ = self.dims
        imgs = self._img.arr[self._ioff:self._ioff + self.n * w * h].reshape(self.n, 1, h, w)   # a view of the mapping
        return imgs, self._lbl.arr[self._loff:self._loff + self.n].astype(np.int32)


class Cifar10DataSource(DataSource):
    """Records of 1 label byte + 3072 planar RGB bytes (src/data_new.rs:797-883)."""
    REC = 3073

    def __init__(self, data_path: str):
        self._m = _Mapped(data_path)
        if self._m.size % self.REC:
            raise ValueError("file size is not a multiple of the CIFAR-10 record size")
        self.n = self._m.size // self.REC
        self.dims = (32, 32, 3)
        self.num_classes = 10

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        o = i * self.REC
        return self._m.arr[o + 1:o + self.REC].reshape(3, 32, 32), int(self._m.arr[o])

    def batch(self, first, count):
        """Contiguous records split into image and label arrays by the native reader."""
        imgs = np.empty((count, 3, 32, 32), dtype=np.uint8)
        lbls = np.empty(count, dtype=np.int32)
        rc = _native.host().rb_cifar_split(self._m.arr.ctypes.data, self._m.size, first, count, imgs.ctypes.data,
                                           lbls.ctypes.data)
        if rc != 0:
            raise IndexError("record range outside the file")
        return imgs, lbls

    def as_arrays(self):
        return self.batch(0, self.n)


def compute_mean(source: DataSource, limit: Optional[int] = None) -> np.ndarray:
    """Per-element mean image [C,H,W] (the reference's calculate-cifar10-mean tool)."""
    n = len(source) if limit is None else min(limit, len(source))
    w, h, c = source.dims
    imgs = np.stack([source[i][0] for i in range(n)]).reshape(n, -1)
    out = np.empty(c * h * w, dtype=np.float32)
    _native.host().rb_mean_u8(np.ascontiguousarray(imgs).ctypes.data, n, c * h * w, out.ctypes.data)
    return out.reshape(c, h, w)


class _IterableAsSource:
    """A sequential shard (database cursor) behind the indexable interface; records are materialised on first use."""

    def __init__(self, shard):
        self._shard, self._items = shard, None

    def _load(self):
        if self._items is None:
            self._items = list(self._shard)
        return self._items

    def __len__(self):
        return len(self._shard)

    def __getitem__(self, i):
        return self._load()[i]

    @property
    def dims(self):
        """(W, H, C) of the records, read off the first one."""
        c, h, w = np.asarray(self._load()[0][0]).shape
        return (w, h, c)


def open_split(split: DatasetSplit, rank: int = 0, world: int = 1) -> DataSource:
    """Open one `[dataset.<split>]` table of a .data file (src/data_new.rs:296-412)."""
    if split.source == "mnist":
        return MnistDataSource(split.data_path, split.labels_path)
    if split.source == "cifar10":
        return Cifar10DataSource(split.data_path)
    if split.source == "synthetic":
        return SyntheticDataSource(getattr(split, "size", 10000), getattr(split, "dims", None) or (28, 28, 1),
                                   getattr(split, "num_classes", 10), separable=True)
    if split.source == "lmdb_caffe":
        from .codecs import JpegDataCodec
        from .lmdb_reader import LmdbCaffeShard
        src = _IterableAsSource(LmdbCaffeShard(split.data_path, rank, world, codec=JpegDataCodec()))
        src.lmdb_path = split.data_path      # lets the native loader read the environment without Python per sample
        return src
    if split.source == "varraydb":
        from .codecs import JpegDataCodec
        from .recorddb import VarrayDbShard
        return VarrayDbShard(split.data_path, split.labels_path, JpegDataCodec(), rank, world)
    if split.source == "episodb":
        from .recorddb import EpisodeDataSource
        dims = tuple(split.frame_dims) if getattr(split, "frame_dims", None) else (19, 19, 1)
        return EpisodeDataSource(split.data_path, dims, lookahead=getattr(split, "lookahead", 1) or 1, rank=rank,
                                 world=world)
    raise ValueError(f"unknown data source {split.source!r}")


def open_data_file(path: str, split: str = "train") -> DataSource:
    return open_split(load_data(path)[split])
