"""Variable-length record stores for image datasets and frame episodes.

The reference reads ImageNet-scale data from `varraydb` (a data store plus a label store of little-endian i32,
src/data/varraydb_data.rs:15-88) and Go positions from `episodb` (episodes of frames with look-ahead labels,
src/data_new.rs:551-646). Both are external crates whose file formats are not part of the reference tree, so the
stores here define their own simple layout:

  <name>.dat   the records back to back
  <name>.idx   little-endian u64 offsets, n + 1 of them (record i is dat[idx[i] : idx[i + 1]])
  <name>.epi   (episode stores only) little-endian u64 pairs (first record, one past the last record) per episode

Readers mmap both files; writers append.
"""
from __future__ import annotations

import mmap
import os
import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..utils.rng import partition_range


class RecordDbWriter:
    def __init__(self, prefix: str):
        os.makedirs(os.path.dirname(os.path.abspath(prefix)), exist_ok=True)
        self._dat = open(prefix + ".dat", "wb")
        self._idx = open(prefix + ".idx", "wb")
        self._epi = None
        self._prefix = prefix
        self._off = 0
        self._n = 0
        self._idx.write(struct.pack("<Q", 0))

    def append(self, record: bytes) -> int:
        self._dat.write(record)
        self._off += len(record)
        self._idx.write(struct.pack("<Q", self._off))
        self._n += 1
        return self._n - 1

    def append_episode(self, records: Sequence[bytes]):
        if self._epi is None:
            self._epi = open(self._prefix + ".epi", "wb")
        first = self._n
        for r in records:
            self.append(r)
        self._epi.write(struct.pack("<QQ", first, self._n))

    def close(self):
        for f in (self._dat, self._idx, self._epi):
            if f is not None:
                f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class RecordDb:
    def __init__(self, prefix: str):
        self._fd = open(prefix + ".dat", "rb")
        size = os.fstat(self._fd.fileno()).st_size
        self._dat = mmap.mmap(self._fd.fileno(), 0, access=mmap.ACCESS_READ) if size else b""
        self._idx = np.fromfile(prefix + ".idx", dtype="<u8")
        if len(self._idx) < 1 or int(self._idx[-1]) != size:
            raise ValueError(f"{prefix}: index and data file disagree")
        self.episodes: Optional[np.ndarray] = None
        if os.path.exists(prefix + ".epi"):
            self.episodes = np.fromfile(prefix + ".epi", dtype="<u8").reshape(-1, 2)

    def __len__(self):
        return len(self._idx) - 1

    def __getitem__(self, i: int) -> bytes:
        if i < 0 or i >= len(self):
            raise IndexError(i)
        return bytes(self._dat[int(self._idx[i]): int(self._idx[i + 1])])

    def close(self):
        if not isinstance(self._dat, bytes):
            self._dat.close()
        self._fd.close()


class VarrayDbShard:
    """Records [lo, hi) of a data store with a parallel label store (i32 little endian), decoded by `codec`
    (JPEG, NdArray, ...): the shard worker `rank` of `world` reads."""

    def __init__(self, data_prefix: str, labels_prefix: str, codec, rank: int = 0, world: int = 1):
        self.data, self.labels = RecordDb(data_prefix), RecordDb(labels_prefix)
        if len(self.data) != len(self.labels):
            raise ValueError("data and label stores have different lengths")
        self.codec = codec
        self.lo, self.hi = partition_range(len(self.data), world, rank)

    def __len__(self):
        return self.hi - self.lo

    def __getitem__(self, i: int):
        j = self.lo + i
        if i < 0 or j >= self.hi:
            raise IndexError(i)
        label, = struct.unpack("<i", self.labels[j])
        return self.codec.decode(self.data[j]), label

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]


class EpisodeDataSource:
    """Frames of an episode store with look-ahead labels: sample i is (frame, [label of this frame, label of the
    next frame of the same episode, ...]) with -1 where the episode has ended; frames whose own label is negative
    are skipped (src/data_new.rs:551-646). A record is `label (i32 le) | frame bytes`."""

    def __init__(self, prefix: str, frame_dims: Tuple[int, int, int], lookahead: int = 1, rank: int = 0,
                 world: int = 1):
        self.db = RecordDb(prefix)
        if self.db.episodes is None:
            raise ValueError(f"{prefix} has no episode index")
        self.dims = frame_dims
        self.lookahead = lookahead
        e_lo, e_hi = partition_range(len(self.db.episodes), world, rank)
        self._samples: List[Tuple[int, int]] = []      # (record, end of its episode)
        self._episodes: List[Tuple[int, int]] = []     # per episode: range of its samples in `_samples`
        for first, end in self.db.episodes[e_lo:e_hi]:
            start = len(self._samples)
            for r in range(int(first), int(end)):
                if self._label(r) >= 0:
                    self._samples.append((r, int(end)))
            self._episodes.append((start, len(self._samples)))

    def episode_ranges(self) -> List[Tuple[int, int]]:
        """[first, end) sample indices of every episode of this shard (frames without a label are not samples)."""
        return list(self._episodes)

    def _label(self, r: int) -> int:
        return struct.unpack_from("<i", self.db[r])[0]

    def __len__(self):
        return len(self._samples)

    def __getitem__(self, i: int):
        r, end = self._samples[i]
        rec = self.db[r]
        w, h, c = self.dims
        frame = np.frombuffer(rec, dtype=np.uint8, offset=4).reshape(c, h, w)
        labels = [self._label(r + k) if r + k < end else -1 for k in range(self.lookahead)]
        return frame, labels if self.lookahead > 1 else labels[0]
