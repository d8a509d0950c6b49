"""NdArray blob codec (native, csrc/host/ndarray_blob.cc) and file helpers.

Record: ``'N' 'D' tag0 tag1 | u32le ndim | u64le dims | little-endian data, first dimension fastest``
(tools/dump-array3d-header.rs:8-15 of the reference). Parameter and state files are plain concatenations of
such records. The tag bytes are opaque: preserved on read, ``00 01`` on write unless given.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, List, Sequence, Tuple

import numpy as np

from .. import _native

_DTYPES = {"f32": np.dtype("<f4"), "u8": np.dtype("u1"), "i32": np.dtype("<i4"), "f64": np.dtype("<f8")}
DEFAULT_TAG = (0x00, 0x01)


class BlobError(ValueError):
    pass


def encode_record(data, dims: Sequence[int], dtype="f32", tag=DEFAULT_TAG) -> bytes:
    """One record; `data` is flattened in memory order (first dimension fastest)."""
    dt = _DTYPES[dtype]
    arr = np.ascontiguousarray(np.asarray(data, dtype=dt).reshape(-1))
    n = 1
    for d in dims:
        n *= int(d)
    if n != arr.size:
        raise BlobError(f"dims {tuple(dims)} do not match {arr.size} elements")
    lib = _native.host()
    cdims = (C.c_uint64 * len(dims))(*[int(d) for d in dims])
    size = lib.rb_blob_record_size(len(dims), cdims, dt.itemsize)
    out = (C.c_uint8 * size)()
    ctag = (C.c_uint8 * 2)(*tag)
    wrote = lib.rb_blob_write(out, size, ctag, len(dims), cdims, arr.ctypes.data, dt.itemsize)
    if wrote != size:
        raise BlobError("record could not be written")
    return bytes(out)


def decode_records(buf: bytes, dtype="f32", offset=0, count=None) -> Tuple[List[Tuple[np.ndarray, tuple, tuple]], int]:
    """Parse records from `offset`; returns ([(flat array, dims, tag)], next offset)."""
    dt = _DTYPES[dtype]
    lib = _native.host()
    rec = _native.BlobRecord()
    out = []
    raw = np.frombuffer(buf, dtype=np.uint8)
    while offset < len(buf) and (count is None or len(out) < count):
        rc = lib.rb_blob_parse(raw.ctypes.data, len(buf), offset, dt.itemsize, C.byref(rec))
        if rc != 0:
            raise BlobError({-1: "truncated header", -2: "bad magic", -3: "too many dimensions",
                             -4: "truncated data"}.get(rc, f"error {rc}") + f" at offset {offset}")
        dims = tuple(int(rec.dims[i]) for i in range(rec.ndim))
        data = np.frombuffer(buf, dtype=dt, count=int(rec.num_elems), offset=int(rec.data_offset)).copy()
        out.append((data, dims, (int(rec.tag[0]), int(rec.tag[1]))))
        offset = int(rec.next_offset)
    return out, offset


def encode_many(records: Iterable[Tuple[object, Sequence[int]]], dtype="f32") -> bytes:
    return b"".join(encode_record(d, dims, dtype) for d, dims in records)


def read_array_file(path: str, dtype="f32") -> np.ndarray:
    """First record of a file as an array shaped with numpy order reversed (so arr[c][h][w] for (W,H,C))."""
    with open(path, "rb") as f:
        buf = f.read()
    recs, _ = decode_records(buf, dtype, count=1)
    data, dims, _ = recs[0]
    return data.reshape(tuple(reversed(dims)))


def write_array_file(path: str, arr: np.ndarray, dtype="f32") -> None:
    """Write `arr` (numpy C order, e.g. [c][h][w]) as one record with dims (w,h,c)."""
    a = np.asarray(arr)
    with open(path, "wb") as f:
        f.write(encode_record(a.reshape(-1), tuple(reversed(a.shape)), dtype))
