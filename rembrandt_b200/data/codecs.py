"""Sample codecs and host-side augmentation (src/data/codec.rs, src/data/augment.rs, src/caffe_proto.proto).

* ``Array3dDataCodec``   NdArray record -> uint8 array;
* ``Bits3dCodec`` / ``BitsThenBytes3dCodec``  bit-plane samples (Go boards): packed bits expanded to 0 / `scale`,
                         optionally followed by byte planes (SampleDatumConfig::{Bits3d, BitsThenBytes3d},
                         src/data_new.rs:22-66);
* ``FakeJpegDataCodec``  returns a zero 256x256x3 image whatever the bytes (the reference's fake for I/O tests);
* ``JpegDataCodec``      real decode through Pillow when it is installed (the reference uses turbojpeg with an
                         stb fallback), grey -> RGB, HWC -> planar;
* ``decode_caffe_datum`` hand-written reader of the Caffe ``Datum`` protobuf message (fields 1-7);
* host preprocs: transpose CWH <-> WHC, random / centre crop, random flip.
"""
from __future__ import annotations

import io
from typing import Optional, Tuple

import numpy as np

from ..utils import blob


class Array3dDataCodec:
    def decode(self, value: bytes) -> np.ndarray:
        recs, _ = blob.decode_records(value, "u8", count=1)
        data, dims, _ = recs[0]
        return data.reshape(tuple(reversed(dims)))


BITS_TAG = (0x42, 0x01)   # 'B': the payload of this record is packed bits


def encode_bits3d(planes) -> bytes:
    """Pack a {0,1}-valued [C, H, W] array into a bit record: the NdArray header with dims (W, H, C) and tag 'B',
    then ceil(W*H*C / 8) bytes, element i (first dimension fastest) in bit i % 8 of byte i // 8.

    The reference's BitArray3d comes from a crate outside its tree, so its byte layout is not known; this layout
    is this framework's own."""
    a = np.ascontiguousarray(np.asarray(planes) != 0)
    c, h, w = a.shape
    packed = np.packbits(a.reshape(-1), bitorder="little")
    return b"ND" + bytes(BITS_TAG) + np.uint32(3).tobytes() + np.asarray([w, h, c], dtype="<u8").tobytes() + packed.tobytes()


def _decode_bits3d(value: bytes, offset: int, scale: int):
    if value[offset:offset + 2] != b"ND" or tuple(value[offset + 2:offset + 4]) != BITS_TAG:
        raise blob.BlobError(f"no bit record at offset {offset}")
    if int(np.frombuffer(value, "<u4", 1, offset + 4)[0]) != 3:
        raise blob.BlobError("bit records are three-dimensional")
    w, h, c = (int(v) for v in np.frombuffer(value, "<u8", 3, offset + 8))
    n = w * h * c
    nbytes = (n + 7) // 8
    start = offset + 32
    if start + nbytes > len(value):
        raise blob.BlobError("truncated bit record")
    from .. import _native
    out = np.empty(n, dtype=np.uint8)
    packed = np.frombuffer(value, np.uint8, nbytes, start)
    if n and _native.host().rb_bits_unpack(packed.ctypes.data, nbytes, n, int(scale) & 0xFF, out.ctypes.data) != 0:
        raise blob.BlobError("truncated bit record")
    return out.reshape(c, h, w), start + nbytes


class Bits3dCodec:
    """Bit planes -> uint8 [C, H, W] holding 0 or `scale`."""

    def __init__(self, scale: int = 255):
        self.scale = scale

    def decode(self, value: bytes) -> np.ndarray:
        return _decode_bits3d(value, 0, self.scale)[0]


class BitsThenBytes3dCodec:
    """A bit record followed by a byte record of the same width and height: channels are concatenated, bit planes
    first (a Go position: stone / liberty planes as bits, then a few byte-valued feature planes)."""

    def __init__(self, scale: int = 255):
        self.scale = scale

    def decode(self, value: bytes) -> np.ndarray:
        bits, off = _decode_bits3d(value, 0, self.scale)
        recs, _ = blob.decode_records(value, "u8", offset=off, count=1)
        data, dims, _ = recs[0]
        planes = data.reshape(tuple(reversed(dims)))
        if planes.shape[1:] != bits.shape[1:]:
            raise blob.BlobError(f"bit planes {bits.shape} and byte planes {planes.shape} differ in size")
        return np.concatenate([bits, planes], axis=0)

    @staticmethod
    def encode(bit_planes, byte_planes) -> bytes:
        b = np.ascontiguousarray(np.asarray(byte_planes, dtype=np.uint8))
        c, h, w = b.shape
        return encode_bits3d(bit_planes) + blob.encode_record(b.reshape(-1), (w, h, c), "u8")


class FakeJpegDataCodec:
    def decode(self, value: bytes) -> np.ndarray:
        return np.zeros((3, 256, 256), dtype=np.uint8)


class JpegDataCodec:
    def __init__(self):
        try:
            from PIL import Image  # noqa: F401
            self._ok = True
        except ImportError:
            self._ok = False

    def decode(self, value: bytes) -> np.ndarray:
        if not self._ok:
            raise RuntimeError("no JPEG decoder available (Pillow is not installed)")
        from PIL import Image
        img = Image.open(io.BytesIO(value)).convert("RGB")
        return np.ascontiguousarray(np.asarray(img, dtype=np.uint8).transpose(2, 0, 1))


def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    out, shift = 0, 0
    while True:
        b = buf[pos]
        pos += 1
        out |= (b & 0x7F) << shift
        if not b & 0x80:
            return out, pos
        shift += 7


def decode_caffe_datum(buf: bytes) -> dict:
    """Fields: 1 channels, 2 height, 3 width, 4 data (bytes), 5 label, 6 float_data (repeated), 7 encoded.
    Parsed by the C++ runtime (csrc/host/sample_codecs.cc); `decode_caffe_datum_py` is the same reader in Python,
    kept as its cross-check."""
    import ctypes as C_
    from .. import _native
    lib = _native.host()
    d = _native.Datum()
    raw = np.frombuffer(buf, dtype=np.uint8)
    rc = lib.rb_datum_parse(raw.ctypes.data if len(buf) else None, len(buf), C_.byref(d))
    if rc != 0:
        raise ValueError({-1: "truncated varint", -2: "a field runs past the end of the message",
                          -3: "packed float_data of odd size", -4: "unsupported wire type"}.get(rc, f"error {rc}"))
    floats = []
    if d.float_count:
        arr = np.empty(int(d.float_count), dtype="<f4")
        n = lib.rb_datum_floats(raw.ctypes.data, len(buf), arr.ctypes.data, int(d.float_count))
        floats = arr[: int(n)].tolist()
    return {"channels": d.channels, "height": d.height, "width": d.width,
            "data": bytes(buf[d.data_offset: d.data_offset + d.data_len]), "label": d.label, "float_data": floats,
            "encoded": bool(d.encoded)}


def decode_caffe_datum_py(buf: bytes) -> dict:
    out = {"channels": 0, "height": 0, "width": 0, "data": b"", "label": 0, "float_data": [], "encoded": False}
    names = {1: "channels", 2: "height", 3: "width", 5: "label"}
    pos = 0
    while pos < len(buf):
        key, pos = _varint(buf, pos)
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, pos = _varint(buf, pos)
            if field in names:
                out[names[field]] = v
            elif field == 7:
                out["encoded"] = bool(v)
        elif wire == 2:
            n, pos = _varint(buf, pos)
            chunk = buf[pos:pos + n]
            pos += n
            if field == 4:
                out["data"] = bytes(chunk)
            elif field == 6:
                out["float_data"].extend(np.frombuffer(chunk, dtype="<f4").tolist())
        elif wire == 5:
            if field == 6:
                out["float_data"].append(float(np.frombuffer(buf[pos:pos + 4], dtype="<f4")[0]))
            pos += 4
        elif wire == 1:
            pos += 8
        else:
            raise ValueError(f"unsupported wire type {wire}")
    return out


def datum_to_sample(d: dict, jpeg: Optional[JpegDataCodec] = None):
    if d["encoded"]:
        return (jpeg or JpegDataCodec()).decode(d["data"]), d["label"]
    arr = np.frombuffer(d["data"], dtype=np.uint8).reshape(d["channels"], d["height"], d["width"])
    return arr, d["label"]


# ---- host-side preprocessing (the GPU input kernel is the fast path; these serve CPU pipelines)
def transpose_cwh_to_whc(img_chw: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(img_chw.transpose(1, 2, 0))


def transpose_whc_to_cwh(img_hwc: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(img_hwc.transpose(2, 0, 1))


class RandomCropPreproc:
    def __init__(self, crop_w, crop_h, seed=0):
        self.cw, self.ch, self.rng = crop_w, crop_h, np.random.default_rng(seed)

    def __call__(self, sample):
        img, label = sample
        _, h, w = img.shape
        oy, ox = int(self.rng.integers(0, h - self.ch + 1)), int(self.rng.integers(0, w - self.cw + 1))
        return img[:, oy:oy + self.ch, ox:ox + self.cw], label


class CenterCropPreproc:
    def __init__(self, crop_w, crop_h):
        self.cw, self.ch = crop_w, crop_h

    def __call__(self, sample):
        img, label = sample
        _, h, w = img.shape
        oy, ox = (h - self.ch) // 2, (w - self.cw) // 2
        return img[:, oy:oy + self.ch, ox:ox + self.cw], label


class RandomFlipXPreproc:
    def __init__(self, seed=0):
        self.rng = np.random.default_rng(seed)

    def __call__(self, sample):
        img, label = sample
        return (img[:, :, ::-1] if self.rng.integers(0, 2) else img), label


def encode_caffe_datum(data: bytes, channels: int, height: int, width: int, label: int = 0, encoded: bool = False) -> bytes:
    """Serialise a Caffe ``Datum`` (fields 1-5 and 7); the inverse of `decode_caffe_datum` for tools and tests."""
    def varint(v):
        out = bytearray()
        while True:
            b = v & 0x7F
            v >>= 7
            out.append(b | (0x80 if v else 0))
            if not v:
                return bytes(out)
    msg = bytearray()
    for field, v in ((1, channels), (2, height), (3, width)):
        msg += varint(field << 3) + varint(v)
    msg += varint((4 << 3) | 2) + varint(len(data)) + data
    msg += varint(5 << 3) + varint(label)
    if encoded:
        msg += varint(7 << 3) + varint(1)
    return bytes(msg)
