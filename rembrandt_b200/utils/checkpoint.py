"""Checkpoint directory layout and resume, as the reference's distributed worker writes it
(src/worker/gossip_dist.rs:1230-1413):

* ``params.t_{t}.blob``      concatenated NdArray records of every hidden operator's parameters (rank 0 only);
* ``params.latest.blob``     symlink to the newest parameter blob;
* ``checkpoint``             text file whose first line is ``t``; ``checkpoint.0`` is the previous copy;
* ``state.latest.blob.{rank}``  per-rank optimizer state: per operator its parameters then its momentum buffers.

gen-2 names (``layer_params.t_{t}.blob`` / ``layer_params.latest.blob``, src/arch_new.rs:472-509) and the gen-1
binary ``checkpoint`` (u64 little-endian ``t``, src/net.rs:158-160) are readable too.
"""
from __future__ import annotations

import os
import shutil
import struct
from typing import Optional


def _atomic_write(path: str, data: bytes) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def checkpoint_params(net, t: int, directory: str, prefix: str = "params") -> str:
    """Write the parameter blob for iteration `t`, refresh the `latest` link and the checkpoint index."""
    os.makedirs(directory, exist_ok=True)
    name = f"{prefix}.t_{t}.blob"
    path = os.path.join(directory, name)
    _atomic_write(path, net.encode_params())
    latest = os.path.join(directory, f"{prefix}.latest.blob")
    tmp_link = latest + ".tmp"
    if os.path.lexists(tmp_link):
        os.remove(tmp_link)
    os.symlink(name, tmp_link)
    os.replace(tmp_link, latest)
    index = os.path.join(directory, "checkpoint")
    if os.path.exists(index):
        shutil.copyfile(index, index + ".0")
    _atomic_write(index, f"{t}\n".encode())
    return path


def checkpoint_state(net, directory: str, rank: int = 0, name: str = "state.latest.blob") -> str:
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, f"{name}.{rank}")
    _atomic_write(path, net.encode_state())
    return path


def latest_iteration(directory: str) -> Optional[int]:
    """First line of `checkpoint` (falls back to `checkpoint.0`, then to the gen-1 binary form)."""
    for name in ("checkpoint", "checkpoint.0"):
        path = os.path.join(directory, name)
        if not os.path.exists(path):
            continue
        raw = open(path, "rb").read()
        try:
            return int(raw.decode().splitlines()[0].strip())
        except (UnicodeDecodeError, ValueError, IndexError):
            if len(raw) == 8:
                return struct.unpack("<Q", raw)[0]
    return None


def can_rollback(directory: Optional[str], rank: int = 0) -> Optional[int]:
    """Iteration a run can resume from: needs the index and this rank's state blob."""
    if not directory or not os.path.isdir(directory):
        return None
    t = latest_iteration(directory)
    if t is None:
        return None
    if not os.path.exists(os.path.join(directory, f"state.latest.blob.{rank}")):
        return None
    return t


def rollback_state(net, directory: str, rank: int = 0) -> None:
    with open(os.path.join(directory, f"state.latest.blob.{rank}"), "rb") as f:
        net.decode_state(f.read())


def rollback_params(net, directory: str, t: Optional[int] = None, prefix: str = "params") -> int:
    """Load `params.t_{t}.blob` (latest when `t` is None); `t` must not exceed the recorded latest iteration."""
    latest = latest_iteration(directory)
    if t is None:
        t = latest
    if t is None:
        raise FileNotFoundError(f"no checkpoint index in {directory}")
    if latest is not None and t > latest:
        raise ValueError(f"requested iteration {t} is newer than the latest checkpoint {latest}")
    for pre in (prefix, "layer_params"):
        path = os.path.join(directory, f"{pre}.t_{t}.blob")
        if os.path.exists(path):
            with open(path, "rb") as f:
                net.decode_params(f.read())
            return t
    raise FileNotFoundError(f"no parameter blob for iteration {t} in {directory}")


def reshape_conv_out_channels(blob_bytes: bytes, op_index_to_channels: dict) -> bytes:
    """Offline blob surgery: keep only the first `k` output channels of the listed parameter records (and of the
    bias that follows each), the equivalent of the reference's ``reshape_params`` (src/arch_new.rs:92-172).
    Keys are record indices of weight arrays within the blob."""
    from . import blob
    recs, _ = blob.decode_records(blob_bytes, "f32")
    out = []
    i = 0
    while i < len(recs):
        data, dims, tag = recs[i]
        if i in op_index_to_channels:
            k = op_index_to_channels[i]
            rows, cols = dims          # (fan_in, out_channels), first dimension fastest
            w = data.reshape(cols, rows)[:k]
            out.append(blob.encode_record(w.reshape(-1), (rows, k), tag=tag))
            bdata, bdims, btag = recs[i + 1]
            out.append(blob.encode_record(bdata[:k], (1, k), tag=btag))
            i += 2
            continue
        out.append(blob.encode_record(data, dims, tag=tag))
        i += 1
    return b"".join(out)
