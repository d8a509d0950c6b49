"""Read-only access to LMDB environments (the Caffe image databases the reference reads through its `lmdb`
bindings: src/data/lmdb_data.rs:50-152, src/data_new.rs:885-997), with no dependency on liblmdb.

Two implementations of the same reader: the C++ cursor in csrc/host/lmdb_reader.cc (`NativeLmdbEnv`, what
`open_env` returns) and the pure-Python `LmdbEnv` below (the executable description of the format, and the
cross-check in the tests).

Only what a reader needs is implemented: the newer of the two meta pages, the main database's B+tree (branch and
leaf pages, overflow pages for large values), ordered iteration, `get` and cursor `seek` (first key >= a given key).
Sub-databases, duplicate-sorted databases and writing real environments are out of scope; `write_env` produces a
small well-formed environment (one B+tree built bottom-up, values on overflow pages when they do not fit) so that
the reader can be tested without liblmdb.

On-disk layout (little endian, 64-bit, LMDB format version 1):
  page header   pgno u64 | pad u16 | flags u16 | lower u16, upper u16  (overflow pages: page count u32 instead)
  meta page     header | magic 0xBEEFC0DE u32 | version u32 | address u64 | mapsize u64 | 2 x db record (48 B:
                pad u32 [page size in the first record], flags u16, depth u16, branch pages, leaf pages, overflow
                pages, entries, root, all u64) | last page u64 | txn id u64
  node          lo u16 | hi u16 | flags u16 | key size u16 | key | data
                branch: child page = lo | hi << 16 | flags << 32;  leaf: data size = lo | hi << 16, flag 0x01 =
                the data is the u64 number of an overflow page whose payload starts 16 bytes in
"""
from __future__ import annotations

import mmap
import os
import struct
from typing import Iterator, List, Optional, Tuple

from ..utils.rng import partition_range

MAGIC = 0xBEEFC0DE
P_BRANCH, P_LEAF, P_OVERFLOW, P_META = 0x01, 0x02, 0x04, 0x08
F_BIGDATA = 0x01
PAGEHDR = 16
INVALID = 0xFFFFFFFFFFFFFFFF


class LmdbError(ValueError):
    pass


class LmdbEnv:
    """One LMDB environment opened read-only (`path` is the directory holding data.mdb, or the file itself)."""

    def __init__(self, path: str):
        if os.path.isdir(path):
            path = os.path.join(path, "data.mdb")
        self._f = open(path, "rb")
        self._m = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        metas = []
        for pg in (0, 1):
            meta = self._read_meta(pg * self._guess_psize())
            if meta is not None:
                metas.append(meta)
        if not metas:
            raise LmdbError("no valid LMDB meta page")
        self.meta = max(metas, key=lambda m: m["txnid"])
        self.psize = self.meta["psize"]
        self.entries = self.meta["entries"]
        self.root = self.meta["root"]
        self.depth = self.meta["depth"]

    def close(self):
        self._m.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- pages
    def _guess_psize(self) -> int:
        # the page size is stored in the first db record of meta page 0 (which always sits at offset 0)
        magic, = struct.unpack_from("<I", self._m, PAGEHDR)
        if magic != MAGIC:
            raise LmdbError("not an LMDB data file")
        psize, = struct.unpack_from("<I", self._m, PAGEHDR + 24)
        if psize < 512 or psize & (psize - 1):
            raise LmdbError(f"implausible page size {psize}")
        return psize

    def _read_meta(self, off: int) -> Optional[dict]:
        if off + PAGEHDR + 136 > len(self._m):
            return None
        magic, version = struct.unpack_from("<II", self._m, off + PAGEHDR)
        if magic != MAGIC or version != 1:
            return None
        psize, = struct.unpack_from("<I", self._m, off + PAGEHDR + 24)
        main = off + PAGEHDR + 24 + 48
        _pad, flags, depth, branch, leaf, overflow, entries, root = struct.unpack_from("<IHHQQQQQ", self._m, main)
        last_pg, txnid = struct.unpack_from("<QQ", self._m, main + 48)
        return {"psize": psize, "flags": flags, "depth": depth, "entries": entries, "root": root, "last_pg": last_pg,
                "txnid": txnid}

    def _page(self, pgno: int) -> Tuple[int, int, List[int]]:
        """(offset, flags, node offsets) of a branch or leaf page."""
        off = pgno * self.psize
        if off + PAGEHDR > len(self._m):
            raise LmdbError(f"page {pgno} lies outside the file")
        _pg, _pad, flags, lower, _upper = struct.unpack_from("<QHHHH", self._m, off)
        n = (lower - PAGEHDR) // 2
        ptrs = list(struct.unpack_from(f"<{n}H", self._m, off + PAGEHDR)) if n > 0 else []
        return off, flags, ptrs

    def _node(self, page_off: int, ptr: int):
        lo, hi, flags, ksize = struct.unpack_from("<HHHH", self._m, page_off + ptr)
        kstart = page_off + ptr + 8
        return lo, hi, flags, bytes(self._m[kstart: kstart + ksize]), kstart + ksize

    def _leaf_value(self, lo, hi, flags, dstart) -> bytes:
        size = lo | (hi << 16)
        if flags & F_BIGDATA:
            opg, = struct.unpack_from("<Q", self._m, dstart)
            start = opg * self.psize + PAGEHDR
            return bytes(self._m[start: start + size])
        return bytes(self._m[dstart: dstart + size])

    # ---- traversal
    def _descend(self, key: Optional[bytes]):
        """Stack of (page offset, node offsets, index) leading to the leaf where `key` would be (leftmost leaf
        for None)."""
        if self.root == INVALID or self.entries == 0:
            return None
        stack = []
        pgno = self.root
        while True:
            off, flags, ptrs = self._page(pgno)
            if flags & P_LEAF:
                stack.append([off, ptrs, 0])
                return stack
            if not flags & P_BRANCH:
                raise LmdbError(f"unexpected page flags {flags:#x} in the tree")
            # branch: node 0 has an empty key and covers everything below node 1's key
            idx = 0
            if key is not None:
                lo_i, hi_i = 1, len(ptrs) - 1
                while lo_i <= hi_i:
                    mid = (lo_i + hi_i) // 2
                    k = self._node(off, ptrs[mid])[3]
                    if k <= key:
                        idx = mid
                        lo_i = mid + 1
                    else:
                        hi_i = mid - 1
            stack.append([off, ptrs, idx])
            lo, hi, fl, _k, _d = self._node(off, ptrs[idx])
            pgno = lo | (hi << 16) | (fl << 32)

    def _advance(self, stack) -> bool:
        """Move the stack to the next leaf; False at the end of the tree."""
        stack.pop()
        while stack:
            off, ptrs, idx = stack[-1]
            if idx + 1 < len(ptrs):
                stack[-1][2] = idx + 1
                lo, hi, fl, _k, _d = self._node(off, ptrs[idx + 1])
                pgno = lo | (hi << 16) | (fl << 32)
                while True:
                    o2, f2, p2 = self._page(pgno)
                    stack.append([o2, p2, 0])
                    if f2 & P_LEAF:
                        return True
                    lo, hi, fl, _k, _d = self._node(o2, p2[0])
                    pgno = lo | (hi << 16) | (fl << 32)
            stack.pop()
        return False

    def items(self, start: Optional[bytes] = None) -> Iterator[Tuple[bytes, bytes]]:
        """(key, value) pairs in key order, from the first key >= `start` (a cursor seek) or from the beginning."""
        stack = self._descend(start)
        if stack is None:
            return
        while True:
            off, ptrs, _ = stack[-1]
            for ptr in ptrs:
                lo, hi, fl, k, d = self._node(off, ptr)
                if start is not None and k < start:
                    continue
                yield k, self._leaf_value(lo, hi, fl, d)
            if not self._advance(stack):
                return

    def get(self, key: bytes) -> Optional[bytes]:
        for k, v in self.items(key):
            return v if k == key else None
        return None

    def __len__(self):
        return self.entries


class NativeLmdbEnv:
    """The same interface as `LmdbEnv` over the C++ reader (memory-mapped file, cursor in native code)."""

    def __init__(self, path: str):
        import ctypes as C
        from .. import _native
        self._C = C
        self._lib = _native.host()
        self._h = self._lib.rb_lmdb_open(os.fsencode(path))
        if not self._h:
            raise LmdbError(f"{path}: not a readable LMDB environment")
        self.entries = int(self._lib.rb_lmdb_entries(self._h))
        self.depth = int(self._lib.rb_lmdb_depth(self._h))
        self.psize = int(self._lib.rb_lmdb_page_size(self._h))

    def close(self):
        if self._h:
            self._lib.rb_lmdb_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return self.entries

    def items(self, start: Optional[bytes] = None) -> Iterator[Tuple[bytes, bytes]]:
        C = self._C
        key = start or b""
        if not self._lib.rb_lmdb_seek(self._h, key, len(key)):
            return
        kp, vp_ = C.c_void_p(), C.c_void_p()
        kl, vl = C.c_uint32(), C.c_uint64()
        while self._lib.rb_lmdb_next(self._h, C.byref(kp), C.byref(kl), C.byref(vp_), C.byref(vl)):
            yield C.string_at(kp.value, kl.value), C.string_at(vp_.value, vl.value)

    def get(self, key: bytes) -> Optional[bytes]:
        for k, v in self.items(key):
            return v if k == key else None
        return None


def open_env(path: str):
    """The native reader when the host library is available, else the Python one."""
    try:
        return NativeLmdbEnv(path)
    except (OSError, AttributeError):
        return LmdbEnv(path)


class LmdbCaffeShard:
    """The part [lo, hi) of a Caffe image database that belongs to worker `rank` of `world`: records are decoded
    from `Datum` messages; the cursor is positioned with a seek on the zero-padded record number, as the reference
    does (src/data/lmdb_data.rs:50-152: keys "{:08}...")."""

    def __init__(self, path: str, rank: int = 0, world: int = 1, codec=None):
        from .codecs import decode_caffe_datum
        self.env = open_env(path)
        self.lo, self.hi = partition_range(len(self.env), world, rank)
        self._decode = decode_caffe_datum
        self.codec = codec

    def __len__(self):
        return self.hi - self.lo

    def __iter__(self):
        """Yields (uint8 array [C, H, W], label)."""
        import numpy as np
        start = b"%08d" % self.lo
        n = 0
        for _k, v in self.env.items(start):
            if n >= len(self):
                return
            d = self._decode(v)
            if d.get("encoded") and self.codec is not None:
                img = self.codec.decode(d["data"])
            else:
                img = np.frombuffer(d["data"], dtype=np.uint8).reshape(d["channels"], d["height"], d["width"])
            yield img, int(d.get("label", 0))
            n += 1


# ------------------------------------------------------------------------------------------------ test writer
def write_env(path: str, items, psize: int = 4096, max_leaf_nodes: int = 0):
    """Write a small well-formed environment holding `items` ((key, value) byte pairs; sorted here). Values that do
    not fit in a quarter of a page go to overflow pages. `max_leaf_nodes` caps the nodes per page (forces depth)."""
    items = sorted(items)
    pages = {}          # pgno -> bytes
    next_pg = [2]

    def alloc(n=1):
        pg = next_pg[0]
        next_pg[0] += n
        return pg

    def build_page(pgno, flags, nodes):
        """nodes: list of raw node bytes; laid out from the end of the page downwards, pointers upwards."""
        buf = bytearray(psize)
        upper = psize
        ptrs = []
        for nd in nodes:
            size = (len(nd) + 1) & ~1
            upper -= size
            buf[upper: upper + len(nd)] = nd
            ptrs.append(upper)
        lower = PAGEHDR + 2 * len(ptrs)
        if lower > upper:
            raise LmdbError("nodes do not fit in the page")
        struct.pack_into("<QHHHH", buf, 0, pgno, 0, flags, lower, upper)
        struct.pack_into(f"<{len(ptrs)}H", buf, PAGEHDR, *ptrs)
        pages[pgno] = bytes(buf)

    overflow_pages = 0
    leaf_nodes = []
    for k, v in items:
        if len(v) > psize // 4:
            n = (PAGEHDR + len(v) + psize - 1) // psize
            opg = alloc(n)
            buf = bytearray(n * psize)
            struct.pack_into("<QHHI", buf, 0, opg, 0, P_OVERFLOW, n)
            buf[PAGEHDR: PAGEHDR + len(v)] = v
            for i in range(n):
                pages[opg + i] = bytes(buf[i * psize: (i + 1) * psize])
            overflow_pages += n
            node = struct.pack("<HHHH", len(v) & 0xFFFF, len(v) >> 16, F_BIGDATA, len(k)) + k + struct.pack("<Q", opg)
        else:
            node = struct.pack("<HHHH", len(v) & 0xFFFF, len(v) >> 16, 0, len(k)) + k + v
        leaf_nodes.append((k, node))

    def pack_level(entries, flags):
        """entries: (first key, node bytes). Returns [(first key of page, pgno)]."""
        out, cur, used = [], [], PAGEHDR
        for k, nd in entries:
            need = ((len(nd) + 1) & ~1) + 2
            if cur and (used + need > psize or (max_leaf_nodes and len(cur) >= max_leaf_nodes)):
                pg = alloc()
                build_page(pg, flags, [n for _, n in cur])
                out.append((cur[0][0], pg))
                cur, used = [], PAGEHDR
            cur.append((k, nd))
            used += need
        if cur:
            pg = alloc()
            build_page(pg, flags, [n for _, n in cur])
            out.append((cur[0][0], pg))
        return out

    depth, leaf_count, branch_count = 0, 0, 0
    root = INVALID
    if leaf_nodes:
        level = pack_level(leaf_nodes, P_LEAF)
        leaf_count = len(level)
        depth = 1
        while len(level) > 1:
            entries = []
            for i, (k, pg) in enumerate(level):
                key = b"" if i == 0 else k
                entries.append((k, struct.pack("<HHHH", pg & 0xFFFF, (pg >> 16) & 0xFFFF, pg >> 32, len(key)) + key))
            # the first node of every branch page carries an empty key
            level2 = []
            cur, used = [], PAGEHDR
            groups = []
            for k, nd in entries:
                need = ((len(nd) + 1) & ~1) + 2
                if cur and (used + need > psize or (max_leaf_nodes and len(cur) >= max_leaf_nodes)):
                    groups.append(cur)
                    cur, used = [], PAGEHDR
                cur.append((k, nd))
                used += need
            if cur:
                groups.append(cur)
            for grp in groups:
                first_key, first_node = grp[0]
                pg_lo, pg_hi, pg_fl, _ks = struct.unpack_from("<HHHH", first_node)
                nodes = [struct.pack("<HHHH", pg_lo, pg_hi, pg_fl, 0)] + [n for _, n in grp[1:]]
                pg = alloc()
                build_page(pg, P_BRANCH, nodes)
                level2.append((first_key, pg))
                branch_count += 1
            level = level2
            depth += 1
        root = level[0][1]

    last_pg = next_pg[0] - 1
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "data.mdb"), "wb") as f:
        for pg in (0, 1):
            buf = bytearray(psize)
            struct.pack_into("<QHHHH", buf, 0, pg, 0, P_META, 0, 0)
            struct.pack_into("<IIQQ", buf, PAGEHDR, MAGIC, 1, 0, 1 << 30)
            struct.pack_into("<IHHQQQQQ", buf, PAGEHDR + 24, psize, 0, 0, 0, 0, 0, 0, INVALID)
            struct.pack_into("<IHHQQQQQ", buf, PAGEHDR + 72, 0, 0, depth, branch_count, leaf_count, overflow_pages,
                             len(items), root)
            struct.pack_into("<QQ", buf, PAGEHDR + 120, last_pg, pg)   # txn ids 0 and 1: page 1 is the newer
            f.write(buf)
        for pg in range(2, last_pg + 1):
            f.write(pages.get(pg, bytes(psize)))
