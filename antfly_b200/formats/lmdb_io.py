"""LMDB environments without the LMDB library: a read-only tree walker and a bulk writer.

The reference keeps an HBC index in an LMDB environment with one named database per namespace (``hbc_nodes``,
``hbc_meta``, ``hbc_quant``, ``hbc_vecs``: zig/pkg/antfly/src/storage/hbc_adapter.zig:1435-1438,
storage/lmdb_backend.zig:29-47; the library is the stock one, zig/lib/lmdb).  To open such an index, and to hand
one back, only the file format is needed (64-bit little-endian builds, format version 1):

* ``data.mdb`` is an array of pages (size in the meta page, 4096 by default).  Every page starts with a 16-byte
  header {page number u64, pad u16, flags u16, lower u16, upper u16}; an overflow page reuses lower / upper as a
  u32 page count.  Flags: 0x01 branch, 0x02 leaf, 0x04 overflow, 0x08 meta.
* Pages 0 and 1 are meta pages: after the header {magic 0xBEEFC0DE u32, version u32, address u64, map size u64,
  two 48-byte database records (free list, main), last page u64, transaction id u64}; the meta page with the larger
  transaction id is current.  A database record is {pad u32 (the page size, in the free-list record), flags u16,
  depth u16, branch pages u64, leaf pages u64, overflow pages u64, entries u64, root page u64 (all ones = empty)}.
* A branch or leaf page holds u16 node offsets from byte 16 up to ``lower`` (sorted by key) and the nodes packed
  downwards from the page end to ``upper``.  A node is {lo u16, hi u16, flags u16, key size u16, key, data}: in a
  branch page lo | hi << 16 | flags << 32 is the child page (the first node's key is empty); in a leaf page
  lo | hi << 16 is the data size, flag 0x01 means the data is a u64 overflow page number (the value starts 16 bytes
  into that page and may span several), flag 0x02 means the data is the 48-byte record of a named database.
* Named databases are entries of the main database keyed by name.

Keys compare as byte strings (no custom comparators, no duplicate-sorted databases: the reference uses neither).
"""
from __future__ import annotations

import functools
import inspect
import mmap
import os
import struct
from typing import Dict, Iterator, List, Optional, Tuple

MAGIC, VERSION = 0xBEEFC0DE, 1
P_BRANCH, P_LEAF, P_OVERFLOW, P_META = 0x01, 0x02, 0x04, 0x08
F_BIGDATA, F_SUBDATA, F_DUPDATA = 0x01, 0x02, 0x04
HDR = 16
NODE = 8
INVALID = 0xFFFFFFFFFFFFFFFF
_DB = struct.Struct("<IHHQQQQQ")          # pad, flags, depth, branch, leaf, overflow, entries, root
_META = struct.Struct("<IIQQ")            # magic, version, address, map size
assert _DB.size == 48


class LmdbError(ValueError):
    pass


_BROKEN = (struct.error, IndexError, OverflowError, UnicodeDecodeError)


def _refuses(fn):
    """Reads that run off a damaged file surface as :class:`LmdbError`, whatever the low-level failure was."""
    if inspect.isgeneratorfunction(fn):
        @functools.wraps(fn)
        def gen(*a, **k):
            try:
                yield from fn(*a, **k)
            except _BROKEN as e:
                raise LmdbError(f"damaged LMDB file: {e}") from e
        return gen

    @functools.wraps(fn)
    def call(*a, **k):
        try:
            return fn(*a, **k)
        except _BROKEN as e:
            raise LmdbError(f"damaged LMDB file: {e}") from e
    return call


class LmdbReader:
    """Read-only view of an LMDB environment (a directory holding ``data.mdb``, or the file itself)."""

    @_refuses
    def __init__(self, path: str):
        if os.path.isdir(path):
            path = os.path.join(path, "data.mdb")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        metas = []
        for pg in (0, 1):
            off = self._meta_offset(pg)
            if off is None:
                continue
            magic, version, _, _ = _META.unpack_from(self._mm, off)
            if magic != MAGIC or version != VERSION:
                continue
            free = _DB.unpack_from(self._mm, off + _META.size)
            main = _DB.unpack_from(self._mm, off + _META.size + _DB.size)
            last_pg, txnid = struct.unpack_from("<QQ", self._mm, off + _META.size + 2 * _DB.size)
            metas.append((txnid, free[0], main, last_pg))
        if not metas:
            raise LmdbError("not an LMDB data file (no valid meta page)")
        self.txnid, self.page_size, self._main, self.last_page = max(metas, key=lambda m: m[0])
        if self.page_size < 512 or self.page_size & (self.page_size - 1):
            raise LmdbError(f"implausible page size {self.page_size}")

    def _meta_offset(self, pg: int) -> Optional[int]:
        # the page size is not known before a meta page is read: page 1 is tried at every power of two
        if pg == 0:
            return HDR if len(self._mm) >= HDR + 136 else None
        for shift in range(9, 17):
            off = (1 << shift) + HDR
            if off + 136 <= len(self._mm):
                flags = struct.unpack_from("<H", self._mm, (1 << shift) + 10)[0]
                magic = struct.unpack_from("<I", self._mm, off)[0]
                if flags & P_META and magic == MAGIC:
                    return off
        return None

    def close(self) -> None:
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- pages -----------------------------------------------------------------------------------------------
    def _page(self, pgno: int) -> Tuple[int, int, int, int]:
        off = pgno * self.page_size
        if pgno > self.last_page or off + HDR > len(self._mm):
            raise LmdbError(f"page {pgno} is outside the file")
        _, _, flags, lower, upper = struct.unpack_from("<QHHHH", self._mm, off)
        return off, flags, lower, upper

    def _nodes(self, pgno: int):
        off, flags, lower, upper = self._page(pgno)
        if not flags & (P_BRANCH | P_LEAF) or lower < HDR or lower > self.page_size or (lower - HDR) % 2:
            raise LmdbError(f"page {pgno} is not a tree page (flags {flags:#x}, lower {lower})")
        for i in range((lower - HDR) // 2):
            ptr = struct.unpack_from("<H", self._mm, off + HDR + 2 * i)[0]
            if ptr < upper or ptr + NODE > self.page_size:
                raise LmdbError(f"page {pgno}: node offset {ptr} out of range")
            lo, hi, nflags, ksize = struct.unpack_from("<HHHH", self._mm, off + ptr)
            yield flags, off + ptr, lo, hi, nflags, ksize

    def _value(self, node_off: int, lo: int, hi: int, nflags: int, ksize: int) -> bytes:
        size = lo | (hi << 16)
        data = node_off + NODE + ksize
        if nflags & F_BIGDATA:
            ov = struct.unpack_from("<Q", self._mm, data)[0]
            off, flags, _, _ = self._page(ov)
            if not flags & P_OVERFLOW:
                raise LmdbError(f"page {ov} is not an overflow page")
            if off + HDR + size > len(self._mm):
                raise LmdbError("overflow value runs past the file")
            return bytes(self._mm[off + HDR: off + HDR + size])
        if data + size > len(self._mm):
            raise LmdbError("value runs past the file")
        return bytes(self._mm[data: data + size])

    def _walk(self, root: int, depth: int = 0) -> Iterator[Tuple[bytes, bytes, int]]:
        if root == INVALID:
            return
        if depth > 64:
            raise LmdbError("tree deeper than 64 levels (a page cycle)")
        for flags, noff, lo, hi, nflags, ksize in self._nodes(root):
            if flags & P_BRANCH:
                yield from self._walk(lo | (hi << 16) | (nflags << 32), depth + 1)
            else:
                if nflags & F_DUPDATA:
                    raise LmdbError("duplicate-sorted databases are not supported")
                key = bytes(self._mm[noff + NODE: noff + NODE + ksize])
                yield key, self._value(noff, lo, hi, nflags, ksize), nflags

    def _seek(self, root: int, key: bytes) -> Optional[bytes]:
        pg = root
        for _ in range(64):
            if pg == INVALID:
                return None
            nodes = list(self._nodes(pg))
            if not nodes:
                return None
            if nodes[0][0] & P_BRANCH:
                child = None
                for i, (_, noff, lo, hi, nflags, ksize) in enumerate(nodes):
                    k = bytes(self._mm[noff + NODE: noff + NODE + ksize])
                    if i == 0 or k <= key:
                        child = lo | (hi << 16) | (nflags << 32)
                    else:
                        break
                pg = child
                continue
            for _, noff, lo, hi, nflags, ksize in nodes:
                if bytes(self._mm[noff + NODE: noff + NODE + ksize]) == key:
                    return self._value(noff, lo, hi, nflags, ksize)
            return None
        raise LmdbError("tree deeper than 64 levels (a page cycle)")

    # -- databases -------------------------------------------------------------------------------------------
    @_refuses
    def databases(self) -> List[str]:
        return [k.decode("utf-8", "replace") for k, _, nf in self._walk(self._main[7]) if nf & F_SUBDATA]

    @staticmethod
    def _sub(v: bytes):
        if len(v) < _DB.size:
            raise LmdbError("named database record is shorter than 48 bytes")
        return _DB.unpack(v[:48])

    def _db_root(self, name: Optional[str]) -> int:
        if name is None:
            return self._main[7]
        for k, v, nf in self._walk(self._main[7]):
            if k == name.encode() and nf & F_SUBDATA:
                return self._sub(v)[7]
        raise KeyError(f"no database named {name!r}")

    @_refuses
    def entries(self, name: Optional[str] = None) -> int:
        if name is None:
            return self._main[6]
        for k, v, nf in self._walk(self._main[7]):
            if k == name.encode() and nf & F_SUBDATA:
                return self._sub(v)[6]
        raise KeyError(f"no database named {name!r}")

    @_refuses
    def items(self, name: Optional[str] = None) -> Iterator[Tuple[bytes, bytes]]:
        """Key / value pairs of a database in key order (``name`` None: the unnamed main database)."""
        for k, v, nf in self._walk(self._db_root(name)):
            if name is None and nf & F_SUBDATA:
                continue
            yield k, v

    @_refuses
    def get(self, name: Optional[str], key: bytes) -> Optional[bytes]:
        return self._seek(self._db_root(name), key)


def _even(n: int) -> int:
    return (n + 1) & ~1


class _Pages:
    def __init__(self, page_size: int):
        self.ps, self.pages = page_size, {}          # pgno -> bytes
        self.next = 2

    def alloc(self, n: int = 1) -> int:
        pg = self.next
        self.next += n
        return pg


def _build_tree(pages: _Pages, items: List[Tuple[bytes, bytes, int]]) -> Tuple[int, int, int, int, int]:
    """Sorted (key, value, node flags) -> pages; returns (root, depth, branch pages, leaf pages, overflow pages)."""
    ps = pages.ps
    if not items:
        return INVALID, 0, 0, 0, 0
    node_max = (((ps - HDR) // 2) & ~1) - 2
    overflow = 0

    def flush(kind: int, nodes: List[bytes]) -> int:
        pg = pages.alloc()
        buf = bytearray(ps)
        upper = ps
        ptrs = []
        for nd in nodes:
            upper -= len(nd)
            buf[upper: upper + len(nd)] = nd
            ptrs.append(upper)
        lower = HDR + 2 * len(nodes)
        struct.pack_into("<QHHHH", buf, 0, pg, 0, kind, lower, upper)
        struct.pack_into(f"<{len(ptrs)}H", buf, HDR, *ptrs)
        pages.pages[pg] = bytes(buf)
        return pg

    # leaves
    level: List[Tuple[bytes, int]] = []               # (first key, page) of every page of the level below
    cur, cur_first, room = [], None, ps - HDR
    for key, val, nflags in items:
        if len(key) == 0 or len(key) > 511:
            raise LmdbError(f"key of {len(key)} bytes (LMDB takes 1..511)")
        if NODE + len(key) + len(val) > node_max and not nflags & F_SUBDATA:
            n_ov = (HDR + len(val) + ps - 1) // ps
            ov = pages.alloc(n_ov)
            body = bytearray(n_ov * ps)
            struct.pack_into("<QHHI", body, 0, ov, 0, P_OVERFLOW, n_ov)
            body[HDR: HDR + len(val)] = val
            for i in range(n_ov):
                pages.pages[ov + i] = bytes(body[i * ps:(i + 1) * ps])
            overflow += n_ov
            nd = struct.pack("<HHHH", len(val) & 0xFFFF, len(val) >> 16, nflags | F_BIGDATA, len(key)) + key + \
                struct.pack("<Q", ov)
        else:
            nd = struct.pack("<HHHH", len(val) & 0xFFFF, len(val) >> 16, nflags, len(key)) + key + val
        nd = nd + b"\0" * (_even(len(nd)) - len(nd))
        if len(nd) + 2 > room:
            level.append((cur_first, flush(P_LEAF, cur)))
            cur, cur_first, room = [], None, ps - HDR
        if cur_first is None:
            cur_first = key
        cur.append(nd)
        room -= len(nd) + 2
    level.append((cur_first, flush(P_LEAF, cur)))
    leaves, branches, depth = len(level), 0, 1
    # branch levels
    while len(level) > 1:
        nxt: List[Tuple[bytes, int]] = []
        cur, cur_first, room = [], None, ps - HDR
        for first, pg in level:
            key = b"" if not cur else first            # the first key of a branch page is implicit
            nd = struct.pack("<HHHH", pg & 0xFFFF, (pg >> 16) & 0xFFFF, (pg >> 32) & 0xFFFF, len(key)) + key
            nd = nd + b"\0" * (_even(len(nd)) - len(nd))
            if len(nd) + 2 > room:
                nxt.append((cur_first, flush(P_BRANCH, cur)))
                cur, cur_first, room = [], None, ps - HDR
                nd = struct.pack("<HHHH", pg & 0xFFFF, (pg >> 16) & 0xFFFF, (pg >> 32) & 0xFFFF, 0)
            if cur_first is None:
                cur_first = first
            cur.append(nd)
            room -= len(nd) + 2
        nxt.append((cur_first, flush(P_BRANCH, cur)))
        branches += len(nxt)
        level = nxt
        depth += 1
    return level[0][1], depth, branches, leaves, overflow


def write_lmdb(path: str, databases: Dict[str, Dict[bytes, bytes]], page_size: int = 4096) -> None:
    """Write an LMDB environment (``path``: a directory; ``data.mdb`` and an empty ``lock.mdb`` inside) holding the
    named databases, every tree bulk-built with full pages, as one committed transaction."""
    pages = _Pages(page_size)
    main_items: List[Tuple[bytes, bytes, int]] = []
    for name in sorted(databases, key=lambda s: s.encode()):
        kv = databases[name]
        items = [(k, kv[k], 0) for k in sorted(kv)]
        root, depth, nb, nl, no = _build_tree(pages, items)
        main_items.append((name.encode(), _DB.pack(0, 0, depth, nb, nl, no, len(items), root), F_SUBDATA))
    root, depth, nb, nl, no = _build_tree(pages, main_items)
    last = pages.next - 1
    size = max((last + 1) * page_size, 1 << 20)

    def meta(pg: int, txnid: int, main: bytes, last_pg: int) -> bytes:
        buf = bytearray(page_size)
        struct.pack_into("<QHHHH", buf, 0, pg, 0, P_META, 0, 0)
        _META.pack_into(buf, HDR, MAGIC, VERSION, 0, size)
        buf[HDR + _META.size: HDR + _META.size + 48] = _DB.pack(page_size, 0x08, 0, 0, 0, 0, 0, INVALID)
        buf[HDR + _META.size + 48: HDR + _META.size + 96] = main
        struct.pack_into("<QQ", buf, HDR + _META.size + 96, last_pg, txnid)
        return bytes(buf)

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "data.mdb"), "wb") as f:
        f.write(meta(0, 0, _DB.pack(0, 0, 0, 0, 0, 0, 0, INVALID), 1))
        f.write(meta(1, 1, _DB.pack(0, 0, depth, nb, nl, no, len(main_items), root), last))
        for pg in range(2, last + 1):
            f.write(pages.pages[pg])
    open(os.path.join(path, "lock.mdb"), "ab").close()
