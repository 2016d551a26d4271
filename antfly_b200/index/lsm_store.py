"""Namespace store over the native log-structured merge engine (``csrc/host/lsm_store.cpp``).

The interface the reference's vector index talks to (zig/lib/vectorindex/src/store.zig:23-28 the four namespaces
``nodes`` / ``meta`` / ``quant`` / ``vecs``; :59-102 cursors with first / last / next / prev / seekAtOrAfter /
seekAtOrBefore; :104-142 read transactions with get / getManySorted / openCursor; :144-190 write transactions that
read their own writes; :192-232 batches with put / appendPut / delete and a ``bulk_ingest`` mode; :234-278 the store
with beginRead / beginWrite / beginBatch), backed by the engine whose design the reference describes in
zig/pkg/antfly/src/storage/lsm/LSM.md: write-ahead log + memory table in the foreground, table files and
level-by-level merges in the background, manifest replaced atomically, read transactions pinned to one version.

A read transaction sees the state at the moment it began, whatever is committed, flushed or merged afterwards.  One
write transaction is open at a time (a second ``begin_write`` waits); its commit is one log record, so it is applied
entirely or not at all after a crash.  A ``bulk_ingest`` batch skips the log: its rows are sorted and written as one
table file that becomes visible when the manifest names it.
"""
from __future__ import annotations

import bisect
import ctypes
import threading
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

from .. import _native as N

NAMESPACES = {"nodes": 0, "meta": 1, "quant": 2, "vecs": 3}
_STATS = ["mutable_bytes", "immutable_bytes", "immutable_tables"] + [f"level{i}_files" for i in range(6)] + \
    [f"level{i}_bytes" for i in range(6)] + ["flushes", "compactions", "compaction_bytes_read",
                                             "compaction_bytes_written", "wal_bytes", "wal_records", "stalls",
                                             "stall_ms", "bloom_skips", "last_sequence", "live_snapshots", "ingests",
                                             "recovered_records", "dropped_tombstones"]
_PUT, _DEL = 1, 2


class LsmError(RuntimeError):
    pass


def _lib():
    lib = N.host()
    if not getattr(lib, "_lsm_typed", False):
        vp, u8p, u64 = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64
        lib.afb_lsm_last_error.restype = ctypes.c_char_p
        lib.afb_lsm_open.restype = vp
        lib.afb_lsm_open.argtypes = [ctypes.c_char_p, vp]
        lib.afb_lsm_close.argtypes = [vp]
        lib.afb_lsm_write.argtypes = [vp, u8p, u64]
        lib.afb_lsm_ingest.argtypes = [vp, u8p, u64]
        lib.afb_lsm_flush.argtypes = [vp]
        lib.afb_lsm_compact.argtypes = [vp, ctypes.c_int]
        lib.afb_lsm_stats.argtypes = [vp, vp, ctypes.c_int]
        lib.afb_lsm_snapshot.restype = vp
        lib.afb_lsm_snapshot.argtypes = [vp]
        lib.afb_lsm_snapshot_free.argtypes = [vp]
        lib.afb_lsm_get.argtypes = [vp, ctypes.c_int, u8p, u64, vp, vp]
        lib.afb_lsm_cursor.restype = vp
        lib.afb_lsm_cursor.argtypes = [vp, ctypes.c_int]
        lib.afb_lsm_cursor_free.argtypes = [vp]
        lib.afb_lsm_cursor_move.argtypes = [vp, ctypes.c_int, u8p, u64]
        lib.afb_lsm_cursor_entry.argtypes = [vp, vp, vp, vp, vp]
        lib._lsm_typed = True
    return lib


def _fail(lib) -> LsmError:
    return LsmError((lib.afb_lsm_last_error() or b"").decode("utf-8", "replace"))


def _ns(namespace) -> int:
    if isinstance(namespace, int):
        if not 0 <= namespace <= 255:
            raise ValueError("a namespace number is 0 to 255")
        return namespace
    try:
        return NAMESPACES[namespace]
    except KeyError:
        raise ValueError(f"unknown namespace {namespace!r} (known: {', '.join(NAMESPACES)})") from None


def _varint(n: int) -> bytes:
    out = bytearray()
    while n >= 0x80:
        out.append((n & 0x7F) | 0x80)
        n >>= 7
    out.append(n)
    return bytes(out)


def _encode(ops: Sequence[Tuple[int, int, bytes, Optional[bytes]]]) -> bytes:
    """[(kind, namespace number, key, value)] -> the engine's batch framing."""
    out = bytearray()
    for kind, ns, key, value in ops:
        v = value or b""
        out.append(kind)
        out += _varint(len(key) + 1)
        out += _varint(len(v))
        out.append(ns)
        out += key
        out += v
    return bytes(out)


class Cursor:
    """Ordered walk over one namespace of a read transaction.  Every move returns ``(key, value)`` or None when it
    leaves the namespace."""

    def __init__(self, txn: "ReadTxn", namespace):
        self._lib, self._txn = _lib(), txn
        self._h = self._lib.afb_lsm_cursor(txn._h, _ns(namespace))
        txn._cursors.append(self)

    def _move(self, op: int, key: Optional[bytes] = None) -> Optional[Tuple[bytes, bytes]]:
        if self._h is None:
            raise LsmError("the cursor is closed")
        r = self._lib.afb_lsm_cursor_move(self._h, op, key, len(key) if key is not None else 0)
        if r < 0:
            raise _fail(self._lib)
        if r == 0:
            return None
        k, v = ctypes.c_void_p(), ctypes.c_void_p()
        kl, vl = ctypes.c_uint64(), ctypes.c_uint64()
        self._lib.afb_lsm_cursor_entry(self._h, ctypes.byref(k), ctypes.byref(kl), ctypes.byref(v), ctypes.byref(vl))
        return ctypes.string_at(k.value, kl.value) if kl.value else b"", \
            ctypes.string_at(v.value, vl.value) if vl.value else b""

    def first(self):
        return self._move(0)

    def last(self):
        return self._move(1)

    def next(self):
        return self._move(2)

    def prev(self):
        return self._move(3)

    def seek_at_or_after(self, key: bytes):
        return self._move(4, bytes(key))

    def seek_at_or_before(self, key: bytes):
        return self._move(5, bytes(key))

    def close(self) -> None:
        if self._h is not None:
            self._lib.afb_lsm_cursor_free(self._h)
            self._h = None

    def __iter__(self) -> Iterator[Tuple[bytes, bytes]]:
        e = self.first()
        while e is not None:
            yield e
            e = self.next()


class ReadTxn:
    def __init__(self, store: "LsmStore"):
        self._lib, self._store = _lib(), store
        self._h = self._lib.afb_lsm_snapshot(store._handle())
        self._cursors: List[Cursor] = []
        store._open_reads.add(self)

    def get(self, namespace, key: bytes) -> Optional[bytes]:
        if self._h is None:
            raise LsmError("the transaction is closed")
        v, vl = ctypes.c_void_p(), ctypes.c_uint64()
        r = self._lib.afb_lsm_get(self._h, _ns(namespace), bytes(key), len(key), ctypes.byref(v), ctypes.byref(vl))
        if r < 0:
            raise _fail(self._lib)
        if r == 0:
            return None
        return ctypes.string_at(v.value, vl.value) if vl.value else b""

    def get_many_sorted(self, namespace, keys: Sequence[bytes]) -> List[Optional[bytes]]:
        """Values of keys given in ascending order (absent: None)."""
        return [self.get(namespace, k) for k in keys]

    def open_cursor(self, namespace) -> Cursor:
        return Cursor(self, namespace)

    def items(self, namespace, prefix: bytes = b"") -> Iterator[Tuple[bytes, bytes]]:
        c = self.open_cursor(namespace)
        try:
            e = c.seek_at_or_after(prefix) if prefix else c.first()
            while e is not None and e[0].startswith(prefix):
                yield e
                e = c.next()
        finally:
            c.close()

    def abort(self) -> None:
        for c in self._cursors:
            c.close()
        self._cursors = []
        if self._h is not None:
            self._lib.afb_lsm_snapshot_free(self._h)
            self._h = None
            self._store._open_reads.discard(self)

    close = abort

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.abort()


class _Overlay:
    """Uncommitted writes of one transaction: {(namespace number, key): value or None for a delete}."""

    def __init__(self):
        self.rows: Dict[Tuple[int, bytes], Optional[bytes]] = {}
        self.order: List[Tuple[int, int, bytes, Optional[bytes]]] = []
        self._sorted: Dict[int, List[bytes]] = {}

    def put(self, ns: int, key: bytes, value: Optional[bytes]) -> None:
        if not 0 < len(key) + 1 <= 1024:
            raise ValueError("a key is 0 to 1023 bytes")
        key = bytes(key)
        self.rows[(ns, key)] = None if value is None else bytes(value)
        self.order.append((_DEL if value is None else _PUT, ns, key, value))
        self._sorted.pop(ns, None)

    def keys(self, ns: int) -> List[bytes]:
        if ns not in self._sorted:
            self._sorted[ns] = sorted(k for (n, k) in self.rows if n == ns)
        return self._sorted[ns]


class _OverlayCursor:
    """A cursor of a write transaction: the snapshot underneath with the transaction's own writes on top."""

    def __init__(self, base: Cursor, overlay: _Overlay, ns: int):
        self._base, self._ov, self._ns, self._at = base, overlay, ns, None

    def _live(self, key: bytes) -> bool:
        return self._ov.rows.get((self._ns, key)) is not None

    def _forward(self, key: Optional[bytes], strict: bool):
        # smallest key >= key (> key when strict) among the base rows the overlay does not replace and the
        # overlay's puts
        e = self._base.first() if key is None else self._base.seek_at_or_after(key)
        while e is not None and ((strict and e[0] == key) or (self._ns, e[0]) in self._ov.rows):
            e = self._base.next()
        keys = self._ov.keys(self._ns)
        i = 0 if key is None else (bisect.bisect_right(keys, key) if strict else bisect.bisect_left(keys, key))
        while i < len(keys) and not self._live(keys[i]):
            i += 1
        if i < len(keys) and (e is None or keys[i] < e[0]):
            e = (keys[i], self._ov.rows[(self._ns, keys[i])])
        self._at = e[0] if e else None
        return e

    def _backward(self, key: Optional[bytes], strict: bool):
        e = self._base.last() if key is None else self._base.seek_at_or_before(key)
        while e is not None and ((strict and e[0] == key) or (self._ns, e[0]) in self._ov.rows):
            e = self._base.prev()
        keys = self._ov.keys(self._ns)
        i = len(keys) if key is None else (bisect.bisect_left(keys, key) if strict else bisect.bisect_right(keys, key))
        i -= 1
        while i >= 0 and not self._live(keys[i]):
            i -= 1
        if i >= 0 and (e is None or keys[i] > e[0]):
            e = (keys[i], self._ov.rows[(self._ns, keys[i])])
        self._at = e[0] if e else None
        return e

    def first(self):
        return self._forward(None, False)

    def last(self):
        return self._backward(None, False)

    def next(self):
        return None if self._at is None else self._forward(self._at, True)

    def prev(self):
        return None if self._at is None else self._backward(self._at, True)

    def seek_at_or_after(self, key: bytes):
        return self._forward(bytes(key), False)

    def seek_at_or_before(self, key: bytes):
        return self._backward(bytes(key), False)

    def close(self) -> None:
        self._base.close()

    def __iter__(self):
        e = self.first()
        while e is not None:
            yield e
            e = self.next()


class WriteTxn:
    """Reads see the snapshot taken at ``begin_write`` plus this transaction's own writes; ``commit`` applies
    everything as one log record."""

    def __init__(self, store: "LsmStore"):
        self._store = store
        store._writer.acquire()
        try:
            self._read = ReadTxn(store)
        except BaseException:
            store._writer.release()
            raise
        self._ov = _Overlay()
        self._open = True

    def get(self, namespace, key: bytes) -> Optional[bytes]:
        ns, key = _ns(namespace), bytes(key)
        if (ns, key) in self._ov.rows:
            return self._ov.rows[(ns, key)]
        return self._read.get(ns, key)

    def put(self, namespace, key: bytes, value: bytes) -> None:
        self._ov.put(_ns(namespace), key, bytes(value))

    append_put = put          # the ascending-key hint changes nothing here: the memory table is ordered anyway

    def delete(self, namespace, key: bytes) -> None:
        self._ov.put(_ns(namespace), key, None)

    def open_cursor(self, namespace) -> _OverlayCursor:
        return _OverlayCursor(self._read.open_cursor(namespace), self._ov, _ns(namespace))

    def _end(self) -> None:
        if self._open:
            self._open = False
            self._read.abort()
            self._store._writer.release()

    def commit(self) -> None:
        if not self._open:
            raise LsmError("the transaction is closed")
        try:
            self._store._write(self._ov.order)
        finally:
            self._end()

    def abort(self) -> None:
        self._end()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, *a):
        if self._open:
            if exc_type is None:
                self.commit()
            else:
                self.abort()


class Batch:
    """Writes collected and applied at ``commit``; ``get`` reads the committed state (not the batch).  Mode
    ``bulk_ingest``: no log record -- the rows are sorted and become one table file."""

    def __init__(self, store: "LsmStore", mode: str = "default"):
        if mode not in ("default", "bulk_ingest"):
            raise ValueError(f"unknown batch mode {mode!r}")
        self._store, self._mode, self._ov, self._open = store, mode, _Overlay(), True

    def get(self, namespace, key: bytes) -> Optional[bytes]:
        with self._store.begin_read() as r:
            return r.get(namespace, key)

    def put(self, namespace, key: bytes, value: bytes) -> None:
        self._ov.put(_ns(namespace), key, bytes(value))

    append_put = put

    def delete(self, namespace, key: bytes) -> None:
        self._ov.put(_ns(namespace), key, None)

    def commit(self) -> None:
        if not self._open:
            raise LsmError("the batch is closed")
        self._open = False
        with self._store._writer:
            self._store._write(self._ov.order, ingest=self._mode == "bulk_ingest")

    def abort(self) -> None:
        self._open = False

    def __enter__(self):
        return self

    def __exit__(self, exc_type, *a):
        if self._open:
            if exc_type is None:
                self.commit()
            else:
                self.abort()


class LsmStore:
    """One store directory.  ``read_only`` opens never create, flush, merge or delete anything (several may be open
    beside one writer; each sees the state as of its own open).  ``sync``: every commit reaches the disk before
    ``commit`` returns.  ``background``: flushes and merges run on the engine's own threads; without them they run
    inside the commit that finds the queues full, or when :meth:`flush` / :meth:`compact` is called."""

    def __init__(self, directory: str, read_only: bool = False, sync: bool = True, background: bool = True,
                 memtable_bytes: int = 8 << 20, block_bytes: int = 16 << 10, target_file_bytes: int = 32 << 20,
                 level1_bytes: int = 64 << 20, level0_compact_files: int = 4, level0_stall_files: int = 12):
        self._lib = _lib()
        opts = (ctypes.c_uint64 * 9)(memtable_bytes, block_bytes, target_file_bytes, level1_bytes,
                                     level0_compact_files, level0_stall_files, int(sync), int(read_only),
                                     int(background))
        self._h = self._lib.afb_lsm_open(directory.encode(), opts)
        if not self._h:
            raise _fail(self._lib)
        self.directory, self.read_only = directory, read_only
        self._writer = threading.Lock()
        self._open_reads: set = set()

    def _handle(self):
        if self._h is None:
            raise LsmError("the store is closed")
        return self._h

    def _write(self, ops, ingest: bool = False) -> None:
        if not ops:
            return
        payload = _encode(ops)
        fn = self._lib.afb_lsm_ingest if ingest else self._lib.afb_lsm_write
        if fn(self._handle(), payload, len(payload)) != 0:
            raise _fail(self._lib)

    def begin_read(self) -> ReadTxn:
        return ReadTxn(self)

    begin_probe_or_read = begin_read

    def begin_write(self) -> WriteTxn:
        if self.read_only:
            raise LsmError("the store is open read-only")
        return WriteTxn(self)

    def begin_batch(self, mode: str = "default") -> Batch:
        if self.read_only:
            raise LsmError("the store is open read-only")
        return Batch(self, mode)

    def flush(self) -> None:
        if self._lib.afb_lsm_flush(self._handle()) != 0:
            raise _fail(self._lib)

    def compact(self, full: bool = False) -> None:
        if self._lib.afb_lsm_compact(self._handle(), int(full)) != 0:
            raise _fail(self._lib)

    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_uint64 * len(_STATS))()
        self._lib.afb_lsm_stats(self._handle(), out, len(_STATS))
        return dict(zip(_STATS, (int(x) for x in out)))

    def close(self) -> None:
        if self._h is not None:
            for r in list(self._open_reads):
                r.abort()
            self._lib.afb_lsm_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def bench(directory: str, rows: int = 200_000, value_bytes: int = 256, batch: int = 500, sync: bool = False,
          seed: int = 0) -> Dict[str, float]:
    """Write / read throughput of a store in ``directory`` (the counterpart of the reference's write bench,
    zig/pkg/antfly/src/lsm_write_bench_root.zig): commits of ``batch`` random-key rows through the log, the same
    rows again as one bulk-ingest batch into a second store, point reads of present and absent keys, a full scan."""
    import os
    import random
    import time

    rng = random.Random(seed)
    keys = [b"%016x" % rng.getrandbits(64) for _ in range(rows)]
    value = bytes(rng.getrandbits(8) for _ in range(value_bytes))
    out: Dict[str, float] = {"rows": rows, "value_bytes": value_bytes, "batch": batch}
    with LsmStore(os.path.join(directory, "logged"), sync=sync) as s:
        t0 = time.perf_counter()
        for i in range(0, rows, batch):
            with s.begin_write() as w:
                for k in keys[i:i + batch]:
                    w.put("vecs", k, value)
        out["logged_rows_per_s"] = rows / (time.perf_counter() - t0)
        s.flush()
        s.compact()
        st = s.stats()
        out["write_amplification"] = (st["compaction_bytes_written"] + sum(st[f"level{i}_bytes"] for i in range(6))) / \
            max(rows * (value_bytes + 17), 1)
        probe = rng.sample(keys, min(20_000, rows))
        with s.begin_read() as r:
            t0 = time.perf_counter()
            for k in probe:
                r.get("vecs", k)
            out["get_hit_per_s"] = len(probe) / (time.perf_counter() - t0)
            t0 = time.perf_counter()
            for k in probe:
                r.get("vecs", k + b"?")
            out["get_miss_per_s"] = len(probe) / (time.perf_counter() - t0)
            t0 = time.perf_counter()
            n = sum(1 for _ in r.items("vecs"))
            out["scan_rows_per_s"] = n / (time.perf_counter() - t0)
        out.update({k: v for k, v in st.items() if k in ("flushes", "compactions", "stalls", "stall_ms")})
    with LsmStore(os.path.join(directory, "bulk"), sync=sync) as s:
        t0 = time.perf_counter()
        with s.begin_batch("bulk_ingest") as b:
            for k in keys:
                b.append_put("vecs", k, value)
        out["bulk_rows_per_s"] = rows / (time.perf_counter() - t0)
    return out
