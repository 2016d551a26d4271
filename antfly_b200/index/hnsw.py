"""Graph index (hierarchical navigable small world) with metadata, filtered search, deletion and persistence.

The reference's second dense index type (go/pkg/antfly/lib/vectorindex/hnsw.go: ``HNSWConfig`` :221-255 -- Neighbors,
NeighborsHigherLayers, EfConstruction, EfSearch, LevelMultiplier; ``BatchInsert`` :1492; ``Search`` :1714 with
``FilterPrefix`` and the direct-scan rule when k >= 20 % of the matching entries or fewer than 100 match;
``DeleteByMetadata`` :1804; the ``VectorIndex`` contract Batch / Search / Delete / Stats,
go/pkg/antfly/lib/vectorindex/index.go:98-129).  The graph itself is the C++ structure of ``csrc/host/hnsw.cpp``
(flat adjacency slabs, searches in parallel over the queries of a batch); this module is its typed front and
adapts it to the ``add`` / ``search`` contract the table layer uses for every dense index.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Sequence

import numpy as np
import torch

from .. import _native as N
from .distance import METRICS
from .flat import SearchResult



def _lib():
    lib = N.host()
    if not getattr(lib, "_hnsw_typed", False):
        lib.afb_hnsw_create.restype = ctypes.c_void_p
        lib.afb_hnsw_create.argtypes = [ctypes.c_int] * 6 + [ctypes.c_double, ctypes.c_uint64]
        lib.afb_hnsw_load.restype = ctypes.c_void_p
        lib.afb_hnsw_load.argtypes = [ctypes.c_char_p, ctypes.c_uint64]
        lib.afb_hnsw_free.argtypes = [ctypes.c_void_p]
        lib.afb_hnsw_free.restype = None
        lib.afb_hnsw_insert.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_long] + [ctypes.c_void_p] * 3
        lib.afb_hnsw_search.restype = ctypes.c_long
        lib.afb_hnsw_search.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.afb_hnsw_delete.restype = ctypes.c_long
        lib.afb_hnsw_delete.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long]
        lib.afb_hnsw_delete_by_metadata.restype = ctypes.c_long
        lib.afb_hnsw_delete_by_metadata.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
        lib.afb_hnsw_stats.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.afb_hnsw_get_metadata.restype = ctypes.c_long
        lib.afb_hnsw_get_metadata.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_long]
        lib.afb_hnsw_get_vector.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
        lib.afb_hnsw_check.argtypes = [ctypes.c_void_p]
        lib.afb_hnsw_save.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        lib._hnsw_typed = True
    return lib


class HNSWIndex:
    def __init__(self, dim: int, metric: str = "cosine", neighbors: int = 16, neighbors_layer0: int = 0,
                 ef_construction: int = 200, ef_search: int = 64, level_multiplier: float = 0.0, seed: int = 0,
                 threads: int = 0, _handle: Optional[int] = None):
        """``neighbors``: links of a new node and the capacity of the upper layers; ``neighbors_layer0``: capacity of
        the bottom layer (0 = twice ``neighbors``); ``level_multiplier`` 0 = 1 / ln(neighbors)."""
        if metric not in METRICS:
            raise ValueError(f"unknown distance metric {metric!r}; expected one of {METRICS}")
        self.dim, self.metric, self.ef_search = dim, metric, ef_search
        self.threads = threads or min(16, os.cpu_count() or 1)
        self._lib = _lib()
        self._h = _handle or self._lib.afb_hnsw_create(dim, METRICS.index(metric), neighbors, neighbors_layer0,
                                                      ef_construction, ef_search, level_multiplier, seed)
        if not self._h:
            raise ValueError("bad HNSW configuration (dim > 0, neighbors >= 2)")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.afb_hnsw_free(h)

    def __len__(self) -> int:
        return self.stats()["active"]

    # -- writes --------------------------------------------------------------------------------------------
    def batch_insert(self, ids: Sequence[int], vectors: torch.Tensor, metadata: Optional[Sequence[bytes]] = None,
                     levels: Optional[Sequence[int]] = None) -> None:
        """Upsert: an id that is already indexed is removed first and inserted again with the new vector."""
        v = np.ascontiguousarray(torch.as_tensor(vectors).detach().float().cpu().numpy())
        if v.ndim != 2 or v.shape[1] != self.dim:
            raise ValueError(f"vectors must be [n, {self.dim}]")
        idv = np.ascontiguousarray(np.asarray(ids, dtype=np.uint64))
        if idv.shape[0] != v.shape[0]:
            raise ValueError("ids and vectors differ in length")
        blob = offs = None
        if metadata is not None:
            if len(metadata) != v.shape[0]:
                raise ValueError("metadata and vectors differ in length")
            offs = np.zeros(len(metadata) + 1, dtype=np.int64)
            offs[1:] = np.cumsum([len(m) for m in metadata])
            blob = np.frombuffer(b"".join(metadata) or b"\0", dtype=np.uint8)
        lv = np.ascontiguousarray(np.asarray(levels, dtype=np.int32)) if levels is not None else None
        p = lambda a: a.ctypes.data if a is not None else None
        rc = self._lib.afb_hnsw_insert(self._h, p(idv), p(v), v.shape[0], p(blob), p(offs), p(lv))
        if rc != 0:
            raise RuntimeError("HNSW insert failed")

    def add(self, vectors: torch.Tensor, ids: torch.Tensor) -> None:
        self.batch_insert(ids.tolist(), vectors)

    def delete(self, ids: Sequence[int]) -> int:
        idv = np.ascontiguousarray(np.asarray(list(ids), dtype=np.uint64))
        return int(self._lib.afb_hnsw_delete(self._h, idv.ctypes.data, idv.shape[0]))

    def delete_by_metadata(self, key: bytes) -> int:
        return int(self._lib.afb_hnsw_delete_by_metadata(self._h, key, len(key)))

    # -- reads ---------------------------------------------------------------------------------------------
    def search(self, queries: torch.Tensor, k: int, ef: int = 0, filter_prefix: Optional[bytes] = None,
               effort: Optional[float] = None) -> SearchResult:
        """queries [Q, dim] -> distances [Q, k] (ascending, +inf padded) and ids [Q, k] int64 (-1 padded).
        ``effort`` in [0, 1] scales the beam between ``max(k, ef_search)`` and 16 times that."""
        q = np.ascontiguousarray(torch.as_tensor(queries).detach().float().cpu().numpy())
        if q.ndim == 1:
            q = q[None]
        if q.shape[1] != self.dim:
            raise ValueError(f"query dimension mismatch: expected {self.dim}, got {q.shape[1]}")
        if ef <= 0 and effort is not None:
            base = max(k, self.ef_search)
            ef = int(base * (1.0 + 15.0 * min(max(float(effort), 0.0), 1.0)))
        out_ids = np.empty((q.shape[0], k), dtype=np.uint64)
        out_d = np.empty((q.shape[0], k), dtype=np.float32)
        rc = self._lib.afb_hnsw_search(self._h, q.ctypes.data, q.shape[0], k, ef, filter_prefix or None,
                                       len(filter_prefix or b""), out_ids.ctypes.data, out_d.ctypes.data, self.threads)
        if rc < 0:
            raise RuntimeError("HNSW search failed")
        ids = torch.from_numpy(out_ids.view(np.int64).copy())             # the pad value ~0 reads as -1
        return SearchResult(torch.from_numpy(out_d), ids)

    def metadata(self, id_: int) -> Optional[bytes]:
        cap = 256
        while True:
            buf = ctypes.create_string_buffer(cap)
            n = self._lib.afb_hnsw_get_metadata(self._h, id_, buf, cap)
            if n < 0:
                return None
            if n <= cap:
                return buf.raw[:n]
            cap = n

    def get_vector(self, id_: int) -> Optional[torch.Tensor]:
        """The stored vector of an id (unit-normalised under the cosine metric), or None."""
        out = np.empty(self.dim, dtype=np.float32)
        if self._lib.afb_hnsw_get_vector(self._h, id_, out.ctypes.data) != 0:
            return None
        return torch.from_numpy(out)

    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_long * 6)()
        self._lib.afb_hnsw_stats(self._h, out)
        return {"active": out[0], "max_layer": out[1], "entry_point": out[2], "edges": out[3], "slots": out[4],
                "upper_layer_nodes": out[5]}

    def check(self) -> int:
        """0 when the graph is structurally sound (see ``afb_hnsw_check``), else the code of the violated rule."""
        return int(self._lib.afb_hnsw_check(self._h))

    # -- persistence ---------------------------------------------------------------------------------------
    def save(self, path: str) -> None:
        tmp = path + ".tmp"
        rc = self._lib.afb_hnsw_save(self._h, tmp.encode())
        if rc != 0:
            raise OSError(f"cannot write {tmp} (code {rc})")
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str, seed: int = 0, threads: int = 0) -> "HNSWIndex":
        lib = _lib()
        h = lib.afb_hnsw_load(path.encode(), seed)
        if not h:
            raise ValueError(f"{path}: not a graph index file, or it fails the structural check")
        # dim / metric / ef_search are in the file; read them back through a second look at the header
        with open(path, "rb") as f:
            head = np.frombuffer(f.read(8 + 80), dtype=np.int64)[1:]
        return cls(int(head[0]), METRICS[int(head[1])], int(head[2]), int(head[3]), int(head[4]), int(head[5]),
                   seed=seed, threads=threads, _handle=h)
