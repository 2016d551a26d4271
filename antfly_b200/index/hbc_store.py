"""An HBC index that lives in a log-structured merge store: every insert / delete batch is one write transaction.

The reference keeps its tree in the namespace store and mutates it through write transactions
(zig/lib/vectorindex/src/hbc_index.zig insert / delete paths over ``store.NamespaceWriteTxn``,
zig/lib/vectorindex/src/store.zig:144-190; row keys zig/lib/vectorindex/src/hbc.zig:89-124).  Here the tree is also
held in memory (searches run on tensors); after a batch the rows that changed -- the touched leaves, their
ancestors' payloads, the new vectors, the ``l:`` rows of vectors a split moved -- are found by comparing row digests
with what the store holds and are written in one commit, so after a crash the store holds the index as of the last
finished batch, never half a split.
"""
from __future__ import annotations

import hashlib
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch

from . import artifact
from .hbc import HBCConfig, HBCIndex
from .lsm_store import LsmStore


def _digest(b: bytes) -> bytes:
    return hashlib.blake2b(b, digest_size=8).digest()


class PersistentHBC:
    def __init__(self, directory: str, **store_options):
        """Opens an index that :meth:`create` (or ``artifact.save_hbc(..., container="lsm")``) wrote."""
        if not os.path.exists(os.path.join(directory, "MANIFEST")):
            raise FileNotFoundError(f"{directory}: no index store here")
        self.store = LsmStore(directory, **store_options)
        self.index = artifact.load_hbc_from(self._spaces())
        self._sig: Dict[Tuple[str, bytes], bytes] = {}
        self._vectors = set()
        with self.store.begin_read() as r:
            for ns in artifact.LMDB_NAMES:
                for k, v in r.items(ns):
                    if ns == "vecs" and k.startswith(b"v:"):
                        self._vectors.add(struct.unpack(">Q", k[2:])[0])     # vector rows never change: no digest
                    else:
                        self._sig[(ns, k)] = _digest(v)
        self.last_commit_rows = 0

    def _spaces(self):
        with self.store.begin_read() as r:
            return {ns: dict(r.items(ns)) for ns in artifact.LMDB_NAMES}

    @classmethod
    def create(cls, directory: str, vectors: torch.Tensor, cfg: HBCConfig, ids: Optional[torch.Tensor] = None,
               **store_options) -> "PersistentHBC":
        artifact.save_hbc(HBCIndex.bulk_build(vectors, cfg, ids), directory, container="lsm")
        return cls(directory, **store_options)

    # -- mutation ------------------------------------------------------------------------------------------
    def _commit(self) -> int:
        rows = artifact.hbc_rows(self.index, known_vectors=self._vectors)
        live = {int(v) for v in self.index.ids[sorted(self.index.leaf_of)].tolist()} if self.index.leaf_of else set()
        written = 0
        with self.store.begin_write() as w:
            seen = set()
            for ns, kv in rows.items():
                for k, v in kv.items():
                    if ns == "vecs" and k.startswith(b"v:"):
                        w.put(ns, k, v)
                        written += 1
                        continue
                    seen.add((ns, k))
                    d = _digest(v)
                    if self._sig.get((ns, k)) != d:
                        w.put(ns, k, v)
                        self._sig[(ns, k)] = d
                        written += 1
            for key in [key for key in self._sig if key not in seen]:
                w.delete(*key)
                del self._sig[key]
                written += 1
            for vid in self._vectors - live:
                w.delete("vecs", b"v:" + struct.pack(">Q", vid))
                written += 1
        self._vectors = live
        self.last_commit_rows = written
        return written

    def insert(self, vectors: torch.Tensor, ids: Optional[torch.Tensor] = None) -> int:
        """-> rows written by the commit."""
        self.index.insert(vectors, ids)
        return self._commit()

    def delete(self, vector_ids: List[int]) -> int:
        """-> vectors found and removed."""
        n = self.index.delete(vector_ids)
        self._commit()
        return n

    # -- reads ---------------------------------------------------------------------------------------------
    def search(self, query: torch.Tensor, k: int, **kw):
        return self.index.search(query, k, **kw)

    def stats(self) -> dict:
        return {**self.index.stats(), "store": self.store.stats()}

    def close(self) -> None:
        self.store.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
