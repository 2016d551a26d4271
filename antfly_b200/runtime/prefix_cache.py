"""Prefix cache: prompts that start with tokens the engine has already prefilled reuse those KV blocks.

Built on the block allocator's shared-prefix attach (reference: zig/pkg/inference/src/runtime/kv/manager.zig
``attachShared``; blocks are shared by reference count, so no KV data moves).  After a request's prompt has been
prefilled, the cache pins the whole blocks of that prompt under an entry of its own; a later request whose prompt
begins with the same tokens attaches to the entry for the longest block-aligned match and only prefills the rest
(RAG-style workloads: a long shared system / context prefix followed by a short question).

Matching is by a chain of block hashes -- hash(previous block's hash, this block's token ids) -- so a lookup walks
the new prompt block by block and stops at the first miss; entries are evicted least-recently-used, either to
respect ``max_entries`` or on demand when the KV pool runs out of blocks.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

from .kv_cache import KvOutOfBlocks

_ENTRY_BASE = -(1 << 40)  # entry sequence ids live far below any request id


class PrefixCache:
    def __init__(self, alloc, page: int, max_entries: int = 256):
        self.alloc, self.page, self.max_entries = alloc, page, max_entries
        self._entries: "OrderedDict[int, List[bytes]]" = OrderedDict()  # entry id -> its block-digest chain
        self._by_hash: Dict[bytes, Tuple[int, int]] = {}                # block digest -> (entry id, blocks covered)
        self._next = 0
        self.hits = self.misses = self.tokens_reused = self.evictions = 0

    def _chain(self, tokens: Sequence[int], n_blocks: int) -> List[bytes]:
        """Chained 128-bit BLAKE2b digests: digest(previous digest || this block's token ids).  A match on the
        digest is taken as a match on the tokens, so the digest has to be collision resistant: with a plain 64-bit
        hash of the ids, colliding prompts could be computed offline and one tenant's request would attach to
        another prompt's KV blocks."""
        import hashlib
        from array import array

        out, h = [], b"antfly-b200-prefix"
        for b in range(n_blocks):
            blk = array("q", tokens[b * self.page:(b + 1) * self.page]).tobytes()
            h = hashlib.blake2b(h + blk, digest_size=16).digest()
            out.append(h)
        return out

    def lookup(self, prompt: Sequence[int]) -> Tuple[Optional[int], int]:
        """(entry id, tokens to share): the longest cached block-aligned prefix that still leaves at least one
        prompt token to prefill; (None, 0) on a miss."""
        usable = (len(prompt) - 1) // self.page
        best: Tuple[Optional[int], int] = (None, 0)
        for i, h in enumerate(self._chain(prompt, usable)):
            hit = self._by_hash.get(h)
            if hit is None or hit[0] not in self._entries:
                break
            best = (hit[0], (i + 1) * self.page)
        if best[0] is None:
            self.misses += 1
        else:
            self.hits += 1
            self.tokens_reused += best[1]
            self._entries.move_to_end(best[0])
        return best

    def insert(self, request_id: int, prompt: Sequence[int]) -> bool:
        """Pin the whole blocks of ``prompt`` (already in the cache under ``request_id``).  Returns False when
        there is nothing to pin, the prefix is cached already, or no entry could be made."""
        n_blocks = len(prompt) // self.page
        if n_blocks == 0:
            return False
        chain = self._chain(prompt, n_blocks)
        known = self._by_hash.get(chain[-1])
        if known is not None and known[0] in self._entries:
            self._entries.move_to_end(known[0])
            return False
        while len(self._entries) >= self.max_entries:
            if not self.evict_one():
                return False
        eid = _ENTRY_BASE - self._next
        self._next += 1
        try:
            self.alloc.attach_shared(eid, request_id, n_blocks * self.page)  # whole blocks: shared, nothing copied
        except (KvOutOfBlocks, KeyError):
            return False
        self._entries[eid] = chain
        for i, h in enumerate(chain):
            self._by_hash[h] = (eid, i + 1)
        return True

    def evict_one(self) -> bool:
        """Drops the least recently used entry (its blocks are freed once no live sequence shares them)."""
        if not self._entries:
            return False
        eid, chain = self._entries.popitem(last=False)
        for h in chain:
            if self._by_hash.get(h, (None,))[0] == eid:
                del self._by_hash[h]
        self.alloc.detach(eid)
        self.evictions += 1
        return True

    def clear(self) -> None:
        while self.evict_one():
            pass

    def stats(self) -> dict:
        return {"entries": len(self._entries), "hits": self.hits, "misses": self.misses,
                "tokens_reused": self.tokens_reused, "evictions": self.evictions}
