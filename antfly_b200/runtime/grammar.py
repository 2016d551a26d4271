"""Grammar-constrained decoding: JSON mode and GBNF grammars.

``JsonGrammar`` and ``GbnfGrammar`` wrap the C++ matchers (``csrc/host/grammar.cpp``).  The engine asks it for the set of tokens
that keep the output a valid JSON prefix, masks every other logit to -inf before arg-max / sampling, and feeds
the chosen token back.  The end-of-sequence token becomes available once the document is complete, and is forced
when nothing else can follow.  Mirrors the reference's JSON grammar masking in the generation pipeline
(zig/pkg/inference/src/pipelines/grammar.zig, zig/pkg/inference/src/pipelines/generation.zig sampling stage).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from .. import _native as N


def token_bytes_table(tokenizer, vocab_size: int) -> List[bytes]:
    """The byte string each token id contributes to the output text.  Tokenizers may expose ``token_bytes(id)``;
    otherwise the single-token decode is used (exact for byte-level and word-piece vocabularies whose tokens are
    whole characters).  Special tokens map to the empty string and are therefore never allowed by a grammar."""
    special = set()
    sp = getattr(tokenizer, "special", None)
    if sp is not None:
        special = {getattr(sp, n) for n in ("bos_id", "eos_id", "pad_id", "unk_id", "cls_id", "sep_id", "mask_id")
                   if getattr(sp, n, None) is not None}
    out: List[bytes] = []
    fn = getattr(tokenizer, "token_bytes", None)
    for t in range(vocab_size):
        if t in special:
            out.append(b"")
            continue
        try:
            b = fn(t) if fn is not None else tokenizer.decode([t]).encode("utf-8")
        except Exception:
            b = b""
        out.append(b)
    return out


class JsonGrammar:
    """One request's matcher state plus the (shared) vocabulary byte table."""

    def __init__(self, token_bytes: Sequence[bytes], eos_id: Optional[int] = None, root_object_only: bool = False):
        self._lib = N.host()
        self._lib.afb_grammar_json_new.restype = ctypes.c_void_p
        self._h = ctypes.c_void_p(self._lib.afb_grammar_json_new(ctypes.c_int(1 if root_object_only else 0)))
        self._set_vocab(token_bytes, eos_id)

    def _set_vocab(self, token_bytes: Sequence[bytes], eos_id: Optional[int]) -> None:
        self.n = len(token_bytes)
        self.eos_id = eos_id
        offsets = np.zeros(self.n + 1, dtype=np.int64)
        np.cumsum([len(b) for b in token_bytes], out=offsets[1:])
        blob = np.frombuffer(b"".join(token_bytes) or b"\0", dtype=np.uint8)
        rc = self._lib.afb_grammar_set_vocab(self._h, blob.ctypes.data_as(ctypes.c_void_p),
                                             offsets.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(self.n))
        assert rc == 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.afb_grammar_free(h)

    def reset(self) -> None:
        self._lib.afb_grammar_reset(self._h)

    @property
    def complete(self) -> bool:
        return bool(self._lib.afb_grammar_complete(self._h))

    def mask(self) -> np.ndarray:
        """uint8 [vocab]: 1 for every token that may come next (the end-of-sequence id included once the document
        is complete, and alone when nothing else fits)."""
        m = np.zeros(self.n, dtype=np.uint8)
        count = self._lib.afb_grammar_mask(self._h, m.ctypes.data_as(ctypes.c_void_p))
        if self.eos_id is not None and 0 <= self.eos_id < self.n:
            if self.complete or count == 0:
                m[self.eos_id] = 1
        return m

    def accept(self, token: int) -> bool:
        if self.eos_id is not None and token == self.eos_id:
            return self.complete
        return bool(self._lib.afb_grammar_accept(self._h, ctypes.c_int(int(token))))

    def accept_text(self, text: str) -> bool:
        b = text.encode("utf-8")
        return bool(self._lib.afb_grammar_accept_bytes(self._h, b, ctypes.c_int(len(b))))


class GbnfGrammar(JsonGrammar):
    """A context-free grammar in GBNF notation (rules ``name ::= ...``, literals, character classes, groups and
    the ``* + ? {m,n}`` operators), matched byte-wise.  Same interface as :class:`JsonGrammar`.  Raises
    ``ValueError`` with the parser's message for a malformed, incomplete or left-recursive grammar."""

    def __init__(self, token_bytes: Sequence[bytes], grammar: str, eos_id: Optional[int] = None, root: str = "root"):
        self._lib = N.host()
        self._lib.afb_grammar_gbnf_new.restype = ctypes.c_void_p
        self._lib.afb_grammar_last_error.restype = ctypes.c_char_p
        h = self._lib.afb_grammar_gbnf_new(grammar.encode("utf-8"), root.encode("utf-8"))
        if not h:
            self._h = None
            raise ValueError("GBNF: " + self._lib.afb_grammar_last_error().decode("utf-8", "replace"))
        self._h = ctypes.c_void_p(h)
        self._set_vocab(token_bytes, eos_id)
