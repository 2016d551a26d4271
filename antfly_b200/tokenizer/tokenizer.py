from __future__ import annotations

import json
import os
import unicodedata
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass
class SpecialTokens:
    cls_id: int = 101
    sep_id: int = 102
    pad_id: int = 0
    unk_id: int = 100
    bos_id: Optional[int] = None
    eos_id: Optional[int] = None


class Tokenizer:
    """Common surface: ``encode`` (no special tokens), ``decode``, special ids, and the model-facing helpers."""

    special = SpecialTokens()
    vocab_size = 0

    def encode(self, text: str) -> List[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int]) -> str:
        raise NotImplementedError

    # zig/lib/tokenizer/src/tokenizer.zig:120-160: [CLS] tokens [SEP], truncated to max_length.
    def encode_for_model(self, text: str, max_length: int = 512) -> List[int]:
        ids = self.encode(text)[: max(max_length - 2, 0)]
        return [self.special.cls_id] + ids + [self.special.sep_id]

    # zig/lib/tokenizer/src/tokenizer.zig:163-215: [CLS] a [SEP] b [SEP]; budget max_length - 3; text a (the
    # query) keeps priority and b gets what is left.  Token types: 0 through the first [SEP], then 1
    # (zig/pkg/inference/src/pipelines/reranking.zig:335-352).
    def encode_pair(self, a: str, b: str, max_length: int = 512) -> Tuple[List[int], List[int]]:
        ia, ib = self.encode(a), self.encode(b)
        budget = max(max_length - 3, 0)
        na = min(len(ia), budget)
        nb = min(len(ib), budget - na)
        ids = [self.special.cls_id] + ia[:na] + [self.special.sep_id] + ib[:nb] + [self.special.sep_id]
        types = [0] * (na + 2) + [1] * (nb + 1)
        return ids, types

    def encode_prompt(self, text: str, add_bos: bool = True) -> List[int]:
        ids = self.encode(text)
        if add_bos and self.special.bos_id is not None:
            ids = [self.special.bos_id] + ids
        return ids


class HFTokenizer(Tokenizer):
    """``tokenizer.json`` through the ``tokenizers`` library."""

    def __init__(self, path: str, config: Optional[dict] = None):
        from tokenizers import Tokenizer as _T

        self.tk = _T.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        cfg = config or {}

        def tid(name, default):
            tok = cfg.get(name)
            if isinstance(tok, dict):
                tok = tok.get("content")
            if tok is not None and self.tk.token_to_id(tok) is not None:
                return self.tk.token_to_id(tok)
            for cand in default:
                i = self.tk.token_to_id(cand)
                if i is not None:
                    return i
            return None

        self.special = SpecialTokens(
            cls_id=tid("cls_token", ["[CLS]", "<s>"]) or 0, sep_id=tid("sep_token", ["[SEP]", "</s>"]) or 0,
            pad_id=tid("pad_token", ["[PAD]", "<pad>"]) or 0, unk_id=tid("unk_token", ["[UNK]", "<unk>"]) or 0,
            bos_id=tid("bos_token", ["<|begin_of_text|>", "<s>", "<bos>"]),
            eos_id=tid("eos_token", ["<|end_of_text|>", "<|eot_id|>", "</s>", "<eos>"]))

    def encode(self, text: str) -> List[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special)

    # -- exact byte string of one token (grammar-constrained decoding needs bytes, not lossy text) -----------------
    _byte_decoder: Optional[Dict[str, int]] = None

    @staticmethod
    def _bytelevel_map() -> Dict[str, int]:
        """Inverse of the byte-level BPE alphabet: the printable stand-in character of every byte value."""
        keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
        chars, n = list(keep), 0
        order = list(keep)
        for b in range(256):
            if b not in keep:
                order.append(b)
                chars.append(256 + n)
                n += 1
        return {chr(c): b for b, c in zip(order, chars)}

    def token_bytes(self, token_id: int) -> bytes:
        piece = self.tk.id_to_token(int(token_id))
        if piece is None:
            return b""
        if len(piece) == 6 and piece.startswith("<0x") and piece.endswith(">"):  # SentencePiece byte fallback
            try:
                return bytes([int(piece[3:5], 16)])
            except ValueError:
                pass
        if HFTokenizer._byte_decoder is None:
            HFTokenizer._byte_decoder = self._bytelevel_map()
        bd = HFTokenizer._byte_decoder
        if "Ġ" in piece or "Ċ" in piece or all(ch in bd for ch in piece) and any(ord(ch) >= 0x100 for ch in piece):
            try:
                return bytes(bd[ch] for ch in piece)
            except KeyError:
                pass
        if "\u2581" in piece:  # SentencePiece word-boundary marker
            return piece.replace("\u2581", " ").encode("utf-8")
        if piece.startswith("##"):  # WordPiece continuation
            return piece[2:].encode("utf-8")
        text = self.tk.decode([int(token_id)], skip_special_tokens=True)
        return text.encode("utf-8")


class SentencePieceTokenizer(Tokenizer):
    """``tokenizer.model`` / ``spiece.model`` / ``sentencepiece.bpe.model`` through the ``sentencepiece`` library
    (the reference parses the same protobuf itself, zig/lib/tokenizer/src/sentencepiece.zig)."""

    def __init__(self, path: str, config: Optional[dict] = None):
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=path)
        self.vocab_size = self.sp.get_piece_size()
        pick = lambda i: i if i is not None and i >= 0 else None
        self.special = SpecialTokens(cls_id=pick(self.sp.bos_id()) or 0, sep_id=pick(self.sp.eos_id()) or 0,
                                     pad_id=pick(self.sp.pad_id()) or 0, unk_id=pick(self.sp.unk_id()) or 0,
                                     bos_id=pick(self.sp.bos_id()), eos_id=pick(self.sp.eos_id()))

    def encode(self, text: str) -> List[int]:
        return list(self.sp.encode(text))

    def decode(self, ids: Sequence[int]) -> str:
        return self.sp.decode([int(i) for i in ids])

    def token_bytes(self, token_id: int) -> bytes:
        t = int(token_id)
        if self.sp.is_control(t) or self.sp.is_unknown(t):
            return b""
        if self.sp.is_byte(t):
            return bytes([int(self.sp.id_to_piece(t)[3:5], 16)])
        return self.sp.id_to_piece(t).replace("\u2581", " ").encode("utf-8")


class WordPieceTokenizer(Tokenizer):
    """BERT WordPiece (basic tokenisation: lower-case, strip accents, split punctuation; greedy longest-match with
    the ``##`` continuation prefix).  Used when only ``vocab.txt`` exists or the ``tokenizers`` wheel is missing."""

    def __init__(self, vocab: Dict[str, int], lower: bool = True, max_chars: int = 100):
        self.vocab, self.lower, self.max_chars = vocab, lower, max_chars
        self.inv = {i: t for t, i in vocab.items()}
        self.vocab_size = len(vocab)
        g = lambda t, d: vocab.get(t, d)
        self.special = SpecialTokens(g("[CLS]", 101), g("[SEP]", 102), g("[PAD]", 0), g("[UNK]", 100))

    @classmethod
    def from_vocab_file(cls, path: str, lower: bool = True) -> "WordPieceTokenizer":
        with open(path, encoding="utf-8") as f:
            return cls({line.rstrip("\n"): i for i, line in enumerate(f)}, lower)

    @staticmethod
    def _is_punct(ch: str) -> bool:
        cp = ord(ch)
        if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
            return True
        return unicodedata.category(ch).startswith("P")

    def _basic(self, text: str) -> List[str]:
        if self.lower:
            text = unicodedata.normalize("NFD", text.lower())
            text = "".join(c for c in text if unicodedata.category(c) != "Mn")
        out, cur = [], []
        for ch in text:
            if ch.isspace():
                if cur:
                    out.append("".join(cur)); cur = []
            elif self._is_punct(ch):
                if cur:
                    out.append("".join(cur)); cur = []
                out.append(ch)
            else:
                cur.append(ch)
        if cur:
            out.append("".join(cur))
        return out

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for word in self._basic(text):
            if len(word) > self.max_chars:
                ids.append(self.special.unk_id)
                continue
            start, sub = 0, []
            while start < len(word):
                end, cur = len(word), None
                while start < end:
                    piece = word[start:end] if start == 0 else "##" + word[start:end]
                    if piece in self.vocab:
                        cur = self.vocab[piece]
                        break
                    end -= 1
                if cur is None:
                    sub = [self.special.unk_id]
                    break
                sub.append(cur)
                start = end
            ids.extend(sub)
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        toks = [self.inv.get(int(i), "[UNK]") for i in ids]
        out = ""
        for t in toks:
            if t in ("[CLS]", "[SEP]", "[PAD]"):
                continue
            out += t[2:] if t.startswith("##") else (" " + t if out else t)
        return out


class ByteTokenizer(Tokenizer):
    """UTF-8 bytes + offset: a dependency-free tokenizer for random-init models, smoke tests and benchmarks."""

    def __init__(self, vocab_size: int = 512, offset: int = 3, bos_id: int = 1, eos_id: int = 2):
        self.vocab_size, self.offset = vocab_size, offset
        self.special = SpecialTokens(cls_id=bos_id, sep_id=eos_id, pad_id=0, unk_id=0, bos_id=bos_id, eos_id=eos_id)

    def encode(self, text: str) -> List[int]:
        return [min(b + self.offset, self.vocab_size - 1) for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        bs = bytes(max(0, min(255, int(i) - self.offset)) for i in ids if int(i) >= self.offset)
        return bs.decode("utf-8", errors="replace")


_BYTE_LEVEL_INV: Dict[str, int] = {}


def _byte_level_inverse() -> Dict[str, int]:
    """Character -> byte of the byte-level BPE alphabet: printable Latin-1 bytes stand for themselves, the other 68
    bytes are spelled as the code points from U+0100 upwards, in byte order."""
    if not _BYTE_LEVEL_INV:
        keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
        extra = 0
        for b in range(256):
            if b in keep:
                _BYTE_LEVEL_INV[chr(b)] = b
            else:
                _BYTE_LEVEL_INV[chr(256 + extra)] = b
                extra += 1
    return _BYTE_LEVEL_INV


class GGUFTokenizer(Tokenizer):
    """The tokenizer a GGUF file carries in its metadata (``tokenizer.ggml.*``).

    ``gpt2`` models: byte-level BPE from the token list and the merge list, control tokens as added tokens -- what
    the reference builds (zig/pkg/inference/src/server/model_manager.zig:406-466).  ``llama`` models: the
    SentencePiece-style BPE of those files (space -> U+2581 with a leading one, adjacent pieces merged in order of
    the vocabulary's scores, ``<0xXX>`` byte tokens for characters the vocabulary lacks)."""

    def __init__(self, metadata: dict):
        md = metadata
        self.kind = str(md.get("tokenizer.ggml.model", ""))
        self.tokens: List[str] = [str(t) for t in md.get("tokenizer.ggml.tokens") or []]
        if not self.tokens or self.kind not in ("gpt2", "llama"):
            raise ValueError(f"no usable tokenizer in the GGUF metadata (model {self.kind!r})")
        self.vocab_size = len(self.tokens)
        self.types = [int(t) for t in md.get("tokenizer.ggml.token_type") or []] or [1] * self.vocab_size
        tid = lambda k: int(md[k]) if md.get(k) is not None and 0 <= int(md[k]) < self.vocab_size else None
        bos, eos = tid("tokenizer.ggml.bos_token_id"), tid("tokenizer.ggml.eos_token_id")
        pad, unk = tid("tokenizer.ggml.padding_token_id"), tid("tokenizer.ggml.unknown_token_id")
        self.special = SpecialTokens(cls_id=bos or 0, sep_id=eos or 0, pad_id=pad or 0, unk_id=unk or 0,
                                     bos_id=bos, eos_id=eos)
        self.chat_template = md.get("tokenizer.chat_template")
        self.index = {t: i for i, t in enumerate(self.tokens)}
        self.control = {i for i, t in enumerate(self.types) if t == 3} | {x for x in (bos, eos, pad) if x is not None}
        if self.kind == "gpt2":
            from tokenizers import Tokenizer as _T, decoders, models, pre_tokenizers

            merges = [tuple(m.split(" ", 1)) for m in md.get("tokenizer.ggml.merges") or []]
            self.tk = _T(models.BPE(vocab=dict(self.index), merges=merges))
            self.tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            self.tk.decoder = decoders.ByteLevel()
            self.tk.add_special_tokens([self.tokens[i] for i in sorted(self.control)])
        else:
            self.scores = [float(x) for x in md.get("tokenizer.ggml.scores") or [0.0] * self.vocab_size]
            self.bytes = {int(t[3:5], 16): i for i, t in enumerate(self.tokens)
                          if len(t) == 6 and t.startswith("<0x") and t.endswith(">")}
            self.add_space_prefix = bool(md.get("tokenizer.ggml.add_space_prefix", True))

    @classmethod
    def from_file(cls, path: str) -> "GGUFTokenizer":
        from ..formats.gguf import GGUFFile

        return cls(GGUFFile(path).metadata)

    def _spm(self, text: str) -> List[int]:
        if not text:
            return []
        s = text.replace(" ", "\u2581")
        if self.add_space_prefix:
            s = "\u2581" + s
        parts = list(s)
        while len(parts) > 1:                       # merge the best-scoring adjacent pair that is a piece
            best, at = None, -1
            for i in range(len(parts) - 1):
                j = self.index.get(parts[i] + parts[i + 1])
                if j is not None and (best is None or self.scores[j] > best):
                    best, at = self.scores[j], i
            if at < 0:
                break
            parts[at:at + 2] = [parts[at] + parts[at + 1]]
        out: List[int] = []
        for p in parts:
            j = self.index.get(p)
            if j is not None:
                out.append(j)
                continue
            for b in p.encode("utf-8"):             # byte fallback, else the unknown token
                out.append(self.bytes.get(b, self.special.unk_id))
        return out

    def encode(self, text: str) -> List[int]:
        if self.kind == "gpt2":
            return list(self.tk.encode(text, add_special_tokens=False).ids)
        return self._spm(text)

    def token_bytes(self, token_id: int) -> bytes:
        t = int(token_id)
        if t in self.control or not 0 <= t < self.vocab_size:
            return b""
        if self.kind == "gpt2":                     # token text is bytes spelled in the byte-level alphabet
            return bytes(_byte_level_inverse()[c] for c in self.tokens[t] if c in _byte_level_inverse())
        piece = self.tokens[t]
        if len(piece) == 6 and piece.startswith("<0x") and piece.endswith(">"):
            return bytes([int(piece[3:5], 16)])
        return piece.replace("\u2581", " ").encode("utf-8")

    def decode(self, ids: Sequence[int]) -> str:
        ids = [int(i) for i in ids if int(i) not in self.control]
        if self.kind == "gpt2":
            return self.tk.decode(ids, skip_special_tokens=True)
        text = b"".join(self.token_bytes(i) for i in ids).decode("utf-8", "replace")
        return text[1:] if self.add_space_prefix and text.startswith(" ") else text


def load_tokenizer(model_dir: str, vocab_size: int = 0) -> Tokenizer:
    """tokenizer.json -> HFTokenizer; vocab.txt -> WordPiece; a GGUF file's own tokenizer; otherwise the byte tokenizer
    (selection order of zig/pkg/inference/src/server/model_manager.zig:383-520)."""
    cfg = {}
    for name in ("tokenizer_config.json", "special_tokens_map.json"):
        p = os.path.join(model_dir, name)
        if os.path.exists(p):
            with open(p, encoding="utf-8") as f:
                cfg.update(json.load(f))
    tj = os.path.join(model_dir, "tokenizer.json")
    if os.path.exists(tj):
        try:
            return HFTokenizer(tj, cfg)
        except ImportError:
            pass
    for name in ("tokenizer.model", "spiece.model", "sentencepiece.bpe.model"):
        sm = os.path.join(model_dir, name)
        if os.path.exists(sm):
            try:
                return SentencePieceTokenizer(sm, cfg)
            except ImportError:
                pass
    vt = os.path.join(model_dir, "vocab.txt")
    if os.path.exists(vt):
        return WordPieceTokenizer.from_vocab_file(vt, lower=cfg.get("do_lower_case", True))
    for name in sorted(os.listdir(model_dir)) if os.path.isdir(model_dir) else []:
        if name.endswith(".gguf"):                      # the tokenizer the weights file carries in its metadata
            try:
                return GGUFTokenizer.from_file(os.path.join(model_dir, name))
            except (ValueError, ImportError, KeyError):
                break
    return ByteTokenizer(vocab_size or 512)
