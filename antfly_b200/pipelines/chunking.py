"""Fixed-size text chunker (the reference's fixed chunker behind ``/chunk``: target tokens, overlap, separator
preference; zig/pkg/inference/src/pipelines/chunking.zig)."""
from __future__ import annotations

from typing import List


def chunk_text(text: str, target_tokens: int = 500, overlap_tokens: int = 50, max_chunks: int = 0,
               separator: str = "\n\n") -> List[dict]:
    words = text.split()
    if not words:
        return []
    step = max(target_tokens - overlap_tokens, 1)
    chunks, i, pos = [], 0, 0
    # Character offsets are tracked so callers can map chunks back into the source text.
    offsets, cursor = [], 0
    for w in words:
        cursor = text.index(w, cursor)
        offsets.append(cursor)
        cursor += len(w)
    while i < len(words):
        j = min(len(words), i + target_tokens)
        start, end = offsets[i], offsets[j - 1] + len(words[j - 1])
        chunks.append({"id": len(chunks), "text": text[start:end], "start_char": start, "end_char": end})
        if max_chunks and len(chunks) >= max_chunks:
            break
        if j == len(words):
            break
        i += step
    return chunks


class NeuralChunker:
    """Semantic chunking with a token-classification model that marks the tokens after which a new chunk starts
    (checkpoints in the style of the reference's ``chunkers/`` models, go/pkg/termite/lib/pipelines/chunking.go: a
    binary ``separator`` label per token).  Long texts are tagged in windows of the model's context; boundaries that
    would make a chunk longer than ``max_tokens`` are supplemented by a hard cut, tiny chunks are merged forward."""

    def __init__(self, tagger, boundary_labels=("separator", "B", "B-SEP", "LABEL_1"), window_tokens: int = 510,
                 threshold: float = 0.5):
        self.tagger, self.labels, self.window, self.threshold = tagger, set(boundary_labels), window_tokens, threshold

    def _pieces(self, text: str):
        """(token id, start char, end char) for the whole text, without special tokens."""
        tk = self.tagger.tokenizer
        inner = getattr(tk, "tk", None)
        if inner is not None and hasattr(inner, "encode"):            # Hugging Face tokenizers: exact offsets
            enc = inner.encode(text, add_special_tokens=False)
            return [(i, a, b) for i, (a, b) in zip(enc.ids, enc.offsets)]
        ids = tk.encode(text)
        out, cursor = [], 0
        for i in ids:                                                   # fall back to decoding token by token
            piece = tk.decode([i])
            at = text.find(piece, cursor) if piece else -1
            if at < 0:
                at = cursor
            out.append((i, at, at + len(piece)))
            cursor = at + len(piece)
        return out

    def chunk(self, text: str, max_tokens: int = 500, min_tokens: int = 8, max_chunks: int = 0) -> List[dict]:
        pieces = self._pieces(text)
        if not pieces:
            return []
        tk = self.tagger.tokenizer
        cls_id, sep_id = tk.special.cls_id, tk.special.sep_id
        cut_after = [False] * len(pieces)
        for lo in range(0, len(pieces), self.window):
            win = pieces[lo:lo + self.window]
            seq = [cls_id] + [p[0] for p in win] + [sep_id]
            tags, scores = self.tagger.tag_ids([seq])[0]
            for j in range(len(win)):
                if tags[j + 1] in self.labels and scores[j + 1] >= self.threshold:
                    cut_after[lo + j] = True
        chunks, start = [], 0
        for i in range(len(pieces)):
            n = i - start + 1
            last = i == len(pieces) - 1
            if last or n >= max_tokens or (cut_after[i] and n >= min_tokens):
                a, b = pieces[start][1], pieces[i][2]
                chunks.append({"id": len(chunks), "text": text[a:b], "start_char": a, "end_char": b, "tokens": n})
                start = i + 1
                if max_chunks and len(chunks) >= max_chunks:
                    break
        return chunks
