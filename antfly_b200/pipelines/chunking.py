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
