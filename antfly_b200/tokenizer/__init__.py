"""Tokenizers: HF ``tokenizer.json`` (through the ``tokenizers`` wheel when present), a built-in WordPiece, and a
byte-level fallback; plus the model-facing encode helpers with the reference's truncation rules
(zig/lib/tokenizer/src/tokenizer.zig:120-215)."""
from .tokenizer import ByteTokenizer, GGUFTokenizer, Tokenizer, WordPieceTokenizer, load_tokenizer  # noqa: F401
