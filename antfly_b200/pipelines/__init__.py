"""Task pipelines: embedding (dense / sparse), reranking (cross-encoder / late interaction), generation, chunking."""
