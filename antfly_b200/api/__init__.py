"""HTTP server: the inference API (/ai/v1/...) and the vector search endpoint, plus model management and metrics."""
