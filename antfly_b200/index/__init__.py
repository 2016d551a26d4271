"""Vector indexes: exact (flat) search, k-means, IVF, RaBitQ, HBC tree, HNSW graph, result fusion, wire codecs."""
from .distance import METRICS, resolve_search_effort  # noqa: F401
