"""Vector indexes: exact (flat) search, k-means, IVF, RaBitQ, HBC tree, result fusion, wire codecs."""
from .distance import METRICS, resolve_search_effort  # noqa: F401
