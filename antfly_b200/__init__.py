"""antfly_b200: a Blackwell-native inference-and-retrieval engine (embedding, reranking, generation with paged
KV cache and speculative decoding, vector search) with hand-written sm_100a kernels under a PyTorch shell."""
__version__ = "0.1.0"
