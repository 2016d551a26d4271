"""antfly_b200: a Blackwell-native inference-and-retrieval engine (embedding, reranking, generation with paged
KV cache and speculative decoding, vector search) with hand-written sm_100a kernels under a PyTorch shell."""
import os as _os

__version__ = "0.1.0"

# The peer-memory kernels of this package use plain loads / stores through peer pointers only, never multimem.
# PyTorch's symmetric-memory allocator would otherwise also bind every symmetric buffer to an NVLink multicast
# object when the fabric supports it; a rank that dies while so bound can raise NVLink faults on its peers' GPUs.
# Nothing here needs the multicast mapping, so ask the allocator not to create it (honoured where the installed
# PyTorch knows the switch; set before the allocator's first use).
_os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
# NCCL would likewise bind its own buffers to NVLink multicast objects (NVLS) for the bootstrap / baseline
# collectives; the same hazard applies when a rank goes away, and nothing here depends on in-switch reduction.
# A caller that wants NVLS back sets the variable before importing the package.
_os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
