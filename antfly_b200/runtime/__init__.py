"""Serving runtime: paged KV cache, continuous-batching scheduler, sampling parameters, generation engine."""
