"""Artifact formats: safetensors (read / write), GGUF v3 (read, dequantise), model-directory manifests."""
