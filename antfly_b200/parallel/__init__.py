"""Multi-GPU plumbing: process-group bootstrap, weight sharding rules, symmetric-memory fused collectives."""
