"""Multi-GPU plumbing: process group helpers, peer-mapped buffers, fused and reference-style synchronisers."""
