"""Fixed-address decode sessions: one C-ABI call per token, capturable in a CUDA graph."""
