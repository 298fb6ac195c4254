"""Runtime twins: the authored functions' signatures over the C-ABI kernels."""
