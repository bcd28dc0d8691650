"""Operators. Every op has a plain-PyTorch reference (the CPU oracle, also used for fp32 runs)
and an sm_100a implementation reached through the native kernel library on CUDA tensors."""
