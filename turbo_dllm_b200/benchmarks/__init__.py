"""Micro-benchmarks of single kernels (CUDA-event timing, L2 flushed between iterations)."""
