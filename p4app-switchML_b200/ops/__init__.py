"""Kernel-level operations: the CPU oracle, the single-GPU emulation of the aggregation
kernels, and the tcgen05 weight-gradient GEMM."""
