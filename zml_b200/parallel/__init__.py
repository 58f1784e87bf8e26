"""Sharding math, process groups, symmetric memory and fused compute+collective kernels."""
