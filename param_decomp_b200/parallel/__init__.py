"""Mesh topology, placement rules, symmetric memory and the fused compute+collective kernels."""
