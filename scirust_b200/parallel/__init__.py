"""Parallel runtime: process groups, symmetric (peer-mapped) memory, fused collectives,
data/tensor parallel layers, logical device meshes, and the host-side fixed-order collectives."""
