"""Parallelism plumbing: tensor-parallel region functions, symmetric-memory collectives,
mesh construction."""
