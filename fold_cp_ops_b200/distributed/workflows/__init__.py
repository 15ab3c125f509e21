"""Distributed workflows: the fused context-parallel TriMul front door."""
