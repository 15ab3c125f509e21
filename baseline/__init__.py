"""Comparison targets measured beside the fused path on the same box (not part of the product)."""
