"""Comparison arms that are not part of the product (timed by bench.py only)."""
