"""Adapter algorithm layer: oft."""
ALGO = "oft"
