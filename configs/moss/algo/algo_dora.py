"""Adapter algorithm layer: dora."""
ALGO = "dora"
