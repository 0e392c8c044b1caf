"""Adapter algorithm layer: lokr."""
ALGO = "lokr"
