"""Adapter algorithm layer: loha."""
ALGO = "loha"
