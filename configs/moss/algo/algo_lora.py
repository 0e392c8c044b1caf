"""Adapter algorithm layer: lora."""
ALGO = "lora"
