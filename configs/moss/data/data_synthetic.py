"""Synthetic packed batches (no files needed)."""
DATASETS = [{"type": "synthetic"}]
MAX_TOKENS = 20480
