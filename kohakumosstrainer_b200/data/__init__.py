"""Data layer: host batches, resolution planning, packing, sources, caches, stateless loader."""

from .types import HostBatch
from .synthetic import SyntheticConfig, SyntheticDataset

__all__ = ["HostBatch", "SyntheticConfig", "SyntheticDataset"]
