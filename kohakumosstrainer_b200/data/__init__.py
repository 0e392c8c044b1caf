"""Data layer: host batches, resolution planning, packing, sources, caches, stateless loader."""

from .types import HostBatch
from .synthetic import SyntheticConfig, SyntheticDataset
from .geometry import Geometry
from .catalog import Catalog, Row
from .planner import PLANNERS, BatchPlan, PlanItem
from .captions import CAPTIONS, build_template
from .sources import SOURCES, build_source
from .store import LatentCache, TensorStore, TextCache, decode_tensor, encode_tensor, merge_shards
from .dataset import DataConfig, MossDataset, build_dataset, data_problems, encode_missing
from .loader import Loader, build_loader

__all__ = ["HostBatch", "SyntheticConfig", "SyntheticDataset", "Geometry", "Catalog", "Row", "PLANNERS", "BatchPlan", "PlanItem",
           "CAPTIONS", "build_template", "SOURCES", "build_source", "LatentCache", "TensorStore", "TextCache", "decode_tensor",
           "encode_tensor", "merge_shards", "DataConfig", "MossDataset", "build_dataset", "data_problems", "encode_missing",
           "Loader", "build_loader"]
