"""Plain data types shared across layers: architecture config, packed-batch layout."""

from .arch import PRESETS, MossArchConfig
from .seqinfo import AttnPlan, SeqInfo, build_seqinfo

__all__ = ["PRESETS", "MossArchConfig", "AttnPlan", "SeqInfo", "build_seqinfo"]
