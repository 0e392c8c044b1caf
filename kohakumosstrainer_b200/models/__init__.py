"""The MOSS-Image DiT: backbone, blocks, swappable linears, runners, checkpoint io."""

from .backbone import KEEP_FP32, MossBackbone
from .block import BlockCtx, JointBlock, TextBlock, TextEmbedder
from .build import build_backbone
from .linear import MossLinear

__all__ = [
    "KEEP_FP32", "MossBackbone", "BlockCtx", "JointBlock", "TextBlock", "TextEmbedder",
    "MossLinear", "build_backbone",
]
