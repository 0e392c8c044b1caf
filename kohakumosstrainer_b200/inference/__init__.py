"""Inference: `MossPipeline` (load, encode, sample, decode) and data-parallel sampling."""

from .pipeline import MossPipeline, SampleRequest

__all__ = ["MossPipeline", "SampleRequest"]
