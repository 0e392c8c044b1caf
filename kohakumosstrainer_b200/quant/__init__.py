"""Stored and compute-time quantised weights: fp8 (tensor / row), MXFP8, int8 weight-only."""

from .weights import Fp8Weight, QuantGroup, apply_base_precision, quantize_group, quantize_linear

__all__ = ["Fp8Weight", "QuantGroup", "apply_base_precision", "quantize_group", "quantize_linear"]
