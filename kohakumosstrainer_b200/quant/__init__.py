"""Stored and compute-time quantised weights: fp8 (tensor / row), MXFP8, int8 weight-only / compute, ConvRot."""

from .weights import Fp8Weight, QuantGroup, apply_base_precision, quantize_group, quantize_linear
from .formats import Int8Weight, MxFp8Weight, group_hadamard, hadamard_matrix, quantize_mxfp8, quantize_rows_int8

__all__ = ["Fp8Weight", "QuantGroup", "apply_base_precision", "quantize_group", "quantize_linear", "Int8Weight", "MxFp8Weight",
           "group_hadamard", "hadamard_matrix", "quantize_mxfp8", "quantize_rows_int8"]
