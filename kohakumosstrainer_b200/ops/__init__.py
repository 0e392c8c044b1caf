"""Op sets: the callables a model uses, resolved once per device.

`eager` is the numerical reference and the CPU path; `native` is the sm_100a CUDA path
(tcgen05 GEMMs, varlen attention, block ops). There is no per-call dispatch and no tuning
table: `resolve_ops(device)` picks the op set when the model is bound
(the reference's rule "select, don't dispatch": `src/kohakumoss/model/opset.py:21-124`).
"""

from __future__ import annotations

import torch

from . import eager
from .opset import EagerOps, OpSet

__all__ = ["eager", "OpSet", "EagerOps", "resolve_ops"]


def resolve_ops(device, kernels: dict | None = None) -> OpSet:
    """Op set for `device`. `kernels` is the `KERNELS` knob: `{"all": "eager"}` forces the
    reference path on CUDA for A/B runs; per-op pins (`{"attention_varlen": "eager"}`)
    replace single ops."""
    device = torch.device(device)
    kernels = dict(kernels or {})
    if device.type != "cuda" or kernels.get("all") == "eager":
        return EagerOps()
    from .native_ops import NativeOps

    return NativeOps(pins=kernels)
