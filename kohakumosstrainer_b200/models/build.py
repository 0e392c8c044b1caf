"""Model construction helpers: meta-device build, random init, dtype placement.

`build_backbone` covers what the reference spreads over `model/build.py:26-110` and
`precision/config.py:45`: build on `meta`, materialise on the target device, keep the
conditioning linears in fp32 (`KEEP_FP32`), cast the trunk to the compute dtype.
"""

from __future__ import annotations

import torch

from ..types.arch import PRESETS, MossArchConfig
from .backbone import KEEP_FP32, MossBackbone


def resolve_arch(variant: str = "base", overrides: dict | None = None) -> MossArchConfig:
    cfg = PRESETS[variant]
    return cfg.override(**overrides) if overrides else cfg


def apply_param_dtypes(model: MossBackbone, dtype: torch.dtype, keep_fp32=KEEP_FP32) -> None:
    """Cast every parameter to `dtype` except the modules named in `keep_fp32`."""
    keep = tuple(keep_fp32)
    for name, module in model.named_children():
        if name in keep:
            module.to(torch.float32)
        else:
            module.to(dtype)


def build_backbone(
    cfg: MossArchConfig | str = "base",
    device="cpu",
    dtype: torch.dtype = torch.float32,
    seed: int | None = 0,
    std: float = 0.02,
    keep_fp32=KEEP_FP32,
    init: bool = True,
) -> MossBackbone:
    """A backbone on `device` with random-init weights (or uninitialised when
    `init=False`, for loading a checkpoint into)."""
    if isinstance(cfg, str):
        cfg = PRESETS[cfg]
    device = torch.device(device)
    with torch.device("meta"):
        model = MossBackbone(cfg)
    model.to_empty(device=device)
    apply_param_dtypes(model, dtype, keep_fp32)
    if init:
        gen = None
        if seed is not None:
            gen = torch.Generator(device=device).manual_seed(seed)
        with torch.no_grad():
            model.init_weights(std, gen)
    model.rope._apply(lambda t: t)
    return model.bind_ops()
