"""Helpers shared by the data scripts: data config from a script's knobs, encoder factories
from dotted paths (`src/kohakumoss_data/scripting.py` in the reference)."""

from __future__ import annotations

import importlib

from .dataset import DataConfig, MossDataset, data_problems


def data_config(knobs: dict, **forced) -> DataConfig:
    cfg = DataConfig.from_knobs({**knobs, **{k.upper(): v for k, v in forced.items()}})
    problems = data_problems(cfg)
    if problems:
        raise SystemExit("data config:\n  " + "\n  ".join(problems))
    return cfg


def build_encoder(path: str, kwargs: dict):
    """`module.factory` -> `factory(**kwargs)`."""
    module, _, name = path.rpartition(".")
    return getattr(importlib.import_module(module), name)(**kwargs)


def open_dataset(knobs: dict, **forced) -> MossDataset:
    return MossDataset(data_config(knobs, **forced))
