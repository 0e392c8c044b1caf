"""Block runners: how one joint block is executed (plain, activation checkpointing).

Modes follow the reference's `CHECKPOINT` knob (`src/kohakumoss/memory/runners.py:94-210`):
`none`, `block` (recompute the whole block in backward), `sub-block` (attention part and
FFN part checkpointed separately), `partial:f` (checkpoint the first fraction f of blocks).
"""

from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint


class PlainRunner:
    name = "none"

    def run(self, index, block, x, ctx):
        return block(x, ctx)


class BlockCheckpointRunner:
    name = "block"

    def run(self, index, block, x, ctx):
        if not torch.is_grad_enabled():
            return block(x, ctx)
        return checkpoint(block, x, ctx, use_reentrant=False)


class SubBlockCheckpointRunner:
    name = "sub-block"

    def run(self, index, block, x, ctx):
        if not torch.is_grad_enabled():
            return block(x, ctx)
        for part in block.sub_blocks():
            x = checkpoint(part, x, ctx, use_reentrant=False)
        return x


class PartialCheckpointRunner:
    """Checkpoint blocks with index < fraction * depth; run the rest plainly."""

    def __init__(self, fraction: float, depth: int):
        self.name = f"partial:{fraction:g}"
        self.cut = int(round(fraction * depth))
        self._ckpt, self._plain = BlockCheckpointRunner(), PlainRunner()

    def run(self, index, block, x, ctx):
        return (self._ckpt if index < self.cut else self._plain).run(index, block, x, ctx)


def build_runner(mode: str, depth: int):
    if mode in ("none", "", None):
        return PlainRunner()
    if mode == "block":
        return BlockCheckpointRunner()
    if mode in ("sub-block", "selective"):
        return SubBlockCheckpointRunner()
    if mode.startswith("partial:"):
        return PartialCheckpointRunner(float(mode.split(":", 1)[1]), depth)
    raise ValueError(f"unknown CHECKPOINT mode {mode!r}")
