"""Numerics helpers around the residual stream.

* `fold_stream_scale(model, s)`: the `weights` form of the reference's fp16 fix
  (`src/kohakumoss/numerics/fp16fix.py`, `numerics/fold.py`): every write into the residual stream
  (the two embedders, each block's `o` and `ffn_down`) is divided by `s`. Every reader normalises
  with RMSNorm first, so the function is unchanged while the stream's magnitude drops by `s` (fp16
  headroom; on a B200 the stream is bf16 and this is only needed to exchange files with fp16
  setups). `unfold_stream_scale` undoes it; the factor is recorded in file metadata
  (`kohakumoss_fp16_fix`).
* `keep_fp32(model, names)`: cast the named sub-modules to fp32 (`KEEP_FP32`).
* `SaturationCounter`: counts block outputs whose magnitude passes a threshold (forward hooks).
"""

from __future__ import annotations

import torch

WRITERS = ("o", "ffn_down")


def _writers(model):
    """Every linear whose output is added to (or starts) a residual stream: the embedders, the text
    blocks' `proj` / `ffn_down`, the joint blocks' `proj.o` / `proj.ffn_down`."""
    mods = [model.video_embedder, model.text_embedder.proj]
    for tb in model.text_embedder.blocks:
        mods += [tb.proj, tb.ffn_down]
    for layer in model.layers:
        mods += [layer.proj[n] for n in WRITERS]
    return mods


@torch.no_grad()
def fold_stream_scale(model, scale: float) -> int:
    n = 0
    for m in _writers(model):
        last = m[-1] if isinstance(m, torch.nn.Sequential) else m
        w = getattr(last, "weight", None)
        if w is None:
            continue
        w.div_(scale)
        if getattr(last, "bias", None) is not None:
            last.bias.div_(scale)
        n += 1
    model.__dict__["stream_scale"] = model.__dict__.get("stream_scale", 1.0) * scale
    return n


def unfold_stream_scale(model) -> int:
    s = model.__dict__.get("stream_scale", 1.0)
    return fold_stream_scale(model, 1.0 / s) if s != 1.0 else 0


def keep_fp32(model, names) -> list[str]:
    done = []
    for name in names:
        mod = getattr(model, name, None)
        if mod is not None:
            mod.float()
            done.append(name)
    return done


class SaturationCounter:
    def __init__(self, model, threshold: float = 6.0e4):
        self.threshold, self.counts, self.peaks = threshold, {}, {}
        for i, layer in enumerate(model.layers):
            layer.register_forward_hook(lambda m, a, out, i=i: self._see(i, out))

    def _see(self, i, out) -> None:
        if isinstance(out, torch.Tensor):
            peak = float(out.detach().abs().max())
            self.peaks[i] = max(self.peaks.get(i, 0.0), peak)
            if peak > self.threshold:
                self.counts[i] = self.counts.get(i, 0) + 1

    def row(self) -> dict:
        return {"detail/stream_peak": max(self.peaks.values(), default=0.0), "detail/saturated_blocks": len(self.counts)}
