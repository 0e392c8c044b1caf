"""Channel statistics and the shrink of massive channels.

A few residual-stream channels of the DiT carry magnitudes hundreds of times the median
("massive channels"); they dominate quantisation ranges and fp16 headroom. The shrink scales
stream channel c by D_c = min(1, tau / M_c) in every WRITER (embedders, text-refiner `proj` /
`ffn_down`, joint `o` / `ffn_down`) and every READER norm gain by 1 / D_c, where M_c is the
channel's peak RMS over the median channel's, across all reader-norm sites
(`src/kohakumoss/heal/channels.py:14-70`, `heal/calibrate.py:28-150`).
"""

from __future__ import annotations

import numpy as np
import torch
from torch import Tensor


def reader_norms(model) -> dict[str, torch.nn.Module]:
    """site name -> RMSNorm module that reads the residual stream."""
    out = {}
    for t, tb in enumerate(model.text_embedder.blocks):
        out[f"text.{t}.norm1"], out[f"text.{t}.norm2"] = tb.norm1, tb.norm2
    for i, layer in enumerate(model.layers):
        out[f"joint.{i}.norm1"], out[f"joint.{i}.norm2"] = layer.norm1, layer.norm2
    out["final"] = model.final_norm_video
    return out


def writer_params(model) -> list[tuple[str, torch.nn.Parameter]]:
    """Every parameter whose rows are stream channels (weights and biases of the writers)."""
    named = []
    mods = {"video_embedder": model.video_embedder, "text_embedder.proj": model.text_embedder.proj}
    for t, tb in enumerate(model.text_embedder.blocks):
        mods[f"text_embedder.blocks.{t}.proj"], mods[f"text_embedder.blocks.{t}.ffn_down"] = tb.proj, tb.ffn_down
    for i, layer in enumerate(model.layers):
        mods[f"layers.{i}.proj.o"], mods[f"layers.{i}.proj.ffn_down"] = layer.proj["o"], layer.proj["ffn_down"]
    for name, m in mods.items():
        last = m[-1] if isinstance(m, torch.nn.Sequential) else m
        for pn in ("weight", "bias"):
            p = getattr(last, pn, None)
            if isinstance(p, torch.nn.Parameter):
                named.append((f"{name}.{pn}", p))
    return named


class _Taps:
    """Per-channel mean square of what each reader norm sees (hooks on the op set's norm calls
    would miss fused paths, so the taps wrap the norm WEIGHT access: the block passes
    `norm.weight` next to `x`; the forward pre-hook of the block records x instead)."""

    def __init__(self, model):
        self.sums: dict[str, Tensor] = {}
        self.counts: dict[str, int] = {}
        self.handles = []
        self.model = model

    def see(self, site: str, x: Tensor) -> None:
        ms = x.detach().float().square().mean(0)
        self.sums[site] = self.sums.get(site, 0) + ms
        self.counts[site] = self.counts.get(site, 0) + 1


def channel_mean_square(model, batches, forward) -> dict[str, np.ndarray]:
    """site -> per-channel mean square of the norm's input over `batches`; `forward(batch)` runs
    the model. The op set is wrapped for the duration, so every stream-reading norm is seen."""
    taps = _Taps(model)
    ops = model.ops

    class Tapped:
        def __getattr__(self, name):
            return getattr(ops, name)

        def rms_norm(self, x, weight, eps):
            taps.see(_site_of(model, weight), x)
            return ops.rms_norm(x, weight, eps)

        def rms_norm_mod(self, x, weight, shift, scale, seg, eps):
            taps.see(_site_of(model, weight), x)
            return ops.rms_norm_mod(x, weight, shift, scale, seg, eps)

    model.bind_ops(Tapped())
    try:
        with torch.no_grad():
            for b in batches:
                forward(b)
    finally:
        model.bind_ops(ops)
    return {s: (taps.sums[s] / taps.counts[s]).cpu().numpy() for s in taps.sums}


def _site_of(model, weight) -> str:
    for site, norm in reader_norms(model).items():
        if norm.weight is weight:
            return site
    return "other"


def peak_ratio(mean_square: dict[str, np.ndarray]) -> np.ndarray:
    """M_c: max over sites of channel c's RMS over the median channel's RMS."""
    rel = [np.sqrt(v) / max(np.median(np.sqrt(v)), 1e-30) for k, v in mean_square.items() if k != "other"]
    return np.stack(rel).max(0)


def shrink_scales(peak: np.ndarray, tau: float) -> Tensor:
    """D_c = min(1, tau / M_c)."""
    return torch.tensor(np.minimum(1.0, tau / np.maximum(peak, 1e-30)), dtype=torch.float32)


def top_channels(peak: np.ndarray, n: int = 32) -> list[list]:
    order = np.argsort(-peak)[:n]
    return [[int(c), round(float(peak[c]), 2)] for c in order]


@torch.no_grad()
def apply_shrink(model, d: Tensor, gains: bool = True) -> None:
    """Writers' rows times D_c; with `gains`, reader norm gains times 1 / D_c (the exact form used
    when norms stay plain RMSNorm requires the channel-weighted norm, see `wnorm`)."""
    for _, p in writer_params(model):
        m = d.to(p.device, torch.float32)
        p.copy_((p.float() * m.reshape(-1, *([1] * (p.dim() - 1)))).to(p.dtype))
    if gains:
        for norm in reader_norms(model).values():
            norm.weight.copy_((norm.weight.float() / d.to(norm.weight.device)).to(norm.weight.dtype))
