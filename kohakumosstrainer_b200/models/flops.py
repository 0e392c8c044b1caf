"""FLOP model of a DiT step and nominal peaks (`src/kohakumoss/model/flops.py:8-56`), with a
B200 row the reference table lacks. Used by the throughput callback for TFLOP/s and MFU."""

from __future__ import annotations

PEAK_TFLOPS = {"B200": {"bf16": 2250.0, "fp8": 4500.0}, "B300": {"bf16": 2500.0, "fp8": 5000.0}, "H100": {"bf16": 989.0, "fp8": 1979.0}}


def forward_flops(cfg, joint_lengths, n_img: int | None = None, n_txt: int | None = None) -> float:
    """Multiply-add FLOPs (x2) of one forward over packed segments of `joint_lengths`."""
    n = sum(joint_lengths)
    d, f = cfg.dim, cfg.ffn_dim
    linear = 2.0 * n * cfg.depth * (4 * d * d + 3 * d * f)
    attn = sum(4.0 * l * l * d for l in joint_lengths) * cfg.depth
    n_txt = n_txt if n_txt is not None else 0
    text = 2.0 * n_txt * (cfg.text_dim * d + cfg.text_blocks * (4 * d * d + 3 * d * f))
    n_img = n_img if n_img is not None else n
    embed = 2.0 * n_img * cfg.latent_channels * d * 2
    return linear + attn + text + embed


def step_flops(cfg, joint_lengths, trainable_base: bool, checkpointing: bool = False, **kw) -> float:
    """Forward + backward: backward = dgrad (1x forward) plus wgrad (1x) when the base trains;
    activation checkpointing adds one forward."""
    fwd = forward_flops(cfg, joint_lengths, **kw)
    return fwd * (3.0 if trainable_base else 2.0) + (fwd if checkpointing else 0.0)
