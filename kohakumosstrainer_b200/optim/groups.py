"""Parameter groups and the weight-decay rules (`WD_RULES`).

`moss`: no decay on tensors with ndim < 2, norm weights, biases and embedders; in full
finetune the q/k norm weights of the last block decay towards one
(`src/kohakumoss/training/optim/groups.py:9-37`, `docs/concepts/training.md:310-353`).
"""

from __future__ import annotations

import re

import torch

NO_DECAY = re.compile(r"(norm|bias|video_embedder|text_embedder\.proj|w_norm|dora_scale|alpha)")


def weight_decay_rule(name: str, p: torch.Tensor, rule: str = "moss") -> bool:
    if rule == "none":
        return False
    if rule == "all":
        return True
    if rule != "moss":
        raise ValueError(f"WD_RULES must be moss|none|all, got {rule}")
    return p.ndim >= 2 and not NO_DECAY.search(name)


def param_groups(named_params, weight_decay: float, rule: str = "moss", decay_to_one: tuple[str, ...] = (),
                 lr_mul: dict | None = None) -> list[dict]:
    """Split `(name, param)` pairs into decay / no-decay / decay-to-one groups; `lr_mul`
    maps a regex to a learning-rate multiplier (LoRA+)."""
    buckets: dict[tuple, list] = {}
    for name, p in named_params:
        if not p.requires_grad:
            continue
        to_one = any(re.search(pat, name) for pat in decay_to_one)
        wd = weight_decay if (to_one or weight_decay_rule(name, p, rule)) else 0.0
        mul = 1.0
        for pat, m in (lr_mul or {}).items():
            if re.search(pat, name):
                mul = m
        buckets.setdefault((wd, to_one, mul), []).append(p)
    return [dict(params=ps, weight_decay=wd, decay_to_one=to_one, lr_mul=mul) for (wd, to_one, mul), ps in buckets.items()]


def is_muon_param(name: str, p: torch.Tensor) -> bool:
    """Muon takes the 2-D hidden matrices of the blocks; embeddings, the head, modulation,
    norms and biases stay on AdamW."""
    if p.ndim != 2:
        return False
    return bool(re.search(r"(layers\.\d+\.proj\.|text_embedder\.blocks\.\d+\.(qkv|proj|ffn_))", name))
