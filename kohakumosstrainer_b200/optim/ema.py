"""Exponential moving averages of the trainable weights (fp32 buffers).

`ConstantEMA`: `ema <- lerp(ema, p, 1 - min(decay, (1 + t) / (10 + t)))`; `PowerEMA`: the
EDM2 power-function profile per `sigma_rel`, with snapshots for post-hoc reconstruction
(`src/kohakumoss/training/ema/averagers.py:85-363`, `ema/posthoc.py`). With the fused AdamW
the first decay's buffers are updated inside the optimiser kernel (`attach_to`), so the EMA
costs no extra pass over the parameters; other decays use one multi-tensor launch each.
Checkpoint keys are `<tag>/<name>` with tags `ema0.9999` / `power0.05`.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor


def _warm(decay: float, t: int) -> float:
    return min(decay, (1 + t) / (10 + t))


class _BufferEMA:
    def __init__(self, named, tags: list[str], device=None):
        self.names, self.params = [], []
        for name, p in named:
            if p.requires_grad:
                self.names.append(name)
                self.params.append(p)
        self.tags = tags
        self.buffers = {
            tag: [p.detach().to(device=device or p.device, dtype=torch.float32).clone() for p in self.params] for tag in tags
        }
        self.fused_tag: str | None = None

    def attach_to(self, optimizer) -> bool:
        """Let `optimizer` (FusedAdamW / MuonHybrid) update the first tag inside its step."""
        if not hasattr(optimizer, "attach_ema") or not self.tags:
            return False
        tag = self.tags[0]
        optimizer.attach_ema({id(p): b for p, b in zip(self.params, self.buffers[tag])})
        self.fused_tag = tag
        self._optimizer = optimizer
        return True

    def _lerp(self, tag: str, weight: float) -> None:
        bufs = self.buffers[tag]
        if tag == self.fused_tag:
            return
        if bufs and bufs[0].device == self.params[0].device:
            torch._foreach_lerp_(bufs, [p.detach().float() for p in self.params], weight)
        else:
            for b, p in zip(bufs, self.params):
                b.lerp_(p.detach().to(b.device, torch.float32), weight)

    def averaged(self, tag: str | None = None) -> dict[str, Tensor]:
        tag = tag or self.tags[0]
        return dict(zip(self.names, self.buffers[tag]))

    def state_dict(self) -> dict[str, Tensor]:
        return {f"{tag}/{name}": b for tag in self.tags for name, b in zip(self.names, self.buffers[tag])}

    def load_state_dict(self, state: dict[str, Tensor]) -> None:
        for tag in self.tags:
            for name, b in zip(self.names, self.buffers[tag]):
                b.copy_(state[f"{tag}/{name}"])

    @torch.no_grad()
    def copy_to(self, tag: str | None = None) -> list[Tensor]:
        """Swap the averaged weights into the parameters; returns the originals for `restore`."""
        tag = tag or self.tags[0]
        saved = [p.detach().clone() for p in self.params]
        for p, b in zip(self.params, self.buffers[tag]):
            p.copy_(b.to(p.device, p.dtype))
        return saved

    @torch.no_grad()
    def restore(self, saved: list[Tensor]) -> None:
        for p, s in zip(self.params, saved):
            p.copy_(s)


class ConstantEMA(_BufferEMA):
    def __init__(self, named, decays=(0.9999,), warmup: bool = True, device=None):
        decays = tuple(decays) if isinstance(decays, (tuple, list)) else (float(decays),)
        super().__init__(named, [f"ema{d:g}" for d in decays], device)
        self.decays, self.warmup = decays, warmup

    def decay_at(self, i: int, step: int) -> float:
        t = step + 1
        return _warm(self.decays[i], t) if self.warmup else self.decays[i]

    def before_step(self, step: int) -> None:
        """Tell the fused optimiser which decay the coming step uses."""
        if self.fused_tag is not None:
            self._optimizer.ema_decay = self.decay_at(0, step)

    @torch.no_grad()
    def update(self, step: int) -> None:
        for i, tag in enumerate(self.tags):
            self._lerp(tag, 1.0 - self.decay_at(i, step))


def power_gamma(sigma_rel: float) -> float:
    """Exponent gamma of the power-function EMA with relative width `sigma_rel` (EDM2):
    the positive root of sigma_rel^2 = (g + 1) / ((g + 2)^2 (g + 3))."""
    lo, hi = 0.0, 1e4
    f = lambda g: (g + 1) / ((g + 2) ** 2 * (g + 3)) - sigma_rel**2
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if f(mid) > 0:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


class PowerEMA(_BufferEMA):
    def __init__(self, named, sigma_rels=(0.05,), device=None):
        sigma_rels = tuple(sigma_rels) if isinstance(sigma_rels, (tuple, list)) else (float(sigma_rels),)
        super().__init__(named, [f"power{s:g}" for s in sigma_rels], device)
        self.sigma_rels = sigma_rels
        self.gammas = tuple(power_gamma(s) for s in sigma_rels)

    def decay_at(self, i: int, step: int) -> float:
        t = step + 1
        return (1 - 1 / t) ** (self.gammas[i] + 1)

    def before_step(self, step: int) -> None:
        if self.fused_tag is not None:
            self._optimizer.ema_decay = self.decay_at(0, step)

    @torch.no_grad()
    def update(self, step: int) -> None:
        for i, tag in enumerate(self.tags):
            self._lerp(tag, 1.0 - self.decay_at(i, step))


def posthoc_weights(snapshot_steps: list[int], gamma_src: float, step_target: int, gamma_target: float) -> Tensor:
    """Least-squares coefficients that combine power-EMA snapshots (all taken with
    `gamma_src`) into the profile `(step_target, gamma_target)` (EDM2 appendix C)."""

    def dot(ta, ga, tb, gb):
        tmax, tmin = max(ta, tb), min(ta, tb)
        ratio = tmin / tmax
        num = (ga + 1) * (gb + 1) * ratio ** (ga if ta >= tb else gb)
        return num / ((ga + gb + 1) * tmax)

    n = len(snapshot_steps)
    a = torch.tensor([[dot(snapshot_steps[i], gamma_src, snapshot_steps[j], gamma_src) for j in range(n)] for i in range(n)], dtype=torch.float64)
    b = torch.tensor([dot(snapshot_steps[i], gamma_src, step_target, gamma_target) for i in range(n)], dtype=torch.float64)
    return torch.linalg.lstsq(a, b.unsqueeze(1)).solution.squeeze(1).float()
