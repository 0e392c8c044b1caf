"""Channel-weighted RMSNorm and the heal anneal.

`WeightedOps` wraps an op set and normalises stream reads by sqrt(mean(lam * x^2) + eps) with a
shared per-channel `lam`: lam = 1 / D^2 makes a D-shrunk stream normalise exactly as the
original, lam = 1 is the plain RMSNorm. The anneal moves lam = (1 / D^2)^(1 - t) from t = 0
(exact) to t = 1 (plain) (`src/kohakumoss/heal/wnorm.py:15-75`).
"""

from __future__ import annotations

import torch
from torch import Tensor


def anneal_t(step: int, anneal_steps: int) -> float:
    return 1.0 if anneal_steps <= 0 else min(1.0, step / anneal_steps)


def anneal_lam(d: Tensor, t: float) -> Tensor:
    return d.reciprocal().square().pow(1.0 - t)


class WeightedOps:
    """Every op of `ops`, with `rms_norm` / `rms_norm_mod` over the weighted mean square for
    inputs of the stream width (other widths, e.g. per-head norms, pass through)."""

    def __init__(self, ops, dim: int, device):
        self._ops = ops
        self.dim = dim
        self.lam = torch.ones(dim, dtype=torch.float32, device=device)

    def __getattr__(self, name):
        return getattr(self.__dict__["_ops"], name)

    def _normed(self, x: Tensor, eps: float) -> Tensor:
        xf = x.float()
        ms = (xf.square() * self.lam).mean(-1, keepdim=True)
        return xf * torch.rsqrt(ms + eps)

    def rms_norm(self, x, weight, eps):
        if x.shape[-1] != self.dim:
            return self._ops.rms_norm(x, weight, eps)
        y = self._normed(x, eps)
        if weight is not None:
            y = y * weight.float()
        return y.to(x.dtype)

    def rms_norm_mod(self, x, weight, shift, scale, seg, eps):
        if x.shape[-1] != self.dim:
            return self._ops.rms_norm_mod(x, weight, shift, scale, seg, eps)
        y = self._normed(x, eps)
        if weight is not None:
            y = y * weight.float()
        if scale is not None:
            y = y * (1.0 + scale.float().index_select(0, seg.long()))
        if shift is not None:
            y = y + shift.float().index_select(0, seg.long())
        return y.to(x.dtype)
