"""Rectified-flow noising, token losses and the global token-count normalisation.

`z_sigma = z0 + sigma (eps - z0)`, target `eps - z0`; the loss is the sum over image tokens of
`weight[sample] * mean_c(err)` divided by the GLOBAL image-token count of the optimiser step
(all micro-batches, all ranks), so gradients are summed across ranks, never averaged
(`src/kohakumoss/diffusion/objective/{flow,loss,weighting,normalize}.py`).
"""

from __future__ import annotations

from collections.abc import Callable

import torch
from torch import Tensor

from ..utils.registry import Registry

LOSSES = Registry("loss")
WEIGHTINGS = Registry("loss weighting")


def noise_latents(z0: Tensor, eps: Tensor, sigma: Tensor, seg_img: Tensor) -> tuple[Tensor, Tensor]:
    """(z_sigma, velocity target) for per-sample sigma [B]."""
    s = sigma.to(z0.dtype).index_select(0, seg_img.long()).unsqueeze(-1)
    return z0 + s * (eps - z0), eps - z0


@LOSSES.register("mse")
def _mse(err: Tensor, **_kw) -> Tensor:
    return err.square().mean(-1)


@LOSSES.register("l1")
def _l1(err: Tensor, **_kw) -> Tensor:
    return err.abs().mean(-1)


@LOSSES.register("huber")
def _huber(err: Tensor, delta: float = 1.0, **_kw) -> Tensor:
    a = err.abs()
    return torch.where(a <= delta, 0.5 * err.square(), delta * (a - 0.5 * delta)).mean(-1)


LOSSES.register("masked_mse", _mse)


@WEIGHTINGS.register("none")
def _w_none(sigma: Tensor) -> Tensor:
    return torch.ones_like(sigma)


@WEIGHTINGS.register("x0")
def _w_x0(sigma: Tensor) -> Tensor:
    """Weight of an x0-prediction loss expressed on velocity: 1 / sigma^2 (clamped)."""
    return 1.0 / sigma.clamp_min(1e-3).square()


@WEIGHTINGS.register("eps")
def _w_eps(sigma: Tensor) -> Tensor:
    return 1.0 / (1.0 - sigma).clamp_min(1e-3).square()


def token_loss(ops, pred: Tensor, target: Tensor, seg: Tensor, weight: Tensor, mask: Tensor | None = None,
               loss: str = "mse", **loss_kwargs) -> Tensor:
    """Sum over tokens of weight[seg] * mask * per-token loss (fp32). `mse` runs the op set's
    fused kernel; the others are composed in torch."""
    if loss in ("mse", "masked_mse") and not loss_kwargs:
        return ops.token_mse(pred, target, seg, weight, mask)
    per_token = LOSSES.get(loss)(pred.float() - target.float(), **loss_kwargs)
    w = weight.float().index_select(0, seg.long())
    if mask is not None:
        w = w * mask.float()
    return (per_token * w).sum()


class TokenNormalizer:
    """Turns local image-token counts into the global denominator (int64 on device).

    `reduce` is an in-place SUM all-reduce over the data-parallel group (identity for one
    rank). The host count reaches the device through pinned memory: no host sync."""

    def __init__(self, reduce: Callable[[Tensor], Tensor] | None = None, world_factor: int = 1):
        self.reduce = reduce or (lambda t: t)
        self.world_factor = world_factor

    def denominator(self, local_count: int | Tensor, device) -> Tensor:
        device = torch.device(device)
        if isinstance(local_count, Tensor):
            t = local_count.to(device=device, dtype=torch.int64).reshape(1).clone()
        elif device.type == "cuda":
            t = torch.tensor([int(local_count)], dtype=torch.int64).pin_memory().to(device, non_blocking=True)
        else:
            t = torch.tensor([int(local_count)], dtype=torch.int64)
        return self.reduce(t).clamp_min(1)

    def __call__(self, loss_sum: Tensor, denom: Tensor) -> Tensor:
        return loss_sum * self.world_factor / denom.to(loss_sum.dtype)
