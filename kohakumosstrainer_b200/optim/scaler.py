"""Loss scaling for fp16 compute (`src/kohakumoss/precision/scaler.py:9-115`).

bf16 (the default on B200) needs none: `NoScaler`. Under fp16 the loss is multiplied by a scale
so that small gradients survive the format; the bundle folds `1 / scale` into the clip
coefficient the optimiser kernel already multiplies gradients by, so unscaling costs no pass
over the gradients. `DeviceScaler` keeps the scale and the clean-step count as 0-d tensors on
the device and updates them from the step's non-finite flag without a host read, which is what
`STEP_SYNC="deferred"` needs; `DynamicScaler` is the same sequence of scales on the host.
"""

from __future__ import annotations

import torch
from torch import Tensor


class NoScaler:
    enabled = False

    def scale_loss(self, loss: Tensor) -> Tensor:
        return loss

    def inv_scale(self, device=None):
        return None

    def update(self, bad) -> None:
        pass

    def host_scale(self) -> float:
        return 1.0

    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, state: dict) -> None:
        pass


class DynamicScaler(NoScaler):
    """Back off (x `backoff`, floored at `floor`) on a non-finite step, grow (x `growth`)
    after `growth_interval` clean steps in a row."""

    enabled = True

    def __init__(self, init_scale: float = 2.0**16, growth: float = 2.0, backoff: float = 0.5, growth_interval: int = 2000,
                 floor: float = 1.0, ceiling: float = 2.0**24):
        self.scale, self.clean = float(init_scale), 0
        self.growth, self.backoff, self.interval, self.floor, self.ceiling = growth, backoff, int(growth_interval), floor, ceiling

    def scale_loss(self, loss: Tensor) -> Tensor:
        return loss * self.scale

    def inv_scale(self, device=None):
        return torch.full((1,), 1.0 / self.scale, device=device)

    def update(self, bad) -> None:
        if bool(bad):
            self.scale, self.clean = max(self.scale * self.backoff, self.floor), 0
            return
        self.clean += 1
        if self.clean >= self.interval:
            self.scale, self.clean = min(self.scale * self.growth, self.ceiling), 0

    def host_scale(self) -> float:
        return self.scale

    def state_dict(self) -> dict:
        return {"scale": self.host_scale(), "clean": int(self.clean)}

    def load_state_dict(self, state: dict) -> None:
        if state:
            self.scale, self.clean = float(state["scale"]), int(state["clean"])


class DeviceScaler(DynamicScaler):
    """The same sequence with scale and count held on `device`; `update` takes the step's
    flag as a tensor (non-zero = non-finite) and launches a handful of 0-d ops, no host read."""

    def __init__(self, device, **kw):
        super().__init__(**kw)
        self.device = torch.device(device)
        self._scale = torch.full((), self.scale, device=self.device)
        self._clean = torch.zeros((), device=self.device)

    def scale_loss(self, loss: Tensor) -> Tensor:
        return loss * self._scale.to(loss.dtype) if loss.dtype == torch.float32 else loss.float() * self._scale

    def inv_scale(self, device=None):
        return self._scale.reciprocal().reshape(1)

    def update(self, bad) -> None:
        bad = torch.as_tensor(bad, device=self.device).reshape(()).float() > 0
        clean = torch.where(bad, torch.zeros_like(self._clean), self._clean + 1)
        grow = clean >= self.interval
        scale = torch.where(bad, (self._scale * self.backoff).clamp_min(self.floor), self._scale)
        scale = torch.where(grow, (scale * self.growth).clamp_max(self.ceiling), scale)
        self._clean.copy_(torch.where(grow, torch.zeros_like(clean), clean))
        self._scale.copy_(scale)

    def host_scale(self) -> float:
        return float(self._scale)

    def state_dict(self) -> dict:
        return {"scale": self.host_scale(), "clean": int(self._clean)}

    def load_state_dict(self, state: dict) -> None:
        if state:
            self._scale.fill_(float(state["scale"]))
            self._clean.fill_(int(state["clean"]))


def build_scaler(precision: str, device, step_sync: str = "step", **kw):
    """`PRECISION` -> scaler: fp16 scales (on the device when the step must not sync), the rest do not."""
    if precision != "fp16":
        return NoScaler()
    return DeviceScaler(device, **kw) if step_sync == "deferred" or torch.device(device).type == "cuda" else DynamicScaler(**kw)
