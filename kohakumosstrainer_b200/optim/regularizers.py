"""Decay terms applied after the optimiser step: start anchors and outlier decay.

* `StartAnchors` (`WD_TARGET="start"`, `src/kohakumoss/training/build/anchors.py:14-60`): the
  optimiser's decoupled decay pulls a weight towards zero, `p -= lr wd p`; adding `lr wd a` with
  `a` the weight the run started from turns that into a pull towards the start,
  `p -= lr wd (p - a)`. The anchors are bf16 copies (2 bytes per decayed parameter).
* `OutlierDecay` (`OUTLIER_DECAY`, `src/kohakumoss/training/optim/outlier.py`): each element's
  excess over `cap` times the tensor's start RMS `r0` decays,
  `p -= lr rate(t) sign(p) relu(|p| - cap(t) r0)`; `rate` warms up linearly over `warmup` steps
  and `cap` anneals from `cap_start` to `cap` over `cap_anneal` steps.

Both run as a few multi-tensor (`torch._foreach_*`) launches over all targeted tensors, read the
group's current lr, and are gated by the step's device skip flag, so they add no host
synchronisation. They are called from the bundle's `post_step`.
"""

from __future__ import annotations

import re

import torch
from torch import Tensor

ANCHOR_OPTIMIZERS = ("adamw", "adamw16", "adamw8bit", "adamw8bit_kernel", "muon")
OUTLIER_DEFAULTS = {"rate": 0.0, "cap": 16.0, "cap_start": 0.0, "cap_anneal": 0, "warmup": 0, "targets": "", "exclude": "",
                    "include_1d": False}


def _gate(skip: Tensor | None, device) -> Tensor | float:
    return 1.0 if skip is None else (1.0 - (skip.reshape(()) != 0).float()).to(device)


class StartAnchors:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.anchors: dict[int, Tensor] = {}
        for g in optimizer.param_groups:
            if g.get("weight_decay", 0.0) > 0 and not g.get("decay_to_one", False):
                for p in g["params"]:
                    self.anchors[id(p)] = p.detach().to(torch.bfloat16).clone()

    def load(self, named_start: dict[str, Tensor], names: dict[int, str]) -> None:
        """Anchors of a resumed run come from the file the run started from, not the restored weights."""
        for pid, name in names.items():
            if pid in self.anchors and name in named_start:
                self.anchors[pid].copy_(named_start[name].to(self.anchors[pid]))

    @torch.no_grad()
    def apply(self, skip: Tensor | None = None) -> None:
        for g in self.optimizer.param_groups:
            wd = g.get("weight_decay", 0.0)
            params = [p for p in g["params"] if id(p) in self.anchors]
            if not params or wd <= 0:
                continue
            coef = g["lr"] * g.get("lr_mul", 1.0) * wd * _gate(skip, params[0].device)
            adds = torch._foreach_mul([self.anchors[id(p)].float() for p in params], coef)
            for p, a in zip(params, adds):
                p.add_(a.to(p.dtype))


class OutlierDecay:
    def __init__(self, named_params, optimizer, spec: dict):
        self.spec = {**OUTLIER_DEFAULTS, **spec}
        unknown = set(spec) - set(OUTLIER_DEFAULTS)
        if unknown:
            raise ValueError(f"OUTLIER_DECAY keys {sorted(unknown)} unknown (have {sorted(OUTLIER_DEFAULTS)})")
        inc = re.compile(self.spec["targets"]) if self.spec["targets"] else None
        exc = re.compile(self.spec["exclude"]) if self.spec["exclude"] else None
        self.optimizer = optimizer
        self.r0: dict[int, Tensor] = {}
        self.names: list[str] = []
        for name, p in named_params:
            if not p.requires_grad or (p.ndim < 2 and not self.spec["include_1d"]):
                continue
            if (inc and not inc.search(name)) or (exc and exc.search(name)):
                continue
            self.r0[id(p)] = p.detach().float().square().mean().sqrt().clamp_min(1e-12)
            self.names.append(name)
        self.step = 0

    def rate(self, t: int) -> float:
        w = int(self.spec["warmup"])
        return float(self.spec["rate"]) * (min(1.0, (t + 1) / w) if w > 0 else 1.0)

    def cap(self, t: int) -> float:
        n, c1 = int(self.spec["cap_anneal"]), float(self.spec["cap"])
        c0 = float(self.spec["cap_start"]) or c1
        return c1 if n <= 0 else c0 + (c1 - c0) * min(1.0, t / n)

    @torch.no_grad()
    def apply(self, skip: Tensor | None = None) -> None:
        rate, cap = self.rate(self.step), self.cap(self.step)
        self.step += 1
        if rate <= 0:
            return
        for g in self.optimizer.param_groups:
            params = [p for p in g["params"] if id(p) in self.r0]
            if not params:
                continue
            coef = g["lr"] * g.get("lr_mul", 1.0) * rate * _gate(skip, params[0].device)
            pf = [p.float() for p in params]
            excess = torch._foreach_abs(pf)
            torch._foreach_sub_(excess, [self.r0[id(p)] * cap for p in params])
            torch._foreach_clamp_min_(excess, 0.0)
            torch._foreach_mul_(excess, torch._foreach_sign(pf))
            torch._foreach_mul_(excess, coef)
            for p, e in zip(params, excess):
                p.sub_(e.to(p.dtype))

    def state_dict(self) -> dict:
        return {"step": self.step}

    def load_state_dict(self, sd: dict) -> None:
        self.step = int(sd.get("step", 0))


def regularizer_problems(k: dict) -> list[str]:
    """Knob cross-checks for WD_TARGET and OUTLIER_DECAY."""
    out = []
    if k.get("WD_TARGET", "zero") == "start":
        if k.get("ALGO") != "full":
            out.append("WD_TARGET='start' trains the base weights (ALGO 'full')")
        if not k.get("WEIGHT_DECAY", 0) > 0:
            out.append("WD_TARGET='start' needs WEIGHT_DECAY > 0")
        if k.get("OPTIMIZER", "adamw") not in ANCHOR_OPTIMIZERS:
            out.append(f"WD_TARGET='start' runs with OPTIMIZER in {ANCHOR_OPTIMIZERS}")
    spec = k.get("OUTLIER_DECAY") or {}
    if spec:
        unknown = set(spec) - set(OUTLIER_DEFAULTS)
        if unknown:
            out.append(f"OUTLIER_DECAY keys {sorted(unknown)} unknown (have {sorted(OUTLIER_DEFAULTS)})")
        if float(spec.get("rate", 0)) < 0 or float(spec.get("cap", 16.0)) <= 0:
            out.append("OUTLIER_DECAY needs rate >= 0 and cap > 0")
    return out
