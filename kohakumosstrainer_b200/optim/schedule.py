"""Learning-rate schedules from the `SCHEDULE` knob: `{"mode": "cosine", "warmup": 100,
"end": -1, "min": 0.1}` (`scripts/train/moss.py:137-151` defaults; modes cosine | linear |
constant, linear warm-up)."""

from __future__ import annotations

import math


def build_schedule(spec: dict | None, total_steps: int):
    spec = dict(spec or {})
    mode = spec.get("mode", "cosine")
    warmup = int(spec.get("warmup", 0))
    end = int(spec.get("end", -1))
    end = total_steps if end < 0 else end
    floor = float(spec.get("min", spec.get("min_value", 0.1)))
    if mode not in ("cosine", "linear", "constant"):
        raise ValueError(f"SCHEDULE mode must be cosine|linear|constant, got {mode}")

    def factor(step: int) -> float:
        if warmup > 0 and step < warmup:
            return (step + 1) / warmup
        if mode == "constant":
            return 1.0
        span = max(1, end - warmup)
        t = min(1.0, max(0.0, (step - warmup) / span))
        if mode == "linear":
            return floor + (1 - floor) * (1 - t)
        return floor + (1 - floor) * 0.5 * (1 + math.cos(math.pi * t))

    return factor
