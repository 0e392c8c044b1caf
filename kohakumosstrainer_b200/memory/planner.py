"""`MEMORY_PROFILE="auto"`: the fastest plan whose estimate fits the device.

Candidates are the named profiles in speed order, then the catalog grid; each is scored with
`estimate.relative_cost` and filtered with `estimate.fits` against the device's total memory
minus what other processes hold. Explicit knobs pin their field in every candidate. The
reference plans the same way on rank 0 and broadcasts the result
(`src/kohakumoss/memory/planner.py:1-139`); here the choice is a pure function of (workload,
device bytes), so every rank computes it locally and a mismatch is caught by the knob
agreement gate of the launcher.
"""

from __future__ import annotations

from dataclasses import replace

from .estimate import Workload, estimate, fits, relative_cost
from .plan import ORDER, PROFILES, MemoryPlan, catalog, plan_problems


def device_bytes(device=None) -> int:
    import torch

    if not torch.cuda.is_available():
        return 180 * (1 << 30)
    free, total = torch.cuda.mem_get_info(device)
    mine = torch.cuda.memory_reserved(device)
    return int(free + mine)


def candidates(pinned: dict) -> list[MemoryPlan]:
    seen, out = set(), []
    specs = [(n, PROFILES[n]) for n in ORDER] + list(catalog().items())
    for name, spec in specs:
        plan = MemoryPlan(profile=name, **{**spec, **pinned})
        key = tuple(sorted((k, str(v)) for k, v in plan.to_dict().items() if k not in ("profile", "overrides")))
        if key in seen or plan_problems(plan):
            continue
        seen.add(key)
        out.append(plan)
    return out


def plan_auto(work: Workload, total_bytes: int, pinned: dict | None = None, margin: float = 0.92, force: bool = False,
              host_bytes: int | None = None) -> tuple[MemoryPlan, dict]:
    """-> (plan, report). `force` returns the smallest plan even when nothing fits. `host_bytes` (default: the
    cgroup-aware room of this host) bounds what a plan may park in host memory."""
    if host_bytes is None:
        from ..utils.hostmem import host_room

        host_bytes = host_room()
    pool = candidates(dict(pinned or {}))
    scored = sorted(pool, key=lambda p: (relative_cost(p), estimate(work, p)["total"]))
    for plan in scored:
        if fits(work, plan, total_bytes, margin) and estimate(work, plan)["host"] <= host_bytes:
            est = estimate(work, plan)
            return replace(plan, profile=f"auto:{plan.profile}"), {"estimate": est, "device_bytes": total_bytes, "considered": len(pool),
                                                                  "relative_cost": relative_cost(plan)}
    smallest = min(pool, key=lambda p: estimate(work, p)["total"])
    est = estimate(work, smallest)
    if not force:
        raise MemoryError(f"no memory plan fits {total_bytes / 2**30:.1f} GiB: the smallest ({smallest.profile}) needs "
                          f"{est['total'] / 2**30:.1f} GiB; lower MAX_TOKENS or set MEMORY_AUTO_FORCE=True")
    return replace(smallest, profile=f"auto:{smallest.profile}"), {"estimate": est, "device_bytes": total_bytes, "considered": len(pool),
                                                                  "forced": True}
