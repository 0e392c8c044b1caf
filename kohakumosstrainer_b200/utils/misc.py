"""Small helpers: no-op callables, dotted imports, greedy runs, weak callbacks, markdown
tables, device strings, host memory room.

Each is the counterpart of a one-file module of the reference's `kohakumoss_common`
(`calls.py`, `imports.py`, `runs.py`, `weak.py`, `markdown.py`, `devices.py`, `hostmem/`).
"""

from __future__ import annotations

import importlib
import os
import weakref
from collections.abc import Callable, Iterable, Sequence


def nothing(*_args, **_kwargs) -> None:
    return None


def identity(x):
    return x


def import_path(path: str):
    """`pkg.mod.attr` or `pkg.mod:attr` -> object."""
    module, _, attr = path.replace(":", ".").rpartition(".")
    return getattr(importlib.import_module(module), attr)


def runs(values: Sequence[int]) -> list[tuple[int, int]]:
    """Greedy maximal runs of consecutive integers: [3,4,5,9] -> [(3,6),(9,10)]."""
    out: list[tuple[int, int]] = []
    for v in values:
        if out and out[-1][1] == v:
            out[-1] = (out[-1][0], v + 1)
        else:
            out.append((v, v + 1))
    return out


def weak_method(method: Callable) -> Callable:
    """A callable that forwards to a bound method while its owner lives, else no-op."""
    ref = weakref.WeakMethod(method)

    def call(*args, **kwargs):
        fn = ref()
        return None if fn is None else fn(*args, **kwargs)

    return call


def markdown_table(rows: Iterable[dict], columns: Sequence[str] | None = None) -> str:
    rows = list(rows)
    if not rows:
        return ""
    cols = list(columns or rows[0])
    lines = ["| " + " | ".join(cols) + " |", "|" + "|".join("---" for _ in cols) + "|"]
    for r in rows:
        lines.append("| " + " | ".join(str(r.get(c, "")) for c in cols) + " |")
    return "\n".join(lines)


def device_index(device: str | int) -> int:
    if isinstance(device, int):
        return device
    return int(device.split(":")[1]) if ":" in device else 0


def streamed_type(device_type: str) -> bool:
    """True when host tensors reach this device type through pinned memory."""
    return device_type in ("cuda", "xpu")


def host_memory_room() -> int:
    """Bytes of host RAM still free for us: min(MemAvailable, cgroup limit - usage)."""
    room = None
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    room = int(line.split()[1]) * 1024
                    break
    except OSError:
        pass
    for limit_path, usage_path in (
        ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
        ("/sys/fs/cgroup/memory/memory.limit_in_bytes", "/sys/fs/cgroup/memory/memory.usage_in_bytes"),
    ):
        try:
            limit = open(limit_path).read().strip()
            usage = int(open(usage_path).read().strip())
            if limit != "max":
                left = int(limit) - usage
                room = left if room is None else min(room, left)
        except (OSError, ValueError):
            continue
    return room if room is not None else os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
