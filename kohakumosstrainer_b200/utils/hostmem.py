"""Host memory room, cgroup aware (`src/kohakumoss_common/hostmem/` there): what pinned staging, host optimiser
state and streamed weights may take before the container's limit bites."""

from __future__ import annotations

from pathlib import Path


def _read_int(path: str) -> int | None:
    try:
        text = Path(path).read_text().strip()
        return None if text in ("", "max") else int(text)
    except (OSError, ValueError):
        return None


def meminfo() -> dict[str, int]:
    out = {}
    try:
        for line in Path("/proc/meminfo").read_text().splitlines():
            key, _, rest = line.partition(":")
            out[key] = int(rest.split()[0]) * 1024
    except (OSError, ValueError, IndexError):
        pass
    return out


def host_limit() -> int | None:
    """The cgroup memory limit of this process (v2, then v1), None when unlimited."""
    for path in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        v = _read_int(path)
        if v is not None and v < 1 << 60:
            return v
    return None


def host_used() -> int | None:
    for path in ("/sys/fs/cgroup/memory.current", "/sys/fs/cgroup/memory/memory.usage_in_bytes"):
        v = _read_int(path)
        if v is not None:
            return v
    return None


def host_room(reserve: float = 0.1) -> int:
    """Bytes this process can still take: min(MemAvailable, cgroup limit - usage), minus a reserve."""
    info = meminfo()
    room = info.get("MemAvailable", 1 << 62)
    limit, used = host_limit(), host_used()
    if limit is not None and used is not None:
        room = min(room, limit - used)
    total = info.get("MemTotal", room)
    return max(0, int(room - reserve * min(total, limit or total)))
