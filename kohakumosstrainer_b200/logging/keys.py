"""Metric key groups and verbosity levels (`src/kohakumoss/logging/keys.py:6-58`)."""

GROUPS = ("loss/", "stream/", "opt/", "amp/", "speed/", "probe/", "detail/", "ddp/", "pipe/", "mem/")
_LEVELS = {"train": ("loss/", "opt/", "speed/", "amp/"), "bench": ("loss/", "opt/", "speed/", "amp/", "ddp/", "pipe/", "mem/"),
           "debug": GROUPS}


def level_allows(level: str, key: str) -> bool:
    return any(key.startswith(g) for g in _LEVELS.get(level, GROUPS)) or "/" not in key
