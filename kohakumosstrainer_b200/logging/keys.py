"""Metric key groups and verbosity levels (`src/kohakumoss/logging/keys.py:6-58`)."""

GROUPS = ("loss/", "val/", "samples/", "stream/", "opt/", "amp/", "speed/", "probe/", "detail/", "ddp/", "pipe/", "mem/", "xfer/", "breakdown/")
_LEVELS = {"train": ("loss/", "val/", "samples/", "stream/", "opt/", "speed/", "amp/"),
           "bench": ("loss/", "val/", "samples/", "stream/", "opt/", "speed/", "amp/", "ddp/", "pipe/", "mem/", "xfer/", "breakdown/"),
           "debug": GROUPS}


def level_allows(level: str, key: str) -> bool:
    return any(key.startswith(g) for g in _LEVELS.get(level, GROUPS)) or "/" not in key
