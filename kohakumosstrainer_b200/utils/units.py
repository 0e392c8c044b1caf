"""Unit constants and small formatters (`src/kohakumoss_common/units.py`)."""

KIB = 1 << 10
MIB = 1 << 20
GIB = 1 << 30
KB = 10**3
MB = 10**6
GB = 10**9
TERA = 10**12


def fmt_bytes(n: float) -> str:
    for unit, size in (("GiB", GIB), ("MiB", MIB), ("KiB", KIB)):
        if abs(n) >= size:
            return f"{n / size:.2f} {unit}"
    return f"{int(n)} B"


def fmt_seconds(s: float) -> str:
    if s >= 3600:
        return f"{int(s // 3600)}h{int(s % 3600 // 60):02d}m"
    if s >= 60:
        return f"{int(s // 60)}m{int(s % 60):02d}s"
    return f"{s:.2f}s"
