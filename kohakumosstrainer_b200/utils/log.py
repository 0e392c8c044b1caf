"""Rank-aware logging: `[HH:MM:SS] [rankN] [module] [LEVEL] msg k=v`.

Same line format and once-only helpers as the reference logger
(`src/kohakumoss_common/log.py`).
"""

from __future__ import annotations

import logging
import os
import sys
import time

_ROOT = "kmoss"
_SEEN: set[str] = set()
_CONFIGURED = False


class _Formatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        stamp = time.strftime("%H:%M:%S", time.localtime(record.created))
        rank = os.environ.get("RANK", "0")
        name = record.name.removeprefix(_ROOT + ".") or _ROOT
        msg = record.getMessage()
        extra = getattr(record, "kv", None)
        if extra:
            msg += " " + " ".join(f"{k}={_fmt(v)}" for k, v in extra.items())
        if record.exc_info:
            msg += "\n" + self.formatException(record.exc_info)
        return f"[{stamp}] [rank{rank}] [{name}] [{record.levelname}] {msg}"


def _fmt(value) -> str:
    if isinstance(value, float):
        return f"{value:.6g}"
    return str(value)


class Logger(logging.LoggerAdapter):
    """Adapter whose calls take keyword pairs: `log.info("step", loss=0.1)`."""

    def process(self, msg, kwargs):
        keep = {}
        for key in ("exc_info", "stack_info", "stacklevel"):
            if key in kwargs:
                keep[key] = kwargs.pop(key)
        keep["extra"] = {"kv": dict(kwargs)}
        return msg, keep

    def once(self, key: str, msg: str, level: int = logging.INFO, **kv) -> None:
        """Log `msg` the first time `key` is seen in this process."""
        if key in _SEEN:
            return
        _SEEN.add(key)
        self.log(level, msg, **kv)

    def table(self, rows: list[dict], title: str = "") -> None:
        """Log a list of dicts as an aligned text table."""
        if not rows:
            return
        cols = list(rows[0])
        width = {c: max(len(c), *(len(_fmt(r.get(c, ""))) for r in rows)) for c in cols}
        lines = [title] if title else []
        lines.append("  ".join(c.ljust(width[c]) for c in cols))
        for r in rows:
            lines.append("  ".join(_fmt(r.get(c, "")).ljust(width[c]) for c in cols))
        self.info("\n".join(lines))


def setup(level: str | int = "INFO", file: str | None = None, all_ranks: bool = False) -> None:
    """Install the console (and optional file) handler; non-zero ranks log warnings only
    unless `all_ranks`."""
    global _CONFIGURED
    root = logging.getLogger(_ROOT)
    root.handlers.clear()
    if isinstance(level, str):
        level = getattr(logging, level.upper())
    rank = int(os.environ.get("RANK", "0"))
    root.setLevel(level if (rank == 0 or all_ranks) else max(level, logging.WARNING))
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(_Formatter())
    root.addHandler(handler)
    if file:
        fh = logging.FileHandler(file)
        fh.setFormatter(_Formatter())
        root.addHandler(fh)
    root.propagate = False
    _CONFIGURED = True


def get_logger(name: str = "") -> Logger:
    if not _CONFIGURED:
        setup()
    name = name.removeprefix("kohakumosstrainer_b200.")
    return Logger(logging.getLogger(f"{_ROOT}.{name}" if name else _ROOT), {})
