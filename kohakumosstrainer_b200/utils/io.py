"""Atomic JSON / text writes (`src/kohakumoss_common/io.py` in the reference)."""

from __future__ import annotations

import json
import os
import tempfile
from pathlib import Path


def write_atomic(path: str | os.PathLike, data: bytes | str) -> None:
    """Write into a temp file in the same directory, fsync, then rename over `path`."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    mode = "wb" if isinstance(data, bytes) else "w"
    fd, tmp = tempfile.mkstemp(dir=path.parent, prefix=path.name + ".", suffix=".tmp")
    try:
        with os.fdopen(fd, mode) as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def write_json(path, obj, indent: int = 2) -> None:
    write_atomic(path, json.dumps(obj, indent=indent, sort_keys=True, default=str))


def read_json(path, default=None):
    try:
        with open(path) as f:
            return json.load(f)
    except FileNotFoundError:
        if default is not None:
            return default
        raise


def append_jsonl(path, obj) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(obj, default=str) + "\n")
