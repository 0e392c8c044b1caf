"""Catalog: every image of one or more sources as columnar planning arrays plus per-row
variable fields.

Planning needs only numbers (size, weight, caption character counts, liveness), so those live
in numpy columns and a million-row dataset plans without touching a Python object per row;
the variable fields (locator, tags, captions, json) are JSON lines addressed through an offset
table and parsed on demand. One catalog is ONE file (`KMC2` container: header JSON, npy
columns, offset table, JSON-lines blob), written atomically by a single writer and memory-mapped
by readers. The same roles as the reference's catalog table and vault
(`src/kohakumoss_data/catalog/table.py:52-180`, `catalog/vault.py`), without a database.

An incremental scan (`merge_scan`) reuses the rows whose `stamp` (path, size, mtime) is
unchanged, marks vanished files dead (`live = False`, ids stay stable so cache keys and plans
of other rows do not move) and appends new files.
"""

from __future__ import annotations

import io
import json
import os
import struct
from dataclasses import asdict, dataclass, field

import numpy as np

MAGIC = b"KMC2"
CHAR_FIELDS = ("tags_chars", "nl_chars", "artist_chars", "rating_chars", "json_chars")


@dataclass
class Row:
    """One image record; `weight` generalises repeats (`src/kohakumoss_data/types.py:18-35`)."""

    locator: str
    w: int
    h: int
    has_alpha: bool = False
    group: str = ""
    weight: float = 1.0
    tags: list | None = None
    caption_nl: str | None = None
    artist: str | None = None
    rating: str | None = None
    json: dict | None = None
    extra: dict = field(default_factory=dict)
    id: int = 0

    def chars(self) -> tuple[int, int, int, int, int]:
        tags = sum(len(t) + 2 for t in self.tags) if self.tags else 0
        js = len(json.dumps(self.json, ensure_ascii=False)) if self.json else 0
        return (tags, len(self.caption_nl or ""), len(self.artist or ""), len(self.rating or ""), js)

    def variable(self) -> dict:
        d = asdict(self)
        for k in ("w", "h", "has_alpha", "weight", "id"):
            d.pop(k)
        return {k: v for k, v in d.items() if v not in (None, "", {}, [])}


class _Blob:
    """JSON lines behind an offset table; parses one row per call, keeps a small cache."""

    def __init__(self, data, offsets: np.ndarray):
        self.data, self.offsets = data, offsets
        self._cache: dict[int, dict] = {}

    def __call__(self, i: int) -> dict:
        hit = self._cache.get(i)
        if hit is None:
            lo, hi = int(self.offsets[i]), int(self.offsets[i + 1])
            hit = json.loads(bytes(self.data[lo:hi]).decode("utf-8"))
            if len(self._cache) >= 4096:
                self._cache.pop(next(iter(self._cache)))
            self._cache[i] = hit
        return hit


class _Concat:
    """Variable fields of concatenated catalogs: global id -> (part, local id). Holds the parts
    themselves, so a file-backed part still pickles as its path."""

    def __init__(self, parts):
        self.parts = list(parts)
        self.bounds = np.cumsum([0] + [len(p) for p in self.parts])

    def __call__(self, i: int) -> dict:
        k = int(np.searchsorted(self.bounds, i, side="right")) - 1
        return self.parts[k]._fetch(i - int(self.bounds[k]))


class Catalog:
    def __init__(self, rows: list[Row] | None = None):
        rows = rows or []
        n = len(rows)
        chars = np.array([r.chars() for r in rows], dtype=np.int64).reshape(n, len(CHAR_FIELDS))
        self.columns = {
            "w": np.array([r.w for r in rows], dtype=np.int64),
            "h": np.array([r.h for r in rows], dtype=np.int64),
            "weight": np.array([r.weight for r in rows], dtype=np.float32),
            "has_alpha": np.array([r.has_alpha for r in rows], dtype=bool),
            "live": np.ones(n, dtype=bool),
            "source": np.zeros(n, dtype=np.int64),
            **{name: chars[:, k].copy() for k, name in enumerate(CHAR_FIELDS)},
        }
        lines = [json.dumps(r.variable(), ensure_ascii=False).encode("utf-8") for r in rows]
        offsets = np.zeros(n + 1, dtype=np.int64)
        if n:
            offsets[1:] = np.cumsum([len(b) for b in lines])
        self._fetch = _Blob(b"".join(lines), offsets)
        self.path: str | None = None

    # -- columns ------------------------------------------------------------------------------
    def __len__(self) -> int:
        return int(self.columns["w"].shape[0])

    def __getattr__(self, name):
        cols = self.__dict__.get("columns")
        if cols is not None and name in cols:
            return cols[name]
        raise AttributeError(name)

    @property
    def chars(self) -> dict:
        return {k: self.columns[k] for k in CHAR_FIELDS}

    def __getitem__(self, i: int) -> Row:
        var = dict(self._fetch(int(i)))
        return Row(locator=var.pop("locator"), w=int(self.w[i]), h=int(self.h[i]), has_alpha=bool(self.has_alpha[i]),
                   weight=float(self.weight[i]), id=int(i), **var)

    def locator(self, i: int) -> str:
        return self._fetch(int(i))["locator"]

    def stamps(self) -> dict[str, int]:
        """locator -> row id, for incremental scans."""
        return {self.locator(i): i for i in range(len(self))}

    # -- composition --------------------------------------------------------------------------
    @classmethod
    def concat(cls, parts: list["Catalog"], weights: list[float] | None = None) -> "Catalog":
        """Rows of several catalogs back to back; `source` = part index; part k's row weights
        are multiplied by `weights[k]`."""
        weights = weights or [1.0] * len(parts)
        out = cls([])
        out.columns = {k: np.concatenate([p.columns[k] for p in parts]) if parts else v for k, v in out.columns.items()}
        out.columns["source"] = np.concatenate([np.full(len(p), k, dtype=np.int64) for k, p in enumerate(parts)]) if parts else out.columns["source"]
        out.columns["weight"] = np.concatenate([p.columns["weight"] * np.float32(w) for p, w in zip(parts, weights)]) if parts else out.columns["weight"]
        out._fetch = _Concat(parts)
        return out

    # -- file ---------------------------------------------------------------------------------
    def save(self, path: str) -> None:
        """Atomic single-writer save (write to `<path>.tmp.<pid>`, fsync, rename)."""
        n = len(self)
        if isinstance(self._fetch, _Blob):
            blob, offsets = bytes(self._fetch.data), self._fetch.offsets
        else:
            lines = [json.dumps(self._fetch(i), ensure_ascii=False).encode("utf-8") for i in range(n)]
            offsets = np.zeros(n + 1, dtype=np.int64)
            if n:
                offsets[1:] = np.cumsum([len(b) for b in lines])
            blob = b"".join(lines)
        sections = {}
        for name, col in {**self.columns, "__offsets__": offsets}.items():
            buf = io.BytesIO()
            np.save(buf, col, allow_pickle=False)
            sections[name] = buf.getvalue()
        sections["__rows__"] = blob
        header, pos = {"rows": n, "sections": {}}, 0
        for name, data in sections.items():
            header["sections"][name] = [pos, len(data)]
            pos += (len(data) + 63) // 64 * 64
        head = json.dumps(header).encode("utf-8")
        tmp = f"{path}.tmp.{os.getpid()}"
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(tmp, "wb") as f:
            f.write(MAGIC + struct.pack("<I", len(head)) + head)
            base = (f.tell() + 63) // 64 * 64
            for name, data in sections.items():
                f.seek(base + header["sections"][name][0])
                f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
        self.path = path

    @classmethod
    def load(cls, path: str) -> "Catalog":
        with open(path, "rb") as f:
            if f.read(4) != MAGIC:
                raise ValueError(f"{path} is not a catalog file of this layout; scan or import the source again")
            (hl,) = struct.unpack("<I", f.read(4))
            header = json.loads(f.read(hl))
            base = (8 + hl + 63) // 64 * 64
        mm = np.memmap(path, dtype=np.uint8, mode="r")
        out = cls([])
        cols = {}
        for name, (pos, size) in header["sections"].items():
            raw = mm[base + pos : base + pos + size]
            if name == "__rows__":
                rows = raw
            else:
                cols[name] = np.load(io.BytesIO(bytes(raw)), allow_pickle=False)
        offsets = cols.pop("__offsets__")
        out.columns = cols
        out._fetch = _Blob(rows, offsets)
        out.path = path
        return out

    def __getstate__(self):
        # a file-backed catalog pickles as its path (loader workers reopen the map)
        if self.path is not None and isinstance(self._fetch, _Blob):
            return {"path": self.path}
        return self.__dict__

    def __setstate__(self, state):
        if set(state) == {"path"}:
            self.__dict__.update(Catalog.load(state["path"]).__dict__)
        else:
            self.__dict__.update(state)


def is_catalog(path: str) -> bool:
    try:
        with open(path, "rb") as f:
            return f.read(4) == MAGIC
    except OSError:
        return False


def merge_scan(old: Catalog | None, found: list[Row]) -> tuple[Catalog, dict]:
    """Incremental scan result: rows of `old` keep their ids; a row whose file vanished turns
    dead; a changed stamp replaces the row's fields in place; new files are appended."""
    if old is None or len(old) == 0:
        return Catalog(found), {"new": len(found), "kept": 0, "changed": 0, "dead": 0}
    by_loc = {r.locator: r for r in found}
    rows, stats = [], {"new": 0, "kept": 0, "changed": 0, "dead": 0}
    live = []
    for i in range(len(old)):
        prev = old[i]
        now = by_loc.pop(prev.locator, None)
        if now is None:
            rows.append(prev)
            live.append(False)
            stats["dead"] += bool(old.live[i])
        elif now.extra.get("hash") == prev.extra.get("hash"):
            rows.append(now)
            live.append(True)
            stats["kept"] += 1
        else:
            rows.append(now)
            live.append(True)
            stats["changed"] += 1
    for r in by_loc.values():
        rows.append(r)
        live.append(True)
        stats["new"] += 1
    out = Catalog(rows)
    out.columns["live"] = np.array(live, dtype=bool)
    return out, stats
